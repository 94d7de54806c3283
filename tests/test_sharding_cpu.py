"""Multi-rank sharding logic on CPU: two gloo ranks each take their row shard of a W4G128
weight, run the matmul (here: the CPU oracle standing in for the device), all-gather, and
must reproduce the unsharded result bit for bit."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
N, K, M = 128, 256, 3


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    blocks = pkg.synth.bg128_weight(5, 1, N, K)
    x = pkg.synth.activations(6, 1, M, K)
    mine, rows, lo = pkg.shard.shard_blocks(blocks, N, K, rank, world)
    y_local = torch.from_numpy(ol.matmul_w4(np.ascontiguousarray(mine), rows, K, x))
    parts = [torch.zeros_like(y_local) for _ in range(world)]
    dist.all_gather(parts, y_local)
    y = torch.cat(parts, dim=1).numpy()
    if rank == 0:
        np.save(os.path.join(out_dir, "y.npy"), y)
    dist.destroy_process_group()


def test_row_sharded_matmul_world2(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    y = np.load(tmp_path / "y.npy")
    blocks = pkg.synth.bg128_weight(5, 1, N, K)
    x = pkg.synth.activations(6, 1, M, K)
    assert y.tobytes() == ol.matmul_w4(blocks, N, K, x).tobytes()


def _k_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, k, m = 72, 1024, 3
    blocks = pkg.synth.bg128_weight(5, 7, n, k)
    x = pkg.synth.activations(6, 7, m, k)
    mine, k0 = pkg.shard.shard_blocks_k(blocks, n, k, rank, world)
    kl = k // world
    y_local, sums = ol.matmul_w4(mine, n, kl, np.ascontiguousarray(x[:, k0:k0 + kl]),
                                 want_sums=True)
    y = torch.from_numpy(y_local.copy())
    dist.all_reduce(y)  # the partial sums meet
    parts = [torch.zeros(sums.shape, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(sums))
    if rank == 0:
        np.save(os.path.join(out_dir, "y_k.npy"), y.numpy())
        np.save(os.path.join(out_dir, "sums_k.npy"), torch.cat(parts, dim=2).numpy())
    dist.destroy_process_group()


def test_input_feature_split_with_all_reduce_world2(tmp_path):
    """The K-split variant: whole 128-groups per rank, partial outputs all-reduced.  Integer
    group sums are the unsharded ones exactly; the fp32 result agrees to rounding."""
    port = 29500 + (os.getpid() + 911) % 2000
    mp.spawn(_k_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    n, k = 72, 1024
    blocks = pkg.synth.bg128_weight(5, 7, n, k)
    x = pkg.synth.activations(6, 7, 3, k)
    want, want_sums = ol.matmul_w4(blocks, n, k, x, want_sums=True)
    assert (np.load(tmp_path / "sums_k.npy") == want_sums).all()
    got = np.load(tmp_path / "y_k.npy")
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-6
    with pytest.raises(ValueError):
        pkg.shard.shard_blocks_k(blocks, n, k, 0, 3)


def test_shard_ranges():
    assert pkg.shard.row_range(9728, 3, 8) == (3648, 4864)
    with pytest.raises(ValueError):
        pkg.shard.row_range(9728 + 8, 0, 8)
    blocks = pkg.synth.bg128_weight(5, 2, 64, 256)
    parts = [pkg.shard.shard_blocks(blocks, 64, 256, r, 4)[0] for r in range(4)]
    assert np.concatenate(parts).tobytes() == blocks.tobytes()
    assert pkg.shard.expert_range(128, 7, 8) == (112, 128)
    with pytest.raises(ValueError):
        pkg.shard.expert_range(128, 0, 3)


# ---- expert-parallel MoE: split at the route outputs, all-reduce, ordered combine --------
E, TOPK, H, I, T = 8, 2, 128, 128, 5


def _moe_inputs():
    router = pkg.synth.router_weight(9, 1, E, H)
    gu = pkg.synth.bg128_weight(9, 2, E * 2 * I, H)
    dn = pkg.synth.bg128_weight(9, 3, E * H, I)
    x = pkg.synth.activations(9, 4, T, H)
    return router, gu, dn, x


class _OracleEngine:
    """The CPU oracle standing in for the device halves of the op."""

    def __init__(self, router, gu_local, dn_local, lo, cnt):
        self.router, self.gu, self.dn, self.lo, self.cnt = router, gu_local, dn_local, lo, cnt

    def expert_outputs(self, hidden):
        logits = ol.router_logits(hidden, self.router)
        idx, w = ol.select_routes(logits, TOPK)
        # local aggregates are indexed from the first expert held
        routes = ol.expert_route_outputs(hidden, idx - self.lo, I, self.gu, self.dn, self.cnt)
        return torch.from_numpy(routes), idx, w

    def combine(self, route_out, idx, w, out):
        out[:] = ol.moe_combine(route_out.numpy(), idx, w)


def _ep_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    router, gu, dn, x = _moe_inputs()
    ep = pkg.expert_parallel
    gu_l, lo, cnt = ep.shard_expert_blocks(gu, E, 2 * I, H, rank, world)
    dn_l, _, _ = ep.shard_expert_blocks(dn, E, H, I, rank, world)
    op = ep.ExpertParallelMoE(_OracleEngine(router, gu_l, dn_l, lo, cnt), dist.all_reduce)
    out = np.zeros((T, H), dtype=np.float32)
    op.forward(x, out)
    np.save(os.path.join(out_dir, f"moe{rank}.npy"), out)
    dist.destroy_process_group()


def test_moe_split_equals_monolithic_oracle():
    router, gu, dn, x = _moe_inputs()
    want, logits, idx, w = ol.moe_forward(x, router, TOPK, I, gu, dn)
    assert ol.router_logits(x, router).tobytes() == logits.tobytes()
    routes = ol.expert_route_outputs(x, idx, I, gu, dn, E)
    assert ol.moe_combine(routes, idx, w).tobytes() == want.tobytes()


def test_expert_parallel_moe_world2(tmp_path):
    port = 31500 + os.getpid() % 2000
    mp.spawn(_ep_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    router, gu, dn, x = _moe_inputs()
    want = ol.moe_forward(x, router, TOPK, I, gu, dn)[0]
    for r in range(2):
        assert np.load(tmp_path / f"moe{r}.npy").tobytes() == want.tobytes()


def test_expert_shard_ranges():
    ep = pkg.expert_parallel
    blocks = pkg.synth.bg128_weight(5, 3, 4 * 16, 128)
    parts = [ep.shard_expert_blocks(blocks, 4, 16, 128, r, 2) for r in range(2)]
    assert np.concatenate([p[0] for p in parts]).tobytes() == blocks.tobytes()
    assert [(p[1], p[2]) for p in parts] == [(0, 2), (2, 2)]
    with pytest.raises(ValueError):
        ep.shard_expert_blocks(blocks, 4, 12, 128, 0, 2)


def _token_rows():
    rng = np.random.default_rng(91)
    plain = rng.standard_normal(64).astype(np.float32)
    ties = np.zeros(64, dtype=np.float32)
    ties[[13, 40, 63]] = 2.5                       # equal maxima on both ranks of a world of 2
    zeros = np.full(64, -3.0, dtype=np.float32)
    zeros[50], zeros[20] = 0.0, -0.0               # -0 on rank 0 ties +0 on rank 1
    nan0 = rng.standard_normal(64).astype(np.float32)
    nan0[0] = np.nan                               # nothing beats a NaN at index 0
    nans = rng.standard_normal(64).astype(np.float32)
    nans[[5, 32, 33]] = np.nan                     # a NaN elsewhere never wins
    ninf = np.full(64, -np.inf, dtype=np.float32)
    ninf[32] = np.nan                              # first row of rank 1 is a NaN: not index 0
    return [plain, ties, zeros, nan0, nans, ninf]


def test_top1_words_order_like_argmax_token():
    """One rank: the largest word of a row is the oracle's argmax_token, corner cases
    included; shards of any split give the same token through pick_token."""
    for row in _token_rows():
        want = ol.argmax_token(row)
        assert pkg.shard.pick_token([pkg.shard.shard_top1_word(row, 0)]) == want
        for world in (2, 4, 8):
            per = len(row) // world
            words = [pkg.shard.shard_top1_word(row[r * per:(r + 1) * per], r * per)
                     for r in range(world)]
            assert pkg.shard.pick_token(words) == want, world


def _token_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    blocks = pkg.synth.bg128_weight(8, 1, N, K)
    x = pkg.synth.activations(9, 1, M, K)
    mine, rows, lo = pkg.shard.shard_blocks(blocks, N, K, rank, world)
    y_local = ol.matmul_w4(np.ascontiguousarray(mine), rows, K, x)
    tokens = []
    for m in range(M):  # each rank hands over one word per activation row
        word = pkg.shard.shard_top1_word(y_local[m], lo)
        mine_t = torch.tensor([word >> 32, word & 0xFFFFFFFF], dtype=torch.int64)
        parts = [torch.zeros_like(mine_t) for _ in range(world)]
        dist.all_gather(parts, mine_t)
        tokens.append(pkg.shard.pick_token([(int(p[0]) << 32) | int(p[1]) for p in parts]))
    np.save(os.path.join(out_dir, f"tok{rank}.npy"), np.array(tokens))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 8])
def test_row_sharded_greedy_token(tmp_path, world):
    """Two and eight gloo ranks, the oracle standing in for the device matmul: every rank ends
    with the token argmax_token picks over the unsharded logits."""
    port = 29500 + (os.getpid() + 7 + world) % 2000
    mp.spawn(_token_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    blocks = pkg.synth.bg128_weight(8, 1, N, K)
    x = pkg.synth.activations(9, 1, M, K)
    full = ol.matmul_w4(blocks, N, K, x)
    want = [ol.argmax_token(full[m]) for m in range(M)]
    for rank in range(world):
        assert np.load(tmp_path / f"tok{rank}.npy").tolist() == want


# ---- sequence-sharded MoE: rows travel to the experts' owners and back (all-to-all) -------
class _OracleRowsEngine:
    """The oracle standing in for the three device pieces AllToAllMoE needs."""

    def __init__(self, router, gu_local, dn_local, local_experts):
        self.router, self.gu, self.dn, self.cnt = router, gu_local, dn_local, local_experts

    def routes(self, hidden):
        if hidden.shape[0] == 0:  # a rank without tokens still takes part in the exchanges
            return (torch.zeros((0, TOPK), dtype=torch.int32),
                    torch.zeros((0, TOPK), dtype=torch.float32))
        idx, w = ol.select_routes(ol.router_logits(hidden.numpy(), self.router), TOPK)
        return torch.from_numpy(idx), torch.from_numpy(w)

    def expert_rows(self, rows, experts):
        if rows.shape[0] == 0:
            return rows.clone()
        # every received row is a one-route token of its expert; the reference's rule sees
        # how many rows each expert holds
        idx = experts.to(torch.int32).numpy().reshape(-1, 1)
        return torch.from_numpy(ol.expert_route_outputs(rows.numpy(), idx, I, self.gu, self.dn,
                                                        self.cnt, rule=ol.ACT_G32))

    def combine(self, route_out, idx, wts, out):
        if out.shape[0]:
            out.copy_(torch.from_numpy(ol.moe_combine(route_out.numpy(), idx.numpy(),
                                                      wts.numpy())))


def _a2a_worker(rank, world, port, out_dir, tokens):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    router, gu, dn, _ = _moe_inputs()
    x = pkg.synth.activations(9, 40 + tokens, tokens, H)
    # uneven contiguous token blocks: rank r takes tokens [cut[r], cut[r + 1])
    cut = [0] + [min(tokens, (r + 1) * tokens // world + (1 if r == 0 else 0))
                 for r in range(world - 1)] + [tokens]
    mine = torch.from_numpy(np.ascontiguousarray(x[cut[rank]:cut[rank + 1]]))
    ep = pkg.expert_parallel
    gu_l, lo, cnt = ep.shard_expert_blocks(gu, E, 2 * I, H, rank, world)
    dn_l, _, _ = ep.shard_expert_blocks(dn, E, H, I, rank, world)
    op = ep.AllToAllMoE(_OracleRowsEngine(router, np.ascontiguousarray(gu_l),
                                          np.ascontiguousarray(dn_l), cnt),
                        dist, rank, world, E)
    out = torch.zeros_like(mine)
    op.forward(mine, out)
    np.save(os.path.join(out_dir, f"a2a_{rank}.npy"), out.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("world,tokens", [(2, 5), (4, 11), (2, 1)])
def test_sequence_sharded_moe_all_to_all(tmp_path, world, tokens):
    """Tokens split over the ranks, rows sent to the experts' owners and back: the one-device
    result bit for bit under the reference's per-expert rule (an expert's owner sees all its
    rows), including a rank with no tokens."""
    port = 29500 + (os.getpid() + 313 * world + tokens) % 2000
    mp.spawn(_a2a_worker, args=(world, port, str(tmp_path), tokens), nprocs=world, join=True)
    router, gu, dn, _ = _moe_inputs()
    x = pkg.synth.activations(9, 40 + tokens, tokens, H)
    want = ol.moe_forward(x, router, TOPK, I, gu, dn, rule=ol.ACT_G32)[0]
    got = np.concatenate([np.load(tmp_path / f"a2a_{r}.npy") for r in range(world)])
    assert got.shape == want.shape
    assert got.tobytes() == want.tobytes()
