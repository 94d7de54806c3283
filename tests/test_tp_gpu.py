"""GPU parity of the tensor-parallel decode matmul (1..8 rows) whose all-gather is done by the kernels
(b2w4_matmul_tp + b2w4_tp_gather): the gathered row equals the unsharded b2w4_matmul and the
CPU oracle bit for bit.  The ranks of a group are emulated on one GPU as contexts that share
one stream (every matmul of an exchange is queued before the gathers, so no kernel ever waits
for another); peer pointers are then plain device pointers."""
import numpy as np
import pytest

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
pytestmark = pytest.mark.gpu


def _group(rank, world, stages):
    g = pkg.capi.TpGroup()
    g.rank, g.world = rank, world
    for p in range(world):
        g.stage_peers[p] = stages[p].data_ptr()
    return g


def _ranks(world, n):
    import torch
    ctxs = [pkg.capi.Context(0) for _ in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    for c in ctxs:
        c.set_stream(stream)
    stages = [torch.zeros(2 + 16 * n, dtype=torch.int64, device="cuda") for _ in range(world)]
    groups = [_group(r, world, stages) for r in range(world)]
    return ctxs, stages, groups


@pytest.mark.parametrize("world,n,k,m", [(1, 64, 256, 1), (2, 96, 384, 1), (2, 9728, 2560, 1),
                                          (4, 1024, 1024, 1), (3, 72, 128, 1),
                                          (8, 512, 640, 1), (2, 96, 384, 2), (2, 2560, 4096, 3),
                                          (4, 1024, 1024, 4), (2, 9728, 2560, 8),
                                          (8, 512, 640, 5)])
def test_gathered_rows_equal_unsharded_matmul(world, n, k, m):
    import torch
    blocks = pkg.synth.bg128_weight(11, 1, n, k)
    ctxs, stages, groups = _ranks(world, n)
    shards = []
    for r in range(world):
        sh, n_local, lo = pkg.shard.shard_blocks(blocks, n, k, r, world)
        shards.append((ctxs[r].upload_weight(sh, n_local, k), lo))
    whole = ctxs[0].upload_weight(blocks, n, k)
    rows = [torch.full((m, n), -3.0, dtype=torch.float32, device="cuda") for _ in range(world)]
    want = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    # several exchanges in a row: both halves of the staging buffer, and their reuse
    for it in range(5):
        x = pkg.synth.activations(20 + it, 0, m, k)
        xd = torch.from_numpy(x).cuda()
        ctxs[0].matmul(whole, xd, want)
        for r in range(world):
            ctxs[r].matmul_tp(shards[r][0], xd, n, shards[r][1], groups[r])
        for r in range(world):
            ctxs[r].tp_gather(groups[r], rows[r], n)
        for c in ctxs:
            c.sync()
        ref = ol.matmul_w4(blocks, n, k, x, rule=ol.ACT_G128)
        for r in range(world):
            assert torch.equal(rows[r], want), (it, r)
            assert np.array_equal(rows[r].cpu().numpy().view(np.uint32), ref.view(np.uint32))
            assert int(stages[r][0].item()) == it + 1  # completed exchanges
    for c in ctxs:
        c.close()


def test_activation_range_in_the_exchange():
    import torch
    world, n, k = 2, 256, 512
    blocks = pkg.synth.bg128_weight(12, 1, n, k)
    ctxs, stages, groups = _ranks(world, n)
    x = pkg.synth.activations(31, 0, 1, k)
    xd = torch.from_numpy(x).cuda()
    whole = ctxs[0].upload_weight(blocks, n, k)
    want = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    ctxs[0].matmul(whole, xd, want, act=pkg.capi.SILU)
    rows = [torch.zeros((1, n), dtype=torch.float32, device="cuda") for _ in range(world)]
    for r in range(world):
        sh, n_local, lo = pkg.shard.shard_blocks(blocks, n, k, r, world)
        w = ctxs[r].upload_weight(sh, n_local, k)
        ctxs[r].matmul_tp(w, xd, n, lo, groups[r], act=pkg.capi.SILU)
    for r in range(world):
        ctxs[r].tp_gather(groups[r], rows[r], n)
        ctxs[r].sync()
        assert torch.equal(rows[r], want)
    for c in ctxs:
        c.close()


def test_gather_without_a_peer_times_out_and_context_stays_usable():
    """A rank whose peer never stores (here: rank 1 of 2 is silent) gets B2W4_E_TIMEOUT from
    the bounded wait at the next sync, not a hang; the context then works again."""
    import torch
    n, k = 64, 256
    blocks = pkg.synth.bg128_weight(13, 1, n, k)
    ctxs, stages, groups = _ranks(2, n)
    sh, n_local, lo = pkg.shard.shard_blocks(blocks, n, k, 0, 2)
    w = ctxs[0].upload_weight(sh, n_local, k)
    xd = torch.from_numpy(pkg.synth.activations(5, 0, 1, k)).cuda()
    row = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    ctxs[0].set_peer_wait_ms(20)  # the default (about 2 s) covers host skew between ranks
    ctxs[0].matmul_tp(w, xd, n, lo, groups[0])
    ctxs[0].tp_gather(groups[0], row, n)
    with pytest.raises(pkg.capi.B200W4Error):
        ctxs[0].sync()
    # this rank's own columns arrived; the silent peer's are NaN, never stale values
    got = row.cpu().numpy()[0]
    assert np.isfinite(got[lo:lo + n_local]).all()
    missing = np.ones(n, dtype=bool)
    missing[lo:lo + n_local] = False
    assert np.isnan(got[missing]).all()
    with pytest.raises(pkg.capi.B200W4Error):
        ctxs[0].set_peer_wait_ms(0)
    whole = ctxs[0].upload_weight(blocks, n, k)
    y = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    ctxs[0].matmul(whole, xd, y)
    ctxs[0].sync()
    ref = ol.matmul_w4(blocks, n, k, pkg.synth.activations(5, 0, 1, k), rule=ol.ACT_G128)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    for c in ctxs:
        c.close()


def test_bad_arguments_are_refused():
    import torch
    n, k = 64, 256
    blocks = pkg.synth.bg128_weight(14, 1, n, k)
    ctxs, stages, groups = _ranks(1, n)
    ctx = ctxs[0]
    w = ctx.upload_weight(blocks, n, k)
    xd = torch.zeros((1, k), dtype=torch.float32, device="cuda")
    row = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.matmul_tp(w, xd, n - 8, 0, groups[0])  # the row is shorter than the shard
    with pytest.raises(pkg.capi.B200W4Error):  # at most 8 rows per exchange
        ctx.matmul_tp(w, torch.zeros((9, k), dtype=torch.float32, device="cuda"), n, 0, groups[0])
    bad = _group(0, 1, stages)
    bad.world = 9
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.matmul_tp(w, xd, n, 0, bad)
    empty = pkg.capi.TpGroup()
    empty.rank, empty.world = 0, 1
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.matmul_tp(w, xd, n, 0, empty)
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.tp_gather(empty, row, n)
    ctx.close()


@pytest.mark.parametrize("world,n,k,m,same_tiles", [(1, 256, 256, 1, False),
                                                     (2, 1024, 512, 1, False),
                                                     (4, 2048, 640, 3, False),
                                                     (8, 151936, 2560, 2, False),
                                                     (2, 4800, 512, 1, True),
                                                     (8, 4096, 256, 8, True)])
def test_tensor_parallel_greedy_token(world, n, k, m, same_tiles):
    """b2w4_matmul_argmax_tp + b2w4_tp_gather_token: every rank ends with the token that
    argmax_token picks over the oracle's full logits; with a weight made of one repeated
    8-row tile the equal maxima sit on different ranks and the lowest index must win."""
    import torch
    if same_tiles:
        blocks = np.tile(pkg.synth.bg128_weight(15, 1, 8, k), n // 8)
    else:
        blocks = pkg.synth.bg128_weight(15, 2, n, k)
    ctxs, stages, groups = _ranks(world, n)
    shards = []
    for r in range(world):
        sh, n_local, lo = pkg.shard.shard_blocks(blocks, n, k, r, world)
        shards.append((ctxs[r].upload_weight(np.ascontiguousarray(sh), n_local, k), lo))
    toks = [torch.full((m,), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    for it in range(3):
        x = pkg.synth.activations(60 + it, 0, m, k)
        xd = torch.from_numpy(x).cuda()
        ref = ol.matmul_w4(blocks, n, k, x, rule=ol.ACT_G128)
        want = [ol.argmax_token(ref[i]) for i in range(m)]
        if same_tiles:
            assert all(t < 8 for t in want)
        for r in range(world):
            ctxs[r].matmul_argmax_tp(shards[r][0], xd, shards[r][1], groups[r])
        for r in range(world):
            ctxs[r].tp_gather_token(groups[r], toks[r])
        for r in range(world):
            ctxs[r].sync()
            assert toks[r].cpu().tolist() == want, (it, r)
            assert int(stages[r][0].item()) == it + 1
    for c in ctxs:
        c.close()


def test_token_gather_with_a_silent_peer_times_out():
    import torch
    n, k = 256, 256
    blocks = pkg.synth.bg128_weight(16, 1, n, k)
    ctxs, stages, groups = _ranks(2, n)
    sh, n_local, lo = pkg.shard.shard_blocks(blocks, n, k, 0, 2)
    w = ctxs[0].upload_weight(np.ascontiguousarray(sh), n_local, k)
    tok = torch.zeros((1,), dtype=torch.int32, device="cuda")
    ctxs[0].set_peer_wait_ms(20)
    ctxs[0].matmul_argmax_tp(w, torch.from_numpy(pkg.synth.activations(6, 0, 1, k)).cuda(), lo,
                             groups[0])
    ctxs[0].tp_gather_token(groups[0], tok)
    with pytest.raises(pkg.capi.B200W4Error):
        ctxs[0].sync()
    assert int(tok.item()) == -1  # no token rather than a guess from one rank's maximum
    for c in ctxs:
        c.close()
