"""The list-of-GEMVs persistent kernel (b2w4_chain_*) through the C ABI: every op must give
the bits of the CPU oracle's one-row W4A8 chain (and therefore of b2w4_matmul), whether its
input comes from device memory or from an earlier op of the list, across the team sizes the
kernel picks (tiles per SM from a fraction to many), deep and shallow K, fp32 scale planes,
ragged N, fused activations, repeated runs of one chain, and the host-buffer entry point."""
import numpy as np
import pytest

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = pkg.capi.Context(0)
    yield c
    c.close()


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("n,k", [(264, 512), (1000, 1280), (9728, 2560), (2560, 4096),
                                 (320, 9728), (8, 128), (1181, 640), (19456, 2560)])
def test_single_op_matches_the_oracle(ctx, n, k):
    import torch
    blocks = pkg.synth.bg128_weight(20261125, 300 + n % 97, n, k)
    x = pkg.synth.activations(7, 300 + k % 89, 1, k)
    w = ctx.upload_weight(blocks, n, k)
    xd = torch.from_numpy(x).cuda()
    yd = torch.full((1, n), -1.0, dtype=torch.float32, device="cuda")
    chain = pkg.capi.Chain(ctx, [dict(w=w, x=xd, y=yd)])
    chain.run()
    ctx.sync()
    want = ol.matmul_w4(blocks, n, k, x)
    assert np.array_equal(_bits(yd.cpu().numpy()), _bits(want))
    chain.free()
    w.free()


def test_fp32_scale_plane_and_fused_activation(ctx):
    import torch
    n, k = 520, 768
    blocks = pkg.synth.bg128_weight(20261125, 311, n, k).copy()
    blocks.reshape(-1, 544)[:, :32].view(np.float32)[:] *= np.float32(1.0001)
    x = pkg.synth.activations(7, 311, 1, k)
    w = ctx.upload_weight(blocks, n, k)
    assert not w.scales_fp16
    xd = torch.from_numpy(x).cuda()
    yd = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    want_d = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    chain = pkg.capi.Chain(ctx, [dict(w=w, x=xd, y=yd, act=pkg.capi.SILU, act_begin=8,
                                      act_len=200)])
    chain.run()
    ctx.matmul(w, xd, want_d, act=pkg.capi.SILU, act_begin=8, act_len=200)
    ctx.sync()
    assert torch.equal(yd, want_d)
    plain = ol.matmul_w4(blocks, n, k, x)
    got = yd.cpu().numpy()
    assert np.array_equal(_bits(got[:, :8]), _bits(plain[:, :8]))
    assert np.array_equal(_bits(got[:, 208:]), _bits(plain[:, 208:]))
    chain.free()
    w.free()


def _dependent_chain(ctx, shapes, seed):
    """ops[i] reads the first K_i outputs of ops[i-1]; returns (chain, weights, x, outputs)."""
    import torch
    ws, ops, ys = [], [], []
    for i, (n, k) in enumerate(shapes):
        w = ctx.upload_weight(pkg.synth.bg128_weight(20261125, seed + i, n, k), n, k)
        ws.append(w)
        y = torch.full((1, n), -1.0, dtype=torch.float32, device="cuda")
        ys.append(y)
        last = i == len(shapes) - 1  # the last op writes the chain's own output only
        if i == 0:
            ops.append(dict(w=w, y=y))  # the chain's own input vector
        else:
            ops.append(dict(w=w, x_from=i - 1, x_offset=0, y=None if last else y))
    return pkg.capi.Chain(ctx, ops), ws, ys


def test_dependent_ops_match_one_by_one_matmuls(ctx):
    """A decoder-layer-like sequence (qkv, o, gate_up, down shapes of a 4B dense model) where
    each op consumes the head of its predecessor's output on the device; every intermediate
    row equals b2w4_matmul run op by op, bit for bit, on three runs of the same chain."""
    import torch
    shapes = [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728), (9728, 2560),
              (9728, 2560), (264, 2560)]
    chain, ws, ys = _dependent_chain(ctx, shapes, 400)
    x = pkg.synth.activations(7, 400, 1, shapes[0][1])
    xin = torch.from_numpy(x).cuda()
    for run in range(3):
        for y in ys:
            y.fill_(-1.0)
        torch.cuda.synchronize()
        assert chain.input_ptr
        y_host = np.zeros(shapes[-1][0], dtype=np.float32)
        chain.run_host(x.reshape(-1), y_host)
        cur = xin
        for i, (n, k) in enumerate(shapes):
            want = torch.zeros((1, n), dtype=torch.float32, device="cuda")
            ctx.matmul(ws[i], cur[:, :k].contiguous(), want)
            ctx.sync()
            if i < len(shapes) - 1:
                assert torch.equal(ys[i], want), f"run {run}, op {i}"
            cur = want
        assert np.array_equal(_bits(y_host), _bits(cur.cpu().numpy().reshape(-1)))
    chain.free()
    for w in ws:
        w.free()


def test_long_chain_of_the_benchmark_shape_and_oracle_at_the_end(ctx):
    """16 dependent GEMVs of the benchmark's shape on independent weights (every op's output
    grows by a factor of about five, which fp32 carries this far); the last row against the
    CPU oracle applied 16 times."""
    import torch
    n, k, depth = 9728, 2560, 16
    blocks = [pkg.synth.bg128_weight(20261125, 600 + i, n, k) for i in range(depth)]
    ws = [ctx.upload_weight(blocks[i], n, k) for i in range(depth)]
    ops = [dict(w=ws[0])] + [dict(w=ws[i], x_from=i - 1) for i in range(1, depth)]
    chain = pkg.capi.Chain(ctx, ops)
    x = pkg.synth.activations(7, 0, 1, k)
    y_host = np.zeros(n, dtype=np.float32)
    chain.run_host(x.reshape(-1), y_host)
    cur = x
    for i in range(depth):
        cur = ol.matmul_w4(blocks[i], n, k, cur[:, :k])
    assert np.isfinite(cur).all()
    assert np.array_equal(_bits(y_host), _bits(cur.reshape(-1)))
    chain.free()
    for w in ws:
        w.free()


def test_independent_ops_and_offsets(ctx):
    """Ops that share one device input (the batch form) and an op that reads a window in the
    middle of an earlier op's output."""
    import torch
    n, k = 1024, 512
    x = pkg.synth.activations(7, 500, 1, k)
    xd = torch.from_numpy(x).cuda()
    blocks = [pkg.synth.bg128_weight(20261125, 500 + i, n, k) for i in range(3)]
    ws = [ctx.upload_weight(b, n, k) for b in blocks]
    ys = [torch.zeros((1, n), dtype=torch.float32, device="cuda") for _ in range(3)]
    ops = [dict(w=ws[0], x=xd, y=ys[0]), dict(w=ws[1], x=xd, y=ys[1]),
           dict(w=ws[2], x_from=0, x_offset=256, y=ys[2])]
    chain = pkg.capi.Chain(ctx, ops)
    chain.run()
    ctx.sync()
    y0 = ol.matmul_w4(blocks[0], n, k, x)
    y1 = ol.matmul_w4(blocks[1], n, k, x)
    y2 = ol.matmul_w4(blocks[2], n, k, y0[:, 256:256 + k])
    for got, want in zip(ys, (y0, y1, y2)):
        assert np.array_equal(_bits(got.cpu().numpy()), _bits(want))
    chain.free()
    for w in ws:
        w.free()


def test_bad_lists_are_refused(ctx):
    n, k = 64, 256
    w = ctx.upload_weight(pkg.synth.bg128_weight(1, 1, n, k), n, k)
    with pytest.raises(pkg.capi.B200W4Error):
        pkg.capi.Chain(ctx, [dict(w=w, x_from=0)])            # reads itself
    with pytest.raises(pkg.capi.B200W4Error):
        pkg.capi.Chain(ctx, [dict(w=w), dict(w=w, x_from=0)])  # needs 256 of 64 outputs
    with pytest.raises(pkg.capi.B200W4Error):
        pkg.capi.Chain(ctx, [dict(w=w, act=9)])
    with pytest.raises(pkg.capi.B200W4Error):
        pkg.capi.Chain(ctx, [])
    w.free()


def _tp_rank_chains(world, shapes_full, x, seed):
    """The ranks of a tensor-parallel group as contexts on this one GPU: per rank its row
    shards of every weight, its scratch and its plain rows; every rank's chain stores into all
    ranks' buffers.  Ops all take the device vector x (no rank waits for another)."""
    import torch
    ctxs = [pkg.capi.Context(0) for _ in range(world)]
    blocks = [pkg.synth.bg128_weight(20261125, seed + i, n, k) for i, (n, k) in enumerate(shapes_full)]
    rows = [[torch.full((1, n), -1.0, dtype=torch.float32, device="cuda") for (n, k) in shapes_full]
            for _ in range(world)]
    tables, scratches = [], []
    for r in range(world):
        sh = []
        for i, (n, k) in enumerate(shapes_full):
            _, n_local, lo = pkg.shard.shard_blocks(blocks[i], n, k, r, world)
            sh.append((lo, n, [rows[p][i].data_ptr() for p in range(world)]))
        tables.append(pkg.capi.Chain.shard_table(sh))
    words = pkg.capi.Chain.scratch_words(tables[0])
    scratches = [torch.zeros((words,), dtype=torch.int64, device="cuda") for _ in range(world)]
    chains, keep = [], []
    for r in range(world):
        group = pkg.capi.TpGroup()
        group.rank, group.world = r, world
        for p in range(world):
            group.stage_peers[p] = scratches[p].data_ptr()
        ops = []
        for i, (n, k) in enumerate(shapes_full):
            shard, n_local, lo = pkg.shard.shard_blocks(blocks[i], n, k, r, world)
            w = ctxs[r].upload_weight(np.ascontiguousarray(shard), n_local, k)
            keep.append(w)
            ops.append(dict(w=w, x=x))
        chains.append(pkg.capi.Chain(ctxs[r], ops, tables[r], group))
    return ctxs, chains, rows, blocks, scratches, keep


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_list_rebuilds_full_rows_on_every_rank(world):
    import torch
    shapes = [(1024, 512), (2560, 512), (9728, 512)]
    x_np = pkg.synth.activations(7, 800, 1, 512)
    x = torch.from_numpy(x_np).cuda()
    ctxs, chains, rows, blocks, scratches, keep = _tp_rank_chains(world, shapes, x, 800)
    for run in range(2):
        for r in range(world):
            chains[r].run()
        for r in range(world):
            ctxs[r].sync()
        for i, (n, k) in enumerate(shapes):
            want = ol.matmul_w4(blocks[i], n, k, x_np)
            for r in range(world):
                assert np.array_equal(_bits(rows[r][i].cpu().numpy()), _bits(want)), (run, r, i)
            rows[0][i].fill_(-1.0) if run == 0 else None
    for c in chains:
        c.free()
    for w in keep:
        w.free()
    for c in ctxs:
        c.close()


def test_tensor_parallel_form_with_one_rank_and_dependent_ops(ctx):
    """world == 1 runs the peer-store epilogue and the scratch supplied by the caller with ops
    that consume earlier ops' rows (several ranks of such a list cannot share one GPU: they
    wait for one another)."""
    import torch
    shapes = [(1024, 512), (512, 1024), (264, 512)]
    blocks = [pkg.synth.bg128_weight(20261125, 820 + i, n, k) for i, (n, k) in enumerate(shapes)]
    ws = [ctx.upload_weight(b, n, k) for b, (n, k) in zip(blocks, shapes)]
    x_np = pkg.synth.activations(7, 820, 1, 512)
    x = torch.from_numpy(x_np).cuda()
    rows = [torch.full((1, n), -1.0, dtype=torch.float32, device="cuda") for (n, k) in shapes]
    table = pkg.capi.Chain.shard_table([(0, n, [rows[i].data_ptr()]) for i, (n, k) in enumerate(shapes)])
    scratch = torch.zeros((pkg.capi.Chain.scratch_words(table),), dtype=torch.int64, device="cuda")
    group = pkg.capi.TpGroup()
    group.rank, group.world = 0, 1
    group.stage_peers[0] = scratch.data_ptr()
    ops = [dict(w=ws[0], x=x), dict(w=ws[1], x_from=0), dict(w=ws[2], x_from=1)]
    chain = pkg.capi.Chain(ctx, ops, table, group)
    chain.run()
    ctx.sync()
    cur = x_np
    for i, (n, k) in enumerate(shapes):
        cur = ol.matmul_w4(blocks[i], n, k, cur[:, :k])
        assert np.array_equal(_bits(rows[i].cpu().numpy()), _bits(cur)), i
    with pytest.raises(pkg.capi.B200W4Error):  # plain rows of a sharded op go to y_peers
        pkg.capi.Chain(ctx, [dict(w=ws[0], x=x, y=rows[0])], table, group)
    chain.free()
    for w in ws:
        w.free()
