"""GPU parity of the routed MoE op (through the C ABI) against the CPU oracle and the
reference's golden routing vectors: expert indices exact, routing weights and outputs
bit-exact (tolerance fallback stated per test)."""
import numpy as np
import pytest

import oracle_lib as ol
from golden_util import case, rel_l2
from __graft_entry__ import load_package

pkg = load_package()
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    # The device takes exp in double and rounds once; the oracle is put in the same mode for
    # this module (its default, the host libm's expf, is what the pins against the reference
    # use; the two differ in the last bit for about 6 in 10000 arguments, which now and then
    # flips an int8 activation code of a SwiGLU row).
    ol.set_exp_mode(True)
    c = pkg.capi.Context(0)
    yield c
    c.close()
    ol.set_exp_mode(False)


@pytest.mark.parametrize("name", ["routes_small_k1", "routes_small_k2", "routes_small_k4",
                                  "routes_64x128_k8"])
def test_routing_matches_reference_vectors(ctx, name):
    import torch
    c = case(name)
    k = c["idx"].shape[1]
    lg = torch.from_numpy(c["logits"]).cuda()
    idx = torch.zeros(c["idx"].shape, dtype=torch.int32, device="cuda")
    w = torch.zeros(c["w"].shape, dtype=torch.float32, device="cuda")
    ctx.select_routes(lg, k, idx, w)
    ctx.sync()
    assert (idx.cpu().numpy() == c["idx"]).all()          # order and tie-break
    assert w.cpu().numpy().tobytes() == c["w"].tobytes()  # softmax over the selected


# The op's activation rule.  REF = the reference's: an expert that holds several rows quantises
# its activations per 32 values (kernels/moe.cpp:1055-1058 -> kernels/matmul_w4.cpp:1125-1154),
# a lone row per 128; the other setting applies per-128 to every row.
REF = ol.ACT_G32


def run_moe(ctx, hidden, router, top_k, inter, gu_blocks, dn_blocks, rule=REF):
    import torch
    ctx.set_moe_rule(rule)
    t, h = hidden.shape
    e = router.shape[0]
    gu = ctx.upload_weight(gu_blocks, e * 2 * inter, h)
    dn = ctx.upload_weight(dn_blocks, e * h, inter)
    xd = torch.from_numpy(hidden).cuda()
    rd = torch.from_numpy(router.view(np.int16)).cuda()
    out = torch.full((t, h), 3.0, dtype=torch.float32, device="cuda")
    logits = torch.zeros((t, e), dtype=torch.float32, device="cuda")
    idx = torch.zeros((t, top_k), dtype=torch.int32, device="cuda")
    w = torch.zeros((t, top_k), dtype=torch.float32, device="cuda")
    ctx.moe_forward(xd, rd, top_k, inter, gu, dn, out, logits, idx, w)
    ctx.sync()
    res = out.cpu().numpy(), logits.cpu().numpy(), idx.cpu().numpy(), w.cpu().numpy()
    gu.free()
    dn.free()
    return res


def check_against_oracle(got, want):
    """Router logits and expert indices bit-exact.  Routing weights: the device takes exp
    in fp64 and rounds once, the host oracle calls expf; the two may differ in the last bit,
    so weights are held to 1 ulp.  Where the weights are identical the output must be
    bit-exact; where a weight differs by an ulp the output is held to 1e-6 relative L2."""
    out, logits, idx, w = got
    o_out, o_logits, o_idx, o_w = want
    assert logits.tobytes() == o_logits.tobytes()
    assert (idx == o_idx).all()
    ulps = np.abs(w.view(np.int32).astype(np.int64) - o_w.view(np.int32).astype(np.int64))
    assert ulps.max() <= 1
    same = (ulps == 0).all(axis=1)
    assert out[same].tobytes() == o_out[same].tobytes()
    if not same.all():
        assert rel_l2(out[~same], o_out[~same]) < 1e-6


def test_small_golden_case(ctx):
    c = case("moe_small")
    t, h, e, top_k, inter = [int(v) for v in c["meta"]]
    router = c["router"].view(np.float16)
    got = run_moe(ctx, c["hidden"], router, top_k, inter, c["gate_up"], c["down"])
    want = ol.moe_forward(c["hidden"], router, top_k, inter, c["gate_up"], c["down"], rule=REF)
    check_against_oracle(got, want)
    # and inside the W4A8-vs-W4A32 gap of the reference's own op on this case
    assert rel_l2(got[0], c["out_ref_w4a32"]) < 3e-2


@pytest.mark.parametrize("t,h,e,top_k,inter", [(1, 256, 16, 4, 128), (7, 256, 16, 4, 256),
                                               (33, 512, 32, 8, 128), (64, 256, 8, 8, 128)])
def test_ragged_expert_groups(ctx, t, h, e, top_k, inter):
    """Experts with zero, one and many routes; top_k == experts (every expert hit by every
    token); one decode token."""
    hidden = pkg.synth.activations(7, t + h, t, h)
    router = pkg.synth.router_weight(20261125, e, e, h, std=0.3)
    gu = pkg.synth.bg128_weight(20261125, 100 + e, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 200 + e, e * h, inter)
    got = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
    want = ol.moe_forward(hidden, router, top_k, inter, gu, dn, rule=REF)
    counts = np.bincount(want[2].ravel(), minlength=e)
    if t < e and top_k < e:
        assert (counts == 0).any()
    check_against_oracle(got, want)


@pytest.mark.parametrize("t,h,e,top_k,inter", [(8, 256, 256, 8, 128), (9, 256, 64, 2, 128),
                                               (3, 128, 512, 16, 128), (5, 128, 1024, 4, 128),
                                               (4, 256, 8, 1, 256), (40, 128, 4, 4, 128)])
def test_routing_path_boundaries(ctx, t, h, e, top_k, inter):
    """Both sides of every switch in the op: 8 tokens (fused decode routing) and 9 (separate
    kernels), 4 tokens (decode grouped kernel, SwiGLU fused) and 5 (prefill kernel), expert
    counts of every logits-per-lane variant (128, 256, 512, 1024), top_k of 1 and of 16, and
    experts with more routes than one pass holds (40 tokens all on 4 experts)."""
    hidden = pkg.synth.activations(7, 900 + t + e, t, h)
    router = pkg.synth.router_weight(20261125, 700 + e, e, h, std=0.3)
    gu = pkg.synth.bg128_weight(20261125, 800 + e, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 900 + e, e * h, inter)
    got = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
    want = ol.moe_forward(hidden, router, top_k, inter, gu, dn, rule=REF)
    check_against_oracle(got, want)


def test_qwen3_30b_shaped_layer(ctx):
    """One Qwen3-30B-A3B-shaped MoE layer: hidden 2048, 128 experts, top-8, expert
    intermediate 768; 16 prompt tokens and 1 decode token."""
    h, e, top_k, inter = 2048, 128, 8, 768
    router = pkg.synth.router_weight(20261125, 1, e, h)
    gu = pkg.synth.bg128_weight(20261125, 2, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 3, e * h, inter)
    for t in (16, 1):
        hidden = pkg.synth.activations(7, 40 + t, t, h)
        got = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
        want = ol.moe_forward(hidden, router, top_k, inter, gu, dn, rule=REF)
        check_against_oracle(got, want)


def _expert_aggregate(tensor_id, experts, rows_per_expert, k, distinct=16):
    """BG128 aggregate [experts * rows_per_expert, k]: `distinct` experts are generated and
    the others are those blocks rotated by whole blocks (a different weight per expert, a
    fraction of the generation time of the full aggregate)."""
    base = pkg.synth.bg128_weight(20261125, tensor_id, distinct * rows_per_expert, k)
    per = base.size // distinct
    parts = []
    for e in range(experts):
        src = base[(e % distinct) * per:(e % distinct + 1) * per]
        parts.append(np.roll(src, 544 * (e // distinct)))
    return np.concatenate(parts)


def test_qwen3_30b_shaped_layer_256_tokens(ctx):
    """The prefill size the benchmark times: 256 tokens x 8 routes over 128 experts (about
    16 routes per expert, ragged), Qwen3-30B-A3B layer shape."""
    h, e, top_k, inter, t = 2048, 128, 8, 768, 256
    router = pkg.synth.router_weight(20261125, 1, e, h)
    gu = _expert_aggregate(2, e, 2 * inter, h)
    dn = _expert_aggregate(3, e, h, inter)
    hidden = pkg.synth.activations(7, 40 + t, t, h)
    got = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
    want = ol.moe_forward(hidden, router, top_k, inter, gu, dn, rule=REF)
    counts = np.bincount(want[2].ravel(), minlength=e)
    assert counts.max() > 16 and counts.min() < 16  # ragged groups on both sides of a pass
    check_against_oracle(got, want)


def test_qwen3_235b_shaped_layer(ctx):
    """One Qwen3-235B-A22B-shaped MoE layer: hidden 4096, 128 experts, top-8, expert
    intermediate 1536 (1.2 GB of expert weights); 16 prompt tokens and 1 decode token."""
    h, e, top_k, inter = 4096, 128, 8, 1536
    router = pkg.synth.router_weight(20261125, 5, e, h)
    gu = _expert_aggregate(6, e, 2 * inter, h, distinct=8)
    dn = _expert_aggregate(7, e, h, inter, distinct=8)
    for t in (16, 1):
        hidden = pkg.synth.activations(7, 60 + t, t, h)
        got = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
        want = ol.moe_forward(hidden, router, top_k, inter, gu, dn, rule=REF)
        check_against_oracle(got, want)


@pytest.mark.parametrize("t,h,e,top_k,inter", [(7, 256, 16, 4, 256), (33, 512, 32, 8, 128),
                                               (3, 128, 8, 4, 128)])
def test_per_128_rule_for_every_row(ctx, t, h, e, top_k, inter):
    """The other setting of the rule: per-128 whatever an expert holds (2..4 tokens then take
    the few-token kernels, SwiGLU fused into the down projection)."""
    hidden = pkg.synth.activations(7, 1200 + t, t, h)
    router = pkg.synth.router_weight(20261125, 1200 + e, e, h, std=0.3)
    gu = pkg.synth.bg128_weight(20261125, 1300 + e, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 1400 + e, e * h, inter)
    got = run_moe(ctx, hidden, router, top_k, inter, gu, dn, rule=ol.ACT_G128)
    want = ol.moe_forward(hidden, router, top_k, inter, gu, dn, rule=ol.ACT_G128)
    check_against_oracle(got, want)
    ctx.set_moe_rule(REF)


def test_bad_shapes_are_errors(ctx):
    import torch
    x = torch.zeros((2, 128), device="cuda")
    r = torch.zeros((4, 128), dtype=torch.int16, device="cuda")
    gu = ctx.upload_weight(pkg.synth.bg128_weight(1, 1, 4 * 2 * 128, 128), 4 * 2 * 128, 128)
    dn = ctx.upload_weight(pkg.synth.bg128_weight(1, 2, 4 * 128, 128), 4 * 128, 128)
    out = torch.zeros((2, 128), device="cuda")
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.moe_forward(x, r, 5, 128, gu, dn, out)      # top_k > experts
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.moe_forward(x, r, 2, 256, gu, dn, out)      # aggregates do not match I
    ctx.moe_forward(x, r, 2, 128, gu, dn, out)
    ctx.sync()
    assert (out.cpu().numpy() == 0).all()               # zero input -> zero output
    gu.free()
    dn.free()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("t,h,e,top_k,inter", [(1, 256, 16, 4, 128), (33, 512, 32, 8, 128),
                                               (16, 2048, 128, 8, 768)])
def test_expert_parallel_split_is_bit_identical(ctx, world, t, h, e, top_k, inter):
    """The expert-parallel halves of the op (b2w4_moe_expert_outputs per rank, sum of the
    route buffers, b2w4_moe_combine) against the one-device op and the oracle's route
    outputs.  The ranks of the group are run one after another on this GPU and their buffers
    summed with a plain add, which is what the all-reduce computes."""
    import torch
    ep = pkg.expert_parallel
    hidden = pkg.synth.activations(7, 300 + t, t, h)
    router = pkg.synth.router_weight(20261125, 50 + e, e, h, std=0.3)
    gu = pkg.synth.bg128_weight(20261125, 300 + e, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 400 + e, e * h, inter)
    one_dev = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
    xd = torch.from_numpy(hidden).cuda()
    rd = torch.from_numpy(router.view(np.int16)).cuda()
    total = torch.zeros((t * top_k, h), dtype=torch.float32, device="cuda")
    owners = np.zeros(t * top_k, dtype=np.int32)
    for rank in range(world):
        gu_l, lo, cnt = ep.shard_expert_blocks(gu, e, 2 * inter, h, rank, world)
        dn_l, _, _ = ep.shard_expert_blocks(dn, e, h, inter, rank, world)
        wg = ctx.upload_weight(np.ascontiguousarray(gu_l), cnt * 2 * inter, h)
        wd = ctx.upload_weight(np.ascontiguousarray(dn_l), cnt * h, inter)
        eng = ep.DeviceEngine(ctx, rd, wg, wd, top_k, inter, lo, cnt)
        routes, idx, w = eng.expert_outputs(xd)
        ctx.sync()
        assert (idx.cpu().numpy() == one_dev[2]).all()
        assert w.cpu().numpy().tobytes() == one_dev[3].tobytes()
        local = (one_dev[2].ravel() >= lo) & (one_dev[2].ravel() < lo + cnt)
        rows = routes.cpu().numpy()
        assert (rows[~local] == 0).all()                   # rows of other ranks stay zero
        owners += local
        total += routes
        wg.free()
        wd.free()
    assert (owners == 1).all()
    want_routes = ol.expert_route_outputs(hidden, one_dev[2], inter, gu, dn, e, rule=REF) \
        if t * top_k <= 64 else None
    if want_routes is not None:
        assert total.cpu().numpy().tobytes() == want_routes.tobytes()
    out = torch.full((t, h), 5.0, dtype=torch.float32, device="cuda")
    eng.combine(total, idx, w, out)
    ctx.sync()
    assert out.cpu().numpy().tobytes() == one_dev[0].tobytes()
    assert out.cpu().numpy().tobytes() == ol.moe_combine(total.cpu().numpy(), one_dev[2],
                                                         one_dev[3]).tobytes()


def test_expert_parallel_bad_range_is_error(ctx):
    import torch
    x = torch.zeros((2, 128), device="cuda")
    r = torch.zeros((4, 128), dtype=torch.int16, device="cuda")
    gu = ctx.upload_weight(pkg.synth.bg128_weight(1, 1, 2 * 2 * 128, 128), 2 * 2 * 128, 128)
    dn = ctx.upload_weight(pkg.synth.bg128_weight(1, 2, 2 * 128, 128), 2 * 128, 128)
    routes = torch.zeros((4, 128), device="cuda")
    idx = torch.zeros((2, 2), dtype=torch.int32, device="cuda")
    w = torch.zeros((2, 2), device="cuda")
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.moe_expert_outputs(x, r, 2, 128, gu, dn, 3, 2, routes, idx, w)   # experts 3..4 of 4
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.moe_expert_outputs(x, r, 2, 128, gu, dn, 0, 4, routes, idx, w)   # aggregates hold 2
    ctx.moe_expert_outputs(x, r, 2, 128, gu, dn, 2, 2, routes, idx, w)
    ctx.sync()
    gu.free()
    dn.free()


def _peer_group(rank, world, stages):
    g = pkg.capi.TpGroup()
    g.rank, g.world = rank, world
    for p in range(world):
        g.stage_peers[p] = stages[p].data_ptr()
    return g


@pytest.mark.parametrize("t,h,e,top_k,inter", [(1, 256, 8, 2, 128), (3, 128, 16, 4, 256),
                                                 (1, 2048, 128, 8, 768), (4, 256, 32, 8, 128),
                                                 (6, 128, 16, 4, 256), (33, 256, 8, 2, 128)])
def test_hand_over_inside_the_kernels_one_rank(ctx, t, h, e, top_k, inter):
    """b2w4_moe_forward_ep with a group of one (this rank owns every expert): the staged
    scatter + combine give b2w4_moe_forward's output bit for bit, over both halves of the
    staging buffer and their reuse; up to four tokens the rows are stored by the
    down-projection's own epilogue, beyond that by a scatter kernel.  (More ranks need more
    GPUs: one call both stores and waits, so ranks cannot be queued one after another on one
    device.)"""
    import torch
    ep = pkg.expert_parallel
    hidden = pkg.synth.activations(7, 500 + t, t, h)
    router = pkg.synth.router_weight(20261125, 60 + e, e, h, std=0.3)
    gu = pkg.synth.bg128_weight(20261125, 500 + e, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 600 + e, e * h, inter)
    want = run_moe(ctx, hidden, router, top_k, inter, gu, dn)
    rows = t * top_k + 3  # more staging rows than routes is allowed
    stage = torch.zeros(ep.PeerExchangeMoE.stage_words(rows, h), dtype=torch.int64, device="cuda")
    group = _peer_group(0, 1, [stage])
    wg = ctx.upload_weight(gu, e * 2 * inter, h)
    wd = ctx.upload_weight(dn, e * h, inter)
    xd = torch.from_numpy(hidden).cuda()
    rd = torch.from_numpy(router.view(np.int16)).cuda()
    op = ep.PeerExchangeMoE(ep.DeviceEngine(ctx, rd, wg, wd, top_k, inter, 0, e), group, rows)
    for it in range(4):
        out = torch.full((t, h), 9.0, dtype=torch.float32, device="cuda")
        op.forward(xd, out)
        ctx.sync()
        assert out.cpu().numpy().tobytes() == want[0].tobytes(), it
        assert int(stage[0].item()) == it + 1
    with pytest.raises(ValueError):
        ep.PeerExchangeMoE(op.engine, group, t * top_k - 1).forward(xd, out)
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.moe_forward_ep(xd, rd, top_k, inter, wg, wd, 0, e, group, t * top_k - 1, out)
    wg.free()
    wd.free()


def test_hand_over_with_a_silent_peer_times_out(ctx):
    """Rank 0 of 2 holds half the experts and its peer never stores: the combine's bounded
    wait runs out, the next sync reports the error, and the context works afterwards."""
    import torch
    ep = pkg.expert_parallel
    t, h, e, top_k, inter = 2, 128, 8, 4, 128
    hidden = pkg.synth.activations(7, 700, t, h)
    router = pkg.synth.router_weight(20261125, 70, e, h, std=0.3)
    gu = pkg.synth.bg128_weight(20261125, 700, e * 2 * inter, h)
    dn = pkg.synth.bg128_weight(20261125, 701, e * h, inter)
    gu_l, lo, cnt = ep.shard_expert_blocks(gu, e, 2 * inter, h, 0, 2)
    dn_l, _, _ = ep.shard_expert_blocks(dn, e, h, inter, 0, 2)
    wg = ctx.upload_weight(np.ascontiguousarray(gu_l), cnt * 2 * inter, h)
    wd = ctx.upload_weight(np.ascontiguousarray(dn_l), cnt * h, inter)
    rows = t * top_k
    stages = [torch.zeros(ep.PeerExchangeMoE.stage_words(rows, h), dtype=torch.int64,
                          device="cuda") for _ in range(2)]
    xd = torch.from_numpy(hidden).cuda()
    rd = torch.from_numpy(router.view(np.int16)).cuda()
    out = torch.zeros((t, h), dtype=torch.float32, device="cuda")
    ctx.set_peer_wait_ms(20)
    ctx.moe_forward_ep(xd, rd, top_k, inter, wg, wd, lo, cnt, _peer_group(0, 2, stages), rows,
                       out)
    with pytest.raises(pkg.capi.B200W4Error):
        ctx.sync()
    ctx.set_peer_wait_ms(2000)
    wg.free()
    wd.free()
    want = run_moe(ctx, hidden, router, top_k, inter, gu, dn)  # the context still works
    assert np.isfinite(want[0]).all()
