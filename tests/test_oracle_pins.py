"""Pins the CPU oracle (oracle/w4a8_oracle.c) against golden vectors produced by the
unmodified reference (tests/golden/make_golden.py) and, where oracle/_ref has been built,
against the reference library itself.  CPU only."""
import numpy as np
import pytest

import oracle_lib as ol
from golden_util import MATMUL_CASES, case, rel_l2


@pytest.mark.parametrize("name", MATMUL_CASES)
def test_block_layout_matches_reference_packer(name):
    c = case(name)
    mine = ol.bg128_encode(c["q"], c["scales"])
    assert mine.tobytes() == c["blocks"].tobytes()
    q, s = ol.bg128_decode(c["blocks"], *c["q"].shape)
    assert (q == c["q"]).all() and (s == c["scales"]).all()


@pytest.mark.parametrize("name", MATMUL_CASES)
def test_quantisers_bit_exact(name):
    c = case(name)
    e, o, s = ol.quantize_g128_even_odd(c["a"][0])
    assert (e == c["qa_even"]).all() and (o == c["qa_odd"]).all()
    assert s.tobytes() == c["a_scales_g128"].tobytes()
    q32, s32 = ol.quantize_g32(c["a"])
    assert (q32 == c["qa_g32"]).all()
    assert s32.tobytes() == c["a_scales_g32"].tobytes()


def test_quantiser_edge_cases():
    c = case("quant_edge")
    e, o, s = ol.quantize_g128_even_odd(c["x"])
    assert (e == c["even"]).all() and (o == c["odd"]).all()
    assert s.tobytes() == c["scales"].tobytes()
    assert s[0] == 1.0 and (e[:64] == 0).all()  # all-zero group: scale 1, codes 0


@pytest.mark.parametrize("name", MATMUL_CASES + ["synth_m5_k512_n72"])
def test_exact_product_matches_reference_x86(name):
    """The decode of the blocks and the per-group structure: exact fp64 product vs the
    reference's W4A32 kernel (fp32 summation noise only)."""
    c = case(name)
    if "q" in c:
        n, k = c["q"].shape
    else:
        n, k = 72, 512
    y = ol.matmul_w4(c["blocks"], n, k, c["a"], rule=ol.ACT_F64)
    assert rel_l2(y, c["y_ref_w4a32"]) < 1e-5


@pytest.mark.parametrize("name", MATMUL_CASES)
@pytest.mark.parametrize("rule", [ol.ACT_G128, ol.ACT_G32])
def test_w4a8_within_reference_test_tolerance(name, rule):
    """tests/test_matmul.cpp:884 holds the NEON W4A8 path to 5e-2 of the fp32 product on
    these inputs; the restatement must sit inside the same bound."""
    c = case(name)
    n, k = c["q"].shape
    y = ol.matmul_w4(c["blocks"], n, k, c["a"], rule=rule)
    exact = c["a"].astype(np.float64) @ (c["q"].astype(np.float64)
                                          * np.repeat(c["scales"], 128, axis=1)).T
    assert np.max(np.abs(y - exact)) < 5e-2


def test_group_sums_are_plain_integer_dots():
    c = case("synth_m5_k512_n72")
    n, k = 72, 512
    y, sums = ol.matmul_w4(c["blocks"], n, k, c["a"], want_sums=True)
    q, s = ol.bg128_decode(c["blocks"], n, k)
    for r in range(c["a"].shape[0]):
        qa, sa = ol.quantize_g128(c["a"][r])
        d = (q.astype(np.int64).reshape(n, k // 128, 128)
             * qa.astype(np.int64).reshape(1, k // 128, 128)).sum(-1)
        assert (sums[r] == d).all()
        # the fp32 chain, restated independently with numpy scalars
        acc = np.zeros(n, dtype=np.float32)
        for g in range(k // 128):
            sc = (s[:, g] * sa[g]).astype(np.float32)
            acc = (d[:, g].astype(np.float32).astype(np.float64) * sc.astype(np.float64)
                   + acc.astype(np.float64)).astype(np.float32)  # one rounding == fma
        assert acc.tobytes() == y[r].tobytes()


def test_int8_matrix_association_of_the_per32_rule():
    """The reference has two ARM kernels for several rows: the dot-product one (ACT_G32, what
    the GPU implements) and, on CPUs with int8 matrix instructions, one that first sums a
    group's four blocks with their activation scales and then applies the weight scale
    (kernels/matmul_w4_i8mm.cpp:100-121, 172-179).  Same integer sums, same scales, another
    association: restated independently here with numpy (a double product plus addend rounded
    once is the fma), equal to the first rule within fp32 rounding and not bit for bit."""
    c = case("synth_m5_k512_n72")
    n, k = 72, 512
    y32, sums = ol.matmul_w4(c["blocks"], n, k, c["a"], rule=ol.ACT_G32, want_sums=True)
    y_mm, sums_mm = ol.matmul_w4(c["blocks"], n, k, c["a"], rule=ol.ACT_G32_I8MM, want_sums=True)
    assert (sums == sums_mm).all()
    q, s = ol.bg128_decode(c["blocks"], n, k)
    for r in range(c["a"].shape[0]):
        sa = ol.quantize_g32(c["a"][r:r + 1])[1][0]
        acc = np.zeros(n, dtype=np.float32)
        for g in range(k // 128):
            t = np.zeros(n, dtype=np.float32)
            for b in range(4):
                d = sums[r][:, g * 4 + b].astype(np.float32).astype(np.float64)
                t = (d * np.float64(sa[g * 4 + b]) + t.astype(np.float64)).astype(np.float32)
            acc = (t.astype(np.float64) * s[:, g].astype(np.float64)
                   + acc.astype(np.float64)).astype(np.float32)
        assert acc.tobytes() == y_mm[r].tobytes()
    assert rel_l2(y_mm, y32) < 1e-6
    assert y_mm.tobytes() != y32.tobytes()


def test_fused_activation_range():
    c = case("synth_m5_k512_n72")
    y = ol.matmul_w4(c["blocks"], 72, 512, c["a"], rule=ol.ACT_F64)
    ya = ol.apply_activation(y.copy(), 1, 8, 40)
    assert rel_l2(ya, c["y_ref_silu_8_40"]) < 1e-5
    assert (ya[:, :8] == y[:, :8]).all() and (ya[:, 48:] == y[:, 48:]).all()


@pytest.mark.parametrize("name", ["routes_small_k1", "routes_small_k2", "routes_small_k4",
                                  "routes_64x128_k8"])
def test_routing_matches_reference(name):
    c = case(name)
    idx, w = ol.select_routes(c["logits"], c["idx"].shape[1])
    assert (idx == c["idx"]).all()
    assert w.tobytes() == c["w"].tobytes()


def test_routing_ties_pick_lowest_expert():
    c = case("routes_small_k4")
    assert list(c["idx"][1]) == [0, 1, 2, 3]      # all equal -> ids ascending
    assert list(c["idx"][0][:3]) == [1, 3, 5]     # three-way tie at 2.0


@pytest.mark.skipif(not ol.have_ref(), reason="reference library not built")
@pytest.mark.parametrize("kind", [0, 1, 2])
def test_routing_score_kinds_groups_bias_match_reference(kind):
    """select_moe_routes with the logistic and sqrt-softplus score kinds, a choice bias,
    expert groups (8 groups, 3 kept), with and without normalisation, a scaling factor, ties
    and large logits: indices and weights identical to the reference's, bit for bit."""
    rng = np.random.default_rng(40 + kind)
    logits = rng.normal(0, 2.5, (37, 64)).astype(np.float32)
    logits[3, 10:14] = logits[3, 10]        # ties inside a group
    logits[4] = 0.0                         # every expert equal
    logits[5, :8] = 60.0                    # exp(-x) underflows / softplus is linear
    logits[6, :8] = -60.0
    bias = rng.normal(0, 0.3, 64).astype(np.float32)
    for normalize in (True, False):
        for groups, kept in ((1, 1), (8, 3), (8, 8), (4, 1)):
            for b in (None, bias):
                got = ol.select_routes_ex(logits, 6, kind, normalize, groups, kept, 2.5, b)
                want = ol.select_routes_ex(logits, 6, kind, normalize, groups, kept, 2.5, b,
                                           which=ol.ref())
                assert (got[0] == want[0]).all(), (kind, normalize, groups, kept)
                assert got[1].tobytes() == want[1].tobytes(), (kind, normalize, groups, kept)


def test_moe_control_flow_matches_reference():
    c = case("moe_small")
    t, h, e, top_k, inter = [int(v) for v in c["meta"]]
    router = c["router"].view(np.float16)
    out, logits, idx, w = ol.moe_forward(c["hidden"], router, top_k, inter, c["gate_up"],
                                         c["down"], rule=ol.ACT_F64)
    assert rel_l2(out, c["out_ref_w4a32"]) < 1e-5
    # and the W4A8 rules stay within the W4A8-vs-W4A32 gap measured on this path
    for rule in (ol.ACT_G128, ol.ACT_G32):
        o8 = ol.moe_forward(c["hidden"], router, top_k, inter, c["gate_up"], c["down"],
                            rule=rule)[0]
        assert rel_l2(o8, c["out_ref_w4a32"]) < 3e-2


@pytest.mark.skipif(not ol.have_ref(), reason="oracle/_ref not built")
def test_live_reference_agrees_on_fresh_inputs():
    import sys, os
    sys.path.insert(0, os.path.join(ol.ROOT, "palm-infra_b200"))
    import synth
    n, k, m = 200, 1024, 3
    blocks = synth.bg128_weight(99, 1, n, k)
    a = synth.activations(98, 2, m, k)
    assert rel_l2(ol.matmul_w4(blocks, n, k, a, rule=ol.ACT_F64),
                  ol.ref_matmul(blocks, n, k, a, threads=4)) < 1e-5
    for r in range(m):
        mine = ol.quantize_g128_even_odd(a[r])
        theirs = ol.ref_quantize_g128_even_odd(a[r])
        assert all((x == y).all() for x, y in zip(mine, theirs))
    q32, s32 = ol.quantize_g32(a)
    rq32, rs32 = ol.ref_quantize_g32(a)
    assert (q32 == rq32).all() and (s32 == rs32).all()


def _argmax_rows():
    rng = np.random.default_rng(77)
    rows = [rng.standard_normal(n).astype(np.float32) for n in (1, 2, 3, 4, 5, 7, 8, 100, 4097)]
    tie = np.zeros(64, dtype=np.float32)
    tie[[9, 17, 40]] = 3.5                       # equal maxima: the first wins
    neg0 = np.full(16, -1.0, dtype=np.float32)
    neg0[5], neg0[11] = -0.0, 0.0                # -0 == +0: the first wins
    nan_mid = rng.standard_normal(40).astype(np.float32)
    nan_mid[[3, 20]] = np.nan                    # a NaN never beats a number
    nan_mid[30] = 10.0
    nan_first = rng.standard_normal(40).astype(np.float32)
    nan_first[0] = np.nan                        # ... but nothing beats a NaN at index 0
    infs = np.array([-np.inf, np.nan, -np.inf, np.inf, np.inf], dtype=np.float32)
    all_ninf = np.full(9, -np.inf, dtype=np.float32)
    return rows + [tie, neg0, nan_mid, nan_first, infs, all_ninf]


def test_argmax_oracle_cases():
    """The scalar rule of argmax_token (engine/sampler.cpp:72-77) on its corner cases."""
    want = [None] * 9 + [9, 5, None, 0, 3, 0]
    for row, w in zip(_argmax_rows(), want):
        got = ol.argmax_token(row)
        if w is None:
            clean = np.where(np.isnan(row), -np.inf, row)
            w = int(np.argmax(clean))            # numpy: first maximum
        assert got == w


@pytest.mark.skipif(not ol.have_ref(), reason="oracle/_ref not built")
def test_argmax_oracle_equals_reference_sampler():
    """Pinned against the reference's own greedy sampling entry (temperature 0)."""
    for row in _argmax_rows():
        assert ol.argmax_token(row) == ol.ref_greedy_token(row)


def test_argmax_oracle_matches_golden_tokens():
    """The committed vectors hold the reference's greedy tokens (sample_token at temperature 0)
    for rows with ties, signed zeros, NaNs and infinities."""
    want = case("greedy_token")["tokens"]
    for i, w in enumerate(want):
        assert ol.argmax_token(case("greedy_token")[f"row{i}"]) == int(w), i
    assert int(want[9]) == 30 and int(want[10]) == 0  # a NaN loses, except at index 0


def test_exp_modes_differ_by_at_most_one_ulp():
    """The oracle's two ways of taking exp of a float -- the host libm's expf (default: what the
    reference built here computes) and double-then-round (what the GPU kernels compute) --
    agree to one unit in the last place, on SiLU arguments and on softmax differences."""
    x = np.concatenate([np.linspace(-20, 20, 40001), np.random.default_rng(3).normal(0, 3, 20000)])
    x = x.astype(np.float32).reshape(1, -1)
    try:
        ol.set_exp_mode(False)
        a = ol.apply_activation(x.copy(), 1)
        ol.set_exp_mode(True)
        b = ol.apply_activation(x.copy(), 1)
    finally:
        ol.set_exp_mode(False)
    ulps = np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))
    assert ulps.max() <= 2  # one ulp of exp moves the quotient by at most two
    assert (ulps != 0).mean() < 5e-3


@pytest.mark.skipif(not ol.have_ref(), reason="reference library not built")
def test_decoder_layer_operators_match_the_reference_bit_for_bit():
    """The C restatements of RMSNorm, add + RMSNorm, SwiGLU, rotary embedding and the x86
    attention head against the reference's own CPU operators (live, oracle/_ref), same inputs,
    identical bits -- including the attention's two-accumulator dot product and the order of
    its 16-lane reduction."""
    rng = np.random.default_rng(11)
    x = rng.normal(0, 1.5, (5, 2560)).astype(np.float32)
    w = rng.normal(1, 0.1, 2560).astype(np.float32)
    assert ol.rms_norm(x, w, 1e-6).tobytes() == ol.rms_norm(x, w, 1e-6, ol.ref()).tobytes()
    u = rng.normal(0, 1, (5, 2560)).astype(np.float32)
    r0, o0 = ol.add_rms_norm(x, u, w, 1e-6)
    r1, o1 = ol.add_rms_norm(x, u, w, 1e-6, ol.ref())
    assert r0.tobytes() == r1.tobytes() and o0.tobytes() == o1.tobytes()
    m = rng.normal(0, 2, (3, 2 * 1000)).astype(np.float32)
    assert ol.swiglu(m).tobytes() == ol.swiglu(m, ol.ref()).tobytes()
    q = rng.normal(0, 1, (4, 6, 128)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (4, 64)).astype(np.float32)
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    assert ol.rope(q, c, s, 128).tobytes() == ol.rope(q, c, s, 128, ol.ref()).tobytes()
    part = ol.rope(q[:, :, :96].copy(), c[:, :32], s[:, :32], 64)  # rope_dim < dim
    assert part.tobytes() == ol.rope(q[:, :, :96].copy(), c[:, :32], s[:, :32], 64,
                                     ol.ref()).tobytes()
    for dim in (128, 80):  # 80: a 16-lane step and a scalar tail in the dot product
        qq = rng.normal(0, 1, (7, dim)).astype(np.float32)
        kk = rng.normal(0, 1, (19, dim)).astype(np.float32)
        vv = rng.normal(0, 1, (19, dim)).astype(np.float32)
        mask = np.zeros((7, 19), dtype=np.float32)
        for t in range(7):
            mask[t, 12 + t + 1:] = -np.inf
        a = ol.sdpa_head(qq, kk, vv, dim ** -0.5, mask)
        b = ol.sdpa_head(qq, kk, vv, dim ** -0.5, mask, ol.ref())
        assert a.tobytes() == b.tobytes()
