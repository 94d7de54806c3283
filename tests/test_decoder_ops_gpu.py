"""The operators between a decoder layer's matmuls (b2w4_rms_norm, b2w4_add_rms_norm,
b2w4_swiglu, b2w4_elementwise, b2w4_rope, b2w4_attention, b2w4_embed_rows) through the C ABI
against the CPU oracle, which is pinned bit for bit against the reference's own CPU operators
(tests/test_oracle_pins.py).  Element-wise arithmetic must be bit-exact; operators that sum
over a row (norms, attention scores, softmax) use tree reductions where the reference's loops
are sequential, and are held to the rounding error of a reassociated fp32 sum: 2e-6 relative
for the norms, 1e-5 relative L2 for attention."""
import numpy as np
import pytest

import oracle_lib as ol
from golden_util import rel_l2
from __graft_entry__ import load_package

pkg = load_package()
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    ol.set_exp_mode(True)  # the device takes exp in double and rounds once
    c = pkg.capi.Context(0)
    yield c
    c.close()
    ol.set_exp_mode(False)


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,dim", [(1, 2560), (7, 2560), (256, 2560), (64, 128), (5, 4096),
                                      (3, 200)])
def test_rms_norm(ctx, rows, dim):
    import torch
    rng = np.random.default_rng(rows * 1000 + dim)
    x = rng.normal(0, 1.7, (rows, dim)).astype(np.float32)
    w = rng.normal(1, 0.2, dim).astype(np.float32)
    out = torch.zeros((rows, dim), dtype=torch.float32, device="cuda")
    ctx.rms_norm(_dev(x), _dev(w), 1e-6, out)
    ctx.sync()
    want = ol.rms_norm(x, w, 1e-6)
    got = out.cpu().numpy()
    assert np.max(np.abs(got - want) / (np.abs(want) + 1e-30)) < 2e-6


def test_add_rms_norm_writes_the_sum_back(ctx):
    import torch
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (9, 2560)).astype(np.float32)
    u = rng.normal(0, 1, (9, 2560)).astype(np.float32)
    w = rng.normal(1, 0.2, 2560).astype(np.float32)
    res = _dev(x)
    out = torch.zeros((9, 2560), dtype=torch.float32, device="cuda")
    ctx.add_rms_norm(res, _dev(u), _dev(w), 1e-6, out)
    ctx.sync()
    want_res, want = ol.add_rms_norm(x, u, w, 1e-6)
    assert res.cpu().numpy().tobytes() == want_res.tobytes()  # one rounded add per element
    got = out.cpu().numpy()
    assert np.max(np.abs(got - want) / (np.abs(want) + 1e-30)) < 2e-6


def test_swiglu_add_mul_rope_embedding_are_bit_exact(ctx):
    import torch
    rng = np.random.default_rng(6)
    m = rng.normal(0, 2.5, (6, 2 * 9728)).astype(np.float32)
    out = torch.zeros((6, 9728), dtype=torch.float32, device="cuda")
    ctx.swiglu(_dev(m), out)
    a = rng.normal(0, 1, (4, 2560)).astype(np.float32)
    b = rng.normal(0, 1, (4, 2560)).astype(np.float32)
    s_add = torch.zeros((4, 2560), dtype=torch.float32, device="cuda")
    s_mul = torch.zeros((4, 2560), dtype=torch.float32, device="cuda")
    ctx.add(_dev(a), _dev(b), s_add)
    ctx.add(_dev(a), _dev(b), s_mul, multiply=True)
    q = rng.normal(0, 1, (5, 8, 128)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (5, 64)).astype(np.float32)
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    qd = _dev(q)
    r_out = torch.zeros_like(qd)
    ctx.rope(qd, r_out, 5, 8, 128, _dev(c), _dev(s), 128)
    r_part = torch.zeros_like(qd)
    ctx.rope(qd, r_part, 5, 8, 128, _dev(c[:, :32]), _dev(s[:, :32]), 64)  # rope_dim < dim
    ctx.rope(qd, qd, 5, 8, 128, _dev(c), _dev(s), 128)                     # in place
    table = rng.normal(0, 0.02, (1000, 256)).astype(np.float16)
    ids = np.array([3, 999, 0, 3], dtype=np.int32)
    emb = torch.zeros((4, 256), dtype=torch.float32, device="cuda")
    ctx.embed_rows(_dev(table.view(np.int16)), _dev(ids), emb)
    ctx.sync()
    assert out.cpu().numpy().tobytes() == ol.swiglu(m).tobytes()
    assert s_add.cpu().numpy().tobytes() == (a + b).tobytes()
    assert s_mul.cpu().numpy().tobytes() == (a * b).tobytes()
    assert r_out.cpu().numpy().tobytes() == ol.rope(q, c, s, 128).tobytes()
    assert r_part.cpu().numpy().tobytes() == ol.rope(q, c[:, :32], s[:, :32], 64).tobytes()
    assert qd.cpu().numpy().tobytes() == ol.rope(q, c, s, 128).tobytes()
    assert emb.cpu().numpy().tobytes() == table[ids].astype(np.float32).tobytes()


@pytest.mark.parametrize("tokens,past,heads,kv_heads", [(1, 37, 8, 2), (33, 0, 8, 2),
                                                        (5, 300, 32, 8), (1, 0, 4, 4)])
def test_attention_over_the_cache(ctx, tokens, past, heads, kv_heads):
    """Causal attention of new tokens over a cache that already holds `past` tokens: the new
    keys and values land at their positions (exact copies) and the output follows the x86
    reference's arithmetic (full-row softmax, P*V key by key)."""
    import torch
    dim, capacity = 128, 512
    rng = np.random.default_rng(tokens * 31 + past)
    k_hist = rng.normal(0, 1, (past, kv_heads, dim)).astype(np.float32)
    v_hist = rng.normal(0, 1, (past, kv_heads, dim)).astype(np.float32)
    q = rng.normal(0, 1, (tokens, heads, dim)).astype(np.float32)
    k = rng.normal(0, 1, (tokens, kv_heads, dim)).astype(np.float32)
    v = rng.normal(0, 1, (tokens, kv_heads, dim)).astype(np.float32)
    kc = np.zeros((kv_heads, capacity, dim), dtype=np.float32)
    vc = np.zeros((kv_heads, capacity, dim), dtype=np.float32)
    kc[:, :past] = k_hist.transpose(1, 0, 2)
    vc[:, :past] = v_hist.transpose(1, 0, 2)
    kcd, vcd = _dev(kc), _dev(vc)
    out = torch.zeros((tokens, heads, dim), dtype=torch.float32, device="cuda")
    scale = dim ** -0.5
    ctx.attention(_dev(q), _dev(k), _dev(v), kcd, vcd, out, tokens, heads, kv_heads, dim, past,
                  capacity, scale)
    ctx.sync()
    k_all = np.concatenate([k_hist, k])
    v_all = np.concatenate([v_hist, v])
    assert kcd.cpu().numpy()[:, :past + tokens].tobytes() == \
        np.ascontiguousarray(k_all.transpose(1, 0, 2)).tobytes()
    assert vcd.cpu().numpy()[:, :past + tokens].tobytes() == \
        np.ascontiguousarray(v_all.transpose(1, 0, 2)).tobytes()
    want = ol.causal_attention(q, k_all, v_all, heads, kv_heads, past, scale)
    assert rel_l2(out.cpu().numpy(), want) < 1e-5
    # the same call with the position read from device memory gives the same bits
    kcd2, vcd2 = _dev(kc), _dev(vc)
    out2 = torch.zeros_like(out)
    past_dev = torch.full((1,), past, dtype=torch.int32, device="cuda")
    ctx.attention(_dev(q), _dev(k), _dev(v), kcd2, vcd2, out2, tokens, heads, kv_heads, dim, 0,
                  capacity, scale, past_dev)
    ctx.sync()
    assert out2.cpu().numpy().tobytes() == out.cpu().numpy().tobytes()
    assert kcd2.cpu().numpy().tobytes() == kcd.cpu().numpy().tobytes()
    with pytest.raises(pkg.capi.B200W4Error):  # the cache is full
        ctx.attention(_dev(q), _dev(k), _dev(v), kcd, vcd, out, tokens, heads, kv_heads, dim,
                      capacity - tokens + 1, capacity, scale)


def test_position_on_the_device(ctx):
    """Rotary rows taken at first_position + t or at *position_dev + t agree with the oracle
    on those rows of the table; b2w4_advance records the token and moves the counter."""
    import torch
    rng = np.random.default_rng(11)
    q = rng.normal(0, 1, (3, 4, 64)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (40, 32)).astype(np.float32)
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    cd, sd, qd = _dev(c), _dev(s), _dev(q)
    a = torch.zeros_like(qd)
    b = torch.zeros_like(qd)
    pos = torch.full((1,), 17, dtype=torch.int32, device="cuda")
    ctx.rope(qd, a, 3, 4, 64, cd, sd, 64, 17)
    ctx.rope(qd, b, 3, 4, 64, cd, sd, 64, 0, pos)
    hist = torch.full((40,), -1, dtype=torch.int32, device="cuda")
    tok = torch.full((1,), 1234, dtype=torch.int32, device="cuda")
    ctx.advance(pos, 1, tok, hist)
    ctx.advance(pos, 2)
    ctx.sync()
    want = ol.rope(q, c[17:20], s[17:20], 64)
    assert a.cpu().numpy().tobytes() == want.tobytes()
    assert b.cpu().numpy().tobytes() == want.tobytes()
    assert int(pos.item()) == 20
    h = hist.cpu().numpy()
    assert h[17] == 1234 and (np.delete(h, 17) == -1).all()


@pytest.mark.parametrize("tokens,past,heads,kv_heads,dim", [(1, 9, 8, 2, 128), (7, 0, 4, 4, 64),
                                                            (3, 20, 2, 1, 256)])
def test_fused_qkv_step_equals_the_separate_operators(ctx, tokens, past, heads, kv_heads, dim):
    """b2w4_qkv_prepare (per-head norm + rotary embedding + cache append in one launch) leaves
    the same bits in q and in the caches as rms_norm, rope and the append of b2w4_attention
    run one after the other; attention without an append then gives the same output."""
    import torch
    capacity = 64
    rng = np.random.default_rng(dim + tokens)
    width = (heads + 2 * kv_heads) * dim
    qkv = rng.normal(0, 1, (tokens, width)).astype(np.float32)
    qw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (capacity, dim // 2)).astype(np.float32)
    c, s = _dev(np.cos(ang).astype(np.float32)), _dev(np.sin(ang).astype(np.float32))
    hist = rng.normal(0, 1, (2, kv_heads, capacity, dim)).astype(np.float32)
    qkv_d, qw_d, kw_d = _dev(qkv), _dev(qw), _dev(kw)
    scale = dim ** -0.5
    # operator by operator
    q = _dev(qkv[:, :heads * dim].reshape(tokens * heads, dim))
    k = _dev(qkv[:, heads * dim:(heads + kv_heads) * dim].reshape(tokens * kv_heads, dim))
    v = _dev(qkv[:, (heads + kv_heads) * dim:])
    kc1, vc1 = _dev(hist[0]), _dev(hist[1])
    out1 = torch.zeros((tokens, heads, dim), dtype=torch.float32, device="cuda")
    ctx.rms_norm(q, qw_d, 1e-6, q)
    ctx.rms_norm(k, kw_d, 1e-6, k)
    ctx.rope(q, q, tokens, heads, dim, c, s, dim, past)
    ctx.rope(k, k, tokens, kv_heads, dim, c, s, dim, past)
    ctx.attention(q, k, v, kc1, vc1, out1, tokens, heads, kv_heads, dim, past, capacity, scale)
    # fused, once with the position as an argument and once from device memory
    for past_dev in (None, torch.full((1,), past, dtype=torch.int32, device="cuda")):
        kc2, vc2 = _dev(hist[0]), _dev(hist[1])
        q2 = torch.zeros((tokens * heads, dim), dtype=torch.float32, device="cuda")
        out2 = torch.zeros_like(out1)
        arg_past = past if past_dev is None else 0
        ctx.qkv_prepare(qkv_d, tokens, heads, kv_heads, dim, qw_d, kw_d, 1e-6, c, s, arg_past, q2,
                        kc2, vc2, capacity, past_dev)
        ctx.attention(q2, None, None, kc2, vc2, out2, tokens, heads, kv_heads, dim, arg_past,
                      capacity, scale, past_dev)
        ctx.sync()
        assert q2.cpu().numpy().tobytes() == q.cpu().numpy().tobytes()
        assert kc2.cpu().numpy().tobytes() == kc1.cpu().numpy().tobytes()
        assert vc2.cpu().numpy().tobytes() == vc1.cpu().numpy().tobytes()
        assert out2.cpu().numpy().tobytes() == out1.cpu().numpy().tobytes()


@pytest.mark.parametrize("tokens,past,heads,kv_heads,dim", [(33, 0, 8, 2, 128),
                                                            (256, 0, 32, 8, 128),
                                                            (40, 100, 4, 4, 64),
                                                            (17, 5, 6, 2, 256),
                                                            (64, 300, 32, 4, 128)])
def test_tile_attention_equals_the_row_kernel(ctx, tokens, past, heads, kv_heads, dim):
    """A run of tokens takes the tile kernel (a block per kv head and tile of query tokens);
    it must leave the same bits as the one-row kernel, and agree with the oracle."""
    import os
    import torch
    os.environ["B2W4_ATTN"] = "row"
    try:
        ctx_row = pkg.capi.Context(0)
    finally:
        del os.environ["B2W4_ATTN"]
    capacity = past + tokens + 3
    rng = np.random.default_rng(tokens + dim)
    q = rng.normal(0, 1, (tokens, heads, dim)).astype(np.float32)
    k_all = rng.normal(0, 1, (past + tokens, kv_heads, dim)).astype(np.float32)
    v_all = rng.normal(0, 1, (past + tokens, kv_heads, dim)).astype(np.float32)
    kc = np.zeros((kv_heads, capacity, dim), dtype=np.float32)
    vc = np.zeros((kv_heads, capacity, dim), dtype=np.float32)
    kc[:, :past + tokens] = k_all.transpose(1, 0, 2)
    vc[:, :past + tokens] = v_all.transpose(1, 0, 2)
    kcd, vcd, qd = _dev(kc), _dev(vc), _dev(q)
    scale = dim ** -0.5
    outs = []
    for c, past_dev in ((ctx_row, None), (ctx, None),
                        (ctx, torch.full((1,), past, dtype=torch.int32, device="cuda"))):
        out = torch.zeros((tokens, heads, dim), dtype=torch.float32, device="cuda")
        c.attention(qd, None, None, kcd, vcd, out, tokens, heads, kv_heads, dim,
                    past if past_dev is None else 0, capacity, scale, past_dev)
        c.sync()
        outs.append(out.cpu().numpy())
    ctx_row.close()
    assert outs[1].tobytes() == outs[0].tobytes()
    assert outs[2].tobytes() == outs[0].tobytes()
    want = ol.causal_attention(q, k_all, v_all, heads, kv_heads, past, scale)
    assert rel_l2(outs[1], want) < 1e-5
