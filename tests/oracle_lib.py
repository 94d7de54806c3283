"""ctypes bindings of the CPU oracle (oracle/w4a8_oracle.c) and, when it has been
built, of the unmodified reference library (oracle/_ref).  Test infrastructure only.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle_w4a8.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libref_shim.so")

ACT_G128, ACT_G32, ACT_F64 = 128, 32, 0
ACT_G32_I8MM = 33  # the per-32 rule as ARM's int8-matrix kernels associate it (oracle only)
BLOCK_BYTES = 544


def _ptr(a, t=C.c_void_p):
    return a.ctypes.data_as(t) if a is not None else None


def build_oracle():
    src = os.path.join(ORACLE_DIR, "w4a8_oracle.c")
    if (not os.path.exists(ORACLE_SO)
            or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src)):
        subprocess.check_call(["make", "-s", "-C", ORACLE_DIR, "oracle"])


_oracle = None


def oracle():
    global _oracle
    if _oracle is None:
        build_oracle()
        lib = C.CDLL(ORACLE_SO)
        lib.orc_bg128_bytes.restype = C.c_size_t
        lib.orc_fp16_to_fp32.restype = C.c_float
        _oracle = lib
    return _oracle


def have_ref():
    return os.path.exists(REF_SO)


_ref = None


def ref():
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_SO)
        lib.ref_isa_name.restype = C.c_char_p
        lib.ref_time_matmul_bg128.restype = C.c_double
        _ref = lib
    return _ref


def ref_engine_generate(package_path, prompt, steps, vocab, w4a8=False, n_ctx=256):
    """The reference's CPU engine (LLMEngine, greedy) on a .mollm package: (tokens, logits of
    the prompt's last position).  w4a8: its INT4 matmuls are answered at the provider seam by
    the oracle's W4A8 arithmetic under the reference's rule per row count (what its ARM build
    computes); everything else stays the reference's code (oracle/ref_shim.cpp)."""
    lib = ref()
    lib.ref_set_w4a8_provider(1 if w4a8 else 0)
    ids = np.asarray(prompt, dtype=np.int32)
    tokens = np.zeros(steps, dtype=np.int32)
    logits = np.zeros(vocab, dtype=np.float32)
    try:
        rc = lib.ref_engine_generate(str(package_path).encode(), _ptr(ids), len(ids), steps,
                                     n_ctx, 1, _ptr(tokens), _ptr(logits), vocab)
    finally:
        lib.ref_set_w4a8_provider(0)
    assert rc == 0, rc
    return tokens.tolist(), logits


# ---------------------------------------------------------------- oracle calls

def set_exp_mode(correctly_rounded):
    """How the oracle takes exp of a float: False = the host libm's expf (the reference built
    on this host; the default, used by the pins against the reference), True = in double,
    rounded once (what the GPU kernels do; independent of the host's libm).  The two differ in
    the last bit for about 6 in 10000 arguments."""
    oracle().orc_set_exp_mode(1 if correctly_rounded else 0)


def bg128_bytes(n, k):
    return ((n + 7) // 8) * (k // 128) * BLOCK_BYTES


def bg128_encode(q, scales):
    """q int8 [N,K] in [-8,7], scales fp32 [N,K/128] -> uint8 blocks."""
    n, k = q.shape
    q = np.ascontiguousarray(q, dtype=np.int8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    out = np.zeros(bg128_bytes(n, k), dtype=np.uint8)
    oracle().orc_bg128_encode(_ptr(q), _ptr(scales), n, k, _ptr(out))
    return out


def bg128_decode(blocks, n, k):
    q = np.zeros((n, k), dtype=np.int8)
    s = np.zeros((n, k // 128), dtype=np.float32)
    oracle().orc_bg128_decode(_ptr(blocks), n, k, _ptr(q), _ptr(s))
    return q, s


def quantize_g128(x):
    k = x.shape[-1]
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.zeros(k, dtype=np.int8)
    s = np.zeros(k // 128, dtype=np.float32)
    oracle().orc_quantize_a_g128(_ptr(x), k, _ptr(q), _ptr(s))
    return q, s


def quantize_g128_even_odd(x):
    k = x.shape[-1]
    x = np.ascontiguousarray(x, dtype=np.float32)
    e = np.zeros(k // 2, dtype=np.int8)
    o = np.zeros(k // 2, dtype=np.int8)
    s = np.zeros(k // 128, dtype=np.float32)
    oracle().orc_quantize_a_g128_even_odd(_ptr(x), k, _ptr(e), _ptr(o), _ptr(s))
    return e, o, s


def quantize_g32(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    q = np.zeros((m, k), dtype=np.int8)
    s = np.zeros((m, k // 32), dtype=np.float32)
    oracle().orc_quantize_a_g32(_ptr(x), m, k, k, _ptr(q), _ptr(s))
    return q, s


def matmul_w4(blocks, n, k, x, rule=ACT_G128, want_sums=False):
    """x fp32 [M,K] -> y fp32 [M,N] (and int32 group sums when asked)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    sums = None
    if want_sums:
        per = k // 128 if rule == ACT_G128 else k // 32
        sums = np.zeros((m, n, per), dtype=np.int32)
    rc = oracle().orc_matmul_w4(_ptr(blocks), n, k, _ptr(x), m, k, _ptr(y), n, rule,
                                _ptr(sums))
    assert rc == 0, rc
    return (y, sums) if want_sums else y


def apply_activation(y, act, begin=0, length=-1):
    y = np.ascontiguousarray(y, dtype=np.float32)
    m, n = y.shape
    oracle().orc_apply_activation(_ptr(y), m, n, n, act, begin, length)
    return y


def select_routes(logits, top_k):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    t, e = logits.shape
    idx = np.zeros((t, top_k), dtype=np.int32)
    w = np.zeros((t, top_k), dtype=np.float32)
    rc = oracle().orc_moe_select_routes_softmax(_ptr(logits), t, e, top_k, _ptr(idx),
                                                _ptr(w))
    assert rc == 0
    return idx, w


def moe_forward(hidden, router_fp16, top_k, intermediate, gate_up, down, rule=ACT_G128):
    hidden = np.ascontiguousarray(hidden, dtype=np.float32)
    t, h = hidden.shape
    e = router_fp16.shape[0]
    router_fp16 = np.ascontiguousarray(router_fp16.view(np.uint16))
    out = np.zeros((t, h), dtype=np.float32)
    logits = np.zeros((t, e), dtype=np.float32)
    idx = np.zeros((t, top_k), dtype=np.int32)
    w = np.zeros((t, top_k), dtype=np.float32)
    rc = oracle().orc_moe_forward(_ptr(hidden), t, h, h, _ptr(router_fp16), e, top_k,
                                  intermediate, _ptr(gate_up), _ptr(down), _ptr(out), h,
                                  rule, _ptr(logits), _ptr(idx), _ptr(w))
    assert rc == 0, rc
    return out, logits, idx, w


def router_logits(hidden, router_fp16):
    hidden = np.ascontiguousarray(hidden, dtype=np.float32)
    t, h = hidden.shape
    e = router_fp16.shape[0]
    router_fp16 = np.ascontiguousarray(router_fp16.view(np.uint16))
    logits = np.zeros((t, e), dtype=np.float32)
    oracle().orc_router_logits(_ptr(hidden), t, h, h, _ptr(router_fp16), e, _ptr(logits))
    return logits


def moe_combine(route_out, idx, w):
    t, top_k = idx.shape
    route_out = np.ascontiguousarray(route_out, dtype=np.float32)
    h = route_out.shape[1]
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.zeros((t, h), dtype=np.float32)
    oracle().orc_moe_combine(_ptr(route_out), t, h, top_k, _ptr(idx), _ptr(w), _ptr(out), h)
    return out


def expert_route_outputs(hidden, idx, intermediate, gate_up, down, experts, lo=0, hi=None,
                         rule=ACT_G128):
    """Per-route expert outputs [tokens*top_k, H] from the oracle's pieces, for the routes
    whose expert lies in [lo, hi); zeros elsewhere.  gate_up / down hold all `experts`.
    rule == ACT_G32: the reference's rule -- an expert's rows go through its matmuls together,
    per-32 activation scales when it holds several, per-128 when it holds one."""
    hidden = np.ascontiguousarray(hidden, dtype=np.float32)
    t, h = hidden.shape
    top_k = idx.shape[1]
    hi = experts if hi is None else hi
    gu_bytes = bg128_bytes(2 * intermediate, h)
    dn_bytes = bg128_bytes(h, intermediate)
    out = np.zeros((t * top_k, h), dtype=np.float32)
    for e in range(lo, hi):
        where = [(tok, j) for tok in range(t) for j in range(top_k) if int(idx[tok, j]) == e]
        if not where:
            continue
        r = ACT_G32 if rule == ACT_G32 and len(where) >= 2 else ACT_G128
        rows = np.ascontiguousarray(hidden[[tok for tok, _ in where]])
        gu = matmul_w4(gate_up[e * gu_bytes:(e + 1) * gu_bytes], 2 * intermediate, h, rows,
                       rule=r)
        gate = apply_activation(gu[:, :intermediate].copy(), 1)  # g * 1/(1+expf(-g))
        inter = (gate * gu[:, intermediate:]).astype(np.float32)
        y = matmul_w4(down[e * dn_bytes:(e + 1) * dn_bytes], h, intermediate, inter, rule=r)
        for i, (tok, j) in enumerate(where):
            out[tok * top_k + j] = y[i]
    return out


# ------------------------------------------------------------- reference calls

def ref_quantize_g128_even_odd(x):
    k = x.shape[-1]
    x = np.ascontiguousarray(x, dtype=np.float32)
    e = np.zeros(k // 2, dtype=np.int8)
    o = np.zeros(k // 2, dtype=np.int8)
    s = np.zeros(k // 128, dtype=np.float32)
    ref().ref_quantize_a_q8_g128_even_odd(_ptr(x), k, _ptr(e), _ptr(o), _ptr(s))
    return e, o, s


def ref_quantize_g32(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    q = np.zeros((m, k), dtype=np.int8)
    s = np.zeros((m, k // 32), dtype=np.float32)
    ref().ref_quantize_a_q8_blocks(_ptr(x), m, k, k, _ptr(q), _ptr(s))
    return q, s


def ref_pack_bg128(q, scales):
    """Through the reference's own packers: row-major nibbles -> q4dot -> BG128."""
    n, k = q.shape
    nib = (q.astype(np.int16) & 15).astype(np.uint8)
    rowmajor = np.ascontiguousarray(nib[:, 0::2] | (nib[:, 1::2] << 4))
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    out = np.zeros(bg128_bytes(n, k), dtype=np.uint8)
    rc = ref().ref_pack_bg128(_ptr(rowmajor), _ptr(scales), n, k, _ptr(out))
    assert rc == 0, rc
    return out


def ref_matmul(blocks, n, k, x, act=0, begin=0, length=-1, threads=1):
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    ref().ref_matmul_bg128(_ptr(x), m, k, k, _ptr(blocks), n, _ptr(y), n, act, begin,
                           length, threads)
    return y


def select_routes_ex(logits, top_k, score_kind, normalize=True, groups=1, topk_groups=1,
                     scaling=1.0, bias=None, which=None):
    """Routing with every parameter of the reference (kernels/moe_routing.h:8-16); `which` =
    ref() runs the reference's own select_moe_routes."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    t, e = logits.shape
    idx = np.zeros((t, top_k), dtype=np.int32)
    w = np.zeros((t, top_k), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    fn = (which.ref_select_moe_routes_ex if which is not None
          else oracle().orc_moe_select_routes)
    rc = fn(_ptr(logits), t, e, top_k, score_kind, 1 if normalize else 0, groups, topk_groups,
            C.c_float(scaling), _ptr(b), _ptr(idx), _ptr(w))
    assert rc == 0, rc
    return idx, w


def ref_select_routes(logits, top_k):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    t, e = logits.shape
    idx = np.zeros((t, top_k), dtype=np.int32)
    w = np.zeros((t, top_k), dtype=np.float32)
    rc = ref().ref_select_moe_routes(_ptr(logits), t, e, top_k, 0, 1, _ptr(idx), _ptr(w))
    assert rc == 0
    return idx, w


def ref_moe(hidden, router_fp16, top_k, intermediate, gate_up, down, threads=1):
    hidden = np.ascontiguousarray(hidden, dtype=np.float32)
    t, h = hidden.shape
    e = router_fp16.shape[0]
    router_fp16 = np.ascontiguousarray(router_fp16.view(np.uint16))
    out = np.zeros((t, h), dtype=np.float32)
    rc = ref().ref_moe_bg128(_ptr(hidden), t, h, _ptr(router_fp16), e, top_k,
                             intermediate, _ptr(gate_up), _ptr(down), _ptr(out), threads)
    assert rc == 0
    return out


def argmax_token(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return int(oracle().orc_argmax_token(_ptr(logits), logits.size))


def ref_greedy_token(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return int(ref().ref_greedy_token(_ptr(logits), logits.size))


# ------------------------------------------- operators between a decoder layer's matmuls
# which = oracle() (the C restatement) or ref() (the reference's own CPU operators); the two
# libraries export the same signatures under the prefixes orc_ / ref_.

def _dec(which, name):
    return getattr(which, ("orc_" if which is oracle() else "ref_") + name)


def rms_norm(x, weight, eps, which=None):
    which = which or oracle()
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.zeros_like(x)
    _dec(which, "rms_norm")(_ptr(x), x.shape[0], x.shape[1], _ptr(w), C.c_float(eps), _ptr(out))
    return out


def add_rms_norm(residual, update, weight, eps, which=None):
    """Returns (new residual, normalised output)."""
    which = which or oracle()
    r = np.array(residual, dtype=np.float32, order="C")
    u = np.ascontiguousarray(update, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.zeros_like(r)
    _dec(which, "add_rms_norm")(_ptr(r), _ptr(u), r.shape[0], r.shape[1], _ptr(w),
                                 C.c_float(eps), _ptr(out))
    return r, out


def swiglu(merged, which=None):
    which = which or oracle()
    m = np.ascontiguousarray(merged, dtype=np.float32)
    out = np.zeros((m.shape[0], m.shape[1] // 2), dtype=np.float32)
    _dec(which, "swiglu")(_ptr(m), m.shape[0], m.shape[1] // 2, _ptr(out))
    return out


def rope(x, cosv, sinv, rope_dim, which=None):
    """x [tokens, heads, dim]; cos / sin [tokens, rope_dim // 2]."""
    which = which or oracle()
    x = np.ascontiguousarray(x, dtype=np.float32)
    c = np.ascontiguousarray(cosv, dtype=np.float32)
    s = np.ascontiguousarray(sinv, dtype=np.float32)
    out = np.zeros_like(x)
    _dec(which, "rope")(_ptr(x), x.shape[0], x.shape[1], x.shape[2], _ptr(c), _ptr(s), rope_dim,
                        _ptr(out))
    return out


def sdpa_head(q, k, v, scale, mask=None, which=None):
    """One head: q [q_tokens, dim], k / v [k_tokens, dim], mask [q_tokens, k_tokens] or None."""
    which = which or oracle()
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    m = None if mask is None else np.ascontiguousarray(mask, dtype=np.float32)
    out = np.zeros((q.shape[0], v.shape[1]), dtype=np.float32)
    _dec(which, "sdpa_head")(_ptr(q), _ptr(k), _ptr(v), _ptr(out), q.shape[0], k.shape[0],
                             q.shape[1], v.shape[1], C.c_float(scale), _ptr(m))
    return out


def causal_attention(q, k_all, v_all, heads, kv_heads, past, scale, which=None):
    """q [tokens, heads, dim]; k_all / v_all [past + tokens, kv_heads, dim]: token t sees keys
    0 .. past + t.  The reference graph expresses that with an additive mask whose invisible
    tail is -inf (engine/input_prep.cpp:8-16), which its kernel trims
    (kernels/attention_x86_avx512.cpp:59-66)."""
    tokens, _, dim = q.shape
    total = k_all.shape[0]
    mask = np.zeros((tokens, total), dtype=np.float32)
    for t in range(tokens):
        mask[t, past + t + 1:] = -np.inf
    out = np.zeros((tokens, heads, dim), dtype=np.float32)
    for h in range(heads):
        kvh = h // (heads // kv_heads)
        out[:, h] = sdpa_head(q[:, h], k_all[:, kvh], v_all[:, kvh], scale, mask, which)
    return out


def set_moe_host_build(x86_avx512):
    """Which build of the reference the MoE operator's router dot product and weighted output
    sum follow: False = the ARM reading the GPU implements, True = the x86 AVX-512 build."""
    oracle().orc_set_moe_host_build(1 if x86_avx512 else 0)


def rope_tables(positions, first_position, rope_dim, theta):
    """(cos, sin) [positions, rope_dim // 2] as the reference's engine fills them."""
    cos = np.zeros((positions, rope_dim // 2), dtype=np.float32)
    sin = np.zeros_like(cos)
    oracle().orc_rope_tables(_ptr(cos), _ptr(sin), positions, first_position, rope_dim,
                             C.c_float(theta))
    return cos, sin


def dense_decoder_tokens(cfg, weights, prompt, steps, multi_row_rule=ACT_G32, every_rule=None,
                         first_logits=None):
    """Greedy tokens of the Qwen3-shaped decoder, dense or with the routed mixture of experts
    as its feed-forward block (the layer structure of the reference's graph builders,
    models/qwen3.py:171-345, models/qwen3_moe.py), computed entirely from the oracle's pieces on the
    CPU: the W4A8 matmul (per 128 values for one row, `multi_row_rule` for several), RMSNorm,
    per-head Q/K norm, rotary embedding with host-computed tables, causal attention over all
    keys so far, SwiGLU, residual adds.  Returns (tokens, margins): margin = top-1 minus top-2
    logit of each step, the quantity that says how fragile the token identity is.
    every_rule: one activation rule for every matmul, whatever its row count (ACT_F64 = the
    exact product of fp32 activations with the dequantised weight, the arithmetic of the
    reference's x86 build up to summation order).  first_logits: a list that receives the
    logits of the prompt's last position."""
    from __graft_entry__ import load_package
    dec = load_package().decoder
    sh = weights["shapes"]
    H, D = cfg.hidden, cfg.head_dim
    embed = weights["embed"].astype(np.float32)
    k_all = [np.zeros((0, cfg.kv_heads, D), np.float32) for _ in range(cfg.layers)]
    v_all = [np.zeros((0, cfg.kv_heads, D), np.float32) for _ in range(cfg.layers)]
    past = 0

    def forward(ids):
        nonlocal past
        T = len(ids)
        rule = ACT_G128 if T == 1 else multi_row_rule
        if every_rule is not None:
            rule = every_rule
        cos, sin = rope_tables(T, past, D, cfg.rope_theta)
        x = embed[np.asarray(ids)]
        h = rms_norm(x, weights["layers"][0]["ln1"], cfg.eps)
        for li, L in enumerate(weights["layers"]):
            qkv = matmul_w4(L["qkv"], *sh["qkv"], h, rule=rule)
            q = qkv[:, :cfg.q_dim].reshape(T * cfg.heads, D)
            k = qkv[:, cfg.q_dim:cfg.q_dim + cfg.kv_dim].reshape(T * cfg.kv_heads, D)
            v = qkv[:, cfg.q_dim + cfg.kv_dim:].reshape(T, cfg.kv_heads, D)
            q = rope(rms_norm(q, L["q_norm"], cfg.eps).reshape(T, cfg.heads, D), cos, sin, D)
            k = rope(rms_norm(k, L["k_norm"], cfg.eps).reshape(T, cfg.kv_heads, D), cos, sin, D)
            k_all[li] = np.concatenate([k_all[li], k])
            v_all[li] = np.concatenate([v_all[li], v])
            attn = causal_attention(q, k_all[li], v_all[li], cfg.heads, cfg.kv_heads, past,
                                    D ** -0.5).reshape(T, cfg.q_dim)
            o = matmul_w4(L["o"], *sh["o"], attn, rule=rule)
            x, h = add_rms_norm(x, o, L["ln2"], cfg.eps)
            if cfg.experts:  # the MOE operator under the reference's rule: an expert that
                # holds several rows quantises per 32 values, a lone row per 128
                dn = moe_forward(h, L["router"], cfg.top_k, cfg.intermediate, L["gate_up"],
                                 L["down"], rule=ACT_G32 if every_rule is None else every_rule)[0]
            else:
                act = swiglu(matmul_w4(L["gate_up"], *sh["gate_up"], h, rule=rule))
                dn = matmul_w4(L["down"], *sh["down"], act, rule=rule)
            nxt = weights["layers"][li + 1]["ln1"] if li + 1 < cfg.layers else weights["final_norm"]
            x, h = add_rms_norm(x, dn, nxt, cfg.eps)
        past += T
        logits = matmul_w4(weights["lm_head"], cfg.vocab, H, h[T - 1:T],
                           rule=ACT_G128 if every_rule is None else every_rule)[0]
        if first_logits is not None and not first_logits:
            first_logits.append(logits.copy())
        top = np.sort(logits)[-2:]
        return argmax_token(logits), float(top[1] - top[0])

    tokens, margins = [], []
    tok, mg = forward(list(prompt))
    for _ in range(steps):
        tokens.append(tok)
        margins.append(mg)
        if len(tokens) < steps:
            tok, mg = forward([tok])
    return tokens, margins
