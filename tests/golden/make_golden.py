"""Regenerates tests/golden/*.npz by running the UNMODIFIED reference library
(oracle/_ref, built by `make -C oracle ref`) on small deterministic inputs.

Run where the reference sources are available:   python tests/golden/make_golden.py

The closed-form inputs restate the fills the reference's own tests use, so the stored
outputs are the reference's answers on its own test cases:
  matmul_m1_k128_n13   tests/test_matmul.cpp:829-888   (M=1 BG128 GEMV)
  matmul_m8_k128_n13   tests/test_matmul.cpp:1418-1477 (M>1 BG128 GEMM)
  matmul_m16_k128_n19  tests/test_matmul.cpp:1479-1529 (odd N)
  cuda_k128_n8 / cuda_k256_n8  tests/test_cuda_backend.cpp:1142-1271 (nibbles -8..7)
  routes_*             tests/test_moe_routing.cpp:29-45,129-144 (order, ties)
The remaining cases are seeded synthetic inputs (palm-infra_b200/synth.py).
Stored per matmul case: the BG128 bytes from the reference packers, the fp32 output of
the reference's kernel_matmul_fp32 (x86 provider, W4A32 arithmetic), and the output of
the reference's activation quantisers on the same activations.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "palm-infra_b200"))
import oracle_lib as ol  # noqa: E402
import synth  # noqa: E402


def closed_form_case(m, k, n, a_mod, a_off, a_mul, s0, s1, s_mod, qa, qb):
    i = np.arange(m * k)
    a = (((i % a_mod) - a_off).astype(np.float32) * np.float32(a_mul)).reshape(m, k)
    nn = np.arange(n)
    scales = (np.float32(s0) + np.float32(s1) * (nn % s_mod).astype(np.float32))
    scales = scales.astype(np.float32).reshape(n, 1).repeat(k // 128, axis=1)
    kk = np.arange(k)
    q = (((nn[:, None] * qa + kk[None, :] * qb) % 15) - 7).astype(np.int8)
    return a, q, scales


def cuda_case(m, k, n):
    groups = k // 128
    i = np.arange(m * k)
    if k == 128:
        a = ((i % 17) - 8).astype(np.float32) / np.float32(19.0)
    else:
        a = ((i % 23) - 11).astype(np.float32) / np.float32(29.0)
    a = a.reshape(m, k)
    q = np.zeros((n, k), dtype=np.int8)
    scales = np.zeros((n, groups), dtype=np.float32)
    for row in range(n):
        for g in range(groups):
            if k == 128:
                scales[row, g] = np.float32(0.0625) + np.float32(row) * np.float32(0.005)
                inner = np.arange(128)
                q[row, :] = (row + inner) % 15 - 7
            else:
                scales[row, g] = np.float32(0.015625) + np.float32(0.001) * np.float32(row + g)
                inner = np.arange(128)
                q[row, g * 128:(g + 1) * 128] = (row + g * 7 + inner) % 16 - 8
    return a, q, scales


def matmul_record(a, q, scales):
    n, k = q.shape
    blocks = ol.ref_pack_bg128(q, scales)
    y = ol.ref_matmul(blocks, n, k, a)
    e, o, s128 = ol.ref_quantize_g128_even_odd(a[0])
    q32, s32 = ol.ref_quantize_g32(a)
    return dict(a=a, q=q, scales=scales, blocks=blocks, y_ref_w4a32=y, qa_even=e,
                qa_odd=o, a_scales_g128=s128, qa_g32=q32, a_scales_g32=s32)


def main():
    assert ol.have_ref(), "build oracle/_ref first: make -C oracle ref"
    out = {}
    cases = {
        "matmul_m1_k128_n13": closed_form_case(1, 128, 13, 23, 11, 0.015625, 0.005, 0.0005, 7, 17, 9),
        "matmul_m8_k128_n13": closed_form_case(8, 128, 13, 23, 11, 0.015625, 0.005, 0.0005, 7, 17, 9),
        "matmul_m16_k128_n19": closed_form_case(16, 128, 19, 29, 14, 0.013671875, 0.0045, 0.0004, 9, 19, 7),
        "cuda_k128_n8": cuda_case(3, 128, 8),
        "cuda_k128_n7": cuda_case(3, 128, 7),
        "cuda_k256_n8": cuda_case(3, 256, 8),
    }
    for name, (a, q, s) in cases.items():
        for key, val in matmul_record(a, q, s).items():
            out[f"{name}/{key}"] = val

    # seeded synthetic matmul, config-1 distributions at a small size
    n, k, m = 72, 512, 5
    blocks = synth.bg128_weight(20261125, 3, n, k)
    a = synth.activations(7, 3, m, k)
    out["synth_m5_k512_n72/blocks"] = blocks
    out["synth_m5_k512_n72/a"] = a
    out["synth_m5_k512_n72/y_ref_w4a32"] = ol.ref_matmul(blocks, n, k, a)
    out["synth_m5_k512_n72/y_ref_silu_8_40"] = ol.ref_matmul(blocks, n, k, a, act=1, begin=8, length=40)
    e, o, s128 = ol.ref_quantize_g128_even_odd(a[2])
    q32, s32 = ol.ref_quantize_g32(a)
    out["synth_m5_k512_n72/qa_even_row2"] = e
    out["synth_m5_k512_n72/qa_odd_row2"] = o
    out["synth_m5_k512_n72/a_scales_g128_row2"] = s128
    out["synth_m5_k512_n72/qa_g32"] = q32
    out["synth_m5_k512_n72/a_scales_g32"] = s32

    # quantiser edge cases: an all-zero group, a constant group, huge and tiny values,
    # exact .5 ties (round half to even)
    edge = np.zeros(512, dtype=np.float32)
    edge[128:256] = 3.0
    edge[256:384] = np.linspace(-1e30, 1e30, 128, dtype=np.float32)
    edge[384:512] = (np.arange(128) - 64).astype(np.float32) * np.float32(0.5) * np.float32(63.5 / 127.0)
    edge[511] = 63.5
    e, o, s = ol.ref_quantize_g128_even_odd(edge)
    out["quant_edge/x"] = edge
    out["quant_edge/even"] = e
    out["quant_edge/odd"] = o
    out["quant_edge/scales"] = s

    # routing: descending order, softmax over the selected, ties -> lower id
    logits = np.array([[0.1, 2.0, -1.0, 2.0, 0.5, 2.0, -3.0, 1.5],
                       [1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0],
                       [-5.0, -4.0, -3.0, -2.0, -1.0, 0.0, 1.0, 2.0]], dtype=np.float32)
    for kk in (1, 2, 4):
        idx, w = ol.ref_select_routes(logits, kk)
        out[f"routes_small_k{kk}/logits"] = logits
        out[f"routes_small_k{kk}/idx"] = idx
        out[f"routes_small_k{kk}/w"] = w
    lg = (synth.normal(11, 5, 64 * 128).astype(np.float32) * np.float32(1.3)).reshape(64, 128)
    idx, w = ol.ref_select_routes(lg, 8)
    out["routes_64x128_k8/logits"] = lg
    out["routes_64x128_k8/idx"] = idx
    out["routes_64x128_k8/w"] = w

    # small routed MoE through the reference op (x86: W4A32 expert arithmetic)
    t, h, e_cnt, top_k, inter = 6, 128, 8, 2, 128
    hidden = synth.activations(7, 9, t, h)
    router = synth.router_weight(20261125, 10, e_cnt, h, std=0.2)
    gu = synth.bg128_weight(20261125, 11, e_cnt * 2 * inter, h)
    dn = synth.bg128_weight(20261125, 12, e_cnt * h, inter)
    out["moe_small/hidden"] = hidden
    out["moe_small/router"] = router.view(np.uint16)
    out["moe_small/gate_up"] = gu
    out["moe_small/down"] = dn
    out["moe_small/out_ref_w4a32"] = ol.ref_moe(hidden, router, top_k, inter, gu, dn)
    out["moe_small/meta"] = np.array([t, h, e_cnt, top_k, inter], dtype=np.int32)

    # greedy token: the reference's own sampling entry at temperature 0 (argmax_token) on
    # rows with equal maxima, signed zeros, NaNs (first, elsewhere), infinities
    rng = np.random.default_rng(77)
    rows = [rng.standard_normal(n).astype(np.float32) for n in (1, 2, 3, 5, 8, 100, 4097)]
    tie = np.zeros(64, dtype=np.float32)
    tie[[9, 17, 40]] = 3.5
    neg0 = np.full(16, -1.0, dtype=np.float32)
    neg0[5], neg0[11] = -0.0, 0.0
    nan_mid = rng.standard_normal(40).astype(np.float32)
    nan_mid[[3, 20]] = np.nan
    nan_mid[30] = 10.0
    nan_first = rng.standard_normal(40).astype(np.float32)
    nan_first[0] = np.nan
    infs = np.array([-np.inf, np.nan, -np.inf, np.inf, np.inf], dtype=np.float32)
    rows += [tie, neg0, nan_mid, nan_first, infs, np.full(9, -np.inf, dtype=np.float32)]
    for i, row in enumerate(rows):
        out[f"greedy_token/row{i}"] = row
    out["greedy_token/tokens"] = np.array([ol.ref_greedy_token(r) for r in rows], dtype=np.int32)

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
