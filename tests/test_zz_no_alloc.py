"""The entry point for callers that cannot allocate device memory while they run a matmul
(a serving loop that forbids cudaMalloc because it synchronises the device, code inside an
open stream capture, a runtime with a memory budget fixed at start-up).
b2w4_matmul_static_scratch keeps the quantised activations in a fixed array inside the
library instead of a cudaMalloc'd pool.  Its result must be bit-identical to b2w4_matmul's,
on two calls in a row (the array is shared and keeps the previous call's contents, so the
second call runs on top of the first one's leftovers), and sizes beyond the array are errors.
This file is collected last so a run that stops at the first failure has already run every
other test."""
import numpy as np
import pytest

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
pytestmark = pytest.mark.gpu


def test_static_scratch_matches_matmul_on_two_calls_in_a_row():
    import torch
    ctx = pkg.capi.Context(0)
    n, k = 1000, 1280
    blocks = pkg.synth.bg128_weight(20261125, 77, n, k)
    w = ctx.upload_weight(blocks, n, k)
    try:
        # first call: 200 rows; second call: 37 rows on top of the first call's leftovers
        for call, m in enumerate((200, 37)):
            x = torch.from_numpy(pkg.synth.activations(7, 900 + call, m, k)).cuda()
            want = torch.zeros((m, n), dtype=torch.float32, device="cuda")
            got = torch.full((m, n), -1.0, dtype=torch.float32, device="cuda")
            ctx.matmul(w, x, want, act=pkg.capi.SILU, act_begin=8, act_len=400)
            ctx.matmul_static_scratch(w, x, got, act=pkg.capi.SILU, act_begin=8, act_len=400)
            ctx.sync()
            assert torch.equal(got, want), f"call {call}: differs from b2w4_matmul"
        # beyond the fixed array: clear errors, nothing launched
        x = torch.zeros((300, k), device="cuda")
        y = torch.zeros((300, n), device="cuda")
        with pytest.raises(pkg.capi.B200W4Error, match="outside 5..256"):
            ctx.matmul_static_scratch(w, x, y)
        with pytest.raises(pkg.capi.B200W4Error, match="outside 5..256"):
            ctx.matmul_static_scratch(w, x[:2], y[:2])
        wide = ctx.upload_weight(pkg.synth.bg128_weight(1, 1, 8, 10368), 8, 10368)
        with pytest.raises(pkg.capi.B200W4Error, match="exceeds 10240"):
            ctx.matmul_static_scratch(wide, torch.zeros((8, 10368), device="cuda"),
                                      torch.zeros((8, 8), device="cuda"))
        wide.free()
    finally:
        w.free()
        ctx.close()


@pytest.mark.parametrize("fp16_scales", [True, False])
def test_static_scratch_against_the_oracle_and_allocates_nothing(fp16_scales):
    """Row counts at the entry point's limits (5, 256) and on both sides of the step where the
    row padding and the kernel variant change (128 / 129), plus 8, in one sequence of calls on
    the shared array; every result bit for bit the CPU oracle's per-128 chain.  The device's
    free memory, read before and after each call, must not move: that is the property the
    entry point exists for.  (Measured on the second call of each size: the very first launch
    of a kernel variant lets the CUDA driver load that kernel's code, which is the driver's
    memory, not this library's.)"""
    import torch
    ctx = pkg.capi.Context(0)
    n, k = 264, 640
    blocks = pkg.synth.bg128_weight(20261125, 78, n, k).copy()
    if not fp16_scales:
        b = blocks.reshape(-1, 544)
        b[:, :32].view(np.float32)[:] *= np.float32(1.0001)  # scale plane stays fp32
    w = ctx.upload_weight(blocks, n, k)
    assert w.scales_fp16 == fp16_scales
    try:
        xs = {m: pkg.synth.activations(7, 950 + m, m, k) for m in (5, 8, 128, 129, 256)}
        xd = {m: torch.from_numpy(x).cuda() for m, x in xs.items()}
        yd = {m: torch.full((m, n), -1.0, dtype=torch.float32, device="cuda") for m in xs}
        for m in xs:  # one-time set-up of this device; every kernel variant's code loaded
            ctx.matmul_static_scratch(w, xd[m], yd[m])
        ctx.sync()
        torch.cuda.synchronize()
        for y in yd.values():
            y.fill_(-1.0)
        torch.cuda.synchronize()
        for m in (256, 5, 129, 128, 8):
            free_before, _ = torch.cuda.mem_get_info()
            ctx.matmul_static_scratch(w, xd[m], yd[m])
            ctx.sync()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, f"M={m}: device memory moved by the call"
            want = ol.matmul_w4(blocks, n, k, xs[m], rule=ol.ACT_G128)
            got = yd[m].cpu().numpy()
            assert got.view(np.uint32).tobytes() == want.view(np.uint32).tobytes(), f"M={m}"
    finally:
        w.free()
        ctx.close()
