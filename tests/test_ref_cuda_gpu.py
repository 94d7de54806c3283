"""The benchmark's GPU comparator: the reference's own CUDA matmul kernels
(engine/cuda_matmul.cu), compiled unmodified for sm_100 by oracle/Makefile (`make refcuda`).
Checked here only for being the computation it is compared as: its outputs agree with the
exact product of the dequantised weight to the reference's own tolerance for that path
(W4A32 for one row; fp16 operands with fp32 accumulation for many rows)."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as ol
from golden_util import rel_l2
from __graft_entry__ import ROOT, load_package

pkg = load_package()
pytestmark = pytest.mark.gpu
LIB = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")


@pytest.mark.skipif(not os.path.exists(LIB),
                    reason="reference CUDA kernels not built (needs the reference tree)")
@pytest.mark.parametrize("m", [1, 32])
def test_reference_cuda_matmul_is_the_w4g128_product(m):
    import torch
    lib = C.CDLL(LIB)
    n, k = 264, 512
    blocks = pkg.synth.bg128_weight(20261125, 5, n, k)
    x = pkg.synth.activations(7, 5 + m, m, k)
    bd = torch.from_numpy(blocks).cuda()
    xd = torch.from_numpy(x).cuda()
    yd = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    vp = C.c_void_p
    if m == 1:
        rc = lib.refcuda_gemv_g128(vp(xd.data_ptr()), vp(bd.data_ptr()), vp(yd.data_ptr()), n, k)
    else:
        rc = lib.refcuda_gemm_g128(vp(xd.data_ptr()), k, vp(bd.data_ptr()), vp(yd.data_ptr()),
                                   m, n, k)
    assert rc == 0
    torch.cuda.synchronize()
    exact = ol.matmul_w4(blocks, n, k, x, rule=ol.ACT_F64)
    # fp32 accumulation over 512 terms (one row) / fp16 operands (many rows)
    assert rel_l2(yd.cpu().numpy(), exact) < (1e-5 if m == 1 else 2e-3)
    lib.refcuda_release()
