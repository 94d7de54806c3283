"""Drop-in check of the C++ CudaBackend replacement (palm-infra_b200/backend/cuda_backend.cpp):
the reference's OWN tests/test_cuda_backend.cpp, compiled unmodified against this backend
(palm-infra_b200/backend/Makefile), must pass on the GPU.  It drives the class through
dispatch() with host and device tensors: FP16 / W8 / W4G32 matmuls (reference bridge),
W4G128 matmuls at M=3 and M=1, N=8 and padded N=7, K=128 and 256 with nibbles over -8..7
(native, libb200w4), zeroes the host blocks after wrap_weight_int4, views, KV cache / SDPA
through the bridge, persistent-storage modes, pool reuse, and REQUIRE_NATIVE rejection."""
import os
import re
import subprocess

import pytest

from __graft_entry__ import PKG_DIR

BIN = os.path.join(PKG_DIR, "build", "backend", "test_cuda_backend")
pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not os.path.exists(BIN),
                    reason="backend test binary not built (needs the reference tree at build time)")
def test_reference_cuda_backend_test_passes_against_this_backend():
    env = dict(os.environ, MOLLM_CUDA_PROFILE="1")
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, f"rc={r.returncode}\nstdout:\n{r.stdout}\nstderr:\n{r.stderr[-3000:]}"
    assert "W4G128 matmul tests passed" in r.stdout
    # The backend counts, per operator type, what ran natively and what went through the
    # reference bridge (printed at tear-down under MOLLM_CUDA_PROFILE).  OpType::MATMUL is 10
    # (graph/graph.h:68).  The reference's test dispatches six W4G128 matmuls on device or host
    # tensors (tests/test_cuda_backend.cpp:1142-1271: M=3 and M=1, N=8 and padded N=7, K=128
    # and 256, and the zeroed-source case) -- those, and only those, must be native -- and
    # eleven matmuls on other formats (FP16, W8, W4G32) or on a sliced weight view, which must
    # all have gone through the bridge.
    counts = {"native": {}, "fallback": {}}
    for line in r.stderr.splitlines():
        m = re.match(r"CudaBackend (native|fallback) op (\d+): (\d+)", line)
        if m:
            counts[m.group(1)][int(m.group(2))] = int(m.group(3))
    assert counts["native"].get(10) == 6, counts
    assert counts["fallback"].get(10) == 11, counts
