"""Loader of the committed golden vectors (tests/golden/reference_vectors.npz)."""
import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                     "reference_vectors.npz")
_cache = None


def golden():
    global _cache
    if _cache is None:
        _cache = dict(np.load(_PATH))
    return _cache


def case(name):
    pre = name + "/"
    return {k[len(pre):]: v for k, v in golden().items() if k.startswith(pre)}


def rel_l2(a, b):
    """The reference's own error metric (tests/test_matmul.cpp:50-62)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


MATMUL_CASES = ["matmul_m1_k128_n13", "matmul_m8_k128_n13", "matmul_m16_k128_n19",
                "cuda_k128_n8", "cuda_k128_n7", "cuda_k256_n8"]
