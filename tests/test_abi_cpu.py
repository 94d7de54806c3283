"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol that
include/b200w4.h declares, and refuses to run without a device (no compute here)."""
import ctypes
import os
import re

import pytest

from __graft_entry__ import ROOT, load_package

pkg = load_package()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200w4.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2w4_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(pkg.capi.SYMBOLS)


def test_library_exports_every_declared_symbol():
    pkg.build_library()
    lib = ctypes.CDLL(pkg.capi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert b"sm_100a" in pkg.capi.lib().b2w4_version()


def test_no_device_is_a_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(pkg.capi.B200W4Error):
        pkg.capi.Context(0)


def test_null_context_is_rejected_not_dereferenced():
    lib = pkg.capi.lib()
    assert lib.b2w4_sync(None) == -1
    assert lib.b2w4_matmul(None, None, None, 0, None, 0, 1, 128, 0, 0, -1) == -1
    assert lib.b2w4_last_error(None) == b"no context"


def test_synth_blocks_follow_the_canonical_layout():
    import numpy as np
    import oracle_lib as ol
    n, k = 21, 256
    blocks = pkg.synth.bg128_weight(5, 2, n, k)
    assert blocks.nbytes == ol.bg128_bytes(n, k) == 3 * 2 * 544
    q, s = ol.bg128_decode(blocks, 24, k)
    assert (s[21:] == 0).all() and (q[21:] == 0).all()           # padded rows
    assert (s[:21] == s[:21].astype(np.float16).astype(np.float32)).all()
    assert q.min() == -8 and q.max() == 7
    assert pkg.synth.bg128_weight(5, 2, n, k).tobytes() == blocks.tobytes()


def test_exchange_group_struct_and_null_contexts():
    """b2w4_tp_group as the header lays it out (two ints, eight pointers), the staging sizes
    the host helpers promise, and the exchange entry points refusing a null context."""
    import ctypes as C
    g = pkg.capi.TpGroup()
    assert C.sizeof(g) == 8 + 8 * 8
    assert pkg.capi.TpGroup.stage_peers.offset == 8
    assert pkg.expert_parallel.PeerExchangeMoE.stage_words(8, 2048) == 2 + 2 * 8 * 2048
    lib = pkg.capi.lib()
    assert lib.b2w4_matmul_tp(None, None, None, 0, 1, 0, 0, None, 0, 0, -1) == -1
    assert lib.b2w4_tp_gather(None, None, None, 1, 0) == -1
    assert lib.b2w4_matmul_argmax(None, None, None, 0, 1, None, 0, None) == -1
    assert lib.b2w4_matmul_argmax_tp(None, None, None, 0, 1, 0, None) == -1
    assert lib.b2w4_tp_gather_token(None, None, None, 1) == -1
