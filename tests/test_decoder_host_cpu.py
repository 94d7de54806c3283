"""Host-side pieces of the decoder driver that need no GPU: the benchmark configurations'
shapes, the synthetic model generator (eager and layer-by-layer forms give the same bytes), the
rotary tables, and the weight bytes a decode token streams."""
import numpy as np
import pytest

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
dec = pkg.decoder


def w4_bytes(n, k):
    return ol.bg128_bytes(n, k)


def test_benchmark_configurations():
    c3, c4, c5 = (dec.DecoderConfig.qwen3_4b(), dec.DecoderConfig.qwen3_30b_a3b(),
                  dec.DecoderConfig.qwen3_235b_a22b())
    assert (c3.layers, c3.hidden, c3.heads, c3.kv_heads, c3.intermediate) == (36, 2560, 32, 8, 9728)
    assert (c4.layers, c4.hidden, c4.experts, c4.top_k, c4.intermediate) == (48, 2048, 128, 8, 768)
    assert (c5.layers, c5.hidden, c5.experts, c5.top_k, c5.intermediate) == (94, 4096, 128, 8, 1536)

    def model_bytes(c):
        per = max(1, c.experts)
        layer = (w4_bytes(c.q_dim + 2 * c.kv_dim, c.hidden) + w4_bytes(c.hidden, c.q_dim)
                 + w4_bytes(per * 2 * c.intermediate, c.hidden)
                 + w4_bytes(per * c.hidden, c.intermediate))
        return c.layers * layer + w4_bytes(c.vocab, c.hidden)

    # 2.1 GB, 16 GB and 125 GB as BG128 blocks (544 bytes per 8 x 128 weights; the device
    # planes with fp16 scales are 3 % smaller: 121 GB for configuration 5)
    assert 2.0e9 < model_bytes(c3) < 2.2e9
    assert 15e9 < model_bytes(c4) < 17e9
    assert 120e9 < model_bytes(c5) < 126e9 < 180e9  # one GPU's memory holds configuration 5


def test_lazy_layers_are_the_eager_layers():
    cfg = dec.DecoderConfig(3, 256, 4, 2, 64, 128, 512, experts=4, top_k=2)
    eager = dec.synthetic_weights(cfg, seed=5, distinct_layers=2)
    lazy = dec.synthetic_weights(cfg, seed=5, distinct_layers=2, lazy=True)
    assert not isinstance(lazy["layers"], list)
    count = 0
    for a, b in zip(eager["layers"], lazy["layers"]):
        assert a.keys() == b.keys()
        for key in a:
            assert np.asarray(a[key]).tobytes() == np.asarray(b[key]).tobytes()
        count += 1
    assert count == 3
    # layer 2 reuses layer 0's blocks rotated by whole blocks: another weight, same size
    l0, l2 = eager["layers"][0], eager["layers"][2]
    assert l0["qkv"].size == l2["qkv"].size and l0["qkv"].tobytes() != l2["qkv"].tobytes()
    assert np.array_equal(np.roll(l0["qkv"], 544), l2["qkv"])
    assert eager["layers"][0]["router"].shape == (4, 256)


def test_rotary_tables_follow_the_engine():
    """engine/input_prep.cpp:18-31: theta_i = 1 / theta^(2i / rope_dim), angle = position *
    theta_i, cos / sin of the angle, in fp32 through the host libm.  The product's host
    function (b2w4_rope_tables) and the oracle's give the same bits, and those are the libm's
    own, which numpy's float cosine does not always match."""
    import ctypes
    cos, sin = dec.rope_tables(range(5, 305), 64, 1e6)
    assert cos.shape == sin.shape == (300, 32) and cos.dtype == np.float32
    o_cos, o_sin = ol.rope_tables(300, 5, 64, 1e6)
    assert cos.tobytes() == o_cos.tobytes() and sin.tobytes() == o_sin.tobytes()
    first = dec.rope_tables([0], 64, 1e6)
    assert (first[0] == 1).all() and (first[1] == 0).all()
    libm = ctypes.CDLL("libm.so.6")
    for f in (libm.cosf, libm.sinf):
        f.restype, f.argtypes = ctypes.c_float, [ctypes.c_float]
    libm.powf.restype, libm.powf.argtypes = ctypes.c_float, [ctypes.c_float, ctypes.c_float]
    for row, i in ((0, 0), (1, 6), (17, 15), (299, 31)):
        inv = np.float32(1.0) / np.float32(libm.powf(1e6, float(np.float32(2.0 * i) /
                                                                np.float32(64))))
        angle = float(np.float32(np.float32(5 + row) * inv))
        assert cos[row, i] == np.float32(libm.cosf(angle))
        assert sin[row, i] == np.float32(libm.sinf(angle))
    with pytest.raises(ValueError):
        dec.rope_tables([0, 2, 3], 64, 1e6)
