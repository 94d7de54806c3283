"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: W4G128 weights written straight into canonical BG128 blocks (every one
of the 16 nibble codes, i.e. int4 in [-8,7], uniformly; per-row group scales |N(0,0.02)|
rounded to fp16 and stored in the block's fp32 slot), fp16 N(0,1) activations widened
to fp32, and fp16 N(0,0.02) router weights.

The generator is counter based (SplitMix64 of seed, tensor id and element index) so any
slice of any tensor can be produced independently, in numpy here and by the same integer
recipe elsewhere.  Block layout: reference kernels/quant_layouts.h:9-14.
"""
import numpy as np

BLOCK_BYTES = 544
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def _stream(seed, tensor_id, count, lane=0):
    with np.errstate(over="ignore"):
        base = splitmix64(np.uint64(seed) * np.uint64(0xD1342543DE82EF95)
                          + np.uint64(tensor_id) * np.uint64(0x2545F4914F6CDD1D)
                          + np.uint64(lane))
        return splitmix64(base + np.arange(count, dtype=np.uint64))


def uniform01(seed, tensor_id, count, lane=0):
    """fp64 uniforms in (0,1) from the top 53 bits."""
    u = _stream(seed, tensor_id, count, lane) >> np.uint64(11)
    return (u.astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed, tensor_id, count, lane=0):
    u1 = uniform01(seed, tensor_id, count, lane)
    u2 = uniform01(seed, tensor_id, count, lane + 1)
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def bg128_bytes(n, k):
    return ((n + 7) // 8) * (k // 128) * BLOCK_BYTES


def bg128_weight(seed, tensor_id, n, k, scale_std=0.02):
    """uint8 array of canonical BG128 blocks for an [N,K] weight.  Rows past N in the
    last 8-row tile carry scale 0 and zero nibbles, as the reference packers write them."""
    assert k % 128 == 0
    tiles, groups = (n + 7) // 8, k // 128
    nblocks = tiles * groups
    blocks = np.zeros((nblocks, BLOCK_BYTES), dtype=np.uint8)
    with np.errstate(over="ignore"):
        raw = _stream(seed, tensor_id, nblocks * 64, lane=7)
    blocks[:, 32:] = raw.view(np.uint8).reshape(nblocks, 512)
    sc = np.abs(normal(seed, tensor_id, nblocks * 8, lane=3) * scale_std)
    sc = sc.astype(np.float16).astype(np.float32).reshape(tiles, groups, 8)
    if n % 8:
        pad = 8 - n % 8
        sc[-1, :, 8 - pad:] = 0.0
        q = blocks[:, 32:].reshape(tiles, groups, 4, 8, 16)
        q[-1, :, :, 8 - pad:, :] = 0
    blocks[:, :32] = sc.reshape(nblocks, 8).view(np.uint8)
    return blocks.reshape(-1)


def activations(seed, tensor_id, m, k):
    """fp16 N(0,1) widened to fp32, shape [M,K]."""
    x = normal(seed, tensor_id, m * k, lane=11)
    return x.astype(np.float16).astype(np.float32).reshape(m, k)


def router_weight(seed, tensor_id, experts, hidden, std=0.02):
    x = normal(seed, tensor_id, experts * hidden, lane=19) * std
    return x.astype(np.float16).reshape(experts, hidden)
