"""Tensor-parallel sharding of a W4G128 weight by output rows.

Every output row of the matmul is independent, so rank r of P keeps rows
[r*N/P, (r+1)*N/P) and the full output is the concatenation of the ranks' outputs: no
reduction, results bit-identical to one GPU.  8-row tiles stay whole, so N must be a multiple
of 8*P.  In the canonical BG128 stream a tile's K/128 blocks are adjacent, which makes a row
shard one contiguous byte range.
"""
BLOCK_BYTES = 544


def row_range(n, rank, world):
    if n % (8 * world):
        raise ValueError(f"N={n} must be a multiple of 8*world={8 * world}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_blocks(blocks, n, k, rank, world):
    """blocks: flat uint8 BG128 array of an [N,K] weight -> (rank's blocks, rows, row offset)."""
    lo, hi = row_range(n, rank, world)
    tile_bytes = (k // 128) * BLOCK_BYTES
    return blocks[(lo // 8) * tile_bytes:(hi // 8) * tile_bytes], hi - lo, lo


def expert_range(num_experts, rank, world):
    """Expert-parallel placement: contiguous blocks of E/P experts per rank."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split over {world} ranks")
    per = num_experts // world
    return rank * per, (rank + 1) * per


# ---- greedy token of a row-sharded lm_head ---------------------------------------------------
# Host statement of what the device does (b2w4_matmul_argmax_tp + b2w4_tp_gather_token), used
# by the CPU tests of the multi-rank logic; the product path runs on the GPUs.

def top1_word(value, index):
    """The 64-bit word a logit becomes: (order-preserving key of the fp32 value << 32) |
    (0xFFFFFFFF - index).  The largest word of a row is its greedy token under the rule of
    the reference's argmax_token (engine/sampler.cpp:72-77): the first maximum wins, a NaN
    never wins -- except at index 0, where nothing beats it.  `index` is the row of the
    UNSHARDED weight, so words of different ranks compare in the one-device order."""
    import numpy as np
    v = np.float32(value)
    bits = int(v.view(np.uint32))
    if v != v:
        key = 0xFFFFFFFF if index == 0 else 0
    else:
        if bits == 0x80000000:
            bits = 0                       # -0 == +0: the lower index wins
        key = (~bits & 0xFFFFFFFF) if bits & 0x80000000 else bits | 0x80000000
    return (key << 32) | (0xFFFFFFFF - index)


def shard_top1_word(logits_shard, row_offset):
    """A rank's hand-over: the largest word over its rows [row_offset, row_offset + n)."""
    return max(top1_word(v, row_offset + i) for i, v in enumerate(logits_shard))


def pick_token(words):
    """The gather: the largest of the ranks' words, decoded to the token."""
    return 0xFFFFFFFF - (max(words) & 0xFFFFFFFF)
