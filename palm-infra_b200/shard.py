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


def shard_blocks_k(blocks, n, k, rank, world):
    """The other way to cut a weight: by input features.  Rank r keeps the 128-wide groups
    [r * G / P, (r + 1) * G / P) of every row, as a BG128 weight [N, K / P] of its own, and
    multiplies them with its slice of the activation row; the ranks' outputs are partial sums
    that an all-reduce adds up.  The int32 group sums and the activation scales are the
    one-GPU ones (groups stay whole), but the fp32 chain of a row is now P chains added in
    another order, so the result equals the one-GPU result to fp32 rounding, not bit for bit --
    the price for an exchange of N values instead of a gather before a wide-K matmul (o and
    down projections).  Returns (blocks [N, K / P], first input feature)."""
    import numpy as np
    groups = k // 128
    if k % 128 or groups % world or n % 8:
        raise ValueError(f"K={k} must split into whole 128-groups over {world} ranks, N={n} "
                         "into 8-row tiles")
    per = groups // world
    tiles = blocks.reshape(n // 8, groups, BLOCK_BYTES)
    mine = np.ascontiguousarray(tiles[:, rank * per:(rank + 1) * per]).reshape(-1)
    return mine, rank * per * 128


def rows_of(blocks, k, lo, hi):
    """The BG128 blocks of rows [lo, hi) (multiples of 8) of a weight with K columns."""
    if lo % 8 or hi % 8:
        raise ValueError(f"rows [{lo}, {hi}) do not fall on 8-row tiles")
    tile_bytes = (k // 128) * BLOCK_BYTES
    return blocks[(lo // 8) * tile_bytes:(hi // 8) * tile_bytes]


def decoder_layer_shard(cfg, shapes, layer, rank, world):
    """Rank `rank`'s share of one decoder layer, every matmul split by output rows:
      qkv      the rank's query heads, then its key heads, then its value heads (so the fused
               projection of the shard is the fused projection of a model with heads / world
               heads), attention then runs on those heads alone with a cache of their own;
      o, down  rows [r * H / P, (r + 1) * H / P) over the full input;
      gate_up  the rank's slice of the gate rows, then the same slice of the up rows (SwiGLU of
               the shard's output is the rank's slice of the activation).
    Inputs of o and down are the concatenation of the ranks' outputs in rank order, which is
    head order and intermediate-feature order.  Norm weights are replicated.  With routed
    experts the feed-forward block is split by expert instead (expert_range): the rank keeps
    its experts' rows of both aggregates and the whole router.  Returns (layer weights,
    shapes)."""
    import numpy as np
    if cfg.heads % world or cfg.kv_heads % world:
        raise ValueError(f"{cfg.heads} / {cfg.kv_heads} heads do not split over {world} ranks")
    D, H, I = cfg.head_dim, cfg.hidden, cfg.intermediate
    q_l, kv_l = cfg.q_dim // world, cfg.kv_dim // world
    h_lo, h_hi = row_range(H, rank, world)
    if D % 8:
        raise ValueError("head_dim must be a multiple of 8")
    qkv = layer["qkv"]
    parts = [rows_of(qkv, H, rank * q_l, (rank + 1) * q_l),
             rows_of(qkv, H, cfg.q_dim + rank * kv_l, cfg.q_dim + (rank + 1) * kv_l),
             rows_of(qkv, H, cfg.q_dim + cfg.kv_dim + rank * kv_l,
                     cfg.q_dim + cfg.kv_dim + (rank + 1) * kv_l)]
    out = {"qkv": np.concatenate(parts), "o": rows_of(layer["o"], cfg.q_dim, h_lo, h_hi)}
    local_shapes = {"qkv": (q_l + 2 * kv_l, H), "o": (H // world, cfg.q_dim)}
    if cfg.experts:
        e_lo, e_hi = expert_range(cfg.experts, rank, world)
        out["gate_up"] = rows_of(layer["gate_up"], H, e_lo * 2 * I, e_hi * 2 * I)
        out["down"] = rows_of(layer["down"], I, e_lo * H, e_hi * H)
        out["router"] = layer["router"]
        local_shapes.update({"gate_up": ((e_hi - e_lo) * 2 * I, H),
                             "down": ((e_hi - e_lo) * H, I)})
    else:
        i_lo, i_hi = row_range(I, rank, world)
        out["gate_up"] = np.concatenate([rows_of(layer["gate_up"], H, i_lo, i_hi),
                                         rows_of(layer["gate_up"], H, I + i_lo, I + i_hi)])
        out["down"] = rows_of(layer["down"], I, h_lo, h_hi)
        local_shapes.update({"gate_up": (2 * (I // world), H), "down": (H // world, I)})
    for key in ("ln1", "ln2", "q_norm", "k_norm"):
        out[key] = layer[key]
    assert all(out[k].size == (n // 8) * (kk // 128) * BLOCK_BYTES
               for k, (n, kk) in local_shapes.items()), shapes
    return out, local_shapes


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
