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
