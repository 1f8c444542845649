"""How one call of the chain is spread over several GPUs (one process per GPU).

Rows and batches are independent, so configurations that shard them need no exchange.
Only the vocab-wide configuration splits the softmax row itself: each rank owns a
contiguous range of columns that starts and ends on 256-column tile boundaries, produces
un-normalised exp values plus one (max, sum) pair per row, and after ONE all-gather of
those pairs ([world, rows, 2] f32, 8 bytes per row per rank) every rank can normalise its
own columns.  The maxima are in the log2 domain: v = scale * log2(e) * s, pair =
(max_j v_j, sum_j 2^(v_j - max)).  The reference has no multi-GPU path to mirror.
"""
from __future__ import annotations

TILE_N = 256


def split_batches(batch: int, world: int) -> list[tuple[int, int]]:
    """[start, stop) of the batches each rank runs; the first `batch % world` ranks get one more."""
    if world < 1 or batch < 0:
        raise ValueError("world must be >= 1 and batch >= 0")
    out, start = [], 0
    for r in range(world):
        n = batch // world + (1 if r < batch % world else 0)
        out.append((start, start + n))
        start += n
    return out


def split_rows(M: int, world: int, block: int = 128) -> list[tuple[int, int]]:
    """[start, stop) of the rows each rank runs, on `block`-row boundaries."""
    blocks = (M + block - 1) // block
    return [(min(M, a * block), min(M, b * block)) for a, b in split_batches(blocks, world)]


def split_columns(N: int, world: int, tile: int = TILE_N) -> list[tuple[int, int]]:
    """[start, stop) of the columns each rank owns, on `tile`-column boundaries
    (32000 columns over 8 ranks: 16,16,16,16,16,15,15,15 tiles)."""
    tiles = (N + tile - 1) // tile
    return [(min(N, a * tile), min(N, b * tile)) for a, b in split_batches(tiles, world)]


def combine_pairs(pairs):
    """Log-sum-exp combination of (max, sum) pairs along axis 0 (any array library whose
    arrays support max/exp2/sum along an axis: numpy or torch).  pairs: [parts, rows, 2].
    Returns (row_max, row_sum)."""
    m = pairs[..., 0]
    l = pairs[..., 1]
    gm = m.max(0) if not hasattr(m.max(0), "values") else m.max(0).values
    scale = 2.0 ** (m - gm)
    return gm, (l * scale).sum(0)
