"""Work partitioning across GPUs for the polynomial hot path.

Nothing on this path is reduced across devices, so multi-GPU means independent shards: contiguous element ranges
for the flat element-wise operators, contiguous row ranges for packed SwiGLU, contiguous expert groups for routed
experts (B4) and contiguous blocks of (batch, head) for attention.  No collective runs on the data path; the only
cross-rank traffic a driver needs is a barrier and a max over ranks for timing.

Every function is pure host arithmetic: the same (rank, world) always yields the same shard, shards never overlap,
and together they cover the whole problem, so concatenating per-rank outputs reproduces the single-GPU output.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def element_range(n: int, rank: int, world: int, align: int = 8) -> tuple[int, int]:
    """Contiguous [lo, hi) of a flat array; interior boundaries are multiples of `align` elements so that every
    shard keeps the 16-byte alignment of the whole."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    units = (n + align - 1) // align
    lo = min(n, (units * rank // world) * align)
    hi = min(n, (units * (rank + 1) // world) * align)
    return lo, hi


def row_range(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range of a [rows, width] tensor (packed SwiGLU)."""
    return element_range(rows, rank, world, align=1)


def zipf_expert_counts(assignments: int, experts: int, exponent: float = 1.1, seed: int = 1234) -> np.ndarray:
    """Tokens per expert for the routed-expert workload: weights 1/k^exponent over a seeded permutation of the
    experts, `assignments` draws from the resulting multinomial."""
    rng = np.random.default_rng(seed)
    weights = 1.0 / np.arange(1, experts + 1, dtype=np.float64) ** exponent
    weights = weights[rng.permutation(experts)]
    weights /= weights.sum()
    return rng.multinomial(assignments, weights).astype(np.int64)


@dataclass(frozen=True)
class ExpertShard:
    first_expert: int
    last_expert: int   # exclusive
    first_row: int
    last_row: int      # exclusive


def expert_group(counts, rank: int, world: int) -> ExpertShard:
    """Rank r owns experts [r*E/W, (r+1)*E/W) and, rows being expert-sorted, the row range they cover."""
    counts = np.asarray(counts, dtype=np.int64)
    lo, hi = element_range(counts.size, rank, world, align=1)
    offsets = np.concatenate([[0], np.cumsum(counts)])
    return ExpertShard(lo, hi, int(offsets[lo]), int(offsets[hi]))


@dataclass(frozen=True)
class HeadBlock:
    batch: int
    first_q_head: int
    last_q_head: int   # exclusive


def attention_blocks(batch: int, q_heads: int, kv_heads: int, rank: int, world: int) -> list[HeadBlock]:
    """Contiguous run of (batch, kv-head group) units; the q heads that share a kv head stay on one GPU."""
    if q_heads % kv_heads:
        raise ValueError("q_heads must be a multiple of kv_heads")
    group = q_heads // kv_heads
    lo, hi = element_range(batch * kv_heads, rank, world, align=1)
    blocks: list[HeadBlock] = []
    for unit in range(lo, hi):
        b, g = divmod(unit, kv_heads)
        if blocks and blocks[-1].batch == b and blocks[-1].last_q_head == g * group:
            blocks[-1] = HeadBlock(b, blocks[-1].first_q_head, (g + 1) * group)
        else:
            blocks.append(HeadBlock(b, g * group, (g + 1) * group))
    return blocks
