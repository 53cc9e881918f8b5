"""How the path is split across GPUs: no exchange step, only independent units.

* m-grouped / masked GEMM: experts are sharded contiguously; each rank keeps its experts' rows of A / D and its
  slices of B, and rebuilds a local psum layout that starts at row 0 (groups are 256-row aligned, so row ranges of
  different ranks never overlap).
* dense GEMM: columns of D (rows of B) are sharded; every rank holds all of A.
"""

from __future__ import annotations

ALIGNMENT = 256


def _align(x: int, a: int = ALIGNMENT) -> int:
    return (x + a - 1) // a * a


def expert_range(num_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block of experts owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(num_experts, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def balanced_expert_ranges(sizes: list[int], world: int) -> list[tuple[int, int]]:
    """Contiguous blocks of experts, one per rank, that minimise the largest number of (256-aligned) rows any rank
    gets: the step time of the sharded grouped GEMM is the slowest rank's. Per-expert sizes ~ U(0.7, 1.3) x 8192 make
    equal expert counts up to 15 % uneven in rows. Every rank computes the same answer from the same `sizes`."""
    rows = [_align(s) for s in sizes]
    n = len(rows)
    if world <= 1 or n == 0:
        return [(0, n)] + [(n, n)] * max(0, world - 1)

    def blocks_needed(cap: int) -> int:
        count, load = 1, 0
        for r in rows:
            if load + r > cap and load > 0:
                count, load = count + 1, 0
            load += r
        return count

    lo, hi = max(rows), sum(rows)
    while lo < hi:                                   # smallest cap that fits in `world` contiguous blocks
        mid = (lo + hi) // 2
        if blocks_needed(mid) <= world:
            hi = mid
        else:
            lo = mid + 1
    ranges, begin, load = [], 0, 0
    for i, r in enumerate(rows):
        remaining_ranks = world - len(ranges) - 1
        # close the block when the next expert would exceed the cap, or when every remaining rank needs an expert
        if i > begin and (load + r > lo) and remaining_ranks > 0:
            ranges.append((begin, i))
            begin, load = i, 0
        load += r
    ranges.append((begin, n))
    while len(ranges) < world:                       # fewer blocks than ranks: the last ranks get nothing
        ranges.append((n, n))
    return ranges


def psum_from_sizes(sizes: list[int]) -> tuple[int, list[int]]:
    """Per-group row counts -> (total rows incl. padding, psum list of end rows); tests/generators.py:212-220."""
    psum, out = 0, []
    for s in sizes:
        out.append(psum + s)
        psum = _align(psum + s)
    return psum, out


def shard_psum_layout(sizes: list[int], world: int, rank: int) -> dict:
    """Local view of a global m-grouped problem for one rank."""
    begin, end = expert_range(len(sizes), world, rank)
    total_global, psum_global = psum_from_sizes(sizes)
    row_begin = _align(psum_global[begin - 1]) if begin > 0 else 0
    local_total, local_psum = psum_from_sizes(sizes[begin:end])
    return {'experts': (begin, end), 'row_begin': row_begin, 'rows': local_total, 'psum': local_psum,
            'global_rows': total_global}


def column_range(n: int, world: int, rank: int, multiple: int = 8) -> tuple[int, int]:
    """Columns of D owned by `rank` for the dense GEMM; boundaries are multiples of `multiple` (TMA alignment)."""
    blocks = (n + multiple - 1) // multiple
    b0, b1 = expert_range(blocks, world, rank)
    return min(b0 * multiple, n), min(b1 * multiple, n)
