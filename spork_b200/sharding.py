"""Host-side partitioning of the two workloads across the GPUs of one box.

The GEMM is sharded over M: rank r owns a contiguous slab of rows of A and of C
and a full replica of B, so no rank ever needs another rank's data while the
clock runs.  Attention is sharded over the (batch x head) index the same way.
There is no counterpart in the reference (it is single-GPU: cudaSetDevice(0),
gemm/gemm_main.cpp:10); the partition is the only multi-GPU logic there is.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Slab:
    rank: int
    world: int
    start: int  # first row (or head) owned
    count: int  # rows (or heads) owned

    @property
    def stop(self) -> int:
        return self.start + self.count


def m_slab(M: int, rank: int, world: int, align: int = 256) -> Slab:
    """Rows [start, start+count) of an M-row problem owned by ``rank`` of ``world``.

    Slabs are contiguous, disjoint, cover [0, M) exactly and start on a multiple of
    ``align`` rows (the kernel's output-tile height) so that no output tile straddles
    two ranks.  When M is not a multiple of world*align the earlier ranks take one
    aligned block more; trailing ranks may own zero rows.
    """
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if M < 0 or align < 1:
        raise ValueError("M must be >= 0 and align >= 1")
    blocks = (M + align - 1) // align
    base, extra = divmod(blocks, world)
    my_blocks = base + (1 if rank < extra else 0)
    first_block = rank * base + min(rank, extra)
    start = min(first_block * align, M)
    stop = min((first_block + my_blocks) * align, M)
    return Slab(rank, world, start, stop - start)


def head_slab(BH: int, rank: int, world: int) -> Slab:
    """Contiguous block of the batch*heads index owned by ``rank`` (attention)."""
    return m_slab(BH, rank, world, align=1)


def whole_job_rate(units_per_rank: list[float], seconds_max_over_ranks: float) -> float:
    """Aggregate throughput of a sharded run: all ranks' work over the slowest rank's time."""
    if seconds_max_over_ranks <= 0:
        raise ValueError("time must be positive")
    return sum(units_per_rank) / seconds_max_over_ranks
