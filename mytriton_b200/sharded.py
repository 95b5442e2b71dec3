"""Row-sharded GEMM over the GPUs of one node.

Rank r owns rows ``[r*M/g, (r+1)*M/g)`` of A, a full copy of B, and computes the
matching rows of C with the tl.dot kernel; because C is row-major the shards are
contiguous, so assembling C on every rank is one in-place all-gather along rows
(NCCL over NVLink).  The reference has no multi-device path; this is the M-sharded
configuration of the benchmark.

The class only orchestrates: the matmul is injected (``gemm(a, b, c_rows)``), so
the partitioning and the gather can be tested on CPU ranks with the ``gloo``
backend and a NumPy/torch matmul in place of the GPU kernel.
"""

from __future__ import annotations

from typing import Callable


def shard_bounds(m_total: int, world: int, rank: int, align: int = 128) -> tuple[int, int]:
    """Half-open row range of ``rank``.  Shards are equal and ``align``-row aligned."""
    if m_total % world:
        raise ValueError(f"M={m_total} does not divide evenly over {world} ranks")
    rows = m_total // world
    if rows % align:
        raise ValueError(f"shard of {rows} rows is not a multiple of the {align}-row tile")
    return rank * rows, (rank + 1) * rows


def symmetric_output(m_total: int, n: int, device, group=None):
    """Allocate C[m_total, n] fp32 in symmetric memory and exchange peer addresses.

    Returns ``(c_full, peer_bases, barrier)``: the local tensor, the device address
    of every rank's copy (index = rank), and a stream-ordered cross-rank barrier.
    Peers are reached with plain stores / TMA stores (no multicast objects are used
    by this package's kernels)."""
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    group = group or dist.group.WORLD
    c_full = symm_mem.empty((m_total, n), dtype=torch.float32, device=device)
    handle = symm_mem.rendezvous(c_full, group)
    peer_bases = [int(ptr) for ptr in handle.buffer_ptrs]

    def barrier() -> None:
        handle.barrier()

    barrier.handle = handle          # type: ignore[attr-defined]  (keeps the mapping alive)
    return c_full, peer_bases, barrier


class RowShardedGemm:
    """``step(a_shard, b)`` leaves the full C on every rank.

    Two schedules:
    * gather (default): local GEMM, then one in-place NCCL all-gather of the row shards;
    * fused (``peer_bases`` given): the GEMM's epilogue writes every finished tile to
      all ranks' C directly, so the transfer overlaps the math tile by tile; a
      stream-ordered barrier afterwards tells each rank its peers are done.
    """

    def __init__(self, m_total: int, n: int, c_full, gemm: Callable, group=None,
                 peer_bases: list[int] | None = None, barrier: Callable | None = None,
                 guard_reuse: bool = True) -> None:
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = shard_bounds(m_total, self.world, self.rank)
        if tuple(c_full.shape) != (m_total, n):
            raise ValueError(f"C must be [{m_total}, {n}], got {tuple(c_full.shape)}")
        if not c_full.is_contiguous():
            raise ValueError("C must be contiguous (row shards are gathered in place)")
        self.c_full = c_full
        self.c_rows = c_full[self.lo:self.hi]
        self.gemm = gemm
        self.barrier = barrier
        self.guard_reuse = guard_reuse
        self._steps = 0
        self.destinations = None
        if peer_bases is not None:
            if len(peer_bases) != self.world or barrier is None:
                raise ValueError("fused mode needs one base address per rank and a barrier")
            offset = self.lo * n * c_full.element_size()
            # own copy first, then the peers in ring order starting after this rank, so
            # that at any moment the ranks are writing to different GPUs
            order = [(self.rank + step) % self.world for step in range(self.world)]
            self.destinations = [peer_bases[peer] + offset for peer in order]

    @property
    def fused(self) -> bool:
        return self.destinations is not None

    def compute(self, a_shard, b) -> None:
        if self.fused:
            self.gemm(a_shard, b, self.c_rows, self.destinations)
        else:
            self.gemm(a_shard, b, self.c_rows)

    def gather(self) -> None:
        if self.world == 1:
            return
        if self.fused:
            self.barrier()
        else:
            self.dist.all_gather_into_tensor(self.c_full, self.c_rows, group=self.group)

    def step(self, a_shard, b) -> None:
        """Leaves the full C on this rank (stream-ordered: work queued on the current stream after
        ``step`` sees it).

        In the fused schedule the peers write straight into this rank's C, so step i+1 of a
        faster peer could overwrite rows that this rank is still reading from step i.  With
        ``guard_reuse`` (the default) every step after the first therefore starts with a barrier:
        the barrier is stream-ordered, so no rank's kernel begins to write until every rank's
        stream has run whatever it queued before this step, its reads of the previous result
        included.  Pass ``guard_reuse=False`` only if C is not read between steps or the caller
        orders the ranks itself."""
        if self.fused and self.guard_reuse and self._steps:
            self.barrier()
        self._steps += 1
        self.compute(a_shard, b)
        self.gather()
