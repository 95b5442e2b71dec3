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
    of every rank's copy (index = rank), and a stream-ordered cross-rank barrier;
    ``barrier.peer_views`` holds every rank's copy as a tensor of this process (for
    peer-to-peer copies).  Peers are reached with plain stores, TMA stores or copy-engine
    copies (no multicast objects are used by this package's kernels)."""
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
    barrier.peer_views = [           # type: ignore[attr-defined]
        handle.get_buffer(peer, (m_total, n), torch.float32) for peer in range(len(peer_bases))]
    return c_full, peer_bases, barrier


class _PanelStreams:
    """The streams of the panel schedule: panel launches alternate between two compute streams,
    so that the CTAs of the next panel's kernel fill the SMs the previous kernel's CTAs leave as
    they run out of tiles (one persistent launch per panel would otherwise idle part of the GPU
    at the end of every panel); peer-to-peer copies run on one stream per peer, each ordered
    after its panel's kernel by an event."""

    def __init__(self, peers: int, copy_streams: int = 0) -> None:
        import torch

        self.torch = torch
        self.compute = [torch.cuda.Stream(), torch.cuda.Stream()]
        # One stream per peer lets the copies to different peers run on different copy engines
        # at once; how streams map to engines is the driver's business, though, and two streams
        # that land on one engine take turns.  With a single stream the copies go out one after
        # the other, each at the full rate of the links, in an order that is the same every time.
        self.copies = [torch.cuda.Stream() for _ in range(copy_streams or peers)]
        self.event = None

    def begin(self) -> None:
        current = self.torch.cuda.current_stream()
        for stream in self.compute:
            stream.wait_stream(current)           # the operands are ready

    def launch(self, panel: int, run) -> None:
        stream = self.compute[panel % 2]
        with self.torch.cuda.stream(stream):
            run()
            self.event = self.torch.cuda.Event()
            self.event.record(stream)

    def copy_panel(self, destinations, source) -> None:
        """Push the panel that was launched last to every peer: one copy-engine copy per peer."""
        for index, destination in enumerate(destinations):
            stream = self.copies[index % len(self.copies)]
            stream.wait_event(self.event)
            with self.torch.cuda.stream(stream):
                destination.copy_(source, non_blocking=True)

    def join(self) -> None:
        current = self.torch.cuda.current_stream()
        for stream in (*self.compute, *self.copies):
            current.wait_stream(stream)


class RowShardedGemm:
    """``step(a_shard, b)`` leaves the full C on every rank.

    Three schedules:
    * gather (default): local GEMM, then one in-place NCCL all-gather of the row shards;
    * fused (``peer_bases`` given): the GEMM's epilogue writes every finished tile to
      all ranks' C directly, so the transfer overlaps the math tile by tile; a
      stream-ordered barrier afterwards tells each rank its peers are done;
    * panels (``peer_views`` and ``panel_rows`` given): the shard is computed in row panels
      by successive launches (alternating between two streams, so that the GPU stays full
      across panel boundaries); as soon as a panel is done the copy engines push it to every
      peer (one stream per peer) while the next panels compute, then the same barrier.
      The SMs do no communication work at all and copy-engine transfers use the links a
      little better than stores issued by SMs, at the price of one panel's GEMM time that
      nothing overlaps.
    """

    def __init__(self, m_total: int, n: int, c_full, gemm: Callable, group=None,
                 peer_bases: list[int] | None = None, barrier: Callable | None = None,
                 guard_reuse: bool = True, peer_views: list | None = None, panel_rows: int = 0,
                 push=None, copy_streams: int = 0) -> None:
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
        self.panel_rows = 0
        if peer_views is not None:
            if peer_bases is not None:
                raise ValueError("give peer_bases (fused epilogue) or peer_views (panel copies), not both")
            if len(peer_views) != self.world or barrier is None:
                raise ValueError("panel mode needs one view of C per rank and a barrier")
            rows = self.hi - self.lo
            if panel_rows <= 0 or rows % panel_rows:
                raise ValueError(f"panel_rows={panel_rows} does not divide the shard of {rows} rows")
            self.panel_rows = panel_rows
            # the peers in ring order starting after this rank, so that at any moment the
            # ranks are sending to different GPUs
            order = [(self.rank + step) % self.world for step in range(1, self.world)]
            self._peer_rows = [peer_views[peer][self.lo:self.hi] for peer in order]
            self._push = push or _PanelStreams(len(order), copy_streams)
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

    @property
    def panelled(self) -> bool:
        return self.panel_rows > 0

    @property
    def schedule(self) -> str:
        return "fused" if self.fused else "panels" if self.panelled else "gather"

    def compute(self, a_shard, b) -> None:
        if self.fused:
            self.gemm(a_shard, b, self.c_rows, self.destinations)
        elif self.panelled and self.world > 1:
            self._push.begin()
            for panel, start in enumerate(range(0, self.hi - self.lo, self.panel_rows)):
                stop = start + self.panel_rows
                self._push.launch(
                    panel, lambda: self.gemm(a_shard[start:stop], b, self.c_rows[start:stop]))
                self._push.copy_panel([peer_rows[start:stop] for peer_rows in self._peer_rows],
                                      self.c_rows[start:stop])
            self._push.join()
        else:
            self.gemm(a_shard, b, self.c_rows)

    def gather(self) -> None:
        if self.world == 1:
            return
        if self.fused or self.panelled:
            self.barrier()
        else:
            self.dist.all_gather_into_tensor(self.c_full, self.c_rows, group=self.group)

    def step(self, a_shard, b) -> None:
        """Leaves the full C on this rank (stream-ordered: work queued on the current stream after
        ``step`` sees it).

        In the fused and panel schedules the peers write straight into this rank's C, so step i+1 of a
        faster peer could overwrite rows that this rank is still reading from step i.  With
        ``guard_reuse`` (the default) every step after the first therefore starts with a barrier:
        the barrier is stream-ordered, so no rank's kernel begins to write until every rank's
        stream has run whatever it queued before this step, its reads of the previous result
        included.  Pass ``guard_reuse=False`` only if C is not read between steps or the caller
        orders the ranks itself."""
        if (self.fused or self.panelled) and self.guard_reuse and self._steps and self.world > 1:
            self.barrier()
        self._steps += 1
        self.compute(a_shard, b)
        self.gather()
