"""World-size-2 test of the row-sharded GEMM orchestration on CPU (gloo): every rank
must end up with the full product, assembled from the row shards in rank order."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mytriton_b200.sharded import RowShardedGemm, shard_bounds


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, n: int, k: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)
        a = torch.randn(m, k, generator=gen)
        b = torch.randn(k, n, generator=gen)
        lo, hi = shard_bounds(m, world, rank)
        c = torch.full((m, n), float("nan"))

        def gemm(a_rows, b_full, c_rows):
            torch.matmul(a_rows, b_full, out=c_rows)

        job = RowShardedGemm(m, n, c, gemm)
        job.step(a[lo:hi], b)
        np.save(os.path.join(out_dir, f"c{rank}.npy"), c.numpy())
        np.save(os.path.join(out_dir, f"ref{rank}.npy"), (a @ b).numpy())
    finally:
        dist.destroy_process_group()


def test_two_ranks_assemble_the_full_product(tmp_path):
    m, n, k, world = 256, 64, 32, 2
    mp.spawn(_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        c = np.load(tmp_path / f"c{rank}.npy")
        ref = np.load(tmp_path / f"ref{rank}.npy")
        assert not np.isnan(c).any()
        np.testing.assert_allclose(c, ref, rtol=1e-5, atol=1e-5)


def test_shard_bounds():
    assert shard_bounds(65536, 8, 3) == (24576, 32768)
    assert shard_bounds(65536, 1, 0) == (0, 65536)
    with pytest.raises(ValueError):
        shard_bounds(1000, 3, 0)
    with pytest.raises(ValueError):
        shard_bounds(256, 4, 0)          # 64-row shards are not tile aligned


def _failing_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    """Rank 1 fails on the host before the step; rank 0 must get an error from the
    gather within the process-group timeout instead of waiting for ever."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=4))
    outcome = "finished"
    try:
        if rank == 1:
            raise RuntimeError("injected host failure before the step")
        c = torch.zeros(256, 8)
        job = RowShardedGemm(256, 8, c, lambda a, b, rows: rows.fill_(1.0))
        started = time.monotonic()
        try:
            job.step(None, None)
        except Exception as error:                      # the collective gives up: good
            outcome = f"error after {time.monotonic() - started:.1f}s: {type(error).__name__}"
    except RuntimeError as error:
        outcome = f"raised: {error}"
    finally:
        with open(os.path.join(out_dir, f"outcome{rank}.txt"), "w") as handle:
            handle.write(outcome)
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_dies_on_the_host_does_not_hang_its_peer(tmp_path):
    mp.spawn(_failing_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    survivor = (tmp_path / "outcome0.txt").read_text()
    failed = (tmp_path / "outcome1.txt").read_text()
    assert failed.startswith("raised: injected host failure")
    assert survivor.startswith("error after"), survivor
    assert float(survivor.split()[2].rstrip("s:")) < 30.0


def test_fused_steps_are_separated_by_a_barrier_so_peers_cannot_overwrite_rows_being_read():
    """Single process, fake kernel and fake barrier: the order of events of three fused steps.
    Every step after the first must open with a barrier (peers may still read the previous C),
    and every step ends with one (the peers' stores have landed)."""
    events = []
    c = torch.zeros(256, 8)

    def gemm(a_rows, b_full, c_rows, destinations):
        events.append(("gemm", tuple(destinations)))

    job = RowShardedGemm(256, 8, c, gemm, peer_bases=[4096], barrier=lambda: events.append("barrier"))
    job.world = 2                                            # as on a rank of a two-rank job
    for _ in range(3):
        job.step(None, None)
    kinds = [e if isinstance(e, str) else e[0] for e in events]
    assert kinds == ["gemm", "barrier", "barrier", "gemm", "barrier", "barrier", "gemm", "barrier"]
    assert events[0][1] == (4096,)                           # own rows of the own copy: offset 0
    events.clear()
    loose = RowShardedGemm(256, 8, c, gemm, peer_bases=[4096], barrier=lambda: events.append("barrier"),
                           guard_reuse=False)
    loose.world = 2
    loose.step(None, None)
    loose.step(None, None)
    assert [e if isinstance(e, str) else e[0] for e in events] == ["gemm", "barrier", "gemm", "barrier"]


def test_panel_schedule_pushes_every_panel_to_every_peer_after_its_gemm():
    """Single process, fake GEMM and fake copy engine: order of events of the panel schedule on
    rank 0 of three, and the rows each copy moves."""
    events = []
    m, n, world = 768, 4, 3
    mine = torch.zeros(m, n)
    peers = [mine, torch.zeros(m, n), torch.zeros(m, n)]

    def gemm(a_rows, b_full, c_rows):
        c_rows.copy_(a_rows)
        events.append(("gemm", a_rows.shape[0]))

    class Push:
        def begin(self):
            events.append("begin")

        def launch(self, panel, run):
            run()
            events.append(("done", panel))

        def copy_panel(self, destinations, source):
            for index, destination in enumerate(destinations):
                destination.copy_(source)
                events.append(("copy", index))

        def join(self):
            events.append("join")

    job = RowShardedGemm.__new__(RowShardedGemm)           # no process group here: fill in what init would
    job.dist, job.group, job.world, job.rank = None, None, world, 0
    job.lo, job.hi = 0, 256
    job.c_full, job.c_rows, job.gemm = mine, mine[0:256], gemm
    job.barrier, job.guard_reuse, job._steps = (lambda: events.append("barrier")), True, 0
    job.destinations, job.panel_rows = None, 128
    job._peer_rows = [peers[1][0:256], peers[2][0:256]]
    job._push = Push()
    a = torch.arange(256 * n, dtype=torch.float32).reshape(256, n)
    job.step(a, None)
    assert events == ["begin", ("gemm", 128), ("done", 0), ("copy", 0), ("copy", 1),
                      ("gemm", 128), ("done", 1), ("copy", 0), ("copy", 1), "join", "barrier"]
    for peer in peers:
        assert torch.equal(peer[0:256], a) and not peer[256:].any()
    events.clear()
    job.step(a, None)
    assert events[0] == "barrier" and events[-1] == "barrier"


def test_panel_rows_must_divide_the_shard():
    with pytest.raises(ValueError, match="does not divide"):
        RowShardedGemm(256, 4, torch.zeros(256, 4), lambda *a: None, peer_views=[torch.zeros(256, 4)],
                       barrier=lambda: None, panel_rows=100)
