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
