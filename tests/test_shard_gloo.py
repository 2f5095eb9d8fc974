"""The N > 1 path on CPU: two gloo ranks shard the rows of a contraction, compute their slices with the CPU
checker, and the slices tile the unsharded answer exactly; the job-level timing reductions (max of the
spans, sum of the units) behave as bench.py relies on."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from plaidml_b200 import shard


def test_row_slices_partition_every_row_once():
    for total in (0, 1, 7, 4096, 4099):
        for world in (1, 2, 3, 8):
            spans = [shard.row_slice(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[r][1] == spans[r + 1][0] for r in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.row_slice(8, 2, 2)
    assert shard.weak_rows(4096, 1, 2) == (4096, 8192)


def test_rank_info_reads_the_launcher_environment():
    info = shard.RankInfo.from_env({"RANK": "5", "LOCAL_RANK": "1", "WORLD_SIZE": "8"})
    assert (info.rank, info.local_rank, info.world, info.device_id) == (5, 1, 8, "cuda.1")
    assert shard.RankInfo.from_env({}).world == 1
    assert shard.shard_seed(10, 0) != shard.shard_seed(10, 1) != 10


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        info = shard.RankInfo.from_env()
        m, n, k = 37, 24, 48                                  # 37 rows do not divide by 2
        g = np.random.Generator(np.random.PCG64(7))           # the replicated operand: same seed everywhere
        b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
        a_full = np.random.Generator(np.random.PCG64(8)).integers(-128, 128, size=(m, k), dtype=np.int8)
        lo, hi = shard.row_slice(m, info.rank, info.world)
        c_part = oracle.gemm_i8_i32(np.ascontiguousarray(a_full[lo:hi]), b)
        np.save(os.path.join(out_dir, f"c{rank}.npy"), c_part)
        shard.barrier(dist)
        slowest = shard.max_over_ranks(dist, 1.0 + rank)
        units = shard.sum_over_ranks(dist, float(hi - lo))
        assert shard.gather_floats(dist, 1.0 + rank) == [1.0 + r for r in range(world)]
        rate = shard.job_throughput(dist, float(hi - lo), 1.0 + rank)
        np.save(os.path.join(out_dir, f"t{rank}.npy"), np.array([slowest, units, rate, lo, hi]))
        # the communicator id of the library's own collectives travels from rank 0 to everyone
        ident = shard.exchange_id(dist, lambda: bytes(range(128)))
        assert ident == bytes(range(128))
        # gathered output: equal slices only (pad the ragged last shard as the caller would)
        mine = torch.full((3, 4), float(rank), dtype=torch.float32)
        whole = shard.all_gather_rows(dist, mine)
        np.save(os.path.join(out_dir, f"g{rank}.npy"), whole.numpy())
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_tile_the_unsharded_result(tmp_path):
    import oracle
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    m, n, k = 37, 24, 48
    b = np.random.Generator(np.random.PCG64(7)).integers(-128, 128, size=(k, n), dtype=np.int8)
    a = np.random.Generator(np.random.PCG64(8)).integers(-128, 128, size=(m, k), dtype=np.int8)
    whole = oracle.gemm_i8_i32(a, b)
    parts = [np.load(tmp_path / f"c{r}.npy") for r in range(world)]
    assert np.array_equal(np.concatenate(parts, axis=0), whole)
    for r in range(world):
        slowest, units, rate, lo, hi = np.load(tmp_path / f"t{r}.npy")
        assert slowest == 2.0 and units == m and rate == m / 2.0
        assert (lo, hi) == shard.row_slice(m, r, world)
        gathered = np.load(tmp_path / f"g{r}.npy")
        assert gathered.shape == (6, 4) and (gathered[:3] == 0).all() and (gathered[3:] == 1).all()


def test_single_process_reductions_are_identities():
    assert shard.max_over_ranks(None, 3.5) == 3.5
    assert shard.sum_over_ranks(None, 3.5) == 3.5
    assert shard.gather_floats(None, 3.5) == [3.5]
    assert shard.job_throughput(None, 10.0, 2.0) == 5.0
    shard.barrier(None)
    assert shard.exchange_id(None, lambda: b"x" * 128) == bytes(128)   # a world of one needs no id
    t = torch.arange(6.0).reshape(2, 3)
    assert torch.equal(shard.all_gather_rows(None, t), t)
    assert isinstance(torch.__version__, str)
