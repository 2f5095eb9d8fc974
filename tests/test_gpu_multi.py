"""Two ranks on two GPUs: each computes its rows of an int8 GEMM, the gathered output equals the
unsharded product.  Needs two devices; skipped otherwise."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from plaidml_b200 import programs, shard
        from plaidml_b200.core import DType, Program
        from plaidml_b200.exec import Runner
        info = shard.RankInfo.from_env()
        rows, n, k = 256, 384, 512
        b = np.random.Generator(np.random.PCG64(7)).integers(-128, 128, size=(k, n), dtype=np.int8)
        a = np.random.Generator(np.random.PCG64(shard.shard_seed(7, rank))).integers(-128, 128, size=(rows, k), dtype=np.int8)
        A, B, C = programs.tile_gemm(DType.INT8, rows, n, k, acc=DType.INT32)
        runner = Runner(Program("shard", [A, B], [C]), info.device_id)
        c_local = runner.run([a, b])[0]
        whole = shard.gather_output(dist, runner.executable, 0).view(torch.int32).reshape(world * rows, n)
        np.save(os.path.join(out_dir, f"whole{rank}.npy"), whole.cpu().numpy())
        np.save(os.path.join(out_dir, f"local{rank}.npy"), c_local)
        # the same two collectives inside the library (its own NCCL communicator): B is marked replicated and
        # every rank's host copy holds only its own 1 / world of the bytes (the rest is poisoned), so a
        # correct product proves that the all-gather completed the operand; the output is gathered by
        # pmlb_exec_gather_output into memory the executable owns
        shard.init_library(dist, info)
        runner2 = Runner(Program("shard_lib", [A, B], [C]), info.device_id)
        runner2.executable.set_input_replicated(1, True)
        flat = b.reshape(-1).copy()
        part = flat.size // world
        poisoned = np.full_like(flat, 77)
        poisoned[rank * part:(rank + 1) * part] = flat[rank * part:(rank + 1) * part]
        c_lib = runner2.run([a, poisoned.reshape(b.shape)])[0]
        ptr, nbytes, _ = runner2.executable.gather_output(0)
        assert nbytes == world * rows * n * 4
        span = shard._DeviceSpan(ptr, nbytes, runner2.executable.stream)
        whole2 = torch.as_tensor(span, device="cuda").view(torch.int32).reshape(world * rows, n)
        np.save(os.path.join(out_dir, f"libwhole{rank}.npy"), whole2.cpu().numpy())
        np.save(os.path.join(out_dir, f"liblocal{rank}.npy"), c_lib)
        del runner2
        shard.shutdown_library()
    finally:
        dist.destroy_process_group()


def test_two_gpus_gather_the_sharded_product(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import oracle
    import torch.multiprocessing as mp
    from plaidml_b200 import shard
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    b = np.random.Generator(np.random.PCG64(7)).integers(-128, 128, size=(512, 384), dtype=np.int8)
    parts = []
    for r in range(2):
        a = np.random.Generator(np.random.PCG64(shard.shard_seed(7, r))).integers(-128, 128, size=(256, 512), dtype=np.int8)
        parts.append(oracle.gemm_i8_i32(a, b))
    ref = np.concatenate(parts, axis=0)
    for r in range(2):
        np.testing.assert_array_equal(np.load(tmp_path / f"whole{r}.npy"), ref)
        np.testing.assert_array_equal(np.load(tmp_path / f"local{r}.npy"), parts[r])
        np.testing.assert_array_equal(np.load(tmp_path / f"libwhole{r}.npy"), ref)
        np.testing.assert_array_equal(np.load(tmp_path / f"liblocal{r}.npy"), parts[r])
