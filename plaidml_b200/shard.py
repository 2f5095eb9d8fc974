"""Data-parallel sharding of a contraction over one process per GPU.

The Tile contraction path has no exchange step: independent rows of the output (the M dimension of a
GEMM, the batch dimension of a convolution) are computed from independent rows of the first operand and a
replicated second operand, like the reference's threading of the outermost parallel loop over output
tiles (pmlc/target/x86/pipeline.cc:133-255 collapses scf.parallel for OpenMP, :374 converts it).  So
ranks share nothing on the data path; the only collectives are the barrier and the max-over-ranks of the
timed span, which use whatever process group is initialised (NCCL on GPUs, gloo in CPU tests).
"""

from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class RankInfo:
    rank: int
    local_rank: int
    world: int

    @staticmethod
    def from_env(env=None) -> "RankInfo":
        env = os.environ if env is None else env
        return RankInfo(int(env.get("RANK", "0")), int(env.get("LOCAL_RANK", "0")), int(env.get("WORLD_SIZE", "1")))

    @property
    def device_id(self) -> str:
        """The device string plaidml_jit takes for this rank (pattern name.N, pmlc/rt/device_id.cc:13-38)."""
        return f"cuda.{self.local_rank}"


def row_slice(total_rows: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the rows rank owns when `total_rows` are split as evenly as possible (strong scaling:
    the first total_rows % world ranks get one row more).  Every row belongs to exactly one rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if total_rows < 0:
        raise ValueError("negative row count")
    base, extra = divmod(total_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def weak_rows(rows_per_rank: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) in the global row numbering when every rank holds `rows_per_rank` rows (weak scaling)."""
    begin, end = row_slice(rows_per_rank * world, rank, world)
    return begin, end


def shard_seed(base_seed: int, rank: int) -> int:
    """Seed of a rank's private operand; the replicated operand uses `base_seed` itself on every rank."""
    return base_seed + 1000 * (rank + 1)


def barrier(dist) -> None:
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def max_over_ranks(dist, value: float, device=None) -> float:
    """The slowest rank's figure; `device` is where the one-element tensor lives (a CUDA device under NCCL)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, value: float, device=None) -> float:
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_floats(dist, value: float, device=None) -> list:
    """Every rank's figure, in rank order, on every rank (one all-gather of one element)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(value)]
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    out = torch.empty(dist.get_world_size(), dtype=torch.float64, device=device or "cpu")
    dist.all_gather_into_tensor(out, t)
    return [float(x) for x in out.tolist()]


def job_throughput(dist, units_this_rank: float, seconds_this_rank: float, device=None) -> float:
    """Whole-job rate: the units all ranks processed divided by the slowest rank's time."""
    units = sum_over_ranks(dist, units_this_rank, device)
    seconds = max_over_ranks(dist, seconds_this_rank, device)
    return units / seconds


# ---------------------------------------------------------------------------- the library's own communicator
#
# libplaidml.so carries the two collectives of the sharded mode itself (a replicated input completed by
# an all-gather, a gathered output), so that a C or C++ host needs no Python for them.  Its NCCL
# communicator is set up from a 128-byte id made on rank 0; here torch.distributed carries the id.

def exchange_id(dist, make_id, id_bytes: int = 128) -> bytes:
    """Rank 0 calls ``make_id()`` (-> bytes); every rank returns rank 0's id.  Works on any backend."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return bytes(id_bytes)
    box = [make_id() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    if not isinstance(box[0], (bytes, bytearray)) or len(box[0]) != id_bytes:
        raise RuntimeError("rank 0 did not deliver a communicator id")
    return bytes(box[0])


def init_library(dist, info: "RankInfo") -> None:
    """Joins this process to the library's communicator (collective over all ranks)."""
    from .ffi import ffi, ffi_call, lib

    def make_id() -> bytes:
        buf = ffi.new("char[128]")
        ffi_call(lib.pmlb_shard_unique_id, buf)
        return bytes(ffi.buffer(buf, 128))

    ident = exchange_id(dist, make_id) if info.world > 1 else bytes(128)
    ffi_call(lib.pmlb_shard_init, info.rank, info.world, ident, info.device_id.encode())


def shutdown_library() -> None:
    from .ffi import ffi_call, lib
    ffi_call(lib.pmlb_shard_shutdown)


# ---------------------------------------------------------------------------- gathered outputs
#
# Outputs stay sharded unless the caller asks for the whole tensor: then one all-gather of equal
# row slices puts every rank's rows on every rank (NCCL over NVLink when the tensors are on GPUs).

def all_gather_rows(dist, local):
    """`local` = this rank's [rows, ...] torch tensor (every rank the same shape); returns the
    [world * rows, ...] tensor holding rank 0's rows, then rank 1's, ...  One collective."""
    import torch
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return local.clone()
    world = dist.get_world_size()
    out = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous())
    return out


class _DeviceSpan:
    """A device address range as an object torch can adopt (CUDA array interface, version 3)."""

    def __init__(self, ptr: int, nbytes: int, stream: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "stream": stream or 1}


def output_tensor(executable, index: int = 0):
    """Output `index` of an executable as a flat uint8 torch tensor over the executable's own device
    memory (no copy; valid while the executable lives and until its next run overwrites it)."""
    import torch
    ptr, nbytes = executable.output_device_ptr(index)
    return torch.as_tensor(_DeviceSpan(ptr, nbytes, executable.stream), device="cuda")


def gather_output(dist, executable, index: int = 0):
    """All ranks' copies of output `index` (sharded along its first dimension), concatenated in rank
    order on every rank: a uint8 tensor of world x nbytes.  The caller views it with the output's
    element type.  The executable's stream is synchronised first."""
    import torch
    local = output_tensor(executable, index)
    torch.cuda.current_stream().synchronize()
    return all_gather_rows(dist, local.reshape(1, -1)).reshape(-1)
