"""Helpers shared by the GPU parity tests: seeded inputs, device buffers (torch is only the
allocator here), bf16 bit views and the comparison rules."""

from __future__ import annotations

import numpy as np
import torch

from plaidml_b200 import kernels as K

TORCH_OF = {
    K.F32: torch.float32, K.F16: torch.float16, K.BF16: torch.bfloat16, K.I8: torch.int8, K.I32: torch.int32,
    K.U8: torch.uint8, K.I16: torch.int16, K.I64: torch.int64, K.F64: torch.float64, K.BOOL: torch.uint8,
}


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def dev_bf16(a_f32: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a_f32, dtype=np.float32)).cuda().to(torch.bfloat16)


def bits16(t: torch.Tensor) -> np.ndarray:
    """uint16 bit pattern of a bf16 / f16 device tensor."""
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def as_f32(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.float32).cpu().numpy()


def empty(shape, dtype: int) -> torch.Tensor:
    return torch.empty(shape, dtype=TORCH_OF[dtype], device="cuda")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def max_rel(x: np.ndarray, ref: np.ndarray) -> float:
    """max |x - ref| / max |ref| (max-norm relative error)."""
    denom = float(np.max(np.abs(ref))) or 1.0
    return float(np.max(np.abs(x.astype(np.float64) - ref.astype(np.float64)))) / denom


def check_close(x: np.ndarray, ref: np.ndarray, tol: float) -> None:
    """The reference fixture's rule, |x - y| <= tol * (|x| + |y|) (plaidml/testenv.cc:52-67), with an
    absolute floor of tol * max|y| so that cancellation near zero does not dominate."""
    x = x.astype(np.float64)
    ref = ref.astype(np.float64)
    floor = tol * (float(np.max(np.abs(ref))) or 1.0)
    bad = np.abs(x - ref) > tol * (np.abs(x) + np.abs(ref)) + floor
    assert not bad.any(), f"{int(bad.sum())} of {bad.size} elements differ; max rel {max_rel(x, ref):.3e}"
