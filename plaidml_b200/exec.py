"""Execution: device list and ``Executable``.  Mirror of ``plaidml/exec/__init__.py:25-66``."""

from __future__ import annotations

import numpy as np

from .core import Buffer, DType, Program, TensorShape
from .ffi import ForeignObject, decode_str, ffi, ffi_call, get_strings, lib


def list_devices() -> list[str]:
    return get_strings(lib.plaidml_devices_get)


class Executable(ForeignObject):
    __ffi_del__ = lib.plaidml_executable_free

    def __init__(self, program: Program, device: str = ""):
        self.program = program
        super().__init__(ffi_call(lib.plaidml_jit, program.as_ptr(), device.encode()))

    def run(self, inputs, outputs) -> float:
        """Runs on ``Buffer`` lists; returns the elapsed milliseconds."""
        raw_in = [x.as_ptr() for x in inputs]
        raw_out = [x.as_ptr() for x in outputs]
        return ffi_call(lib.plaidml_executable_run, self.as_ptr(), len(raw_in), raw_in, len(raw_out), raw_out)

    # ---- inspection (additions of this library)
    def describe(self) -> str:
        return decode_str(ffi_call(lib.pmlb_exec_describe, self.as_ptr()))

    @property
    def launch_count(self) -> int:
        return ffi_call(lib.pmlb_exec_launch_count, self.as_ptr())

    @property
    def uses_graph(self) -> bool:
        """True once passes replay a captured CUDA graph of the kernel sequence."""
        return bool(ffi_call(lib.pmlb_exec_uses_graph, self.as_ptr()))

    @property
    def upload_groups(self) -> int:
        """Groups the inputs are uploaded in (1: all, then the kernels; more: uploads overlap the kernels)."""
        return int(ffi_call(lib.pmlb_exec_upload_groups, self.as_ptr()))

    def run_resident(self, iters: int = 1) -> float:
        """Mean milliseconds per iteration of the kernel sequence on device-resident inputs."""
        return ffi_call(lib.pmlb_exec_run_resident, self.as_ptr(), iters)

    def time_steps(self, iters: int = 1, flush_l2: bool = True) -> float:
        """Mean milliseconds per pass, each pass timed alone (CUDA events), L2 flushed before it."""
        return ffi_call(lib.pmlb_exec_time_steps, self.as_ptr(), iters, flush_l2)

    def time_passes(self, iters: int, flush_l2: bool = True) -> np.ndarray:
        """Milliseconds of each of ``iters`` passes, each timed alone (CUDA events), L2 flushed before it."""
        out = ffi.new("double[]", max(1, iters))
        ffi_call(lib.pmlb_exec_time_passes, self.as_ptr(), iters, flush_l2, out)
        return np.array([out[i] for i in range(iters)], dtype=np.float64)

    def time_each_step(self, iters: int = 3, flush_l2: bool = False) -> list[tuple[str, float]]:
        """(plan line, mean milliseconds) of every kernel step launched on its own."""
        n = ffi_call(lib.pmlb_exec_time_each_step, self.as_ptr(), iters, flush_l2, ffi.NULL, 0)
        out = ffi.new("double[]", max(1, n))
        ffi_call(lib.pmlb_exec_time_each_step, self.as_ptr(), iters, flush_l2, out, n)
        return list(zip(self.describe().strip().splitlines(), [out[i] for i in range(n)]))

    def set_input_replicated(self, index: int, replicated: bool = True) -> None:
        """Sharded mode: input ``index`` holds the same data on every rank; a run uploads this rank's
        1 / world slice and one all-gather over NVLink completes it on every GPU."""
        ffi_call(lib.pmlb_exec_set_input_replicated, self.as_ptr(), index, int(replicated))

    def gather_output(self, index: int = 0, iters: int = 1) -> tuple[int, int, float]:
        """Sharded mode: all ranks' copies of output ``index`` in rank order, in device memory the
        executable owns.  Returns (device address, bytes, mean milliseconds of one all-gather)."""
        nbytes = ffi.new("size_t*")
        ms = ffi.new("double*")
        ptr = ffi_call(lib.pmlb_exec_gather_output, self.as_ptr(), index, nbytes, iters, ms)
        return int(ffi.cast("uintptr_t", ptr)), int(nbytes[0]), float(ms[0])

    def output_device_ptr(self, index: int = 0) -> tuple[int, int]:
        nbytes = ffi.new("size_t*")
        ptr = ffi_call(lib.pmlb_exec_output_device_ptr, self.as_ptr(), index, nbytes)
        return int(ffi.cast("uintptr_t", ptr)), int(nbytes[0])

    @property
    def stream(self) -> int:
        return int(ffi.cast("uintptr_t", ffi_call(lib.pmlb_exec_stream, self.as_ptr())))


class Runner:
    """Convenience wrapper: numpy in, numpy out, buffers allocated once."""

    def __init__(self, program: Program, device: str = "", target: str = "cuda"):
        program.compile(target)
        self.program = program
        self.executable = Executable(program, device)
        self.inputs = [Buffer(shape) for shape in program.inputs]
        self.outputs = [Buffer(shape) for shape in program.outputs]
        self.last_ms = 0.0

    def run(self, arrays) -> list[np.ndarray]:
        for buf, arr in zip(self.inputs, arrays):
            buf.copy_from_ndarray(arr)
        self.last_ms = self.executable.run(self.inputs, self.outputs)
        return [buf.as_ndarray() for buf in self.outputs]


def run(program: Program, inputs, device: str = "cuda.0", target: str = "cuda") -> list[np.ndarray]:
    return Runner(program, device, target).run(inputs)
