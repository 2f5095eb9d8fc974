"""Core objects: ``DType``, ``TensorShape``, ``Buffer``, ``Program``, settings.

Python mirror of the reference's ``plaidml/core/__init__.py:72-338`` over the same C calls.
"""

from __future__ import annotations

import enum

import numpy as np

from .ffi import Error, ForeignObject, decode_str, ffi, ffi_call, get_strings, lib


class DType(enum.IntEnum):
    INVALID = 0
    INTX = 1
    UINTX = 2
    FLOATX = 3
    BOOLEAN = 4
    INT8 = 5
    UINT8 = 6
    INT16 = 7
    UINT16 = 8
    INT32 = 9
    UINT32 = 10
    INT64 = 11
    UINT64 = 12
    FLOAT16 = 13
    FLOAT32 = 14
    FLOAT64 = 15
    BFLOAT16 = 16  # addition of this library; numpy sees it as uint16 bit patterns

    @staticmethod
    def from_numpy(dtype) -> "DType":
        return _NP_TO_DTYPE[np.dtype(dtype).name]

    def into_numpy(self):
        return _DTYPE_TO_NP[self]


_NP_TO_DTYPE = {
    "bool": DType.BOOLEAN, "int8": DType.INT8, "uint8": DType.UINT8, "int16": DType.INT16,
    "uint16": DType.UINT16, "int32": DType.INT32, "uint32": DType.UINT32, "int64": DType.INT64,
    "uint64": DType.UINT64, "float16": DType.FLOAT16, "float32": DType.FLOAT32, "float64": DType.FLOAT64,
}
_DTYPE_TO_NP = {v: k for k, v in _NP_TO_DTYPE.items()}
_DTYPE_TO_NP[DType.BFLOAT16] = "uint16"
_DTYPE_TO_NP[DType.INTX] = "int32"
_DTYPE_TO_NP[DType.UINTX] = "uint32"
_DTYPE_TO_NP[DType.FLOATX] = "float32"


def _integers(raw) -> list[int]:
    try:
        return [raw.elts[i] for i in range(raw.size)]
    finally:
        ffi_call(lib.plaidml_integers_free, raw)


class TensorShape(ForeignObject):
    __ffi_del__ = lib.plaidml_shape_free
    __ffi_repr__ = lib.plaidml_shape_repr

    def __init__(self, dtype=None, sizes=(), strides=None, ptr=None):
        if ptr is None:
            sizes = [int(s) for s in sizes]
            raw_strides = ffi.NULL if strides is None else ffi.new("int64_t[]", [int(s) for s in strides])
            ptr = ffi_call(lib.plaidml_shape_alloc, int(dtype), len(sizes), ffi.new("int64_t[]", sizes), raw_strides)
        super().__init__(ptr)

    @property
    def dtype(self) -> DType:
        return DType(ffi_call(lib.plaidml_shape_get_dtype, self.as_ptr()))

    @property
    def rank(self) -> int:
        return ffi_call(lib.plaidml_shape_get_rank, self.as_ptr())

    @property
    def sizes(self) -> list[int]:
        return _integers(ffi_call(lib.plaidml_shape_get_sizes, self.as_ptr()))

    @property
    def strides(self) -> list[int]:
        return _integers(ffi_call(lib.plaidml_shape_get_strides, self.as_ptr()))

    @property
    def byte_size(self) -> int:
        return ffi_call(lib.plaidml_shape_get_nbytes, self.as_ptr())

    def into_TensorShape(self):
        return self


class Buffer(ForeignObject):
    """Host storage of a tensor (page-locked when a CUDA driver is present)."""

    __ffi_del__ = lib.plaidml_buffer_free

    def __init__(self, shape: TensorShape = None, data=None, ptr=None):
        self._keepalive = None
        if ptr is None:
            if data is not None and shape is None:
                arr = np.ascontiguousarray(data)
                shape = TensorShape(DType.from_numpy(arr.dtype), arr.shape)
            ptr = ffi_call(lib.plaidml_buffer_alloc, shape.as_ptr())
        super().__init__(ptr)
        if data is not None:
            self.copy_from_ndarray(np.asarray(data))

    @staticmethod
    def adopt(array: np.ndarray, dtype: DType = None) -> "Buffer":
        """Borrows the memory of a C-contiguous array for the buffer's lifetime."""
        if not array.flags["C_CONTIGUOUS"]:
            raise ValueError("only C-contiguous arrays can be adopted")
        shape = TensorShape(dtype if dtype is not None else DType.from_numpy(array.dtype), array.shape)
        raw = ffi.from_buffer(array, require_writable=True)
        buf = Buffer(ptr=ffi_call(lib.plaidml_buffer_adopt, shape.as_ptr(), ffi.cast("char*", raw), array.nbytes))
        buf._keepalive = (array, raw)
        return buf

    @property
    def shape(self) -> TensorShape:
        return TensorShape(ptr=ffi_call(lib.plaidml_buffer_shape, self.as_ptr()))

    @property
    def size(self) -> int:
        return ffi_call(lib.plaidml_buffer_size, self.as_ptr())

    def _view(self) -> np.ndarray:
        shape = self.shape
        data = ffi_call(lib.plaidml_buffer_data, self.as_ptr())
        raw = ffi.buffer(data, self.size)
        return np.frombuffer(raw, dtype=shape.dtype.into_numpy()).reshape(shape.sizes)

    def as_ndarray(self) -> np.ndarray:
        """A copy of the contents (bf16 comes back as uint16 bit patterns)."""
        return self._view().copy()

    def copy_from_ndarray(self, src: np.ndarray) -> None:
        view = self._view()
        np.copyto(view, np.asarray(src).reshape(view.shape), casting="unsafe")

    def copy_to_ndarray(self, dst: np.ndarray) -> None:
        np.copyto(dst, self._view().reshape(dst.shape), casting="unsafe")


class Program(ForeignObject):
    """A built program; ``compile`` selects the target (default: ``$PLAIDML_TARGET``)."""

    __ffi_del__ = lib.plaidml_program_free
    __ffi_repr__ = lib.plaidml_program_repr

    def __init__(self, name, inputs, outputs, shapes=None, ptr=None):
        if ptr is None:
            raw_in = [x.as_ptr() for x in inputs]
            raw_out = [x.as_ptr() for x in outputs]
            raw_shapes = ffi.NULL if shapes is None else [s.as_ptr() for s in shapes]
            ptr = ffi_call(lib.plaidml_build, name.encode(), len(raw_in), raw_in, raw_shapes, len(raw_out), raw_out)
        super().__init__(ptr)

    def compile(self, target="", debug=False):
        ffi_call(lib.plaidml_program_compile, self.as_ptr(), debug, target.encode())
        return self

    def _shapes(self, func) -> list[TensorShape]:
        raw = ffi_call(func, self.as_ptr())
        try:
            return [TensorShape(ptr=raw.elts[i]) for i in range(raw.size)]
        finally:
            ffi_call(lib.plaidml_shapes_free, raw)

    @property
    def inputs(self) -> list[TensorShape]:
        return self._shapes(lib.plaidml_program_get_inputs)

    @property
    def outputs(self) -> list[TensorShape]:
        return self._shapes(lib.plaidml_program_get_outputs)

    @property
    def passes(self) -> list[tuple[str, str]]:
        raw = ffi_call(lib.plaidml_program_get_passes, self.as_ptr())
        try:
            return [(decode_str(raw.elts[i].key), decode_str(raw.elts[i].value)) for i in range(raw.size)]
        finally:
            ffi_call(lib.plaidml_kvps_free, raw)


def list_targets() -> list[str]:
    return get_strings(lib.plaidml_targets_get)


def settings_get(key: str) -> str:
    return decode_str(ffi_call(lib.plaidml_settings_get, key.encode()))


def settings_set(key: str, value: str) -> None:
    ffi_call(lib.plaidml_settings_set, key.encode(), value.encode())


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Rounds float32 to bfloat16 (nearest even) and returns the uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (0x7FFF + ((u >> 16) & 1))
    return (rounded >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
