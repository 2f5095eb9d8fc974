"""ctypes mirror of ``include/pmlb_kernels.h`` -- the kernel-level C ABI of ``libplaidml.so``.

The EDSL / exec layers do not need this module (the C++ planner calls the kernels
directly); it exists so that tests and benchmarks can drive single kernels with raw
device pointers, the way JIT-compiled code drives ``plaidml_rt_xsmm_*`` in the reference.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_NAME = "libplaidml.so"

# element types (== plaidml_datatype, BFLOAT16 appended)
BOOL, I8, U8, I16, U16, I32, U32, I64, U64, F16, F32, F64, BF16 = 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16
AGG_NONE, AGG_SUM, AGG_MAX, AGG_MIN, AGG_PROD, AGG_ASSIGN = range(6)
COMBO_NONE, COMBO_MUL, COMBO_ADD, COMBO_EQ, COMBO_COND = range(5)
EPI_BIAS, EPI_RESIDUAL, EPI_RELU, EPI_ROWMAX = 1, 2, 4, 8
GEMM_TRANSPOSE_B = 1
GEMM_PLAIN_STORES = 2
GEMM_PLAIN_RESIDUAL = 4
GEMM_CTA_PAIRS = 8
GEMM_NO_CTA_PAIRS = 16
GEMM_NO_TAIL_SPLIT = 32
GEMM_NO_SPLIT_K = 64
GEMM_SPLIT_K = 128
CONV_NO_PACKED_ROWS = 1
CONV_NO_HALO = 2
CONV_NO_S2D = 4
CONV_CTA_PAIRS = 8
CONV_NO_CTA_PAIRS = 16
CONV_NO_COLUMN_MERGE = 32
CONV_MAX_POOL_3X3_S2 = 64
SPECIAL_GATHER, SPECIAL_SCATTER, SPECIAL_ARGSORT, SPECIAL_PRNG = range(4)
OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT = range(5)

MAX_IDX, MAX_RANK, MAX_CONS = 10, 8, 8


class GemmDesc(C.Structure):
    _fields_ = [
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("batch", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64),
        ("b_is_nk", C.c_int32), ("epilogue", C.c_int32),
        ("ldr", C.c_int64), ("stride_r", C.c_int64),
        ("tile_n", C.c_int32), ("flags", C.c_int32),
        ("k_first", C.c_int32), ("a2_stride", C.c_int32), ("lda2", C.c_int64),
        ("a2_n", C.c_int32), ("a2_h", C.c_int32), ("a2_w", C.c_int32), ("reserved0", C.c_int32),
    ]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "in_dtype", "out_dtype", "n", "h", "w", "c", "r", "s", "k", "p", "q", "stride_h", "stride_w",
        "pad_h", "pad_w", "dil_h", "dil_w", "epilogue", "tile_n", "flags")]


class ReduceDesc(C.Structure):
    _fields_ = [
        ("agg", C.c_int32), ("dtype", C.c_int32), ("out_dtype", C.c_int32), ("divide", C.c_int32),
        ("outer", C.c_int64), ("reduce", C.c_int64), ("inner", C.c_int64), ("scale", C.c_double),
    ]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "agg", "dtype", "n", "h", "w", "c", "r", "s", "p", "q", "stride_h", "stride_w", "pad_h", "pad_w",
        "average", "include_padding")]


class Access(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("rank", C.c_int32),
        ("sizes", C.c_int64 * MAX_RANK), ("strides", C.c_int64 * MAX_RANK),
        ("coef", (C.c_int32 * MAX_IDX) * MAX_RANK),
        ("off", C.c_int64 * MAX_RANK), ("den", C.c_int32 * MAX_RANK),
    ]


class ContractDesc(C.Structure):
    _fields_ = [
        ("agg", C.c_int32), ("combo", C.c_int32), ("n_idx", C.c_int32), ("n_src", C.c_int32),
        ("range", C.c_int64 * MAX_IDX),
        ("out", Access), ("src", Access * 3),
        ("n_cons", C.c_int32), ("has_init", C.c_int32),
        ("cons_coef", (C.c_int32 * MAX_IDX) * MAX_CONS),
        ("cons_off", C.c_int64 * MAX_CONS), ("cons_range", C.c_int64 * MAX_CONS),
        ("init", Access),
    ]


class EltwiseDesc(C.Structure):
    _fields_ = [
        ("op", C.c_char * 24), ("n_in", C.c_int32), ("rank", C.c_int32), ("out_dtype", C.c_int32),
        ("in_dtype", C.c_int32 * 3),
        ("sizes", C.c_int64 * MAX_RANK), ("in_strides", (C.c_int64 * MAX_RANK) * 3),
    ]


class SpecialDesc(C.Structure):
    """gather / scatter / argsort / prng (``pmlb_special_desc``)."""
    _fields_ = [
        ("op", C.c_int32), ("dtype", C.c_int32), ("idx_dtype", C.c_int32),
        ("rank", C.c_int32), ("idx_rank", C.c_int32), ("upd_rank", C.c_int32),
        ("sizes", C.c_int64 * MAX_RANK), ("idx_sizes", C.c_int64 * MAX_RANK), ("upd_sizes", C.c_int64 * MAX_RANK),
        ("axis", C.c_int32), ("mode", C.c_int32), ("batch_dims", C.c_int32), ("interpolation", C.c_int32),
        ("nearest", C.c_int32), ("out_of_bounds", C.c_int32),
        ("cube_coeff", C.c_double), ("state_elems", C.c_int64),
    ]


class KernelError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"pmlb status {status}: {message}")
        self.status = status


def lib_path() -> Path:
    override = os.environ.get("PLAIDML_LIB_PATH")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / LIB_NAME


_lib = None


def load() -> C.CDLL:
    """Loads ``libplaidml.so``; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m plaidml_b200.build` (nvcc, sm_100a). "
            "There is no CPU fallback.")
    lib = C.CDLL(str(path))
    vp = C.c_void_p
    lib.pmlb_last_error.restype = C.c_char_p
    lib.pmlb_version.restype = C.c_char_p
    lib.pmlb_plan_kind.restype = C.c_char_p
    lib.pmlb_plan_kind.argtypes = [vp]
    lib.pmlb_plan_split_k.restype = C.c_int
    lib.pmlb_plan_split_k.argtypes = [vp]
    lib.pmlb_plan_arm_timeout_test.restype = C.c_int
    lib.pmlb_plan_arm_timeout_test.argtypes = [vp, C.c_int]
    lib.pmlb_plan_free.argtypes = [vp]
    lib.pmlb_plan_free.restype = None
    lib.pmlb_plan_scratch_bytes.argtypes = [vp]
    lib.pmlb_plan_scratch_bytes.restype = C.c_size_t
    lib.pmlb_plan_check.argtypes = [vp, vp]
    for name, desc in (("gemm", GemmDesc), ("conv", ConvDesc), ("reduce", ReduceDesc), ("pool", PoolDesc),
                       ("contract", ContractDesc), ("eltwise", EltwiseDesc), ("special", SpecialDesc)):
        getattr(lib, f"pmlb_{name}_dispatch").argtypes = [C.POINTER(desc), C.POINTER(vp)]
    lib.pmlb_gemm_invoke.argtypes = [vp] * 8
    lib.pmlb_gemm_invoke_two.argtypes = [vp] * 9
    lib.pmlb_conv_set_filter.argtypes = [vp, vp, vp, C.c_int32]
    lib.pmlb_conv_invoke.argtypes = [vp] * 6
    lib.pmlb_reduce_invoke.argtypes = [vp] * 4
    lib.pmlb_pool_invoke.argtypes = [vp] * 4
    lib.pmlb_contract_invoke.argtypes = [vp] * 7
    lib.pmlb_eltwise_invoke.argtypes = [vp] * 6
    lib.pmlb_special_invoke.argtypes = [vp] * 7
    lib.pmlb_special_out_elems.argtypes = [C.POINTER(SpecialDesc)]
    lib.pmlb_special_out_elems.restype = C.c_int64
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise KernelError(status, load().pmlb_last_error().decode())


class Plan:
    """Owns a ``pmlb_plan``; ``kind`` is 'gemm', 'conv', 'reduce', 'pool', 'contract', 'eltwise' or 'special'."""

    def __init__(self, kind: str, desc):
        self.lib = load()
        self.kind = kind
        self.desc = desc
        handle = C.c_void_p()
        check(getattr(self.lib, f"pmlb_{kind}_dispatch")(C.byref(desc), C.byref(handle)))
        self.handle = handle

    def __del__(self):
        h = getattr(self, "handle", None)
        if h:
            self.lib.pmlb_plan_free(h)
            self.handle = None

    @property
    def scratch_bytes(self) -> int:
        return self.lib.pmlb_plan_scratch_bytes(self.handle)

    @property
    def kernel(self) -> str:
        return self.lib.pmlb_plan_kind(self.handle).decode()

    @property
    def split_k(self) -> int:
        return self.lib.pmlb_plan_split_k(self.handle)

    def arm_timeout_test(self, wait_limit_ms: int = 5) -> None:
        check(self.lib.pmlb_plan_arm_timeout_test(self.handle, wait_limit_ms))

    def check(self, stream: int = 0) -> None:
        check(self.lib.pmlb_plan_check(self.handle, stream))

    # invoke wrappers take raw device addresses (ints) and a stream handle (int, 0 = default)
    def gemm(self, a, b, c, bias=None, residual=None, rowmax=None, stream=0):
        check(self.lib.pmlb_gemm_invoke(self.handle, stream, a, b, c, bias, residual, rowmax))

    def gemm_two(self, a, a2, b, c, bias=None, residual=None, rowmax=None, stream=0):
        """A plan whose descriptor has k_first > 0: `a2` holds columns k_first.. of A."""
        check(self.lib.pmlb_gemm_invoke_two(self.handle, stream, a, a2, b, c, bias, residual, rowmax))

    def set_filter(self, filt, dtype, stream=0):
        check(self.lib.pmlb_conv_set_filter(self.handle, stream, filt, dtype))

    def conv(self, x, out, bias=None, residual=None, stream=0):
        check(self.lib.pmlb_conv_invoke(self.handle, stream, x, out, bias, residual))

    def reduce(self, x, out, stream=0):
        check(self.lib.pmlb_reduce_invoke(self.handle, stream, x, out))

    def pool(self, x, out, stream=0):
        check(self.lib.pmlb_pool_invoke(self.handle, stream, x, out))

    def contract(self, srcs, out, init=None, stream=0):
        s = list(srcs) + [None] * (3 - len(srcs))
        check(self.lib.pmlb_contract_invoke(self.handle, stream, s[0], s[1], s[2], init, out))

    def eltwise(self, ins, out, stream=0):
        s = list(ins) + [None] * (3 - len(ins))
        check(self.lib.pmlb_eltwise_invoke(self.handle, stream, s[0], s[1], s[2], out))


    def special(self, ins, out0, out1=None, stream=0):
        """gather (tensor, indices), scatter (data, indices, updates), argsort (tensor), prng (state -> out0, out1)."""
        s = list(ins) + [None] * (3 - len(ins))
        check(self.lib.pmlb_special_invoke(self.handle, stream, s[0], s[1], s[2], out0, out1))


def special_desc(op: int, dtype: int = 0, sizes=(), idx_dtype: int = 0, idx_sizes=(), upd_sizes=(), axis: int = 0,
                 mode: int = 0, batch_dims: int = 0, interpolation: int = 3, nearest: int = 0, out_of_bounds: int = 0,
                 cube_coeff: float = -0.75, state_elems: int = 0) -> SpecialDesc:
    d = SpecialDesc()
    d.op, d.dtype, d.idx_dtype = op, dtype, idx_dtype
    d.rank, d.idx_rank, d.upd_rank = len(sizes), len(idx_sizes), len(upd_sizes)
    for i, v in enumerate(sizes):
        d.sizes[i] = v
    for i, v in enumerate(idx_sizes):
        d.idx_sizes[i] = v
    for i, v in enumerate(upd_sizes):
        d.upd_sizes[i] = v
    d.axis, d.mode, d.batch_dims = axis, mode, batch_dims
    d.interpolation, d.nearest, d.out_of_bounds = interpolation, nearest, out_of_bounds
    d.cube_coeff, d.state_elems = cube_coeff, state_elems
    return d


def make_access(dtype: int, sizes, coef_rows, offs=None, dens=None, strides=None) -> Access:
    """Builds an ``Access``: ``coef_rows[d]`` maps index-variable number -> coefficient."""
    a = Access()
    a.dtype = dtype
    a.rank = len(sizes)
    stride = 1
    dense = [0] * len(sizes)
    for d in range(len(sizes) - 1, -1, -1):
        dense[d] = stride
        stride *= sizes[d]
    for d, size in enumerate(sizes):
        a.sizes[d] = size
        a.strides[d] = (strides or dense)[d]
        a.off[d] = (offs or [0] * len(sizes))[d]
        a.den[d] = (dens or [1] * len(sizes))[d]
        for var, c in (coef_rows[d] if coef_rows else {}).items():
            a.coef[d][var] = c
    return a
