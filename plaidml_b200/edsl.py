"""The Tile EDSL in Python: ``TensorDim``, ``TensorIndex``, ``Tensor``, ``Contraction`` and the
element-wise intrinsics, over the C calls of ``include/plaidml_ffi.h``.

API mirror of the reference's ``plaidml/edsl/__init__.py:32-1180`` (same class and function
names, same operator overloads) so that programs written against it run unchanged.
"""

from __future__ import annotations

import enum

import numpy as np

from .core import Buffer, DType, Program, TensorShape
from .ffi import ForeignObject, decode_str, ffi, ffi_call, lib


# ---------------------------------------------------------------------- dims

def _as_dim(x) -> "TensorDim":
    if isinstance(x, TensorDim):
        return x
    if isinstance(x, (int, np.integer)):
        return TensorDim(expr=ffi_call(lib.plaidml_dim_expr_int, int(x)))
    raise TypeError(f"cannot use {type(x).__name__} as a tensor dimension")


def _dim_op(op, *args) -> "TensorDim":
    dims = [_as_dim(a) for a in args]  # keeps temporaries alive across the call
    raw = [d.as_ptr() for d in dims]
    return TensorDim(expr=ffi_call(lib.plaidml_dim_expr_op, op, len(raw), raw))


class TensorDim(ForeignObject):
    """A symbolic tensor dimension, bound to a size by ``Tensor.bind_dims``."""

    __ffi_del__ = lib.plaidml_dim_expr_free
    __ffi_repr__ = lib.plaidml_dim_expr_repr

    def __init__(self, expr=None):
        if expr is None:
            expr = ffi_call(lib.plaidml_dim_expr_none)
        elif isinstance(expr, (int, np.integer)):
            expr = ffi_call(lib.plaidml_dim_expr_int, int(expr))
        super().__init__(expr)

    def _bind(self, expr):
        self.take_ptr()
        self._ffi_obj = expr

    def __neg__(self):
        return _dim_op(lib.PLAIDML_INT_OP_NEG, self)

    def __add__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_ADD, self, o)

    def __radd__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_ADD, o, self)

    def __sub__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_SUB, self, o)

    def __rsub__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_SUB, o, self)

    def __mul__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_MUL, self, o)

    def __rmul__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_MUL, o, self)

    def __floordiv__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_DIV, self, o)

    def __rfloordiv__(self, o):
        return _dim_op(lib.PLAIDML_INT_OP_DIV, o, self)


def dim_max(a, b):
    return _dim_op(lib.PLAIDML_INT_OP_MAX, a, b)


def dim_min(a, b):
    return _dim_op(lib.PLAIDML_INT_OP_MIN, a, b)


# ---------------------------------------------------------------------- indices

def _as_poly(x) -> "TensorIndex":
    if isinstance(x, TensorIndex):
        return x
    if isinstance(x, (int, np.integer)):
        return TensorIndex(expr=ffi_call(lib.plaidml_poly_expr_literal, int(x)))
    if isinstance(x, TensorDim):
        return TensorIndex(expr=ffi_call(lib.plaidml_poly_expr_dim, x.as_ptr()))
    raise TypeError(f"cannot use {type(x).__name__} in an index expression")


def _poly_op(op, *args) -> "TensorIndex":
    polys = [_as_poly(a) for a in args]  # keeps temporaries alive across the call
    raw = [p.as_ptr() for p in polys]
    return TensorIndex(expr=ffi_call(lib.plaidml_poly_expr_op, op, len(raw), raw))


class Constraint:
    """``lhs < rhs`` (and implicitly ``0 <= lhs``)."""

    def __init__(self, lhs, rhs):
        self.lhs = lhs
        self.rhs = rhs


class TensorIndex(ForeignObject):
    """An index variable of a contraction, or an affine expression of such variables."""

    __ffi_del__ = lib.plaidml_poly_expr_free
    __ffi_repr__ = lib.plaidml_poly_expr_repr

    def __init__(self, expr=None, name=""):
        if expr is None:
            expr = ffi_call(lib.plaidml_poly_expr_index, name.encode())
        super().__init__(expr)

    def __lt__(self, rhs):
        return Constraint(self, _as_dim(rhs))  # the Constraint keeps both operands alive

    def __neg__(self):
        return _poly_op(lib.PLAIDML_INT_OP_NEG, self)

    def __add__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_ADD, self, o)

    def __radd__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_ADD, o, self)

    def __sub__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_SUB, self, o)

    def __rsub__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_SUB, o, self)

    def __mul__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_MUL, self, o)

    def __rmul__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_MUL, o, self)

    def __floordiv__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_DIV, self, o)

    def __rfloordiv__(self, o):
        return _poly_op(lib.PLAIDML_INT_OP_DIV, o, self)


def TensorDims(count):
    return [TensorDim() for _ in range(count)]


def TensorIndexes(count):
    return [TensorIndex() for _ in range(count)]


# ---------------------------------------------------------------------- tensors

class IndexedTensor:
    """``T[i, j]`` or a combination of such accesses inside a contraction."""

    def __init__(self, op, ref=None, idxs=None, args=None):
        self._op = op
        self._ref = ref
        self._idxs = idxs
        self._args = args

    def __add__(self, rhs):
        return IndexedTensor(lib.PLAIDML_COMBO_OP_ADD, args=(self, rhs))

    def __mul__(self, rhs):
        return IndexedTensor(lib.PLAIDML_COMBO_OP_MUL, args=(self, rhs))

    def __eq__(self, rhs):
        return IndexedTensor(lib.PLAIDML_COMBO_OP_EQ, args=(self, rhs))


def cond(lhs, rhs, true_case):
    """``(lhs == rhs) ? true_case : 0`` as a contraction combination."""
    return IndexedTensor(lib.PLAIDML_COMBO_OP_COND, args=(lhs, rhs, true_case))


def _as_tensor(x) -> "Tensor":
    if isinstance(x, Tensor):
        return x
    if isinstance(x, bool):
        return Tensor(expr=ffi_call(lib.plaidml_expr_int, int(x)))
    if isinstance(x, (int, np.integer)):
        return Tensor(expr=ffi_call(lib.plaidml_expr_int, int(x)))
    if isinstance(x, (float, np.floating)):
        return Tensor(expr=ffi_call(lib.plaidml_expr_float, float(x)))
    if isinstance(x, TensorDim):
        return Tensor(expr=ffi_call(lib.plaidml_expr_dim, x.as_ptr()))
    raise TypeError(f"cannot use {type(x).__name__} as a tensor")


def intrinsic(fn, *args, name=""):
    tensors = [_as_tensor(a) for a in args]
    raw = [t.as_ptr() for t in tensors]
    return Tensor(expr=ffi_call(lib.plaidml_expr_intrinsic, fn.encode(), len(raw), raw, name.encode()))


class TensorLens:
    """Reorders dimensions and indexes written in a `source` layout (say 'NCHW') into the `target` layout
    the code was written for ('NHWC'); position p of the result is taken from where target[p]'s letter
    stands in source.  The empty lens is the identity.  (plaidml/edsl/__init__.py:292-309)"""

    def __init__(self, source="", target=""):
        if len(source) != len(target):
            raise ValueError("source and target rank mismatch")
        self.map = []
        for letter in source:
            pos = target.find(letter)
            if pos < 0:
                raise ValueError("source and target dims mismatch")
            self.map.append(pos)

    def apply(self, items):
        if not self.map:
            return list(items)
        if len(items) != len(self.map):
            raise ValueError("rank mismatch in TensorLens apply")
        return [items[p] for p in self.map]


class Tensor(ForeignObject):
    __ffi_del__ = lib.plaidml_expr_free
    __ffi_repr__ = lib.plaidml_expr_repr

    def __init__(self, expr=None, value=None, lens=None):
        self._lens = lens if lens is not None else TensorLens()
        if expr is None:
            if value is None:
                raise ValueError("a Tensor needs an expression or a literal value")
            expr = _as_tensor(value).take_ptr()
        super().__init__(expr)

    def __getitem__(self, key):
        if not isinstance(key, (tuple, list)):
            key = (key,)
        return IndexedTensor(lib.PLAIDML_COMBO_OP_NONE, ref=self, idxs=tuple(key))

    def __hash__(self):
        return id(self)

    # element-wise arithmetic
    def __neg__(self):
        return intrinsic("neg", self)

    def __invert__(self):
        return intrinsic("bit_not", self)

    def __add__(self, o):
        return intrinsic("add", self, o)

    def __radd__(self, o):
        return intrinsic("add", o, self)

    def __sub__(self, o):
        return intrinsic("sub", self, o)

    def __rsub__(self, o):
        return intrinsic("sub", o, self)

    def __mul__(self, o):
        return intrinsic("mul", self, o)

    def __rmul__(self, o):
        return intrinsic("mul", o, self)

    def __truediv__(self, o):
        return intrinsic("div", self, o)

    def __rtruediv__(self, o):
        return intrinsic("div", o, self)

    __div__ = __truediv__
    __rdiv__ = __rtruediv__

    def __mod__(self, o):
        return intrinsic("mod", self, o)

    def __eq__(self, o):
        return intrinsic("cmp_eq", self, o)

    def __ne__(self, o):
        return intrinsic("cmp_ne", self, o)

    def __lt__(self, o):
        return intrinsic("cmp_lt", self, o)

    def __gt__(self, o):
        return intrinsic("cmp_gt", self, o)

    def __le__(self, o):
        return intrinsic("cmp_le", self, o)

    def __ge__(self, o):
        return intrinsic("cmp_ge", self, o)

    def __lshift__(self, o):
        return intrinsic("bit_shl", self, o)

    def __rshift__(self, o):
        return intrinsic("bit_shr", self, o)

    def __and__(self, o):
        return intrinsic("bit_and", self, o)

    def __or__(self, o):
        return intrinsic("bit_or", self, o)

    def __xor__(self, o):
        return intrinsic("bit_xor", self, o)

    # shape queries
    def compute_shape(self) -> TensorShape:
        return TensorShape(ptr=ffi_call(lib.plaidml_expr_get_shape, self.as_ptr()))

    @property
    def dtype(self) -> DType:
        return DType(ffi_call(lib.plaidml_expr_get_dtype, self.as_ptr()))

    @property
    def rank(self) -> int:
        return ffi_call(lib.plaidml_expr_get_rank, self.as_ptr())

    def bind_dims(self, *dims):
        """Binds unbound ``TensorDim`` objects to this tensor's sizes and checks bound ones."""
        dims = self._lens.apply([d if isinstance(d, TensorDim) else _as_dim(d) for d in dims])
        handles = [d.as_ptr() for d in dims]
        ffi_call(lib.plaidml_expr_bind_dims, self.as_ptr(), len(handles), handles)

    def use(self, lens: TensorLens) -> "Tensor":
        """The same tensor seen through `lens` (its own handle, so both views can be freed independently)."""
        return Tensor(expr=ffi_call(lib.plaidml_expr_clone, self.as_ptr()), lens=lens)

    def element(self, ordinal):
        return Tensor(expr=ffi_call(lib.plaidml_expr_element, self.as_ptr(), ordinal))


class Contraction:
    """``Contraction().outShape(..).outAccess(..).sum(A[i, k] * B[k, j]).build()``"""

    def __init__(self, lens=None, name=""):
        if isinstance(lens, str):  # Contraction("name")
            lens, name = None, lens
        self._lens = lens if lens is not None else TensorLens()
        self._name = name
        self._dims = ()
        self._idxs = ()
        self._constraints = []
        self._rhs = None
        self._agg = None
        self._init = None

    def outShape(self, *dims):
        self._dims = dims[0] if len(dims) == 1 and isinstance(dims[0], (list, tuple)) else dims
        return self

    def outAccess(self, *idxs):
        self._idxs = idxs[0] if len(idxs) == 1 and isinstance(idxs[0], (list, tuple)) else idxs
        return self

    def _set(self, agg, rhs):
        self._agg = agg
        self._rhs = rhs
        return self

    def assign(self, rhs):
        return self._set(lib.PLAIDML_AGG_OP_ASSIGN, rhs)

    def max(self, rhs):
        return self._set(lib.PLAIDML_AGG_OP_MAX, rhs)

    def min(self, rhs):
        return self._set(lib.PLAIDML_AGG_OP_MIN, rhs)

    def product(self, rhs):
        return self._set(lib.PLAIDML_AGG_OP_PROD, rhs)

    def sum(self, rhs):
        return self._set(lib.PLAIDML_AGG_OP_SUM, rhs)

    def init(self, rhs):
        self._init = rhs
        return self

    def add_constraint(self, constraint):
        self._constraints.append(constraint)
        return self

    def add_constraints(self, constraints):
        self._constraints.extend(constraints)
        return self

    def build(self) -> Tensor:
        rhs = self._rhs
        if isinstance(rhs, Tensor):
            rhs = IndexedTensor(lib.PLAIDML_COMBO_OP_NONE, ref=rhs, idxs=())
        elif not isinstance(rhs, IndexedTensor):
            rhs = IndexedTensor(lib.PLAIDML_COMBO_OP_NONE, ref=_as_tensor(rhs), idxs=())
        dims = self._lens.apply([_as_dim(d) for d in self._dims])
        idxs = self._lens.apply([_as_poly(i) for i in self._idxs])
        init = self._init.as_ptr() if self._init is not None else ffi.NULL
        tensor = Tensor(expr=ffi_call(lib.plaidml_expr_contraction, self._agg, rhs._op, len(idxs),
                                      [i.as_ptr() for i in idxs], [d.as_ptr() for d in dims], init,
                                      self._name.encode()))
        operands = [rhs] if rhs._op == lib.PLAIDML_COMBO_OP_NONE else list(rhs._args)
        for operand in operands:
            if not isinstance(operand, IndexedTensor) or operand._ref is None:
                raise TypeError("contraction operands must be indexed tensors, e.g. A[i, k]")
            polys = operand._ref._lens.apply([_as_poly(i) for i in operand._idxs])
            ffi_call(lib.plaidml_contraction_add_operand, tensor.as_ptr(), operand._ref.as_ptr(), len(polys),
                     [p.as_ptr() for p in polys])
        for c in self._constraints:
            ffi_call(lib.plaidml_contraction_add_constraint, tensor.as_ptr(), c.lhs.as_ptr(), c.rhs.as_ptr())
        ffi_call(lib.plaidml_contraction_build, tensor.as_ptr())
        return tensor


def Placeholder(dtype_or_shape, dims=(), name=""):
    if isinstance(dtype_or_shape, TensorShape):
        shape = dtype_or_shape
    elif isinstance(dtype_or_shape, DType):
        shape = TensorShape(dtype_or_shape, dims)
    else:
        raise TypeError(f"Unsupported type {type(dtype_or_shape)} for dtype_or_shape")
    return Tensor(expr=ffi_call(lib.plaidml_expr_input, shape.as_ptr(), name.encode()))


def Constant(buffer_or_array, name="", dtype=None):
    """A constant tensor from a ``Buffer`` or a numpy array (``dtype`` relabels uint16 as bf16)."""
    if isinstance(buffer_or_array, Buffer):
        buf = buffer_or_array
    else:
        arr = np.ascontiguousarray(buffer_or_array)
        shape = TensorShape(dtype if dtype is not None else DType.from_numpy(arr.dtype), arr.shape)
        buf = Buffer(shape)
        buf.copy_from_ndarray(arr)
    t = Tensor(expr=ffi_call(lib.plaidml_expr_constant, buf.as_ptr(), name.encode()))
    t._buffer = buf
    return t


# ---------------------------------------------------------------------- intrinsics

def cast(x, dtype):
    t = _as_tensor(x)  # held until the call returns
    return Tensor(expr=ffi_call(lib.plaidml_expr_cast, t.as_ptr(), int(dtype)))


def _unary(name):
    def fn(x):
        return intrinsic(name, x)
    fn.__name__ = name
    fn.__doc__ = f"Element-wise ``{name}``."
    return fn


abs = _unary("abs")
ceil = _unary("ceil")
cos = _unary("cos")
cosh = _unary("cosh")
exp = _unary("exp")
floor = _unary("floor")
ident = _unary("ident")
log = _unary("log")
relu = _unary("relu")
round = _unary("round")
sigmoid = _unary("sigmoid")
sin = _unary("sin")
sinh = _unary("sinh")
sqrt = _unary("sqrt")
tan = _unary("tan")
tanh = _unary("tanh")
erf = _unary("erf")


def max(x, y):
    return intrinsic("max", x, y)


def min(x, y):
    return intrinsic("min", x, y)


def pow(x, y):
    return intrinsic("pow", x, y)


def select(cond_, true_case, false_case):
    return intrinsic("select", cond_, true_case, false_case)


def reshape(x, dims):
    return intrinsic("reshape", x, *dims)


def index(dims, axis):
    return intrinsic("index", axis, *dims)


def shape(x):
    return intrinsic("shape", x)


# The operations that are not contractions (plaidml/edsl/edsl.h:809-811, 971-979, 1034-1068, 1623-1770); the
# enumerations carry the reference's values.
class SortDirection(enum.IntEnum):
    ASC = 0
    DESC = 1


class InterpolationMode(enum.IntEnum):
    NEAREST = 0
    LINEAR = 1
    CUBIC = 2
    NONE = 3


class NearestMode(enum.IntEnum):
    ROUND_PREFER_FLOOR = 0
    ROUND_PREFER_CEIL = 1
    FLOOR = 2
    CEIL = 3
    SIMPLE = 4
    NONE = 5


class GatherMode(enum.IntEnum):
    NORMAL = 0
    ND = 1


class OutOfBoundsMode(enum.IntEnum):
    GATHER_EDGE_PADDED_INPUT = 0
    RETURN_ZERO = 1


class ScatterMode(enum.IntEnum):
    NORMAL = 0
    UPDATE_SLICE = 1
    UPDATE_ELT = 2
    UPDATE_ND = 3


def argsort(x, axis=-1, direction=SortDirection.ASC):
    """int32 positions that sort `x` along `axis`; equal elements keep their order."""
    return intrinsic("argsort", x, int(axis), int(direction))


def gather(x, y, axis=0, interpolation_mode=InterpolationMode.NONE, nearest_mode=NearestMode.ROUND_PREFER_FLOOR,
           cube_coeff=-0.75, out_of_bounds_mode=OutOfBoundsMode.GATHER_EDGE_PADDED_INPUT, mode=GatherMode.NORMAL,
           batch_dims=0):
    """`x` gathered along `axis` at the positions in `y` (float positions interpolate); with ``mode=GatherMode.ND``
    the last dim of `y` addresses `batch_dims`.. dims of `x`.  A Python number for `y` picks one position."""
    if not isinstance(y, Tensor):
        kind = DType.FLOAT32 if isinstance(y, (float, np.floating)) else DType.INT32
        y = cast(index([1], 0), kind) + y
    if axis < 0:
        axis += x.rank
    return intrinsic("gather", x, y, int(axis), int(interpolation_mode), int(nearest_mode), float(cube_coeff), int(mode),
                     int(batch_dims), int(out_of_bounds_mode))


def scatter(data, indices, updates, axis=0, mode=ScatterMode.NORMAL):
    """A copy of `data` with `updates` added (NORMAL) or stored (the UPDATE modes) at the places `indices` name."""
    if axis < 0:
        axis += data.rank
    return intrinsic("scatter", data, indices, updates, int(axis), int(mode))


def prng(state, dims):
    """(numbers in [0, 1) of shape `dims` as f32, the state after them) from a state of three uint32 words."""
    both = intrinsic("prng", state, *[_as_dim(d) if not isinstance(d, (int, np.integer)) else int(d) for d in dims])
    return both.element(0), both.element(1)


def pragma(x, op, attrs):
    """``tile.pragma``: `x` annotated with an operation name and attributes (plaidml/edsl/__init__.py:1159-1171).
    The cuda target runs it as a copy of `x`."""
    t = _as_tensor(x)
    keys, values, raw = [], [], []
    for key, value in attrs.items():
        keys.append(ffi.new("char[]", key.encode()))
        values.append(Value(value))
        raw.append(ffi.new("plaidml_attr*", {"key": keys[-1], "value": values[-1].as_ptr()}))
    return Tensor(expr=ffi_call(lib.plaidml_expr_pragma, t.as_ptr(), op.encode(), len(raw), raw))


def layer(op, operands, fn, attrs=None):
    """A named region of the program (edsl.h `layer(op, operands, attrs, fn)`): the operations `fn` builds are
    printed as the body of a ``layer.box`` whose block arguments stand for `operands`; constants made inside are
    added to the operands.  `fn` returns one Tensor or a list of them, and so does ``layer``.  The body may read
    the tensors around it only through `operands` (the program is rejected otherwise)."""
    ops = [_as_tensor(t) for t in operands]
    keys, values, raw = [], [], []
    for key, value in (attrs or {}).items():
        keys.append(ffi.new("char[]", key.encode()))
        values.append(Value(value))
        raw.append(ffi.new("plaidml_attr*", {"key": keys[-1], "value": values[-1].as_ptr()}))
    handle = ffi_call(lib.plaidml_expr_layer_begin, op.encode(), len(ops), [t.as_ptr() for t in ops], len(raw), raw)
    try:
        inner = fn()
    except BaseException:
        # close the layer so that later expressions do not end up inside it
        done = ffi_call(lib.plaidml_expr_layer_end, handle, 0, [])
        ffi_call(lib.plaidml_exprs_free, done)
        ffi_call(lib.plaidml_expr_free, handle)
        raise
    single = isinstance(inner, Tensor)
    outs = [inner] if single else list(inner)
    outer = ffi_call(lib.plaidml_expr_layer_end, handle, len(outs), [t.as_ptr() for t in outs])
    tensors = [Tensor(expr=outer.elts[i]) for i in range(outer.size)]
    ffi_call(lib.plaidml_exprs_free, outer)
    ffi_call(lib.plaidml_expr_free, handle)
    return tensors[0] if single else tensors


def trace(x, msg):
    """A trace point: ``pragma(x, "trace", msg=...)``; the cuda target records no host-side trace."""
    return pragma(x, "trace", dict(msg=msg))


# ---------------------------------------------------------------------- values (op-library arguments)

class Value(ForeignObject):
    __ffi_del__ = lib.plaidml_value_free
    __ffi_repr__ = lib.plaidml_value_repr

    def __init__(self, value):
        if isinstance(value, Value):
            ptr = ffi_call(lib.plaidml_value_clone, value.as_ptr())
        elif isinstance(value, ffi.CData):
            ptr = value
        elif value is None:
            ptr = ffi_call(lib.plaidml_value_none)
        elif isinstance(value, bool):
            ptr = ffi_call(lib.plaidml_value_int, int(value))
        elif isinstance(value, (int, np.integer)):
            ptr = ffi_call(lib.plaidml_value_int, int(value))
        elif isinstance(value, TensorDim):
            ptr = ffi_call(lib.plaidml_value_dim, value.as_ptr())
        elif isinstance(value, (float, np.floating)):
            ptr = ffi_call(lib.plaidml_value_float, float(value))
        elif isinstance(value, Tensor):
            ptr = ffi_call(lib.plaidml_value_expr, value.as_ptr())
        elif isinstance(value, (list, tuple)):
            elts = [Value(v) for v in value]
            ptr = ffi_call(lib.plaidml_value_tuple, len(elts), [e.as_ptr() for e in elts])
        elif isinstance(value, str):
            ptr = ffi_call(lib.plaidml_value_str, value.encode())
        elif hasattr(value, "value") and isinstance(value.value, int):  # enums
            ptr = ffi_call(lib.plaidml_value_int, int(value.value))
        else:
            raise TypeError(f"Unsupported type {type(value)} for value={value}")
        super().__init__(ptr)

    def as_tensor(self) -> Tensor:
        return Tensor(expr=ffi_call(lib.plaidml_value_expr_get, self.as_ptr()))

    def as_tuple(self):
        """The elements of a tuple value, each as its own ``Value`` (plaidml/edsl/__init__.py Value.as_tuple)."""
        raw = ffi_call(lib.plaidml_value_tuple_get, self.as_ptr())
        try:
            return [Value(ffi_call(lib.plaidml_value_clone, raw.elts[i])) for i in range(raw.size)]
        finally:
            ffi_call(lib.plaidml_tuple_free, raw)


def build_program(name, inputs, outputs, shapes=None) -> Program:
    return Program(name, inputs, outputs, shapes=shapes)
