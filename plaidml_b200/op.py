"""The operation library from Python.  Mirror of ``plaidml/op/__init__.py`` / ``plaidml/op/op.h``:
each function packs its arguments into a value tuple for ``plaidml_op_make``."""

from __future__ import annotations

import enum

from . import edsl
from .ffi import ffi_call, lib


def op(op_name, args):
    value = edsl.Value(args)
    return edsl.Value(ffi_call(lib.plaidml_op_make, op_name.encode(), value.as_ptr()))


class AutoGroupMode(enum.IntEnum):
    UNGROUPED = 0
    EXPLICIT = 1
    AUTO = 2
    DEPTHWISE = 3


class AutoPadMode(enum.IntEnum):
    EXPLICIT = 0
    SAME_LOWER = 1
    SAME_UPPER = 2
    VALID = 3


class ConvDerivMode(enum.IntEnum):
    NONE = 0
    DATA = 1
    FILTER = 2


class GroupLayout(enum.IntEnum):
    NONE = 0
    SEPARATE = 1
    IN_C = 2
    IN_K = 3


class PoolMode(enum.IntEnum):
    AVG = 0
    MAX = 1
    MIN = 2
    SUM = 3


class TensorLayout(enum.IntEnum):
    NXC = 0
    NCX = 1
    KCX = 2
    XCK = 3
    GKCX = 4
    XGCK = 5


def convolution(I, F, strides=None, dilations=None, data_dilations=None, filter_shape=None, groups=1,
                autopad_mode=AutoPadMode.SAME_UPPER, manual_padding=None, input_layout=TensorLayout.NXC,
                filter_layout=TensorLayout.XCK, group_layout=GroupLayout.NONE, winograd_allowed=False, name="",
                autogroup_mode=AutoGroupMode.UNGROUPED, deriv_mode=ConvDerivMode.NONE, result_shape=None,
                infer_result_shape=False):
    args = [I, F, list(strides or []), list(dilations or []), list(data_dilations or []), list(filter_shape or []),
            groups, int(autopad_mode), list(manual_padding or []), int(input_layout), int(filter_layout),
            int(group_layout), winograd_allowed, name, int(autogroup_mode), int(deriv_mode),
            list(result_shape or []), infer_result_shape]
    return op("convolution", args).as_tensor()


def pool(I, pool_mode, pool_size, strides, autopad_mode, manual_padding, input_layout, include_padding_in_avg=False,
         use_ceil_for_output_shape=False, name=""):
    args = [I, int(pool_mode), list(pool_size), list(strides), int(autopad_mode), list(manual_padding),
            int(input_layout), include_padding_in_avg, use_ceil_for_output_shape, name]
    return op("pool", args).as_tensor()


def dot(x, y, name=""):
    return op("dot", [x, y, name]).as_tensor()


def relu(x, alpha=None, max_value=None, threshold=0.0, name=""):
    return op("relu", [x, alpha, max_value, threshold, name]).as_tensor()


def mean(x, axes=None, keepdims=False):
    return op("mean", [x, axes, keepdims]).as_tensor()


def sum(x, axes=None, keepdims=False):
    return op("sum", [x, axes, keepdims]).as_tensor()


def max(x, axes=None, keepdims=False):
    return op("max", [x, axes, keepdims]).as_tensor()


def min(x, axes=None, keepdims=False):
    return op("min", [x, axes, keepdims]).as_tensor()


def prod(x, axes=None, keepdims=False):
    return op("prod", [x, axes, keepdims]).as_tensor()


def variance(x, axes=None, keepdims=False):
    return op("variance", [x, axes, keepdims]).as_tensor()


def softmax(x, axis, name=""):
    return op("softmax", [x, axis, name]).as_tensor()


def maximum(x, y):
    return op("maximum", [x, y]).as_tensor()


def minimum(x, y):
    return op("minimum", [x, y]).as_tensor()


def clip(x, lo=None, hi=None):
    return op("clip", [x, lo, hi]).as_tensor()


def abs(x):
    return op("abs", [x]).as_tensor()


def sigmoid(x):
    return op("sigmoid", [x]).as_tensor()


def square(x):
    return op("square", x).as_tensor()


def reshape(x, dims):
    return op("reshape", [x, list(dims)]).as_tensor()


def transpose(x, axes=None):
    return op("transpose", [x, None if axes is None else list(axes)]).as_tensor()


def squeeze(x, axes):
    return op("squeeze", [x, list(axes)]).as_tensor()


def unsqueeze(x, axes):
    return op("unsqueeze", [x, list(axes)]).as_tensor()


def flip(x, axis):
    return op("flip", [x, axis]).as_tensor()


def cumsum(x, axis, exclusive=False):
    return op("cumsum", [x, axis, exclusive]).as_tensor()


def elu(x, alpha):
    return op("elu", [x, alpha]).as_tensor()


def spatial_padding(x, lo_pads, hi_pads, data_layout=TensorLayout.NXC):
    return op("spatial_padding", [x, list(lo_pads), list(hi_pads), int(data_layout)]).as_tensor()


# ---- the rest of the contraction-built operations of plaidml/op/__init__.py (same names and arguments)

class EpsMode(enum.IntEnum):
    ADD = 0
    MAX = 1


class InterpolationMode(enum.IntEnum):
    NEAREST = 0
    BILINEAR = 1


class PadMode(enum.IntEnum):
    CONSTANT = 0
    EDGE = 1
    REFLECT = 2
    SYMMETRIC = 3


def all(x, axis=None, keepdims=False):
    return op("all", [x, axis, keepdims]).as_tensor()


def any(x, axis=None, keepdims=False):
    return op("any", [x, axis, keepdims]).as_tensor()


def argmax(x, axis=-1):
    return op("argmax", [x, axis]).as_tensor()


def binary_crossentropy(targets, preds, epsilon):
    return op("binary_crossentropy", [targets, preds, float(epsilon)]).as_tensor()


def broadcast(x, result_shape, bcast_axes):
    return op("broadcast", [x, list(result_shape), list(bcast_axes)]).as_tensor()


def concatenate(tensors, axis=-1):
    return op("concatenate", [list(tensors), axis]).as_tensor()


def cumprod(x, axis):
    return op("cumprod", [x, axis]).as_tensor()


def explicit_padding(x, lo_pads, hi_pads, mode=PadMode.CONSTANT, padval=0.0):
    return op("explicit_padding", [x, list(lo_pads), list(hi_pads), int(mode), padval]).as_tensor()


def hard_sigmoid(x, slope):
    return op("hard_sigmoid", [x, float(slope)]).as_tensor()


def l2norm(x, axes, epsilon, eps_mode=EpsMode.ADD):
    return op("l2norm", [x, list(axes), float(epsilon), int(eps_mode)]).as_tensor()


def image_resize(x, factors, interp, layout):
    return op("image_resize", [x, list(factors), int(interp), int(layout)]).as_tensor()


def lrn(x, window_size, axes=(-1,), alpha=1.0, beta=0.5, epsilon=1.0):
    return op("lrn", [x, list(window_size), list(axes), float(alpha), float(beta), float(epsilon)]).as_tensor()


def mvn(x, axes=None, normalize_variance=True, epsilon=1e-9, across_channels=True, layout=""):
    return op("mvn", [x, None if axes is None else list(axes), normalize_variance, float(epsilon), across_channels,
                      layout]).as_tensor()


def reorg_yolo(x, stride, decrease, layout="NCHW"):
    return op("reorg_yolo", [x, stride, decrease, layout]).as_tensor()


def repeat(x, repeats, axis):
    return op("repeat", [x, repeats, axis]).as_tensor()


def scale_gradient(x, scale=-1.0):
    return op("scale_gradient", [x, float(scale)]).as_tensor()


def slice_of(x, slices):
    """`slices`: one entry per axis, an int (the axis disappears) or a Python slice."""
    packed = []
    for s in slices:
        if isinstance(s, int):
            packed.append(s)
        elif isinstance(s, slice):
            packed.append([s.start, s.stop, s.step])
        else:
            raise ValueError("Unexpected type {} used to slice tensor".format(type(s)))
    return op("slice", [x, packed]).as_tensor()


def tile(x, n):
    return op("tile", [x, list(n)]).as_tensor()


class TopKSortType(enum.IntEnum):
    VALUE = 0
    INDEX = 1


def gatherND(x, indices, batch_dims=0, interpolation_mode=edsl.InterpolationMode.NONE):
    """`x` at the index rows of `indices` (their last dim addresses dims batch_dims.. of `x`); LINEAR blends the
    corners around float rows, the data seen as zero-padded."""
    return op("gatherND", [x, indices, batch_dims, int(interpolation_mode)]).as_tensor()


def sort(x, axis=-1, direction=edsl.SortDirection.ASC):
    return op("sort", [x, axis, int(direction)]).as_tensor()


def topk(x, k, axis=-1, sort_direction=edsl.SortDirection.DESC, sort_type=TopKSortType.VALUE, index_element_type=None):
    """(values, positions) of the first `k` elements along `axis` in sorted order."""
    from .core import DType
    values, positions = op("topk", [x, k, axis, int(sort_direction), int(sort_type),
                                    int(index_element_type if index_element_type is not None else DType.INT32)]).as_tuple()
    return values.as_tensor(), positions.as_tensor()


class BoxesDecodeMode(enum.IntEnum):
    NMS = 0
    SSD = 1


class NmsStyle(enum.IntEnum):
    CAFFE = 0
    MXNET = 1
    OV = 2


def nms(boxes, scores, iou_threshold, score_threshold, max_output_boxes_per_class, soft_nms_sigma=0.0,
        center_point_box=False, sort_result_descending=True, box_output_type=None, clip_before_nms=False,
        nms_style=NmsStyle.OV, share_location=True, hard_suppression=True):
    """Non-maximum suppression over boxes [batch, boxes, 4] and scores [batch, classes, boxes]: returns (rows of
    (batch, class, box), rows of (batch, class, score), number of valid rows); rows that found nothing hold -1.
    (plaidml/op/op.h `nms`; the SSD box decoding is not offered.)"""
    from .core import DType
    out_type = int(box_output_type if box_output_type is not None else DType.INT32)
    b, s, v = op("nms", [boxes, scores, iou_threshold, score_threshold, int(max_output_boxes_per_class), float(soft_nms_sigma),
                         bool(center_point_box), bool(sort_result_descending), out_type, int(BoxesDecodeMode.NMS),
                         bool(clip_before_nms), False, 0, 0, None, None, False, None, int(nms_style), bool(share_location),
                         bool(hard_suppression)]).as_tuple()
    return b.as_tensor(), s.as_tensor(), v.as_tensor()
