"""CPU oracle for the Tile contraction path -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` may
import this package; the product (``plaidml_b200``) never does.  See ``tile_oracle.c`` for the
reference files each function restates.
"""

from .binding import (  # noqa: F401
    build,
    contract,
    conv2d_nhwc_f32,
    gemm_f32,
    gemm_f32_acc64,
    gemm_h16_f32,
    gemm_i8_i32,
    lib,
    pool2d_nhwc_f32,
    reduce_f32,
    bf16_to_f32,
    f32_to_bf16,
)
from . import special  # noqa: F401,E402  (gather / scatter / argsort / prng, numpy)
