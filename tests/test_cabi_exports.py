"""The C-ABI library loads without a GPU and exports every function the headers under include/ declare
(and the headers declare the reference's complete export list)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "plaidml_b200" / "libplaidml.so"
DECL = re.compile(r"\b((?:plaidml|pmlb)_[a-z0-9_]+)\s*\(", re.M)

# The functions plaidml/{core,edsl,op,exec}/ffi.h declare in the reference, by header.
REFERENCE_EXPORTS = """
plaidml_buffer_adopt plaidml_buffer_alloc plaidml_buffer_clone plaidml_buffer_data plaidml_buffer_free
plaidml_buffer_shape plaidml_buffer_size plaidml_init plaidml_integers_free plaidml_kvps_free plaidml_program_compile
plaidml_program_free plaidml_program_get_inputs plaidml_program_get_outputs plaidml_program_get_passes
plaidml_program_repr plaidml_program_save plaidml_settings_get plaidml_settings_list plaidml_settings_load
plaidml_settings_save plaidml_settings_set plaidml_shape_alloc plaidml_shape_clone plaidml_shape_free
plaidml_shape_get_dtype plaidml_shape_get_nbytes plaidml_shape_get_rank plaidml_shape_get_sizes
plaidml_shape_get_strides plaidml_shape_repr plaidml_shapes_free plaidml_shutdown plaidml_string_free
plaidml_string_ptr plaidml_strings_free plaidml_version
plaidml_build plaidml_contraction_add_constraint plaidml_contraction_add_operand plaidml_contraction_build
plaidml_dim_expr_free plaidml_dim_expr_int plaidml_dim_expr_none plaidml_dim_expr_op plaidml_dim_expr_repr
plaidml_edsl_init plaidml_expr_bind_dims plaidml_expr_cast plaidml_expr_clone plaidml_expr_constant
plaidml_expr_contraction plaidml_expr_dim plaidml_expr_element plaidml_expr_float plaidml_expr_free
plaidml_expr_get_dim plaidml_expr_get_dtype plaidml_expr_get_rank plaidml_expr_get_shape plaidml_expr_input
plaidml_expr_int plaidml_expr_intrinsic plaidml_expr_layer_begin plaidml_expr_layer_end plaidml_expr_pragma
plaidml_expr_ptr plaidml_expr_repr plaidml_expr_uint plaidml_exprs_free plaidml_poly_expr_dim plaidml_poly_expr_free
plaidml_poly_expr_index plaidml_poly_expr_literal plaidml_poly_expr_op plaidml_poly_expr_repr plaidml_targets_get
plaidml_tuple_free plaidml_value_clone plaidml_value_dim plaidml_value_dim_get plaidml_value_expr
plaidml_value_expr_get plaidml_value_float plaidml_value_float_get plaidml_value_free plaidml_value_get_kind
plaidml_value_int plaidml_value_int_get plaidml_value_none plaidml_value_repr plaidml_value_str plaidml_value_str_get
plaidml_value_tuple plaidml_value_tuple_get
plaidml_op_make
plaidml_devices_get plaidml_exec_init plaidml_executable_free plaidml_executable_run plaidml_jit
""".split()


def declared(header: Path) -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"^\s*#[^\n]*(\\\n[^\n]*)*", "", text, flags=re.M)
    return sorted(set(DECL.findall(text)))


@pytest.fixture(scope="module")
def library():
    assert LIB.exists(), "build the library first: python -m plaidml_b200.build"
    return ctypes.CDLL(str(LIB))


@pytest.mark.parametrize("header", sorted((ROOT / "include").glob("*.h")), ids=lambda p: p.name)
def test_every_declared_function_is_exported(library, header):
    names = declared(header)
    assert names, f"no declarations parsed from {header.name}"
    missing = [n for n in names if not hasattr(library, n)]
    assert not missing, f"declared in {header.name} but not exported: {missing}"


def test_header_covers_the_reference_export_list(library):
    names = set(declared(ROOT / "include" / "plaidml_ffi.h"))
    missing = [n for n in REFERENCE_EXPORTS if n not in names]
    assert not missing, f"reference exports absent from include/plaidml_ffi.h: {missing}"
    assert all(hasattr(library, n) for n in REFERENCE_EXPORTS)


def test_nothing_else_leaks_out_of_the_library():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(LIB)], capture_output=True, text=True, check=True).stdout
    symbols = [line.split()[-1] for line in out.splitlines() if line.strip()]
    stray = [s for s in symbols if not s.startswith(("plaidml_", "pmlb_"))]
    assert not stray, f"unexpected exported symbols: {stray[:10]}"


def test_version_and_error_calls_work_without_a_gpu(library):
    library.pmlb_version.restype = ctypes.c_char_p
    library.pmlb_last_error.restype = ctypes.c_char_p
    assert library.pmlb_version()
    library.pmlb_device_count.restype = ctypes.c_int
    assert library.pmlb_device_count() >= 0


def test_special_descriptor_layout_and_result_sizes_without_a_device():
    # pmlb_special_out_elems is host arithmetic on the descriptor: it checks that the ctypes mirror of
    # pmlb_special_desc has the layout of the C struct and that inconsistent descriptors are recognised
    from plaidml_b200 import kernels as K
    lib = K.load()
    C = K.C

    def count(d):
        return lib.pmlb_special_out_elems(C.byref(d))

    # gather along axis 1 of [3, 5, 7] with indices [2, 4]: 3 * (2 * 4) * 7
    assert count(K.special_desc(K.SPECIAL_GATHER, K.F32, [3, 5, 7], K.I32, [2, 4], axis=1)) == 168
    # nd with one batch dim: indices [3, 6, 2] address dims 1..2 of [3, 5, 7, 9]: 3 * 6 * 9
    assert count(K.special_desc(K.SPECIAL_GATHER, K.F32, [3, 5, 7, 9], K.I32, [3, 6, 2], mode=1, batch_dims=1)) == 162
    assert count(K.special_desc(K.SPECIAL_SCATTER, K.F32, [8, 4], K.I32, [3], [3, 4])) == 32
    assert count(K.special_desc(K.SPECIAL_ARGSORT, K.I32, [6, 5], axis=1)) == 30
    assert count(K.special_desc(K.SPECIAL_PRNG, sizes=[2, 3], state_elems=3)) == 6
    # refused: axis outside the tensor, float indices without an interpolation, nd indices past the rank,
    # 64-bit scatter indices, a state of two words
    assert count(K.special_desc(K.SPECIAL_GATHER, K.F32, [3, 5], K.I32, [2], axis=2)) == 0
    assert count(K.special_desc(K.SPECIAL_GATHER, K.F32, [3, 5], K.F32, [2], interpolation=3)) == 0
    assert count(K.special_desc(K.SPECIAL_GATHER, K.F32, [3, 5], K.I32, [2, 3], mode=1)) == 0
    assert count(K.special_desc(K.SPECIAL_SCATTER, K.F32, [8], K.I64, [3], [3])) == 0
    assert count(K.special_desc(K.SPECIAL_PRNG, sizes=[4], state_elems=2)) == 0
