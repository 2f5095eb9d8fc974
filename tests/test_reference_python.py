"""The reference's own Python package and Python tests on this repository's libplaidml.so.

The reference ships a cffi front end (plaidml/{__init__,ffi}.py, plaidml/{core,edsl,exec,op}/__init__.py) that binds
`libplaidml.so` by name, and Python test modules for it (plaidml/edsl/tests/edsl_test.py: 37 tests with expected
values; plaidml/edsl/examples/example_tests.py with the seven example modules it imports; plaidml/core/core_test.py: settings, and the target list, which is asked for `llvm_cpu` -- the one test that
cannot hold against a library whose only target is `cuda`, pinned below).  Here that package is byte-compiled UNMODIFIED from the checkout into
tests/host/_build/pyref/ (byte code without sources, like the compiled C++ test binaries: build products, not sources),
completed by the two modules the reference's build generates (tests/host/pyshim/plaidml/_ffi.py: the C declarations,
taken from include/plaidml_ffi.h; core/_version.py) and pointed at this library through PLAIDML_LIB_PATH.

The same edsl_test.py also runs on this repository's OWN Python package (`plaidml_b200.{core,edsl,exec,op}`) reached
under the name `plaidml` through a few lines of aliasing (tests/host/pyshim_mirror/plaidml/__init__.py): the mirror of
the reference's Python API is a drop-in for code written against it.

The CPU half needs the checkout (``PLAIDML_REFERENCE_DIR``; skipped when unset): it assembles the package and runs the
tests with --build-only (every program is built and compiled for the `cuda` target through the reference's Python API;
nothing runs).  The GPU half runs whatever tests/host/_build/pyref/ holds on cuda.0 with the tests' own expected
values; it never reads the checkout.
"""

import os
import py_compile
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SHIM = ROOT / "tests" / "host" / "pyshim"
OUT = ROOT / "tests" / "host" / "_build" / "pyref"

# file of the checkout -> module file of the assembled tree
PACKAGE = {
    "plaidml/__init__.py": "plaidml/__init__",
    "plaidml/ffi.py": "plaidml/ffi",
    "plaidml/core/__init__.py": "plaidml/core/__init__",
    "plaidml/core/settings.py": "plaidml/core/settings",
    "plaidml/edsl/__init__.py": "plaidml/edsl/__init__",
    "plaidml/exec/__init__.py": "plaidml/exec/__init__",
    "plaidml/op/__init__.py": "plaidml/op/__init__",
    "plaidml/edsl/tests/edsl_test.py": "ref_edsl_test",
    "plaidml/core/core_test.py": "ref_core_test",
    "plaidml/edsl/examples/example_tests.py": "ref_example_tests",
}
PACKAGE.update({f"plaidml/edsl/examples/{name}.py": f"plaidml/edsl/examples/{name}"
                for name in ("complex_conv_2d", "conv_1d", "conv_2d_dilated", "gemm", "gemv", "max_pool_1d", "quantize")})
# The byte code is kept under this suffix (snapshots of the tree leave *.pyc files behind as caches) and given its
# importable name in a scratch copy when the tests run.
STORED = ".bytecode"
TEST_MODULES = ["ref_edsl_test", "ref_core_test", "ref_example_tests"]
EXPECTED_TESTS = 48      # 37 of edsl_test.py, 2 of core_test.py, 9 of examples/example_tests.py
# (not taken: plaidml/edsl/edsl_docs.py, whose tests use names the reference's own package no longer has --
# LogicalShape, Tensor(shape), Program(name, outputs))


def assemble(ref: Path) -> None:
    if OUT.exists():
        shutil.rmtree(OUT)
    for src, dst in PACKAGE.items():
        target = OUT / (dst + STORED)
        target.parent.mkdir(parents=True, exist_ok=True)
        py_compile.compile(str(ref / src), cfile=str(target), doraise=True,
                           invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)


def run_tests(scratch: Path, *flags) -> str:
    tree = scratch / "pyref"
    for stored in OUT.rglob("*" + STORED):
        target = tree / stored.relative_to(OUT).with_suffix(".pyc")
        target.parent.mkdir(parents=True, exist_ok=True)
        shutil.copy(stored, target)
    shutil.copy(SHIM / "plaidml" / "_ffi.py", tree / "plaidml" / "_ffi.py")
    shutil.copy(SHIM / "plaidml" / "core" / "_version.py", tree / "plaidml" / "core" / "_version.py")
    env = dict(os.environ)
    env.update({
        "PYTHONPATH": str(tree),
        "PLAIDML_LIB_PATH": str(ROOT / "plaidml_b200" / "libplaidml.so"),
        "PLAIDML_FFI_HEADER": str(ROOT / "include" / "plaidml_ffi.h"),
        "PLAIDML_DEVICE": "cuda.0",
        "PLAIDML_TARGET": "cuda",
    })
    res = subprocess.run([sys.executable, str(SHIM / "run_reference_tests.py"), *flags, *TEST_MODULES], cwd=str(tree), env=env,
                         capture_output=True, text=True, timeout=900)
    assert res.returncode in (0, 1), (res.stdout[-2000:], res.stderr[-3000:])
    return res.stdout + "\n--- stderr ---\n" + res.stderr


# The one test that cannot hold here, and why: it asks the target list for the reference's CPU target.
NOT_THIS_LIBRARY = {"ref_core_test.TestCore.test_get_strings": "'llvm_cpu' not found in ['cuda']"}


def check(out: str, suffix: str) -> None:
    failed = [ln.split("]", 1)[1].strip() for ln in out.splitlines() if ln.startswith("[ FAIL]")]
    assert sorted(failed) == sorted(NOT_THIS_LIBRARY), (failed, out[-4000:])
    for reason in NOT_THIS_LIBRARY.values():
        assert reason in out, out[-4000:]
    assert f"{EXPECTED_TESTS} tests, {len(NOT_THIS_LIBRARY)} failures{suffix}" in out, out[-3000:]
    # (the reference itself skips test_assignment_exceptions)
    assert out.count("[ SKIP]") == 1 and out.count("[  OK ]") == EXPECTED_TESTS - len(NOT_THIS_LIBRARY) - 1


def run_against_own_package(scratch: Path, *flags) -> str:
    """The reference's edsl_test.py on this repository's own Python package, reached under the name `plaidml`."""
    tree = scratch / "mirror"
    tree.mkdir(parents=True, exist_ok=True)
    shutil.copy(OUT / ("ref_edsl_test" + STORED), tree / "ref_edsl_test.pyc")
    env = dict(os.environ)
    env.update({
        "PYTHONPATH": os.pathsep.join([str(SHIM.parent / "pyshim_mirror"), str(ROOT), str(tree)]),
        "PLAIDML_DEVICE": "cuda.0",
        "PLAIDML_TARGET": "cuda",
    })
    env.pop("PLAIDML_LIB_PATH", None)
    res = subprocess.run([sys.executable, str(SHIM / "run_reference_tests.py"), *flags, "ref_edsl_test"], cwd=str(tree), env=env,
                         capture_output=True, text=True, timeout=900)
    assert res.returncode in (0, 1), (res.stdout[-2000:], res.stderr[-3000:])
    return res.stdout + "\n--- stderr ---\n" + res.stderr


def check_own_package(out: str, suffix: str) -> None:
    failed = [ln for ln in out.splitlines() if ln.startswith("[ FAIL]")]
    assert not failed and f"37 tests, 0 failures{suffix}" in out, (failed, out[-4000:])


def test_reference_python_package_builds_its_programs(tmp_path):
    ref = os.environ.get("PLAIDML_REFERENCE_DIR")
    if not ref or not (Path(ref) / "plaidml/edsl/__init__.py").exists():
        pytest.skip("PLAIDML_REFERENCE_DIR does not point at a checkout of the reference")
    if not (ROOT / "plaidml_b200" / "libplaidml.so").exists():
        pytest.skip("needs a built libplaidml.so")
    assemble(Path(ref))
    check(run_tests(tmp_path, "--build-only"), " (build only)")
    # ... and the same EDSL tests on this repository's own Python package under the reference's name
    check_own_package(run_against_own_package(tmp_path, "--build-only"), " (build only)")


@pytest.mark.gpu
def test_reference_python_tests_run_on_the_cuda_device(tmp_path):
    if not (OUT / ("ref_edsl_test" + STORED)).exists():
        pytest.skip("tests/host/_build/pyref/ is empty (assembled by the CPU half where the checkout is mounted)")
    out = run_tests(tmp_path)
    assert "build only" not in out
    check(out, "")
    out = run_against_own_package(tmp_path)
    assert "build only" not in out
    check_own_package(out, "")
