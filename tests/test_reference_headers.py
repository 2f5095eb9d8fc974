"""Test sources of the reference checkout, compiled UNMODIFIED against the reference's own C++ headers and
linked with this repository's libplaidml.so (tests/host/ref_driver.cc and the stand-in headers under
tests/host/refshim/ replace googletest, gflags and three LLVM ADT headers, nothing of plaidml):

  * plaidml/edsl/examples/gemm.cc: five GEMM tests with exact expected outputs;
  * networks/oplib/resnet50.cc: the reference's ResNet-50 builder, built at batch 1;
  * plaidml/edsl/tests/edsl_test.cc: the reference's whole C++ EDSL suite, 119 tests with their own checkExact /
    checkClose / EXPECT_* expectations (contractions, element-wise operations, layers, gather / scatter / argsort /
    prng): all pass;
  * plaidml/edsl/examples/{complex_conv_2d,conv_1d,conv_2d_dilated,gemv,max_pool_1d,quantize}.cc and
    plaidml/edsl/edsl_docs.cc (the code blocks of the documentation): 23 tests, all pass;
  * networks/oplib/run.cc and layer.cc: the reference's two command-line programs (one ResNet-50 pass; one convolution
    layer of a given shape ten times);
  * networks/oplib/benchmark.cc: the reference's ResNet-50 benchmark program (with its own main(); a stand-in for Google
    Benchmark under refshim/benchmark/ runs and times the registered benchmarks);
  * plaidml/op/op_test.cc: the reference's op-library suite, 60 tests (67 with the parameterised convolution cases),
    among them exact expected outputs for explicit paddings, transposed and grouped convolutions and a sort: all pass.

The CPU half needs the checkout (``PLAIDML_REFERENCE_DIR``; skipped when unset) and g++: it compiles the
binaries into tests/host/_build/ and runs them with --build-only (programs are built, printed and compiled
for the `cuda` target; no device).  The GPU half runs whatever binaries tests/host/_build/ already holds --
they link libplaidml.so dynamically, so they always exercise the current library -- on cuda.0 and applies
the tests' own expectations; it never reads the checkout.
"""

import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HOST = ROOT / "tests" / "host"
OUT = HOST / "_build"
LIB_DIR = ROOT / "plaidml_b200"

BINARIES = {
    "ref_gemm": (["plaidml/edsl/examples/gemm.cc"], []),
    "ref_resnet": (["networks/oplib/resnet50.cc"], ["-DPMLB_REF_RESNET"]),
    "ref_edsl": (["plaidml/edsl/tests/edsl_test.cc"], []),
    "ref_op": (["plaidml/op/op_test.cc"], []),
    # the other EDSL examples (gemm.cc has its own binary above) and the documentation's code blocks
    # (not taken: plaidml/exec/tests/list_devices_test.cc, one test that looks for the device "llvm_cpu.0")
    "ref_examples": (["plaidml/edsl/examples/complex_conv_2d.cc", "plaidml/edsl/examples/conv_1d.cc",
                      "plaidml/edsl/examples/conv_2d_dilated.cc", "plaidml/edsl/examples/gemv.cc",
                      "plaidml/edsl/examples/max_pool_1d.cc", "plaidml/edsl/examples/quantize.cc",
                      "plaidml/edsl/edsl_docs.cc"], []),
    # the reference's ResNet-50 benchmark program (its own main(); Google Benchmark replaced by refshim/benchmark/)
    "ref_benchmark": (["networks/oplib/benchmark.cc", "networks/oplib/resnet50.cc"], ["-DPMLB_OWN_MAIN"]),
    # ... and its two small command-line programs: run the ResNet-50 once; one convolution layer of given shape 10 times
    "ref_run": (["networks/oplib/run.cc", "networks/oplib/resnet50.cc"], ["-DPMLB_OWN_MAIN"]),
    "ref_layer": (["networks/oplib/layer.cc"], ["-DPMLB_OWN_MAIN"]),
}

def _check_edsl_suite(out: str) -> None:
    ran = [ln for ln in out.splitlines() if ln.startswith("[ RUN ]")]
    failed = [ln for ln in out.splitlines() if ln.startswith("[ FAIL]")]
    assert len(ran) == 119 and not failed and "119 tests, 0 failures" in out, (failed, out[-1500:])


def build_binaries(ref_dir: Path) -> list:
    """Compiles the reference's sources where they lie; outputs only under tests/host/_build/."""
    OUT.mkdir(parents=True, exist_ok=True)
    built = []
    for name, (sources, defines) in BINARIES.items():
        driver = [] if "-DPMLB_OWN_MAIN" in defines else [str(HOST / "ref_driver.cc")]
        cmd = ["g++", "-std=c++17", "-O1", "-w", *defines, "-I", str(HOST / "refshim"), "-I", str(ref_dir), "-o", str(OUT / name),
               *driver, *[str(ref_dir / s) for s in sources], "-L", str(LIB_DIR), "-l:libplaidml.so",
               "-Wl,-rpath,$ORIGIN/../../../plaidml_b200"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        assert res.returncode == 0, res.stderr[-4000:]
        built.append(OUT / name)
    return built


def _check_op_suite(out: str) -> None:
    failed = [ln for ln in out.splitlines() if ln.startswith("[ FAIL]")]
    assert "67 tests, 0 failures" in out and not failed, (failed, out[-1500:])


def _run(binary: Path, *args, ok_codes=(0,)) -> str:
    res = subprocess.run([str(binary), *args], capture_output=True, text=True, timeout=600)
    assert res.returncode in ok_codes, (res.stdout[-3000:], res.stderr[-2000:])
    return res.stdout


def test_reference_sources_compile_and_build_their_programs():
    ref = os.environ.get("PLAIDML_REFERENCE_DIR")
    if not ref or not (Path(ref) / "plaidml/edsl/edsl.h").exists():
        pytest.skip("PLAIDML_REFERENCE_DIR does not point at a checkout of the reference")
    if shutil.which("g++") is None or not (LIB_DIR / "libplaidml.so").exists():
        pytest.skip("needs g++ and a built libplaidml.so")
    gemm, resnet, edsl_suite, op_suite, examples = build_binaries(Path(ref))[:5]   # (the three programs with a main() of their own need a device)
    assert "23 tests, 0 failures" in _run(examples, "--build-only")
    _check_edsl_suite(_run(edsl_suite, "--build-only"))
    _check_op_suite(_run(op_suite, "--build-only"))
    out = _run(gemm, "--build-only")
    assert "5 tests, 0 failures" in out
    # the printed programs are the tile module of the reference's own FileCheck expectations
    assert out.count("tile.contract add, mul") == 5 and "tensor<3x3xsi8>" in out and "tensor<3x3xui64>" in out
    out = _run(resnet, "--build-only")
    assert "1 tests, 0 failures" in out and "109 inputs, 1 output" in out


@pytest.mark.gpu
def test_reference_sources_run_on_the_cuda_device():
    if not (OUT / "ref_gemm").exists():
        pytest.skip("tests/host/_build/ holds no binaries (built by the CPU half where the checkout is mounted)")
    out = _run(OUT / "ref_gemm", "--device", "cuda.0")
    assert "5 tests, 0 failures" in out and "build only" not in out
    if (OUT / "ref_resnet").exists():
        out = _run(OUT / "ref_resnet", "--device", "cuda.0")
        assert "1 tests, 0 failures" in out
    if (OUT / "ref_edsl").exists():
        # the reference's EDSL suite with its own expected values (checkExact / checkClose at the reference's
        # tolerances), on the device
        out = _run(OUT / "ref_edsl", "--device", "cuda.0")
        assert "build only" not in out
        _check_edsl_suite(out)
    if (OUT / "ref_op").exists():
        out = _run(OUT / "ref_op", "--device", "cuda.0")
        assert "build only" not in out
        _check_op_suite(out)
    if (OUT / "ref_benchmark").exists():
        # networks/oplib/benchmark.cc: compile and run of the reference's ResNet-50 (batch 1, fp32, 109 host buffers per run)
        env = dict(os.environ, PLAIDML_TARGET="cuda", PLAIDML_DEVICE="cuda.0", PMLB_BENCH_ITERS="12")
        res = subprocess.run([str(OUT / "ref_benchmark")], capture_output=True, text=True, timeout=600, env=env)
        assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-2000:])
        assert "resnet50/compile: 12 iterations" in res.stdout and "resnet50/run: 12 iterations" in res.stdout, res.stdout
    env = dict(os.environ, PLAIDML_TARGET="cuda", PLAIDML_DEVICE="cuda.0")
    if (OUT / "ref_run").exists():
        res = subprocess.run([str(OUT / "ref_run")], capture_output=True, text=True, timeout=600, env=env)
        assert res.returncode == 0 and "Running..." in res.stdout and "tile.contract" in res.stdout, (res.stdout[-1500:], res.stderr[-1500:])
    if (OUT / "ref_layer").exists():
        # N K C H W R S stride: a 3 x 3 convolution on 56 x 56 x 64 in fp32 (the tensor-core route with three TF32 products)
        res = subprocess.run([str(OUT / "ref_layer"), "8", "64", "64", "56", "56", "3", "3", "1"], capture_output=True, text=True,
                             timeout=600, env=env)
        assert res.returncode == 0 and "Running..." in res.stdout and "conv2d:8:64:64:56:56:3:3:1" in res.stdout, \
            (res.stdout[-1500:], res.stderr[-1500:])
    if (OUT / "ref_examples").exists():
        # the remaining EDSL examples (1-D / dilated / complex convolutions, GEMV, max pool, quantisation) and the
        # code blocks of the reference's documentation
        out = _run(OUT / "ref_examples", "--device", "cuda.0")
        assert "23 tests, 0 failures" in out and "build only" not in out
