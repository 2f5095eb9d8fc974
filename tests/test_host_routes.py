"""Pure host-side decision code of the kernel library (division constants for tile coordinates,
convolution routes), compiled with g++ and run on the CPU."""

import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def cuda_include():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    inc = Path(nvcc).resolve().parent.parent / "include"
    return inc if (inc / "cuda.h").exists() else None


def test_route_and_division_checks(tmp_path):
    inc = cuda_include()
    if inc is None or shutil.which("g++") is None:
        pytest.skip("needs g++ and the CUDA headers")
    exe = tmp_path / "route_check"
    cmd = ["g++", "-std=c++17", "-O2", "-I", str(ROOT / "include"), "-I", str(ROOT / "plaidml_b200/csrc/kernels"),
           "-I", str(inc), str(ROOT / "tests/host/route_check.cc"), "-o", str(exe)]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    lines = res.stdout.strip().splitlines()
    assert lines and all(ln.startswith("ok ") for ln in lines), res.stdout
    assert res.returncode == 0
    assert len(lines) >= 15
