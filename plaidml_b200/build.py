"""Builds ``libplaidml.so`` (the C-ABI boundary plus the sm_100a kernels) in-tree with nvcc.

Usage: ``python -m plaidml_b200.build [--force] [--verbose]``.  Objects are cached under
``build/`` next to the repository root and rebuilt when a source or any header is newer.
Cross-compiles without a GPU.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = ROOT / "build" / "obj"
LIB_PATH = PKG_DIR / "libplaidml.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libplaidml.so")
    return cand


def _sources() -> list[Path]:
    srcs = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "host").glob("*.cc"))
    return srcs


def _headers_mtime() -> float:
    newest = 0.0
    for pat in ("**/*.h", "**/*.cuh"):
        for p in CSRC.glob(pat):
            newest = max(newest, p.stat().st_mtime)
    for p in (ROOT / "include").glob("*.h"):
        newest = max(newest, p.stat().st_mtime)
    return newest


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> None:
    cmd = [
        nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC",
        "-I", str(ROOT / "include"), "-I", str(CSRC / "kernels"), "-I", str(CSRC / "host"),
        "-DPMLB_BUILDING_LIBRARY",
    ]
    if src.suffix == ".cc":
        cmd += ["-x", "cu"]  # host files include cuda_runtime.h; one toolchain for everything
    if os.environ.get("PMLB_TC_TRACE"):
        cmd += ["-DPMLB_TC_TRACE"]   # the kernel's timeline records (see pmlb_debug_set_trace)
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _headers_mtime()
    jobs = []
    objs = []
    for src in _sources():
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_mtime)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o in jobs]
            for f in futs:
                f.result()
    need_link = force or bool(jobs) or not LIB_PATH.exists()
    if need_link:
        cmd = [
            nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *[str(o) for o in objs],
            "-Xlinker", f"--version-script={CSRC / 'exports.lds'}",
        ]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link of libplaidml.so failed")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
