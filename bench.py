#!/usr/bin/env python
"""Benchmark of the Tile contraction hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--extras 0|1] [--resnet 0|1]

Headline workload: the int8 x int8 -> int32 Tile GEMM with M = N = K = 4096, built through the EDSL
(operands cast to int32, sum-of-products contraction) and executed by the `cuda` target.  It is ONE
fixed problem: at N GPUs every rank computes its 4096 / N rows of M against the replicated B
(`"scaling": "strong"`), no data-path collective.  `value` is the whole-job TOP/s with inputs resident
in HBM (one CUDA-event pair per step on the executable's stream, L2 flushed before every step, max
over ranks); `e2e` is the same metric through `plaidml_executable_run` with host buffers, copies
inside the timed region (at N > 1 every rank uploads 1 / N of B and one NCCL all-gather inside the
library completes it).  One step = one pass of the compiled program over one (A, B) pair.

Every line also carries: `long_run` (the same pass repeated for at least 0.5 s: median, spread,
time x SM clock), `weak` (4096 rows per GPU, N > 1 only), `gathered` (the all-gather of the sharded
output over NCCL, N > 1 only), `host_link` (pinned copies in both directions on all GPUs at once: the
ceiling of any end-to-end figure on this box) and `resnet50` (ResNet-50 v1.5 inference, batch 256 in
all, 256 / N images per rank: images/s device-timed and end to end, with its own roofline).  At N = 1
`other_configs` times the remaining configurations, each with a roofline block.

Prints ONE JSON line.  `--impl reference` times the CPU restatement of the reference's path (the
checker library, all host threads) on the same workload: the reference itself cannot be built here.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from plaidml_b200 import shard  # noqa: E402  (pure Python; the CUDA library loads on first use)

M_DIM, N_DIM, K_DIM = 4096, 4096, 4096
WORKLOAD = ("cfg2: int8 x int8 -> int32 Tile GEMM, M=N=K=4096 (M = 4096 in all: rows of M sharded across the "
            "GPUs, B replicated)")
CONFIG = {"workload": WORKLOAD, "seed": "PCG64, 1234 + configuration index",
          "l2": "256 MiB device buffer overwritten before every timed pass"}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 4096-row kernel, from an ncu capture of
# this kernel at this shape (a profiler figure cannot be taken inside a timed run)
NCU_TRAFFIC_BYTES_4096 = 52.58e6
RESNET_BATCH = 256

emit = None  # set by main(): writes the result line


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "_fallback": True}


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: NVML polled every millisecond
    from a thread, nvidia-smi -lms as the fallback."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.nvml = None
        self.samples = []      # (sm MHz, reasons bitmask)
        self.stop_flag = False
        self.thread = None
        self.sm_max = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu
            if visible:
                ids = [x for x in visible.split(",") if x.strip() != ""]
                if self.gpu < len(ids) and ids[self.gpu].strip().isdigit():
                    index = int(ids[self.gpu])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _poll(self):
        nv = self.nvml
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, mask))
            except Exception:
                pass
            time.sleep(0.001)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
            bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
            sm = sorted(m for m, _ in self.samples)
            reasons = sorted(name for name, bit in bits.items() if any(mask & bit for _, mask in self.samples))
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.sm_max, "reasons": reasons,
                    "samples": len(sm), "source": "nvml polled at 1 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi -lms 100"}


def seeded_operands():
    """The whole cfg2 problem: A [4096, 4096] and B [4096, 4096], uniform integers in [-128, 127]."""
    g = np.random.Generator(np.random.PCG64(1234 + 2))
    a = g.integers(-128, 128, size=(M_DIM, K_DIM), dtype=np.int8)
    b = g.integers(-128, 128, size=(K_DIM, N_DIM), dtype=np.int8)
    return a, b


# ------------------------------------------------------------------------------------------ CPU arm

_CPU_INPUTS = None


def cpu_baseline(rows: int, threads: int, repeats: int = 1) -> dict:
    """Times the checker's int8 GEMM loop nest on `rows` rows of the workload (inputs generated once, untimed)."""
    # The launcher of multi-process runs exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core,
    # so the variable is set here, before the OpenMP runtime of the checker library starts.
    os.environ["OMP_NUM_THREADS"] = str(threads)
    import oracle
    global _CPU_INPUTS
    if _CPU_INPUTS is None:
        _CPU_INPUTS = seeded_operands()
    a, b = _CPU_INPUTS
    a = np.ascontiguousarray(a[:rows])
    oracle.gemm_i8_i32(a[:8], b)  # load the library, warm the caches
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.gemm_i8_i32(a, b)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    ops = 2.0 * rows * N_DIM * K_DIM
    return {"value": ops / best / 1e12, "unit": "TOP/s", "cores": threads, "kind": "port",
            "sample": f"{rows} of 4096 rows of A against the full 4096x4096 B (CPU restatement, OpenMP)",
            "seconds": best}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = args.cpu_baseline_rows
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_baseline(min(rows, 256), threads)
    results = [cpu_baseline(rows, threads) for _ in range(args.steps)]
    seconds = float(np.mean([r["seconds"] for r in results]))
    value = 2.0 * rows * N_DIM * K_DIM / seconds / 1e12
    line = {
        "impl": "reference", "metric": "tile_contraction_throughput", "value": value, "unit": "TOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * seconds, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8->int32", "data": "synthetic",
        "config": dict(CONFIG),
        "note": ("CPU restatement of the reference path on the host cores (the reference's LLVM/MLIR + libxsmm build "
                 "cannot be produced offline); int8 contractions take plain loops in the reference too"),
        "cpu_baseline": {"value": value, "unit": "TOP/s", "cores": threads, "kind": "port", "sample": results[0]["sample"]},
        "e2e": {"value": value, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# ------------------------------------------------------------------------------------------ helpers

def spread(ms: np.ndarray) -> dict:
    s = np.sort(np.asarray(ms, dtype=np.float64))
    n = len(s)
    return {"passes": int(n), "median_ms": float(s[n // 2]), "mean_ms": float(s.mean()), "p10_ms": float(s[int(0.1 * (n - 1))]),
            "p90_ms": float(s[int(0.9 * (n - 1))]), "min_ms": float(s[0]), "max_ms": float(s[-1])}


def long_run(exe, local_rank: int, est_ms: float, min_passes: int = 200, seconds: float = 0.5, max_passes: int = 4000) -> dict:
    """The same pass repeated until the timed passes alone add up to `seconds` (at least `min_passes`), every
    pass between its own event pair, clocks sampled throughout."""
    passes = int(min(max_passes, max(min_passes, math.ceil(seconds * 1e3 / max(est_ms, 1e-3)))))
    sampler = ClockSampler(local_rank).start()
    ms = exe.time_passes(passes, True)
    clocks = sampler.stop()
    out = spread(ms)
    out["timed_seconds"] = float(ms.sum() / 1e3)
    out["sm_mhz_median"] = clocks.get("sm_mhz")
    out["reasons"] = clocks.get("reasons")
    out["clock_samples"] = clocks.get("samples")
    if clocks.get("sm_mhz"):
        out["median_ms_x_sm_mhz"] = out["median_ms"] * clocks["sm_mhz"]
    return out


def build_gemm_runner(device: str, rows: int):
    from plaidml_b200 import programs as progs
    from plaidml_b200.core import DType, Program
    from plaidml_b200.exec import Runner
    A, B, C = progs.tile_gemm(DType.INT8, rows, N_DIM, K_DIM, acc=DType.INT32)
    return Runner(Program("tile_gemm_int8", [A, B], [C]), device)


def host_link_ceiling(torch, barrier, gather_floats, local_rank: int, mib: int = 64, reps: int = 8) -> dict:
    """Pinned host <-> device copies on every GPU of the job at once, one copy call per buffer: host -> device
    alone, device -> host alone, then both directions together on two streams.  GB/s summed over the ranks."""
    nbytes = mib << 20
    dev = torch.device("cuda", local_rank)
    h_up = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_dn = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_up = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_dn = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def timed(up: bool, down: bool) -> float:
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s1):
                    d_up.copy_(h_up, non_blocking=True)
            if down:
                with torch.cuda.stream(s2):
                    h_dn.copy_(d_dn, non_blocking=True)
        s1.synchronize()
        s2.synchronize()
        barrier()
        return time.perf_counter() - t0

    timed(True, True)
    out = {}
    for name, up, down in (("h2d", True, False), ("d2h", False, True), ("both", True, True)):
        secs = max(gather_floats(timed(up, down)))
        world = len(gather_floats(0.0))
        moved = world * reps * nbytes * ((1 if up else 0) + (1 if down else 0))
        out[name + "_gbs"] = moved / secs / 1e9
    out["what"] = f"{mib} MiB pinned buffers, {reps} copies per direction per rank, all ranks at once, wall clock, max over ranks"
    return out


def check_int8_rows(c_rows: np.ndarray, a_rows: np.ndarray, b: np.ndarray) -> bool:
    """Bit-exactness of a few rows against numpy's int64 product, and the row-sum identity on all given rows."""
    want = a_rows.astype(np.int64) @ b.astype(np.int64)
    return bool(np.array_equal(c_rows.astype(np.int64), want))


# ------------------------------------------------------------------------------------------ ResNet-50

def resnet_block(device: str, local_rank: int, world: int, steps: int, barrier, max_over_ranks, peaks) -> dict:
    from plaidml_b200 import programs as progs
    from plaidml_b200.core import f32_to_bf16_bits
    from plaidml_b200.exec import Runner
    if RESNET_BATCH % world != 0:
        return {"skipped": f"batch {RESNET_BATCH} does not divide by {world} ranks"}
    per_rank = RESNET_BATCH // world
    prog, _ = progs.resnet50(per_rank)
    r = Runner(prog, device)
    exe = r.executable
    g = np.random.Generator(np.random.PCG64(shard.shard_seed(1234 + 4, local_rank)))
    r.inputs[0].copy_from_ndarray(f32_to_bf16_bits(g.uniform(0, 1, (per_rank, 224, 224, 3)).astype(np.float32)))
    # end to end: image batch host -> device, the network, logits device -> host, every step
    for _ in range(3):
        exe.run(r.inputs, r.outputs)
    e2e_steps = max(5, min(steps, 20))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        exe.run(r.inputs, r.outputs)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0) / e2e_steps
    logits = r.outputs[0].as_ndarray()
    finite = bool(np.isfinite(logits).all())
    # device-resident: the kernel sequence (a replayed CUDA graph), each pass between its own events
    exe.time_steps(5, True)
    est = exe.time_steps(3, True)
    passes = int(min(400, max(20, math.ceil(500.0 / max(est, 1e-3)))))
    sampler = ClockSampler(local_rank).start()
    barrier()
    ms = exe.time_passes(passes, True)
    barrier()
    clocks = sampler.stop()
    sp = spread(ms)
    mean_ms = max_over_ranks(sp["mean_ms"])
    median_ms = max_over_ranks(sp["median_ms"])
    flops = RESNET_BATCH * progs.RESNET50_GFLOP_PER_IMAGE * 1e9
    peak = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    per_gpu_tflops = per_rank * progs.RESNET50_GFLOP_PER_IMAGE / mean_ms
    in_bytes = per_rank * 224 * 224 * 3 * 2
    return {
        "workload": f"cfg4: ResNet-50 v1.5 inference, batch {RESNET_BATCH} in all ({per_rank} images per GPU), NHWC 224x224x3, "
                    "bf16 with fp32 accumulation, He-normal weights",
        "images_per_s": RESNET_BATCH / mean_ms * 1e3, "ms_per_step": mean_ms, "median_ms_per_step": median_ms,
        "passes": passes, "timed_seconds": float(ms.sum() / 1e3), "kernels_per_pass": exe.launch_count,
        "cuda_graph": bool(exe.uses_graph),
        "e2e": {"images_per_s": RESNET_BATCH / e2e_s, "ms_per_step": 1e3 * e2e_s, "steps": e2e_steps,
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": per_rank * 1000 * 4, "logits_finite": finite},
        "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu_tflops / peak,
                     "traffic": None, "per": "GPU", "flop_per_image": progs.RESNET50_GFLOP_PER_IMAGE * 1e9,
                     "job_tflops": flops / (mean_ms * 1e-3) / 1e12,
                     "peak_source": "bf16_tflops_sustained of MEASURED_PEAKS.json (a kernel sequence inside a long step)"},
        "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons", "samples")},
    }


# ------------------------------------------------------------------------------------------ other configurations

def extras(device: str, local_rank: int, peaks: dict) -> dict:
    """Device-resident timings of the other configurations (kernel sequence only), each with its roofline."""
    import torch
    from plaidml_b200 import programs as progs
    from plaidml_b200.core import DType, Program, bf16_bits_to_f32, f32_to_bf16_bits
    from plaidml_b200.edsl import Contraction, TensorIndexes
    from plaidml_b200.exec import Runner
    out = {}
    burst = float(peaks["bf16_tflops"])
    hbm = float(peaks["hbm_gbs"])
    dev = torch.device("cuda", local_rank)

    def timed(r, est_passes=200):
        r.executable.time_steps(5, True)
        sampler = ClockSampler(local_rank).start()
        ms = r.executable.time_passes(est_passes, True)
        clocks = sampler.stop()
        sp = spread(ms)
        sp["sm_mhz_median"] = clocks.get("sm_mhz")
        sp["reasons"] = clocks.get("reasons")
        return sp

    # write-only bandwidth of HBM: a fill over 1 GiB (the bound of the output-heavy launches below)
    buf = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for _ in range(2):
        buf.fill_(1)
    best = None
    for i in range(5):
        ev[0].record()
        buf.fill_(i)
        ev[1].record()
        ev[1].synchronize()
        t = ev[0].elapsed_time(ev[1])
        best = t if best is None else min(best, t)
    del buf
    write_gbs = (1 << 30) / best / 1e6
    out["hbm_write_only"] = {"gbs": write_gbs, "what": "fill of a 1 GiB device buffer, best of 5 (CUDA events)"}

    # cfg1: fp32 1024^3 via 3xTF32
    g = np.random.Generator(np.random.PCG64(1234 + 1))
    A, B, C = progs.tile_gemm(DType.FLOAT32, 1024, 1024, 1024)
    r = Runner(Program("cfg1", [A, B], [C]), device)
    a = g.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    b = g.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    got = r.run([a, b])[0]
    rows = [0, 511, 1023]
    want = a[rows].astype(np.float64) @ b.astype(np.float64)
    err = float(np.max(np.abs(got[rows] - want)) / np.max(np.abs(want)))
    sp = timed(r)
    tf = 2 * 1024**3 / sp["mean_ms"] / 1e9
    # three TF32 products per fp32 product, TF32 at half the bf16 rate
    out["cfg1_fp32_gemm_1024"] = {
        **sp, "tflops": tf, "kernels": r.executable.launch_count, "check": {"rows_vs_f64": err, "ok": err < 1e-5},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": burst / 6.0, "unit": "TFLOP/s", "frac": tf / (burst / 6.0),
                     "traffic": None, "peak_source": "bf16_tflops / 6: TF32 runs at half the bf16 rate and an fp32 product is three TF32 products"}}

    # bf16 4096^3 Tile GEMM
    g = np.random.Generator(np.random.PCG64(1234 + 6))
    A, B, C = progs.tile_gemm(DType.BFLOAT16, 4096, 4096, 4096, acc=DType.FLOAT32, out_bf16=True)
    r = Runner(Program("bf16_gemm", [A, B], [C]), device)
    x = f32_to_bf16_bits(g.standard_normal((4096, 4096)))
    y = f32_to_bf16_bits(g.standard_normal((4096, 4096)))
    got = bf16_bits_to_f32(r.run([x, y])[0][[0, 4095]])
    want = bf16_bits_to_f32(x[[0, 4095]]).astype(np.float64) @ bf16_bits_to_f32(y).astype(np.float64)
    err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
    sp = timed(r)
    tf = 2 * 4096**3 / sp["mean_ms"] / 1e9
    out["bf16_gemm_4096"] = {**sp, "tflops": tf, "check": {"rows_vs_f64": err, "ok": err < 1e-2},
                             "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s",
                                          "frac": tf / burst, "traffic": None, "peak_source": "bf16_tflops of MEASURED_PEAKS.json"}}

    # cfg3: conv 3x3 N128 56x56 64->64 + bias + relu, bf16
    g = np.random.Generator(np.random.PCG64(1234 + 3))
    f = f32_to_bf16_bits(g.standard_normal((3, 3, 64, 64)) * np.sqrt(2.0 / 576))
    prog = progs.conv_bias_relu(128, 56, 56, 64, 64, filt=f, bias=np.zeros(64, np.float32))
    r = Runner(prog, device)
    img = f32_to_bf16_bits(g.uniform(0, 1, (128, 56, 56, 64)))
    got = bf16_bits_to_f32(r.run([img])[0])
    # a corner, an edge and an interior pixel of two images against the definition
    xf, ff = bf16_bits_to_f32(img), bf16_bits_to_f32(f).astype(np.float64)
    err = 0.0
    for (n_, y_, x_) in [(0, 0, 0), (0, 0, 17), (5, 30, 41), (127, 55, 55), (64, 55, 0)]:
        acc = np.zeros(64)
        for fr in range(3):
            for fs in range(3):
                yy, xx = y_ + fr - 1, x_ + fs - 1
                if 0 <= yy < 56 and 0 <= xx < 56:
                    acc += xf[n_, yy, xx].astype(np.float64) @ ff[fr, fs]
        err = max(err, float(np.max(np.abs(got[n_, y_, x_] - np.maximum(acc, 0))) / max(1e-6, float(np.max(np.abs(acc))))))
    sp = timed(r)
    flops = 2.0 * 128 * 56 * 56 * 64 * 64 * 9
    tf = flops / sp["mean_ms"] / 1e9
    out["cfg3_conv3x3_bias_relu"] = {
        **sp, "tflops": tf, "hbm_gbs": 102.8e6 / sp["mean_ms"] / 1e6, "plan": r.executable.describe().strip(),
        "check": {"pixels_vs_f64": err, "ok": err < 1e-2},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst, "traffic": None,
                     "peak_source": "bf16_tflops of MEASURED_PEAKS.json", "algorithmic_bytes": 102.8e6}}

    # cfg5: QK^T-shaped batched GEMM + row max
    g = np.random.Generator(np.random.PCG64(1234 + 5))
    Q, Kt, S = progs.tile_gemm(DType.BFLOAT16, 512, 512, 64, acc=DType.FLOAT32, batch=1024, b_transposed=True)
    bb, i, j = TensorIndexes(3)
    R = Contraction(name="rowmax").outShape(1024, 512).outAccess(bb, i).max(S[bb, i, j]).build()
    r = Runner(Program("cfg5", [Q, Kt], [S, R]), device)
    q = f32_to_bf16_bits(g.standard_normal((1024, 512, 64)))
    kk = f32_to_bf16_bits(g.standard_normal((1024, 512, 64)))
    s_out, r_out = r.run([q, kk])
    ok = bool(np.array_equal(r_out[:8], s_out[:8].max(axis=2)))
    want = bf16_bits_to_f32(q[3]).astype(np.float64) @ bf16_bits_to_f32(kk[3]).astype(np.float64).T
    err = float(np.max(np.abs(s_out[3] - want)) / np.max(np.abs(want)))
    del s_out
    sp = timed(r, 100)
    alg = 2 * 1024 * 512 * 64 * 2 + 1024 * 512 * 512 * 4 + 1024 * 512 * 4   # operands once, S and R written once
    gbs = alg / sp["mean_ms"] / 1e6
    out["cfg5_qk_gemm_rowmax"] = {
        **sp, "gemm_tflops_equiv": 2.0 * 1024 * 512 * 512 * 64 / sp["mean_ms"] / 1e9, "hbm_gbs": gbs,
        "plan": r.executable.describe().strip(), "check": {"rowmax_equals_max_of_S": ok, "entry_vs_f64": err, "ok": ok and err < 1e-2},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None,
                     "peak_source": "hbm_gbs of MEASURED_PEAKS.json (a copy: half reads, half writes)",
                     "write_only_gbs_this_run": write_gbs, "frac_of_write_only": (1024 * 512 * 512 * 4) / sp["mean_ms"] / 1e6 / write_gbs,
                     "algorithmic_bytes": alg}}
    # the same contractions when only R is asked for: S is an intermediate, never written
    r = Runner(Program("cfg5_r_only", [Q, Kt], [R]), device)
    r_only = r.run([q, kk])[0]
    sp = timed(r)
    tf = 2.0 * 1024 * 512 * 512 * 64 / sp["mean_ms"] / 1e9
    out["cfg5_qk_rowmax_only"] = {
        **sp, "gemm_tflops_equiv": tf, "plan": r.executable.describe().strip(),
        "check": {"equals_rowmax_with_S_stored": bool(np.array_equal(r_only, r_out)), "ok": bool(np.array_equal(r_only, r_out))},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst, "traffic": None,
                     "peak_source": "bf16_tflops of MEASURED_PEAKS.json"}}
    # the operations beside the path that are not contractions; a failure here must not take the line down
    try:
        out["gather_argsort_prng"] = special_extras(device, hbm, timed)
    except Exception as exc:  # noqa: BLE001
        out["gather_argsort_prng"] = {"error": str(exc)[:300]}
    return out


def special_extras(device: str, hbm: float, timed) -> dict:
    """gather / argsort / prng on large inputs: device time per launch, algorithmic bytes, a check of sampled results."""
    from plaidml_b200 import edsl
    from plaidml_b200.core import DType, Program
    from plaidml_b200.edsl import Placeholder
    from plaidml_b200.exec import Runner
    out = {}
    g = np.random.Generator(np.random.PCG64(1234 + 7))
    rows, width, picks = 1 << 20, 64, 1 << 21
    T, I = Placeholder(DType.FLOAT32, [rows, width]), Placeholder(DType.INT32, [picks])
    r = Runner(Program("gather_rows", [T, I], [edsl.gather(T, I)]), device)
    table = g.standard_normal((rows, width), dtype=np.float32)
    idx = g.integers(0, rows, picks, dtype=np.int32)
    got = r.run([table, idx])[0]
    sample = g.integers(0, picks, 2000)
    ok = bool(np.array_equal(got[sample], table[idx[sample]]))
    del got
    sp = timed(r, 50)
    alg = picks * 4 + 2 * picks * width * 4
    gbs = alg / sp["mean_ms"] / 1e6
    out["gather_2m_rows_of_64_f32"] = {**sp, "check": {"sampled_rows_equal": ok, "ok": ok},
                                       "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                                                    "traffic": None, "algorithmic_bytes": alg,
                                                    "peak_source": "hbm_gbs of MEASURED_PEAKS.json"}}
    lines, n = 2048, 4096
    X = Placeholder(DType.FLOAT32, [lines, n])
    r = Runner(Program("argsort", [X], [edsl.argsort(X, 1)]), device)
    x = g.standard_normal((lines, n), dtype=np.float32)
    got = r.run([x])[0]
    ok = bool(np.array_equal(got[:8], np.argsort(x[:8], axis=1, kind="stable").astype(np.int32)))
    sp = timed(r, 50)
    out["argsort_2048_lines_of_4096_f32"] = {**sp, "keys_per_s": lines * n / sp["mean_ms"] * 1e3,
                                             "check": {"first_lines_equal_stable_sort": ok, "ok": ok}}
    count = 1 << 26
    S = Placeholder(DType.UINT32, [3])
    numbers, state = edsl.prng(S, [count])
    r = Runner(Program("prng", [S], [numbers, state]), device)
    got, after = r.run([np.array([5, 6, 7], dtype=np.uint32)])
    s = [5, 6, 7]
    want = []
    for _ in range(64):   # the sequential generator (pmlc/rt/prng.cc:26-39)
        want.append(np.float32((s[0] ^ s[1] ^ s[2]) / 4294967296.0))
        s = [(((s[0] & 4294967294) << 12) & 0xFFFFFFFF) ^ ((((s[0] << 13) & 0xFFFFFFFF) ^ s[0]) >> 19),
             (((s[1] & 4294967288) << 4) & 0xFFFFFFFF) ^ ((((s[1] << 2) & 0xFFFFFFFF) ^ s[1]) >> 25),
             (((s[2] & 4294967280) << 17) & 0xFFFFFFFF) ^ ((((s[2] << 3) & 0xFFFFFFFF) ^ s[2]) >> 11)]
    ok = bool(np.array_equal(got[:64], np.array(want, dtype=np.float32)))
    del got
    sp = timed(r, 50)
    gbs = count * 4 / sp["mean_ms"] / 1e6
    out["prng_64m_numbers"] = {**sp, "check": {"first_64_equal_the_sequential_generator": ok, "ok": ok},
                               "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                                            "traffic": None, "algorithmic_bytes": count * 4,
                                            "peak_source": "hbm_gbs of MEASURED_PEAKS.json",
                                            "note": "bound by the generators' integer operations, not by HBM"}}
    return out


def library_int8_tops(torch, local_rank: int) -> float | None:
    """What the vendor library reaches on the headline shape in this run (torch._int_mm, best of 10)."""
    try:
        dev = torch.device("cuda", local_rank)
        a = torch.randint(-128, 128, (M_DIM, K_DIM), dtype=torch.int8, device=dev)
        b = torch.randint(-128, 128, (K_DIM, N_DIM), dtype=torch.int8, device=dev)
        for _ in range(3):
            torch._int_mm(a, b)
        best = None
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for _ in range(10):
            ev[0].record()
            torch._int_mm(a, b)
            ev[1].record()
            ev[1].synchronize()
            t = ev[0].elapsed_time(ev[1])
            best = t if best is None else min(best, t)
        return 2.0 * M_DIM * N_DIM * K_DIM / best / 1e9
    except Exception:
        return None


# ------------------------------------------------------------------------------------------ main

def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--extras", type=int, default=1)
    ap.add_argument("--resnet", type=int, default=1)
    ap.add_argument("--cpu-baseline-rows", type=int, default=4096)
    args = ap.parse_args()
    # Exactly one line goes to standard output: libraries that print there (NCCL's version banner) are sent
    # to standard error for the duration of the run and the result line is written to the saved descriptor.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)
    global emit

    def emit(line: dict) -> None:
        os.write(result_fd, (json.dumps(line) + "\n").encode())

    if args.impl == "reference":
        run_reference_arm(args)
        return

    info = shard.RankInfo.from_env()
    rank, local_rank, world = info.rank, info.local_rank, info.world
    warm = max(3, args.warmup)

    import torch
    dist = None
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        shard.init_library(dist, info)     # the library's own communicator (replicated B, gathered output)

    cuda_dev = f"cuda:{local_rank}"

    def barrier():
        shard.barrier(dist)
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        return shard.max_over_ranks(dist, x, cuda_dev)

    def gather_floats(x: float) -> list:
        return shard.gather_floats(dist, x, cuda_dev)

    peaks = measured_peaks()
    device = info.device_id
    lo, hi = shard.row_slice(M_DIM, rank, world)
    rows = hi - lo
    runner = build_gemm_runner(device, rows)
    exe = runner.executable
    a_full, b = seeded_operands()
    a = np.ascontiguousarray(a_full[lo:hi])
    runner.inputs[0].copy_from_ndarray(a)
    runner.inputs[1].copy_from_ndarray(b)
    if world > 1:
        exe.set_input_replicated(1, True)

    # ---- e2e: plaidml_executable_run with host buffers (H2D and D2H inside the timed region)
    for _ in range(warm):
        exe.run(runner.inputs, runner.outputs)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        exe.run(runner.inputs, runner.outputs)   # synchronous: outputs are in host memory on return
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    ops_total = 2.0 * M_DIM * N_DIM * K_DIM
    ops_rank = 2.0 * rows * N_DIM * K_DIM
    e2e_value = ops_total * args.steps / e2e_s / 1e12
    c_host = runner.outputs[0].as_ndarray()
    sample = [0, rows // 2, rows - 1]
    parity_ok = check_int8_rows(c_host[sample], a[sample], b)
    parity_ok = parity_ok and bool(np.array_equal(c_host.astype(np.int64).sum(axis=1),
                                                  a.astype(np.int64) @ b.astype(np.int64).sum(axis=1)))

    # ---- device-resident: the kernel sequence alone, CUDA events per pass, L2 flushed between passes.
    # Warm-up: at least 30 passes, because the phase before this one leaves the GPU waiting on host copies
    # and its clocks take a few milliseconds of work to come back up.
    exe.time_steps(max(warm, 30), True)
    sampler = ClockSampler(local_rank).start()
    barrier()
    step_ms = exe.time_passes(args.steps, True)   # exactly K steps, one event pair each, enqueued ahead of the host's wait
    barrier()
    ms_rank = float(step_ms.mean())
    rank_ms = gather_floats(ms_rank)
    ms = max(rank_ms)
    median_ms = max_over_ranks(float(np.median(step_ms)))
    value = ops_total / (ms * 1e-3) / 1e12
    # the timed steps above last about a millisecond: the same pass repeated for half a second under the same
    # sampler gives the median, the spread and the clock the kernel settles at
    lr = long_run(exe, local_rank, ms_rank + 0.07)
    clocks = sampler.stop()
    lr_median = max_over_ranks(lr["median_ms"])
    lr["median_ms_max_over_ranks"] = lr_median
    lr["value_at_median"] = ops_total / (lr_median * 1e-3) / 1e12
    barrier()

    line_extra = {}
    if world > 1:
        # weak-scaled secondary figure: 4096 rows on every GPU
        wr = build_gemm_runner(device, M_DIM)
        wr.inputs[0].copy_from_ndarray(a_full)
        wr.inputs[1].copy_from_ndarray(b)
        wr.executable.run(wr.inputs, wr.outputs)
        wr.executable.time_steps(30, True)
        barrier()
        wms = max_over_ranks(float(wr.executable.time_passes(max(args.steps, 50), True).mean()))
        barrier()
        line_extra["weak"] = {"workload": "4096 rows of M per GPU (M = 4096 x N in all)", "ms_per_step": wms,
                              "value": world * ops_total / (wms * 1e-3) / 1e12, "unit": "TOP/s"}
        del wr
        # the sharded output gathered on every GPU: one NCCL all-gather inside the library
        barrier()
        _, gbytes, gms = exe.gather_output(0, iters=20)
        gms = max_over_ranks(gms)
        line_extra["gathered"] = {"what": "all-gather of the sharded C (int32) over NCCL, in the library, 20 in a row",
                                  "bytes_out_per_rank": gbytes, "ms": gms, "algbw_gbs": gbytes / gms / 1e6,
                                  "busbw_gbs": gbytes * (world - 1) / world / gms / 1e6}
    host_link = host_link_ceiling(torch, barrier, gather_floats, local_rank)
    h2d_step = int(a.nbytes + (b.nbytes // world if world > 1 else b.nbytes))
    d2h_step = int(rows * N_DIM * 4)
    # the time the step's bytes need on the measured link if both directions overlap perfectly
    floor_s = max(world * h2d_step / (host_link["h2d_gbs"] * 1e9), world * d2h_step / (host_link["d2h_gbs"] * 1e9))
    e2e_ms = 1e3 * e2e_s / args.steps

    resnet = None
    if args.resnet:
        try:
            barrier()
            resnet = resnet_block(device, local_rank, world, args.steps, barrier, max_over_ranks, peaks)
        except Exception as e:  # the headline line must still be printed
            resnet = {"error": f"{type(e).__name__}: {e}"}
        barrier()

    if rank != 0:
        if dist is not None:
            shard.shutdown_library()
            dist.destroy_process_group()
        return

    int8_peak = 2.0 * float(peaks["bf16_tflops"])
    per_gpu = ops_rank / (ms * 1e-3) / 1e12
    line = {
        "metric": "tile_contraction_throughput", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "median_ms_per_step": median_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8->int32", "data": "synthetic",
        "config": dict(CONFIG),
        "method": {"timing": "CUDA events on the executable's stream around each step; mean of the K steps, max over ranks",
                   "rows_per_gpu": rows, "plan": exe.describe().strip()},
        "e2e": {"value": e2e_value, "unit": "TOP/s", "h2d_bytes_per_step": h2d_step, "d2h_bytes_per_step": d2h_step,
                "ms_per_step": e2e_ms, "replicated_operand": ("1/N of B per rank + NCCL all-gather" if world > 1 else "whole B"),
                "host_link_floor_ms": 1e3 * floor_s, "frac_of_host_link": 1e3 * floor_s / e2e_ms},
        "gpu_launches": int(exe.launch_count * args.steps),
        "ms_per_step_by_rank": [round(x, 5) for x in rank_ms],
        "parity": {"check": "rows 0, mid, last bit-exact against numpy int64; row-sum identity on every row of this rank's C "
                            "(output of the end-to-end phase)", "ok": parity_ok},
        "clocks": clocks,
        "long_run": lr,
        "host_link": host_link,
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": int8_peak, "unit": "TOP/s",
                     "frac": per_gpu / int8_peak,
                     "traffic": NCU_TRAFFIC_BYTES_4096 if rows == M_DIM else None,
                     "traffic_source": ("ncu capture of this kernel at this shape (dram read + write bytes of one launch); "
                                        "a constant of the source, not measured in this run" if rows == M_DIM else
                                        "no capture at this shard shape"),
                     "peak_source": ("2 x bf16_tflops of MEASURED_PEAKS.json (int8 dense peak derived from the measured "
                                     "bf16 burst figure; the file carries no int8 number)"
                                     if "_fallback" not in peaks else "2 x fallback bf16 figure"),
                     "per": "GPU",
                     "kernel": "tc_contract_kernel (int8, tcgen05.mma kind::i8, B read as [k][n])",
                     "algorithmic_ops_per_launch": ops_rank},
    }
    line["clocks"]["covers"] = "the K timed steps and the long run after them (same kernel)"
    line.update(line_extra)
    if resnet is not None:
        line["resnet50"] = resnet
    lib = library_int8_tops(torch, local_rank) if world == 1 else None
    if lib is not None:
        line["roofline"]["library_int8_tops_this_run"] = lib
        line["roofline"]["frac_of_library"] = per_gpu / lib
    if args.gpus == 1 and world == 1:
        line["cpu_baseline"] = {k: v for k, v in cpu_baseline(args.cpu_baseline_rows, os.cpu_count() or 1).items() if k != "seconds"}
        if args.extras:
            try:
                line["other_configs"] = extras(device, local_rank, peaks)
            except Exception as e:  # the headline line must still be printed
                line["other_configs"] = {"error": f"{type(e).__name__}: {e}"}
    emit(line)
    if dist is not None:
        shard.shutdown_library()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
