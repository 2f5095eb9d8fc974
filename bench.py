#!/usr/bin/env python
"""Benchmark of the Tile contraction hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--extras 0|1]

Workload (BASELINE.json configs[1]): the int8 x int8 -> int32 Tile GEMM, N = K = 4096, built
through the EDSL (operands cast to int32, sum-of-products contraction) and executed by the
`cuda` target.  Rows of M are sharded across GPUs with 4096 rows per GPU (weak scaling: the B
matrix is replicated, no data-path collective); `value` is the whole-job TOP/s with inputs
resident in HBM, `e2e` the same metric through `plaidml_executable_run` with host buffers.

One step = one pass of the compiled program over one (A, B) pair.  Prints ONE JSON line.
`--impl reference` times the CPU restatement of the reference's path (the oracle, all host
threads) on a bounded sample of the same workload: the reference itself cannot be built here.
"""

from __future__ import annotations

import argparse
import json
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

M_PER_GPU, N_DIM, K_DIM = 4096, 4096, 4096
WORKLOAD = "cfg2: int8 x int8 -> int32 Tile GEMM, N=K=4096, M=4096 rows per GPU (rows of M sharded)"
# dram__bytes_read.sum + dram__bytes_write.sum of one tc_contract launch of this workload, from
# the ncu capture summarised in profiles/tc_gemm_i8_4096.md
NCU_TRAFFIC_BYTES = 52.58e6


emit = None  # set by main(): writes the result line


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "_fallback": True}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled every millisecond
    from a thread (the region lasts a few milliseconds), nvidia-smi -lms as the fallback."""

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
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

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
            nv = self.nvml
            bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
            sm = sorted(m for m, _ in self.samples)
            reasons = sorted(name for name, bit in bits.items() if any(mask & bit for _, mask in self.samples))
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.sm_max, "reasons": reasons,
                    "samples": len(sm), "source": "nvml polled at 1 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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


def seeded_inputs(rank: int):
    # PRNG of the measurement plan: PCG64, seed = 1234 + configuration index (+ rank for the shard)
    g = np.random.Generator(np.random.PCG64(1234 + 2))
    b = g.integers(-128, 128, size=(K_DIM, N_DIM), dtype=np.int8)
    ga = np.random.Generator(np.random.PCG64(shard.shard_seed(1234 + 2, rank)))
    a = ga.integers(-128, 128, size=(M_PER_GPU, K_DIM), dtype=np.int8)
    return a, b


_CPU_INPUTS = None


def cpu_baseline(rows: int, threads: int, repeats: int = 1) -> dict:
    """Times the oracle's int8 GEMM loop nest on `rows` rows of the workload (inputs generated once, untimed)."""
    # The launcher of multi-process runs exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core,
    # so the variable is set here, before the OpenMP runtime of the checker library starts.
    os.environ["OMP_NUM_THREADS"] = str(threads)
    import oracle
    global _CPU_INPUTS
    if _CPU_INPUTS is None:
        _CPU_INPUTS = seeded_inputs(0)
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
        "ms_per_step": 1e3 * seconds, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8->int32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference path (the reference's LLVM/MLIR + "
                   "libxsmm build cannot be produced offline); int8 contractions take plain loops in the reference too"},
        "cpu_baseline": {"value": value, "unit": "TOP/s", "cores": threads, "kind": "port", "sample": results[0]["sample"]},
        "e2e": {"value": value, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def build_gemm_runner(device: str):
    from plaidml_b200 import programs as progs
    from plaidml_b200.core import DType, Program
    from plaidml_b200.exec import Runner
    A, B, C = progs.tile_gemm(DType.INT8, M_PER_GPU, N_DIM, K_DIM, acc=DType.INT32)
    return Runner(Program("tile_gemm_int8", [A, B], [C]), device)


def extras(device: str, iters: int) -> dict:
    """Short device-resident timings of the other configurations (kernel sequence only)."""
    from plaidml_b200 import programs as progs
    from plaidml_b200.core import DType, Program, f32_to_bf16_bits
    from plaidml_b200.edsl import Contraction, TensorIndexes
    from plaidml_b200.exec import Runner
    out = {}
    g = np.random.Generator(np.random.PCG64(99))
    # cfg1: fp32 1024^3 via 3xTF32
    A, B, C = progs.tile_gemm(DType.FLOAT32, 1024, 1024, 1024)
    r = Runner(Program("cfg1", [A, B], [C]), device)
    r.run([g.uniform(-1, 1, (1024, 1024)).astype(np.float32), g.uniform(-1, 1, (1024, 1024)).astype(np.float32)])
    ms = r.executable.time_steps(iters, True)
    out["cfg1_fp32_gemm_1024"] = {"ms": ms, "tflops": 2 * 1024**3 / ms / 1e9, "kernels": r.executable.launch_count}
    # bf16 4096^3 Tile GEMM
    A, B, C = progs.tile_gemm(DType.BFLOAT16, 4096, 4096, 4096, acc=DType.FLOAT32, out_bf16=True)
    r = Runner(Program("bf16_gemm", [A, B], [C]), device)
    x = f32_to_bf16_bits(g.standard_normal((4096, 4096)))
    r.run([x, x])
    ms = r.executable.time_steps(iters, True)
    out["bf16_gemm_4096"] = {"ms": ms, "tflops": 2 * 4096**3 / ms / 1e9}
    # cfg3: conv 3x3 N128 56x56 64->64 + bias + relu, bf16
    f = f32_to_bf16_bits(g.standard_normal((3, 3, 64, 64)) * np.sqrt(2.0 / 576))
    prog = progs.conv_bias_relu(128, 56, 56, 64, 64, filt=f, bias=np.zeros(64, np.float32))
    r = Runner(prog, device)
    r.run([f32_to_bf16_bits(g.uniform(0, 1, (128, 56, 56, 64)))])
    ms = r.executable.time_steps(iters, True)
    flops = 2.0 * 128 * 56 * 56 * 64 * 64 * 9
    out["cfg3_conv3x3_bias_relu"] = {"ms": ms, "tflops": flops / ms / 1e9, "hbm_gbs": 102.8e6 / ms / 1e6,
                                     "plan": r.executable.describe().strip()}
    # cfg5: QK^T-shaped batched GEMM + row max
    Q, Kt, S = progs.tile_gemm(DType.BFLOAT16, 512, 512, 64, acc=DType.FLOAT32, batch=1024, b_transposed=True)
    bb, i, j = TensorIndexes(3)
    R = Contraction(name="rowmax").outShape(1024, 512).outAccess(bb, i).max(S[bb, i, j]).build()
    r = Runner(Program("cfg5", [Q, Kt], [S, R]), device)
    q = f32_to_bf16_bits(g.standard_normal((1024, 512, 64)))
    r.run([q, q])
    ms = r.executable.time_steps(iters, True)
    out["cfg5_qk_gemm_rowmax"] = {"ms": ms, "gemm_tflops_equiv": 2.0 * 1024 * 512 * 512 * 64 / ms / 1e9,
                                  # operands once, S written once, R written once (the row maxima come out of
                                  # the GEMM's epilogue, S is not read back)
                                  "hbm_gbs": (2 * 1024 * 512 * 64 * 2 + 1024 * 512 * 512 * 4 + 1024 * 512 * 4) / ms / 1e6,
                                  "plan": r.executable.describe().strip()}
    # the same contractions when only R is asked for: S is an intermediate, never written
    r = Runner(Program("cfg5_r_only", [Q, Kt], [R]), device)
    r.run([q, q])
    ms = r.executable.time_steps(iters, True)
    out["cfg5_qk_rowmax_only"] = {"ms": ms, "gemm_tflops_equiv": 2.0 * 1024 * 512 * 512 * 64 / ms / 1e9,
                                  "hbm_gbs": (2 * 1024 * 512 * 64 * 2 + 1024 * 512 * 4) / ms / 1e6,
                                  "plan": r.executable.describe().strip()}
    # cfg4: ResNet-50 v1.5 inference, batch 256, 224x224x3 (device-resident kernel sequence)
    prog, _ = progs.resnet50(256)
    r = Runner(prog, device)
    r.run([f32_to_bf16_bits(g.uniform(0, 1, (256, 224, 224, 3)).astype(np.float32))])
    ms = r.executable.time_steps(max(3, iters // 2), True)
    out["cfg4_resnet50_b256"] = {"ms": ms, "images_per_s": 256 / ms * 1e3,
                                 "tflops": 256 * progs.RESNET50_GFLOP_PER_IMAGE / ms, "kernels": r.executable.launch_count}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--extras", type=int, default=1)
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
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        shard.barrier(dist)
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        return shard.max_over_ranks(dist, x, f"cuda:{local_rank}")

    device = info.device_id
    runner = build_gemm_runner(device)
    exe = runner.executable
    a, b = seeded_inputs(rank)
    runner.inputs[0].copy_from_ndarray(a)
    runner.inputs[1].copy_from_ndarray(b)

    # ---- e2e: plaidml_executable_run with host buffers (H2D and D2H inside the timed region)
    for _ in range(warm):
        exe.run(runner.inputs, runner.outputs)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        exe.run(runner.inputs, runner.outputs)   # synchronous: outputs are in host memory on return
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    ops_per_step = 2.0 * M_PER_GPU * N_DIM * K_DIM
    e2e_value = world * ops_per_step * args.steps / e2e_s / 1e12

    # ---- device-resident: the kernel sequence alone, CUDA events per pass, L2 flushed between passes
    # Warm-up: at least 30 passes, because the phase before this one leaves the GPU waiting on PCIe copies
    # (at 8 ranks most of the time) and its clocks take a few milliseconds of work to come back up.
    exe.time_steps(max(warm, 30), True)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    ms = exe.time_steps(args.steps, True)   # one CUDA-event pair per pass, passes enqueued ahead of the host's wait
    clocks = sampler.stop()
    barrier()
    rank_ms = shard.gather_floats(dist, ms, f"cuda:{local_rank}")
    # The timed region lasts a few milliseconds, less than most clock queries take; so the same kernel
    # sequence is also run back to back for about 0.3 s (untimed) under a second sampler: the clock and the
    # throttle reasons the kernel settles at under sustained load.
    probe = ClockSampler(local_rank)
    probe.start()
    exe.run_resident(max(1, int(300.0 / max(ms, 1e-3))))
    sustained = probe.stop()
    clocks["sustained_probe"] = {k: sustained.get(k) for k in ("sm_mhz", "reasons", "samples")}
    clocks["reasons"] = sorted(set(clocks.get("reasons", [])) | set(sustained.get("reasons", [])))
    barrier()
    ms = max_over_ranks(ms)
    value = world * ops_per_step / (ms * 1e-3) / 1e12

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    int8_peak = 2.0 * float(peaks["bf16_tflops"])
    per_gpu = ops_per_step / (ms * 1e-3) / 1e12
    line = {
        "metric": "tile_contraction_throughput", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8->int32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "256 MiB device buffer overwritten before every timed pass",
                   "timing": "CUDA events on the executable's stream around each pass; max over ranks",
                   "plan": exe.describe().strip()},
        "e2e": {"value": e2e_value, "unit": "TOP/s", "h2d_bytes_per_step": int(a.nbytes + b.nbytes),
                "d2h_bytes_per_step": int(M_PER_GPU * N_DIM * 4), "ms_per_step": 1e3 * e2e_s / args.steps},
        "gpu_launches": int(exe.launch_count * args.steps),
        "ms_per_step_by_rank": [round(x, 5) for x in rank_ms],
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": int8_peak, "unit": "TOP/s",
                     "frac": per_gpu / int8_peak, "traffic": NCU_TRAFFIC_BYTES,
                     "peak_source": ("2 x bf16_tflops of MEASURED_PEAKS.json (int8 dense peak derived from the measured "
                                     "bf16 burst figure; the file carries no int8 number)"
                                     if "_fallback" not in peaks else "2 x fallback bf16 figure"),
                     "kernel": "tc_contract_kernel (int8, CTA pairs on 256x256 tiles, cta_group::2 MMAs, B read as [k][n])",
                     "algorithmic_ops_per_launch": ops_per_step},
    }
    if args.gpus == 1 and world == 1:
        line["cpu_baseline"] = {k: v for k, v in cpu_baseline(args.cpu_baseline_rows, os.cpu_count() or 1).items() if k != "seconds"}
        if args.extras:
            try:
                line["other_configs"] = extras(device, max(5, args.steps // 2))
            except Exception as e:  # the headline line must still be printed
                line["other_configs"] = {"error": str(e)}
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
