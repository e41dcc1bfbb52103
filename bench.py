#!/usr/bin/env python
"""Benchmark of the SOFIE inference hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  A step is one pass of the hot path over one batch of synthetic
input.  The default workload is the int8 QLinearMatMul M=N=K=4096 (per-tensor symmetric scales
0.02 / 0.01, output scale 0.5, zero points 0): A [M,K] and B [K,N] int8 uniform in [-127,127],
int32 accumulation, ONNX requantisation to int8 fused in the kernel's epilogue.

  value      whole-job TOPS with operands resident in HBM (CUDA events, max over ranks)
  e2e        the same metric through the C ABI's host-operand call (sofie_b200_gemm_run_host_many, a queue of inferences):
             pinned host A and B copied in, Y copied out, inside the timed region
  roofline   the contraction kernel against the dense tensor peak measured on this pool
  cpu_baseline  the CPU restatement (oracle/) timed on the host cores on a bounded row sample

With --impl reference the CPU implementation is the thing timed (rank 0 only).  Multi-GPU runs
are launched with torchrun; every rank runs its own replica of the workload on its own GPU and
nothing crosses NVLink on the data path (weak scaling).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (None until a capture exists for that workload).
NCU_TRAFFIC_BYTES = {
    "qlinear_matmul_4096": 33.64e6 + 0.03e6,  # profiles/umma_gemm_i8_qlinear_matmul_4096.md
    "fp8_gemm_8192": None,
    "layernorm_bf16_65536x512": None,
    "softmax_bf16_524288x128": None,
}


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (NVML, read-only)."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            uuid_index = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                ent = vis.split(",")[self.index]
                uuid_index = int(ent) if ent.isdigit() else self.index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(uuid_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
            return
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()

    def _run(self):
        nv = self._nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period)

    def stop(self) -> dict:
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
class QLinearMatMul:
    """int8 x int8 -> int32 -> requantised int8 (ONNX QLinearMatMul), square."""

    def __init__(self, n: int, name: str):
        self.name, self.n = name, n
        self.ops = 2.0 * n * n * n
        self.unit = "TOPS"
        self.metric = f"int8 QLinearMatMul {n}^3 throughput"
        self.dtype = "int8"
        self.a_scale, self.b_scale, self.y_scale = np.float32(0.02), np.float32(0.01), np.float32(0.5)
        self.mult = float(np.float32(self.a_scale * self.b_scale) / self.y_scale)  # fp32 on the host, once
        self.bytes_alg = 3.0 * n * n

    def host_operands(self, seed: int):
        rng = np.random.default_rng(seed)
        a = rng.integers(-127, 128, size=(self.n, self.n), dtype=np.int8)
        b = rng.integers(-127, 128, size=(self.n, self.n), dtype=np.int8)
        return a, b

    def epilogue(self):
        from sofie_b200.ops import make_epilogue
        return make_epilogue(alpha=self.mult)

    def plan(self, ctx):
        import torch
        from sofie_b200.ops import GemmPlan
        return GemmPlan(ctx, self.n, self.n, self.n, torch.int8, torch.int8, trans_b=False)

    def torch_dtypes(self):
        import torch
        return torch.int8, torch.int8

    # CPU restatement on `rows` rows of A (all of B): ops = 2*rows*n*n
    def cpu_rows(self, lib, a, b, rows: int) -> float:
        from sofie_b200 import lib as L
        d = L.GemmDesc()
        d.M, d.N, d.K, d.batch = rows, self.n, self.n, 1
        d.ab_dtype, d.y_dtype = L.I8, L.I8
        e = L.Epilogue()
        e.alpha, e.beta, e.out_scale = self.mult, 1.0, 1.0
        y = np.zeros((rows, self.n), dtype=np.int8)
        t0 = time.perf_counter()
        lib.so_gemm(C.byref(d), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), C.byref(e))
        return time.perf_counter() - t0


class Fp8Gemm(QLinearMatMul):
    """FP8 e4m3 x e4m3 -> fp32, per-row / per-column scales, bias, Gelu, bf16 output."""

    def __init__(self, n: int, name: str):
        super().__init__(n, name)
        self.metric = f"FP8 e4m3 GEMM {n}^3 + scales + bias + Gelu -> bf16 throughput"
        self.unit = "TFLOP/s"
        self.dtype = "fp8_e4m3"
        self.bytes_alg = 2.0 * n * n + 2.0 * n * n

    def host_operands(self, seed: int):
        import torch
        g = torch.Generator().manual_seed(seed)
        a = torch.randn(self.n, self.n, generator=g)
        b = torch.randn(self.n, self.n, generator=g)
        self.sa = (a.abs().amax(dim=1) / 448.0).contiguous()
        self.sb = (b.abs().amax(dim=0) / 448.0).contiguous()
        self.bias = (torch.randn(self.n, generator=g) * 0.1).contiguous()
        a8 = (a / self.sa[:, None]).to(torch.float8_e4m3fn)
        b8 = (b / self.sb[None, :]).to(torch.float8_e4m3fn)
        return a8.view(torch.uint8).numpy(), b8.view(torch.uint8).numpy()

    def epilogue(self):
        from sofie_b200 import lib as L
        from sofie_b200.ops import make_epilogue
        dev = "cuda"
        self._keep = (self.sa.to(dev), self.sb.to(dev), self.bias.to(dev))
        return make_epilogue(row_scale=self._keep[0], col_scale=self._keep[1], bias=self._keep[2], act=L.ACT_GELU_ERF)

    def plan(self, ctx):
        import torch
        from sofie_b200.ops import GemmPlan
        return GemmPlan(ctx, self.n, self.n, self.n, torch.float8_e4m3fn, torch.bfloat16, trans_b=False)

    def torch_dtypes(self):
        import torch
        return torch.float8_e4m3fn, torch.bfloat16

    def cpu_rows(self, lib, a, b, rows: int) -> float:
        from sofie_b200 import lib as L
        d = L.GemmDesc()
        d.M, d.N, d.K, d.batch = rows, self.n, self.n, 1
        d.ab_dtype, d.y_dtype = L.F8E4M3, L.BF16
        e = L.Epilogue()
        sa, sb, bias = self.sa.numpy(), self.sb.numpy(), self.bias.numpy()
        e.row_scale, e.col_scale = sa.ctypes.data_as(C.c_void_p), sb.ctypes.data_as(C.c_void_p)
        e.alpha, e.beta, e.out_scale = 1.0, 1.0, 1.0
        e.bias_mode, e.bias, e.act = L.BIAS_COL_F32, bias.ctypes.data_as(C.c_void_p), L.ACT_GELU_ERF
        y = np.zeros((rows, self.n), dtype=np.uint16)
        t0 = time.perf_counter()
        lib.so_gemm(C.byref(d), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), C.byref(e))
        return time.perf_counter() - t0


WORKLOADS = {
    "qlinear_matmul_4096": lambda: QLinearMatMul(4096, "qlinear_matmul_4096"),
    "fp8_gemm_8192": lambda: Fp8Gemm(8192, "fp8_gemm_8192"),
}


def load_oracle():
    """The CPU checker library; only the CPU-baseline legs use it."""
    so = ROOT / "oracle" / "libsofie_oracle.so"
    if not so.exists():
        import subprocess
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    lib = C.CDLL(str(so))
    lib.so_threads.restype = C.c_int
    lib.so_set_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1; the CPU arm gets every host core
    return lib


def cpu_sample(w, budget_s: float):
    """Times the CPU restatement on a row sample sized to about `budget_s` seconds."""
    lib = load_oracle()
    a, b = w.host_operands(seed=1)
    t = w.cpu_rows(lib, a, b, 8)  # calibration
    rows = int(max(8, min(w.n, 8 * budget_s / max(t, 1e-6))))
    t = w.cpu_rows(lib, a, b, rows)
    ops = 2.0 * rows * w.n * w.n
    return ops / t / 1e12, lib.so_threads(), f"{rows} of {w.n} rows of A against all of B ({ops / 1e9:.1f} GOP, {t:.1f} s)", rows


# ---------------------------------------------------------------------------------------------
def run_reference(args, w) -> None:
    """The reference has no int8 / FP8 operator (ROperator_Gemm is fp32 only), so its arm is the
    CPU restatement of the operator, on every host thread OpenMP gives it; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    lib = load_oracle()
    a, b = w.host_operands(seed=1)
    total = max(1, args.steps + args.warmup)
    t_cal = w.cpu_rows(lib, a, b, 8)
    rows = int(max(1, min(w.n, 8 * (90.0 / total) / max(t_cal, 1e-6))))
    for _ in range(args.warmup):
        w.cpu_rows(lib, a, b, rows)
    t = 0.0
    for _ in range(args.steps):
        t += w.cpu_rows(lib, a, b, rows)
    ops = 2.0 * rows * w.n * w.n * args.steps
    val = ops / t / 1e12
    sample = f"each step = {rows} of {w.n} rows of A against all of B"
    line = {"impl": "reference", "metric": w.metric, "value": val, "unit": w.unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": w.name, "note": "CPU restatement of the operator on host threads; the reference itself has no int8/FP8 path"},
            "cpu_baseline": {"value": val, "unit": w.unit, "cores": lib.so_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_ours(args, w) -> None:
    import torch
    from sofie_b200 import replicas
    from sofie_b200.ops import Context

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    rep = replicas.init_from_env("nccl")
    torch.cuda.set_device(rep.local_rank)
    dev = f"cuda:{rep.local_rank}"
    ctx = Context(rep.local_rank)
    in_dt, out_dt = w.torch_dtypes()

    # operand sets rotated between steps so that each step's inputs come from HBM, not L2
    set_bytes = w.bytes_alg
    nsets = int(max(3, np.ceil(1.6 * L2_BYTES / set_bytes)))
    ha, hb = w.host_operands(seed=1 + rep.rank)
    sets = []
    for s in range(nsets):
        a = torch.from_numpy(np.roll(ha, s, axis=0).copy()).to(dev).view(in_dt)
        b = torch.from_numpy(np.roll(hb, s, axis=1).copy()).to(dev).view(in_dt)
        y = torch.empty((w.n, w.n), dtype=out_dt, device=dev)
        sets.append((a, b, y))
    plan = w.plan(ctx)
    ep, keep = w.epilogue()

    def step(i):
        a, b, y = sets[i % nsets]
        plan.enqueue(a, b, y, ep)

    for i in range(max(3, args.warmup)):
        step(i)
    ctx.sync()
    sampler = ClockSampler(rep.local_rank)
    replicas.barrier(rep)
    torch.cuda.synchronize()
    launches0 = ctx.launches
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ctx.sync()
    launches = ctx.launches - launches0
    ms_local = e0.elapsed_time(e1)
    replicas.barrier(rep)
    ms = replicas.max_over_ranks(rep, ms_local)
    value = rep.world * w.ops * args.steps / (ms * 1e-3) / 1e12

    # end to end through the host-operand entry point of the C ABI
    pa = torch.from_numpy(ha).pin_memory()
    pb = torch.from_numpy(hb).pin_memory()
    py = torch.empty((w.n, w.n), dtype=out_dt).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    py2 = torch.empty((w.n, w.n), dtype=out_dt).pin_memory()
    plan.run_host(pa, pb, py, ep)
    plan.run_host_many([pa] * 2, [pb] * 2, [py, py2], ep)
    replicas.barrier(rep)
    # a queue of e2e_steps inferences through one call: every inference copies its A and B in and its Y out; the copies of
    # neighbouring inferences overlap the contraction (sofie_b200_gemm_run_host_many)
    t0 = time.perf_counter()
    plan.run_host_many([pa] * e2e_steps, [pb] * e2e_steps, [py if i % 2 == 0 else py2 for i in range(e2e_steps)], ep)
    t_e2e = replicas.max_over_ranks(rep, time.perf_counter() - t0)
    e2e_val = rep.world * w.ops * e2e_steps / t_e2e / 1e12
    h2d = pa.numel() * pa.element_size() + pb.numel() * pb.element_size()
    d2h = py.numel() * py.element_size()

    line = None
    if rep.is_root:
        peaks = measured_peaks()
        # dense int8 / FP8 tensor peak = 2 x the bf16 figure measured on this pool (the file has no 8-bit entry)
        peak = 2.0 * peaks["bf16_tflops"]
        ach = w.ops / (ms_local / args.steps * 1e-3) / 1e12
        cpu_val, cores, sample, _ = cpu_sample(w, budget_s=12.0)
        line = {"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": rep.world, "steps": args.steps, "warmup": max(3, args.warmup),
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
                "data": "synthetic",
                "config": {"workload": w.name, "M": w.n, "N": w.n, "K": w.n, "b_layout": "[K,N] row-major (ONNX)",
                           "l2": f"{nsets} operand sets rotated ({nsets * set_bytes / 2**20:.0f} MiB > 126 MiB L2)",
                           "kernel": plan.kernel, "replicas": rep.world},
                "clocks": clocks, "gpu_launches": int(launches),
                "e2e": {"value": e2e_val, "unit": w.unit, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps},
                "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": w.unit, "frac": ach / peak,
                             "traffic": NCU_TRAFFIC_BYTES.get(w.name),
                             "peak_source": f"2 x bf16_tflops of {peaks['source']} MEASURED_PEAKS.json (no 8-bit figure there); nominal dense 4500"},
                "cpu_baseline": {"value": cpu_val, "unit": w.unit, "cores": cores, "kind": "port", "sample": sample}}
    plan.close()
    ctx.close()
    replicas.shutdown(rep)
    if line is not None:
        print(json.dumps(line), flush=True)


class RowOp:
    """LayerNormalization / Softmax over bf16 rows: the HBM-bound operators of the transformer configuration."""

    def __init__(self, kind: str, rows: int, cols: int, name: str):
        self.kind, self.rows, self.cols, self.name = kind, rows, cols, name
        self.metric = f"{kind} bf16 {rows}x{cols} effective bandwidth"
        self.unit, self.dtype = "GB/s", "bf16"
        self.bytes_alg = 2.0 * rows * cols * 2  # read once + write once


def run_rowop(args, w) -> None:
    import torch
    from sofie_b200 import lib as L
    from sofie_b200 import replicas
    from sofie_b200.ops import Context

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        lib = load_oracle()
        rows = min(w.rows, 8192)
        x = (np.random.default_rng(1).standard_normal((rows, w.cols)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        y = np.zeros_like(x)
        g, b = np.ones(w.cols, dtype=np.float32), np.zeros(w.cols, dtype=np.float32)
        def cpu_step():
            t0 = time.perf_counter()
            if w.kind == "layernorm":
                lib.so_layernorm(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), L.BF16, L.BF16, C.c_int64(rows), C.c_int64(w.cols),
                                 g.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), C.c_float(1e-5), None, None)
            else:
                lib.so_softmax(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), L.BF16, L.BF16, C.c_int64(rows), C.c_int64(w.cols), 0)
            return time.perf_counter() - t0
        for _ in range(args.warmup):
            cpu_step()
        t = sum(cpu_step() for _ in range(args.steps))
        val = 2.0 * rows * w.cols * 2 * args.steps / t / 1e9
        print(json.dumps({"impl": "reference", "metric": w.metric, "value": val, "unit": w.unit, "n_gpus": args.gpus, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": 1e3 * t / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": w.dtype, "data": "synthetic", "config": {"workload": w.name},
                          "cpu_baseline": {"value": val, "unit": w.unit, "cores": 1, "kind": "port", "sample": f"each step = {rows} of {w.rows} rows"},
                          "e2e": {"value": val, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return

    rep = replicas.init_from_env("nccl")
    torch.cuda.set_device(rep.local_rank)
    dev = f"cuda:{rep.local_rank}"
    ctx = Context(rep.local_rank)
    nsets = int(max(3, np.ceil(1.6 * L2_BYTES / w.bytes_alg)))
    xs = [torch.randn(w.rows, w.cols, device=dev).to(torch.bfloat16) for _ in range(nsets)]
    ys = [torch.empty_like(x) for x in xs]
    g, b = torch.ones(w.cols, device=dev), torch.zeros(w.cols, device=dev)

    def step(i):
        if w.kind == "layernorm":
            ctx.layernorm(xs[i % nsets], ys[i % nsets], g, b, 1e-5)
        else:
            ctx.softmax(xs[i % nsets], ys[i % nsets])

    for i in range(max(3, args.warmup)):
        step(i)
    ctx.sync()
    sampler = ClockSampler(rep.local_rank)
    replicas.barrier(rep)
    torch.cuda.synchronize()
    l0 = ctx.launches
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_local = e0.elapsed_time(e1)
    ms = replicas.max_over_ranks(rep, ms_local)
    launches = ctx.launches - l0
    value = rep.world * w.bytes_alg * args.steps / (ms * 1e-3) / 1e9
    hx = xs[0].cpu().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        xs[0].copy_(hx, non_blocking=True)
        step(0)
        hy.copy_(ys[0], non_blocking=True)
        ctx.sync()
        torch.cuda.synchronize()
    t_e2e = replicas.max_over_ranks(rep, time.perf_counter() - t0)
    if rep.is_root:
        peaks = measured_peaks()
        ach = w.bytes_alg / (ms_local / args.steps * 1e-3) / 1e9
        print(json.dumps({"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": rep.world, "steps": args.steps, "warmup": max(3, args.warmup),
                          "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
                          "data": "synthetic", "config": {"workload": w.name, "rows": w.rows, "cols": w.cols,
                                                          "l2": f"{nsets} tensor pairs rotated ({nsets * w.bytes_alg / 2**20:.0f} MiB > 126 MiB L2)"},
                          "clocks": clocks, "gpu_launches": int(launches),
                          "e2e": {"value": rep.world * w.bytes_alg * e2e_steps / t_e2e / 1e9, "unit": w.unit,
                                  "h2d_bytes_per_step": int(w.bytes_alg / 2), "d2h_bytes_per_step": int(w.bytes_alg / 2), "steps": e2e_steps},
                          "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                                       "traffic": NCU_TRAFFIC_BYTES.get(w.name), "peak_source": f"hbm_gbs of {peaks['source']} MEASURED_PEAKS.json"}}),
              flush=True)
    ctx.close()
    replicas.shutdown(rep)


WORKLOADS["layernorm_bf16_65536x512"] = lambda: RowOp("layernorm", 65536, 512, "layernorm_bf16_65536x512")
WORKLOADS["softmax_bf16_524288x128"] = lambda: RowOp("softmax", 524288, 128, "softmax_bf16_524288x128")


class EncoderWorkload:
    """Transformer encoder: 6 pre-LN layers, d_model 512, 8 heads, FFN 2048, Gelu, seq 128; bf16 activations, int8
    per-channel weights dequantised in the contraction epilogue.  One step = one batch through all layers."""

    def __init__(self, name: str, batch: int):
        self.name, self.batch = name, batch
        self.layers, self.seq, self.d_model, self.heads, self.ffn = 6, 128, 512, 8, 2048
        self.metric = "transformer encoder inferences/s (sequences of 128 tokens)"
        self.unit, self.dtype = "inferences/s", "bf16"


def pipelined_e2e(torch, compute, step, x_bufs, hx, hy, steps: int) -> float:
    """A queue of `steps` inferences from pinned host memory, end to end.  Inference i's input is copied in on a copy
    stream (two device input buffers), its output is copied to a second device buffer and from there to the host on
    another copy stream, so the copies of inferences i+1 and i-1 overlap the kernels of inference i (`compute` is the
    stream `step` enqueues on).  Returns the wall-clock seconds until the last output is in host memory."""
    cin, cout = torch.cuda.Stream(), torch.cuda.Stream()
    ev = lambda: [torch.cuda.Event(), torch.cuda.Event()]
    ready, consumed, kept, left = ev(), ev(), ev(), ev()
    keep = [None, None]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(steps):
        s = i & 1
        with torch.cuda.stream(cin):
            if i >= 2:
                cin.wait_event(consumed[s])
            x_bufs[s].copy_(hx, non_blocking=True)
            ready[s].record(cin)
        with torch.cuda.stream(compute):
            compute.wait_event(ready[s])
            y = step(x_bufs[s])
            consumed[s].record(compute)
            if keep[s] is None:
                keep[s] = torch.empty_like(y)
            if i >= 2:
                compute.wait_event(left[s])
            keep[s].copy_(y)   # the next inference may overwrite the network's output buffer
            kept[s].record(compute)
        with torch.cuda.stream(cout):
            cout.wait_event(kept[s])
            hy.copy_(keep[s], non_blocking=True)
            left[s].record(cout)
    torch.cuda.synchronize()
    return time.perf_counter() - t0


def run_encoder(args, w) -> None:
    import torch
    import bench_encoder as be
    from sofie_b200 import lib as L

    flops = be.flops_per_sample(w.layers, w.seq, w.d_model, w.ffn)
    rng = np.random.default_rng(7)
    weights = be.make_weights(rng, w.layers, w.d_model, w.ffn)
    config = {"workload": w.name, "layers": w.layers, "d_model": w.d_model, "heads": w.heads, "ffn": w.ffn, "seq_len": w.seq,
              "batch_per_gpu": w.batch, "weights": "int8 per output channel, scale fused in the contraction epilogue",
              "gflop_per_inference": flops / 1e9}

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        sys.path.insert(0, str(ROOT / "tests"))
        from oracle_api import Oracle
        load_oracle()   # builds the checker library if needed
        o = Oracle(ROOT / "oracle" / "libsofie_oracle.so")
        o.lib.so_threads.restype = C.c_int
        o.lib.so_set_threads(os.cpu_count() or 1)
        nb = 2   # sequences per CPU step: a bounded sample of the batch
        x = be.f32_to_bf16_bits(rng.standard_normal((nb * w.seq, w.d_model)).astype(np.float32))
        def cpu_step():
            t0 = time.perf_counter()
            be.encoder_oracle(o, x, weights, nb, w.seq, w.d_model, w.heads)
            return time.perf_counter() - t0
        for _ in range(min(args.warmup, 1)):
            cpu_step()
        steps = max(1, min(args.steps, 5))
        t = sum(cpu_step() for _ in range(steps))
        val = nb * steps / t
        cores = int(o.lib.so_threads())
        print(json.dumps({"impl": "reference", "metric": w.metric, "value": val, "unit": w.unit, "n_gpus": args.gpus, "steps": steps,
                          "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * t / steps, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f64 accumulate, bf16 tensors", "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": val, "unit": w.unit, "cores": cores, "kind": "port",
                                           "sample": f"each step = {nb} of {w.batch} sequences through all {w.layers} layers"},
                          "e2e": {"value": val, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return

    from sofie_b200 import replicas
    from sofie_b200.ops import Context
    rep = replicas.init_from_env("nccl")
    torch.cuda.set_device(rep.local_rank)
    dev = f"cuda:{rep.local_rank}"
    # --cuda-graph: the step is captured once per input buffer on a side stream (an enqueue is nothing but kernel
    # launches on the context's stream) and the timed loop replays the graphs
    side = torch.cuda.Stream(device=dev) if args.cuda_graph else torch.cuda.current_stream(dev)
    ctx = Context(rep.local_rank, stream=side)
    enc = be.EncoderB200(ctx, weights, w.batch, w.seq, w.d_model, w.heads, w.ffn, dev)
    m = w.batch * w.seq
    xs = [torch.randn(m, w.d_model, device=dev).to(torch.bfloat16) for _ in range(3)]   # activations per step: ~1.5 GB > L2
    torch.cuda.synchronize()
    for i in range(max(3, args.warmup)):
        enc(xs[i % 3])
    ctx.sync()
    step = lambda i: enc(xs[i % 3])
    per_step = 0
    if args.cuda_graph:
        config["cuda_graph"] = True
        graphs = []
        for x in xs:
            g, c0 = torch.cuda.CUDAGraph(), ctx.launches
            with torch.cuda.graph(g, stream=side):
                enc(x)
            per_step = ctx.launches - c0
            graphs.append(g)
        step = lambda i: graphs[i % 3].replay()
    sampler = ClockSampler(rep.local_rank)
    replicas.barrier(rep)
    torch.cuda.synchronize()
    l0 = ctx.launches
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(side):
        if args.cuda_graph:
            for i in range(3):
                step(i)
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
    torch.cuda.synchronize()
    ctx.sync()
    clocks = sampler.stop()
    ms_local = e0.elapsed_time(e1)
    ms = replicas.max_over_ranks(rep, ms_local)
    launches = per_step * args.steps if args.cuda_graph else ctx.launches - l0
    value = rep.world * w.batch * args.steps / (ms * 1e-3)
    # end to end: tokens from pinned host memory in, final activations back out, every step
    hx = xs[0].cpu().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    pipelined_e2e(torch, side, enc, xs[:2], hx, hy, 2)
    t_e2e = replicas.max_over_ranks(rep, pipelined_e2e(torch, side, enc, xs[:2], hx, hy, e2e_steps))
    if rep.is_root:
        peaks = measured_peaks()
        ach = flops * w.batch / (ms_local / args.steps * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]
        print(json.dumps({"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": rep.world, "steps": args.steps, "warmup": max(3, args.warmup),
                          "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
                          "data": "synthetic", "config": dict(config, l2="three input batches rotated; one step streams ~1.5 GB of activations (> 126 MiB L2)"),
                          "clocks": clocks, "gpu_launches": int(launches),
                          "e2e": {"value": rep.world * w.batch * e2e_steps / t_e2e, "unit": w.unit, "h2d_bytes_per_step": int(hx.numel() * 2),
                                  "d2h_bytes_per_step": int(hy.numel() * 2), "steps": e2e_steps},
                          "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                                       "peak_source": f"bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS.json; whole step (all "
                                                      f"{launches // max(1, args.steps)} launches), not one kernel"}}), flush=True)
    enc.close()
    ctx.close()
    replicas.shutdown(rep)


WORKLOADS["transformer_encoder_b512"] = lambda: EncoderWorkload("transformer_encoder_b512", 512)
WORKLOADS["transformer_encoder_b64"] = lambda: EncoderWorkload("transformer_encoder_b64", 64)


class ConvNetWorkload:
    """Conv net: 8 Conv3x3 (+ folded BatchNormalization + Relu) layers, global average pool, Gemm 512 -> 1000, on NCHW
    3 x img x img inputs; fp32 or per-channel int8 (QLinearConv)."""

    def __init__(self, name: str, batch: int, img: int, int8: bool):
        self.name, self.batch, self.img, self.int8 = name, batch, img, int8
        self.metric = f"conv net inferences/s ({img}x{img} images, {'int8 QLinearConv' if int8 else 'fp32'})"
        self.unit, self.dtype = "inferences/s", ("int8" if int8 else "fp32 (3xTF32 on tcgen05 where large, fp32 FMA else)")


def run_convnet(args, w) -> None:
    import torch
    import bench_convnet as bc

    flops = bc.flops_per_image(w.img)
    rng = np.random.default_rng(11)
    weights = bc.make_weights(rng, w.int8)
    config = {"workload": w.name, "batch_per_gpu": w.batch, "image": [3, w.img, w.img], "layers": "8 x Conv3x3+BN+Relu, avgpool, Gemm 512->1000",
              "strides": bc.STRIDES, "gflop_per_inference": flops / 1e9}

    def host_input(n):
        x = rng.random((n, 3, w.img, w.img), dtype=np.float32)
        return np.clip(np.rint(x * 127.0), 0, 127).astype(np.int8) if w.int8 else x

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        sys.path.insert(0, str(ROOT / "tests"))
        from oracle_api import Oracle
        load_oracle()
        o = Oracle(ROOT / "oracle" / "libsofie_oracle.so")
        o.lib.so_threads.restype = C.c_int
        o.lib.so_set_threads(os.cpu_count() or 1)
        x = host_input(1)
        def cpu_step():
            t0 = time.perf_counter()
            bc.convnet_oracle(o, x, weights, w.int8)
            return time.perf_counter() - t0
        steps = max(1, min(args.steps, 3))
        if args.warmup:
            cpu_step()
        t = sum(cpu_step() for _ in range(steps))
        val = steps / t
        print(json.dumps({"impl": "reference", "metric": w.metric, "value": val, "unit": w.unit, "n_gpus": args.gpus, "steps": steps,
                          "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * t / steps, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "int32 accumulate" if w.int8 else "f64 accumulate", "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": val, "unit": w.unit, "cores": int(o.lib.so_threads()), "kind": "port",
                                           "sample": f"each step = 1 of {w.batch} images through the whole network"},
                          "e2e": {"value": val, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return

    from sofie_b200 import replicas
    from sofie_b200.ops import Context
    rep = replicas.init_from_env("nccl")
    torch.cuda.set_device(rep.local_rank)
    dev = f"cuda:{rep.local_rank}"
    ctx = Context(rep.local_rank)
    net = bc.ConvNetB200(ctx, weights, w.batch, w.img, w.int8, dev)
    hx = torch.from_numpy(host_input(w.batch)).pin_memory()
    x = hx.to(dev)
    for _ in range(max(3, args.warmup)):
        net(x)
    ctx.sync()
    sampler = ClockSampler(rep.local_rank)
    replicas.barrier(rep)
    torch.cuda.synchronize()
    l0 = ctx.launches
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        net(x)
    e1.record()
    torch.cuda.synchronize()
    ctx.sync()
    clocks = sampler.stop()
    ms_local = e0.elapsed_time(e1)
    ms = replicas.max_over_ranks(rep, ms_local)
    launches = ctx.launches - l0
    value = rep.world * w.batch * args.steps / (ms * 1e-3)
    hy = torch.empty((w.batch, bc.CLASSES), dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    x_bufs = [x, torch.empty_like(x)]
    pipelined_e2e(torch, torch.cuda.current_stream(dev), net, x_bufs, hx, hy, 2)
    t_e2e = replicas.max_over_ranks(rep, pipelined_e2e(torch, torch.cuda.current_stream(dev), net, x_bufs, hx, hy, e2e_steps))
    if rep.is_root:
        peaks = measured_peaks()
        ach = flops * w.batch / (ms_local / args.steps * 1e-3) / 1e12
        base = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]
        peak = 2.0 * base if w.int8 else base / 6.0
        how = "2 x bf16_tflops_sustained (int8 dense)" if w.int8 else "bf16_tflops_sustained / 6 (TF32 is half the bf16 rate, 3xTF32 does three passes)"
        print(json.dumps({"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": rep.world, "steps": args.steps, "warmup": max(3, args.warmup),
                          "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
                          "data": "synthetic", "config": dict(config, contraction_kernels=net.kernels,
                                                              l2="activations of one step are several GB (> 126 MiB L2)"),
                          "clocks": clocks, "gpu_launches": int(launches),
                          "e2e": {"value": rep.world * w.batch * e2e_steps / t_e2e, "unit": w.unit, "h2d_bytes_per_step": int(hx.numel() * hx.element_size()),
                                  "d2h_bytes_per_step": int(hy.numel() * 4), "steps": e2e_steps},
                          "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s" if not w.int8 else "TOP/s", "frac": ach / peak,
                                       "traffic": None, "peak_source": f"{how} of {peaks['source']} MEASURED_PEAKS.json; whole step "
                                                                       f"({launches // max(1, args.steps)} launches), not one kernel"}}), flush=True)
    net.close()
    ctx.close()
    replicas.shutdown(rep)


WORKLOADS["convnet_fp32_b256"] = lambda: ConvNetWorkload("convnet_fp32_b256", 256, 224, False)
WORKLOADS["convnet_int8_b256"] = lambda: ConvNetWorkload("convnet_int8_b256", 256, 224, True)
WORKLOADS["convnet_fp32_b32"] = lambda: ConvNetWorkload("convnet_fp32_b32", 32, 224, False)
WORKLOADS["convnet_int8_b32"] = lambda: ConvNetWorkload("convnet_int8_b32", 32, 224, True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qlinear_matmul_4096", choices=sorted(WORKLOADS))
    ap.add_argument("--cuda-graph", action="store_true", help="transformer_encoder_* only: replay the step from a CUDA graph")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]()
    if isinstance(w, RowOp):
        run_rowop(args, w)
    elif isinstance(w, EncoderWorkload):
        run_encoder(args, w)
    elif isinstance(w, ConvNetWorkload):
        run_convnet(args, w)
    elif args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
