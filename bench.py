#!/usr/bin/env python
"""Benchmark of the SOFIE inference hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-also]

Prints ONE JSON line (rank 0).  A "pass" is one run of the hot path over one batch of synthetic input (one
contraction, or one batch through a whole network); a "step" is `launches_per_step` passes back to back, chosen so
that the K timed steps last about `--seconds` (2.5 s): long enough for the GPU to reach the clocks it sustains under
its power limit and for the clock sampler to see it.  ms_per_step x steps is the timed region.

The headline workload is the int8 QLinearMatMul M = N = K = 4096 (per-tensor scales 0.02 / 0.01, output scale 0.5, zero
points 0): A [M,K] int8 uniform in [-127,127], the weight B [K,N] an initializer (kept K-major by the plan), int32
accumulation, ONNX requantisation to int8 fused in the kernel's epilogue.  Without --workload the same line carries an
"also" array with one record per other configuration: FP8 GEMM 8192^3 + bias + Gelu, the conv net (int8 and fp32,
batch 256), the transformer encoder (512 sequences over all GPUs), LayerNorm and Softmax.

  value         whole-job throughput with inputs resident in HBM (CUDA events on the launching stream, max over ranks)
  e2e           the same metric from HOST buffers: weights on the device once (Session construction), every inference's
                input copied from pinned memory and its output copied back inside the timed region, copies of
                neighbouring inferences overlapping the kernels
  roofline      achieved / peak of the dominant kernel (contractions: dense tensor peak; row operators: HBM), against
                the burst and the sustained figure measured on this pool
  cpu_baseline  rank 0, one GPU only: the reference's own emitted CPU code (oracle/_ref, linked to the BLAS found in
                the process) where the reference has the operators, the CPU restatement (oracle/) otherwise, on a
                bounded sample

With --impl reference the CPU implementation is the thing timed (rank 0 only).  Multi-GPU runs are launched with
torchrun; every rank runs its own replica on its own GPU and nothing crosses NVLink on the data path.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures summarised
# under profiles/ (None where no capture of that workload exists).
NCU_TRAFFIC_BYTES = {
    "qlinear_matmul_4096": 33.65e6 + 0.13e6,  # profiles/umma_gemm_i8_qlinear_matmul_4096.md
    "fp8_gemm_8192": 339.3e6 + 111.1e6,       # profiles/umma_gemm_f8_gemm_8192.md
}


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained") or d["bf16_tflops"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while the timed region runs (NVML, read-only)."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.power, self.reasons = [], [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        self._nv = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            idx = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                ent = vis.split(",")[self.index]
                idx = int(ent) if ent.isdigit() else self.index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(idx)
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
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
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
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------------------------
# CPU side: the checker library, the reference's emitted code, the BLAS of the process
def load_oracle():
    """The CPU restatement (oracle/libsofie_oracle.so); only the CPU-baseline legs use it."""
    so = ROOT / "oracle" / "libsofie_oracle.so"
    if not so.exists():
        import subprocess
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    lib = C.CDLL(str(so))
    lib.so_threads.restype = C.c_int
    lib.so_set_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1; the CPU arm gets every host core
    return lib


def find_blas():
    """sgemm_ of a BLAS this process can load: MKL inside libtorch_cpu.so, else none (the reference models then run on
    the plain loops of oracle/ref_sgemm.c).  Returns (address or None, description)."""
    try:
        import torch
        torch.set_num_threads(os.cpu_count() or 1)   # also sets the MKL thread count (torchrun exports OMP_NUM_THREADS=1)
        lib = C.CDLL(str(Path(torch.__file__).parent / "lib" / "libtorch_cpu.so"))
        return C.cast(lib.sgemm_, C.c_void_p).value, f"MKL sgemm_ of libtorch_cpu.so, {torch.get_num_threads()} threads"
    except Exception:
        return None, "plain loops (oracle/ref_sgemm.c)"


class RefModel:
    """A Session of the reference's own emitted CPU code (oracle/_ref/models/lib<name>.so, built by `make -C oracle ref`)."""

    def __init__(self, name: str):
        so = ROOT / "oracle" / "_ref" / "models" / f"lib{name}.so"
        if not so.exists():
            raise FileNotFoundError(so)
        self.lib = C.CDLL(str(so))
        self.lib.ref_open.restype = C.c_void_p
        self.lib.ref_open.argtypes = [C.c_char_p]
        self.lib.ref_infer.restype = C.c_long
        self.lib.ref_infer.argtypes = [C.c_void_p, C.POINTER(C.POINTER(C.c_float)), C.POINTER(C.c_float), C.c_long]
        self.lib.ref_close.argtypes = [C.c_void_p]
        self.lib.ref_last_error.restype = C.c_char_p
        addr, self.blas = find_blas()
        if addr:
            self.lib.ref_blas_use(C.c_void_p(addr))
        self.h = self.lib.ref_open(str(ROOT / "oracle" / "_ref" / "gen").encode())
        if not self.h:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def infer(self, inputs, out=None) -> float:
        """Seconds of one Session::infer (the reference's std::vector result is dropped unless `out` is given)."""
        ins = [np.ascontiguousarray(x, dtype=np.float32) for x in inputs]
        ptrs = (C.POINTER(C.c_float) * len(ins))(*[x.ctypes.data_as(C.POINTER(C.c_float)) for x in ins])
        t0 = time.perf_counter()
        n = self.lib.ref_infer(self.h, ptrs, out.ctypes.data_as(C.POINTER(C.c_float)) if out is not None else None, out.size if out is not None else 0)
        dt = time.perf_counter() - t0
        if n < 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return dt

    def close(self):
        if self.h:
            self.lib.ref_close(self.h)
            self.h = None


def timed_cpu(fn, budget_s: float, max_steps: int = 50):
    """Runs fn() (returns seconds) once untimed, then until the budget is spent; returns (mean seconds, steps)."""
    first = fn()
    if first > budget_s:
        return first, 1
    tot, n = 0.0, 0
    while n < max_steps and tot < budget_s:
        tot += fn()
        n += 1
    return tot / n, n


# ---------------------------------------------------------------------------------------------
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


def e2e_measure(torch, rep, compute, step, x_bufs, hx, hy, units_per_inference: float, target_s: float = 1.0) -> dict:
    from sofie_b200 import replicas
    pipelined_e2e(torch, compute, step, x_bufs, hx, hy, 3)
    t_probe = pipelined_e2e(torch, compute, step, x_bufs, hx, hy, 6) / 6
    n = int(max(6, min(4000, target_s / max(t_probe, 1e-6))))
    n = int(replicas.max_over_ranks(rep, float(n)))
    replicas.barrier(rep)
    t = replicas.max_over_ranks(rep, pipelined_e2e(torch, compute, step, x_bufs, hx, hy, n))
    return {"value": rep.world * units_per_inference * n / t, "h2d_bytes_per_step": int(hx.numel() * hx.element_size()),
            "d2h_bytes_per_step": int(hy.numel() * hy.element_size()), "inferences": n, "seconds": t}


def session_e2e(torch, rep, sess, host_inputs, out_shape, out_dtype, units_per_inference: float, target_s: float = 1.0) -> dict:
    """A queue of inferences through Session::infer_host_many of the emitted code: every inference's inputs come from pinned
    host memory and its output goes back to pinned host memory (two output buffers in turn); weights were uploaded once, at
    Session construction.  Returns the e2e record (value still in plain units per second)."""
    from sofie_b200 import replicas
    outs = [torch.empty(out_shape, dtype=out_dtype).pin_memory() for _ in range(2)]

    def run(count):
        t0 = time.perf_counter()
        sess.infer_host_many([[t.data_ptr()] * count for t in host_inputs], [outs[k & 1].data_ptr() for k in range(count)])
        return time.perf_counter() - t0
    run(3)
    t_probe = run(6) / 6
    n = int(replicas.max_over_ranks(rep, float(max(6, min(4000, target_s / max(t_probe, 1e-6))))))
    replicas.barrier(rep)
    t = replicas.max_over_ranks(rep, run(n))
    return {"value": rep.world * units_per_inference * n / t, "h2d_bytes_per_step": int(sum(x.numel() * x.element_size() for x in host_inputs)),
            "d2h_bytes_per_step": int(outs[0].numel() * outs[0].element_size()), "inferences": n, "seconds": t,
            "api": "Session::infer_host_many of the emitted code (ONNX model -> sofie_b200_emit -> g++); weights uploaded once at Session construction"}


# ---------------------------------------------------------------------------------------------
class Workload:
    name = metric = unit = dtype = ""
    scaling = "weak"
    unit_scale = 1.0        # value = units / seconds / unit_scale

    def stream(self, torch, dev):
        """The CUDA stream the passes are enqueued on (the timing events are recorded there)."""
        return torch.cuda.current_stream(dev)

    def sync(self):
        self.ctx.sync()

    def launches(self) -> int:
        """Kernels enqueued so far."""
        return self.ctx.launches

    def setup(self, torch, ctx, dev, rep): ...
    def one_pass(self, i): ...
    def units_per_pass(self) -> float: ...
    def config(self) -> dict: return {"workload": self.name}
    def roofline(self, s_per_pass: float, peaks: dict, sustained: bool, launches_per_pass: float) -> dict: ...
    def e2e(self, torch, rep, compute) -> dict: ...
    def cpu_baseline(self, budget_s: float) -> dict: ...
    def reference_step(self): ...   # -> (fn returning seconds, units per step, description dict)
    def close(self): ...


def tensor_roofline(ach, peaks, sustained, factor, unit, what, traffic=None, extra=""):
    burst, sust = factor * peaks["bf16_tflops"], factor * peaks["bf16_tflops_sustained"]
    peak = sust if sustained else burst
    return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak, "traffic": traffic,
            "frac_of_burst": ach / burst, "frac_of_sustained": ach / sust, "peak_burst": burst, "peak_sustained": sust,
            "peak_source": f"{what} of {peaks['source']} MEASURED_PEAKS.json ({'sustained: the timed region is seconds long' if sustained else 'burst: short region'}){extra}"}


class GemmWorkload(Workload):
    """One square contraction with a constant weight B: int8 QLinearMatMul or FP8 e4m3 GEMM + scales + bias + Gelu -> bf16."""

    def __init__(self, name: str, n: int, kind: str):
        self.name, self.n, self.kind = name, n, kind
        self.ops = 2.0 * n * n * n
        self.unit_scale = 1e12
        if kind == "int8":
            self.metric, self.unit, self.dtype = f"int8 QLinearMatMul {n}^3 throughput", "TOPS", "int8"
            self.a_scale, self.b_scale, self.y_scale = np.float32(0.02), np.float32(0.01), np.float32(0.5)
            self.mult = float(np.float32(self.a_scale * self.b_scale) / self.y_scale)  # fp32 on the host, once
            self.bytes_alg = 3.0 * n * n
        else:
            self.metric, self.unit, self.dtype = f"FP8 e4m3 GEMM {n}^3 + scales + bias + Gelu -> bf16 throughput", "TFLOP/s", "fp8_e4m3"
            self.bytes_alg = 2.0 * n * n + 2.0 * n * n

    # ---- synthetic operands
    def host_operands(self, seed: int):
        n = self.n
        if self.kind == "int8":
            rng = np.random.default_rng(seed)
            return rng.integers(-127, 128, size=(n, n), dtype=np.int8), rng.integers(-127, 128, size=(n, n), dtype=np.int8)
        import torch
        g = torch.Generator().manual_seed(seed)
        a, b = torch.randn(n, n, generator=g), torch.randn(n, n, generator=g)
        self.sa = (a.abs().amax(dim=1) / 448.0).contiguous()
        self.sb = (b.abs().amax(dim=0) / 448.0).contiguous()
        self.bias = (torch.randn(n, generator=g) * 0.1).contiguous()
        a8 = (a / self.sa[:, None]).to(torch.float8_e4m3fn)
        b8 = (b / self.sb[None, :]).to(torch.float8_e4m3fn)
        return a8.view(torch.uint8).numpy(), b8.view(torch.uint8).numpy()

    def setup(self, torch, ctx, dev, rep):
        from sofie_b200 import lib as L
        from sofie_b200.ops import GemmPlan, make_epilogue
        self.torch, self.ctx = torch, ctx
        n = self.n
        in_dt = torch.int8 if self.kind == "int8" else torch.float8_e4m3fn
        out_dt = torch.int8 if self.kind == "int8" else torch.bfloat16
        self.out_dt = out_dt
        self.ha, self.hb = self.host_operands(seed=1 + rep.rank)
        # operand sets rotated between passes so that every pass reads its operands from HBM, not L2; each set has a plan
        # of its own because a plan keeps the K-major copy of ITS weight
        self.nsets = int(max(3, math.ceil(1.6 * L2_BYTES / self.bytes_alg)))
        self.sets = []
        for s in range(self.nsets):
            a = torch.from_numpy(np.roll(self.ha, s, axis=0).copy()).to(dev).view(in_dt)
            b = torch.from_numpy(np.roll(self.hb, s, axis=1).copy()).to(dev).view(in_dt)
            y = torch.empty((n, n), dtype=out_dt, device=dev)
            plan = GemmPlan(ctx, n, n, n, in_dt, out_dt, trans_b=False, flags=L.GEMM_B_CONSTANT)
            self.sets.append((a, b, y, plan))
        if self.kind == "int8":
            self.ep, self._keep = make_epilogue(alpha=self.mult)
        else:
            self._dev = (self.sa.to(dev), self.sb.to(dev), self.bias.to(dev))
            self.ep, self._keep = make_epilogue(row_scale=self._dev[0], col_scale=self._dev[1], bias=self._dev[2], act=L.ACT_GELU_ERF)
        self.kernel = self.sets[0][3].kernel

    def one_pass(self, i):
        a, b, y, plan = self.sets[i % self.nsets]
        plan.enqueue(a, b, y, self.ep)

    def units_per_pass(self):
        return self.ops

    def config(self):
        n = self.n
        return {"workload": self.name, "M": n, "N": n, "K": n,
                "b_layout": "[K,N] row-major as ONNX stores it; a constant weight (initializer): the plan keeps a K-major copy made on first use",
                "l2": f"{self.nsets} operand sets rotated ({self.nsets * self.bytes_alg / 2**20:.0f} MiB > 126 MiB L2)", "kernel": self.kernel}

    def roofline(self, s_per_pass, peaks, sustained, launches_per_pass):
        ach = self.ops / s_per_pass / 1e12
        return tensor_roofline(ach, peaks, sustained, 2.0, self.unit, "2 x bf16_tflops" + ("_sustained" if sustained else ""),
                               NCU_TRAFFIC_BYTES.get(self.name), "; the file has no 8-bit figure; nominal dense 4500")

    def session(self):
        """The workload as a model file handed to the C++ generator: parsed, emitted, compiled and constructed the way a user
        of the generated code does it.  The weight B (and the per-column scales and bias) are initializers."""
        import tempfile
        from sofie_b200.session import EmittedSession
        n = self.n
        if self.kind == "int8":
            w = {"B": self.hb, "a_scale": np.array(self.a_scale), "a_zp": np.array(0, dtype=np.int8), "b_scale": np.array(self.b_scale),
                 "b_zp": np.array(0, dtype=np.int8), "y_scale": np.array(self.y_scale), "y_zp": np.array(0, dtype=np.int8)}
            nodes = [{"op": "QLinearMatMul", "in": ["A", "a_scale", "a_zp", "B", "b_scale", "b_zp", "y_scale", "y_zp"], "out": ["Y"], "attrs": {}}]
            return EmittedSession(self.name, nodes, w, [("A", [n, n])], ["Y"], tempfile.mkdtemp(prefix="sofie_b200_"), input_types={"A": 3})
        w = {"B": self.hb, "col_scale": self.sb.numpy(), "bias": self.bias.numpy()}
        nodes = [{"op": "ScaledGemm", "in": ["A", "B", "row_scale", "col_scale", "bias"], "out": ["P"], "attrs": {}},
                 {"op": "Gelu", "in": ["P"], "out": ["Y"], "attrs": {}}]
        return EmittedSession(self.name, nodes, w, [("A", [n, n]), ("row_scale", [n])], ["Y"], tempfile.mkdtemp(prefix="sofie_b200_"),
                              input_types={"A": 17, "row_scale": 1}, initializer_types={"B": 17})

    def e2e(self, torch, rep, compute):
        """Through the emitted Session's infer_host_many: A (and its row scales) from pinned host memory in, Y back out, per
        inference; the weights were uploaded once, when the Session was constructed."""
        sess = self.session()
        ins = [torch.from_numpy(self.ha).pin_memory()]
        if self.kind != "int8":
            ins.append(self.sa.pin_memory())
        r = session_e2e(torch, rep, sess, ins, (self.n, self.n), self.out_dt, self.ops)
        r["value"] /= 1e12
        r["unit"] = self.unit
        sess.close()
        return r

    # ---- CPU
    def _port_rows(self, lib, a, b, rows: int) -> float:
        from sofie_b200 import lib as L
        d = L.GemmDesc()
        d.M, d.N, d.K, d.batch = rows, self.n, self.n, 1
        e = L.Epilogue()
        e.alpha, e.beta, e.out_scale = 1.0, 1.0, 1.0
        if self.kind == "int8":
            d.ab_dtype, d.y_dtype = L.I8, L.I8
            e.alpha = self.mult
            y = np.zeros((rows, self.n), dtype=np.int8)
            keep = None
        else:
            d.ab_dtype, d.y_dtype = L.F8E4M3, L.BF16
            keep = (self.sa.numpy(), self.sb.numpy(), self.bias.numpy())
            e.row_scale, e.col_scale = keep[0].ctypes.data_as(C.c_void_p), keep[1].ctypes.data_as(C.c_void_p)
            e.bias_mode, e.bias, e.act = L.BIAS_COL_F32, keep[2].ctypes.data_as(C.c_void_p), L.ACT_GELU_ERF
            y = np.zeros((rows, self.n), dtype=np.uint16)
        t0 = time.perf_counter()
        lib.so_gemm(C.byref(d), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), C.byref(e))
        return time.perf_counter() - t0

    def _dequantised(self):
        a, b = self.host_operands(seed=1)
        if self.kind == "int8":
            return [a.astype(np.float32) * self.a_scale, b.astype(np.float32) * self.b_scale]
        import torch
        af = torch.from_numpy(a).view(torch.float8_e4m3fn).float() * self.sa[:, None]
        bf = torch.from_numpy(b).view(torch.float8_e4m3fn).float() * self.sb[None, :]
        return [af.numpy(), bf.numpy(), self.bias.numpy()]

    def cpu_baseline(self, budget_s):
        lib = load_oracle()
        a, b = self.host_operands(seed=1)
        t = self._port_rows(lib, a, b, 8)
        rows = int(max(8, min(self.n, 8 * 0.5 * budget_s / max(t, 1e-6))))
        t = self._port_rows(lib, a, b, rows)
        out = {"value": 2.0 * rows * self.n * self.n / t / 1e12, "unit": self.unit, "cores": lib.so_threads(), "kind": "port",
               "sample": f"CPU restatement of the operator on {rows} of {self.n} rows of A against all of B ({t:.1f} s)"}
        try:   # what the reference itself can run: its emitted fp32 Gemm on the dequantised operands, on the process's BLAS
            ref_name = "MatMul_C2" if self.kind == "int8" else "Gemm_C3"
            if (self.kind, self.n) in (("int8", 4096), ("fp8", 8192)):
                m = RefModel(ref_name)
                ins = self._dequantised()
                sec, n = timed_cpu(lambda: m.infer(ins), 0.5 * budget_s, 5)
                m.close()
                out["fp32_blas_standin"] = {"value": self.ops / sec / 1e12, "unit": "TFLOP/s", "kind": "reference", "cores": os.cpu_count(),
                                            "sample": f"SOFIE-emitted fp32 Gemm (oracle/_ref {ref_name}) on the dequantised operands, full size, {n} runs; {m.blas}"}
        except Exception as e:   # the reference build is not on this machine: the port stands alone
            out["fp32_blas_standin"] = {"unavailable": str(e)[:200]}
        return out

    def reference_step(self):
        ref_name = "MatMul_C2" if self.kind == "int8" else "Gemm_C3"
        try:
            if (self.kind, self.n) not in (("int8", 4096), ("fp8", 8192)):
                raise FileNotFoundError("no reference model of this size")
            m = RefModel(ref_name)
            ins = self._dequantised()
            return (lambda: m.infer(ins)), self.ops, {"kind": "reference", "cores": os.cpu_count(),
                                                        "sample": f"each step = the SOFIE-emitted fp32 Gemm (oracle/_ref {ref_name}) on the dequantised operands at full size "
                                                                  f"(the reference has no int8 / FP8 operator); {m.blas}"}
        except Exception:
            lib = load_oracle()
            a, b = self.host_operands(seed=1)
            t = self._port_rows(lib, a, b, 8)
            rows = int(max(1, min(self.n, 8 * 3.0 / max(t, 1e-6))))
            return (lambda: self._port_rows(lib, a, b, rows)), 2.0 * rows * self.n * self.n, {
                "kind": "port", "cores": lib.so_threads(), "sample": f"each step = the CPU restatement on {rows} of {self.n} rows of A against all of B"}

    def close(self):
        for s in self.sets:
            s[3].close()
        self.sets = []


class RowOpWorkload(Workload):
    """LayerNormalization / Softmax over bf16 rows: the HBM-bound operators of the transformer configuration."""

    def __init__(self, kind: str, rows: int, cols: int, name: str):
        self.kind, self.rows, self.cols, self.name = kind, rows, cols, name
        self.metric = f"{kind} bf16 {rows}x{cols} effective bandwidth"
        self.unit, self.dtype = "GB/s", "bf16"
        self.unit_scale = 1e9
        self.bytes_alg = 2.0 * rows * cols * 2  # read once + write once

    def setup(self, torch, ctx, dev, rep):
        self.torch, self.ctx = torch, ctx
        self.nsets = int(max(3, math.ceil(1.6 * L2_BYTES / self.bytes_alg)))
        self.xs = [torch.randn(self.rows, self.cols, device=dev).to(torch.bfloat16) for _ in range(self.nsets)]
        self.ys = [torch.empty_like(x) for x in self.xs]
        self.g, self.b = torch.ones(self.cols, device=dev), torch.zeros(self.cols, device=dev)

    def one_pass(self, i):
        s = i % self.nsets
        if self.kind == "layernorm":
            self.ctx.layernorm(self.xs[s], self.ys[s], self.g, self.b, 1e-5)
        else:
            self.ctx.softmax(self.xs[s], self.ys[s])

    def units_per_pass(self):
        return self.bytes_alg

    def config(self):
        return {"workload": self.name, "rows": self.rows, "cols": self.cols,
                "l2": f"{self.nsets} tensor pairs rotated ({self.nsets * self.bytes_alg / 2**20:.0f} MiB > 126 MiB L2)"}

    def roofline(self, s_per_pass, peaks, sustained, launches_per_pass):
        ach = self.bytes_alg / s_per_pass / 1e9
        return {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "traffic": NCU_TRAFFIC_BYTES.get(self.name), "peak_source": f"hbm_gbs of {peaks['source']} MEASURED_PEAKS.json (copy, read + write); nominal 8000"}

    def e2e(self, torch, rep, compute):
        hx = self.xs[0].cpu().pin_memory()
        hy = torch.empty_like(hx).pin_memory()

        def step(x):
            if self.kind == "layernorm":
                self.ctx.layernorm(x, self.ys[0], self.g, self.b, 1e-5)
            else:
                self.ctx.softmax(x, self.ys[0])
            return self.ys[0]
        r = e2e_measure(torch, rep, compute, step, [self.xs[0], self.xs[1]], hx, hy, self.bytes_alg, 0.5)
        r["value"] /= 1e9
        r["unit"] = self.unit
        return r

    def _cpu_fn(self):
        from sofie_b200 import lib as L
        lib = load_oracle()
        rows = min(self.rows, 8192)
        x = (np.random.default_rng(1).standard_normal((rows, self.cols)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        y = np.zeros_like(x)
        g, b = np.ones(self.cols, dtype=np.float32), np.zeros(self.cols, dtype=np.float32)

        def fn():
            t0 = time.perf_counter()
            if self.kind == "layernorm":
                lib.so_layernorm(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), L.BF16, L.BF16, C.c_int64(rows), C.c_int64(self.cols),
                                 g.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), C.c_float(1e-5), None, None)
            else:
                lib.so_softmax(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), L.BF16, L.BF16, C.c_int64(rows), C.c_int64(self.cols), 0)
            return time.perf_counter() - t0
        return fn, 2.0 * rows * self.cols * 2, rows

    def cpu_baseline(self, budget_s):
        fn, units, rows = self._cpu_fn()
        sec, n = timed_cpu(fn, budget_s)
        return {"value": units / sec / 1e9, "unit": self.unit, "cores": 1, "kind": "port", "sample": f"CPU restatement on {rows} of {self.rows} rows, {n} runs"}

    def reference_step(self):
        fn, units, rows = self._cpu_fn()
        return fn, units, {"kind": "port", "cores": 1, "sample": f"each step = the CPU restatement on {rows} of {self.rows} rows"}

    def close(self):
        self.xs = self.ys = None


class SessionWorkload(Workload):
    """A whole model through the generator: written as an ONNX file, emitted by sofie_b200_emit, compiled with g++, constructed,
    and driven through the emitted Session -- infer_nosync on device-resident inputs for `value` (two input buffers in turn;
    after the first, eager call the Session replays its CUDA graph: one graph launch per pass), infer_host_many for e2e."""

    def model(self): ...            # -> (nodes, initializers, inputs, outputs, input_types)
    def host_input(self): ...       # -> numpy array of one batch
    out_shape, out_torch_dtype = None, None

    def setup(self, torch, ctx, dev, rep):
        import tempfile
        from sofie_b200.session import EmittedSession
        self.torch, self.ctx = torch, ctx
        nodes, init, ins, outs, types = self.model()
        self.sess = EmittedSession(self.name, nodes, init, ins, outs, tempfile.mkdtemp(prefix="sofie_b200_"), input_types=types)
        self.hx = torch.from_numpy(self.host_input()).pin_memory()
        self.xs = [self.hx.to(dev), torch.roll(self.hx, 1, 0).to(dev)]
        torch.cuda.synchronize()
        self._stream = torch.cuda.ExternalStream(self.sess.stream, device=dev)
        l0 = self.sess.launches
        self.sess.infer_nosync(self.xs[0].data_ptr())       # the eager call: every operator is one kernel launch
        self.sess.sync()
        self.kernels_per_pass = self.sess.launches - l0
        self.passes = 0

    def stream(self, torch, dev):
        return self._stream

    def sync(self):
        self.sess.sync()

    def launches(self):
        return self.kernels_per_pass * self.passes   # kernels executed: a replayed graph runs the kernels of the eager call

    def one_pass(self, i):
        self.sess.infer_nosync(self.xs[i & 1].data_ptr())
        self.passes += 1

    def e2e(self, torch, rep, compute):
        r = session_e2e(torch, rep, self.sess, [self.hx], self.out_shape, self.out_torch_dtype, self.units_per_pass())
        r["unit"] = self.unit
        return r

    def session_config(self):
        return {"session": "emitted by sofie_b200_emit from an ONNX model; passes replay the Session's CUDA graph",
                "kernels_per_pass": self.kernels_per_pass, "generator_decisions": len(json.loads(self.sess.report)["fusions"])}

    def close(self):
        self.sess.close()
        self.xs = None


class EncoderWorkload(SessionWorkload):
    """Transformer encoder: 6 pre-LN layers, d_model 512, 8 heads, FFN 2048, Gelu, seq 128; bf16 activations, int8
    per-channel weights dequantised in the contraction epilogue.  One pass = one batch through all layers."""

    def __init__(self, name: str, batch: int, scaling: str = "weak"):
        self.name, self.batch, self.scaling = name, batch, scaling
        self.layers, self.seq, self.d_model, self.heads, self.ffn = 6, 128, 512, 8, 2048
        self.metric = "transformer encoder inferences/s (sequences of 128 tokens)"
        self.unit, self.dtype = "inferences/s", "bf16"

    def model(self):
        from sofie_b200 import encoder as be
        self.flops = be.flops_per_sample(self.layers, self.seq, self.d_model, self.ffn)
        return be.onnx_model(be.make_weights(7, self.layers, self.d_model, self.ffn), self.batch, self.seq, self.d_model, self.heads)

    def host_input(self):
        from sofie_b200 import encoder as be
        x = np.random.default_rng(7).standard_normal((self.batch * self.seq, self.d_model)).astype(np.float32)
        return be.f32_to_bf16_bits(x).view(np.int16)

    def setup(self, torch, ctx, dev, rep):
        self.out_shape, self.out_torch_dtype = (self.batch * self.seq, self.d_model), torch.int16
        super().setup(torch, ctx, dev, rep)

    def units_per_pass(self):
        return float(self.batch)

    def config(self):
        return dict({"workload": self.name, "layers": self.layers, "d_model": self.d_model, "heads": self.heads, "ffn": self.ffn, "seq_len": self.seq,
                     "batch_per_gpu": self.batch, "weights": "int8 per output channel behind DequantizeLinear; the scale is fused in the contraction epilogue",
                     "gflop_per_inference": self.flops / 1e9,
                     "l2": "two input batches in turn; the activations of one pass " + ("exceed" if self.batch >= 64 else "do not exceed") + " the 126 MiB L2"},
                    **self.session_config())

    def roofline(self, s_per_pass, peaks, sustained, launches_per_pass):
        ach = self.flops * self.batch / s_per_pass / 1e12
        return tensor_roofline(ach, peaks, sustained, 1.0, "TFLOP/s", "bf16_tflops" + ("_sustained" if sustained else ""), None,
                               f"; whole pass (all {launches_per_pass:.0f} kernels), not one kernel")

    def _cpu(self):
        """The reference's emitted fp32 code of the 6-layer encoder on the dequantised weights, 2 sequences per step."""
        from sofie_b200 import synth
        try:
            m = RefModel("Encoder_C5t")
            x = synth.normal_f32(synth.tensor_seed(7, 900), (2 * self.seq, self.d_model), 1.0)
            return (lambda: m.infer([x])), 2.0, {"kind": "reference", "cores": os.cpu_count(),
                                                 "sample": f"each step = 2 of {self.batch} sequences through the SOFIE-emitted fp32 code of all {self.layers} layers "
                                                           f"(oracle/_ref Encoder_C5t, dequantised weights); {m.blas}"}
        except Exception:
            sys.path.insert(0, str(ROOT / "tests"))
            import model_oracles as mo
            from oracle_api import Oracle
            from sofie_b200 import encoder as be
            load_oracle()
            o = Oracle(ROOT / "oracle" / "libsofie_oracle.so")
            o.lib.so_threads.restype = C.c_int
            o.lib.so_set_threads(os.cpu_count() or 1)
            w = be.make_weights(7, self.layers, self.d_model, self.ffn)
            x = be.f32_to_bf16_bits(np.random.default_rng(7).standard_normal((2 * self.seq, self.d_model)).astype(np.float32))

            def fn():
                t0 = time.perf_counter()
                mo.encoder_oracle(o, x, w, 2, self.seq, self.d_model, self.heads)
                return time.perf_counter() - t0
            return fn, 2.0, {"kind": "port", "cores": int(o.lib.so_threads()), "sample": f"each step = 2 of {self.batch} sequences through the CPU restatement"}

    def cpu_baseline(self, budget_s):
        fn, units, d = self._cpu()
        sec, n = timed_cpu(fn, budget_s, 10)
        return dict(d, value=units / sec, unit=self.unit)

    def reference_step(self):
        return self._cpu()


class ConvNetWorkload(SessionWorkload):
    """Conv net: 8 Conv3x3 (+ BatchNormalization + Relu) layers, global average pool, Gemm 512 -> 1000, on NCHW
    3 x img x img inputs; fp32 or per-channel int8 (QLinearConv).  One pass = one batch through the network."""

    def __init__(self, name: str, batch: int, img: int, int8: bool):
        self.name, self.batch, self.img, self.int8 = name, batch, img, int8
        self.metric = f"conv net inferences/s ({img}x{img} images, {'int8 QLinearConv' if int8 else 'fp32'})"
        self.unit, self.dtype = "inferences/s", ("int8" if int8 else "fp32 (3xTF32 on tcgen05 where large, fp32 FMA else)")

    def model(self):
        from sofie_b200 import convnet as bc
        self.bc = bc
        self.flops = bc.flops_per_image(self.img)
        return bc.onnx_model(11, self.batch, self.img, self.int8)

    def host_input(self, n=None):
        x = np.random.default_rng(11).random((n or self.batch, 3, self.img, self.img), dtype=np.float32)
        return np.clip(np.rint(x * 127.0), 0, 127).astype(np.int8) if self.int8 else x

    def setup(self, torch, ctx, dev, rep):
        self.out_shape, self.out_torch_dtype = (self.batch, 1000), torch.float32
        super().setup(torch, ctx, dev, rep)

    def units_per_pass(self):
        return float(self.batch)

    def config(self):
        return dict({"workload": self.name, "batch_per_gpu": self.batch, "image": [3, self.img, self.img],
                     "layers": "8 x Conv3x3+BN+Relu, avgpool, Gemm 512->1000", "strides": self.bc.STRIDES, "gflop_per_inference": self.flops / 1e9,
                     "l2": "two input batches in turn; the activations of one pass are several GB (> 126 MiB L2)"}, **self.session_config())

    def roofline(self, s_per_pass, peaks, sustained, launches_per_pass):
        ach = self.flops * self.batch / s_per_pass / 1e12
        if self.int8:
            return tensor_roofline(ach, peaks, sustained, 2.0, "TOP/s", "2 x bf16_tflops" + ("_sustained" if sustained else "") + " (int8 dense)", None,
                                   f"; whole pass ({launches_per_pass:.0f} kernels), not one kernel")
        return tensor_roofline(ach, peaks, sustained, 1.0 / 6.0, "TFLOP/s", "bf16_tflops" + ("_sustained" if sustained else "") +
                               " / 6 (TF32 runs at half the bf16 rate and 3xTF32 makes three passes)", None,
                               f"; whole pass ({launches_per_pass:.0f} kernels), not one kernel")

    def _cpu(self):
        if not self.int8:
            try:   # the reference's emitted fp32 code (Conv -> BatchNormalization+Relu unfused, as it emits them), 4 images per step
                if self.img != 224:
                    raise FileNotFoundError("reference model is built for 224 x 224")
                m = RefModel("ConvNet_C4t")
                x = np.random.default_rng(11).random((4, 3, 224, 224), dtype=np.float32)
                return (lambda: m.infer([x])), 4.0, {"kind": "reference", "cores": os.cpu_count(),
                                                     "sample": f"each step = 4 of {self.batch} images through the SOFIE-emitted fp32 code (oracle/_ref ConvNet_C4t); {m.blas}; "
                                                               "Im2col and BatchNormalization loops of the emitted code are single-threaded"}
            except Exception:
                pass
        sys.path.insert(0, str(ROOT / "tests"))
        import model_oracles as mo
        from oracle_api import Oracle
        from sofie_b200 import convnet as bc
        load_oracle()
        o = Oracle(ROOT / "oracle" / "libsofie_oracle.so")
        o.lib.so_threads.restype = C.c_int
        o.lib.so_set_threads(os.cpu_count() or 1)
        w = bc.make_weights(11, self.int8)
        x = self.host_input(1)

        def fn():
            t0 = time.perf_counter()
            mo.convnet_oracle(o, x, w, self.int8)
            return time.perf_counter() - t0
        return fn, 1.0, {"kind": "port", "cores": int(o.lib.so_threads()),
                         "sample": f"each step = 1 of {self.batch} images through the CPU restatement" + (" (the reference has no QLinearConv)" if self.int8 else "")}

    def cpu_baseline(self, budget_s):
        fn, units, d = self._cpu()
        sec, n = timed_cpu(fn, budget_s, 10)
        return dict(d, value=units / sec, unit=self.unit)

    def reference_step(self):
        return self._cpu()


def make_workload(name: str, world: int) -> Workload:
    if name == "qlinear_matmul_4096":
        return GemmWorkload(name, 4096, "int8")
    if name == "qlinear_matmul_8192":
        return GemmWorkload(name, 8192, "int8")
    if name == "fp8_gemm_8192":
        return GemmWorkload(name, 8192, "fp8")
    if name == "layernorm_bf16_65536x512":
        return RowOpWorkload("layernorm", 65536, 512, name)
    if name == "softmax_bf16_524288x128":
        return RowOpWorkload("softmax", 524288, 128, name)
    if name == "transformer_encoder":          # the configuration's 512 sequences over all GPUs (64 per GPU at 8 GPUs)
        return EncoderWorkload(name, max(1, 512 // world), "strong")
    if name == "transformer_encoder_b512":
        return EncoderWorkload(name, 512)
    if name == "transformer_encoder_b64":
        return EncoderWorkload(name, 64)
    if name.startswith("convnet_"):
        _, kind, b = name.split("_")
        return ConvNetWorkload(name, int(b[1:]), 224, kind == "int8")
    raise SystemExit(f"bench.py: unknown workload {name}")


WORKLOAD_NAMES = ["qlinear_matmul_4096", "qlinear_matmul_8192", "fp8_gemm_8192", "layernorm_bf16_65536x512", "softmax_bf16_524288x128",
                  "transformer_encoder", "transformer_encoder_b512", "transformer_encoder_b64", "convnet_fp32_b256", "convnet_int8_b256",
                  "convnet_fp32_b32", "convnet_int8_b32"]
ALSO = ["fp8_gemm_8192", "convnet_int8_b256", "convnet_fp32_b256", "transformer_encoder", "layernorm_bf16_65536x512", "softmax_bf16_524288x128"]


# ---------------------------------------------------------------------------------------------
def measure(torch, rep, ctx, dev, w: Workload, steps: int, warmup: int, seconds: float, cpu_budget: float) -> dict:
    """Warm-up, calibration of the passes per step, the timed region, end-to-end and (one GPU) the CPU baseline."""
    from sofie_b200 import replicas
    w.setup(torch, ctx, dev, rep)
    stream = w.stream(torch, dev)
    n_warm = max(3, warmup)
    for i in range(n_warm):
        w.one_pass(i)
    w.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(6):
        w.one_pass(i)
    e1.record(stream)
    torch.cuda.synchronize()
    t_pass = max(1e-6, e0.elapsed_time(e1) * 1e-3 / 6)
    inner = int(max(1, math.ceil(seconds / steps / t_pass)))
    inner = int(replicas.max_over_ranks(rep, float(inner)))
    # at least 200 ms of warm-up in all (the reference's rule, benchmark/src/WarmupUtil.hxx:25-39)
    for i in range(int(min(inner * steps, math.ceil(0.2 / t_pass)))):
        w.one_pass(i)
    w.sync()
    sampler = ClockSampler(rep.local_rank)
    replicas.barrier(rep)
    torch.cuda.synchronize()
    l0 = w.launches()
    sampler.start()
    e0.record(stream)
    k = 0
    for _ in range(steps):
        for _ in range(inner):
            w.one_pass(k)
            k += 1
    e1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    w.sync()
    launches = w.launches() - l0
    ms_local = e0.elapsed_time(e1)
    replicas.barrier(rep)
    ms = replicas.max_over_ranks(rep, ms_local)
    passes = steps * inner
    value = rep.world * w.units_per_pass() * passes / (ms * 1e-3) / w.unit_scale
    e2e = w.e2e(torch, rep, stream)
    rec = None
    if rep.is_root:
        peaks = measured_peaks()
        s_per_pass = ms_local * 1e-3 / passes
        sustained = ms * 1e-3 >= 1.0
        rec = {"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": rep.world, "steps": steps, "warmup": n_warm,
               "ms_per_step": ms / steps, "higher_is_better": True, "scaling": w.scaling, "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
               "config": dict(w.config(), launches_per_step=launches // steps, passes_per_step=inner, ms_per_pass=ms / passes, replicas=rep.world,
                              timed_region_s=ms * 1e-3),
               "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e,
               "roofline": w.roofline(s_per_pass, peaks, sustained, launches / passes)}
        if clocks.get("sm_mhz"):
            rec["roofline"]["ms_per_pass_x_sm_mhz"] = ms_local / passes * clocks["sm_mhz"]
        if rep.world == 1 and cpu_budget > 0:
            rec["cpu_baseline"] = w.cpu_baseline(cpu_budget)
    w.close()
    torch.cuda.empty_cache()
    return rec


def run_ours(args) -> None:
    import torch
    from sofie_b200 import replicas
    from sofie_b200.ops import Context

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    rep = replicas.init_from_env("nccl")
    torch.cuda.set_device(rep.local_rank)
    dev = f"cuda:{rep.local_rank}"
    ctx = Context(rep.local_rank)
    main = args.workload or "qlinear_matmul_4096"
    line = measure(torch, rep, ctx, dev, make_workload(main, rep.world), args.steps, args.warmup, args.seconds, 12.0)
    if args.workload is None and not args.no_also:
        also = []
        for name in ALSO:
            rec = measure(torch, rep, ctx, dev, make_workload(name, rep.world), args.steps, args.warmup, min(args.seconds, 2.0), 4.0)
            if rec is not None:
                rec["workload"] = name
                also.append(rec)
        if line is not None:
            line["also"] = also
    ctx.close()
    replicas.shutdown(rep)
    if line is not None:
        print(json.dumps(line), flush=True)


def run_reference(args) -> None:
    """The reference arm: the reference's own CPU implementation of the workload, on every host core it can use; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = make_workload(args.workload or "qlinear_matmul_4096", world)
    fn, units, desc = w.reference_step()
    for _ in range(min(args.warmup, 2)):
        fn()
    t = 0.0
    done = 0
    for _ in range(args.steps):       # bounded: the whole arm ends within a few minutes
        t += fn()
        done += 1
        if t > 150.0:
            break
    val = units * done / t / w.unit_scale
    cfg = {"workload": w.name}
    if isinstance(w, GemmWorkload):
        cfg.update(M=w.n, N=w.n, K=w.n)
    line = {"impl": "reference", "metric": w.metric, "value": val, "unit": w.unit, "n_gpus": args.gpus, "steps": done, "warmup": min(args.warmup, 2),
            "ms_per_step": 1e3 * t / done, "higher_is_better": True, "scaling": w.scaling, "vs_baseline": None, "dtype": "fp32" if desc["kind"] == "reference" else w.dtype,
            "data": "synthetic", "config": cfg, "cpu_baseline": dict(desc, value=val, unit=w.unit),
            "e2e": {"value": val, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=WORKLOAD_NAMES)
    ap.add_argument("--seconds", type=float, default=2.5, help="length of the timed region the passes per step are sized for")
    ap.add_argument("--no-also", action="store_true", help="measure the headline workload only")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("bench.py: --steps must be at least 1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
