"""Host-side handles over the C ABI: a Context (the Session's queue + blas object) and plans.

torch is used for device memory and streams only; every computation is a call into
libsofie_b200.so.  Tensors must live on the context's CUDA device.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
from typing import Optional

import torch

from . import lib as L

_DT = {
    torch.float32: L.F32,
    torch.bfloat16: L.BF16,
    torch.int8: L.I8,
    torch.float8_e4m3fn: L.F8E4M3,
    torch.int32: L.I32,
    torch.uint8: L.U8,
}


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise TypeError(f"dtype {t} is not part of the sofie_b200 ABI") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("sofie_b200 operators take CUDA tensors; host data goes through run_host()")
    return t.data_ptr()


class Context:
    """One per Session / GPU / stream (sofie_b200_ctx)."""

    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None):
        self._lib = L.load()
        self.device = device
        self.stream = stream
        h = C.c_void_p()
        sp = C.c_void_p(stream.cuda_stream) if stream is not None else C.c_void_p(
            torch.cuda.current_stream(device).cuda_stream)
        L.check(self._lib.sofie_b200_ctx_create(C.byref(h), device, sp), "ctx_create")
        self._h = h

    def sync(self) -> None:
        L.check(self._lib.sofie_b200_ctx_sync(self._h), "ctx_sync")

    @property
    def launches(self) -> int:
        return int(self._lib.sofie_b200_ctx_launch_count(self._h))

    # another GPU's memory, for GemmPlan.enqueue_peers
    def enable_peer(self, peer_device: int) -> None:
        """One process driving several GPUs: this ctx's kernels may then store to `peer_device`'s memory."""
        L.check(self._lib.sofie_b200_ctx_enable_peer(self._h, int(peer_device)), "ctx_enable_peer")

    def peer_export(self, t: torch.Tensor) -> bytes:
        """The 72 bytes another process needs to open `t`'s first element (send them by any means)."""
        h = L.PeerHandle()
        L.check(self._lib.sofie_b200_peer_export(self._h, _ptr(t), C.byref(h)), "peer_export")
        return bytes(h)

    def peer_open(self, handle: bytes) -> int:
        """Device pointer, valid in this process, to the byte another process exported."""
        h = L.PeerHandle.from_buffer_copy(handle)
        p = C.c_void_p()
        L.check(self._lib.sofie_b200_peer_open(self._h, C.byref(h), C.byref(p)), "peer_open")
        return int(p.value)

    def peer_close(self, ptr: int) -> None:
        L.check(self._lib.sofie_b200_peer_close(self._h, C.c_void_p(ptr)), "peer_close")

    def close(self) -> None:
        if self._h:
            self._lib.sofie_b200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- memory-bound operators -----------------------------------------------------
    def layernorm(self, x, y, scale=None, bias=None, eps=1e-5, mean_out=None, invstd_out=None):
        cols = x.shape[-1]
        rows = x.numel() // cols
        L.check(self._lib.sofie_b200_layernorm_enqueue(
            self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), dtype_code(y.dtype), rows, cols, _ptr(scale),
            _ptr(bias), eps, _ptr(mean_out), _ptr(invstd_out)), "layernorm_enqueue")

    def softmax(self, x, y, log_softmax=False):
        cols = x.shape[-1]
        rows = x.numel() // cols if cols else 0
        L.check(self._lib.sofie_b200_softmax_enqueue(
            self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), dtype_code(y.dtype), rows, cols, int(log_softmax)),
            "softmax_enqueue")

    def softmax_axis(self, x, y, axis, log_softmax=False):
        """Softmax over `axis` of a contiguous tensor (any axis)."""
        axis = axis + x.dim() if axis < 0 else axis
        outer = int(np.prod(x.shape[:axis])) if axis else 1
        inner = int(np.prod(x.shape[axis + 1:])) if axis + 1 < x.dim() else 1
        L.check(self._lib.sofie_b200_softmax_axis_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), outer, x.shape[axis], inner,
                                                          int(log_softmax)), "softmax_axis_enqueue")

    def sdpa(self, q, k, v, y, mask=None, scale=0.0, heads=0, ldq=0, ldk=0, ldv=0):
        """Scaled dot-product attention through an SDPA plan made for this call.  Rank-4 tensors are [B,H,S,D]; rank-3
        tensors are folded [B,S,H*D] and need `heads` (ldq / ldk / ldv: row pitches when Q, K, V are column blocks of a
        wider tensor).  Returns the kernel family that ran ("attention" or "chain")."""
        import torch
        d = L.SdpaDesc()
        if q.dim() == 4:
            d.batch, d.heads, d.seq, d.head_dim = q.shape
            d.v_head_dim, d.folded = v.shape[3], 0
        else:
            d.batch, d.seq = q.shape[0], q.shape[1]
            d.heads, d.folded = heads, 1
            d.head_dim, d.v_head_dim = q.shape[2] // heads, y.shape[2] // heads
            d.ldq, d.ldk, d.ldv = ldq, ldk, ldv
        d.dtype, d.has_mask, d.scale = dtype_code(q.dtype), int(mask is not None), float(scale)
        h = C.c_void_p()
        L.check(self._lib.sofie_b200_sdpa_plan_create(self._h, C.byref(d), C.byref(h)), "sdpa_plan_create")
        try:
            ws = torch.empty(max(256, self._lib.sofie_b200_sdpa_workspace_bytes(h)), dtype=torch.uint8, device=q.device)
            L.check(self._lib.sofie_b200_sdpa_enqueue(h, _ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(y), _ptr(ws)), "sdpa_enqueue")
            kernel = self._lib.sofie_b200_sdpa_plan_kernel(h).decode()
            self.sync()   # the workspace is released on return
        finally:
            self._lib.sofie_b200_sdpa_plan_destroy(h)
        return kernel

    def unary(self, x, y, act, act_alpha=0.0):
        L.check(self._lib.sofie_b200_unary_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), x.numel(), act,
                                                   act_alpha), "unary_enqueue")

    def binary(self, a, b, y, op=0, act=L.ACT_NONE):
        L.check(self._lib.sofie_b200_binary_enqueue(self._h, _ptr(a), _ptr(b), _ptr(y), dtype_code(a.dtype),
                                                    a.numel(), b.numel(), op, act), "binary_enqueue")

    def batchnorm(self, x, y, fused_scale, bias, mean, act=L.ACT_NONE):
        outer, ch = x.shape[0], x.shape[1]
        inner = x.numel() // (outer * ch) if outer * ch else 0
        L.check(self._lib.sofie_b200_batchnorm_enqueue(self._h, _ptr(x), _ptr(y), outer, ch, inner,
                                                       _ptr(fused_scale), _ptr(bias), _ptr(mean), act),
                "batchnorm_enqueue")

    def global_avgpool(self, x, y):
        nc = x.shape[0] * x.shape[1]
        inner = x.numel() // nc if nc else 0
        L.check(self._lib.sofie_b200_global_avgpool_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), nc,
                                                            inner), "global_avgpool_enqueue")

    def global_avgpool_nhwc(self, x, y):
        """x: channels-last [n, ..., c]; y: [n, c] fp32."""
        n, c = x.shape[0], x.shape[-1]
        pixels = x.numel() // (n * c) if n * c else 0
        L.check(self._lib.sofie_b200_global_avgpool_nhwc_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), n, pixels, c),
                "global_avgpool_nhwc_enqueue")

    def quantize(self, x, q, scale, zero_point, channels=1, inner=1):
        L.check(self._lib.sofie_b200_quantize_enqueue(self._h, _ptr(x), _ptr(q), dtype_code(q.dtype), x.numel(),
                                                      _ptr(scale), _ptr(zero_point), channels, inner),
                "quantize_enqueue")

    def dequantize(self, q, x, scale, zero_point, channels=1, inner=1):
        L.check(self._lib.sofie_b200_dequantize_enqueue(self._h, _ptr(q), _ptr(x), dtype_code(q.dtype), q.numel(),
                                                        _ptr(scale), _ptr(zero_point), channels, inner),
                "dequantize_enqueue")

    def attention(self, qkv, out, batch, seq, heads, head_dim, scale):
        """qkv [batch, seq, 3, heads, head_dim] -> out [batch, seq, heads * head_dim] (fused Softmax(scale Q K^T) V)."""
        L.check(self._lib.sofie_b200_attention_enqueue(self._h, _ptr(qkv), _ptr(out), dtype_code(qkv.dtype), batch, seq, heads, head_dim,
                                                       float(scale)), "attention_enqueue")

    def depth_unfold(self, x, y, taps, d_out, stride_d=1, pad_front=0, dil_d=1):
        """x [n, c, d, h, w] -> y [n * d_out, c * taps, h, w]: the depth taps of a 3-D convolution as channels."""
        n, c, d = x.shape[:3]
        hw = int(x[0, 0, 0].numel())
        L.check(self._lib.sofie_b200_depth_unfold_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), n, c, d, hw, taps, d_out, stride_d, pad_front, dil_d),
                "depth_unfold_enqueue")

    def transpose(self, x, y, perm):
        shape = (C.c_int64 * x.dim())(*x.shape)
        pm = (C.c_int32 * x.dim())(*perm)
        L.check(self._lib.sofie_b200_transpose_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype), x.dim(), shape, pm),
                "transpose_enqueue")

    def convert(self, x, y, row_scale=None):
        cols = x.shape[-1]
        rows = x.numel() // cols if cols else 0
        L.check(self._lib.sofie_b200_convert_enqueue(self._h, _ptr(x), _ptr(y), dtype_code(x.dtype),
                                                     dtype_code(y.dtype), rows, cols, _ptr(row_scale)),
                "convert_enqueue")


def make_epilogue(row_scale=None, col_scale=None, alpha=1.0, beta=1.0, bias=None, bias_mode=None, ldc=0,
                  residual=None, ldr=0, act=L.ACT_NONE, act_alpha=0.0, out_scale=1.0,
                  out_zero_point=0) -> tuple[L.Epilogue, list]:
    """Builds a sofie_b200_epilogue from torch tensors; returns it with the tensors to keep alive."""
    e = L.Epilogue()
    e.row_scale = _ptr(row_scale)
    e.col_scale = _ptr(col_scale)
    e.alpha = alpha
    e.beta = beta
    if bias is not None and bias_mode is None:
        bias_mode = L.BIAS_COL_I32 if bias.dtype == torch.int32 else L.BIAS_COL_F32
    e.bias_mode = bias_mode or L.BIAS_NONE
    e.bias = _ptr(bias)
    e.ldc = ldc
    e.residual = _ptr(residual)
    e.residual_dtype = dtype_code(residual.dtype) if residual is not None else L.F32
    e.ldr = ldr
    e.act = act
    e.act_alpha = act_alpha
    e.out_scale = out_scale
    e.out_zero_point = out_zero_point
    return e, [row_scale, col_scale, bias, residual]


class GemmPlan:
    """One registered contraction (sofie_b200_gemm_plan)."""

    def __init__(self, ctx: Context, M, N, K, ab_dtype, y_dtype, trans_a=False, trans_b=False, batch=1, lda=0,
                 ldb=0, ldy=0, stride_a=0, stride_b=0, stride_y=0, stride_c=0, stride_r=0, precise=True, flags=0):
        self.ctx = ctx
        self._lib = ctx._lib
        d = L.GemmDesc()
        d.M, d.N, d.K, d.batch = M, N, K, batch
        d.trans_a, d.trans_b = int(trans_a), int(trans_b)
        d.ab_dtype = dtype_code(ab_dtype)
        d.y_dtype = dtype_code(y_dtype)
        d.lda, d.ldb, d.ldy = lda, ldb, ldy
        d.stride_a, d.stride_b, d.stride_y = stride_a, stride_b, stride_y
        d.stride_c, d.stride_r = stride_c, stride_r
        d.precise = int(precise)
        d.flags = int(flags)
        self.desc = d
        h = C.c_void_p()
        L.check(self._lib.sofie_b200_gemm_plan_create(ctx._h, C.byref(d), C.byref(h)), "gemm_plan_create")
        self._h = h

    @property
    def kernel(self) -> str:
        return self._lib.sofie_b200_gemm_plan_kernel(self._h).decode()

    def enqueue(self, A, B, Y, epilogue: Optional[L.Epilogue] = None) -> None:
        ep = C.byref(epilogue) if epilogue is not None else None
        L.check(self._lib.sofie_b200_gemm_enqueue(self._h, _ptr(A), _ptr(B), _ptr(Y), ep), "gemm_enqueue")

    def enqueue_peers(self, A, B, y_ptr: int, peer_ptrs, epilogue: Optional[L.Epilogue] = None) -> None:
        """The contraction with every finished row segment stored to `y_ptr` and to each of `peer_ptrs` (raw device
        pointers: this rank's columns inside its own and inside the other ranks' full-width results)."""
        ep = C.byref(epilogue) if epilogue is not None else None
        n = len(peer_ptrs)
        arr = (C.c_void_p * max(n, 1))(*peer_ptrs)
        L.check(self._lib.sofie_b200_gemm_enqueue_peers(self._h, _ptr(A), _ptr(B), C.c_void_p(y_ptr), arr, n, ep), "gemm_enqueue_peers")

    def run_host(self, hostA, hostB, hostY, epilogue: Optional[L.Epilogue] = None) -> None:
        """Host operands (pinned or pageable CPU tensors): H2D, contraction, D2H, wait."""
        for t in (hostA, hostB, hostY):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("run_host takes contiguous CPU tensors")
        ep = C.byref(epilogue) if epilogue is not None else None
        L.check(self._lib.sofie_b200_gemm_run_host(self._h, hostA.data_ptr(), hostB.data_ptr(), hostY.data_ptr(), ep),
                "gemm_run_host")

    def run_host_many(self, hostA, hostB, hostY, epilogue: Optional[L.Epilogue] = None) -> None:
        """Lists of host operands, one entry per inference: copies and contractions of successive inferences overlap."""
        n = len(hostA)
        if len(hostB) != n or len(hostY) != n:
            raise ValueError("run_host_many takes three lists of the same length")
        for t in (*hostA, *hostB, *hostY):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("run_host_many takes contiguous CPU tensors")
        arr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() for t in ts])
        ep = C.byref(epilogue) if epilogue is not None else None
        L.check(self._lib.sofie_b200_gemm_run_host_many(self._h, n, arr(hostA), arr(hostB), arr(hostY), ep), "gemm_run_host_many")

    def close(self) -> None:
        if self._h:
            self._lib.sofie_b200_gemm_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
