"""numpy front-end of the CPU checker (oracle/libsofie_oracle.so) for the tests."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from sofie_b200 import lib as L

ROOT = Path(__file__).resolve().parent.parent
NP_OF = {L.F32: np.float32, L.BF16: np.uint16, L.I8: np.int8, L.F8E4M3: np.uint8, L.I32: np.int32, L.U8: np.uint8}


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Oracle:
    def __init__(self, so_path):
        self.lib = C.CDLL(str(so_path))

    def epilogue(self, row_scale=None, col_scale=None, alpha=1.0, beta=1.0, bias=None, bias_mode=None, ldc=0, residual=None,
                 residual_dtype=L.F32, ldr=0, act=L.ACT_NONE, act_alpha=0.0, out_scale=1.0, out_zero_point=0):
        e = L.Epilogue()
        e.row_scale, e.col_scale, e.alpha, e.beta = _p(row_scale), _p(col_scale), alpha, beta
        if bias is not None and bias_mode is None:
            bias_mode = L.BIAS_COL_I32 if bias.dtype == np.int32 else L.BIAS_COL_F32
        e.bias_mode, e.bias, e.ldc = bias_mode or L.BIAS_NONE, _p(bias), ldc
        e.residual, e.residual_dtype, e.ldr = _p(residual), residual_dtype, ldr
        e.act, e.act_alpha, e.out_scale, e.out_zero_point = act, act_alpha, out_scale, out_zero_point
        return e

    def gemm(self, a, b, M, N, K, ab_dtype, y_dtype, trans_a=False, trans_b=False, batch=1, ep=None, **strides):
        d = L.GemmDesc()
        d.M, d.N, d.K, d.batch = M, N, K, batch
        d.trans_a, d.trans_b, d.ab_dtype, d.y_dtype = int(trans_a), int(trans_b), ab_dtype, y_dtype
        d.stride_a = strides.get("stride_a", (K * M) if batch > 1 else 0)
        d.stride_b = strides.get("stride_b", (K * N) if batch > 1 else 0)
        d.stride_y = M * N if batch > 1 else 0
        d.stride_c, d.stride_r = strides.get("stride_c", 0), strides.get("stride_r", 0)
        y = np.zeros((batch, M, N), dtype=NP_OF[y_dtype])
        rc = self.lib.so_gemm(C.byref(d), _p(a), _p(b), _p(y), C.byref(ep) if ep is not None else None)
        assert rc == 0
        return y if batch > 1 else y[0]

    def conv(self, x, w, desc: L.ConvDesc, ho, wo, ep=None):
        y = np.zeros((desc.N, desc.K, ho, wo), dtype=NP_OF[desc.y_dtype])
        rc = self.lib.so_conv(C.byref(desc), _p(x), _p(w), _p(y), C.byref(ep) if ep is not None else None)
        assert rc == 0
        return y

    def layernorm(self, x, scale, bias, eps, dtype=L.F32):
        y = np.zeros_like(x)
        rows, cols = x.shape
        self.lib.so_layernorm(_p(x), _p(y), dtype, dtype, C.c_int64(rows), C.c_int64(cols), _p(scale), _p(bias), C.c_float(eps), None, None)
        return y

    def softmax(self, x, dtype=L.F32, log=False):
        y = np.zeros_like(x)
        rows, cols = x.shape
        self.lib.so_softmax(_p(x), _p(y), dtype, dtype, C.c_int64(rows), C.c_int64(cols), int(log))
        return y

    def unary(self, x, act, act_alpha=0.0, dtype=L.F32):
        y = np.zeros_like(x)
        self.lib.so_unary(_p(x), _p(y), dtype, C.c_int64(x.size), act, C.c_float(act_alpha))
        return y

    def binary(self, a, b, op, dtype=L.F32):
        y = np.zeros_like(a)
        self.lib.so_binary(_p(a), _p(b), _p(y), dtype, C.c_int64(a.size), C.c_int64(b.size), op, 0)
        return y

    def quantize(self, x, scale, zp, q_dtype, channels=1, inner=1):
        q = np.zeros(x.shape, dtype=NP_OF[q_dtype])
        self.lib.so_quantize(_p(x), _p(q), q_dtype, C.c_int64(x.size), _p(scale), _p(zp), C.c_int64(channels), C.c_int64(inner))
        return q

    def dequantize(self, q, scale, zp, q_dtype, channels=1, inner=1):
        x = np.zeros(q.shape, dtype=np.float32)
        self.lib.so_dequantize(_p(q), _p(x), q_dtype, C.c_int64(q.size), _p(scale), _p(zp), C.c_int64(channels), C.c_int64(inner))
        return x

    def convert(self, x, x_dtype, y_dtype, row_scale=None):
        y = np.zeros(x.shape, dtype=NP_OF[y_dtype])
        rows, cols = x.shape
        self.lib.so_convert(_p(x), _p(y), x_dtype, y_dtype, C.c_int64(rows), C.c_int64(cols), _p(row_scale))
        return y

    def global_avgpool(self, x, x_dtype=L.F32):
        nc = x.shape[0] * x.shape[1]
        inner = x.size // nc
        y = np.zeros((x.shape[0], x.shape[1]), dtype=np.float32)
        self.lib.so_global_avgpool(_p(x), _p(y), x_dtype, C.c_int64(nc), C.c_int64(inner))
        return y


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)
