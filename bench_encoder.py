"""The transformer-encoder configuration on libsofie_b200, for bench.py and the parity tests.

Pre-LayerNorm encoder layers: LN -> QKV projection -> per-head Softmax(Q K^T / sqrt(d_h)) V -> output projection
+ residual -> LN -> FFN (Gelu) -> + residual.  Activations are bf16; the four projection weights of a layer are
int8 with one fp32 scale per output channel, converted to bf16 once at construction, the scale applied as the
column scale of the contraction's epilogue together with bias, Gelu and the residual add.  Every operator is one
call of the C ABI (sofie_b200/ops.py); all buffers are allocated once, a step allocates nothing.

`encoder_oracle` composes the same graph from the CPU restatement (oracle/), rounding to bf16 at the same tensor
boundaries; it is the checker of the tests and the CPU arm of the benchmark.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns of an fp32 array (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def make_weights(rng, layers: int, d_model: int, ffn: int):
    """int8 per-output-channel weights ~N(0, 0.02) with scale = absmax/127, fp32 biases, LN gamma 1 / beta 0."""
    def qlinear(n_out, n_in):
        w = rng.standard_normal((n_out, n_in)).astype(np.float32) * 0.02
        scale = (np.abs(w).max(axis=1) / 127.0).astype(np.float32)
        q = np.clip(np.rint(w / scale[:, None]), -127, 127).astype(np.int8)
        return q, scale, (rng.standard_normal(n_out) * 0.02).astype(np.float32)
    out = []
    for _ in range(layers):
        out.append({"qkv": qlinear(3 * d_model, d_model), "out": qlinear(d_model, d_model), "ff1": qlinear(ffn, d_model),
                    "ff2": qlinear(d_model, ffn), "g1": np.ones(d_model, np.float32), "b1": np.zeros(d_model, np.float32),
                    "g2": np.ones(d_model, np.float32), "b2": np.zeros(d_model, np.float32)})
    return out


def flops_per_sample(layers: int, seq: int, d_model: int, ffn: int) -> float:
    proj = 2.0 * seq * d_model * (3 * d_model + d_model + 2 * ffn)
    attn = 2.0 * 2.0 * seq * seq * d_model
    return layers * (proj + attn)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def attention_oracle(o, qkv_bits: np.ndarray, batch: int, seq: int, heads: int, dh: int, scale: float) -> np.ndarray:
    """Checker of the fused attention kernel, with its roundings: fp32 scores, exp(scale*s - max) rounded to bf16
    (unnormalised), second contraction on those, division by the sum of the rounded values, bf16 result.
    qkv_bits: [batch, seq, 3, heads, dh] bf16 bit patterns; returns [batch*seq, heads*dh] bf16 bit patterns."""
    from sofie_b200 import lib as L
    t = np.ascontiguousarray(qkv_bits.reshape(batch, seq, 3 * heads, dh).transpose(2, 0, 1, 3))   # [3H, B, S, dh]
    q, k, v = (np.ascontiguousarray(t[i * heads:(i + 1) * heads]).reshape(heads * batch, seq, dh) for i in range(3))
    sc = o.gemm(q, k, seq, seq, dh, L.BF16, L.F32, False, True, batch=heads * batch).reshape(heads * batch, seq, seq)
    z = sc.astype(np.float64) * scale
    e = np.exp(z - z.max(axis=-1, keepdims=True)).astype(np.float32)
    pb = f32_to_bf16_bits(e)
    den = bf16_bits_to_f32(pb).astype(np.float64).sum(axis=-1, keepdims=True)
    ov = o.gemm(pb, v, seq, dh, seq, L.BF16, L.F32, False, False, batch=heads * batch).reshape(heads * batch, seq, dh)
    a = f32_to_bf16_bits((ov / den).astype(np.float32))
    return np.ascontiguousarray(a.reshape(heads, batch, seq, dh).transpose(1, 2, 0, 3)).reshape(batch * seq, heads * dh)


def encoder_oracle(o, x_bits: np.ndarray, weights, batch: int, seq: int, d_model: int, heads: int, fused_attention: bool = False):
    """x_bits: [batch*seq, d_model] bf16 bit patterns.  Returns the output activations as bf16 bit patterns.
    `fused_attention` selects the roundings of the fused attention kernel instead of those of the operator chain."""
    from sofie_b200 import lib as L
    dh = d_model // heads
    m = batch * seq
    x = x_bits

    def linear(a, wq, scale, bias, act=L.ACT_NONE, residual=None):
        w = f32_to_bf16_bits(wq.astype(np.float32))  # int8 values are exact in bf16
        ep = o.epilogue(col_scale=scale, bias=bias, act=act, residual=residual, residual_dtype=L.BF16)
        return o.gemm(a, w, m, wq.shape[0], wq.shape[1], L.BF16, L.BF16, False, True, ep=ep)

    for ly in weights:
        h = o.layernorm(x, ly["g1"], ly["b1"], 1e-5, L.BF16)
        qkv = linear(h, *ly["qkv"])
        if fused_attention:
            a = attention_oracle(o, qkv, batch, seq, heads, dh, 1.0 / np.sqrt(dh))
        else:
            t = np.ascontiguousarray(qkv.reshape(batch, seq, 3 * heads, dh).transpose(2, 0, 1, 3))   # [3H, B, S, dh]
            q, k, v = (np.ascontiguousarray(t[i * heads:(i + 1) * heads]).reshape(heads * batch, seq, dh) for i in range(3))
            sc = o.gemm(q, k, seq, seq, dh, L.BF16, L.BF16, False, True, batch=heads * batch, ep=o.epilogue(alpha=1.0 / np.sqrt(dh)))
            p = o.softmax(sc.reshape(-1, seq), L.BF16).reshape(heads * batch, seq, seq)
            a = o.gemm(p, v, seq, dh, seq, L.BF16, L.BF16, False, False, batch=heads * batch)
            a = np.ascontiguousarray(a.reshape(heads, batch, seq, dh).transpose(1, 2, 0, 3)).reshape(m, d_model)
        x = linear(a, *ly["out"], residual=x)
        h = o.layernorm(x, ly["g2"], ly["b2"], 1e-5, L.BF16)
        f = linear(h, *ly["ff1"], act=L.ACT_GELU_ERF)
        x = linear(f, *ly["ff2"], residual=x)
    return x


class EncoderB200:
    """The encoder on one GPU through the C ABI.  `ctx` is a sofie_b200.ops.Context on that GPU."""

    LAUNCHES_PER_LAYER = 7            # 4 projections, 2 LayerNorms, 1 fused attention
    LAUNCHES_PER_LAYER_UNFUSED = 11   # attention as 2 batched contractions, Softmax and 2 transposes

    def __init__(self, ctx, weights, batch: int, seq: int, d_model: int, heads: int, ffn: int, device: str, fused_attention: bool = True):
        import torch
        from sofie_b200.ops import GemmPlan, make_epilogue
        from sofie_b200 import lib as L
        t, bf = torch, torch.bfloat16
        self.ctx, self.batch, self.seq, self.d, self.heads, self.ffn = ctx, batch, seq, d_model, heads, ffn
        self.dh = dh = d_model // heads
        self.fused = fused_attention and dh == 64 and seq <= 128
        m, hb = batch * seq, heads * batch
        dev = device
        # activations, allocated once
        self.h = t.empty((m, d_model), dtype=bf, device=dev)
        self.qkv = t.empty((m, 3 * d_model), dtype=bf, device=dev)
        self.tq = t.empty((3 * heads, batch, seq, dh), dtype=bf, device=dev)
        self.sc = t.empty((hb, seq, seq), dtype=bf, device=dev)
        self.p = t.empty_like(self.sc)
        self.a = t.empty((heads, batch, seq, dh), dtype=bf, device=dev)
        self.am = t.empty((batch, seq, heads, dh), dtype=bf, device=dev)
        self.x1 = t.empty((m, d_model), dtype=bf, device=dev)
        self.x2 = t.empty((m, d_model), dtype=bf, device=dev)
        self.f = t.empty((m, ffn), dtype=bf, device=dev)
        self.keep = []
        self.layers = []
        for ly in weights:
            d = {}
            for name, act in (("qkv", L.ACT_NONE), ("out", L.ACT_NONE), ("ff1", L.ACT_GELU_ERF), ("ff2", L.ACT_NONE)):
                wq, scale, bias = ly[name]
                w8 = t.from_numpy(wq).to(dev)
                wb = t.empty(wq.shape, dtype=bf, device=dev)
                ctx.convert(w8, wb)   # weights become bf16 once; the per-channel scale stays in the epilogue
                d[name] = dict(w=wb, scale=t.from_numpy(scale).to(dev), bias=t.from_numpy(bias).to(dev), act=act,
                               plan=GemmPlan(ctx, m, wq.shape[0], wq.shape[1], bf, bf, trans_b=True))
                assert d[name]["plan"].kernel == "umma"
            for name in ("g1", "b1", "g2", "b2"):
                d[name] = t.from_numpy(ly[name]).to(dev)
            self.layers.append(d)
        ctx.sync()
        self.qk = GemmPlan(ctx, seq, seq, dh, bf, bf, trans_b=True, batch=hb, stride_a=seq * dh, stride_b=seq * dh, stride_y=seq * seq)
        self.pv = GemmPlan(ctx, seq, dh, seq, bf, bf, trans_b=False, batch=hb, stride_a=seq * seq, stride_b=seq * dh, stride_y=seq * dh)
        assert self.qk.kernel == "umma" and self.pv.kernel == "umma"
        self.ep_qk, k = make_epilogue(alpha=float(1.0 / np.sqrt(dh)))
        self.keep.append(k)
        self._make_epilogue = make_epilogue

    def _linear(self, a, layer, name, y, residual=None):
        e = layer[name]
        ep, keep = self._make_epilogue(col_scale=e["scale"], bias=e["bias"], act=e["act"], residual=residual)
        e["plan"].enqueue(a, e["w"], y, ep)

    def __call__(self, x):
        """x: [batch*seq, d_model] bf16 on the device; returns the output activations (a buffer owned by this object,
        overwritten by the next call).  Work is only enqueued; the caller synchronises."""
        ctx, heads, b, s, dh = self.ctx, self.heads, self.batch, self.seq, self.dh
        m = b * s
        cur = x
        for i, ly in enumerate(self.layers):
            ctx.layernorm(cur, self.h, ly["g1"], ly["b1"], 1e-5)
            self._linear(self.h, ly, "qkv", self.qkv)
            if self.fused:
                ctx.attention(self.qkv, self.am, b, s, heads, dh, 1.0 / np.sqrt(dh))
            else:
                ctx.transpose(self.qkv.view(b, s, 3 * heads, dh), self.tq, (2, 0, 1, 3))
                q, k, v = self.tq[:heads], self.tq[heads:2 * heads], self.tq[2 * heads:]
                self.qk.enqueue(q, k, self.sc, self.ep_qk)
                ctx.softmax(self.sc, self.p)
                self.pv.enqueue(self.p, v, self.a)
                ctx.transpose(self.a, self.am, (1, 2, 0, 3))
            self._linear(self.am.view(m, self.d), ly, "out", self.x1, residual=cur)
            ctx.layernorm(self.x1, self.h, ly["g2"], ly["b2"], 1e-5)
            self._linear(self.h, ly, "ff1", self.f)
            self._linear(self.f, ly, "ff2", self.x2, residual=self.x1)
            cur = self.x2
            # the next layer reads x2 as its residual and writes x1 then x2 again: x2 is consumed (by the out
            # projection's residual) before ff2 overwrites it, in stream order
        return cur

    def close(self):
        for ly in self.layers:
            for name in ("qkv", "out", "ff1", "ff2"):
                ly[name]["plan"].close()
        self.qk.close()
        self.pv.close()
