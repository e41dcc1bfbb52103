"""The transformer-encoder configuration on libsofie_b200: weights, work count and the device assembly.

Pre-LayerNorm encoder layers: LN -> QKV projection -> per-head Softmax(Q K^T / sqrt(d_h)) V -> output projection
+ residual -> LN -> FFN (Gelu) -> + residual.  Activations are bf16; the four projection weights of a layer are
int8 with one fp32 scale per output channel, converted to bf16 once at construction, the scale applied as the
column scale of the contraction's epilogue together with bias, Gelu and the residual add.  Every operator is one
call of the C ABI (sofie_b200/ops.py); all buffers are allocated once, a step allocates nothing.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns of an fp32 array (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def make_weights(seed: int, layers: int, d_model: int, ffn: int):
    """int8 per-output-channel weights ~N(0, 0.02) with scale = absmax/127, fp32 biases ~N(0, 0.02), LN gamma 1 / beta 0,
    from the reproducible generator of sofie_b200/synth.py (oracle/ref_emit.cxx builds the reference's fp32 model from the
    same draws, with the weights dequantised: float(q) * scale)."""
    from . import synth

    def qlinear(sw, sb, n_out, n_in):
        w = synth.normal_f32(sw, (n_out, n_in), 0.02)
        scale = (np.abs(w).max(axis=1) / np.float32(127.0)).astype(np.float32)
        q = np.clip(np.rint(w / scale[:, None]), -127, 127).astype(np.int8)
        return q, scale, synth.normal_f32(sb, n_out, 0.02)
    out = []
    for l in range(layers):
        ts = lambda j: synth.tensor_seed(seed, 10 * l + j)
        out.append({"qkv": qlinear(ts(0), ts(1), 3 * d_model, d_model), "out": qlinear(ts(2), ts(3), d_model, d_model),
                    "ff1": qlinear(ts(4), ts(5), ffn, d_model), "ff2": qlinear(ts(6), ts(7), d_model, ffn),
                    "g1": np.ones(d_model, np.float32), "b1": np.zeros(d_model, np.float32),
                    "g2": np.ones(d_model, np.float32), "b2": np.zeros(d_model, np.float32)})
    return out


def flops_per_sample(layers: int, seq: int, d_model: int, ffn: int) -> float:
    proj = 2.0 * seq * d_model * (3 * d_model + d_model + 2 * ffn)
    attn = 2.0 * 2.0 * seq * seq * d_model
    return layers * (proj + attn)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


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


def onnx_model(weights, batch: int, seq: int, d_model: int, heads: int):
    """The encoder as an ONNX graph for the C++ generator (sofie_b200/onnx_min.save): bf16 activations [batch*seq, d_model];
    every projection is DequantizeLinear(int8 weight [out, in], per-output-channel scale) -> Gemm(transB = 1) with an fp32
    bias; attention is Split -> Reshape -> ScaledDotProductAttention(num_heads) on the folded [batch, seq, d_model] layout.
    Returns (nodes, initializers, inputs, outputs, input_types)."""
    m = batch * seq
    init = {"shape_bsd": np.array([batch, seq, d_model], dtype=np.int64), "shape_md": np.array([m, d_model], dtype=np.int64)}
    nodes = []

    def linear(x, name, l, out):
        wq, scale, bias = weights[l][name]
        init[f"{name}_q_{l}"], init[f"{name}_s_{l}"], init[f"{name}_b_{l}"] = wq, scale, bias
        nodes.append({"op": "DequantizeLinear", "in": [f"{name}_q_{l}", f"{name}_s_{l}"], "out": [f"{name}_w_{l}"], "attrs": {"axis": 0}})
        nodes.append({"op": "Gemm", "in": [x, f"{name}_w_{l}", f"{name}_b_{l}"], "out": [out], "attrs": {"transB": 1}})

    x = "X"
    for l, ly in enumerate(weights):
        for k in ("g1", "b1", "g2", "b2"):
            init[f"{k}_{l}"] = ly[k]
        nodes.append({"op": "LayerNormalization", "in": [x, f"g1_{l}", f"b1_{l}"], "out": [f"h1_{l}"], "attrs": {"axis": -1, "epsilon": 1e-5}})
        linear(f"h1_{l}", "qkv", l, f"qkv_{l}")
        nodes.append({"op": "Split", "in": [f"qkv_{l}"], "out": [f"q_{l}", f"k_{l}", f"v_{l}"], "attrs": {"axis": 1}})
        for t in "qkv":
            nodes.append({"op": "Reshape", "in": [f"{t}_{l}", "shape_bsd"], "out": [f"{t}3_{l}"], "attrs": {}})
        nodes.append({"op": "ScaledDotProductAttention", "in": [f"q3_{l}", f"k3_{l}", f"v3_{l}"], "out": [f"att3_{l}"], "attrs": {"num_heads": heads}})
        nodes.append({"op": "Reshape", "in": [f"att3_{l}", "shape_md"], "out": [f"att_{l}"], "attrs": {}})
        linear(f"att_{l}", "out", l, f"proj_{l}")
        nodes.append({"op": "Add", "in": [f"proj_{l}", x], "out": [f"x1_{l}"], "attrs": {}})
        nodes.append({"op": "LayerNormalization", "in": [f"x1_{l}", f"g2_{l}", f"b2_{l}"], "out": [f"h2_{l}"], "attrs": {"axis": -1, "epsilon": 1e-5}})
        linear(f"h2_{l}", "ff1", l, f"f_{l}")
        nodes.append({"op": "Gelu", "in": [f"f_{l}"], "out": [f"g_{l}"], "attrs": {}})
        linear(f"g_{l}", "ff2", l, f"ff_{l}")
        out = "Y" if l + 1 == len(weights) else f"x2_{l}"
        nodes.append({"op": "Add", "in": [f"ff_{l}", f"x1_{l}"], "out": [out], "attrs": {}})
        x = out
    return nodes, init, [("X", [m, d_model])], ["Y"], {"X": 16}
