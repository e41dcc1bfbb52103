"""The two model configurations composed from the CPU restatement (oracle/): the checkers of the model-level GPU
tests and the "port" CPU arm of bench.py.  Test infrastructure; nothing in the package imports this file.

`encoder_oracle` rounds to bf16 at the same tensor boundaries as the device assembly (sofie_b200/encoder.py);
`convnet_oracle` runs the network of sofie_b200/convnet.py layer by layer.
"""
from __future__ import annotations

import numpy as np

from sofie_b200.convnet import CLASSES, STRIDES, Y_SCALE, conv_desc
from sofie_b200.encoder import bf16_bits_to_f32, f32_to_bf16_bits


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


def convnet_oracle(o, x: np.ndarray, weights, int8: bool) -> np.ndarray:
    """x: [n, 3, img, img] fp32 in [0,1) (fp32 variant) or int8 0..127 (int8 variant).  Returns [n, 1000] fp32 logits."""
    from sofie_b200 import lib as L
    layers, fc_w, fc_b = weights
    dt = L.I8 if int8 else L.F32
    for ly, st in zip(layers, STRIDES):
        n, c, h, w = x.shape
        d = conv_desc(n, c, h, w, ly["w"].shape[0], st, dt, dt)
        ho = (h + 2 - 3) // st + 1
        x = o.conv(x, ly["w"], d, ho, ho, ep=o.epilogue(col_scale=ly["scale"], bias=ly["bias"], act=L.ACT_RELU))
    pooled = o.global_avgpool(x, dt) if int8 else o.global_avgpool(x)
    ep = o.epilogue(alpha=float(Y_SCALE), bias=fc_b) if int8 else o.epilogue(bias=fc_b)
    return o.gemm(np.ascontiguousarray(pooled, dtype=np.float32), fc_w, x.shape[0], CLASSES, 512, L.F32, L.F32, ep=ep)
