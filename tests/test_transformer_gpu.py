"""Transformer-encoder configuration (pre-LayerNorm, 8 heads, d_model 512, FFN 2048, Gelu, seq 128) at a
reduced batch and depth: bf16 activations, int8 per-output-channel weights whose dequantisation is the
column scale of the GEMM epilogue, Softmax attention.  Every operator runs through the C ABI; the checker
composes the same graph from the CPU restatement, rounding to bf16 at the same tensor boundaries.
Bar: 2e-2 relative + 1e-2 absolute on the final activations.
"""
import numpy as np
import pytest
import torch

from oracle_api import Oracle, bf16_bits_to_f32
from sofie_b200 import lib as L

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
B, S, D_MODEL, HEADS, FFN, LAYERS = 2, 128, 512, 8, 2048, 2
DH = D_MODEL // HEADS


def f32_to_bf16_bits(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def make_weights(rng):
    def qlinear(n_out, n_in):
        w = rng.standard_normal((n_out, n_in)).astype(np.float32) * 0.02
        scale = (np.abs(w).max(axis=1) / 127.0).astype(np.float32)          # per output channel
        q = np.clip(np.rint(w / scale[:, None]), -127, 127).astype(np.int8)
        return q, scale, (rng.standard_normal(n_out) * 0.02).astype(np.float32)
    layers = []
    for _ in range(LAYERS):
        layers.append({"qkv": qlinear(3 * D_MODEL, D_MODEL), "out": qlinear(D_MODEL, D_MODEL), "ff1": qlinear(FFN, D_MODEL),
                       "ff2": qlinear(D_MODEL, FFN), "g1": np.ones(D_MODEL, np.float32), "b1": np.zeros(D_MODEL, np.float32),
                       "g2": np.ones(D_MODEL, np.float32), "b2": np.zeros(D_MODEL, np.float32)})
    return layers


# ---- checker: numpy + oracle/libsofie_oracle.so on bf16 bit patterns -----------------------------------
def encoder_oracle(o: Oracle, x, layers):
    M = B * S
    def linear(a, wq, scale, bias, act=L.ACT_NONE, residual=None):
        w = f32_to_bf16_bits(wq.astype(np.float32))  # int8 values are exact in bf16
        ep = o.epilogue(col_scale=scale, bias=bias, act=act, residual=residual, residual_dtype=L.BF16)
        return o.gemm(a, w, M, wq.shape[0], wq.shape[1], L.BF16, L.BF16, False, True, ep=ep)
    for ly in layers:
        h = o.layernorm(x, ly["g1"], ly["b1"], 1e-5, L.BF16)
        qkv = linear(h, *ly["qkv"])
        t = np.ascontiguousarray(qkv.reshape(B, S, 3 * HEADS, DH).transpose(2, 0, 1, 3))   # [3H, B, S, DH]
        q, k, v = (np.ascontiguousarray(t[i * HEADS:(i + 1) * HEADS]).reshape(HEADS * B, S, DH) for i in range(3))
        sc = o.gemm(q, k, S, S, DH, L.BF16, L.BF16, False, True, batch=HEADS * B, ep=o.epilogue(alpha=1.0 / 8.0))
        p = o.softmax(sc.reshape(-1, S), L.BF16).reshape(HEADS * B, S, S)
        a = o.gemm(p, v, S, DH, S, L.BF16, L.BF16, False, False, batch=HEADS * B)
        a = np.ascontiguousarray(a.reshape(HEADS, B, S, DH).transpose(1, 2, 0, 3)).reshape(M, D_MODEL)
        x = linear(a, *ly["out"], residual=x)
        h = o.layernorm(x, ly["g2"], ly["b2"], 1e-5, L.BF16)
        f = linear(h, *ly["ff1"], act=L.ACT_GELU_ERF)
        x = linear(f, *ly["ff2"], residual=x)
    return x


# ---- product path: libsofie_b200 through the C ABI ---------------------------------------------------------
class EncoderB200:
    def __init__(self, ctx, layers):
        from sofie_b200.ops import GemmPlan
        self.ctx, t = ctx, torch
        M = B * S
        self.layers = []
        for ly in layers:
            d = {}
            for name in ("qkv", "out", "ff1", "ff2"):
                wq, scale, bias = ly[name]
                w8 = t.from_numpy(wq).to(DEV)
                wb = t.empty(wq.shape, dtype=t.bfloat16, device=DEV)
                ctx.convert(w8, wb)   # weights become bf16 once, at construction; the scale stays in the epilogue
                d[name] = (wb, t.from_numpy(scale).to(DEV), t.from_numpy(bias).to(DEV),
                           GemmPlan(ctx, M, wq.shape[0], wq.shape[1], t.bfloat16, t.bfloat16, trans_b=True))
            for name in ("g1", "b1", "g2", "b2"):
                d[name] = t.from_numpy(ly[name]).to(DEV)
            self.layers.append(d)
        hb = HEADS * B
        self.qk = GemmPlan(ctx, S, S, DH, t.bfloat16, t.bfloat16, trans_b=True, batch=hb, stride_a=S * DH, stride_b=S * DH, stride_y=S * S)
        self.pv = GemmPlan(ctx, S, DH, S, t.bfloat16, t.bfloat16, trans_b=False, batch=hb, stride_a=S * S, stride_b=S * DH, stride_y=S * DH)
        assert self.qk.kernel == "umma" and self.pv.kernel == "umma"

    def linear(self, a, layer, name, act=L.ACT_NONE, residual=None):
        from sofie_b200.ops import make_epilogue
        w, scale, bias, plan = layer[name]
        y = torch.empty((a.shape[0], w.shape[0]), dtype=torch.bfloat16, device=DEV)
        ep, keep = make_epilogue(col_scale=scale, bias=bias, act=act, residual=residual)
        plan.enqueue(a, w, y, ep)
        assert plan.kernel == "umma"
        return y

    def __call__(self, x):
        from sofie_b200.ops import make_epilogue
        ctx, t = self.ctx, torch
        M = B * S
        for ly in self.layers:
            h = t.empty_like(x)
            ctx.layernorm(x, h, ly["g1"], ly["b1"], 1e-5)
            qkv = self.linear(h, ly, "qkv")
            tq = t.empty((3 * HEADS, B, S, DH), dtype=t.bfloat16, device=DEV)
            ctx.transpose(qkv.view(B, S, 3 * HEADS, DH), tq, (2, 0, 1, 3))
            q, k, v = tq[:HEADS], tq[HEADS:2 * HEADS], tq[2 * HEADS:]
            sc = t.empty((HEADS * B, S, S), dtype=t.bfloat16, device=DEV)
            ep, _ = make_epilogue(alpha=1.0 / 8.0)
            self.qk.enqueue(q, k, sc, ep)
            p = t.empty_like(sc)
            ctx.softmax(sc, p)
            a = t.empty((HEADS, B, S, DH), dtype=t.bfloat16, device=DEV)
            self.pv.enqueue(p, v, a)
            am = t.empty((B, S, HEADS, DH), dtype=t.bfloat16, device=DEV)
            ctx.transpose(a, am, (1, 2, 0, 3))
            x = self.linear(am.view(M, D_MODEL), ly, "out", residual=x)
            h2 = t.empty_like(x)
            ctx.layernorm(x, h2, ly["g2"], ly["b2"], 1e-5)
            f = self.linear(h2, ly, "ff1", act=L.ACT_GELU_ERF)
            x = self.linear(f, ly, "ff2", residual=x)
        ctx.sync()
        return x


def test_transformer_encoder_matches_checker(b200_lib, oracle_lib):
    from sofie_b200.ops import Context
    rng = np.random.default_rng(5)
    layers = make_weights(rng)
    x0 = f32_to_bf16_bits(rng.standard_normal((B * S, D_MODEL)).astype(np.float32))
    want = bf16_bits_to_f32(encoder_oracle(Oracle(oracle_lib), x0, layers))
    ctx = Context(0)
    enc = EncoderB200(ctx, layers)
    launches0 = ctx.launches
    xg = torch.from_numpy(x0.view(np.int16)).to(DEV).view(torch.bfloat16)
    got = enc(xg).float().cpu().numpy()
    assert ctx.launches - launches0 == LAYERS * 11   # 4 projections, 2 attention GEMMs, 2 LayerNorms, 1 Softmax, 2 transposes
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 * np.abs(want) + 1e-2), f"max abs err {err.max():.4f}"
    assert np.isfinite(got).all() and np.abs(want).max() > 1.0
    ctx.close()


@pytest.mark.parametrize("shape,perm", [((2, 128, 24, 64), (2, 0, 1, 3)), ((8, 2, 128, 64), (1, 2, 0, 3)), ((5, 7, 9), (2, 0, 1)),
                                        ((33, 65), (1, 0)), ((3, 4, 5, 6), (3, 2, 1, 0))])
def test_transpose(b200_lib, shape, perm):
    from sofie_b200.ops import Context
    ctx = Context(0)
    for dt in (torch.bfloat16, torch.float32, torch.int8):
        x = (torch.randn(shape, device=DEV) * 50).to(dt)
        y = torch.empty([shape[p] for p in perm], dtype=dt, device=DEV)
        ctx.transpose(x, y, perm)
        ctx.sync()
        assert torch.equal(y, x.permute(*perm).contiguous())
    ctx.close()
