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


@pytest.mark.parametrize("batch,seq,heads", [(2, 128, 8), (3, 77, 4), (1, 1, 2), (40, 128, 8)])
def test_fused_attention_matches_unfused_checker(b200_lib, oracle_lib, batch, seq, heads):
    """Softmax(Q K^T / 8) V per head from the packed QKV tensor, against the checker with the kernel's roundings."""
    from sofie_b200.ops import Context
    import model_oracles as mo
    from sofie_b200 import encoder as be
    o = Oracle(oracle_lib)
    dh = 64
    rng = np.random.default_rng(batch * 1000 + seq)
    qkv = be.f32_to_bf16_bits((rng.standard_normal((batch, seq, 3, heads, dh)) * 1.5).astype(np.float32))
    want = bf16_bits_to_f32(mo.attention_oracle(o, qkv, batch, seq, heads, dh, 0.125)).reshape(batch, seq, heads * dh)
    ctx = Context(0)
    tq = torch.from_numpy(qkv.view(np.int16)).to(DEV).view(torch.bfloat16)
    out = torch.full((batch, seq, heads * dh), 7.0, dtype=torch.bfloat16, device=DEV)
    n0 = ctx.launches
    ctx.attention(tq, out, batch, seq, heads, dh, 0.125)
    ctx.sync()
    assert ctx.launches - n0 == 1
    got = out.float().cpu().numpy()
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 * np.abs(want) + 1e-2), f"max abs err {err.max():.4f}"
    with pytest.raises(L.SofieB200Error):
        ctx.attention(tq, out, batch, 129, heads, dh, 0.125)      # longer sequences: the caller emits the unfused graph
    with pytest.raises(L.SofieB200Error):
        ctx.attention(tq, out, batch, seq, heads, 32, 0.125)
    ctx.close()


@pytest.mark.parametrize("fused", [True, False])
def test_transformer_encoder_matches_checker(b200_lib, oracle_lib, fused):
    import model_oracles as mo
    from sofie_b200 import encoder as be
    from sofie_b200.ops import Context
    rng = np.random.default_rng(5)
    weights = be.make_weights(5, LAYERS, D_MODEL, FFN)
    x0 = be.f32_to_bf16_bits(rng.standard_normal((B * S, D_MODEL)).astype(np.float32))
    want = bf16_bits_to_f32(mo.encoder_oracle(Oracle(oracle_lib), x0, weights, B, S, D_MODEL, HEADS, fused_attention=fused))
    ctx = Context(0)
    enc = be.EncoderB200(ctx, weights, B, S, D_MODEL, HEADS, FFN, DEV, fused_attention=fused)
    launches0 = ctx.launches
    xg = torch.from_numpy(x0.view(np.int16)).to(DEV).view(torch.bfloat16)
    y = enc(xg)
    ctx.sync()
    got = y.float().cpu().numpy()
    assert ctx.launches - launches0 == LAYERS * (be.EncoderB200.LAUNCHES_PER_LAYER if fused else be.EncoderB200.LAUNCHES_PER_LAYER_UNFUSED)
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 * np.abs(want) + 1e-2), f"max abs err {err.max():.4f}"
    assert np.isfinite(got).all() and np.abs(want).max() > 1.0
    # a second call reuses every buffer and gives the same answer
    y2 = enc(xg)
    ctx.sync()
    assert torch.equal(y2.float().cpu(), torch.from_numpy(got))
    enc.close()
    ctx.close()


def test_encoder_step_replays_from_a_cuda_graph(b200_lib):
    """Every enqueue of a step is a plain kernel launch on the context's stream (tensor maps travel by value in the
    launch parameters, no allocation, no synchronisation), so a step can be captured once into a CUDA graph and
    replayed: same bits as the eager step, one graph launch instead of 14 kernel launches."""
    import model_oracles as mo
    from sofie_b200 import encoder as be
    from sofie_b200.ops import Context
    rng = np.random.default_rng(9)
    weights = be.make_weights(5, LAYERS, D_MODEL, FFN)
    x0 = be.f32_to_bf16_bits(rng.standard_normal((B * S, D_MODEL)).astype(np.float32))
    side = torch.cuda.Stream(device=DEV)
    ctx = Context(0, stream=side)
    enc = be.EncoderB200(ctx, weights, B, S, D_MODEL, HEADS, FFN, DEV, fused_attention=True)
    xg = torch.from_numpy(x0.view(np.int16)).to(DEV).view(torch.bfloat16)
    torch.cuda.synchronize()
    eager = enc(xg).clone()          # also the warm-up: tensor maps are encoded, function attributes set
    ctx.sync()
    eager = eager.cpu()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        out = enc(xg)
    out.zero_()
    n0 = ctx.launches
    graph.replay()
    torch.cuda.synchronize()
    assert ctx.launches == n0        # the replay goes through no enqueue
    assert torch.equal(out.cpu(), eager)
    xg.copy_(torch.from_numpy(be.f32_to_bf16_bits(rng.standard_normal((B * S, D_MODEL)).astype(np.float32)).view(np.int16)).to(DEV).view(torch.bfloat16))
    graph.replay()                   # new input in the same buffer
    torch.cuda.synchronize()
    replayed = out.cpu().clone()
    want = enc(xg)
    ctx.sync()
    assert torch.equal(replayed, want.cpu())
    del graph
    enc.close()
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


@pytest.mark.parametrize("fused", [True, False])
def test_encoder_matches_the_references_emitted_code(b200_lib, fused):
    """2 layers, 2 sequences, against the reference's emitted fp32 code run on the dequantised weights (fixture made by
    tests/golden/make_golden.py from oracle/_ref Encoder_C5r, whose attention is the reference's ROperator_SDPA)."""
    from pathlib import Path
    from sofie_b200 import encoder as be
    from sofie_b200.ops import Context
    fx = np.load(Path(__file__).parent / "golden" / "configs" / "Encoder_C5r.npz")
    batch, layers = int(fx["batch"]), int(fx["layers"])
    weights = be.make_weights(int(fx["seed"]), layers, D_MODEL, FFN)
    ctx = Context(0)
    enc = be.EncoderB200(ctx, weights, batch, S, D_MODEL, HEADS, FFN, DEV, fused_attention=fused)
    xg = torch.from_numpy(be.f32_to_bf16_bits(fx["x"]).view(np.int16)).to(DEV).view(torch.bfloat16)
    got = enc(xg)
    ctx.sync()
    got = got.float().cpu().numpy()
    enc.close()
    ctx.close()
    err = np.abs(got - fx["y"])
    assert np.all(err <= 2e-2 * np.abs(fx["y"]) + 1e-2), f"max abs err {err.max():.4f}"
