"""Conv-net configuration (8 Conv3x3 layers 64-64-128-128-256-256-512-512, strides 1,2,1,2,1,2,1,2, each with a
folded BatchNormalization and Relu, global average pool, Gemm 512 -> 1000) at a reduced batch and image size,
in its fp32 and per-channel int8 (QLinearConv) variants, through the C ABI against the CPU restatement.
fp32: 1e-5 relative with an rms floor per layer output chain end; int8: every layer bit-exact.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import graph_runner as gr
from oracle_api import Oracle
from sofie_b200 import lib as L
from test_gpu_parity import run_conv, run_gemm, close_f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CHANNELS = [3, 64, 64, 128, 128, 256, 256, 512, 512]
STRIDES = [1, 2, 1, 2, 1, 2, 1, 2]
BATCH, IMG, CLASSES = 2, 32, 1000


def geometry(stride):
    return dict(pads=[1, 1, 1, 1], strides=[stride, stride], dil=[1, 1], group=1)


def out_hw(ctx, d):
    ho, wo = C.c_int64(), C.c_int64()
    assert ctx._lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    return ho.value, wo.value


@pytest.fixture(scope="module")
def ctx(b200_lib):
    from sofie_b200.ops import Context
    c = Context(0)
    yield c
    c.close()


def make_fp32_net(rng):
    layers = []
    for i in range(8):
        cin, cout = CHANNELS[i], CHANNELS[i + 1]
        w = (rng.standard_normal((cout, cin, 3, 3)) * np.sqrt(2.0 / (cin * 9))).astype(np.float32)   # He-normal
        gamma, beta = (rng.random(cout) + 0.5).astype(np.float32), (rng.standard_normal(cout) * 0.1).astype(np.float32)
        mean, var = (rng.standard_normal(cout) * 0.1).astype(np.float32), (rng.random(cout) + 0.5).astype(np.float32)
        scale = (gamma / np.sqrt(var + np.float32(1e-5))).astype(np.float32)      # BatchNormalization folded:
        shift = (beta - mean * scale).astype(np.float32)                           # y*scale + shift per channel
        layers.append((w, scale, shift))
    fc_w = (rng.standard_normal((512, CLASSES)) * np.sqrt(2.0 / 512)).astype(np.float32)
    fc_b = np.zeros(CLASSES, dtype=np.float32)
    return layers, fc_w, fc_b


def test_convnet_fp32(ctx, oracle_lib):
    o = Oracle(oracle_lib)
    rng = np.random.default_rng(21)
    layers, fc_w, fc_b = make_fp32_net(rng)
    x_ref = rng.random((BATCH, 3, IMG, IMG), dtype=np.float32)
    x_gpu = x_ref
    for (w, scale, shift), st in zip(layers, STRIDES):
        d = gr.conv_desc(geometry(st), x_ref.shape, w.shape)
        ho, wo = out_hw(ctx, d)
        x_ref = o.conv(x_ref, w, d, ho, wo, ep=o.epilogue(col_scale=scale, bias=shift, act=L.ACT_RELU))
        x_gpu = run_conv(ctx, np.ascontiguousarray(x_gpu), w, d, ho, wo, torch.float32, col_scale=scale, bias=shift, act=L.ACT_RELU)
        assert close_f32(x_gpu, x_ref, rel=2e-5), f"stride {st}: {np.abs(x_gpu - x_ref).max():.3g}"
    pooled_ref = o.global_avgpool(x_ref)
    tp = torch.empty((BATCH, 512), dtype=torch.float32, device=DEV)
    ctx.global_avgpool(torch.from_numpy(x_gpu).to(DEV), tp)
    ctx.sync()
    pooled_gpu = tp.cpu().numpy()
    want = o.gemm(pooled_ref, fc_w, BATCH, CLASSES, 512, L.F32, L.F32, ep=o.epilogue(bias=fc_b))
    got = run_gemm(ctx, pooled_gpu, fc_w, BATCH, CLASSES, 512, torch.float32, torch.float32, bias=fc_b).cpu().numpy()
    assert close_f32(got, want, rel=5e-5), np.abs(got - want).max()


def test_convnet_int8_every_layer_bit_exact(ctx, oracle_lib):
    o = Oracle(oracle_lib)
    rng = np.random.default_rng(22)
    x = rng.integers(0, 128, size=(BATCH, 3, IMG, IMG), dtype=np.int8)   # quantised U(0,1) input, scale 1/127
    x_gpu = x
    a_scale = np.float32(1.0 / 127.0)
    for i, st in enumerate(STRIDES):
        cin, cout = CHANNELS[i], CHANNELS[i + 1]
        wf = rng.standard_normal((cout, cin, 3, 3)) * np.sqrt(2.0 / (cin * 9))
        w_scale = (np.abs(wf).reshape(cout, -1).max(axis=1) / 127.0).astype(np.float32)          # per output channel
        w = np.clip(np.rint(wf / w_scale[:, None, None, None]), -127, 127).astype(np.int8)
        y_scale = np.float32(0.05)
        mult = (a_scale * w_scale / y_scale).astype(np.float32)                                 # fp32, left to right
        bias = rng.integers(-2000, 2000, size=cout, dtype=np.int32)                              # folded BN shift at scale a*w[c]
        d = gr.conv_desc(geometry(st), x.shape, w.shape, L.I8, L.I8)
        ho, wo = out_hw(ctx, d)
        x = o.conv(x, w, d, ho, wo, ep=o.epilogue(col_scale=mult, bias=bias, act=L.ACT_RELU))
        x_gpu = run_conv(ctx, np.ascontiguousarray(x_gpu), w, d, ho, wo, torch.int8, col_scale=mult, bias=bias, act=L.ACT_RELU)
        assert np.array_equal(x_gpu, x), f"layer {i}: {(x_gpu != x).sum()} of {x.size} differ"
        assert x.max() > 0   # the layer is not dead
        a_scale = y_scale
    pooled = o.global_avgpool(x, L.I8)
    tp = torch.empty((BATCH, 512), dtype=torch.float32, device=DEV)
    ctx.global_avgpool(torch.from_numpy(x_gpu).to(DEV), tp)
    ctx.sync()
    assert np.abs(tp.cpu().numpy() - pooled).max() <= 1e-5 * max(1.0, np.abs(pooled).max())


@pytest.mark.parametrize("channels_last", [True, False])
@pytest.mark.parametrize("int8", [False, True])
def test_benchmark_network_object_matches_checker(ctx, oracle_lib, int8, channels_last):
    """sofie_b200.convnet.ConvNetB200 (plans and buffers created once, as the benchmark runs it) against the checker."""
    import model_oracles as mo
    from sofie_b200 import convnet as bc
    o = Oracle(oracle_lib)
    rng = np.random.default_rng(5)
    weights = bc.make_weights(5, int8)
    x = rng.random((3, 3, 48, 48), dtype=np.float32)
    if int8:
        x = np.clip(np.rint(x * 127.0), 0, 127).astype(np.int8)
    want = mo.convnet_oracle(o, x, weights, int8)
    net = bc.ConvNetB200(ctx, weights, 3, 48, int8, DEV, channels_last=channels_last)
    n0 = ctx.launches
    for _ in range(2):   # the second call reuses every buffer
        got = net(torch.from_numpy(x).to(DEV))
        ctx.sync()
    assert ctx.launches - n0 == 2 * net.launches
    assert net.kernels[0] == "direct"
    if channels_last and int8:   # conv -> conv on channels-last int8 tensors: no unfolded copy
        assert net.kernels[1:] == ["umma_im2col"] * 7 and net.launches == 1 + 7 + 2
    got = got.cpu().numpy()
    assert close_f32(got, want, rel=1e-4 if not int8 else 1e-5), np.abs(got - want).max()
    net.close()


@pytest.mark.parametrize("int8", [True, False])
def test_full_size_layer_two_data_paths_agree(ctx, int8, monkeypatch):
    """Layer 3 of the benchmark network at its full size (256 images of 112 x 112 x 64 -> 128 channels, 473 GFLOP), too
    large for the CPU checker: the implicit convolution (input read in place by im2col-mode TMA loads) against the
    unfold + contraction path, which shares nothing with it up to the accumulator.  int8: every output bit for bit.
    fp32: TF32 pairs read in place against the split unfold; the same three products, summed in different chunks."""
    import model_oracles as mo
    from sofie_b200 import convnet as bc
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    n, c, hw, k = 256, 64, 112, 128
    gen = torch.Generator(device=DEV).manual_seed(3)
    if int8:
        x = torch.randint(-127, 128, (n, hw, hw, c), dtype=torch.int8, device=DEV, generator=gen)
        w = torch.randint(-127, 128, (k, c, 3, 3), dtype=torch.int8, device=DEV, generator=gen)
        ep_kw = dict(col_scale=torch.rand(k, device=DEV, generator=gen) * 1e-4 + 2e-5,
                     bias=torch.randint(-20000, 20000, (k,), dtype=torch.int32, device=DEV, generator=gen), act=L.ACT_RELU)
        code, dt = L.I8, torch.int8
    else:
        x = torch.rand((n, hw, hw, c), device=DEV, generator=gen)
        w = torch.randn((k, c, 3, 3), device=DEV, generator=gen) * 0.05
        ep_kw = dict(col_scale=torch.rand(k, device=DEV, generator=gen) + 0.5, bias=torch.randn(k, device=DEV, generator=gen), act=L.ACT_RELU)
        code, dt = L.F32, torch.float32

    def run(xl, xin, kernel, flags=0):
        d = bc.conv_desc(n, c, hw, hw, k, 1, code, code, xl, 1, flags)
        h = C.c_void_p()
        L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), w.data_ptr(), C.byref(h)), "conv_plan_create")
        assert lib.sofie_b200_conv_plan_kernel(h).decode() == kernel
        ws = torch.empty(max(16, lib.sofie_b200_conv_workspace_bytes(h)), dtype=torch.uint8, device=DEV)
        y = torch.empty((n, hw, hw, k), dtype=dt, device=DEV)
        ep, keep = make_epilogue(**ep_kw)
        L.check(lib.sofie_b200_conv_enqueue(h, xin.data_ptr(), y.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
        ctx.sync()
        lib.sofie_b200_conv_plan_destroy(h)
        del ws
        return y

    if int8:
        a = run(1, x, "umma_im2col_x2")   # 64-byte pixels, unit stride: read as pixel pairs, even and odd output columns apart
        b = run(1, x, "umma", flags=L.CONV_UNFOLD)
        assert torch.equal(a, b)
        assert int((a != 0).sum()) > a.numel() // 10   # not a dead layer
    else:
        # the pairs, made on the device with the library's rounding (ties away from zero on the 13 dropped bits)
        bits = x.view(torch.int32)
        hi = ((bits + 0x1000) & ~0x1FFF).view(torch.float32)
        rem = (x - hi).view(torch.int32)
        lo = ((rem + 0x1000) & ~0x1FFF).view(torch.float32)
        a = run(2, torch.cat([hi, lo], dim=3).contiguous(), "umma3x_im2col")
        b = run(1, x, "umma3x")
        err = (a - b).abs().max().item()
        scale = b.abs().max().item()
        assert err <= 2e-6 * scale, (err, scale)


def test_network_matches_the_references_emitted_code(ctx):
    """The fp32 network on 2 images of 32 x 32 against what the reference's own emitted CPU code computed (fixture made by
    tests/golden/make_golden.py from oracle/_ref ConvNet_C4r; same weights through the reproducible generator)."""
    from pathlib import Path
    from sofie_b200 import convnet as bc
    fx = np.load(Path(__file__).parent / "golden" / "configs" / "ConvNet_C4r.npz")
    weights = bc.make_weights(int(fx["seed"]), False)
    for channels_last in (True, False):
        net = bc.ConvNetB200(ctx, weights, 2, 32, False, DEV, channels_last=channels_last)
        got = net(torch.from_numpy(fx["x"]).to(DEV))
        ctx.sync()
        got = got.cpu().numpy()
        net.close()
        assert close_f32(got, fx["y"], rel=1e-5), (channels_last, np.abs(got - fx["y"]).max())
