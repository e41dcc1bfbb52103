"""Parity of the CUDA path (through the C ABI) with the CPU checker and the golden fixtures.

Bars: bit-exact for int8 paths; |got-want| <= 1e-5*max(|want|, rms) for fp32; 2e-2 relative +
1e-2 absolute for bf16 / FP8.  Everything here needs a B200.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

import graph_runner as gr
from oracle_api import Oracle, bf16_bits_to_f32
from sofie_b200 import lib as L

pytestmark = pytest.mark.gpu
GOLDEN = sorted(p.stem for p in (Path(__file__).parent / "golden").glob("*.npz"))
DEV = "cuda:0"


def close_f32(got, want, rel=1e-5):
    floor = float(np.sqrt(np.mean(np.square(want)))) if want.size else 0.0
    return bool(np.all(np.abs(got - want) <= rel * np.maximum(np.abs(want), floor) + 1e-30))


def close_lowp(got, want):
    return bool(np.all(np.abs(got - want) <= 2e-2 * np.abs(want) + 1e-2))


@pytest.fixture(scope="module")
def ctx(b200_lib):
    from sofie_b200.ops import Context
    c = Context(0)
    yield c
    c.close()


@pytest.fixture(scope="module")
def oracle(oracle_lib):
    return Oracle(oracle_lib)


@pytest.fixture(scope="module")
def backend(b200_lib):
    return gr.B200Backend()


# ---- the reference's own test models --------------------------------------------------------
@pytest.mark.parametrize("name", GOLDEN)
def test_golden_models(name, backend):
    fx = gr.load_fixture(name)
    for tag in ("A", "B"):
        if f"out{tag}" not in fx:
            continue
        ins = [fx[k] for k in sorted(fx) if k.startswith(f"in{tag}")]
        got = gr.run_graph(fx, ins, backend)
        want = fx[f"out{tag}"]
        assert got.shape == want.shape
        assert close_f32(got, want), f"{name}/{tag}: max abs diff {np.abs(got - want).max():.3g}"
    if "expected" in fx:
        ins = [fx[k] for k in sorted(fx) if k.startswith("inA")]
        assert np.abs(gr.run_graph(fx, ins, backend) - fx["expected"]).max() <= 2e-4


# ---- int8 QLinearMatMul: bit-exact --------------------------------------------------------------
def run_gemm(ctx, a, b, M, N, K, in_dt, out_dt, trans_a=False, trans_b=False, batch=1, precise=True, expect=None, flags=0, **ep_kw):
    from sofie_b200.ops import GemmPlan, make_epilogue
    ta, tb = torch.from_numpy(a).to(DEV).view(in_dt), torch.from_numpy(b).to(DEV).view(in_dt)
    y = torch.zeros((batch, M, N) if batch > 1 else (M, N), dtype=out_dt, device=DEV)
    plan = GemmPlan(ctx, M, N, K, in_dt, out_dt, trans_a=trans_a, trans_b=trans_b, batch=batch,
                    stride_a=(M * K if batch > 1 else 0), stride_b=(K * N if batch > 1 else 0), stride_y=(M * N if batch > 1 else 0),
                    precise=precise, flags=flags)
    dev_kw = {k: (torch.from_numpy(v).to(DEV) if isinstance(v, np.ndarray) else v) for k, v in ep_kw.items()}
    ep, keep = make_epilogue(**dev_kw)
    plan.enqueue(ta, tb, y, ep)
    ctx.sync()
    if expect is not None:
        assert plan.kernel == expect, plan.kernel
    plan.close()
    return y


MULT = float(np.float32(np.float32(0.02) * np.float32(0.01)) / np.float32(0.5))


@pytest.mark.parametrize("M,N,K,ta,tb,kernel", [
    (256, 384, 512, False, False, "umma"), (256, 384, 512, False, True, "umma"), (256, 384, 512, True, False, "umma"),
    (1000, 700, 400, False, True, "umma"), (1000, 704, 400, False, False, "umma"), (1, 1, 16, False, True, "umma"),
    (130, 50, 33, False, True, "simt"), (7, 300, 1, False, False, "simt"), (129, 257, 4096, False, False, "simt"), (129, 272, 4096, False, False, "umma"),
])
def test_qlinear_matmul_bit_exact(ctx, oracle, M, N, K, ta, tb, kernel):
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    a = rng.integers(-127, 128, size=(K, M) if ta else (M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(N, K) if tb else (K, N), dtype=np.int8)
    want = oracle.gemm(a, b, M, N, K, L.I8, L.I8, ta, tb, ep=oracle.epilogue(alpha=MULT))
    got = run_gemm(ctx, a, b, M, N, K, torch.int8, torch.int8, ta, tb, alpha=MULT, expect=kernel).cpu().numpy()
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} differ"
    want32 = oracle.gemm(a, b, M, N, K, L.I8, L.I32, ta, tb)
    got32 = run_gemm(ctx, a, b, M, N, K, torch.int8, torch.int32, ta, tb).cpu().numpy()
    assert np.array_equal(got32, want32)


def test_qlinear_per_channel_bias_relu_zero_point(ctx, oracle):
    M, N, K = 384, 320, 640
    rng = np.random.default_rng(11)
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    cs = (rng.random(N, dtype=np.float32) * 1e-3 + 1e-4).astype(np.float32)
    bias = rng.integers(-50000, 50000, size=N, dtype=np.int32)
    for out_dt, odt, zp in ((torch.int8, L.I8, -7), (torch.uint8, L.U8, 128)):
        want = oracle.gemm(a, b, M, N, K, L.I8, odt, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU, out_zero_point=zp))
        got = run_gemm(ctx, a, b, M, N, K, torch.int8, out_dt, col_scale=cs, bias=bias, act=L.ACT_RELU, out_zero_point=zp).cpu().numpy()
        assert np.array_equal(got, want)


def test_qlinear_batched_and_shared_weight(ctx, oracle):
    from sofie_b200.ops import GemmPlan, make_epilogue
    B, M, N, K = 5, 200, 136, 256
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, size=(B, M, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    want = oracle.gemm(a, w, M, N, K, L.I8, L.I32, False, True, batch=B, stride_b=0)
    ta, tw = torch.from_numpy(a).to(DEV), torch.from_numpy(w).to(DEV)
    y = torch.zeros((B, M, N), dtype=torch.int32, device=DEV)
    plan = GemmPlan(ctx, M, N, K, torch.int8, torch.int32, trans_b=True, batch=B, stride_a=M * K, stride_b=0, stride_y=M * N)
    plan.enqueue(ta, tw, y)
    ctx.sync()
    assert np.array_equal(y.cpu().numpy(), want)


def test_empty_and_invalid(ctx):
    from sofie_b200.ops import GemmPlan
    y = torch.zeros((0, 8), dtype=torch.int8, device=DEV)
    a = torch.zeros((0, 16), dtype=torch.int8, device=DEV)
    b = torch.zeros((16, 8), dtype=torch.int8, device=DEV)
    plan = GemmPlan(ctx, 0, 8, 16, torch.int8, torch.int8)
    plan.enqueue(a, b, y)  # empty output: nothing is launched
    ctx.sync()
    with pytest.raises(L.SofieB200Error):
        GemmPlan(ctx, 8, 8, 8, torch.bfloat16, torch.int32)  # int32 output needs int8 operands
    with pytest.raises(L.SofieB200Error):
        GemmPlan(ctx, 8, 8, 8, torch.int8, torch.int8, lda=4)  # pitch smaller than the row


def test_qlinear_matmul_4096_sampled_rows(ctx, oracle):
    """The benchmark configuration at full size: 96 sampled rows of the output, bit for bit."""
    n = 4096
    rng = np.random.default_rng(1)
    a = rng.integers(-127, 128, size=(n, n), dtype=np.int8)
    b = rng.integers(-127, 128, size=(n, n), dtype=np.int8)
    got = run_gemm(ctx, a, b, n, n, n, torch.int8, torch.int8, alpha=MULT, expect="umma").cpu().numpy()
    rows = np.concatenate([np.arange(32), rng.choice(np.arange(32, n), size=64, replace=False)])
    want = oracle.gemm(np.ascontiguousarray(a[rows]), b, len(rows), n, n, L.I8, L.I8, ep=oracle.epilogue(alpha=MULT))
    assert np.array_equal(got[rows], want)
    # size-independent property: the int32 product is linear in A
    got32 = run_gemm(ctx, a, b, n, n, n, torch.int8, torch.int32).cpu().numpy().astype(np.int64)
    a2 = (a.astype(np.int16) // 2).astype(np.int8)
    r = (a.astype(np.int16) - 2 * a2.astype(np.int16)).astype(np.int8)
    g2 = run_gemm(ctx, a2, b, n, n, n, torch.int8, torch.int32).cpu().numpy().astype(np.int64)
    gr_ = run_gemm(ctx, r, b, n, n, n, torch.int8, torch.int32).cpu().numpy().astype(np.int64)
    assert np.array_equal(got32, 2 * g2 + gr_)


@pytest.mark.parametrize("M,tb", [(37500, True), (37786, False)])
def test_tall_tiles_with_ragged_last_tile(ctx, oracle, M, tb):
    """Long K, one tile across N and more row tiles than SMs: the plan takes 256-row tiles (two 128-row halves sharing every
    B slice).  37500 rows leave a last tile whose lower half does not exist, 37786 one whose lower half has 26 rows.  The rows
    of the last tiles and a random sample of the rest, bit for bit, with a per-channel epilogue."""
    N, K = 256, 4096
    rng = np.random.default_rng(M)
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(N, K) if tb else (K, N), dtype=np.int8)
    cs = (rng.random(N, dtype=np.float32) * 2e-5 + 1e-5).astype(np.float32)
    bias = rng.integers(-50000, 50000, size=N, dtype=np.int32)
    got = run_gemm(ctx, a, b, M, N, K, torch.int8, torch.int8, False, tb, col_scale=cs, bias=bias, act=L.ACT_RELU, expect="umma").cpu().numpy()
    rows = np.concatenate([np.arange(M - 420, M), rng.choice(M - 420, size=60, replace=False)])
    want = oracle.gemm(np.ascontiguousarray(a[rows]), b, len(rows), N, K, L.I8, L.I8, False, tb,
                       ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU))
    assert np.array_equal(got[rows], want), f"{(got[rows] != want).sum()} of {want.size} differ"


@pytest.mark.parametrize("N,tb", [(4096, True), (4032, True), (4000, False)])
def test_tall_tiles_over_a_wide_result(ctx, oracle, N, tb):
    """4096 x N x 4096: 16 bands of tall tiles (256 rows) and 16 tiles across N -- more tiles than SMs, so the CTAs take a
    second tile; N = 4032 and 4000 leave a narrower last tile (4000 with B stored [K, N]: the plan's K-major copy).  Rows
    from every band, all columns, bit for bit."""
    M, K = 4096, 4096
    rng = np.random.default_rng(N)
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(N, K) if tb else (K, N), dtype=np.int8)
    cs = (rng.random(N, dtype=np.float32) * 2e-5 + 1e-5).astype(np.float32)
    bias = rng.integers(-50000, 50000, size=N, dtype=np.int32)
    got = run_gemm(ctx, a, b, M, N, K, torch.int8, torch.int8, False, tb, col_scale=cs, bias=bias, expect="umma",
                   flags=0 if tb else L.GEMM_B_CONSTANT).cpu().numpy()
    rows = np.sort(np.concatenate([np.arange(16) * 256 + rng.integers(0, 256, size=16), rng.choice(M, size=48, replace=False), [0, 127, 128, 255, M - 1]]))
    want = oracle.gemm(np.ascontiguousarray(a[rows]), b, len(rows), N, K, L.I8, L.I8, False, tb, ep=oracle.epilogue(col_scale=cs, bias=bias))
    assert np.array_equal(got[rows], want), f"{(got[rows] != want).sum()} of {want.size} differ"


@pytest.mark.parametrize("M,N,K", [(20000, 768, 1024), (56832, 1536, 512)])
def test_short_k_many_bands_int8(ctx, oracle, M, N, K):
    """Short K, several tiles across N, more 128-row bands than SMs (the shape class of the encoder's projections), int8:
    rows of the first, a middle and the last bands (20000 rows: the last band has 32) and a random sample, all columns, bit
    for bit, per-channel epilogue."""
    rng = np.random.default_rng(M + K)
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    cs = (rng.random(N, dtype=np.float32) * 4e-5 + 1e-5).astype(np.float32)
    bias = rng.integers(-50000, 50000, size=N, dtype=np.int32)
    got = run_gemm(ctx, a, b, M, N, K, torch.int8, torch.int8, False, True, col_scale=cs, bias=bias, act=L.ACT_RELU, expect="umma").cpu().numpy()
    rows = np.unique(np.concatenate([np.arange(0, 130), np.arange(148 * 128 - 3, 148 * 128 + 131), np.arange(M - 200, M), rng.choice(M, size=100, replace=False)]))
    rows = rows[rows < M]
    want = oracle.gemm(np.ascontiguousarray(a[rows]), b, len(rows), N, K, L.I8, L.I8, False, True, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU))
    assert np.array_equal(got[rows], want), f"{(got[rows] != want).sum()} of {want.size} differ"


def test_short_k_many_bands_bf16_with_residual(ctx, oracle):
    """The encoder's output projection shape class (bf16, K = 512, bias, residual add) against an fp32 product of the same
    bf16 operands."""
    M, N, K = 24000, 512, 512
    rng = np.random.default_rng(5)
    a = torch.from_numpy((rng.standard_normal((M, K)) * 0.5).astype(np.float32)).to(torch.bfloat16)
    b = torch.from_numpy((rng.standard_normal((N, K)) * 0.05).astype(np.float32)).to(torch.bfloat16)
    res = torch.from_numpy((rng.standard_normal((M, N)) * 0.5).astype(np.float32)).to(torch.bfloat16)
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    an, bn = a.view(torch.int16).numpy(), b.view(torch.int16).numpy()
    got = run_gemm(ctx, an, bn, M, N, K, torch.bfloat16, torch.bfloat16, False, True, bias=bias, residual=res.to(DEV), ldr=N, expect="umma").float().cpu().numpy()
    want = a.float().numpy() @ b.float().numpy().T + bias + res.float().numpy()
    assert close_lowp(got, want), np.abs(got - want).max()


# ---- FP8 / bf16 / fp32 contractions -------------------------------------------------------------
def fp8_operands(rng, M, N, K, tb):
    a = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32))
    b = torch.from_numpy(rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32))
    sa = (a.abs().amax(dim=1) / 448.0)
    sb = (b.abs().amax(dim=1 if tb else 0) / 448.0)
    a8 = (a / sa[:, None]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    b8 = (b / (sb[:, None] if tb else sb[None, :])).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    return a8, b8, sa.numpy(), sb.numpy()


@pytest.mark.parametrize("M,N,K,tb", [(512, 768, 1024, False), (300, 200, 528, True)])
def test_fp8_gemm_scales_bias_gelu(ctx, oracle, M, N, K, tb):
    rng = np.random.default_rng(M + N)
    a8, b8, sa, sb = fp8_operands(rng, M, N, K, tb)
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    want = bf16_bits_to_f32(oracle.gemm(a8, b8, M, N, K, L.F8E4M3, L.BF16, False, tb,
                                        ep=oracle.epilogue(row_scale=sa, col_scale=sb, bias=bias, act=L.ACT_GELU_ERF)))
    got = run_gemm(ctx, a8, b8, M, N, K, torch.float8_e4m3fn, torch.bfloat16, False, tb, row_scale=sa, col_scale=sb, bias=bias,
                   act=L.ACT_GELU_ERF, expect="umma").float().cpu().numpy()
    assert close_lowp(got, want), np.abs(got - want).max()


def test_fp8_gemm_8192_sampled_rows(ctx, oracle):
    n = 8192
    rng = np.random.default_rng(2)
    a8, b8, sa, sb = fp8_operands(rng, n, n, n, False)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    got = run_gemm(ctx, a8, b8, n, n, n, torch.float8_e4m3fn, torch.bfloat16, row_scale=sa, col_scale=sb, bias=bias,
                   act=L.ACT_GELU_ERF, expect="umma").float().cpu().numpy()
    rows = rng.choice(n, size=16, replace=False)
    want = bf16_bits_to_f32(oracle.gemm(np.ascontiguousarray(a8[rows]), b8, 16, n, n, L.F8E4M3, L.BF16,
                                        ep=oracle.epilogue(row_scale=np.ascontiguousarray(sa[rows]), col_scale=sb, bias=bias, act=L.ACT_GELU_ERF)))
    assert close_lowp(got[rows], want), np.abs(got[rows] - want).max()


@pytest.mark.parametrize("M,N,K,ta,tb,batch", [(256, 512, 320, False, False, 1), (200, 130, 64, False, True, 4), (128, 64, 128, False, False, 6),
                                                (264, 128, 72, True, True, 1)])
def test_bf16_gemm(ctx, oracle, M, N, K, ta, tb, batch):
    rng = np.random.default_rng(K)
    a = torch.from_numpy(rng.standard_normal((batch, K, M) if ta else (batch, M, K)).astype(np.float32)).to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((batch, N, K) if tb else (batch, K, N)).astype(np.float32)).to(torch.bfloat16)
    an, bn = a.view(torch.int16).numpy().view(np.uint16), b.view(torch.int16).numpy().view(np.uint16)
    want = oracle.gemm(an, bn, M, N, K, L.BF16, L.F32, ta, tb, batch=batch)
    got = run_gemm(ctx, an.view(np.int16), bn.view(np.int16), M, N, K, torch.bfloat16, torch.float32, ta, tb, batch=batch, expect="umma").cpu().numpy()
    assert close_lowp(got.reshape(want.shape), want)
    assert np.abs(got.reshape(want.shape) - want).max() <= 1e-3 * np.abs(want).max()  # fp32 accumulation: far inside the bf16 bar


@pytest.mark.parametrize("M,N,K,ta,tb", [(1024, 256, 64, False, False), (100, 37, 19, True, False), (64, 10, 256, False, True)])
def test_fp32_gemm_bias_relu(ctx, oracle, M, N, K, ta, tb):
    rng = np.random.default_rng(N)
    a = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    want = oracle.gemm(a, b, M, N, K, L.F32, L.F32, ta, tb, ep=oracle.epilogue(bias=bias, act=L.ACT_RELU))
    got = run_gemm(ctx, a, b, M, N, K, torch.float32, torch.float32, ta, tb, bias=bias, act=L.ACT_RELU).cpu().numpy()
    assert close_f32(got, want), np.abs(got - want).max()


# ---- convolution -----------------------------------------------------------------------------------
def run_conv(ctx, x, w, desc, ho, wo, out_dt, expect=None, **ep_kw):
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    tx, tw = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(desc), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    if expect is not None:
        assert lib.sofie_b200_conv_plan_kernel(h).decode() == expect
    ws = torch.empty(max(16, lib.sofie_b200_conv_workspace_bytes(h)), dtype=torch.uint8, device=DEV)
    y = torch.zeros((desc.N, desc.K, ho, wo), dtype=out_dt, device=DEV)
    dev_kw = {k: (torch.from_numpy(v).to(DEV) if isinstance(v, np.ndarray) else v) for k, v in ep_kw.items()}
    ep, keep = make_epilogue(**dev_kw)
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    return y.cpu().numpy()


@pytest.mark.parametrize("N,Ci,H,W,Co,st,g", [(2, 64, 28, 28, 128, 1, 1), (3, 32, 30, 26, 64, 2, 1), (2, 16, 9, 11, 32, 1, 4), (1, 3, 32, 32, 64, 1, 1)])
def test_qlinear_conv_bit_exact(ctx, oracle, N, Ci, H, W, Co, st, g):
    rng = np.random.default_rng(Ci + Co)
    x = rng.integers(-127, 128, size=(N, Ci, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(Co, Ci // g, 3, 3), dtype=np.int8)
    geo = dict(pads=[1, 1, 1, 1], strides=[st, st], dil=[1, 1], group=g)
    d = gr.conv_desc(geo, x.shape, w.shape, L.I8, L.I8)
    ho, wo = C.c_int64(), C.c_int64()
    assert ctx._lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    cs = (rng.random(Co, dtype=np.float32) * 2e-4 + 5e-5).astype(np.float32)  # a_scale*w_scale[c]/y_scale
    bias = rng.integers(-20000, 20000, size=Co, dtype=np.int32)
    want = oracle.conv(x, w, d, ho.value, wo.value, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU))
    got = run_conv(ctx, x, w, d, ho.value, wo.value, torch.int8, col_scale=cs, bias=bias, act=L.ACT_RELU)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size}"


@pytest.mark.parametrize("dtype", ["int8", "fp32", "fp32_tensor"])
@pytest.mark.parametrize("xl,yl", [(0, 1), (1, 1), (1, 0)])
def test_conv_channels_last_layouts(ctx, oracle, dtype, xl, yl):
    """x_layout / y_layout = 1: the same convolution on [N,H,W,C] tensors (grouped, strided, with a residual in Y's layout)."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    int8 = dtype == "int8"
    N, Ci, H, W, Co, g, st = (12, 64, 40, 36, 96, 2, 1) if dtype == "fp32_tensor" else (2, 32, 13, 10, 48, 2, 2)
    rng = np.random.default_rng(xl * 2 + yl + (7 if int8 else 0))
    if int8:
        x = rng.integers(-127, 128, size=(N, Ci, H, W), dtype=np.int8)
        w = rng.integers(-127, 128, size=(Co, Ci // g, 3, 3), dtype=np.int8)
        cs = (rng.random(Co, dtype=np.float32) * 2e-4 + 5e-5).astype(np.float32)
        bias = rng.integers(-20000, 20000, size=Co, dtype=np.int32)
        code, tdt, res = L.I8, torch.int8, None
    else:
        x = rng.random((N, Ci, H, W), dtype=np.float32)
        w = (rng.standard_normal((Co, Ci // g, 3, 3)) * 0.1).astype(np.float32)
        cs = rng.random(Co, dtype=np.float32) + 0.5
        bias = rng.standard_normal(Co).astype(np.float32)
        code, tdt = L.F32, torch.float32
    geo = dict(pads=[1, 1, 1, 1], strides=[st, st], dil=[1, 1], group=g)
    d = gr.conv_desc(geo, x.shape, w.shape, code, code)
    ho, wo = C.c_int64(), C.c_int64()
    assert lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    res = None if int8 else rng.standard_normal((N, Co, ho.value, wo.value)).astype(np.float32)
    want = oracle.conv(x, w, d, ho.value, wo.value, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU, residual=res))
    d.x_layout, d.y_layout = xl, yl
    to_dev = lambda a, cl: torch.from_numpy(np.ascontiguousarray(a.transpose(0, 2, 3, 1)) if cl else a).to(DEV)
    tx, tw = to_dev(x, xl), torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    if dtype == "fp32_tensor":
        assert lib.sofie_b200_conv_plan_kernel(h).decode() == "umma3x"
    ws = torch.empty(max(16, lib.sofie_b200_conv_workspace_bytes(h)), dtype=torch.uint8, device=DEV)
    y = torch.zeros((N, ho.value, wo.value, Co) if yl else (N, Co, ho.value, wo.value), dtype=tdt, device=DEV)
    ep, keep = make_epilogue(col_scale=torch.from_numpy(cs).to(DEV), bias=torch.from_numpy(bias).to(DEV), act=L.ACT_RELU,
                             residual=None if res is None else to_dev(res, yl))
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    got = y.cpu().numpy()
    if yl:
        got = got.transpose(0, 3, 1, 2)
    if int8:
        assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size}"
    else:
        assert close_f32(got, want), np.abs(got - want).max()


@pytest.mark.parametrize("K,kernel", [(64, "direct"), (256, "simt")])
def test_three_channel_first_layer_channels_last_fp32(ctx, oracle, K, kernel):
    """The 3-channel 3x3 first layer writing a channels-last F32 tensor: the direct kernel while its filters and staging
    fit its shared memory (up to 252 filters), the unfold path for wider layers -- both must run and agree with the checker."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    rng = np.random.default_rng(K)
    x = rng.random((2, 3, 20, 18), dtype=np.float32)
    w = (rng.standard_normal((K, 3, 3, 3)) * 0.2).astype(np.float32)
    bias = rng.standard_normal(K).astype(np.float32)
    geo = dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1)
    d = gr.conv_desc(geo, x.shape, w.shape, L.F32, L.F32)
    want = oracle.conv(x, w, d, 20, 18, ep=oracle.epilogue(bias=bias, act=L.ACT_RELU))
    d.y_layout = 1
    tx, tw = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    assert lib.sofie_b200_conv_plan_kernel(h).decode() == kernel
    ws = torch.empty(max(16, lib.sofie_b200_conv_workspace_bytes(h)), dtype=torch.uint8, device=DEV)
    y = torch.zeros((2, 20, 18, K), dtype=torch.float32, device=DEV)
    ep, keep = make_epilogue(bias=torch.from_numpy(bias).to(DEV), act=L.ACT_RELU)
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    assert close_f32(y.cpu().numpy().transpose(0, 3, 1, 2), want)


@pytest.mark.parametrize("case", ["same", "stride2_zero_point", "dilated_ragged"])
def test_three_channel_first_layer_int8_on_tensor_cores(ctx, oracle, case):
    """The int8 3-channel 3x3 first layer with a channels-last output and enough output pixels: one gather kernel writes
    the unfolded [pixels][32] matrix and the tensor-core contraction does the rest; bit-exact against the checker, also
    with a zero point in the padding, a stride, a dilation and a last tile that is not full."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    N, H, W, K, pads, strides, dil, zp = {"same": (2, 96, 96, 64, [1, 1, 1, 1], [1, 1], [1, 1], 0),
                                          "stride2_zero_point": (3, 161, 150, 32, [1, 1, 1, 1], [2, 2], [1, 1], -7),
                                          "dilated_ragged": (2, 101, 99, 48, [2, 1, 0, 2], [1, 1], [2, 1], 0)}[case]
    rng = np.random.default_rng(len(case))
    x = rng.integers(-127, 128, size=(N, 3, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(K, 3, 3, 3), dtype=np.int8)
    cs = (rng.random(K, dtype=np.float32) * 2e-3 + 2e-4).astype(np.float32)
    bias = rng.integers(-2000, 2000, size=K, dtype=np.int32)
    d = gr.conv_desc(dict(pads=pads, strides=strides, dil=dil, group=1), x.shape, w.shape, L.I8, L.I8)
    d.x_zero_point = zp
    ho, wo = C.c_int64(), C.c_int64()
    assert lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    want = oracle.conv(x, w, d, ho.value, wo.value, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU))
    d.y_layout = 1
    tx, tw = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    assert lib.sofie_b200_conv_plan_kernel(h).decode() == "umma"
    assert lib.sofie_b200_conv_workspace_bytes(h) == N * ho.value * wo.value * 32
    ws = torch.empty(lib.sofie_b200_conv_workspace_bytes(h), dtype=torch.uint8, device=DEV)
    y = torch.zeros((N, ho.value, wo.value, K), dtype=torch.int8, device=DEV)
    ep, keep = make_epilogue(col_scale=torch.from_numpy(cs).to(DEV), bias=torch.from_numpy(bias).to(DEV), act=L.ACT_RELU)
    launches = ctx.launches
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
    ctx.sync()
    # unfold + contraction, plus one small kernel that repeats the per-channel vectors when the contraction packs 2 or 4
    # output pixels per row (as many as keep the packed columns within 256 and divide the pixel count)
    pack = 4
    while pack > 1 and (K * pack > 256 or (N * ho.value * wo.value) % pack):
        pack //= 2
    assert ctx.launches - launches == (3 if pack > 1 else 2)
    lib.sofie_b200_conv_plan_destroy(h)
    got = y.cpu().numpy().transpose(0, 3, 1, 2)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size}"


@pytest.mark.parametrize("dt", [torch.float32, torch.int8])
def test_depth_taps_as_channels(ctx, dt):
    """sofie_b200_depth_unfold_enqueue against the same gather in numpy: stride, dilation and padding in depth."""
    rng = np.random.default_rng(5)
    n, c, d, h, w, taps, stride, pad, dil = 2, 3, 7, 4, 5, 3, 2, 2, 2
    d_out = (d + 2 * pad - (taps + (dil - 1) * (taps - 1))) // stride + 1
    x = (rng.standard_normal((n, c, d, h, w)) * 50).astype(np.float32 if dt == torch.float32 else np.int8)
    want = np.zeros((n, d_out, c, taps, h, w), dtype=x.dtype)
    for od in range(d_out):
        for t in range(taps):
            z = od * stride - pad + t * dil
            if 0 <= z < d:
                want[:, od, :, t] = x[:, :, z]
    tx = torch.from_numpy(x).to(DEV)
    ty = torch.full((n * d_out, c * taps, h, w), 77, dtype=dt, device=DEV)
    ctx.depth_unfold(tx, ty, taps, d_out, stride, pad, dil)
    ctx.sync()
    assert np.array_equal(ty.cpu().numpy(), want.reshape(n * d_out, c * taps, h, w))


IMPLICIT_CASES = {
    # name: (N, C, H, W, K, R, S, pads [top, left, bottom, right], strides [h, w], dilations [h, w], x zero point)
    "c64_3x3_tail": (2, 64, 13, 10, 48, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1], 0),         # 64-byte K blocks, 260 pixels: a partial tile
    "c128_3x3_stride2": (3, 128, 17, 12, 64, 3, 3, [1, 1, 1, 1], [2, 2], [1, 1], 0),    # 128-byte K blocks
    "c64_asymmetric": (2, 64, 15, 11, 40, 3, 2, [2, 0, 1, 1], [2, 1], [1, 2], 0),       # every W / H parameter different
    "c256_1x1_zero_point": (2, 256, 9, 7, 96, 1, 1, [0, 0, 0, 0], [1, 1], [1, 1], 3),   # no padding: a zero point is allowed
    "c192_5x5_wide": (1, 192, 20, 33, 272, 5, 5, [2, 2, 2, 2], [1, 1], [1, 1], 0),      # 3 x 64-byte blocks per tap, two N tiles
    "c64_many_tiles": (5, 64, 56, 56, 64, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1], 0),       # more tiles than SMs, windows wrap rows and images
    # stride 2 on even extents
    "s2_c64_3x3": (2, 64, 16, 12, 48, 3, 3, [1, 1, 1, 1], [2, 2], [1, 1], 0),
    "s2_c128_pads": (3, 128, 14, 10, 64, 3, 3, [0, 1, 1, 0], [2, 2], [1, 1], 0),
    "s2_c64_5x5": (2, 64, 18, 20, 32, 5, 5, [2, 2, 2, 2], [2, 2], [1, 1], 0),
    "s2_c256_1x1": (2, 256, 12, 8, 128, 1, 1, [0, 0, 0, 0], [2, 2], [1, 1], 5),
    "s2_c64_dilated": (2, 64, 20, 16, 64, 3, 3, [2, 3, 2, 3], [2, 2], [2, 3], 0),
    "s2_c64_many_tiles": (4, 64, 112, 112, 128, 3, 3, [1, 1, 1, 1], [2, 2], [1, 1], 0),
    # 64-byte pixels under a horizontal stride of 2 are read as pixel pairs (two-tap convolution over [N, H, W/2, 2C])
    "pairs_w_stride_only": (2, 64, 11, 14, 80, 3, 3, [1, 1, 1, 0], [1, 2], [1, 1], 0),
    "pairs_two_rows": (2, 64, 9, 16, 32, 2, 3, [0, 1, 1, 1], [2, 2], [1, 1], 0),
    "pairs_row_dilation": (3, 64, 20, 18, 64, 3, 3, [2, 1, 2, 1], [2, 2], [2, 1], 0),
    # ... and under a horizontal stride of 1 (16384 pixels or more) as two contractions over the pairs: even and odd output columns
    "pairs1_many_tiles": (6, 64, 56, 56, 128, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1], 0),
    "pairs1_row_dilation": (4, 64, 70, 72, 48, 3, 3, [2, 1, 2, 1], [1, 1], [2, 1], 0),
    "pairs1_row_stride": (8, 64, 64, 80, 64, 3, 3, [1, 1, 1, 1], [2, 1], [1, 1], 0),
    # 128-byte K blocks, output rows of 40 to 112 pixels: windows that wrap rows inside a tile, with every W / H parameter in turn
    "rows_c128_two_per_tile": (3, 128, 24, 56, 96, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1], 0),
    "rows_c128_w112_dilated": (2, 128, 10, 112, 64, 3, 3, [2, 2, 2, 2], [1, 1], [2, 2], 0),
    "rows_c256_row_stride": (2, 256, 35, 40, 64, 3, 3, [1, 1, 1, 1], [2, 1], [1, 1], 0),
    "rows_c128_5x3_asymmetric": (2, 128, 20, 48, 272, 5, 3, [3, 0, 1, 2], [1, 1], [1, 1], 0),
}


@pytest.mark.parametrize("case", list(IMPLICIT_CASES))
def test_conv_implicit_int8(ctx, oracle, case):
    """Channels-last int8 convolutions whose contraction reads the input tensor itself (im2col-mode TMA loads, no unfolded
    copy, no workspace): bit-exact against the oracle's direct convolution."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    N, Ci, H, W, Co, R, S, pads, strides, dil, zp = IMPLICIT_CASES[case]
    rng = np.random.default_rng(len(case) + Ci)
    x = rng.integers(-127, 128, size=(N, Ci, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, size=(Co, Ci, R, S), dtype=np.int8)
    cs = (rng.random(Co, dtype=np.float32) * 1e-4 + 2e-5).astype(np.float32)
    bias = rng.integers(-20000, 20000, size=Co, dtype=np.int32)
    d = gr.conv_desc(dict(pads=pads, strides=strides, dil=dil, group=1), x.shape, w.shape, L.I8, L.I8)
    d.x_zero_point = zp
    ho, wo = C.c_int64(), C.c_int64()
    assert lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    want = oracle.conv(x, w, d, ho.value, wo.value, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU))
    d.x_layout = d.y_layout = 1
    tx = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).to(DEV)
    tw = torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    assert lib.sofie_b200_conv_plan_kernel(h).decode() == ("umma_im2col_x2" if case.startswith("pairs1") else "umma_im2col")
    assert lib.sofie_b200_conv_workspace_bytes(h) == 0
    y = torch.zeros((N, ho.value, wo.value, Co), dtype=torch.int8, device=DEV)
    ep, keep = make_epilogue(col_scale=torch.from_numpy(cs).to(DEV), bias=torch.from_numpy(bias).to(DEV), act=L.ACT_RELU)
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), None, C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    got = y.cpu().numpy().transpose(0, 3, 1, 2)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size}"


def tf32_rn(x):
    """x rounded to the nearest TF32 value (ties away from zero), as the library splits fp32 operands."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = np.where((b & 0x7F800000) >= 0x7F000000, b, b + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
    return r.view(np.float32)


PAIR_CASES = {
    # name: (N, C, H, W, K, R, S, pads, strides, dilations, y_layout)
    "c32_3x3_pairs_out": (2, 32, 14, 12, 64, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1], 2),
    "c64_3x3_stride2_plain_out": (3, 64, 16, 18, 96, 3, 3, [1, 1, 1, 1], [2, 2], [1, 1], 1),
    "c96_asymmetric_pairs_out": (2, 96, 11, 13, 40, 2, 3, [0, 2, 1, 1], [1, 2], [2, 1], 2),
    "c64_many_tiles_pairs_out": (4, 64, 56, 56, 128, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1], 2),
}


@pytest.mark.parametrize("case", list(PAIR_CASES))
def test_conv_fp32_from_tf32_pairs(ctx, oracle, case):
    """x_layout = 2: fp32 convolution at the fp32 bar whose input is a channels-last tensor of TF32 pairs ([N,H,W,2C]: hi
    channels, then lo channels), read in place by the 3xTF32 contraction (no unfold, no workspace); y_layout = 2 writes
    the same form for the next convolution."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    N, Ci, H, W, Co, R, S, pads, strides, dil, yl = PAIR_CASES[case]
    rng = np.random.default_rng(len(case))
    x = (rng.random((N, Ci, H, W), dtype=np.float32) * 2).astype(np.float32)   # same-sign data: the hard case for a truncating accumulator
    w = (rng.standard_normal((Co, Ci, R, S)) * 0.1).astype(np.float32)
    cs = rng.random(Co, dtype=np.float32) + 0.5
    bias = rng.standard_normal(Co).astype(np.float32)
    d = gr.conv_desc(dict(pads=pads, strides=strides, dil=dil, group=1), x.shape, w.shape, L.F32, L.F32)
    ho, wo = C.c_int64(), C.c_int64()
    assert lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    want = oracle.conv(x, w, d, ho.value, wo.value, ep=oracle.epilogue(col_scale=cs, bias=bias, act=L.ACT_RELU))
    d.x_layout, d.y_layout = 2, yl
    xcl = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    hi = tf32_rn(xcl)
    pairs = np.concatenate([hi, tf32_rn(xcl - hi)], axis=3)
    tx, tw = torch.from_numpy(pairs).to(DEV), torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    assert lib.sofie_b200_conv_plan_kernel(h).decode() == "umma3x_im2col"
    assert lib.sofie_b200_conv_workspace_bytes(h) == 0
    y = torch.zeros((N, ho.value, wo.value, Co * (2 if yl == 2 else 1)), dtype=torch.float32, device=DEV)
    ep, keep = make_epilogue(col_scale=torch.from_numpy(cs).to(DEV), bias=torch.from_numpy(bias).to(DEV), act=L.ACT_RELU)
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), None, C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    got = y.cpu().numpy()
    if yl == 2:
        ghi, glo = got[..., :Co], got[..., Co:]
        assert np.array_equal(ghi, tf32_rn(ghi)) and np.array_equal(glo, tf32_rn(glo))   # both halves are TF32 values
        assert np.all(np.abs(glo) <= np.abs(ghi) * 2.0 ** -10 + 1e-37)                    # lo is the rounding remainder of hi
        got = ghi + glo
    got = got.transpose(0, 3, 1, 2)
    assert close_f32(got, want), np.abs(got - want).max()


def test_conv_first_layer_writes_tf32_pairs(ctx, oracle):
    """The 3-channel first layer (direct kernel) with y_layout = 2."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    N, H, W, Co = 3, 20, 18, 64
    rng = np.random.default_rng(12)
    x = rng.random((N, 3, H, W), dtype=np.float32)
    w = (rng.standard_normal((Co, 3, 3, 3)) * 0.3).astype(np.float32)
    bias = rng.standard_normal(Co).astype(np.float32)
    d = gr.conv_desc(dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1), x.shape, w.shape, L.F32, L.F32)
    want = oracle.conv(x, w, d, H, W, ep=oracle.epilogue(bias=bias, act=L.ACT_RELU))
    d.y_layout = 2
    tx, tw = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    assert lib.sofie_b200_conv_plan_kernel(h).decode() == "direct"
    y = torch.zeros((N, H, W, 2 * Co), dtype=torch.float32, device=DEV)
    ep, keep = make_epilogue(bias=torch.from_numpy(bias).to(DEV), act=L.ACT_RELU)
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), None, C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    got = y.cpu().numpy()
    ghi, glo = got[..., :Co], got[..., Co:]
    assert np.array_equal(ghi, tf32_rn(ghi)) and np.array_equal(glo, tf32_rn(glo))
    assert close_f32((ghi + glo).transpose(0, 3, 1, 2), want), np.abs((ghi + glo).transpose(0, 3, 1, 2) - want).max()


def test_conv_implicit_tf32(ctx, oracle):
    """precise = 0 on fp32 channels-last tensors: single-pass TF32 through the same im2col-mode producer."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    N, Ci, H, W, Co = 2, 32, 14, 14, 64
    rng = np.random.default_rng(5)
    x = rng.random((N, Ci, H, W), dtype=np.float32)
    w = (rng.standard_normal((Co, Ci, 3, 3)) * 0.1).astype(np.float32)
    bias = rng.standard_normal(Co).astype(np.float32)
    d = gr.conv_desc(dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1), x.shape, w.shape, L.F32, L.F32)
    want = oracle.conv(x, w, d, H, W, ep=oracle.epilogue(bias=bias))
    d.x_layout = d.y_layout = 1
    d.precise = 0
    tx = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).to(DEV)
    tw = torch.from_numpy(w).to(DEV)
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    assert lib.sofie_b200_conv_plan_kernel(h).decode() == "umma_im2col"
    y = torch.zeros((N, H, W, Co), dtype=torch.float32, device=DEV)
    ep, keep = make_epilogue(bias=torch.from_numpy(bias).to(DEV))
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y.data_ptr(), None, C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)
    got = y.cpu().numpy().transpose(0, 3, 1, 2)
    # TF32 operands (10-bit mantissa): the tolerance of the reduced-precision contractions
    assert np.allclose(got, want, rtol=2e-2, atol=1e-2), np.abs(got - want).max()


def test_conv_fp32_with_folded_batchnorm(ctx, oracle):
    rng = np.random.default_rng(9)
    x = rng.random((2, 8, 20, 20), dtype=np.float32)
    w = (rng.standard_normal((16, 8, 3, 3)) * np.sqrt(2.0 / 72)).astype(np.float32)
    geo = dict(pads=[1, 1, 1, 1], strides=[2, 2], dil=[1, 1], group=1)
    d = gr.conv_desc(geo, x.shape, w.shape)
    gamma, beta = rng.random(16, dtype=np.float32) + 0.5, (rng.standard_normal(16) * 0.1).astype(np.float32)
    mean, var = (rng.standard_normal(16) * 0.1).astype(np.float32), rng.random(16, dtype=np.float32) + 0.5
    fs = (gamma / np.sqrt(var + np.float32(1e-5))).astype(np.float32)
    shift = (beta - mean * fs).astype(np.float32)
    want = oracle.conv(x, w, d, 10, 10, ep=oracle.epilogue(col_scale=fs, bias=shift, act=L.ACT_RELU))
    got = run_conv(ctx, x, w, d, 10, 10, torch.float32, col_scale=fs, bias=shift, act=L.ACT_RELU)
    assert close_f32(got, want), np.abs(got - want).max()


@pytest.mark.parametrize("N,Ci,H,W,Co,st,g,k", [(4, 64, 56, 56, 64, 1, 1, 3), (16, 96, 28, 28, 192, 1, 2, 3), (8, 3, 112, 112, 64, 2, 1, 7)])
def test_conv_fp32_on_tensor_cores_meets_fp32_bar(ctx, oracle, N, Ci, H, W, Co, st, g, k):
    """Large fp32 convolutions unfold into hi/lo TF32 segments and run as 3xTF32 (K = 27..576, not a multiple of 32)."""
    rng = np.random.default_rng(N + Ci + Co)
    x = rng.random((N, Ci, H, W), dtype=np.float32)                         # post-Relu-like: all one sign, the worst case for
    w = np.abs(rng.standard_normal((Co, Ci // g, k, k)) * 0.1).astype(np.float32)   # a truncating accumulator
    geo = dict(pads=[k // 2] * 4, strides=[st, st], dil=[1, 1], group=g)
    d = gr.conv_desc(geo, x.shape, w.shape)
    ho, wo = C.c_int64(), C.c_int64()
    assert ctx._lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    fs, shift = rng.random(Co, dtype=np.float32) + 0.5, (rng.standard_normal(Co) * 0.1).astype(np.float32)
    want = oracle.conv(x, w, d, ho.value, wo.value, ep=oracle.epilogue(col_scale=fs, bias=shift, act=L.ACT_RELU))
    got = run_conv(ctx, x, w, d, ho.value, wo.value, torch.float32, expect="umma3x", col_scale=fs, bias=shift, act=L.ACT_RELU)
    assert close_f32(got, want), f"max abs {np.abs(got - want).max():.3g} at scale {np.abs(want).max():.3g}"


# ---- row-wise and elementwise operators ---------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1000, 512), (333, 128), (17, 100), (64, 4096), (5, 10000), (4096, 8), (1, 1), (3, 2049)])
def test_layernorm_softmax_fp32(ctx, oracle, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g, b = rng.standard_normal(cols).astype(np.float32), rng.standard_normal(cols).astype(np.float32)
    tx = torch.from_numpy(x).to(DEV)
    ty = torch.empty_like(tx)
    ctx.layernorm(tx, ty, torch.from_numpy(g).to(DEV), torch.from_numpy(b).to(DEV), 1e-5)
    ctx.sync()
    want = oracle.layernorm(x, g, b, 1e-5)
    assert np.abs(ty.cpu().numpy() - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    for log in (False, True):
        ctx.softmax(tx, ty, log_softmax=log)
        ctx.sync()
        want = oracle.softmax(x, log=log)
        assert np.abs(ty.cpu().numpy() - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("rows,cols,bf", [(5000, 512, True), (4099, 384, True), (70001, 200, True), (4100, 128, False), (4097, 256, False), (9000, 200, False)])
def test_layernorm_many_rows(ctx, oracle, rows, cols, bf):
    """Rows of 17 to 64 sixteen-byte chunks, thousands of them: the one-warp-per-row kernel that keeps the next rows' loads in
    flight (row counts that leave warps with different numbers of rows; 384 and 200 columns: lanes without a chunk).  With
    scale and bias, mean and 1/std not requested."""
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal((rows, cols)) * 2 + 0.5).astype(np.float32)
    g, b = rng.standard_normal(cols).astype(np.float32), rng.standard_normal(cols).astype(np.float32)
    if bf:
        tx = torch.from_numpy(x).to(torch.bfloat16)
        dx = tx.to(DEV)
        dy = torch.empty_like(dx)
        ctx.layernorm(dx, dy, torch.from_numpy(g).to(DEV), torch.from_numpy(b).to(DEV), 1e-5)
        ctx.sync()
        want = bf16_bits_to_f32(oracle.layernorm(tx.view(torch.int16).numpy().view(np.uint16), g, b, 1e-5, L.BF16))
        assert close_lowp(dy.float().cpu().numpy(), want)
    else:
        dx = torch.from_numpy(x).to(DEV)
        dy = torch.empty_like(dx)
        ctx.layernorm(dx, dy, torch.from_numpy(g).to(DEV), torch.from_numpy(b).to(DEV), 1e-5)
        ctx.sync()
        want = oracle.layernorm(x, g, b, 1e-5)
        assert np.abs(dy.cpu().numpy() - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("rows,cols", [(2048, 512), (4096, 128), (9, 72)])
def test_layernorm_softmax_bf16(ctx, oracle, rows, cols):
    rng = np.random.default_rng(cols)
    tx = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).to(torch.bfloat16)
    xn = tx.view(torch.int16).numpy().view(np.uint16)
    g, b = np.ones(cols, dtype=np.float32), np.zeros(cols, dtype=np.float32)
    dx = tx.to(DEV)
    dy = torch.empty_like(dx)
    ctx.layernorm(dx, dy, torch.from_numpy(g).to(DEV), torch.from_numpy(b).to(DEV), 1e-5)
    ctx.sync()
    assert close_lowp(dy.float().cpu().numpy(), bf16_bits_to_f32(oracle.layernorm(xn, g, b, 1e-5, L.BF16)))
    ctx.softmax(dx, dy)
    ctx.sync()
    assert close_lowp(dy.float().cpu().numpy(), bf16_bits_to_f32(oracle.softmax(xn, L.BF16)))


def test_elementwise_operators(ctx, oracle):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal(100003) * 3).astype(np.float32)
    tx = torch.from_numpy(x).to(DEV)
    ty = torch.empty_like(tx)
    for act, aa in ((L.ACT_RELU, 0.0), (L.ACT_GELU_ERF, 0.0), (L.ACT_GELU_TANH, 0.0), (L.ACT_LEAKY_RELU, 0.1), (L.ACT_SIGMOID, 0.0)):
        ctx.unary(tx, ty, act, aa)
        ctx.sync()
        want = oracle.unary(x, act, aa)
        assert np.abs(ty.cpu().numpy() - want).max() <= 1e-6 * max(1.0, np.abs(want).max()), act
    a = rng.standard_normal((65, 1000)).astype(np.float32)
    b = rng.standard_normal(1000).astype(np.float32) + 3.0
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    tz = torch.empty_like(ta)
    for op in range(4):
        ctx.binary(ta, tb, tz, op)
        ctx.sync()
        assert np.array_equal(tz.cpu().numpy(), oracle.binary(a, b, op)), op


def test_quantize_dequantize_convert_pool(ctx, oracle):
    rng = np.random.default_rng(6)
    x = (rng.standard_normal((4, 6, 5, 7)) * 2).astype(np.float32)
    scale = (rng.random(6, dtype=np.float32) * 0.05 + 0.01).astype(np.float32)
    zp = rng.integers(-5, 5, size=6, dtype=np.int32)
    tx = torch.from_numpy(x).to(DEV)
    q = torch.zeros(x.shape, dtype=torch.int8, device=DEV)
    ctx.quantize(tx, q, torch.from_numpy(scale).to(DEV), torch.from_numpy(zp).to(DEV), channels=6, inner=35)
    ctx.sync()
    wq = oracle.quantize(x, scale, zp, L.I8, 6, 35)
    assert np.array_equal(q.cpu().numpy(), wq)
    back = torch.empty_like(tx)
    ctx.dequantize(q, back, torch.from_numpy(scale).to(DEV), torch.from_numpy(zp).to(DEV), channels=6, inner=35)
    ctx.sync()
    assert np.array_equal(back.cpu().numpy(), oracle.dequantize(wq, scale, zp, L.I8, 6, 35))
    pooled = torch.empty((4, 6), dtype=torch.float32, device=DEV)
    ctx.global_avgpool(tx, pooled)
    ctx.sync()
    assert np.abs(pooled.cpu().numpy() - oracle.global_avgpool(x)).max() <= 1e-6
    # the same pool on the channels-last copy of x (fp32), and on an int8 channels-last tensor (exact sums)
    x4 = x.reshape(4, 6, 5, 7)
    pooled_cl = torch.empty((4, 6), dtype=torch.float32, device=DEV)
    ctx.global_avgpool_nhwc(torch.from_numpy(np.ascontiguousarray(x4.transpose(0, 2, 3, 1))).to(DEV), pooled_cl)
    ctx.sync()
    assert np.abs(pooled_cl.cpu().numpy() - oracle.global_avgpool(x)).max() <= 1e-6
    xi = rng.integers(-128, 128, size=(3, 40, 9, 11), dtype=np.int8)
    pooled_i = torch.empty((3, 40), dtype=torch.float32, device=DEV)
    ctx.global_avgpool_nhwc(torch.from_numpy(np.ascontiguousarray(xi.transpose(0, 2, 3, 1))).to(DEV), pooled_i)
    ctx.sync()
    assert np.array_equal(pooled_i.cpu().numpy(), oracle.global_avgpool(xi, L.I8))
    m = (rng.standard_normal((50, 64)) * 30).astype(np.float32)
    rs = (np.abs(m).max(axis=1) / 448.0).astype(np.float32)
    t8 = torch.zeros((50, 64), dtype=torch.float8_e4m3fn, device=DEV)
    ctx.convert(torch.from_numpy(m).to(DEV), t8, torch.from_numpy(rs).to(DEV))
    ctx.sync()
    assert np.array_equal(t8.view(torch.uint8).cpu().numpy(), oracle.convert(m, L.F32, L.F8E4M3, rs))


# ---- fp32 at fp32 accuracy on the tensor cores (3xTF32) ---------------------------------------------------
@pytest.mark.parametrize("M,N,K,ta,tb,batch", [(1024, 768, 1000, False, False, 1), (640, 512, 2304, False, True, 1), (512, 768, 515, True, False, 1),
                                                (256, 320, 1152, False, True, 3), (384, 200, 8192, False, True, 1)])
def test_fp32_gemm_3xtf32_meets_fp32_bar(ctx, oracle, M, N, K, ta, tb, batch):
    rng = np.random.default_rng(M + K)
    a = rng.standard_normal((batch, K, M) if ta else (batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, N, K) if tb else (batch, K, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    want = oracle.gemm(a, b, M, N, K, L.F32, L.F32, ta, tb, batch=batch, ep=oracle.epilogue(bias=bias, act=L.ACT_RELU))
    got = run_gemm(ctx, a, b, M, N, K, torch.float32, torch.float32, ta, tb, batch=batch, bias=bias, act=L.ACT_RELU, expect="umma3x").cpu().numpy()
    got = got.reshape(want.shape)
    assert close_f32(got, want), f"max abs {np.abs(got - want).max():.3g} at scale {np.abs(want).max():.3g}"
    # single-pass TF32 on the same inputs is far outside the bar: the compensation is what meets it
    tf32 = run_gemm(ctx, a, b, M, N, K, torch.float32, torch.float32, ta, tb, batch=batch, bias=bias, act=L.ACT_RELU, precise=False).cpu().numpy()
    if not ta and tb:
        assert not close_f32(tf32.reshape(want.shape), want)


def test_constant_weight_is_relaid_once_and_follows_its_address(ctx, oracle):
    """SOFIE_B200_GEMM_B_CONSTANT: a weight stored [K,N] is kept as a K-major copy.  Same bits as without the flag; a
    second weight at another address is picked up; the same address is not read again (the documented contract)."""
    from sofie_b200.ops import GemmPlan, make_epilogue
    rng = np.random.default_rng(23)
    for (M, N, K, batch) in ((384, 320, 640, 1), (200, 272, 144, 3)):
        a = rng.integers(-127, 128, size=(batch, M, K), dtype=np.int8)
        b1 = rng.integers(-127, 128, size=(batch, K, N), dtype=np.int8)
        b2 = rng.integers(-127, 128, size=(batch, K, N), dtype=np.int8)
        plan = GemmPlan(ctx, M, N, K, torch.int8, torch.int8, batch=batch, stride_a=M * K if batch > 1 else 0,
                        stride_b=K * N if batch > 1 else 0, stride_y=M * N if batch > 1 else 0, flags=L.GEMM_B_CONSTANT)
        assert plan.kernel == "umma"
        ta, t1, t2 = (torch.from_numpy(v).to(DEV) for v in (a, b1, b2))
        y = torch.zeros((batch, M, N), dtype=torch.int8, device=DEV)
        ep, keep = make_epilogue(alpha=MULT)
        for tb, hb in ((t1, b1), (t2, b2), (t1, b1)):
            plan.enqueue(ta, tb, y, ep)
            ctx.sync()
            want = oracle.gemm(a, hb, M, N, K, L.I8, L.I8, batch=batch, ep=oracle.epilogue(alpha=MULT)).reshape(batch, M, N)
            assert np.array_equal(y.cpu().numpy(), want)
        plan.close()
    # bf16 weights, and fp32 at fp32 accuracy (the constant weight's hi | lo split is made once)
    a = rng.standard_normal((1024, 256)).astype(np.float32)
    b = rng.standard_normal((256, 1024)).astype(np.float32)
    ab, bb = (a.view(np.uint32) >> 16).astype(np.uint16), (b.view(np.uint32) >> 16).astype(np.uint16)
    want = bf16_bits_to_f32(oracle.gemm(ab, bb, 1024, 1024, 256, L.BF16, L.BF16))
    got = run_gemm(ctx, ab.view(np.int16), bb.view(np.int16), 1024, 1024, 256, torch.bfloat16, torch.bfloat16, flags=L.GEMM_B_CONSTANT, expect="umma")
    assert close_lowp(got.float().cpu().numpy(), want)
    plan = GemmPlan(ctx, 1024, 1024, 256, torch.float32, torch.float32, flags=L.GEMM_B_CONSTANT)
    assert plan.kernel == "umma3x"
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    y = torch.zeros((1024, 1024), dtype=torch.float32, device=DEV)
    want = oracle.gemm(a, b, 1024, 1024, 256, L.F32, L.F32)
    for _ in range(2):
        y.zero_()
        plan.enqueue(ta, tb, y)
        ctx.sync()
        assert close_f32(y.cpu().numpy(), want)
    plan.close()


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(ctx, oracle):
    """The kernels' bounded wait on a barrier that nothing signals gives up after its limit, the status word carries the
    code to the next sync (once), and the context keeps working.  The waiting kernel returns normally."""
    lib = ctx._lib
    assert lib.sofie_b200_selftest_wait_timeout(ctx._h, 2000) == 0        # 2 ms
    rc = lib.sofie_b200_ctx_sync(ctx._h)
    assert rc == L.ERR_DEVICE_WAIT
    assert "stage never filled" in lib.sofie_b200_last_error().decode()
    assert lib.sofie_b200_ctx_sync(ctx._h) == 0                            # the word was cleared
    assert lib.sofie_b200_selftest_wait_timeout(ctx._h, 0) == L.ERR_INVALID
    rng = np.random.default_rng(5)
    a = rng.integers(-127, 128, size=(256, 256), dtype=np.int8)
    b = rng.integers(-127, 128, size=(256, 256), dtype=np.int8)
    got = run_gemm(ctx, a, b, 256, 256, 256, torch.int8, torch.int32, expect="umma").cpu().numpy()
    assert np.array_equal(got, a.astype(np.int32) @ b.astype(np.int32))


def test_plans_of_different_sizes_coexist(ctx, oracle):
    """A small plan created AFTER a large one must not make the large one unlaunchable (the shared-memory opt-in is per function)."""
    from sofie_b200.ops import GemmPlan
    rng = np.random.default_rng(2)
    big = GemmPlan(ctx, 512, 512, 512, torch.int8, torch.int32, trans_b=True)      # bn = 256: the largest stage ring
    small = GemmPlan(ctx, 128, 32, 64, torch.int8, torch.int32, trans_b=True)      # bn = 32
    a = torch.from_numpy(rng.integers(-127, 128, size=(512, 512), dtype=np.int8)).to(DEV)
    b = torch.from_numpy(rng.integers(-127, 128, size=(512, 512), dtype=np.int8)).to(DEV)
    y = torch.zeros((512, 512), dtype=torch.int32, device=DEV)
    big.enqueue(a, b, y)
    ctx.sync()
    assert torch.equal(y.cpu(), a.cpu().int() @ b.cpu().int().T)
    big.close(); small.close()


def test_conv_layout_rules_and_empty_batch(ctx):
    """Layout combinations the header rules out are refused at plan creation; an empty batch enqueues nothing."""
    lib = ctx._lib
    w64 = torch.zeros((64, 64, 3, 3), dtype=torch.float32, device=DEV)
    w48 = torch.zeros((64, 48, 3, 3), dtype=torch.float32, device=DEV)
    w8 = torch.zeros((64, 64, 3, 3), dtype=torch.int8, device=DEV)

    def create(w, xshape, x_dtype, y_dtype, xl, yl, groups=1, precise=1):
        d = gr.conv_desc(dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=groups), xshape, tuple(w.shape), x_dtype, y_dtype)
        d.x_layout, d.y_layout, d.precise = xl, yl, precise
        h = C.c_void_p()
        rc = lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), w.data_ptr(), C.byref(h))
        return rc, h

    for args in [
        (w48, (2, 48, 8, 8), L.F32, L.F32, 2, 1),        # pairs need C % 32 == 0
        (w64, (2, 64, 8, 8), L.F32, L.F32, 2, 0),        # pairs in, NCHW out
        (w64, (2, 64, 8, 8), L.F32, L.F32, 1, 2),        # pairs out from a plain channels-last input
        (w8, (2, 64, 8, 8), L.I8, L.I8, 2, 2),           # pairs are an fp32 format
        (w64, (2, 64, 8, 8), L.F32, L.F32, 2, 2, 1, 0),  # ... at precise = 1 only
        (w64, (2, 64, 8, 8), L.F32, L.F32, 3, 0),        # unknown layout
    ]:
        rc, h = create(*args)
        assert rc == L.ERR_INVALID, (args[1:], rc)
        assert h.value is None
    # an empty batch: the plan is created, the enqueue is a no-op
    n0 = ctx.launches
    rc, h = create(w8, (0, 64, 8, 8), L.I8, L.I8, 1, 1)
    assert rc == 0
    created = ctx.launches - n0        # the filter re-layout at plan creation
    assert lib.sofie_b200_conv_enqueue(h, None, None, None, None) == 0
    assert ctx.launches - n0 == created
    lib.sofie_b200_conv_plan_destroy(h)
