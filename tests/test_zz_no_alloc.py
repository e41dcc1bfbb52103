"""The allocation-free convolution entry point against the regular plan-based one.

Some users of this library (fixed-memory-budget services, e.g. online event filters) are not allowed to
allocate device memory once they are configured; sofie_b200_conv_enqueue_noalloc serves them from a
16 MiB array inside the library image.  Here it is called through the C ABI twice in a row, the second
time on a smaller, different problem so that stale bytes of the first call would show, and each
result is compared with sofie_b200_conv_enqueue on the same inputs and with the CPU checker: bit for
bit for the int8 path, 1e-5 for fp32.  A convolution that does not fit the array, or one with an
argument the call does not support, must be refused with a clear message before anything is launched.
After one warm-up call per input type (CUDA loads kernels and the library's static array on first
use) further calls must leave the device's free memory where it was.
The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import graph_runner as gr
from oracle_api import Oracle
from sofie_b200 import lib as L

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def conv_checker(oracle, x, w, geo, x_dtype, y_dtype, **ep_kw):
    """The same convolution on the CPU checker (numpy operands)."""
    d = gr.conv_desc(geo, x.shape, w.shape, x_dtype, y_dtype)
    g = gr.conv_geometry(dict(pads=geo["pads"], strides=geo["strides"], dilations=geo["dil"], group=geo["group"]), x.shape, w.shape)
    return oracle.conv(x, w, d, g["ho"], g["wo"], oracle.epilogue(**ep_kw))


def conv_both_ways(ctx, x, w, geo, x_dtype, y_dtype, out_torch_dtype, **ep_kw):
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    d = gr.conv_desc(geo, x.shape, w.shape, x_dtype, y_dtype)
    ho, wo = C.c_int64(), C.c_int64()
    assert lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    tx, tw = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV)
    dev_kw = {k: (torch.from_numpy(v).to(DEV) if isinstance(v, np.ndarray) else v) for k, v in ep_kw.items()}
    ep, keep = make_epilogue(**dev_kw)
    shape = (d.N, d.K, ho.value, wo.value)

    # regular path: plan (owns padded weights) + caller workspace
    h = C.c_void_p()
    L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), tw.data_ptr(), C.byref(h)), "conv_plan_create")
    ws = torch.empty(max(16, lib.sofie_b200_conv_workspace_bytes(h)), dtype=torch.uint8, device=DEV)
    y_ref = torch.zeros(shape, dtype=out_torch_dtype, device=DEV)
    L.check(lib.sofie_b200_conv_enqueue(h, tx.data_ptr(), y_ref.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
    ctx.sync()
    lib.sofie_b200_conv_plan_destroy(h)

    # allocation-free path: inputs and outputs only
    y_new = torch.full(shape, 77, dtype=out_torch_dtype, device=DEV)
    L.check(lib.sofie_b200_conv_enqueue_noalloc(ctx._h, C.byref(d), tx.data_ptr(), tw.data_ptr(), y_new.data_ptr(), C.byref(ep)),
            "conv_enqueue_noalloc")
    ctx.sync()
    return y_new.cpu().numpy(), y_ref.cpu().numpy()


@pytest.fixture(scope="module")
def ctx(b200_lib):
    from sofie_b200.ops import Context
    c = Context(0)
    yield c
    c.close()


def test_noalloc_convolution_matches_plan_based_twice_in_a_row(ctx, oracle_lib):
    oracle = Oracle(oracle_lib)
    rng = np.random.default_rng(42)
    geo1 = dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1)
    geo2 = dict(pads=[1, 1, 1, 1], strides=[2, 2], dil=[1, 1], group=2)
    # call 1: int8, 4 x 32 x 24 x 24 -> 64 channels; per-channel requantisation, int32 bias, Relu
    x1 = rng.integers(-127, 128, size=(4, 32, 24, 24), dtype=np.int8)
    w1 = rng.integers(-127, 128, size=(64, 32, 3, 3), dtype=np.int8)
    cs1 = (rng.random(64, dtype=np.float32) * 2e-4 + 5e-5).astype(np.float32)
    b1 = rng.integers(-20000, 20000, size=64, dtype=np.int32)
    got, want = conv_both_ways(ctx, x1, w1, geo1, L.I8, L.I8, torch.int8, col_scale=cs1, bias=b1, act=L.ACT_RELU)
    assert np.array_equal(got, want), f"first call: {(got != want).sum()} of {got.size} differ"
    assert np.array_equal(got, conv_checker(oracle, x1, w1, geo1, L.I8, L.I8, col_scale=cs1, bias=b1, act=L.ACT_RELU))
    # call 2, straight after: smaller, grouped, strided, other values -- leftovers of call 1 must not matter
    x2 = rng.integers(-127, 128, size=(2, 16, 13, 11), dtype=np.int8)
    w2 = rng.integers(-127, 128, size=(8, 8, 3, 3), dtype=np.int8)
    got, want = conv_both_ways(ctx, x2, w2, geo2, L.I8, L.I32, torch.int32)
    assert np.array_equal(got, want), f"second call: {(got != want).sum()} of {got.size} differ"
    assert np.array_equal(got, conv_checker(oracle, x2, w2, geo2, L.I8, L.I32))
    # and once in fp32 with a folded BatchNormalization epilogue
    x3 = rng.random((2, 8, 20, 20), dtype=np.float32)
    w3 = (rng.standard_normal((16, 8, 3, 3)) * 0.2).astype(np.float32)
    fs, sh = rng.random(16, dtype=np.float32) + 0.5, rng.standard_normal(16).astype(np.float32)
    got, want = conv_both_ways(ctx, x3, w3, geo1, L.F32, L.F32, torch.float32, col_scale=fs, bias=sh, act=L.ACT_RELU)
    floor = float(np.sqrt(np.mean(np.square(want))))
    assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), floor))
    chk = conv_checker(oracle, x3, w3, geo1, L.F32, L.F32, col_scale=fs, bias=sh, act=L.ACT_RELU)
    assert np.all(np.abs(got - chk) <= 1e-5 * np.maximum(np.abs(chk), floor))


def test_noalloc_convolution_refuses_what_does_not_fit(ctx):
    lib = ctx._lib
    x = torch.zeros((64, 64, 56, 56), dtype=torch.int8, device=DEV)   # unfolded: 64*3136*576 bytes = 115 MB > 16 MiB
    w = torch.zeros((64, 64, 3, 3), dtype=torch.int8, device=DEV)
    y = torch.zeros((64, 64, 56, 56), dtype=torch.int8, device=DEV)
    d = gr.conv_desc(dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1), tuple(x.shape), tuple(w.shape), L.I8, L.I8)
    rc = lib.sofie_b200_conv_enqueue_noalloc(ctx._h, C.byref(d), x.data_ptr(), w.data_ptr(), y.data_ptr(), None)
    assert rc == L.ERR_TOO_LARGE
    msg = lib.sofie_b200_last_error().decode()
    assert "static scratch holds 16777216 bytes" in msg and "plan-based" in msg
    ctx.sync()  # the refusal launched nothing and left the context usable


def test_noalloc_convolution_refuses_bad_arguments_before_launching(ctx):
    """A row scale, a full-matrix bias or an I32 output of an F32 convolution are refused; the refusal comes before
    the first launch (the launch counter does not move), so the shared array is not touched either."""
    from sofie_b200.ops import make_epilogue
    lib = ctx._lib
    geo = dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1)
    x = torch.ones((1, 8, 10, 10), dtype=torch.float32, device=DEV)
    w = torch.ones((8, 8, 3, 3), dtype=torch.float32, device=DEV)
    y = torch.zeros((1, 8, 10, 10), dtype=torch.float32, device=DEV)
    vec = torch.ones(8, dtype=torch.float32, device=DEV)
    full = torch.ones((8, 100), dtype=torch.float32, device=DEV)
    d = gr.conv_desc(geo, tuple(x.shape), tuple(w.shape), L.F32, L.F32)
    cases = []
    ep, keep1 = make_epilogue(row_scale=vec)
    cases.append((d, ep, "row_scale"))
    ep, keep2 = make_epilogue(bias=full, bias_mode=L.BIAS_FULL_F32)
    cases.append((d, ep, "bias_mode"))
    d32 = gr.conv_desc(geo, tuple(x.shape), tuple(w.shape), L.F32, L.I32)
    ep, keep3 = make_epilogue()
    cases.append((d32, ep, "I32 output"))
    before = lib.sofie_b200_ctx_launch_count(ctx._h)
    for desc, e, word in cases:
        rc = lib.sofie_b200_conv_enqueue_noalloc(ctx._h, C.byref(desc), x.data_ptr(), w.data_ptr(), y.data_ptr(), C.byref(e))
        assert rc == L.ERR_INVALID, word
        assert word in lib.sofie_b200_last_error().decode()
    assert lib.sofie_b200_ctx_launch_count(ctx._h) == before
    ctx.sync()


def test_noalloc_convolution_moves_no_device_memory_once_warm(ctx):
    """One warm-up call per input type loads the kernels and the static array; after that the free device memory
    reported by the driver is the same before and after further calls."""
    lib = ctx._lib
    geo = dict(pads=[1, 1, 1, 1], strides=[1, 1], dil=[1, 1], group=1)
    sets = []
    for tdt, ldt in ((torch.int8, L.I8), (torch.float32, L.F32)):
        x = torch.ones((2, 16, 12, 12), dtype=tdt, device=DEV)
        w = torch.ones((16, 16, 3, 3), dtype=tdt, device=DEV)
        y = torch.zeros((2, 16, 12, 12), dtype=torch.int32 if ldt == L.I8 else torch.float32, device=DEV)
        d = gr.conv_desc(geo, tuple(x.shape), tuple(w.shape), ldt, L.I32 if ldt == L.I8 else L.F32)
        sets.append((d, x, w, y))

    def call_all():
        for d, x, w, y in sets:
            L.check(lib.sofie_b200_conv_enqueue_noalloc(ctx._h, C.byref(d), x.data_ptr(), w.data_ptr(), y.data_ptr(), None), "noalloc")
        ctx.sync()

    call_all()                                  # warm-up: modules and the array are loaded here
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        call_all()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes"
    assert int(sets[0][3][0, 0, 5, 5]) == 16 * 9 and float(sets[1][3][0, 0, 5, 5]) == 16.0 * 9
