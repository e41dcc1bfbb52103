"""Emitted Sessions on the GPU beyond the fp32 golden models: quantised operators, the safetensors weight file, CUDA-graph
replay, the pipelined host queue, and the external-stream / custom-memory options, modelled on the reference's own
device tests (tests/alpaka/TestAlpakaExternalStream.cxx:5-45, tests/alpaka/TestAlpakaCustomMemory.cxx:113-183).

Every model is written as an ONNX file, emitted by the C++ generator, compiled with g++ against include/sofie_b200.h and
run through a small C wrapper; results are compared with the CPU checker (bit for bit for int8).
"""
import ctypes as C
import subprocess

import numpy as np
import pytest

import graph_runner as gr
from oracle_api import Oracle
from sofie_b200 import build as B
from sofie_b200 import lib as L
from sofie_b200 import onnx_min

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def emit():
    return B.build_host()


# infer_host three times (eager, captured, replayed) and a queue of 5 through infer_host_many: all results must agree
TYPED_WRAPPER = """
#include "{header}"
#include <cstring>
static std::string g_err;
extern "C" const char *session_error() {{ return g_err.c_str(); }}
extern "C" long session_run(const char *file, const {tin} *x, {tout} *out, long cap, long long *launches)
{{
   try {{
      SOFIE_{name}::Session s(file);
      std::vector<{tout}> y0 = s.infer_host(x);
      const long long eager = s.GetLaunchCount();
      std::vector<{tout}> y1 = s.infer_host(x), y2 = s.infer_host(x);
      if (y1 != y0 || y2 != y0) {{ g_err = "graph capture / replay changed the result"; return -2; }}
      launches[0] = eager;
      launches[1] = s.GetLaunchCount();
      std::vector<std::vector<{tout}>> q(5, std::vector<{tout}>(y0.size()));
      const {tin} *ins[5] = {{x, x, x, x, x}};
      {tout} *outs[5];
      for (int i = 0; i < 5; ++i) outs[i] = q[i].data();
      s.infer_host_many(5, ins, outs);
      for (int i = 0; i < 5; ++i) if (q[i] != y0) {{ g_err = "infer_host_many differs from infer_host at " + std::to_string(i); return -3; }}
      std::memcpy(out, y0.data(), sizeof({tout}) * (y0.size() < (size_t)cap ? y0.size() : (size_t)cap));
      return (long)y0.size();
   }} catch (const std::exception &e) {{ g_err = e.what(); return -1; }}
}}
"""


def emit_and_load(emit, tmp_path, name, nodes, weights, inputs, outputs, wrapper, flags=(), **onnx_kw):
    onnx_min.save(str(tmp_path / f"{name}.onnx"), nodes, weights, inputs, outputs, **onnx_kw)
    r = subprocess.run([str(emit), str(tmp_path / f"{name}.onnx"), str(tmp_path / f"{name}.hxx"), *flags], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    so = B.compile_session(tmp_path / f"{name}.hxx", tmp_path / f"libsession_{name}.so", wrapper)
    lib = C.CDLL(str(so))
    lib.session_error.restype = C.c_char_p
    return lib


def test_qlinear_matmul_session_bit_exact_from_safetensors(emit, tmp_path, oracle_lib, b200_lib):
    """A parsed QLinearMatMul model (per-column weight scales, non-zero input zero point, uint8 output) as an emitted
    Session reading its int8 weights from a safetensors file."""
    o = Oracle(oracle_lib)
    rng = np.random.default_rng(31)
    M, K, N = 200, 256, 144
    a = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    a_scale, y_scale, a_zp, y_zp = np.float32(0.02), np.float32(0.4), 3, 120
    b_scale = (rng.random(N, dtype=np.float32) * 0.01 + 0.005).astype(np.float32)
    w = {"B": b, "a_scale": np.array(a_scale), "a_zp": np.array(a_zp, dtype=np.int8), "b_scale": b_scale, "b_zp": np.zeros(N, dtype=np.int8),
         "y_scale": np.array(y_scale), "y_zp": np.array(y_zp, dtype=np.uint8)}
    nodes = [{"op": "QLinearMatMul", "in": ["A", "a_scale", "a_zp", "B", "b_scale", "b_zp", "y_scale", "y_zp"], "out": ["Y"], "attrs": {}}]
    src = TYPED_WRAPPER.format(header=tmp_path / "qmm.hxx", name="qmm", tin="int8_t", tout="uint8_t")
    lib = emit_and_load(emit, tmp_path, "qmm", nodes, w, [("A", [M, K])], ["Y"], src, flags=("--safetensors",), input_types={"A": 3})
    # checker: acc = sum (a - a_zp) b;  y = sat(rint(acc * (a_scale * b_scale[j] / y_scale)) + y_zp)
    mult = (a_scale * b_scale / y_scale).astype(np.float32)
    corr = (-a_zp * b.astype(np.int32).sum(axis=0)).astype(np.int32)
    want = o.gemm(a, b, M, N, K, L.I8, L.U8, ep=o.epilogue(col_scale=mult, bias=corr, out_zero_point=y_zp))
    got = np.zeros((M, N), dtype=np.uint8)
    launches = (C.c_longlong * 2)()
    n = lib.session_run(str(tmp_path / "qmm.safetensors").encode(), a.ctypes.data_as(C.c_void_p), got.ctypes.data_as(C.c_void_p), got.size, launches)
    assert n == got.size, lib.session_error().decode()
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} differ"
    # the first call enqueued the operators (and the one-time K-major copy of the weight); the captured call enqueued them
    # once more; the replay enqueued nothing
    assert launches[0] >= 1 and launches[1] - launches[0] <= launches[0]


def test_qlinear_conv_session_bit_exact(emit, tmp_path, oracle_lib, b200_lib):
    """QLinearConv (per-channel weight scales, int32 bias, input zero point) -> QLinearConv: a parsed two-layer int8 model."""
    o = Oracle(oracle_lib)
    rng = np.random.default_rng(32)
    x = rng.integers(-100, 100, size=(2, 16, 12, 10), dtype=np.int8)
    w1 = rng.integers(-127, 128, size=(32, 16, 3, 3), dtype=np.int8)
    w2 = rng.integers(-127, 128, size=(16, 32, 1, 1), dtype=np.int8)
    s1 = (rng.random(32, dtype=np.float32) * 0.01 + 0.002).astype(np.float32)
    s2 = (rng.random(16, dtype=np.float32) * 0.01 + 0.002).astype(np.float32)
    b1 = rng.integers(-3000, 3000, size=32, dtype=np.int32)
    xs, h_s, ys, x_zp = np.float32(0.05), np.float32(0.9), np.float32(1.1), 4
    w = {"w1": w1, "w2": w2, "s1": s1, "s2": s2, "b1": b1, "xs": np.array(xs), "hs": np.array(h_s), "ys": np.array(ys),
         "xzp": np.array(x_zp, dtype=np.int8), "z8": np.array(0, dtype=np.int8), "wz1": np.zeros(32, dtype=np.int8), "wz2": np.zeros(16, dtype=np.int8)}
    nodes = [{"op": "QLinearConv", "in": ["X", "xs", "xzp", "w1", "s1", "wz1", "hs", "z8", "b1"], "out": ["H"],
              "attrs": {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [2, 1]}},
             {"op": "QLinearConv", "in": ["H", "hs", "z8", "w2", "s2", "wz2", "ys", "z8"], "out": ["Y"], "attrs": {"kernel_shape": [1, 1], "pads": [0, 0, 0, 0]}}]
    src = TYPED_WRAPPER.format(header=tmp_path / "qconv.hxx", name="qconv", tin="int8_t", tout="int8_t")
    lib = emit_and_load(emit, tmp_path, "qconv", nodes, w, [("X", list(x.shape))], ["Y"], src, input_types={"X": 3})
    # checker: layer by layer, padding filled with the input zero point
    g1 = gr.conv_geometry({"pads": [1, 1, 1, 1], "strides": [2, 1]}, x.shape, w1.shape)
    d1 = gr.conv_desc(g1, x.shape, w1.shape, L.I8, L.I8)
    d1.x_zero_point = x_zp
    bias1 = (b1 - x_zp * w1.astype(np.int32).reshape(32, -1).sum(axis=1)).astype(np.int32)
    h = o.conv(x, w1, d1, g1["ho"], g1["wo"], ep=o.epilogue(col_scale=(xs * s1 / h_s).astype(np.float32), bias=bias1))
    g2 = gr.conv_geometry({"pads": [0, 0, 0, 0]}, h.shape, w2.shape)
    d2 = gr.conv_desc(g2, h.shape, w2.shape, L.I8, L.I8)
    want = o.conv(h, w2, d2, g2["ho"], g2["wo"], ep=o.epilogue(col_scale=(h_s * s2 / ys).astype(np.float32)))
    got = np.zeros(want.shape, dtype=np.int8)
    launches = (C.c_longlong * 2)()
    n = lib.session_run(str(tmp_path / "qconv.dat").encode(), x.ctypes.data_as(C.c_void_p), got.ctypes.data_as(C.c_void_p), got.size, launches)
    assert n == got.size, lib.session_error().decode()
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} differ"


EXT_WRAPPER = """
#include "{header}"
#include <cstring>
using namespace SOFIE_{name};
static std::string g_err;
extern "C" const char *session_error() {{ return g_err.c_str(); }}
struct State {{ int allocs = 0, deallocs = 0; size_t bytes = 0; char *block = nullptr; }};
static void *my_alloc(size_t bytes, void *user)
{{
   State *s = static_cast<State *>(user);
   ++s->allocs;
   s->bytes = bytes;
   if (cudaMalloc(reinterpret_cast<void **>(&s->block), bytes + 4096) != cudaSuccess) return nullptr;
   return s->block + 4096;   // not the start of an allocation: the Session must use exactly what it is given
}}
static void my_dealloc(void *, void *user)
{{
   State *s = static_cast<State *>(user);
   ++s->deallocs;
   cudaFree(s->block);
}}
static void *null_alloc(size_t, void *) {{ return nullptr; }}
// counts: allocations, deallocations, block size == arena size, result inside the block, null block rejected, empty provider rejected
extern "C" long session_run(const char *file, const float *x_host, long nx, float *out, long cap, int *counts)
{{
   cudaStream_t st = nullptr;
   float *x_d = nullptr;
   long n = -1;
   try {{
      if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) throw std::runtime_error("stream");
      if (cudaMalloc(reinterpret_cast<void **>(&x_d), sizeof(float) * nx) != cudaSuccess) throw std::runtime_error("malloc");
      cudaMemcpy(x_d, x_host, sizeof(float) * nx, cudaMemcpyHostToDevice);
      State state;
      {{
         MemoryProvider prov{{my_alloc, my_dealloc, &state}};
         Session s(prov, st, file);
         counts[0] = state.allocs;
         counts[2] = state.bytes == s.GetArenaSize();
         for (int rep = 0; rep < 3; ++rep) {{              // eager, captured on the caller's stream, replayed
            float *r = s.infer_nosync(x_d);                 // records on the caller's stream only
            if (cudaStreamSynchronize(st) != cudaSuccess) throw std::runtime_error("sync");
            counts[3] = reinterpret_cast<char *>(r) >= state.block + 4096 && reinterpret_cast<char *>(r) < state.block + 4096 + state.bytes;
            cudaMemcpy(out, r, sizeof(float) * cap, cudaMemcpyDeviceToHost);
         }}
         n = cap;
      }}
      counts[1] = state.deallocs;
      State other;
      try {{ MemoryProvider bad{{null_alloc, my_dealloc, &other}}; Session s2(bad, st, file); counts[4] = 0; }} catch (const std::runtime_error &) {{ counts[4] = 1; }}
      try {{ MemoryProvider none{{}}; Session s3(none, st, file); counts[5] = 0; }} catch (const std::runtime_error &) {{ counts[5] = 1; }}
   }} catch (const std::exception &e) {{ g_err = e.what(); n = -1; }}
   if (x_d) cudaFree(x_d);
   if (st) cudaStreamDestroy(st);
   return n;
}}
"""


def test_external_stream_and_custom_memory_session(emit, tmp_path, b200_lib):
    """The reference's ExternalStreamGemmRelu model (ones [3,5] x 0.5 [5,4] + 1, Relu = 3.5) in a Session that borrows the
    caller's stream and takes its one block of device memory from the caller's provider."""
    w = {"W": np.full((5, 4), 0.5, dtype=np.float32), "B": np.ones(4, dtype=np.float32)}
    nodes = [{"op": "Gemm", "in": ["X", "W", "B"], "out": ["G"], "attrs": {}}, {"op": "Relu", "in": ["G"], "out": ["Y"], "attrs": {}}]
    src = EXT_WRAPPER.format(header=tmp_path / "ext.hxx", name="ext")
    lib = emit_and_load(emit, tmp_path, "ext", nodes, w, [("X", [3, 5])], ["Y"], src, flags=("--external-stream", "--custom-memory"))
    text = (tmp_path / "ext.hxx").read_text()
    assert "cudaMalloc(" not in text          # no allocation of its own (the reference's GeneratedCodeHasNoAlpakaDeviceAllocation)
    x = np.ones((3, 5), dtype=np.float32)
    out = np.zeros(12, dtype=np.float32)
    counts = (C.c_int * 6)()
    n = lib.session_run(str(tmp_path / "ext.dat").encode(), x.ctypes.data_as(C.c_void_p), x.size, out.ctypes.data_as(C.c_void_p), out.size, counts)
    assert n == 12, lib.session_error().decode()
    assert np.all(np.abs(out - 3.5) <= 1e-6)
    assert list(counts) == [1, 1, 1, 1, 1, 1], list(counts)


def test_encoder_configuration_from_the_generator_matches_the_reference(tmp_path, b200_lib):
    """The transformer-encoder configuration as a parsed ONNX model (int8 weights behind DequantizeLinear, Split -> SDPA): the
    generator folds the dequantisation, the Gelu and the residual adds into the contractions and lets the fused attention
    kernel read Q, K, V in place -- 7 launches per layer -- and the emitted Session reproduces what the reference's own
    emitted fp32 code computed on the dequantised weights (fixture of tests/golden/make_golden.py), at the bf16 bar."""
    from pathlib import Path
    from sofie_b200 import encoder as be
    from sofie_b200.session import EmittedSession
    fx = np.load(Path(__file__).parent / "golden" / "configs" / "Encoder_C5r.npz")
    batch, layers = int(fx["batch"]), int(fx["layers"])
    weights = be.make_weights(int(fx["seed"]), layers, 512, 2048)
    nodes, init, ins, outs, in_types = be.onnx_model(weights, batch, 128, 512, 8)
    sess = EmittedSession("encoder", nodes, init, ins, outs, tmp_path, input_types=in_types)
    header = (tmp_path / "encoder.hxx").read_text()
    assert "cudaMemcpy2DAsync(" not in header            # no Split copies: attention reads the projection's output in place
    x = be.f32_to_bf16_bits(fx["x"])
    y = np.zeros((batch * 128, 512), dtype=np.uint16)
    l0 = sess.launches
    assert sess.infer_host([x], y) == y.size
    assert sess.launches - l0 == 7 * layers
    got = be.bf16_bits_to_f32(y)
    err = np.abs(got - fx["y"])
    assert np.all(err <= 2e-2 * np.abs(fx["y"]) + 1e-2), f"max abs err {err.max():.4f}"
    y2 = np.zeros_like(y)
    sess.infer_host([x], y2)     # captured into a CUDA graph
    sess.infer_host([x], y2)     # replayed
    assert np.array_equal(y, y2)
    sess.close()


@pytest.mark.parametrize("int8", [False, True])
def test_convnet_configuration_from_the_generator(tmp_path, oracle_lib, b200_lib, int8):
    """The conv-net configuration as a parsed ONNX model.  fp32: Conv -> BatchNormalization -> Relu per layer, which the
    generator folds and keeps channels-last as TF32 pairs (10 launches), against the reference's own emitted code (fixture
    of tests/golden/make_golden.py) at 1e-5.  int8: QLinearConv -> Relu chains running as implicit convolutions, the final
    DequantizeLinear folded behind the pooling, against the CPU checker."""
    from pathlib import Path
    import model_oracles as mo
    from sofie_b200 import convnet as bc
    from sofie_b200.session import EmittedSession
    fx = np.load(Path(__file__).parent / "golden" / "configs" / "ConvNet_C4r.npz")
    seed = int(fx["seed"])
    nodes, init, ins, outs, in_types = bc.onnx_model(seed, 2, 32, int8)
    sess = EmittedSession("convnet_i8" if int8 else "convnet_f32", nodes, init, ins, outs, tmp_path, input_types=in_types)
    if int8:
        x = np.clip(np.rint(fx["x"] * 127.0), 0, 127).astype(np.int8)
        want = mo.convnet_oracle(Oracle(oracle_lib), x, bc.make_weights(seed, True), True)
    else:
        x, want = fx["x"], fx["y"]
    y = np.zeros((2, 1000), dtype=np.float32)
    l0 = sess.launches
    assert sess.infer_host([x], y) == y.size
    assert sess.launches - l0 == 10
    floor = float(np.sqrt(np.mean(np.square(want))))
    assert np.all(np.abs(y - want) <= 1e-5 * np.maximum(np.abs(want), floor)), np.abs(y - want).max()
    y2 = np.zeros_like(y)
    sess.infer_host([x], y2)
    sess.infer_host([x], y2)     # replayed from the captured graph
    assert np.array_equal(y, y2)
    sess.close()


def test_int8_convnet_session_with_the_first_layer_on_tensor_cores(tmp_path, oracle_lib, b200_lib):
    """2 images of 96 x 96: 18432 output pixels, enough for the int8 first layer to take the unfold + tensor-core path
    (three launches: gather, the per-channel vectors repeated for the four pixels a row of the contraction holds, the
    contraction; a [pixels][32] scratch region the generator reserved in the arena) instead of the direct kernel; the logits
    against the CPU checker, 12 launches."""
    import model_oracles as mo
    from sofie_b200 import convnet as bc
    from sofie_b200.session import EmittedSession
    seed = 11
    nodes, init, ins, outs, in_types = bc.onnx_model(seed, 2, 96, True)
    sess = EmittedSession("convnet_i8_96", nodes, init, ins, outs, tmp_path, input_types=in_types)
    x = np.clip(np.rint(np.random.default_rng(seed).random((2, 3, 96, 96), dtype=np.float32) * 127.0), 0, 127).astype(np.int8)
    want = mo.convnet_oracle(Oracle(oracle_lib), x, bc.make_weights(seed, True), True)
    y = np.zeros((2, 1000), dtype=np.float32)
    l0 = sess.launches
    assert sess.infer_host([x], y) == y.size
    assert sess.launches - l0 == 12
    floor = float(np.sqrt(np.mean(np.square(want))))
    assert np.all(np.abs(y - want) <= 1e-5 * np.maximum(np.abs(want), floor)), np.abs(y - want).max()
    sess.close()


def test_span_infer_and_pool_statistics(tmp_path, b200_lib):
    """The span form of infer (device views in, results copied into caller-owned device buffers, as the reference's
    infer(span<ViewConst>, span<View>)) against infer_host on the MLP, a wrong number of views refused, and the pool's
    free-space figures of the reference's Session (pool size, free bytes and largest free block when the footprint last
    grew, the fragmentation derived from them)."""
    import torch
    from sofie_b200.session import EmittedSession
    rng = np.random.default_rng(3)
    w1, w2 = (rng.standard_normal((64, 256)) * 0.1).astype(np.float32), (rng.standard_normal((256, 10)) * 0.1).astype(np.float32)
    b1, b2 = rng.standard_normal(256).astype(np.float32), rng.standard_normal(10).astype(np.float32)
    nodes = [{"op": "Gemm", "in": ["X", "w1", "b1"], "out": ["h"], "attrs": {}}, {"op": "Relu", "in": ["h"], "out": ["r"], "attrs": {}},
             {"op": "Gemm", "in": ["r", "w2", "b2"], "out": ["Y"], "attrs": {}}]
    sess = EmittedSession("mlp_span", nodes, {"w1": w1, "b1": b1, "w2": w2, "b2": b2}, [("X", [128, 64])], ["Y"], tmp_path)
    x = rng.standard_normal((128, 64)).astype(np.float32)
    want = np.zeros((128, 10), dtype=np.float32)
    assert sess.infer_host([x], want) == want.size
    assert np.allclose(want, np.maximum(x @ w1 + b1, 0) @ w2 + b2, rtol=1e-4, atol=1e-4)
    dx = torch.from_numpy(x).cuda()
    dy = torch.zeros((128, 10), dtype=torch.float32, device="cuda:0")
    sess.infer_span([dx.data_ptr()], [dy.data_ptr()])
    assert np.array_equal(dy.cpu().numpy(), want)
    with pytest.raises(RuntimeError, match="expected 1 input and 1 output"):
        sess.infer_span([dx.data_ptr(), dx.data_ptr()], [dy.data_ptr()])
    st = sess.pool_stats()
    assert st["pool"] > 0 and st["largest_free"] <= st["free"] <= st["pool"] and 0.0 <= st["fragmentation"] < 1.0
    sess.close()


@pytest.mark.parametrize("n", [1, 8])
def test_dynamic_linear_takes_the_batch_in_the_constructor(n, tmp_path, b200_lib):
    """The reference's DynamicLinear test (tests/alpaka/TestAlpakaLinear.cxx:121-160): Gemm + Relu on an input [N, 4] whose
    leading dimension is symbolic; Session(file, N), infer(N, input); its weights, inputs and 1e-5 bar.  One emitted header
    serves both values of N."""
    import torch
    from sofie_b200.session import EmittedSession
    w = np.array([[0.5, -1.0, 0.25], [0.75, 0.5, -0.5], [-0.25, 1.0, 0.75], [1.5, -0.75, 0.5]], dtype=np.float32)
    b = np.array([0.5, -0.5, 0.25], dtype=np.float32)
    nodes = [{"op": "Gemm", "in": ["X", "W", "B"], "out": ["H"], "attrs": {}}, {"op": "Relu", "in": ["H"], "out": ["Y"], "attrs": {}}]
    sess = EmittedSession("DynamicLinear", nodes, {"W": w, "B": b}, [("X", ["N", 4])], ["Y"], tmp_path, symbolic_dim=n)
    x = ((np.arange(n * 4) % 7) - 3.0).astype(np.float32).reshape(n, 4)
    want = np.maximum(x @ w + b, 0)
    dx = torch.from_numpy(x).cuda()
    out = sess.infer_dim(n, dx.data_ptr())
    got = np.zeros((n, 3), dtype=np.float32)
    assert sess.infer_host([x], got) == 3 * n
    assert np.abs(got - want).max() <= 1e-5
    y = torch.empty((n, 3), dtype=torch.float32, device="cuda:0")
    sess.infer_span([dx.data_ptr()], [y.data_ptr()])
    assert np.abs(y.cpu().numpy() - want).max() <= 1e-5 and out
    with pytest.raises(RuntimeError, match="another value of N"):
        sess.infer_dim(n + 1, dx.data_ptr())
    sess.close()


@pytest.mark.parametrize("n", [1, 5])
def test_dynamic_batched_matmul(n, tmp_path, b200_lib):
    """The reference's DynamicMatMulBatched test (tests/alpaka/TestAlpakaLinear.cxx:162-203): A[N,4,8] x B[N,8,6], both inputs
    with the symbolic leading dimension, which becomes the batch count of one strided-batched contraction."""
    from sofie_b200.session import EmittedSession
    nodes = [{"op": "MatMul", "in": ["A", "B"], "out": ["Y"], "attrs": {}}]
    sess = EmittedSession("DynamicMatMulBatched", nodes, {}, [("A", ["N", 4, 8]), ("B", ["N", 8, 6])], ["Y"], tmp_path, symbolic_dim=n)
    a = (((np.arange(n * 32) % 11) - 5.0) * 0.3).astype(np.float32).reshape(n, 4, 8)
    b = (((np.arange(n * 48) % 7) - 3.0) * 0.5).astype(np.float32).reshape(n, 8, 6)
    got = np.zeros((n, 4, 6), dtype=np.float32)
    assert sess.infer_host([a, b], got) == 24 * n
    assert np.abs(got - np.einsum("nik,nkj->nij", a, b)).max() <= 1e-5
    outs = [np.zeros((n, 4, 6), dtype=np.float32) for _ in range(3)]      # the pipelined queue sizes its buffers from N too
    sess.infer_host_many([[a.ctypes.data] * 3, [b.ctypes.data] * 3], [o.ctypes.data for o in outs])
    assert all(np.array_equal(o, got) for o in outs)
    sess.close()


@pytest.mark.parametrize("n", [1, 6])
def test_dynamic_batchnorm_layernorm_softmax_chain(n, tmp_path, b200_lib):
    """The operators that opt in to a symbolic leading dimension besides the contractions, in one model: BatchNormalization on
    [N, 5, 4, 4] (the reference's DynamicBatchNorm4D shape class), Flatten, LayerNormalization and Softmax over the rows, an
    Add with a per-column tensor.  Against numpy in fp32 at 1e-5."""
    from sofie_b200.session import EmittedSession
    rng = np.random.default_rng(17)
    c = 5
    w = {"s": rng.random(c).astype(np.float32) + 0.5, "b": rng.standard_normal(c).astype(np.float32), "m": rng.standard_normal(c).astype(np.float32),
         "v": rng.random(c).astype(np.float32) + 0.5, "g": rng.standard_normal(80).astype(np.float32), "h": rng.standard_normal(80).astype(np.float32),
         "t": rng.standard_normal(80).astype(np.float32)}
    nodes = [{"op": "BatchNormalization", "in": ["X", "s", "b", "m", "v"], "out": ["B"], "attrs": {"epsilon": 1e-5}},
             {"op": "Flatten", "in": ["B"], "out": ["F"], "attrs": {"axis": 1}},
             {"op": "LayerNormalization", "in": ["F", "g", "h"], "out": ["L"], "attrs": {"axis": -1, "epsilon": 1e-5}},
             {"op": "Softmax", "in": ["L"], "out": ["S"], "attrs": {"axis": -1}},
             {"op": "Add", "in": ["S", "t"], "out": ["Y"], "attrs": {}}]
    sess = EmittedSession("DynamicChain", nodes, w, [("X", ["N", c, 4, 4])], ["Y"], tmp_path, symbolic_dim=n)
    x = rng.standard_normal((n, c, 4, 4)).astype(np.float32)
    bn = (x - w["m"][None, :, None, None]) / np.sqrt(w["v"][None, :, None, None] + 1e-5) * w["s"][None, :, None, None] + w["b"][None, :, None, None]
    f = bn.reshape(n, 80).astype(np.float64)
    ln = (f - f.mean(axis=1, keepdims=True)) / np.sqrt(f.var(axis=1, keepdims=True) + 1e-5) * w["g"] + w["h"]
    e = np.exp(ln - ln.max(axis=1, keepdims=True))
    want = (e / e.sum(axis=1, keepdims=True) + w["t"]).astype(np.float32)
    got = np.zeros((n, 80), dtype=np.float32)
    assert sess.infer_host([x], got) == 80 * n
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    sess.close()
