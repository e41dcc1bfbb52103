"""The C++ code generator (sofie_b200/host): ONNX -> RModel -> fusion -> arena -> emitted Session.

CPU part: every golden model is written as an ONNX file, parsed and emitted; the emitted header must
compile against include/sofie_b200.h and the CUDA runtime headers, and generation must take the
decisions the design states (activation / BatchNormalization / residual folding, lifetime reuse in the
arena, loud errors for what is off the path).  GPU part: the emitted Session is compiled, loaded and run
on cuda:0, and must reproduce what the reference's own emitted CPU code computed.
"""
import ctypes as C
import json
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

import graph_runner as gr
from sofie_b200 import onnx_min
from sofie_b200 import build as B

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = sorted(p.stem for p in (ROOT / "tests" / "golden").glob("*.npz"))
EMITTABLE = GOLDEN


@pytest.fixture(scope="session")
def emit():
    return B.build_host()


def write_onnx(fx, path):
    g = fx["graph"]
    onnx_min.save(str(path), g["nodes"], fx["weights"], [(n, s) for n, s in g["inputs"]], g["outputs"])


def run_emit(emit, onnx_path, out_hxx, *flags):
    r = subprocess.run([str(emit), str(onnx_path), str(out_hxx), *flags], capture_output=True, text=True)
    return r.returncode, r.stdout, r.stderr


def syntax_check(header):
    cmd = ["g++", "-std=c++20", "-fsyntax-only", f"-I{ROOT / 'include'}", f"-I{B.cuda_include_dir()}", "-x", "c++", "-"]
    src = f'#include "{header}"\n'
    return subprocess.run(cmd, input=src, capture_output=True, text=True)


@pytest.mark.parametrize("name", EMITTABLE)
def test_emit_and_compile_every_golden_model(name, emit, tmp_path):
    fx = gr.load_fixture(name)
    write_onnx(fx, tmp_path / f"{name}.onnx")
    rc, out, err = run_emit(emit, tmp_path / f"{name}.onnx", tmp_path / f"{name}.hxx")
    assert rc == 0, err
    rep = json.loads(out)
    assert rep["model"] == name and rep["arena_bytes"] % 256 == 0
    text = (tmp_path / f"{name}.hxx").read_text()
    assert f"namespace SOFIE_{name}" in text and "struct Session" in text
    for member in ("infer(", "infer_nosync(", "_infer_impl(", "infer_host(", "resetState()"):
        assert member in text
    # one arena allocation at construction; the only other one is the lazy queue buffer of infer_host_many
    assert "alpaka" not in text and text.count('"arena allocation"') == 1 and text.count("cudaMalloc(") == 2 and '"queue buffers"' in text
    for member in ("Enqueue(", "SetUseCudaGraph(", "infer_host_many(", "cudaGraphLaunch("):
        assert member in text
    # the reference's span form of infer and its pool statistics (RModel_ALPAKA.cxx:814-838, 1262-1269)
    for member in ("infer(std::span<const void *const> inputs, std::span<void *const> outputs)", "GetTotalFreeMemory()", "GetLargestFreeBlock()",
                   "GetFragmentation()", "GetIntermediateMemoryPoolSize()"):
        assert member in text
    chk = syntax_check(tmp_path / f"{name}.hxx")
    assert chk.returncode == 0, chk.stderr[:2000]


def test_activation_folds_into_gemm(emit, tmp_path):
    fx = gr.load_fixture("Linear_16")
    write_onnx(fx, tmp_path / "Linear_16.onnx")
    rc, out, err = run_emit(emit, tmp_path / "Linear_16.onnx", tmp_path / "Linear_16.hxx")
    rep = json.loads(out)
    n_gemm = sum(n["op"] == "Gemm" for n in fx["graph"]["nodes"])
    n_relu = sum(n["op"] == "Relu" for n in fx["graph"]["nodes"])
    assert len(rep["fusions"]) == n_relu  # every Relu became a Gemm epilogue
    text = (tmp_path / "Linear_16.hxx").read_text()
    assert text.count("sofie_b200_gemm_enqueue(") == n_gemm and "sofie_b200_unary_enqueue" not in text
    assert text.count("SOFIE_B200_ACT_RELU") == n_relu
    # 9 hidden activations of 16x50 floats are alive two at a time: the pool holds two of them
    assert rep["pool_bytes"] == 2 * 3328 and rep["unplanned_pool_bytes"] == 9 * 3328


def test_batchnorm_and_residual_fold_into_conv(emit, tmp_path):
    rng = np.random.default_rng(0)
    w = {"W": rng.standard_normal((8, 4, 3, 3)).astype(np.float32), "B": rng.standard_normal(8).astype(np.float32),
         "scale": rng.random(8).astype(np.float32) + 0.5, "beta": rng.standard_normal(8).astype(np.float32),
         "mean": rng.standard_normal(8).astype(np.float32), "var": rng.random(8).astype(np.float32) + 0.5}
    nodes = [{"op": "Conv", "in": ["X", "W", "B"], "out": ["c"], "attrs": {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]}},
             {"op": "BatchNormalization", "in": ["c", "scale", "beta", "mean", "var"], "out": ["bn"], "attrs": {"epsilon": 1e-5}},
             {"op": "Relu", "in": ["bn"], "out": ["r"], "attrs": {}},
             {"op": "Conv", "in": ["r", "W2"], "out": ["c2"], "attrs": {"kernel_shape": [1, 1], "pads": [0, 0, 0, 0]}},
             {"op": "Add", "in": ["c2", "r"], "out": ["Y"], "attrs": {}}]
    w["W2"] = rng.standard_normal((8, 8, 1, 1)).astype(np.float32)
    onnx_min.save(str(tmp_path / "m.onnx"), nodes, w, [("X", [2, 4, 6, 6])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "m.onnx", tmp_path / "m.hxx")
    assert rc == 0, err
    rep = json.loads(out)
    kinds = " ".join(rep["fusions"])
    assert "BatchNormalization as column scale + shift" in kinds and "residual Add" in kinds and "activation" in kinds
    text = (tmp_path / "m.hxx").read_text()
    assert text.count("sofie_b200_conv_enqueue(") == 2
    assert "batchnorm_enqueue" not in text and "binary_enqueue" not in text and "unary_enqueue" not in text
    assert ".residual = tensor_r" in text
    assert syntax_check(tmp_path / "m.hxx").returncode == 0


def test_a_shared_output_is_not_folded(emit, tmp_path):
    # the Gemm result feeds a Relu AND is a graph output: the reference's legality rule forbids the fold
    rng = np.random.default_rng(1)
    w = {"W": rng.standard_normal((8, 4)).astype(np.float32), "b": rng.standard_normal(4).astype(np.float32)}
    nodes = [{"op": "Gemm", "in": ["X", "W", "b"], "out": ["g"], "attrs": {}}, {"op": "Relu", "in": ["g"], "out": ["r"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "m.onnx"), nodes, w, [("X", [3, 8])], ["r", "g"])
    rc, out, err = run_emit(emit, tmp_path / "m.onnx", tmp_path / "m.hxx")
    assert rc == 0, err
    assert json.loads(out)["fusions"] == []
    assert "sofie_b200_unary_enqueue" in (tmp_path / "m.hxx").read_text()


def test_batchnorm_after_a_stacked_matmul_is_not_folded(emit, tmp_path):
    # [B,S,S] product: BatchNormalization's channel axis is dimension 1, the ROWS of each product, so a per-column fold
    # would scale the wrong axis even though the sizes match
    rng = np.random.default_rng(4)
    w = {"W": rng.standard_normal((6, 6)).astype(np.float32), "scale": rng.random(6).astype(np.float32) + 0.5,
         "beta": rng.standard_normal(6).astype(np.float32), "mean": rng.standard_normal(6).astype(np.float32),
         "var": rng.random(6).astype(np.float32) + 0.5}
    nodes = [{"op": "MatMul", "in": ["X", "W"], "out": ["m"], "attrs": {}},
             {"op": "BatchNormalization", "in": ["m", "scale", "beta", "mean", "var"], "out": ["Y"], "attrs": {"epsilon": 1e-5}}]
    onnx_min.save(str(tmp_path / "m.onnx"), nodes, w, [("X", [2, 6, 6])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "m.onnx", tmp_path / "m.hxx")
    assert rc == 0, err
    assert json.loads(out)["fusions"] == []
    assert "sofie_b200_batchnorm_enqueue" in (tmp_path / "m.hxx").read_text()
    # the rank-2 product does fold
    onnx_min.save(str(tmp_path / "n.onnx"), nodes, w, [("X", [5, 6])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "n.onnx", tmp_path / "n.hxx")
    assert rc == 0, err
    assert len(json.loads(out)["fusions"]) == 1 and "batchnorm_enqueue" not in (tmp_path / "n.hxx").read_text()


def test_matmul_add_becomes_gemm_with_bias_and_transpose_is_absorbed(emit, tmp_path):
    rng = np.random.default_rng(2)
    w = {"Wt": rng.standard_normal((5, 8)).astype(np.float32), "b": rng.standard_normal(5).astype(np.float32)}
    nodes = [{"op": "Transpose", "in": ["Wt"], "out": ["W"], "attrs": {"perm": [1, 0]}},
             {"op": "MatMul", "in": ["X", "W"], "out": ["m"], "attrs": {}},
             {"op": "Add", "in": ["m", "b"], "out": ["Y"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "m.onnx"), nodes, w, [("X", [3, 8])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "m.onnx", tmp_path / "m.hxx")
    assert rc == 0, err
    text = (tmp_path / "m.hxx").read_text()
    assert json.loads(out)["operators"] == 1
    assert "d.trans_b = 1" in text and "SOFIE_B200_BIAS_COL_F32" in text and "binary_enqueue" not in text


def test_quantised_nodes_parse_and_fix_the_multiplier(emit, tmp_path):
    rng = np.random.default_rng(3)
    w = {"B": rng.integers(-127, 128, size=(64, 32), dtype=np.int8), "a_scale": np.array(0.02, dtype=np.float32),
         "a_zp": np.array(0, dtype=np.int8), "b_scale": np.array(0.01, dtype=np.float32), "b_zp": np.array(0, dtype=np.int8),
         "y_scale": np.array(0.5, dtype=np.float32), "y_zp": np.array(0, dtype=np.int8)}
    nodes = [{"op": "QLinearMatMul", "in": ["A", "a_scale", "a_zp", "B", "b_scale", "b_zp", "y_scale", "y_zp"], "out": ["Y"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "q.onnx"), nodes, w, [("A", [16, 64])], ["Y"], input_types={"A": 3})
    rc, out, err = run_emit(emit, tmp_path / "q.onnx", tmp_path / "q.hxx")
    assert rc == 0, err
    text = (tmp_path / "q.hxx").read_text()
    mult = np.float32(np.float32(0.02) * np.float32(0.01)) / np.float32(0.5)
    assert "d.ab_dtype = SOFIE_B200_I8; d.y_dtype = SOFIE_B200_I8" in text
    assert f"{mult:.9g}" in text  # the fp32 multiplier a_scale*b_scale/y_scale is a generation-time constant
    assert "int8_t *infer(const int8_t *tensor_A)" in text
    assert syntax_check(tmp_path / "q.hxx").returncode == 0


def test_options_change_the_session_surface(emit, tmp_path):
    fx = gr.load_fixture("Linear_16")
    write_onnx(fx, tmp_path / "Linear_16.onnx")
    rc, out, err = run_emit(emit, tmp_path / "Linear_16.onnx", tmp_path / "a.hxx", "--external-stream", "--custom-memory", "--profile", "--debug",
                            "--no-weight-file")
    assert rc == 0, err
    text = (tmp_path / "a.hxx").read_text()
    assert "Session(MemoryProvider provider, cudaStream_t externalStream" in text
    assert "cudaMalloc(" not in text and "fProvider.alloc(kArenaBytes" in text and "fProvider.dealloc(" in text
    assert "ValidateMemory()" in text and "GetOpAvgTime" in text and "fWeights_0_weight[]" in text
    assert not (tmp_path / "Linear_16.dat").exists()
    assert syntax_check(tmp_path / "a.hxx").returncode == 0


def test_unsupported_operators_fail_loudly(emit, tmp_path):
    onnx_min.save(str(tmp_path / "u.onnx"), [{"op": "LSTM", "in": ["X"], "out": ["Y"], "attrs": {}}], {}, [("X", [2, 3])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "u.onnx", tmp_path / "u.hxx")
    assert rc != 0 and "SOFIE Operator type LSTM is not yet supported" in err
    rc, out, err = run_emit(emit, tmp_path / "u.onnx", tmp_path / "u.hxx", "--check")
    assert rc == 1 and "operator LSTM is not supported" in out
    # a Gemm bias that cannot broadcast to the result: the reference's message
    w = {"W": np.zeros((8, 4), dtype=np.float32), "b": np.zeros(3, dtype=np.float32)}
    onnx_min.save(str(tmp_path / "g.onnx"), [{"op": "Gemm", "in": ["X", "W", "b"], "out": ["Y"], "attrs": {}}], w, [("X", [3, 8])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "g.onnx", tmp_path / "g.hxx")
    assert rc != 0 and "cannot be uni-directional broadcasted" in err
    # a batch size fixes the dimensions named bs / batch_size / input_size at generation
    onnx_min.save(str(tmp_path / "d.onnx"), [{"op": "Relu", "in": ["X"], "out": ["Y"], "attrs": {}}], {}, [("X", ["bs", 3])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "d.onnx", tmp_path / "d.hxx", "--batch", "7")
    assert rc == 0 and "unary_enqueue(ctx, tensor_X, tensor_Y, SOFIE_B200_F32, 21," in (tmp_path / "d.hxx").read_text()


def test_a_symbolic_leading_dimension_reaches_the_session_constructor(emit, tmp_path):
    """The reference's dynamic models (tests/alpaka/TestAlpakaLinear.cxx:121-203): Session(file, N) and infer(N, inputs)."""
    w = {"W": np.ones((4, 3), dtype=np.float32), "B": np.zeros(3, dtype=np.float32), "g": np.ones(3, dtype=np.float32)}
    nodes = [{"op": "Gemm", "in": ["X", "W", "B"], "out": ["H"], "attrs": {}}, {"op": "Relu", "in": ["H"], "out": ["R"], "attrs": {}},
             {"op": "Softmax", "in": ["R"], "out": ["S"], "attrs": {"axis": -1}}, {"op": "Add", "in": ["S", "g"], "out": ["Y"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "dyn.onnx"), nodes, w, [("X", ["N", 4])], ["Y"])
    for flags in ((), ("--debug", "--profile"), ("--external-stream", "--custom-memory"), ("--safetensors",), ("--no-weight-file",)):
        rc, out, err = run_emit(emit, tmp_path / "dyn.onnx", tmp_path / "dyn.hxx", *flags)
        assert rc == 0, err
        text = (tmp_path / "dyn.hxx").read_text()
        assert "std::string filename, size_t N_value) : fDim_N(N_value)" in text
        assert "d.M = (size_t(1) * fDim_N);" in text and "*infer(size_t N_value, const float *tensor_X)" in text
        assert "softmax_enqueue(ctx, tensor_R, tensor_S, SOFIE_B200_F32, SOFIE_B200_F32, (size_t(1) * fDim_N), 3, 0)" in text
        assert "static constexpr size_t kArenaBytes" not in text and "const size_t kArenaBytes = (size_t(" in text
        assert re.search(r"(?<![\w.])\d{11,}(?![\w.])", text) is None          # no number still carries the stand-in for N
        chk = syntax_check(tmp_path / "dyn.hxx")
        assert chk.returncode == 0, chk.stderr[-2000:]
    # every offset of the arena is a sum of aligned sizes: a multiple of 256 for every N
    for m in re.finditer(r"fArena \+ \(size_t\((\d+)\) \* fDim_N(?: \+ (\d+))?\)", text):
        assert int(m.group(1)) % 256 == 0 and int(m.group(2) or 0) % 256 == 0
    # a Reshape that keeps the dimension in front is free (an alias); one that moves it inward is refused
    rw = {"W": np.ones((48, 5), dtype=np.float32), "keep": np.array([0, -1], dtype=np.int64), "move": np.array([4, -1], dtype=np.int64)}
    rn = [{"op": "Relu", "in": ["X"], "out": ["R"], "attrs": {}}, {"op": "Reshape", "in": ["R", "keep"], "out": ["F"], "attrs": {}},
          {"op": "MatMul", "in": ["F", "W"], "out": ["Y"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "resh.onnx"), rn, rw, [("X", ["N", 3, 4, 4])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "resh.onnx", tmp_path / "resh.hxx", "--no-weight-file")
    text = (tmp_path / "resh.hxx").read_text()
    assert rc == 0 and "d.M = (size_t(1) * fDim_N); d.N = 5; d.K = 48;" in text and "fWeights_W[] = {1,1,1," in text
    assert json.loads(out)["arena_bytes_per_unit"] == 768 and syntax_check(tmp_path / "resh.hxx").returncode == 0
    rn[1]["in"] = ["R", "move"]
    onnx_min.save(str(tmp_path / "resh2.onnx"), rn[:2], rw, [("X", ["N", 3, 4, 4])], ["F"])
    rc, out, err = run_emit(emit, tmp_path / "resh2.onnx", tmp_path / "resh2.hxx")
    assert rc != 0 and "in an inner position" in err
    # what the target cannot carry is refused with the reason
    onnx_min.save(str(tmp_path / "two.onnx"), [{"op": "Add", "in": ["A", "B"], "out": ["Y"], "attrs": {}}], {}, [("A", ["N", 4]), ("B", ["M", 4])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "two.onnx", tmp_path / "two.hxx")
    assert rc != 0 and "one symbolic dimension per model" in err
    onnx_min.save(str(tmp_path / "inner.onnx"), [{"op": "Relu", "in": ["X"], "out": ["Y"], "attrs": {}}], {}, [("X", [2, "L"])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "inner.onnx", tmp_path / "inner.hxx")
    assert rc != 0 and "only a leading (batch) dimension may be symbolic" in err
    cw = {"F": np.zeros((4, 3, 3, 3), dtype=np.float32)}
    onnx_min.save(str(tmp_path / "conv.onnx"), [{"op": "Conv", "in": ["X", "F"], "out": ["Y"], "attrs": {"kernel_shape": [3, 3]}}], cw, [("X", ["N", 3, 8, 8])], ["Y"])
    rc, out, err = run_emit(emit, tmp_path / "conv.onnx", tmp_path / "conv.hxx")
    assert rc != 0 and "needs static shapes" in err and "symbolic dimension N" in err


# ---- on the GPU: the emitted Session against the reference's own results ----------------------------------
WRAPPER = """
#include "{header}"
#include <cstring>
static std::string g_err;
extern "C" const char *session_error() {{ return g_err.c_str(); }}
extern "C" long session_run(const char *datfile, const float *const *in, float *out, long cap, long long *launches) {{
   try {{
      SOFIE_{name}::Session s(datfile);
      std::vector<float> y = s.infer_host({args});
      *launches = s.GetLaunchCount();
      std::memcpy(out, y.data(), sizeof(float) * (y.size() < (size_t)cap ? y.size() : (size_t)cap));
      return (long)y.size();
   }} catch (const std::exception &e) {{ g_err = e.what(); return -1; }}
}}
"""


@pytest.mark.gpu
@pytest.mark.parametrize("name", EMITTABLE)
def test_emitted_session_reproduces_reference_results(name, emit, tmp_path, b200_lib):
    fx = gr.load_fixture(name)
    write_onnx(fx, tmp_path / f"{name}.onnx")
    rc, out, err = run_emit(emit, tmp_path / f"{name}.onnx", tmp_path / f"{name}.hxx", "--debug")
    assert rc == 0, err
    nin = len(fx["graph"]["inputs"])
    src = WRAPPER.format(header=tmp_path / f"{name}.hxx", name=name, args=", ".join(f"in[{i}]" for i in range(nin)))
    so = B.compile_session(tmp_path / f"{name}.hxx", tmp_path / f"libsession_{name}.so", src)
    lib = C.CDLL(str(so))
    lib.session_run.restype = C.c_long
    lib.session_error.restype = C.c_char_p
    for tag in ("A", "B"):
        if f"out{tag}" not in fx:
            continue
        ins = [np.ascontiguousarray(fx[k], dtype=np.float32) for k in sorted(fx) if k.startswith(f"in{tag}")]
        ptrs = (C.POINTER(C.c_float) * nin)(*[x.ctypes.data_as(C.POINTER(C.c_float)) for x in ins])
        want = fx[f"out{tag}"]
        got = np.zeros(want.size, dtype=np.float32)
        launches = C.c_longlong()
        n = lib.session_run(str(tmp_path / f"{name}.dat").encode(), ptrs, got.ctypes.data_as(C.POINTER(C.c_float)), got.size, C.byref(launches))
        assert n == want.size, lib.session_error().decode()
        floor = float(np.sqrt(np.mean(np.square(want))))
        assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), floor)), f"{name}/{tag}: {np.abs(got - want).max():.3g}"
        assert launches.value >= 1


def test_safetensors_weight_file_round_trips_low_precision_types(emit, tmp_path):
    """Options::kSafetensorsWeightFile: the generator writes <model>.safetensors in the reference's layout (8-byte header size,
    JSON header with sorted names, raw payload; core/src/RModel.cxx:1967-2010) with I8, F32 and the other types of this
    target; every weight must come back bit for bit, and the emitted Session must read that file."""
    from safetensors import safe_open
    rng = np.random.default_rng(9)
    w = {"B": rng.integers(-127, 128, size=(64, 32), dtype=np.int8), "a_scale": np.array(0.02, dtype=np.float32),
         "a_zp": np.array(0, dtype=np.int8), "b_scale": np.array(0.01, dtype=np.float32), "b_zp": np.array(0, dtype=np.int8),
         "y_scale": np.array(0.5, dtype=np.float32), "y_zp": np.array(0, dtype=np.int8)}
    nodes = [{"op": "QLinearMatMul", "in": ["A", "a_scale", "a_zp", "B", "b_scale", "b_zp", "y_scale", "y_zp"], "out": ["Y"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "q.onnx"), nodes, w, [("A", [16, 64])], ["Y"], input_types={"A": 3})
    rc, out, err = run_emit(emit, tmp_path / "q.onnx", tmp_path / "q.hxx", "--safetensors")
    assert rc == 0, err
    assert not (tmp_path / "q.dat").exists()
    with safe_open(str(tmp_path / "q.safetensors"), framework="numpy") as f:
        assert "tensor_B" in f.keys()
        assert np.array_equal(f.get_tensor("tensor_B"), w["B"]) and f.get_tensor("tensor_B").dtype == np.int8
    text = (tmp_path / "q.hxx").read_text()
    assert 'std::string filename = "q.safetensors"' in text and 'FindSafetensor(blob, "tensor_B", "I8", 2048)' in text
    assert "ReadTensorFromStream(f" not in text
    assert syntax_check(tmp_path / "q.hxx").returncode == 0
    # bf16 and fp8 initializers: written as BF16 / F8_E4M3, payload bytes untouched
    bits16 = rng.integers(0, 0x7F00, size=(8, 16)).astype(np.uint16)
    bits8 = rng.integers(0, 0x70, size=(16, 8)).astype(np.uint8)
    nodes = [{"op": "Add", "in": ["X", "W16"], "out": ["Y"], "attrs": {}}]
    onnx_min.save(str(tmp_path / "b.onnx"), nodes, {"W16": bits16, "unused8": bits8}, [("X", [8, 16])], ["Y"], input_types={"X": 16},
                  initializer_types={"W16": 16, "unused8": 17})
    rc, out, err = run_emit(emit, tmp_path / "b.onnx", tmp_path / "b.hxx", "--safetensors")
    assert rc == 0, err
    raw = (tmp_path / "b.safetensors").read_bytes()
    hs = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + hs])
    e = header["tensor_W16"]
    assert e["dtype"] == "BF16" and e["shape"] == [8, 16]
    assert raw[8 + hs + e["data_offsets"][0]:8 + hs + e["data_offsets"][1]] == bits16.tobytes()
    if "tensor_unused8" in header:
        assert header["tensor_unused8"]["dtype"] == "F8_E4M3"
