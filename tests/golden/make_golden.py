"""Generates the golden fixtures under tests/golden/ (run where the reference checkout exists).

For every model listed in oracle/ref_models.list (the reference's own hot-path test models) plus
the benchmark MLP, one <Name>.npz is written holding
  graph     JSON: nodes (op_type, inputs, outputs, attrs), graph inputs with shapes, outputs
  w:<name>  every initializer
  inA<i>    the input the reference's own test feeds (all ones for Linear_*, iota for Conv*, the
            literal vectors of the test source for the others)
  outA      what the UNMODIFIED reference's emitted CPU code (oracle/_ref) computes for inA
  expected  the reference's checked-in expected vector (tests/models/onnx/references/*.ref.hxx),
            when the test that uses it feeds inA
  inB<i>, outB   a seeded N(0,1) input and the reference code's output for it

usage:  make -C oracle ref REF=<reference checkout> && python tests/golden/make_golden.py <reference checkout>
"""
from __future__ import annotations

import ctypes as C
import json
import os
import re
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
from sofie_b200 import onnx_min  # noqa: E402

if len(sys.argv) < 2 and "SOFIE_REFERENCE" not in os.environ:
    sys.exit("usage: make_golden.py <reference checkout>   (or SOFIE_REFERENCE=<path>)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["SOFIE_REFERENCE"])
ONNX_DIR = REF / "tests" / "models" / "onnx"
GEN = ROOT / "oracle" / "_ref" / "gen"

def ref_infer(name: str, inputs: list[np.ndarray], cap: int = 1 << 22) -> np.ndarray:
    """Runs the reference's emitted Session for `name` (oracle/_ref/models/lib<name>.so)."""
    lib = C.CDLL(str(ROOT / "oracle" / "_ref" / "models" / f"lib{name}.so"))
    lib.ref_run.restype = C.c_long
    lib.ref_run.argtypes = [C.POINTER(C.POINTER(C.c_float)), C.c_char_p, C.POINTER(C.c_float), C.c_long]
    lib.ref_last_error.restype = C.c_char_p
    ins = [np.ascontiguousarray(x, dtype=np.float32) for x in inputs]
    ptrs = (C.POINTER(C.c_float) * len(ins))(*[x.ctypes.data_as(C.POINTER(C.c_float)) for x in ins])
    out = np.zeros(cap, dtype=np.float32)
    n = lib.ref_run(ptrs, str(GEN).encode(), out.ctypes.data_as(C.POINTER(C.c_float)), cap)
    if n < 0:
        raise RuntimeError(f"reference code for {name} failed: {lib.ref_last_error().decode()}")
    return out[:n].copy()


def parse_ref_hxx(name: str) -> dict[str, np.ndarray]:
    """Every `float <id>[] = {...};` array of references/<name>.ref.hxx (or .hxx)."""
    for cand in (ONNX_DIR / "references" / f"{name}.ref.hxx", ONNX_DIR / "references" / f"{name}.hxx"):
        if cand.exists():
            text = cand.read_text()
            out = {}
            for m in re.finditer(r"float\s+(\w+)\s*\[\s*\d*\s*\]\s*=\s*\{([^}]*)\}", text, re.S):
                vals = [float(v.rstrip("fF")) for v in re.split(r"[,\s]+", m.group(2).strip()) if v]
                out[m.group(1)] = np.array(vals, dtype=np.float32)
            return out
    return {}


def test_literal_input(test_file: str, test_name: str) -> np.ndarray | None:
    """First brace-enclosed float list after TEST_F(..., <test_name>) in a reference test source."""
    text = (REF / "tests" / "alpaka" / test_file).read_text()
    m = re.search(r"TEST_F\(SofieAlpakaTest,\s*" + re.escape(test_name) + r"\)(.*?)(?=TEST_F\(|\Z)", text, re.S)
    if not m:
        return None
    body = re.sub(r"//[^\n]*", "", m.group(1))
    lst = re.search(r"\{\s*((?:-?[\d.]+(?:e-?\d+)?f?\s*,?\s*)+)\}", body)
    if not lst:
        return None
    vals = [float(v.rstrip("f")) for v in re.split(r"[,\s]+", lst.group(1).strip()) if v]
    return np.array(vals, dtype=np.float32)


# name -> (kind of the reference test's input, test file, test name)
TEST_INPUT = {
    "BatchNorm": ("literal", "TestAlpakaNormalization.cxx", "BatchNormalization"),
    "BatchNormRelu": ("literal", "TestAlpakaNormalization.cxx", "BatchNormalizationRelu"),
    "LayerNorm": ("literal", "TestAlpakaNormalization.cxx", "LayerNorm"),
    "LayerNormScaleBias": ("literal", "TestAlpakaNormalization.cxx", "LayerNormScaleBias"),
    "LayerNorm3D": ("iota", None, None),
    "LinearWithLeakyRelu": ("random", None, None),
    "Softmax1d": ("literal", "TestAlpakaNormalization.cxx", "Softmax1d"),
    "Softmax2d": ("literal", "TestAlpakaNormalization.cxx", "Softmax2d"),
    "Softmax3d": ("literal", "TestAlpakaNormalization.cxx", "Softmax3d"),
    "Softmax4d": ("literal", "TestAlpakaNormalization.cxx", "Softmax4d"),
}


def graph_json(g: onnx_min.Graph) -> str:
    def clean(v):
        if isinstance(v, np.ndarray):
            return v.tolist()
        return v
    return json.dumps({
        "nodes": [{"op": n.op_type, "in": n.inputs, "out": n.outputs, "attrs": {k: clean(v) for k, v in n.attrs.items()}}
                  for n in g.nodes],
        "inputs": [[n, s] for n, s in g.inputs],
        "outputs": g.outputs,
    })


def read_dat(path: Path) -> dict[str, np.ndarray]:
    """Text weight file written by the reference (core/src/RModel.cxx:1919-1961)."""
    toks = path.read_text().split()
    out, i = {}, 0
    while i < len(toks):
        name, n = toks[i], int(toks[i + 1])
        out[name.removeprefix("tensor_")] = np.array(toks[i + 2:i + 2 + n], dtype=np.float64).astype(np.float32)
        i += 2 + n
    return out


def main() -> None:
    names = [l.strip() for l in (ROOT / "oracle" / "ref_models.list").read_text().splitlines() if l.strip() and not l.startswith("#")]
    rng = np.random.default_rng(20240607)
    for name in names:
        g = onnx_min.load(str(ONNX_DIR / f"{name}.onnx"))
        shapes = [tuple(s) for _, s in g.inputs]
        kind = TEST_INPUT.get(name, ("ones" if name.startswith("Linear") else "iota" if name.startswith("Conv") else "random", None, None))
        ins_a = []
        for shp in shapes:
            n = int(np.prod(shp))
            if kind[0] == "ones":
                ins_a.append(np.ones(shp, dtype=np.float32))
            elif kind[0] == "iota":
                ins_a.append(np.arange(n, dtype=np.float32).reshape(shp))
            elif kind[0] == "literal":
                lit = test_literal_input(kind[1], kind[2])
                if lit is None or lit.size != n:
                    raise RuntimeError(f"{name}: literal input not found in {kind[1]} ({None if lit is None else lit.size} vs {n})")
                ins_a.append(lit.reshape(shp))
            else:
                ins_a.append(rng.standard_normal(shp).astype(np.float32))
        ins_b = [rng.standard_normal(shp).astype(np.float32) for shp in shapes]
        if name == "SDPA":      # the reference test's own operands (tests/alpaka/TestAlpakaSequenceOps.cxx: SDPA)
            lit = parse_ref_hxx("SDPA_input")
            ins_a = [lit[k].reshape(shp) for k, shp in zip(("Q", "K", "V"), shapes)]
        if name == "SDPABig":   # the generator of the reference test (same file: SDPABig): an LCG, every fifth key masked
            state = 12345
            def rnd():
                nonlocal state
                state = (1103515245 * state + 12345) & 0xFFFFFFFF
                return np.float32(np.float32(state & 0x7FFFFFFF) / np.float32(0x7FFFFFFF)) * np.float32(2.0) - np.float32(1.0)
            n = int(np.prod(shapes[0]))
            qkv = np.array([rnd() for _ in range(3 * n)], dtype=np.float32).reshape(n, 3)
            mask = np.where(np.arange(int(np.prod(shapes[3]))) % 5 == 0, np.float32(-1e9), np.float32(0)).astype(np.float32)
            ins_a = [qkv[:, 0].reshape(shapes[0]).copy(), qkv[:, 1].reshape(shapes[1]).copy(), qkv[:, 2].reshape(shapes[2]).copy(), mask.reshape(shapes[3])]
            ins_b[3] = np.where(rng.random(shapes[3]) < 0.2, np.float32(-1e9), np.float32(0)).astype(np.float32)
            ins_b[3][..., 0] = 0   # never a fully masked row
        out_a, out_b = ref_infer(name, ins_a), ref_infer(name, ins_b)
        arrays = {"graph": np.array(graph_json(g)), "outA": out_a, "outB": out_b}
        for i, (a, b) in enumerate(zip(ins_a, ins_b)):
            arrays[f"inA{i}"], arrays[f"inB{i}"] = a, b
        for k, v in g.initializers.items():
            arrays[f"w:{k}"] = v
        exp = parse_ref_hxx(name)
        if exp and (kind[0] in ("ones", "iota", "literal") or name == "SDPA"):
            first = next(iter(exp.values()))
            if first.size == out_a.size:
                arrays["expected"] = first
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        tag = ""
        if "expected" in arrays:
            tag = f" max|ref_code - expected| = {np.abs(out_a - arrays['expected']).max():.3g}"
        print(f"{name}: out {out_a.size}{tag}")

    # the benchmark MLP built through the reference's C++ model API by oracle/ref_emit.cxx
    w = read_dat(GEN / "MLP_C1.dat")
    nodes = []
    prev = "X"
    for l in range(3):
        out = "Y" if l == 2 else f"H{l}"
        nodes.append({"op": "Gemm", "in": [prev, f"W{l}", f"B{l}"], "out": [out], "attrs": {"alpha": 1.0, "beta": 1.0}})
        if l < 2:
            nodes.append({"op": "Relu", "in": [out], "out": [out + "r"], "attrs": {}})
            prev = out + "r"
    dims = [64, 256, 256, 10]
    x = rng.standard_normal((1024, 64)).astype(np.float32)
    arrays = {"graph": np.array(json.dumps({"nodes": nodes, "inputs": [["X", [1024, 64]]], "outputs": ["Y"]})),
              "inA0": x, "outA": ref_infer("MLP_C1", [x])}
    for l in range(3):
        arrays[f"w:W{l}"] = w[f"W{l}"].reshape(dims[l], dims[l + 1])
        arrays[f"w:B{l}"] = w[f"B{l}"]
    np.savez_compressed(HERE / "MLP_C1.npz", **arrays)
    print("MLP_C1: out", arrays["outA"].size)

    # The conv-net and transformer-encoder configurations at reduced size, built through the reference's C++ model API by
    # oracle/ref_emit.cxx with weights from the reproducible generator (sofie_b200/synth.py): the fixtures hold only the
    # input and what the reference's emitted code computed; the tests draw the same weights again.
    sys.path.insert(0, str(ROOT))
    from sofie_b200 import synth
    from sofie_b200.encoder import bf16_bits_to_f32, f32_to_bf16_bits
    (HERE / "configs").mkdir(exist_ok=True)
    x = synth.uniform_f32(synth.tensor_seed(11, 900), (2, 3, 32, 32), 0.0, 1.0)
    y = ref_infer("ConvNet_C4r", [x]).reshape(2, 1000)
    np.savez_compressed(HERE / "configs" / "ConvNet_C4r.npz", x=x, y=y, seed=np.int64(11))
    print("ConvNet_C4r: out", y.shape, "rms", float(np.sqrt(np.mean(y * y))))
    # encoder input: N(0,1) tokens rounded to bf16 (the GPU path's activation type), given to the reference as fp32
    xe = bf16_bits_to_f32(f32_to_bf16_bits(synth.normal_f32(synth.tensor_seed(7, 900), (2 * 128, 512), 1.0)))
    ye = ref_infer("Encoder_C5r", [xe]).reshape(2 * 128, 512)
    np.savez_compressed(HERE / "configs" / "Encoder_C5r.npz", x=xe, y=ye, seed=np.int64(7), layers=np.int64(2), batch=np.int64(2))
    print("Encoder_C5r: out", ye.shape, "absmax", float(np.abs(ye).max()))


if __name__ == "__main__":
    main()
