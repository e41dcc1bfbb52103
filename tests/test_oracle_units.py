"""Known-answer tests of the checker's element conversions and quantisation rules."""
import ctypes as C

import numpy as np
import pytest
import torch

from sofie_b200 import lib as L


@pytest.fixture(scope="module")
def o(oracle_lib):
    lib = C.CDLL(str(oracle_lib))
    lib.so_e4m3_to_f32.restype = C.c_float
    lib.so_e4m3_to_f32.argtypes = [C.c_uint8]
    lib.so_f32_to_e4m3.restype = C.c_uint8
    lib.so_f32_to_e4m3.argtypes = [C.c_float]
    lib.so_bf16_to_f32.restype = C.c_float
    lib.so_bf16_to_f32.argtypes = [C.c_uint16]
    lib.so_f32_to_bf16.restype = C.c_uint16
    lib.so_f32_to_bf16.argtypes = [C.c_float]
    return lib


def test_e4m3_decode_matches_torch_for_all_codes(o):
    codes = torch.arange(256, dtype=torch.uint8)
    want = codes.view(torch.float8_e4m3fn).float().numpy()
    got = np.array([o.so_e4m3_to_f32(int(c)) for c in range(256)], dtype=np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])


def test_e4m3_encode_round_trips_every_finite_code(o):
    for c in range(256):
        v = o.so_e4m3_to_f32(c)
        if v != v:
            continue
        back = o.so_f32_to_e4m3(v)
        assert back == c or (v == 0.0 and back in (0x00, 0x80)), (c, v, back)


def test_e4m3_encode_rounds_to_nearest_even_and_saturates(o):
    assert o.so_e4m3_to_f32(o.so_f32_to_e4m3(1.0625)) == 1.0    # tie between 1.0 and 1.125 -> even mantissa
    assert o.so_e4m3_to_f32(o.so_f32_to_e4m3(1.1875)) == 1.25   # tie between 1.125 and 1.25 -> even mantissa
    assert o.so_e4m3_to_f32(o.so_f32_to_e4m3(500.0)) == 448.0
    assert o.so_e4m3_to_f32(o.so_f32_to_e4m3(-1e9)) == -448.0
    assert o.so_e4m3_to_f32(o.so_f32_to_e4m3(2.0 ** -10)) == 0.0       # half of the smallest subnormal: ties to even (0)
    assert o.so_e4m3_to_f32(o.so_f32_to_e4m3(3 * 2.0 ** -10)) == 2.0 ** -8  # 1.5 quanta -> 2 quanta (even)
    x = torch.randn(20000) * 40
    x = x[x.abs() <= 448]
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([o.so_f32_to_e4m3(float(v)) for v in x.numpy()], dtype=np.uint8)
    assert np.array_equal(got, want)


def test_bf16_matches_torch(o):
    x = torch.randn(20000) * 1e3
    want = x.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    got = np.array([o.so_f32_to_bf16(float(v)) for v in x.numpy()], dtype=np.uint16)
    assert np.array_equal(got, want)
    assert o.so_bf16_to_f32(0x3F80) == 1.0


def test_qlinear_requantisation_known_answers(oracle_lib):
    """acc * M with round-half-to-even and saturation (ONNX QLinearMatMul)."""
    lib = C.CDLL(str(oracle_lib))
    a = np.array([[1, 1, 1, 1], [127, 127, 127, 127], [-127, 127, 0, 3]], dtype=np.int8)
    b = np.array([[1, 2], [1, 2], [1, 2], [2, -1]], dtype=np.int8).copy()
    d = L.GemmDesc()
    d.M, d.N, d.K, d.batch, d.ab_dtype, d.y_dtype = 3, 2, 4, 1, L.I8, L.I8
    e = L.Epilogue()
    e.alpha, e.beta, e.out_scale = 0.5, 1.0, 1.0
    y = np.zeros((3, 2), dtype=np.int8)
    lib.so_gemm(C.byref(d), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), C.byref(e))
    # acc = [[5,5],[635,635],[6,-3]] -> *0.5 = [[2.5,2.5],[317.5,..],[3,-1.5]] -> half to even, saturate
    assert y.tolist() == [[2, 2], [127, 127], [3, -2]]
    e.out_zero_point = 10
    y2 = np.zeros((3, 2), dtype=np.int8)
    lib.so_gemm(C.byref(d), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), y2.ctypes.data_as(C.c_void_p), C.byref(e))
    assert y2.tolist() == [[12, 12], [127, 127], [13, 8]]


def test_quantize_dequantize_per_channel(oracle_lib):
    lib = C.CDLL(str(oracle_lib))
    x = np.array([[0.26, -0.74], [1.0, 300.0]], dtype=np.float32)  # channels on axis 0, inner 2
    scale = np.array([0.5, 2.0], dtype=np.float32)
    zp = np.array([0, -3], dtype=np.int32)
    q = np.zeros(4, dtype=np.int8)
    lib.so_quantize(x.ctypes.data_as(C.c_void_p), q.ctypes.data_as(C.c_void_p), L.I8, C.c_int64(4), scale.ctypes.data_as(C.c_void_p),
                    zp.ctypes.data_as(C.c_void_p), C.c_int64(2), C.c_int64(2))
    # 0.26/0.5 = 0.52 -> 1;  -0.74/0.5 = -1.48 -> -1;  1/2 = 0.5 -> 0 (half to even), -3 -> -3;  150 - 3 -> saturates
    assert q.tolist() == [1, -1, -3, 127]
