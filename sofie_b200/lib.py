"""ctypes binding of libsofie_b200.so (the C ABI declared in include/sofie_b200.h).

This module only loads the library and describes its structs and prototypes.  There is no
fallback: if the library has not been built, or a symbol is missing, importing the package on a
GPU machine fails loudly instead of computing anything on the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libsofie_b200.so"

# enums of include/sofie_b200.h
F32, BF16, I8, F8E4M3, I32, U8 = range(6)
ACT_NONE, ACT_RELU, ACT_GELU_ERF, ACT_GELU_TANH, ACT_LEAKY_RELU, ACT_SIGMOID = range(6)
BIAS_NONE, BIAS_COL_F32, BIAS_ROW_F32, BIAS_SCALAR_F32, BIAS_COL_I32, BIAS_FULL_F32, BIAS_ROW_I32 = range(7)
OK, ERR_INVALID, ERR_CUDA, ERR_DEVICE_WAIT, ERR_NO_DEVICE, ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5
ABI_VERSION = 2
GEMM_B_CONSTANT = 1
GEMM_WIDE_STORES = 2
CONV_UNFOLD = 1


class Epilogue(C.Structure):
    _fields_ = [
        ("row_scale", C.c_void_p),
        ("col_scale", C.c_void_p),
        ("alpha", C.c_float),
        ("beta", C.c_float),
        ("bias_mode", C.c_int32),
        ("bias", C.c_void_p),
        ("ldc", C.c_int64),
        ("residual", C.c_void_p),
        ("residual_dtype", C.c_int32),
        ("ldr", C.c_int64),
        ("act", C.c_int32),
        ("act_alpha", C.c_float),
        ("out_scale", C.c_float),
        ("out_zero_point", C.c_int32),
    ]


class PeerHandle(C.Structure):
    _fields_ = [("ipc", C.c_ubyte * 64), ("offset", C.c_uint64)]


class GemmDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("batch", C.c_int64),
        ("trans_a", C.c_int32), ("trans_b", C.c_int32),
        ("ab_dtype", C.c_int32), ("y_dtype", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldy", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_y", C.c_int64),
        ("stride_c", C.c_int64), ("stride_r", C.c_int64),
        ("precise", C.c_int32), ("flags", C.c_int32),
    ]


class ConvDesc(C.Structure):
    _fields_ = [
        ("N", C.c_int64), ("C", C.c_int64), ("H", C.c_int64), ("W", C.c_int64),
        ("K", C.c_int64), ("R", C.c_int64), ("S", C.c_int64),
        ("pad_top", C.c_int32), ("pad_left", C.c_int32), ("pad_bottom", C.c_int32), ("pad_right", C.c_int32),
        ("stride_h", C.c_int32), ("stride_w", C.c_int32),
        ("dil_h", C.c_int32), ("dil_w", C.c_int32),
        ("groups", C.c_int32),
        ("x_dtype", C.c_int32), ("y_dtype", C.c_int32),
        ("x_zero_point", C.c_int32),
        ("precise", C.c_int32),
        ("x_layout", C.c_int32), ("y_layout", C.c_int32),
        ("flags", C.c_int32),
    ]


class SdpaDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int64), ("heads", C.c_int64), ("seq", C.c_int64), ("head_dim", C.c_int64), ("v_head_dim", C.c_int64),
        ("dtype", C.c_int32), ("folded", C.c_int32), ("has_mask", C.c_int32), ("scale", C.c_float),
        ("ldq", C.c_int64), ("ldk", C.c_int64), ("ldv", C.c_int64),
    ]


class TensorLife(C.Structure):
    _fields_ = [("begin", C.c_int64), ("end", C.c_int64), ("size", C.c_int64)]


_P = C.c_void_p
_I32, _I64, _F = C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); every symbol include/sofie_b200.h declares
PROTOTYPES = {
    "sofie_b200_abi_version": (C.c_int, []),
    "sofie_b200_status_string": (C.c_char_p, [C.c_int]),
    "sofie_b200_last_error": (C.c_char_p, []),
    "sofie_b200_ctx_create": (C.c_int, [C.POINTER(_P), C.c_int, _P]),
    "sofie_b200_ctx_destroy": (C.c_int, [_P]),
    "sofie_b200_ctx_sync": (C.c_int, [_P]),
    "sofie_b200_ctx_launch_count": (_I64, [_P]),
    "sofie_b200_selftest_wait_timeout": (C.c_int, [_P, _I64]),
    "sofie_b200_ctx_enable_peer": (C.c_int, [_P, _I32]),
    "sofie_b200_peer_export": (C.c_int, [_P, _P, C.POINTER(PeerHandle)]),
    "sofie_b200_peer_open": (C.c_int, [_P, C.POINTER(PeerHandle), C.POINTER(_P)]),
    "sofie_b200_peer_close": (C.c_int, [_P, _P]),
    "sofie_b200_gemm_plan_create": (C.c_int, [_P, C.POINTER(GemmDesc), C.POINTER(_P)]),
    "sofie_b200_gemm_plan_destroy": (C.c_int, [_P]),
    "sofie_b200_gemm_plan_kernel": (C.c_char_p, [_P]),
    "sofie_b200_gemm_enqueue": (C.c_int, [_P, _P, _P, _P, C.POINTER(Epilogue)]),
    "sofie_b200_gemm_enqueue_peers": (C.c_int, [_P, _P, _P, _P, C.POINTER(C.c_void_p), _I32, C.POINTER(Epilogue)]),
    "sofie_b200_gemm_run_host": (C.c_int, [_P, _P, _P, _P, C.POINTER(Epilogue)]),
    "sofie_b200_gemm_run_host_many": (C.c_int, [_P, _I64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(Epilogue)]),
    "sofie_b200_conv_plan_create": (C.c_int, [_P, C.POINTER(ConvDesc), _P, C.POINTER(_P)]),
    "sofie_b200_conv_plan_destroy": (C.c_int, [_P]),
    "sofie_b200_conv_out_shape": (C.c_int, [C.POINTER(ConvDesc), C.POINTER(_I64), C.POINTER(_I64)]),
    "sofie_b200_conv_workspace_bytes": (_I64, [_P]),
    "sofie_b200_conv_plan_kernel": (C.c_char_p, [_P]),
    "sofie_b200_conv_enqueue": (C.c_int, [_P, _P, _P, _P, C.POINTER(Epilogue)]),
    "sofie_b200_conv_enqueue_noalloc": (C.c_int, [_P, C.POINTER(ConvDesc), _P, _P, _P, C.POINTER(Epilogue)]),
    "sofie_b200_attention_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _I64, _I32, _I32, _F]),
    "sofie_b200_sdpa_plan_create": (C.c_int, [_P, C.POINTER(SdpaDesc), C.POINTER(_P)]),
    "sofie_b200_sdpa_plan_destroy": (C.c_int, [_P]),
    "sofie_b200_sdpa_plan_kernel": (C.c_char_p, [_P]),
    "sofie_b200_sdpa_workspace_bytes": (_I64, [_P]),
    "sofie_b200_sdpa_enqueue": (C.c_int, [_P, _P, _P, _P, _P, _P, _P]),
    "sofie_b200_layernorm_enqueue": (C.c_int, [_P, _P, _P, _I32, _I32, _I64, _I64, _P, _P, _F, _P, _P]),
    "sofie_b200_softmax_enqueue": (C.c_int, [_P, _P, _P, _I32, _I32, _I64, _I64, _I32]),
    "sofie_b200_softmax_axis_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _I64, _I64, _I32]),
    "sofie_b200_unary_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _I32, _F]),
    "sofie_b200_binary_enqueue": (C.c_int, [_P, _P, _P, _P, _I32, _I64, _I64, _I32, _I32]),
    "sofie_b200_batchnorm_enqueue": (C.c_int, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _I32]),
    "sofie_b200_global_avgpool_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _I64]),
    "sofie_b200_global_avgpool_nhwc_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _I64, _I64]),
    "sofie_b200_quantize_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _P, _P, _I64, _I64]),
    "sofie_b200_dequantize_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _P, _P, _I64, _I64]),
    "sofie_b200_transpose_enqueue": (C.c_int, [_P, _P, _P, _I32, _I32, C.POINTER(_I64), C.POINTER(_I32)]),
    "sofie_b200_depth_unfold_enqueue": (C.c_int, [_P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64]),
    "sofie_b200_convert_enqueue": (C.c_int, [_P, _P, _P, _I32, _I32, _I64, _I64, _P]),
    "sofie_b200_plan_arena": (C.c_int, [C.POINTER(TensorLife), _I64, C.POINTER(_I64), C.POINTER(_I64)]),
}

_lib = None


class SofieB200Error(RuntimeError):
    """Raised for every non-zero status, as the emitted Session wrapper throws std::runtime_error."""

    def __init__(self, status: int, where: str, detail: str):
        self.status = status
        super().__init__(f"{where}: status {status}: {detail}")


def load() -> C.CDLL:
    """Loads libsofie_b200.so and binds every prototype; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sofie_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.sofie_b200_abi_version() != ABI_VERSION:
        raise ImportError("libsofie_b200.so has a different ABI version than this binding")
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != 0:
        lib = load()
        raise SofieB200Error(status, where, lib.sofie_b200_last_error().decode())
