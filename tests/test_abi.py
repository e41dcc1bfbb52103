"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares, and
refuses to compute without a GPU instead of falling back to anything."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from sofie_b200 import lib as L

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "sofie_b200.h").read_text()


def declared_functions():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(sofie_b200_\w+)\s*\(", body)))


def test_library_exports_every_declared_symbol(b200_lib):
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(b200_lib, n), f"{n} is declared in include/sofie_b200.h but not exported"
    assert set(names) == set(L.PROTOTYPES), set(names) ^ set(L.PROTOTYPES)


def test_struct_layouts_match_header():
    # field order of the ctypes mirrors follows the header's declarations
    for struct, cname in ((L.Epilogue, "sofie_b200_epilogue"), (L.GemmDesc, "sofie_b200_gemm_desc"), (L.ConvDesc, "sofie_b200_conv_desc"),
                          (L.SdpaDesc, "sofie_b200_sdpa_desc")):
        m = re.search(r"typedef struct " + cname + r" \{(.*?)\} " + cname, HEADER, re.S)
        body = re.sub(r"/\*.*?\*/", "", m.group(1), flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.split(None, 1)[1] if not decl.startswith("const") else decl.split(None, 2)[2]
            fields += [x.strip().lstrip("*") for x in names.split(",")]
        assert fields == [f[0] for f in struct._fields_], (cname, fields)


def test_abi_version_and_status_strings(b200_lib):
    assert b200_lib.sofie_b200_abi_version() == L.ABI_VERSION == 2
    assert b200_lib.sofie_b200_status_string(0) == b"ok"
    assert b"wait" in b200_lib.sofie_b200_status_string(L.ERR_DEVICE_WAIT)


def test_no_gpu_means_loud_failure(b200_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = b200_lib.sofie_b200_ctx_create(C.byref(h), 0, None)
    assert rc == L.ERR_NO_DEVICE and not h.value
    assert b"no CUDA device" in b200_lib.sofie_b200_last_error()
    with pytest.raises(L.SofieB200Error):
        L.check(rc, "ctx_create")


def test_null_arguments_are_rejected(b200_lib):
    assert b200_lib.sofie_b200_ctx_create(None, 0, None) == L.ERR_INVALID
    assert b200_lib.sofie_b200_gemm_enqueue(None, None, None, None, None) == L.ERR_INVALID
    assert b200_lib.sofie_b200_layernorm_enqueue(None, None, None, 0, 0, 1, 1, None, None, 1e-5, None, None) == L.ERR_INVALID


def test_conv_out_shape_follows_reference_rules(b200_lib):
    d = L.ConvDesc()
    d.N, d.C, d.H, d.W, d.K, d.R, d.S = 1, 1, 7, 5, 1, 3, 3
    d.pad_top = d.pad_left = d.pad_bottom = d.pad_right = 1
    d.stride_h = d.stride_w = 2
    d.dil_h = d.dil_w = 1
    ho, wo = C.c_int64(), C.c_int64()
    assert b200_lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == 0
    assert (ho.value, wo.value) == (4, 3)  # ConvWithStridesPadding: 7x5 -> 4x3
    d.dil_h = d.dil_w = 0
    assert b200_lib.sofie_b200_conv_out_shape(C.byref(d), C.byref(ho), C.byref(wo)) == L.ERR_INVALID


# ---- arena planner (host-only code in the library) --------------------------------------------
def plan(lib, fn, lives):
    arr = (L.TensorLife * len(lives))(*[L.TensorLife(b, e, s) for b, e, s in lives])
    offs = (C.c_int64 * len(lives))()
    total = C.c_int64()
    rc = getattr(lib, fn)(arr, len(lives), offs, C.byref(total))
    return rc, list(offs), total.value


def check_no_overlap(lives, offs):
    for i, (b1, e1, s1) in enumerate(lives):
        assert offs[i] % 256 == 0
        for j in range(i):
            b2, e2, s2 = lives[j]
            if b1 < e2 and b2 < e1 and s1 and s2:  # alive together
                r1, r2 = (s1 + 255) // 256 * 256, (s2 + 255) // 256 * 256
                assert offs[i] + r1 <= offs[j] or offs[j] + r2 <= offs[i], (i, j)


def test_arena_reuses_dead_tensors(b200_lib):
    # a chain x0 -> x1 -> x2 -> x3: only two neighbours are alive together
    lives = [(0, 2, 1000), (1, 3, 1000), (2, 4, 1000), (3, 5, 1000)]
    rc, offs, total = plan(b200_lib, "sofie_b200_plan_arena", lives)
    assert rc == 0 and total == 2 * 1024
    check_no_overlap(lives, offs)


def test_arena_best_fit_and_coalescing(b200_lib):
    lives = [(0, 1, 512), (0, 3, 256), (0, 1, 1024), (1, 4, 1024), (1, 4, 512), (2, 5, 300)]
    rc, offs, total = plan(b200_lib, "sofie_b200_plan_arena", lives)
    assert rc == 0
    check_no_overlap(lives, offs)
    assert offs[3] == offs[2] and offs[4] == offs[0]  # exact-size blocks are taken (best fit)
    assert total == 512 + 256 + 1024 + 512  # tensor 5 needs fresh space: nothing fitting is free at t=2


def test_arena_rejects_empty_lifetime(b200_lib):
    rc, _, _ = plan(b200_lib, "sofie_b200_plan_arena", [(3, 3, 10)])
    assert rc == L.ERR_INVALID


def test_arena_matches_oracle_on_random_lifetimes(b200_lib, oracle_lib):
    olib = C.CDLL(str(oracle_lib))
    rng = np.random.default_rng(5)
    for trial in range(50):
        n = int(rng.integers(1, 40))
        lives = []
        for i in range(n):
            b = int(rng.integers(0, 30))
            lives.append((b, b + int(rng.integers(1, 10)), int(rng.integers(1, 64)) * 256))
        rc1, o1, t1 = plan(b200_lib, "sofie_b200_plan_arena", lives)
        rc2, o2, t2 = plan(olib, "so_plan_arena", lives)
        assert rc1 == 0 and rc2 == 0
        assert (o1, t1) == (o2, t2), trial
        check_no_overlap(lives, o1)
        assert t1 <= sum((s + 255) // 256 * 256 for _, _, s in lives)
