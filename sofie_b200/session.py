"""Emits, compiles and drives a Session of the C++ generator from Python (ctypes): the path a user of the generated code
takes -- ONNX file -> sofie_b200_emit -> <model>.hxx + weight file -> g++ -> Session -- wrapped so that tests and the
benchmark can call infer_nosync / infer_host / infer_host_many of the emitted code.  Nothing here computes: the wrapper
forwards to the Session, which calls libsofie_b200.
"""
from __future__ import annotations

import ctypes as C
import re
import subprocess
from pathlib import Path

from . import build as B
from . import onnx_min

# ONNX element type -> C type of the emitted Session's pointers
C_TYPE = {1: "float", 2: "uint8_t", 3: "int8_t", 6: "int32_t", 7: "int64_t", 16: "uint16_t", 17: "uint8_t"}

_WRAPPER = """
#include "{header}"
#include <cstring>
using S = SOFIE_{name}::Session;
static thread_local std::string g_err;
extern "C" const char *sess_error() {{ return g_err.c_str(); }}
// `dim`: the value of the model's symbolic dimension (a model without one ignores it)
extern "C" void *sess_create(const char *file, unsigned long long dim)
{{
   (void)dim;
   try {{ return new S(file{dim_arg}); }} catch (const std::exception &e) {{ g_err = e.what(); return nullptr; }}
}}
// the reference's dynamic form of infer: the dimension again, then the inputs; waits for the result
extern "C" const void *sess_infer_dim(void *s, unsigned long long dim, const void *const *in)
{{
   (void)dim;
   try {{ return static_cast<S *>(s)->infer({dim_lead}{dev_args}); }} catch (const std::exception &e) {{ g_err = e.what(); return nullptr; }}
}}
extern "C" void sess_destroy(void *s) {{ delete static_cast<S *>(s); }}
extern "C" void *sess_stream(void *s) {{ return static_cast<S *>(s)->stream; }}
extern "C" long long sess_launches(void *s) {{ return static_cast<S *>(s)->GetLaunchCount(); }}
extern "C" unsigned long long sess_arena_bytes(void *s) {{ return static_cast<S *>(s)->GetArenaSize(); }}
extern "C" void sess_use_graph(void *s, int on) {{ static_cast<S *>(s)->SetUseCudaGraph(on != 0); }}
extern "C" const void *sess_infer_nosync(void *s, const void *const *in)
{{
   try {{ return static_cast<S *>(s)->infer_nosync({dev_args}); }} catch (const std::exception &e) {{ g_err = e.what(); return nullptr; }}
}}
// the span form: device views of the inputs in, results copied into the caller's device buffers, returns when done
extern "C" int sess_infer_span(void *s, const void *const *in, unsigned long long n_in, void *const *out, unsigned long long n_out)
{{
   try {{ static_cast<S *>(s)->infer(std::span<const void *const>(in, n_in), std::span<void *const>(out, n_out)); return 0; }}
   catch (const std::exception &e) {{ g_err = e.what(); return -1; }}
}}
extern "C" void sess_pool_stats(void *s, unsigned long long *pool, unsigned long long *free_bytes, unsigned long long *largest, double *fragmentation)
{{
   const S *p = static_cast<S *>(s);
   *pool = p->GetIntermediateMemoryPoolSize(); *free_bytes = p->GetTotalFreeMemory(); *largest = p->GetLargestFreeBlock(); *fragmentation = p->GetFragmentation();
}}
extern "C" int sess_sync(void *s)
{{
   try {{ S::Check(sofie_b200_ctx_sync(static_cast<S *>(s)->ctx), "sync"); return 0; }} catch (const std::exception &e) {{ g_err = e.what(); return -1; }}
}}
extern "C" long sess_infer_host(void *s, const void *const *in, void *out, long cap_bytes)
{{
   try {{
      auto y = static_cast<S *>(s)->infer_host({dev_args});
      const size_t bytes = y.size() * sizeof(y[0]);
      std::memcpy(out, y.data(), bytes < (size_t)cap_bytes ? bytes : (size_t)cap_bytes);
      return (long)y.size();
   }} catch (const std::exception &e) {{ g_err = e.what(); return -1; }}
}}
// ins[i] is the array of `count` host pointers of input i
extern "C" int sess_infer_host_many(void *s, unsigned long long count, const void *const *const *ins, void *const *outs)
{{
   try {{ static_cast<S *>(s)->infer_host_many(count, {many_args}reinterpret_cast<{tout} *const *>(outs)); return 0; }}
   catch (const std::exception &e) {{ g_err = e.what(); return -1; }}
}}
"""


class EmittedSession:
    """One emitted, compiled and constructed Session."""

    def __init__(self, name: str, nodes, weights, inputs, outputs, workdir, flags=("--safetensors",), input_types=None, initializer_types=None,
                 symbolic_dim=None):
        """symbolic_dim: the value for the model's symbolic dimension (an input shape with a string in it), given to the
        Session constructor as the reference's dynamic Sessions take it."""
        workdir = Path(workdir)
        workdir.mkdir(parents=True, exist_ok=True)
        self.name, self.workdir = name, workdir
        emit = B.build_host()
        onnx = workdir / f"{name}.onnx"
        onnx_min.save(str(onnx), nodes, weights, inputs, outputs, input_types=input_types, initializer_types=initializer_types)
        r = subprocess.run([str(emit), str(onnx), str(workdir / f"{name}.hxx"), *flags], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"sofie_b200_emit failed for {name}: {r.stderr}")
        self.report = r.stdout
        header = (workdir / f"{name}.hxx").read_text()
        self.out_ctype = re.search(r"(\w+) \*infer_nosync\(", header).group(1)
        self.n_in = len(inputs)
        types = [C_TYPE[(input_types or {}).get(n, 1)] for n, _ in inputs]
        dev_args = ", ".join(f"static_cast<const {t} *>(in[{i}])" for i, t in enumerate(types))
        many_args = "".join(f"reinterpret_cast<const {t} *const *>(ins[{i}]), " for i, t in enumerate(types))
        dynamic = symbolic_dim is not None
        src = _WRAPPER.format(header=workdir / f"{name}.hxx", name=name, dev_args=dev_args, many_args=many_args, tout=self.out_ctype,
                              dim_arg=", size_t(dim)" if dynamic else "", dim_lead="size_t(dim), " if dynamic else "")
        so = B.compile_session(workdir / f"{name}.hxx", workdir / f"libsession_{name}.so", src)
        lib = C.CDLL(str(so))
        lib.sess_error.restype = C.c_char_p
        lib.sess_create.restype = C.c_void_p
        lib.sess_create.argtypes = [C.c_char_p, C.c_ulonglong]
        lib.sess_infer_dim.restype = C.c_void_p
        lib.sess_infer_dim.argtypes = [C.c_void_p, C.c_ulonglong, C.POINTER(C.c_void_p)]
        lib.sess_destroy.argtypes = [C.c_void_p]
        lib.sess_stream.restype = C.c_void_p
        lib.sess_stream.argtypes = [C.c_void_p]
        lib.sess_launches.restype = C.c_longlong
        lib.sess_launches.argtypes = [C.c_void_p]
        lib.sess_arena_bytes.restype = C.c_ulonglong
        lib.sess_arena_bytes.argtypes = [C.c_void_p]
        lib.sess_use_graph.argtypes = [C.c_void_p, C.c_int]
        lib.sess_infer_nosync.restype = C.c_void_p
        lib.sess_infer_nosync.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        lib.sess_sync.argtypes = [C.c_void_p]
        lib.sess_infer_span.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_ulonglong, C.POINTER(C.c_void_p), C.c_ulonglong]
        lib.sess_pool_stats.argtypes = [C.c_void_p, C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), C.POINTER(C.c_double)]
        lib.sess_infer_host.restype = C.c_long
        lib.sess_infer_host.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.c_long]
        lib.sess_infer_host_many.argtypes = [C.c_void_p, C.c_ulonglong, C.POINTER(C.POINTER(C.c_void_p)), C.POINTER(C.c_void_p)]
        self.lib = lib
        ext = ".safetensors" if "--safetensors" in flags else ".dat"
        self.h = lib.sess_create(str(workdir / f"{name}{ext}").encode(), int(symbolic_dim or 0))
        if not self.h:
            raise RuntimeError(f"Session {name}: {lib.sess_error().decode()}")

    # ---- device pointers in, device pointer out; only enqueues
    def infer_nosync(self, *device_ptrs: int) -> int:
        arr = (C.c_void_p * self.n_in)(*device_ptrs)
        r = self.lib.sess_infer_nosync(self.h, arr)
        if not r:
            raise RuntimeError(f"Session {self.name}: {self.lib.sess_error().decode()}")
        return r

    def infer_dim(self, dim: int, *device_ptrs: int) -> int:
        """infer(dim, inputs...) of a Session with a symbolic dimension; returns the output's device pointer after the wait."""
        arr = (C.c_void_p * self.n_in)(*device_ptrs)
        p = self.lib.sess_infer_dim(self.h, int(dim), arr)
        if not p:
            raise RuntimeError(f"Session {self.name}: {self.lib.sess_error().decode()}")
        return p

    def infer_span(self, device_in_ptrs, device_out_ptrs) -> None:
        """The Session's span form of infer: device pointers of the inputs and of caller-owned output buffers; returns when
        the outputs are written."""
        ins = (C.c_void_p * len(device_in_ptrs))(*device_in_ptrs)
        outs = (C.c_void_p * len(device_out_ptrs))(*device_out_ptrs)
        if self.lib.sess_infer_span(self.h, ins, len(device_in_ptrs), outs, len(device_out_ptrs)) != 0:
            raise RuntimeError(f"Session {self.name}: {self.lib.sess_error().decode()}")

    def pool_stats(self) -> dict:
        pool, free, largest, frag = C.c_ulonglong(), C.c_ulonglong(), C.c_ulonglong(), C.c_double()
        self.lib.sess_pool_stats(self.h, C.byref(pool), C.byref(free), C.byref(largest), C.byref(frag))
        return {"pool": pool.value, "free": free.value, "largest_free": largest.value, "fragmentation": frag.value}

    def sync(self) -> None:
        if self.lib.sess_sync(self.h) != 0:
            raise RuntimeError(f"Session {self.name}: {self.lib.sess_error().decode()}")

    @property
    def stream(self) -> int:
        return self.lib.sess_stream(self.h)

    @property
    def launches(self) -> int:
        return self.lib.sess_launches(self.h)

    def use_graph(self, on: bool) -> None:
        self.lib.sess_use_graph(self.h, int(on))

    # ---- host arrays (numpy, contiguous) in, host array out
    def infer_host(self, ins, out) -> int:
        arr = (C.c_void_p * self.n_in)(*[x.ctypes.data for x in ins])
        n = self.lib.sess_infer_host(self.h, arr, out.ctypes.data, out.nbytes)
        if n < 0:
            raise RuntimeError(f"Session {self.name}: {self.lib.sess_error().decode()}")
        return n

    def infer_host_many(self, in_ptr_lists, out_ptrs) -> None:
        """in_ptr_lists[i][k]: host address of input i of inference k; out_ptrs[k]: host address of its first output."""
        count = len(out_ptrs)
        per_input = [(C.c_void_p * count)(*ptrs) for ptrs in in_ptr_lists]
        ins = (C.POINTER(C.c_void_p) * self.n_in)(*[C.cast(a, C.POINTER(C.c_void_p)) for a in per_input])
        outs = (C.c_void_p * count)(*out_ptrs)
        if self.lib.sess_infer_host_many(self.h, count, ins, outs) != 0:
            raise RuntimeError(f"Session {self.name}: {self.lib.sess_error().decode()}")

    def close(self) -> None:
        if self.h:
            self.lib.sess_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
