"""Builds libsofie_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch extension).

`python -m sofie_b200.build` compiles every .cu under sofie_b200/csrc into objects under
sofie_b200/csrc/build/ and links sofie_b200/libsofie_b200.so.  Only stale objects are rebuilt.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libsofie_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; libsofie_b200 can only be built with the CUDA toolkit")
    return cand


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "sofie_b200.h"]
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0 or ptxas_info:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(run, jobs))

    objs = [OBJ / (s.stem + ".o") for s in sources]
    if jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-Xlinker", "--no-undefined"]
        run(cmd)
    return LIB


HOST = PKG / "host"
HOST_LIB = HOST / "libsofie_b200_host.so"
EMIT = HOST / "sofie_b200_emit"


def build_host(verbose: bool = False) -> Path:
    """The C++ code generator: libsofie_b200_host.so (RModel, operators, ONNX front-end) and the
    sofie_b200_emit tool.  Plain g++, no CUDA needed."""
    cxx = shutil.which("g++") or "g++"
    srcs = [HOST / "src" / "RModel.cxx", HOST / "src" / "RModelParser_ONNX.cxx"]
    deps = srcs + sorted((HOST / "inc").rglob("*.hxx"))
    flags = ["-std=c++20", "-O1", "-Wall", f"-I{HOST / 'inc'}"]

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("g++ failed for the host generator")

    if _stale(HOST_LIB, deps):
        run([cxx, *flags, "-fPIC", "-shared", "-o", str(HOST_LIB), *map(str, srcs)])
    if _stale(EMIT, deps + [HOST / "src" / "sofie_b200_emit.cxx", HOST_LIB]):
        run([cxx, *flags, "-o", str(EMIT), str(HOST / "src" / "sofie_b200_emit.cxx"), f"-L{HOST}", "-lsofie_b200_host",
             "-Wl,-rpath,$ORIGIN"])
    return EMIT


def cuda_include_dir() -> Path:
    return Path(_nvcc()).resolve().parent.parent / "include"


def compile_session(header: Path, out_so: Path, wrapper_src: str) -> Path:
    """Compiles an emitted Session header plus a small C wrapper into a shared library that links
    libsofie_b200 and the CUDA runtime (what a user of the emitted code does)."""
    cxx = shutil.which("g++") or "g++"
    src = out_so.with_suffix(".cxx")
    src.write_text(wrapper_src)
    cuda = cuda_include_dir().parent
    cmd = [cxx, "-std=c++20", "-O1", "-fPIC", "-shared", "-o", str(out_so), str(src), f"-I{header.parent}",
           f"-I{PKG.parent / 'include'}", f"-I{cuda / 'include'}", f"-L{PKG}", "-lsofie_b200", f"-Wl,-rpath,{PKG}",
           f"-L{cuda / 'lib64'}", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compiling the emitted Session failed:\n" + r.stdout + r.stderr)
    return out_so


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
    print(build_host(verbose="-v" in sys.argv))
