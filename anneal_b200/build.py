"""Builds libanneal_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
SO = os.path.join(LIBDIR, "libanneal_cuda.so")
SOURCES = ["kir.cpp", "codegen.cpp", "comm.cpp", "runtime.cu", "gemm.cu", "gemm_f32.cu", "static_sum.cu", "beam.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", "-I", LIBDIR,
         "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-cudart", "static"]


def _stale() -> bool:
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "anneal_cuda.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return SO
    os.makedirs(LIBDIR, exist_ok=True)
    # the two-CTA contraction kernel is compiled at run time: its text travels inside the library
    with open(os.path.join(CSRC, "gemm_pair_kernel.cuh")) as f:
        text = f.read()
    assert ')ANLSRC"' not in text
    inc = os.path.join(LIBDIR, "gemm_pair_src.inc")
    lit = 'R"ANLSRC(' + text + ')ANLSRC"\n'
    if not os.path.exists(inc) or open(inc).read() != lit:
        with open(inc, "w") as f:
            f.write(lit)
    objs = []
    for src in SOURCES:
        obj = os.path.join(LIBDIR, src.rsplit(".", 1)[0] + ".o")
        path = os.path.join(CSRC, src)
        # every object depends on its source, on every header beside it and on the public header (struct
        # layouts such as anl_stats are part of anl_device, which all of them see)
        deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".hpp", ".h", ".cuh")) or f == src]
        deps.append(os.path.join(HERE, "..", "include", "anneal_cuda.h"))
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(d) for d in deps):
            cmd = [NVCC, *FLAGS, "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            subprocess.check_call(cmd)
        objs.append(obj)
    cmd = [NVCC, "-shared", "-cudart", "static", "-o", SO, *objs, "-lnvrtc", "-ldl", "-Xlinker", "-rpath=/usr/local/cuda/lib64"]
    subprocess.check_call(cmd)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
