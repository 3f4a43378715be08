"""In-tree build of libkurumi_cuda.so (the product) and of the CPU oracle used by the tests.

Host code is C++17 compiled by nvcc's host compiler; hand-written kernel templates under
csrc/cuda/kernels/ are embedded as text and compiled at run time by NVRTC for sm_100a, and are
also compiled here once by nvcc (-gencode arch=compute_100a,code=sm_100a) as the build check.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIBDIR = os.path.join(ROOT, "lib")
LIB = os.path.join(LIBDIR, "libkurumi_cuda.so")
ORACLE_DIR = os.path.join(os.path.dirname(ROOT), "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "_build", "libkurumi_oracle.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

SOURCES = ["core/graph.cc", "core/serialize.cc", "core/split.cc", "capi/capi.cc", "lower/view.cc", "cuda/hostmem.cc", "cuda/runtime.cc", "cuda/fuse.cc", "cuda/emit.cc", "cuda/emit_index.cc", "cuda/sched.cc",
           "cuda/kernels.cc", "cuda/backend.cc", "cuda/pipeline.cc", "cuda/comm.cc", "cuda/capi_cuda.cc"]


def _run(cmd, **kw):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout)
    return r.stdout


def _embed_kernels() -> str:
    """Turn csrc/cuda/kernels/*.cuh into one C++ source of raw string literals."""
    kdir = os.path.join(CSRC, "cuda", "kernels")
    out = os.path.join(LIBDIR, "kernel_sources.gen.cc")
    parts = ['#include <string>\nnamespace ku::cu {\n']
    for name in sorted(os.listdir(kdir)) if os.path.isdir(kdir) else []:
        if not name.endswith(".cuh"):
            continue
        text = open(os.path.join(kdir, name)).read()
        ident = "kSrc_" + name[:-4]
        # MSVC-style literal length limits do not apply to g++; split anyway to stay portable
        chunks = [text[i:i + 12000] for i in range(0, len(text), 12000)]
        lit = "\n".join('R"KUSRC(' + c + ')KUSRC"' for c in chunks)
        parts.append(f"extern const std::string {ident} = std::string({lit});\n")
    parts.append("}\n")
    os.makedirs(LIBDIR, exist_ok=True)
    new = "".join(parts)
    if not os.path.exists(out) or open(out).read() != new:
        open(out, "w").write(new)
    return out


def _stamp(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.encode())
        h.update(open(p, "rb").read())
    return h.hexdigest()


def _all_inputs():
    files = []
    for d, _, names in os.walk(CSRC):
        files += [os.path.join(d, n) for n in names if n.endswith((".cc", ".h", ".cuh", ".cu"))]
    files.append(os.path.join(os.path.dirname(ROOT), "include", "kurumi.h"))
    files.append(os.path.join(os.path.dirname(ROOT), "include", "kurumi_cuda.h"))
    files.append(os.path.abspath(__file__))
    return files


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    stamp_file = os.path.join(LIBDIR, ".stamp")
    stamp = _stamp(_all_inputs())
    if not force and os.path.exists(LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return LIB
    gen = _embed_kernels()
    srcs = [os.path.join(CSRC, s) for s in SOURCES] + [gen]
    cu = [os.path.join(CSRC, "cuda", n) for n in sorted(os.listdir(os.path.join(CSRC, "cuda"))) if n.endswith(".cu")]
    cmd = [NVCC, "-std=c++17", "-O2", "-lineinfo", "-shared", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-parameter", *ARCH, "-cudart", "static",
           "-I" + os.path.join(CUDA_HOME, "include"), "-o", LIB, *srcs, *cu, "-L" + os.path.join(CUDA_HOME, "lib64"), "-lnvrtc",
           "-Xlinker", "-rpath," + os.path.join(CUDA_HOME, "lib64"), "-ldl", "-lpthread"]
    out = _run(cmd)
    if verbose:
        print(out)
    open(stamp_file, "w").write(stamp)
    return LIB


def build_oracle(force: bool = False) -> str:
    cmd = ["make", "-C", ORACLE_DIR] + (["-B"] if force else [])
    _run(cmd)
    return ORACLE_LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
    print(build_oracle())
