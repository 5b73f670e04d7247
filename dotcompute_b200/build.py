"""Build libdcb200.so in-tree with nvcc for sm_100a.

Steps: (1) embed dcb_kernels.cuh as a string for NVRTC, (2) build the translator and the generator tool with
g++, (3) generate the ahead-of-time pipeline table, (4) compile the .cu files for sm_100a, (5) link the shared
library next to this file. Run as ``python -m dotcompute_b200.build`` or through ``__graft_entry__.build()``.
No GPU is needed to build.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libdcb200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
AOT_UNROLL = "4"


def _run(cmd, log=None):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return proc.stdout


def _digest(paths):
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target, paths):
    """True if the library is missing or was built from other sources (content hash, not mtime: a copy of the tree
    to another machine must not trigger a rebuild)."""
    stamp = os.path.join(BUILD, "sources.sha256")
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != _digest(paths)


def sources():
    names = ["dcb_kernels.cuh", "dcb_translate.h", "dcb_translate.cpp", "dcb_api.cu", "dcb_builtin.h",
             "dcb_builtin_pipelines.txt", "dcb_gen.cpp", "dcb_noalloc.cu", "dcb_peer.cuh", "dcb_internal.h", "dcb_relational.cu"]
    out = [os.path.join(CSRC, n) for n in names if os.path.exists(os.path.join(CSRC, n))]
    out.append(os.path.join(HERE, "..", "include", "dcb200.h"))
    out.append(os.path.abspath(__file__))
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile everything if any source is newer than the library; return the library path."""
    if not force and not _stale(LIB, sources()):
        return LIB
    if not os.path.exists(NVCC):
        raise RuntimeError(f"nvcc not found at {NVCC}")
    os.makedirs(BUILD, exist_ok=True)
    # (1) kernel templates as a raw string literal for NVRTC
    with open(os.path.join(CSRC, "dcb_kernels.cuh")) as f:
        text = f.read()
    assert ')DCBSRC"' not in text
    with open(os.path.join(BUILD, "dcb_kernels_embed.inc"), "w") as f:
        f.write('R"DCBSRC(' + text + ')DCBSRC"\n')
    # (2) translator + generator
    tr_o = os.path.join(BUILD, "dcb_translate.o")
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-c", os.path.join(CSRC, "dcb_translate.cpp"), "-o", tr_o])
    gen = os.path.join(BUILD, "dcb_gen")
    _run(["g++", "-O1", "-std=c++17", os.path.join(CSRC, "dcb_gen.cpp"), tr_o, "-o", gen])
    # (3) ahead-of-time table
    gen_cu = os.path.join(BUILD, "dcb_builtin_gen.cu")
    _run([gen, os.path.join(CSRC, "dcb_builtin_pipelines.txt"), gen_cu, AOT_UNROLL])
    # (4) device code. -fmad=false: a Select must round like the C# lambda, never contract a*b+c.
    common = [NVCC, *ARCH, "-I" + CSRC, "-lineinfo", "-O3", "-std=c++17", "-fmad=false", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
    objs = [tr_o]
    cu_files = [os.path.join(CSRC, "dcb_api.cu"), gen_cu]
    for extra in ("dcb_noalloc.cu", "dcb_relational.cu"):
        if os.path.exists(os.path.join(CSRC, extra)):
            cu_files.append(os.path.join(CSRC, extra))
    for cu in cu_files:
        o = os.path.join(BUILD, os.path.basename(cu).replace(".cu", ".o"))
        log = os.path.join(BUILD, os.path.basename(cu) + ".ptxas.log")
        out = _run(common + ["-c", cu, "-o", o], log=log)
        if verbose:
            print(out)
        objs.append(o)
    # (5) link. cudart is linked statically; NVRTC stays dynamic (it ships with the CUDA toolkit).
    libdir = os.path.join(CUDA_HOME, "lib64")
    _run([NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-L" + libdir, "-lnvrtc", "-Xlinker", "-rpath=" + libdir])
    with open(os.path.join(BUILD, "sources.sha256"), "w") as f:
        f.write(_digest(sources()))
    return LIB


def clean() -> None:
    if os.path.isdir(BUILD):
        shutil.rmtree(BUILD)
    if os.path.exists(LIB):
        os.remove(LIB)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
