"""Build libquactlize_b200.so in-tree with nvcc for sm_100a (no torch types; a plain C-ABI shared library).

    python -m quactlize_b200.build [-v] [--force]
    python -m quactlize_b200.build --variant NAME --define MACRO[=VALUE] [--define ...]

Each .cu is compiled to an object only when it or a header changed, then linked into
quactlize_b200/csrc/libquactlize_b200.so.

A variant is the same library with compile-time switches of the kernels set (the ablation and tuning macros the sources
name: QB_ABL_*, QB_GABL_*, QB_SWAP_*, QB_GEMM_*, QB_Q4_WARPS ...): the sources that mention one of the macros are
recompiled with them, the other objects are shared with the main build, and the result is
csrc/libquactlize_b200_NAME.so, which QUACTLIZE_B200_LIB=<that path> selects at run time, e.g.

    python -m quactlize_b200.build --variant nodeq --define QB_GABL_NODEQ
    QUACTLIZE_B200_LIB=quactlize_b200/csrc/libquactlize_b200_nodeq.so python -m quactlize_b200.bench_suite --only cfg4_gate
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(CSRC, "libquactlize_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-I", os.path.join(os.path.dirname(HERE), "include")]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers_mtime():
    hs = glob.glob(os.path.join(CSRC, "*.hpp")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hm = _headers_mtime()
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hm):
            cmd = [NVCC, *FLAGS, "-c", src, "-o", obj]
            if ptxas_info:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        if (verbose or ptxas_info) and (r.stdout or r.stderr):
            print(r.stdout + r.stderr, flush=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([NVCC, "-shared", "-o", LIB, *objs, "-cudart", "shared"])
    return LIB


def build_variant(name: str, defines, verbose: bool = False) -> str:
    """The library with `defines` (["MACRO", "MACRO=VALUE", ...]) set in every source that mentions one of the macros."""
    if not name.isidentifier() or not defines:
        raise ValueError("a variant needs a name (letters, digits, underscores) and at least one --define")
    build(verbose=verbose)                                   # the shared objects are the main build's
    vdir = os.path.join(OBJ, "variant_" + name)
    os.makedirs(vdir, exist_ok=True)
    macros = [d.split("=")[0] for d in defines]
    objs, jobs = [], []
    for src in sources():
        base = os.path.basename(src)[:-3] + ".o"
        text = open(src).read()
        if any(m in text for m in macros):
            obj = os.path.join(vdir, base)
            jobs.append([NVCC, *FLAGS, *["-D" + d for d in defines], "-c", src, "-o", obj])
        else:
            obj = os.path.join(OBJ, base)
        objs.append(obj)
    if not jobs:
        raise ValueError("no source mentions " + ", ".join(macros))
    for cmd in jobs:
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    lib = os.path.join(CSRC, "libquactlize_b200_" + name + ".so")
    r = subprocess.run([NVCC, "-shared", "-o", lib, *objs, "-cudart", "shared"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return lib


if __name__ == "__main__":
    if "--variant" in sys.argv:
        args = sys.argv[1:]
        name = args[args.index("--variant") + 1]
        defines = [args[i + 1] for i, a in enumerate(args) if a == "--define" and i + 1 < len(args)]
        print(build_variant(name, defines, verbose="-v" in args))
    else:
        print(build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv))
