"""Builds libwein_b200.so (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python -m inferulm_b200.build            # build if sources are newer than the library
    python -m inferulm_b200.build --force
    python -m inferulm_b200.build -v         # with ptxas resource usage per kernel
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libwein_b200.so")
OBJ = os.path.join(HERE, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-I", CSRC, "-I", os.path.join(os.path.dirname(HERE), "include")]
# (source, extra flags).  Files holding bit-parity kernels are built with -fmad=false: the compiler must
# never contract a*b+c, fused multiply-adds appear only where written as fmaf().
SOURCES = [
    ("capi.cu", []),
    ("ops_exact.cu", ["-fmad=false"]),
    ("gdn.cu", ["-fmad=false"]),
    ("accept.cu", ["-fmad=false"]),
    ("fused_glue.cu", ["-fmad=false"]),
    ("attn.cu", []),
    ("gemm.cu", []),
    ("gemm_umma.cu", []),
    ("engine.cu", []),
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [
        os.path.join(os.path.dirname(HERE), "include", "wein_b200.h")]


def build(force=False, verbose=False):
    return _build(LIB, OBJ, [], force, verbose)


def _build(LIB, OBJ, defs, force, verbose):
    os.makedirs(OBJ, exist_ok=True)
    hdr_m = max((os.path.getmtime(h) for h in _headers() if os.path.exists(h)), default=0)
    objs, changed = [], False
    procs = []
    for src, extra in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(path), hdr_m):
            cmd = [_nvcc()] + ARCH + COMMON + defs + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, path]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
            changed = True
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
    if changed or not os.path.exists(LIB):
        cmd = [_nvcc()] + ARCH + ["-shared", "-o", LIB] + objs
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
