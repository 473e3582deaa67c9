#!/usr/bin/env python3
"""Build libdk_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python deformable-kernels_b200/build.py [--force] [--verbose]

The library depends on the CUDA runtime only (no torch, no ATen).  Output:
deformable-kernels_b200/lib/libdk_b200.so (git-ignored).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libdk_b200.so")
SOURCES = ["dk_api.cu", "dk_local.cu", "dk_local_mma.cu", "dk_local_ring.cu", "dk_deform.cu", "dk_deform_mma.cu", "dk_nd.cu", "dk_scale.cu", "dk_global.cu", "dk_static_scratch.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _deps():
    out = [os.path.join(ROOT, "include", "dk_b200.h")]
    for f in os.listdir(CSRC):
        if f.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, f))
    return out


def build(force=False, verbose=False, defines=()):
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    newest = max(os.path.getmtime(p) for p in _deps())
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= newest:
        return LIB
    objs, procs = [], []
    for src in SOURCES:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [_nvcc()] + NVCC_FLAGS + list(defines) + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    subprocess.check_call([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-lcudart"])
    return LIB


if __name__ == "__main__":
    # -DNAME arguments are passed to nvcc (e.g. -DDK_TUNING enables the experiment knobs read from the environment)
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, defines=[a for a in sys.argv[1:] if a.startswith("-D")]))
