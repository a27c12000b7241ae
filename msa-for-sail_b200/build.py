#!/usr/bin/env python3
"""Build libmsa_b200.so in-tree with nvcc for sm_100a (no other architecture).

    python build.py [-v] [-f]            the shipped library
    python build.py --bounds-check       libmsa_b200_check.so: the same sources with -DMSA_BOUNDS_CHECK (every index a
                                         kernel reads from a caller's table is range-checked, clamped and reported in
                                         the status word) and -DMSA_DEBUG_HOOKS (clock traces, test hooks); loaded
                                         instead of the shipped library when MSA_BOUNDS_CHECK=1 is set in the environment
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "python", "msa_for_sail", "libmsa_b200.so")
OUT_CHECK = os.path.join(HERE, "python", "msa_for_sail", "libmsa_b200_check.so")
CHECK_FLAGS = ["-DMSA_BOUNDS_CHECK", "-DMSA_DEBUG_HOOKS"]
SOURCES = ["api.cu", "fmha_mma.cu", "fmha_tc.cu", "fmha_sparse_tc.cu", "fmha_decode_tc.cu", "score_gemv.cu", "plan_device.cu", "topk_select.cu", "lse_merge.cu", "static_scratch.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
         "--expt-relaxed-constexpr"]


def _stale(obj, src):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    deps = [src, os.path.join(ROOT, "include", "msa_b200.h")] + [
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, check=False):
    objdir = os.path.join(HERE, "build", "check" if check else "")
    out = OUT_CHECK if check else OUT
    os.makedirs(objdir, exist_ok=True)
    objs, jobs = [], []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, src):
            cmd = [NVCC] + FLAGS + (CHECK_FLAGS if check else []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(out):
        run([NVCC, "-shared", "-o", out] + objs)   # cudart is linked statically (nvcc default)
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, check="--bounds-check" in sys.argv))
