"""Build libflh_b200.so (sm_100a only) in-tree with nvcc.

    python -m flh_b200.build          # or: from flh_b200.build import build; build()

The library has no Python or torch dependency: it is the C ABI declared in
include/flh_b200.h.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["api.cu", "quant_group.cu", "quant_token.cu", "quant_token_warp.cu", "quant_token_factor.cu", "quant_token_tc.cu", "act.cu", "gemm_mma.cu", "gemm_tcgen05.cu", "gemm_i8.cu", "gemm_decode_tc.cu", "gptq.cu", "allreduce.cu"]
LIB = os.path.join(HERE, "libflh_b200.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "nvcc")
    headers = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "token_common.cuh"), os.path.join(CSRC, "tc_common.cuh"), os.path.join(CSRC, "act_common.cuh"), os.path.join(CSRC, "tc_quant_common.cuh"), os.path.join(HERE, "..", "include", "flh_b200.h")]
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", s, "-o", o] + (["-Xptxas", "-v"] if verbose else [])
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    with ThreadPoolExecutor(max_workers=min(4, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if force or jobs or not os.path.exists(LIB):
        run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
