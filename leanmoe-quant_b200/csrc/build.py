"""Build liblemoq_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python leanmoe-quant_b200/csrc/build.py [--verbose]

The library has no dependency on torch or Python: it links against the CUDA runtime
only.  Objects are rebuilt when a source or header is newer than the object.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SOURCES = ["cabi.cu", "gemv_w8.cu", "stream_gemv.cu", "moe_grouped.cu", "attn_decode.cu", "small_ops.cu", "step.cu", "step_tile.cu", "batched_w8.cu", "ep_exchange.cu"]
HEADERS = ["common.cuh", "gemv_common.cuh", "stream.cuh", "stream_gemv.cuh", "step_kernel.h", "kernels.h", os.path.join(ROOT, "include", "lemoq_b200.h")]
LIB = os.path.join(HERE, "liblemoq_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
] + os.environ.get("LEMOQ_NVCC_EXTRA", "").split()


def _newer(src: str, dst: str) -> bool:
    return not os.path.exists(dst) or os.path.getmtime(src) > os.path.getmtime(dst)


def build(verbose: bool = False) -> str:
    deps = [h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS]
    objs, jobs = [], []
    for s in SOURCES:
        src = os.path.join(HERE, s)
        obj = os.path.join(HERE, s.replace(".cu", ".o"))
        objs.append(obj)
        if _newer(src, obj) or any(_newer(d, obj) for d in deps) or _newer(__file__, obj):
            cmd = [NVCC, *FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for %s" % cmd[-3])
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv))
