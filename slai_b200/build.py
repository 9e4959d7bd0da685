"""Builds libslai_b200.so (sm_100a only) in-tree with nvcc.  No JIT cache: the built library sits next to
its sources so that it travels with the repository snapshot."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libslai_b200.so")
SOURCES = ["gemv.cu", "gemv_batch.cu", "attention.cu", "ops.cu", "model.cu", "tp.cu", "sampler.cu", "prefill.cu"]
HEADERS = ["common.cuh", "dequant.cuh", "gemv_frag.cuh", "gemv_formats.cuh", "gemv_kernel.cuh", "attention.cuh", "layout.cuh", os.path.join("..", "..", "include", "slai_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """trace=True builds libslai_b200_trace.so with -DSLAI_TRACE (device-side timeline, read by slai_b200/trace.py)."""
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objdir = os.path.join(HERE, "build_trace" if trace else "build")
    lib = os.path.join(HERE, "libslai_b200_trace.so") if trace else LIB
    flags = NVCC_FLAGS + (["-DSLAI_TRACE"] if trace else []) + os.environ.get("SLAI_NVCC_EXTRA", "").split()
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    objs = []
    for src in SOURCES:
        sp = os.path.join(CSRC, src)
        op = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(op)
        if force or _stale(op, [sp] + hdrs):
            jobs.append([_nvcc(), *flags, "-c", sp, "-o", op] + (["-Xptxas", "-v"] if verbose else []))

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=4) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        for l in logs:
            sys.stderr.write(l)
    if jobs or force or _stale(lib, objs):
        run([_nvcc(), "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
             "-lcudart", "-ldl"])
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
