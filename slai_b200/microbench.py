"""Quantised GEMV microbenchmark mirroring slai-bench (crates/slai-bench/src/main.rs:73-247): one M x K matrix per
format, warm-up discarded, repeated timed launches, mean time per launch and the GB/s of packed weights + vectors.
Unlike the reference it rotates over several distinct weight copies so that the working set exceeds the L2 cache.

    python -m slai_b200.microbench --fmt q4_k --M 32000 --K 4096 [--copies 3] [--reps 20]

Also the small, self-contained launch sequence used for kernel profiling.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import synth
from .ops import Backend, GpuQuantMatrix, LlmContext


def run(fmt: int, M: int, K: int, copies: int, reps: int, warmup: int, device: int = 0):
    backend = Backend(device)
    ctx = LlmContext(backend)
    mats = [GpuQuantMatrix.synthetic(backend, fmt, M, K, 1000 + i, 0.02) for i in range(copies)]
    x = backend.vector(np.random.default_rng(1).standard_normal(K).astype(np.float32))
    out = backend.zeros(M)
    for i in range(warmup):
        ctx.matmul_quant_assign(out, mats[i % copies], x)
    backend.synchronize()
    backend.timer_start()
    for _ in range(reps):
        for m in mats:
            ctx.matmul_quant_assign(out, m, x)
    ms = backend.timer_stop()
    per = ms * 1e-3 / (reps * copies)
    algo = synth.gemv_bytes(fmt, M, K)
    return {"fmt": synth.FMT_NAMES[fmt], "M": M, "K": K, "copies": copies, "launches": reps * copies, "us_per_launch": per * 1e6,
            "algorithmic_bytes": algo, "GBs": algo / per / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fmt", default="q4_k", choices=["q8_0", "q4_k", "q5_k", "q6_k"])
    ap.add_argument("--M", type=int, default=32000)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--copies", type=int, default=3)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    print(json.dumps(run(synth.FMT_BY_NAME[a.fmt], a.M, a.K, a.copies, a.reps, a.warmup)))


if __name__ == "__main__":
    main()
