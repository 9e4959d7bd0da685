"""Quantised GEMV microbenchmark mirroring slai-bench (crates/slai-bench/src/main.rs:73-247): one M x K matrix per
format, warm-up discarded, repeated timed launches, mean time per launch and the GB/s of packed weights + vectors.
Unlike the reference it rotates over several distinct weight copies so that the working set exceeds the L2 cache.

    python -m slai_b200.microbench --fmt q4_k --M 32000 --K 4096 [--copies 3] [--reps 20]
    python -m slai_b200.microbench --fmt q4_k --M 11008 --K 4096 --pair      # RmsNorm + gate/up pair + SiLU in one kernel
    python -m slai_b200.microbench --fmt q4_k --M 11008 --K 4096 --batch 8   # eight vectors in one pass over the matrix

Also the small, self-contained launch sequence used for kernel profiling.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import synth
from .ops import Backend, GpuQuantMatrix, LlmContext


def run(fmt: int, M: int, K: int, copies: int, reps: int, warmup: int, device: int = 0, pair: bool = False, batch: int = 1):
    """pair: the decode step's feed-forward front half (slai_ffn_gate_up) on `copies` distinct (gate, up) pairs of M x K.
    batch: vectors per launch (slai_gemv_quant with n_batch; the algorithmic bytes count the matrix once)."""
    backend = Backend(device)
    ctx = LlmContext(backend)
    n_mat = 2 if pair else 1
    mats = [[GpuQuantMatrix.synthetic(backend, fmt, M, K, 1000 + n_mat * i + j, 0.02) for j in range(n_mat)] for i in range(copies)]
    x = backend.vector(np.random.default_rng(1).standard_normal(K * batch).astype(np.float32))
    nw = backend.vector(np.ones(K, dtype=np.float32))
    out = backend.zeros(M * batch)

    def launch(ms_):
        if pair:
            ctx.ffn_gate_up(out, ms_[0], ms_[1], x, nw, 1e-5)
        else:
            ctx.matmul_quant_assign(out, ms_[0], x, n_batch=batch)

    for i in range(warmup):
        launch(mats[i % copies])
    backend.synchronize()
    backend.timer_start()
    for _ in range(reps):
        for m in mats:
            launch(m)
    ms = backend.timer_stop()
    per = ms * 1e-3 / (reps * copies)
    algo = n_mat * synth.gemv_bytes(fmt, M, K) - (n_mat - 1) * 4 * (K + M) + (batch - 1) * 4 * (K + M)
    return {"fmt": synth.FMT_NAMES[fmt], "M": M, "K": K, "pair": pair, "batch": batch, "copies": copies, "launches": reps * copies, "us_per_launch": per * 1e6,
            "algorithmic_bytes": algo, "GBs": algo / per / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fmt", default="q4_k", choices=["q8_0", "q4_k", "q5_k", "q6_k"])
    ap.add_argument("--M", type=int, default=32000)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--copies", type=int, default=3)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--pair", action="store_true", help="RmsNorm + gate/up GEMV pair + SiLU (two M x K matrices per launch)")
    ap.add_argument("--batch", type=int, default=1, help="vectors per launch (1..8)")
    a = ap.parse_args()
    print(json.dumps(run(synth.FMT_BY_NAME[a.fmt], a.M, a.K, a.copies, a.reps, a.warmup, pair=a.pair, batch=a.batch)))


if __name__ == "__main__":
    main()
