"""Reader of the trace build's device-side timeline.

    python -m slai_b200.build --trace          # builds slai_b200/libslai_b200_trace.so (-DSLAI_TRACE)
    python -m slai_b200.trace [--tokens 4] [--prompt 512] [--model 7b|70b|gpt2xl] [--layers N]

The trace library stamps %globaltimer inside the decode kernels (block 0 of every GEMV / attention launch: start,
ring requested, predecessor done, input staged, main loop done, partials reduced, end) and appends one record per
launch to a device-side list, in execution order and inside the replayed CUDA graph, so the token is seen as it
really runs.  This module loads that library instead of the shipped one, decodes a few tokens of a synthetic
model and prints, per kernel of a layer, where the time goes, plus the gaps between kernels.  It is the tool
behind the per-kernel tables in the design notes; the shipped library contains none of the instrumentation.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
TRACE_LIB = os.environ.get("SLAI_B200_TRACE_LIB") or os.path.join(_HERE, "libslai_b200_trace.so")

PRO = {0: "", 1: "rms+", 2: "ln+"}
EPI = {0: "store", 1: "resid", 2: "silu", 3: "gelu", 4: "qkv", 5: "xchg"}


def kernel_name(kid: int) -> str:
    if kid == 999:
        return "attention"
    k256, rest = divmod(kid, 1000)
    nmat, rest = divmod(rest, 100)
    pro, epi = divmod(rest, 10)
    return f"gemv K={256 * k256} {PRO.get(pro, '?')}{EPI.get(epi, '?')}" + (" x2" if nmat == 2 else "")


SLOTS, CAP = 16, 4096
# Stamps of a GEMV launch (block 0), see common.cuh: the columns printed are the differences between consecutive ones.
COLS = (("init", 0, 1), ("fill", 1, 2), ("pre", 2, 3), ("wait", 3, 4), ("setup", 4, 5), ("load", 5, 6), ("stats", 6, 7),
        ("digits", 7, 8), ("bar", 8, 9), ("loop", 9, 10), ("sync", 10, 11), ("epi", 11, 12), ("exit", 12, 13))


def read_timeline(backend, cap=CAP):
    lib = backend.lib
    buf = np.zeros(SLOTS * cap, dtype=np.uint64)
    cnt = C.c_uint(0)
    rc = lib.slai_debug_timeline(backend.h, buf.ctypes.data_as(C.c_void_p), C.c_size_t(buf.nbytes), C.byref(cnt))
    if rc != 0:
        raise RuntimeError(f"slai_debug_timeline failed ({rc})")
    n = min(int(cnt.value), cap)
    return buf[: SLOTS * n].reshape(n, SLOTS).astype(np.int64)


def summarise(rec: np.ndarray):
    """rec: one token's records [id, stamp 0..14] in execution order.  Per kernel (in order of first appearance): mean
    microseconds of every phase of block 0, the whole kernel, the period (start to the next kernel's start) and the
    hand-over (this kernel's end to the moment the next kernel sees its predecessor done)."""
    rows, order = {}, []
    for i in range(len(rec)):
        kid = int(rec[i, 0])
        t = rec[i, 1:].astype(np.float64) * 1e-3
        key = kernel_name(kid)
        if key not in rows:
            rows[key] = []
            order.append(key)
        if kid == 999:
            parts = [0.0] * len(COLS)
            parts[3] = t[4] - t[0]
            parts[9] = t[13] - t[4]
        else:
            parts = [t[b] - t[a] for _, a, b in COLS]
        period = (rec[i + 1, 1] * 1e-3 - t[0]) if i + 1 < len(rec) else np.nan
        handover = (rec[i + 1, 5] * 1e-3 - t[13]) if i + 1 < len(rec) else np.nan
        rows[key].append(parts + [t[13] - t[0], period, handover])
    return [(key, len(rows[key]), *np.nanmean(np.array(rows[key]), axis=0)) for key in order]


def block_report(backend, nblocks):
    """Per-block view of the GEMV launches still in the trace ring (the graph's launches stamp into fixed slots, so
    after a replay every slot holds its launch of the last token): for every stamp the earliest, median and latest
    block, relative to the earliest start of the launch."""
    lib = backend.lib
    ring = np.zeros(64 * 256 * 16, dtype=np.uint64)
    n = C.c_ulonglong(0)
    lib.slai_debug_trace_ring.restype = C.c_int
    rc = lib.slai_debug_trace_ring(backend.h, ring.ctypes.data_as(C.c_void_p), C.c_size_t(ring.nbytes), C.byref(n))
    if rc != 0:
        raise RuntimeError(f"slai_debug_trace_ring failed ({rc})")
    ring = ring.reshape(64, 256, 16).astype(np.int64)
    names = ["start", "init", "fill", "pre", "waited", "setup", "loaded", "stats", "digits", "staged", "loop", "synced", "epi", "end"]
    out = []
    for slot in range(64):
        t = ring[slot, :nblocks, :14].astype(np.float64) * 1e-3
        used = t[:, 0] > 0
        if used.sum() < 2:
            continue
        t = t[used]
        t0 = t[:, 0].min()
        out.append((t0, slot, int(used.sum()), t - t0))
    out.sort()
    for t0, slot, nb, t in out[-6:]:
        print(f"slot {slot}: {nb} blocks; microseconds after the earliest block start: min / median / max over blocks")
        print("   " + " ".join(f"{nm:>17s}" for nm in names))
        print("   " + " ".join(f"{t[:, k].min():5.2f}/{np.median(t[:, k]):5.2f}/{t[:, k].max():5.2f}" for k in range(14)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", action="store_true", help="also print the per-block spread of the last GEMV launches")
    ap.add_argument("--tokens", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--model", default="7b", choices=["7b", "70b", "gpt2xl"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the architecture has (0 = all)")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--tp", action="store_true", help="70b only: shard the model over the ranks of a torch.distributed launch "
                    "(python -m torch.distributed.run --nproc-per-node N -m slai_b200.trace --model 70b --tp); rank 0 prints its timeline")
    a = ap.parse_args()
    if not os.path.exists(TRACE_LIB):
        sys.exit("build the trace library first: python -m slai_b200.build --trace")
    os.environ["SLAI_B200_LIB"] = TRACE_LIB
    from . import synth
    from .ops import Backend
    rank, world = 0, 1
    if a.tp:
        import torch
        import torch.distributed as dist
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl")
    backend = Backend(int(os.environ.get("LOCAL_RANK", "0")) if a.tp else 0)
    lib = backend.lib
    lib.slai_debug_timeline.restype = C.c_int
    if a.tp:
        import dataclasses
        from . import tp
        from .models import LLAMA2_70B
        cfg = dataclasses.replace(LLAMA2_70B, n_layers=a.layers) if a.layers > 0 else LLAMA2_70B
        if world > 1:
            tp.join_group(backend, rank, world, tp.torch_broadcast)
            tp.enable_peer_exchange(backend, world, tp.torch_all_gather, tp.torch_barrier)
        m = tp.synthetic_llama_device_tp(backend, cfg, synth.FMT_Q4_K, synth.FMT_Q6_K, rank, world)
        vocab = cfg.vocab_size
        backend.synchronize()
        tp.torch_barrier()
    elif a.model in ("7b", "70b"):
        import dataclasses
        from .models import LLAMA2_7B, LLAMA2_70B, synthetic_llama_device
        cfg = LLAMA2_7B if a.model == "7b" else LLAMA2_70B
        if a.layers > 0:
            cfg = dataclasses.replace(cfg, n_layers=a.layers)
        m = synthetic_llama_device(backend, cfg, synth.FMT_Q4_K, synth.FMT_Q6_K)
        vocab = cfg.vocab_size
    else:
        from .models import GPT2_XL, synthetic_gpt2_device
        cfg = GPT2_XL
        m = synthetic_gpt2_device(backend, cfg, synth.FMT_Q8_0, seed=0)
        vocab = cfg.n_vocab
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, vocab, size=a.prompt).astype(np.int32)
    m.prefill(prompt[:-1], 0)
    toks = m.generate(int(prompt[-1]), a.prompt - 1, 3)  # graph warm-up
    read_timeline(backend)  # drop what has accumulated
    toks = m.generate(int(toks[-1]), a.prompt + 2, a.tokens)
    rec = read_timeline(backend)
    per_tok = len(rec) // a.tokens
    last = rec[(a.tokens - 1) * per_tok:]
    rows = summarise(last)
    t_tok = (last[-1, 14] - last[0, 1]) * 1e-3
    names = [c[0] for c in COLS] + ["kernel", "period", "handover"]
    if a.tp:  # every rank leaves the group the same way; only rank 0 reports
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
        if rank != 0:
            return
    if a.json:
        print(json.dumps({"token_us": t_tok, "records_per_token": per_tok,
                          "kernels": [dict(zip(["name", "n"] + names, r)) for r in rows]}))
        return
    if a.blocks:
        block_report(backend, backend.device_info()[1])
    print(f"last token: {per_tok} traced launches, {t_tok:.1f} us from the first traced start to the last traced end (us, block 0)")
    print(f"{'kernel':28s} {'n':>3s} " + " ".join(f"{n:>6s}" for n in names))
    for r in rows:
        print(f"{r[0]:28s} {r[1]:3d} " + " ".join(f"{x:6.2f}" for x in r[2:]))


if __name__ == "__main__":
    main()
