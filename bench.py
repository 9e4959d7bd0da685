#!/usr/bin/env python
"""Benchmark of the decode hot path: Llama-2-7B architecture, Q4_K weights (Q6_K logits matrix), batch 1,
fp16 KV cache, 512-token prompt, greedy decoding (the headline benchmark configuration).  Synthetic seeded weights generated on
the GPU stand in for a checkpoint.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--gemv]

One step = one decoded token.  Prints ONE JSON line (rank 0).  `value` is tokens/s with everything resident in
HBM (device-side greedy loop, CUDA events); `e2e` is the same metric through the per-token public call with the
token id going host->device and the logits + greedy token coming back to pinned host memory every step.
With N > 1 the path does not shard at this model size (replicas only): every rank decodes its own sequence.
`--impl reference` times the reference's CPU operator path (CPU oracle port, all host threads) on a bounded
sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 512
WORKLOAD = "llama2-7b-arch q4_k (q6_k logits) bs1 decode, 512-token prompt, fp16 KV (the headline benchmark configuration)"


def workload_config(world: int, steps: int, warmup: int) -> dict:
    """The `config` object of the JSON line, identical for the CUDA arm and the reference arm."""
    first = PROMPT_LEN - 1 + warmup
    return {"workload": WORKLOAD, "prompt_len": PROMPT_LEN, "decode_positions": [first, first + steps - 1],
            "parallelism": "single GPU" if world == 1 else f"replicas x{world} (path does not shard at this model size)",
            "l2": "every token streams 3.75 GB of weights, far larger than the 126 MB L2 (no flush needed)"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, burst copy)"
    return 6650.0, "fallback (6.65 TB/s earlier measurement on this pool)"


def measured_tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier measurement on this pool)"


def prefill_record(cfg, n_tokens, seconds, sequential_ms_per_token=None, n_gpus=1):
    """Prompt processing of `n_tokens` through the tensor-core GEMM path: model FLOPs = 2 x layer weights x tokens (the
    logits matrix is applied to the last token only).  Every model product is issued as three fp16 products
    (hi*hi, hi*lo, lo*hi of fp16 operand pairs, f32 accumulation), so the tensor cores execute three times the model
    FLOPs; both figures are given against the measured dense bf16 peak (of all `n_gpus` GPUs for a sharded model, whose
    ranks each run their shard of every GEMM and sum the row-parallel products with an all-reduce)."""
    peak, src = measured_tensor_peak()
    peak *= n_gpus
    layer_params = sum(r * c for r, c in cfg.matrix_shapes().values())
    flops = 2.0 * cfg.n_layers * layer_params * n_tokens
    rec = {"tokens": n_tokens, "seconds": seconds, "tok_s": n_tokens / seconds, "model_tflops": flops / seconds / 1e12,
           "tensor_tflops_executed": 3 * flops / seconds / 1e12, "operands": "fp16 pairs (hi + lo) for weights and activations, f32 accumulators in TMEM",
           "peak_tflops": peak, "frac_model": flops / seconds / 1e12 / peak, "frac_executed": 3 * flops / seconds / 1e12 / peak, "peak_source": src}
    if sequential_ms_per_token:
        rec["sequential_estimate_s"] = sequential_ms_per_token * 1e-3 * n_tokens
        rec["speedup_vs_sequential"] = rec["sequential_estimate_s"] / seconds
    return rec


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [r.strip().split(", ") for r in open(self.f.name) if r.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons, power = [], [], set(), []
        for r in rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); power.append(float(r[3]))
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.strip().lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "power_w_max": float(max(power)),
                "samples": len(sm), "reasons": sorted(reasons)}


def build_model(backend, seed=0):
    """Llama-2-7B-architecture model with device-generated weights; layer 0 and the logits matrix keep their raw
    GGUF blocks so the CPU baseline can run on exactly the same bytes."""
    from slai_b200 import synth
    from slai_b200.models import LLAMA2_7B, Llama2
    from slai_b200.ops import GpuQuantMatrix, GpuVector
    cfg = LLAMA2_7B
    m = Llama2(backend, cfg)
    sid = seed * 1_000_003
    raw = {}
    mats = {}
    for l in range(cfg.n_layers):
        for i, (name, (r, c)) in enumerate(cfg.matrix_shapes().items()):
            qm = GpuQuantMatrix.synthetic(backend, synth.FMT_Q4_K, r, c, sid + 100 * l + i + 1, 0.02, keep_raw=(l == 0))
            m.set_matrix(name, l, qm)
            mats[(name, l)] = qm
            if l == 0:
                raw[name] = qm
        ones = np.ones(cfg.dim, dtype=np.float32)
        m.set_f32("attn_norm", l, ones)
        m.set_f32("ffn_norm", l, ones)
    emb = GpuVector(backend, cfg.vocab_size * cfg.dim)
    backend.check(backend.lib.slai_synth_normal_f32(backend.h, C.c_void_p(emb.ptr), emb.n, sid + 7_000_001, 0.02))
    m.set_f32("token_embd", -1, emb)
    del emb
    m.set_f32("out_norm", -1, np.ones(cfg.dim, dtype=np.float32))
    out = GpuQuantMatrix.synthetic(backend, synth.FMT_Q6_K, cfg.vocab_size, cfg.dim, sid + 7_000_002, 0.02, keep_raw=True)
    m.set_matrix("output", -1, out)
    raw["output"] = out
    return cfg, m, mats, raw


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate/up kernel on 2 x 11008 x 4096 Q4_K, from an ncu capture
# of `python -m slai_b200.microbench --fmt q4_k --M 11008 --K 4096 --pair` (summary under profiles/): 2 x 688 tiles x 16 steps x 2368-byte blocks = 52 137 984 bytes of weights (the 2.8 % above the
# GGUF byte count being the unpacked scales) plus the vectors
DOMINANT_KERNEL_DRAM_BYTES = 52_230_000


def time_dominant_kernel(backend, ctx, cfg, mats, rounds=8):
    """Average duration of the decode step's dominant kernel: RmsNorm + gate/up GEMV pair + SiLU (2 x 11008 x 4096 Q4_K, the
    largest share of the step), run on the gate / up matrices of all 32 layers in turn (1.6 GB, larger than L2) as one
    recorded pass, CUDA events on the launching stream.  Algorithmic bytes: both matrices' GGUF bytes + input + output."""
    from slai_b200 import synth
    x = backend.vector(np.random.default_rng(0).standard_normal(cfg.dim).astype(np.float32))
    nw = backend.vector(np.ones(cfg.dim, dtype=np.float32))
    out = backend.zeros(cfg.hidden_dim)
    pairs = [(mats[("w_gate", l)], mats[("w_up", l)]) for l in range(cfg.n_layers)]
    for g, u in pairs[:4]:
        ctx.ffn_gate_up(out, g, u, x, nw, 1e-5)
    backend.synchronize()
    with backend.record() as rec:  # one recorded pass over the 32 layers: no host work between the launches
        for g, u in pairs:
            ctx.ffn_gate_up(out, g, u, x, nw, 1e-5)
    rec.launch(2)
    backend.synchronize()
    backend.timer_start()
    rec.launch(rounds)
    ms = backend.timer_stop()
    rec.close()
    n = rounds * len(pairs)
    per = ms / n * 1e-3
    algo = 2 * synth.gemv_bytes(synth.FMT_Q4_K, cfg.hidden_dim, cfg.dim) - 4 * cfg.dim - 4 * cfg.hidden_dim  # one input, one output
    return algo, per, n


def gemv_microbench(backend, ctx, peak):
    """The GEMV microbenchmark configuration: quantised GEMV on the four Llama-2-7B shapes x four formats, rotating over enough
    distinct weight copies that the working set exceeds L2."""
    from slai_b200 import synth
    from slai_b200.ops import GpuQuantMatrix
    res = []
    for (M, K) in ((4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)):
        for fmt in (synth.FMT_Q8_0, synth.FMT_Q4_K, synth.FMT_Q5_K, synth.FMT_Q6_K):
            algo = synth.gemv_bytes(fmt, M, K)
            ncopies = max(2, int(np.ceil(200e6 / algo)) + 1)
            mats = [GpuQuantMatrix.synthetic(backend, fmt, M, K, 1000 + i, 0.02) for i in range(ncopies)]
            x = backend.vector(np.random.default_rng(1).standard_normal(K).astype(np.float32))
            out = backend.zeros(M)
            for m_ in mats[:3]:
                ctx.matmul_quant_assign(out, m_, x)
            backend.synchronize()
            reps = max(1, 60 // ncopies)
            with backend.record() as rec:
                for m_ in mats:
                    ctx.matmul_quant_assign(out, m_, x)
            rec.launch(1)
            backend.synchronize()
            backend.timer_start()
            rec.launch(reps)
            ms = backend.timer_stop()
            rec.close()
            per = ms * 1e-3 / (reps * ncopies)
            res.append({"M": M, "K": K, "fmt": synth.FMT_NAMES[fmt], "us": round(per * 1e6, 2), "GBs": round(algo / per / 1e9, 1),
                        "frac": round(algo / per / 1e9 / peak, 3)})
            del mats
    return res


def host_layer_blocks(cfg, seed=0):
    """Layer 0 and the logits matrix of the benchmark model as raw GGUF blocks made on the host (numpy quantisers of
    slai_b200/synth.py): what the reference arm runs on, with no GPU and no CUDA library involved."""
    from slai_b200 import synth
    raw = {}
    for i, (name, (r, c)) in enumerate(cfg.matrix_shapes().items()):
        raw[name] = synth.quantize(synth.FMT_Q4_K, synth.normal_matrix(seed * 1_000_003 + i + 1, r, c, 0.02))
    raw["output"] = synth.quantize(synth.FMT_Q6_K, synth.normal_matrix(seed * 1_000_003 + 7_000_002, cfg.vocab_size, cfg.dim, 0.02))
    return raw


class CpuLayer:
    """The reference's CPU path on layer 0 and the logits matrix of the benchmark model: weights dequantised to f32
    at load (models/llama2/cpu.rs:200-219), dense f32 gemv per matrix (:370-376), attention over `pos`+1 positions."""

    def __init__(self, cfg, raw_blocks):
        from oracle import oracle as O
        from slai_b200 import synth
        self.cfg = cfg
        self.W = {name: O.dequantize(synth.FMT_Q4_K, raw_blocks[name]).reshape(r, c) for name, (r, c) in cfg.matrix_shapes().items()}
        self.Wout = O.dequantize(synth.FMT_Q6_K, raw_blocks["output"]).reshape(cfg.vocab_size, cfg.dim)
        rng = np.random.default_rng(0)
        self.x = rng.standard_normal(cfg.dim).astype(np.float32)
        self.kc = rng.standard_normal((cfg.seq_len, cfg.kv_dim)).astype(np.float32)
        self.vc = rng.standard_normal((cfg.seq_len, cfg.kv_dim)).astype(np.float32)

    def times(self, pos, nthreads, reps=2):
        """(seconds per layer, seconds for the logits gemv), best of `reps`."""
        from oracle import oracle as O
        cfg, W, x = self.cfg, self.W, self.x
        ones = np.ones(cfg.dim, np.float32)
        kc, vc = self.kc[: pos + 1], self.vc[: pos + 1]
        best_layer, best_out = 1e9, 1e9
        for _ in range(reps):
            t0 = time.perf_counter()
            xb = O.rms_norm(x, ones, cfg.rms_norm_eps)
            q = O.gemv_f32(W["wq"], xb, nthreads)
            k = O.gemv_f32(W["wk"], xb, nthreads)
            v = O.gemv_f32(W["wv"], xb, nthreads)
            q, k = O.rope(q, k, cfg.head_size, cfg.kv_dim, pos)
            kc[pos], vc[pos] = k, v
            att, _ = O.attention(q, kc, vc, seq_len=pos + 1, kv_dim=cfg.kv_dim, kv_mul=1, n_heads=cfg.n_q_heads, head_size=cfg.head_size, pos=pos)
            x2 = x + O.gemv_f32(W["wo"], att, nthreads)
            xb = O.rms_norm(x2, ones, cfg.rms_norm_eps)
            hb = O.silu_gate(O.gemv_f32(W["w_gate"], xb, nthreads), O.gemv_f32(W["w_up"], xb, nthreads))
            x2 = x2 + O.gemv_f32(W["w_down"], hb, nthreads)
            t1 = time.perf_counter()
            O.gemv_f32(self.Wout, O.rms_norm(x2, ones, cfg.rms_norm_eps), nthreads)
            t2 = time.perf_counter()
            best_layer, best_out = min(best_layer, t1 - t0), min(best_out, t2 - t1)
        return best_layer, best_out


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU implementation of the path (the oracle port; the Rust reference cannot be
    built here) with all host threads, on a bounded sample per step: one full layer + the logits GEMV of the same
    model shape, extrapolated to 32 layers.  Runs on the host alone: the CUDA library is not loaded."""
    if rank != 0:
        return
    from slai_b200.models import LLAMA2_7B
    cfg = LLAMA2_7B
    layer = CpuLayer(cfg, host_layer_blocks(cfg))
    nthreads = os.cpu_count() or 1
    times = []
    for i in range(args.warmup + args.steps):
        tl, to = layer.times(PROMPT_LEN - 1 + i, nthreads, reps=1)
        if i >= args.warmup:
            times.append(cfg.n_layers * tl + to)
    ms = 1e3 * float(np.mean(times))
    val = 1e3 / ms
    line = {"impl": "reference", "metric": "decode tok/s bs1 (Llama-2-7B Q4_K)", "value": val, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(world, args.steps, args.warmup),
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": nthreads, "kind": "port",
                             "sample": "per step: one full layer (7 dense f32 gemvs on dequantised weights, attention over the "
                                       "prompt) + the logits gemv on the host, layer time x32"},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def run_gpt2(args):
    """The GPT-2 XL benchmark configuration (48 layers, dim 1600, 25 heads, FFN 6400, vocab 50257, tied logits, Q8_0
    weights, fp16 KV, batch 1): 128-token prompt, then the timed greedy tokens.  Not the default workload: `--gpt2`."""
    from slai_b200 import synth
    from slai_b200.models import GPT2_XL, synthetic_gpt2_device
    from slai_b200.ops import Backend
    backend = Backend(0)
    p = GPT2_XL
    m = synthetic_gpt2_device(backend, p, synth.FMT_Q8_0, seed=0)
    peak, peak_src = measured_peaks()
    K, W, PL = args.steps, args.warmup, 128
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, p.n_vocab, size=PL).astype(np.int32)
    m.prefill(prompt[:-1], 0)  # warm-up (the prompt buffers get their size), overwritten by the timed pass
    backend.synchronize()
    t0 = time.perf_counter()
    m.prefill(prompt[:-1], 0)
    prefill_s = time.perf_counter() - t0
    warm = m.generate(int(prompt[-1]), PL - 1, W)
    tok, pos = int(warm[-1]), PL - 1 + W
    sampler = ClockSampler(0)
    backend.synchronize()
    backend.timer_start()
    toks = m.generate(tok, pos, K)
    ms = backend.timer_stop()
    clocks = sampler.stop()
    esz = 2
    kv = float(np.mean([2 * p.n_layer * p.n_embd * esz * (q + 1) for q in range(pos, pos + K)]))
    bytes_tok = p.weight_bytes_per_token(synth.FMT_Q8_0) + kv
    t = ms * 1e-3 / K
    line = {"metric": "decode tok/s bs1 (GPT-2 XL Q8_0)", "value": K / (ms * 1e-3), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "gpt2-xl-arch q8_0 bs1 decode, 128-token prompt, fp16 KV", "decode_positions": [pos, pos + K - 1]},
            "clocks": clocks,
            "prefill": {"tokens": PL - 1, "seconds": prefill_s, "tok_s": (PL - 1) / prefill_s, "sequential_estimate_s": (PL - 1) * ms / K * 1e-3,
                        "speedup_vs_sequential": (PL - 1) * ms / K * 1e-3 / prefill_s,
                        "path": "tcgen05 GEMMs, fp16-pair operands (LayerNorm / bias / GELU variants of the Llama prompt pass)"},
            "roofline": {"bound": "hbm", "bytes_per_token": bytes_tok, "achieved": bytes_tok / t / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": bytes_tok / t / 1e9 / peak, "peak_source": peak_src}}
    emit(line)


def measure_batch(m, cfg, n_seq, prompt_len, steps, warmup, bs1_ms_per_token):
    """`n_seq` sequences decoded together through slai_llama_decode_batch (one KV cache and position per sequence, every
    weight matrix read once per step for all of them): the prompts advance in lockstep, one token of every sequence per
    step, then `warmup` + `steps` greedy steps; wall-clock per step of the blocking call (ids read back every step)."""
    rng = np.random.default_rng(7)
    prompts = rng.integers(0, cfg.vocab_size, size=(n_seq, prompt_len)).astype(np.int32)
    m.batch_reserve(n_seq)
    try:
        nxt = prompts[:, 0]
        for p in range(prompt_len):
            _, nxt = m.decode_batch(prompts[:, p], [p] * n_seq, want_logits=False)
        pos = prompt_len
        for _ in range(warmup):
            _, nxt = m.decode_batch(nxt, [pos] * n_seq, want_logits=False)
            pos += 1
        t0 = time.perf_counter()
        for _ in range(steps):
            _, nxt = m.decode_batch(nxt, [pos] * n_seq, want_logits=False)
            pos += 1
        dt = time.perf_counter() - t0
    finally:
        m.batch_reserve(0)
    return {"n_seq": n_seq, "value": n_seq * steps / dt, "unit": "tok/s (all sequences)", "ms_per_step": dt / steps * 1e3, "steps": steps,
            "warmup": warmup, "prompt_len": prompt_len, "decode_positions": [pos - steps, pos - 1],
            "vs_one_sequence_at_a_time": (n_seq * steps / dt) / (1e3 / bs1_ms_per_token),
            "timing": "wall clock around the blocking per-step call: token ids and positions H2D, greedy ids D2H every step"}


def _tp_bit_identity(backend, group, cfg70):
    """Two layers of the 70B shape decoded twice, the half-layer sums once through NCCL all-reduce and once through
    the peer-memory exchange inside the GEMV kernels: same logits bit for bit and same greedy ids."""
    from slai_b200 import synth, tp
    from slai_b200.models import Llama2Config
    small = Llama2Config(**{**cfg70.__dict__, "n_layers": 2, "seq_len": 64})
    res = []
    for force_nccl in (True, False):
        if force_nccl:
            os.environ["SLAI_TP_NCCL"] = "1"
        else:
            os.environ.pop("SLAI_TP_NCCL", None)
        m = tp.synthetic_llama_device_tp(backend, small, synth.FMT_Q4_K, synth.FMT_Q6_K, group.rank, group.world, seed=3)
        backend.synchronize()
        group.barrier()
        lg, _ = m.forward_logits(0, 11)
        ids = list(m.generate(12, 1, 16))
        res.append((lg.copy(), ids))
        m.close()
    os.environ.pop("SLAI_TP_NCCL", None)
    same = bool(np.array_equal(res[0][0].view(np.uint32), res[1][0].view(np.uint32)) and res[0][1] == res[1][1])
    (agree,) = group.sum_over_ranks([1.0 if same else 0.0])
    return agree == group.world


def measure_tp(args, group, n_layers=0, prompt_len=1024, steps=None, warmup=None, nccl_only=False):
    """The 70B benchmark configuration (Llama-2-70B architecture, Q4_K + Q6_K logits, fp16 KV, batch 1, 1024-token
    prompt) sharded over all ranks: tensor parallel, one sum per half-layer, logits matrix sharded by rows.  Returns the
    record rank 0 reports (None on the other ranks).  At one rank it is the unsharded model on one GPU."""
    from slai_b200 import synth, tp
    from slai_b200.models import LLAMA2_70B, Llama2Config
    from slai_b200.ops import Backend
    rank, world = group.rank, group.world
    backend = Backend(group.local_rank)
    cfg = LLAMA2_70B if n_layers <= 0 else Llama2Config(**{**LLAMA2_70B.__dict__, "n_layers": n_layers})
    K = steps or min(args.steps, 64)
    W = warmup or max(3, min(args.warmup, 8))
    exchange, identical = "none (one GPU)", None
    if world > 1:
        tp.join_group(backend, rank, world, tp.torch_broadcast)
        exchange = "NCCL all-reduce of 8192 f32 after wo and w_down"
        if not nccl_only:
            tp.enable_peer_exchange(backend, world, tp.torch_all_gather, tp.torch_barrier)
            exchange = "peer-memory stores from the wo / w_down kernels, summed in the next kernel's prologue (no collective kernel)"
            identical = _tp_bit_identity(backend, group, cfg)
        m = tp.synthetic_llama_device_tp(backend, cfg, synth.FMT_Q4_K, synth.FMT_Q6_K, rank, world)
    else:
        from slai_b200.models import synthetic_llama_device
        m = synthetic_llama_device(backend, cfg, synth.FMT_Q4_K, synth.FMT_Q6_K)
    peak, peak_src = measured_peaks()
    PL = prompt_len
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, cfg.vocab_size, size=PL).astype(np.int32)
    # The peer exchange waits a bounded time (about a second) for the other ranks' partial sums: start the first step together,
    # not whenever each rank has finished building its shard.
    backend.synchronize()
    group.barrier()
    # warm-up, overwritten by the timed pass: the whole prompt, so that the prompt buffers (grown on demand and kept by the
    # library) have their size before the timed pass, as for every prompt after a server's first
    m.prefill(prompt[:-1], 0)
    backend.synchronize()
    group.barrier()
    t0 = time.perf_counter()
    m.prefill(prompt[:-1], 0)
    prefill_s = time.perf_counter() - t0
    tok, pos = int(prompt[-1]), PL - 1
    warm = m.generate(tok, pos, W)
    tok, pos = int(warm[-1]), pos + W
    sampler = ClockSampler(group.local_rank)
    group.barrier()
    backend.synchronize()
    backend.timer_start()
    toks = m.generate(tok, pos, K)
    ms = backend.timer_stop()
    group.barrier()
    clocks = sampler.stop()
    ids = group.gather_ids(toks)
    ms, prefill_s = group.max_over_ranks([ms, prefill_s])
    batch = None
    if world == 1 and not getattr(args, "no_batch", False):
        try:  # BASELINE configs[4] also names batch 8: eight sequences per step, the weights read once
            batch = measure_batch(m, cfg, 8, 128, 16, 3, ms / K)
        except Exception as e:
            batch = {"error": f"{type(e).__name__}: {e}"}
    rec = None
    if rank == 0:
        per_rank = tp.bytes_per_token_per_rank(cfg, synth.FMT_Q4_K, synth.FMT_Q6_K, world)
        kv = float(np.mean([cfg.kv_bytes_at(p) for p in range(pos, pos + K)])) / world
        t = ms * 1e-3 / K
        rec = {"metric": "decode tok/s bs1 (Llama-2-70B Q4_K, tensor parallel)", "value": K / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
               "steps": K, "warmup": W, "ms_per_step": ms / K, "scaling": "strong",
               "config": {"workload": "llama2-70b-arch q4_k (q6_k logits) bs1 decode, fp16 KV", "n_layers": cfg.n_layers,
                          "prompt_len": PL, "decode_positions": [pos, pos + K - 1], "parallelism": f"tp{world}", "exchange": exchange,
                          "logits": "output matrix sharded by rows, logits all-gathered" if world > 1 else "whole output matrix"},
               "prefill_s": prefill_s,
               "prefill": prefill_record(cfg, PL - 1, prefill_s, ms / K, n_gpus=world),
               "clocks": clocks, "launches_per_token": m.launches_per_token(), "gpu_launches": m.launches_per_token() * K,
               "ranks_agree": all(r == ids[0] for r in ids), "nccl_and_peer_exchange_bit_identical": identical, "batch8": batch,
               "roofline": {"bound": "hbm", "per_gpu_bytes_per_token": per_rank + kv, "achieved": (per_rank + kv) / t / 1e9, "peak": peak,
                            "unit": "GB/s", "frac": (per_rank + kv) / t / 1e9 / peak, "peak_source": peak_src}}
    m.close()
    if world > 1:
        backend.check(backend.lib.slai_tp_shutdown(backend.h))
    backend.close()
    return rec


def run_tp(args, group):
    """`--tp`: only the sharded 70B measurement, as the one JSON line."""
    rec = measure_tp(args, group, n_layers=args.tp_layers, prompt_len=args.prompt_len if args.prompt_len != 512 else 1024,
                     steps=args.steps, warmup=args.warmup, nccl_only=args.tp_nccl)
    if rec is not None:
        rec.update({"higher_is_better": True, "vs_baseline": None, "dtype": "f32", "data": "synthetic (shards seeded per rank)"})
        emit(rec)
    group.close()


_RESULT_FD = None


def emit(line: dict) -> None:
    """The one JSON line, on the process's original standard output."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # Libraries print to file descriptor 1 as they please (NCCL's version banner, for one): everything written there during
    # the run is sent to stderr, and the one JSON line goes to the original standard output.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--gemv", action="store_true", help="also run the 16-case quantised GEMV microbenchmark")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--prompt-len", type=int, default=512, help="prompt length (512 = the benchmark; smaller for profiling)")
    ap.add_argument("--gpt2", action="store_true", help="GPT-2 XL architecture (Q8_0) instead of Llama-2-7B; one GPU")
    ap.add_argument("--tp", action="store_true", help="Llama-2-70B architecture sharded over all ranks instead of 7B replicas")
    ap.add_argument("--tp-layers", type=int, default=0, help="with --tp: fewer layers than 80 (0 = the full model)")
    ap.add_argument("--tp-nccl", action="store_true", help="with --tp: exchange through NCCL all-reduce instead of peer memory")
    ap.add_argument("--no-batch", action="store_true", help="skip the eight-sequences-per-step measurement (`batch8`, one GPU only)")
    ap.add_argument("--no-tp", action="store_true", help="skip the sharded 70B measurement that the default run attaches as `tp`")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global PROMPT_LEN
    PROMPT_LEN = args.prompt_len

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if args.gpt2:
        if rank == 0:
            run_gpt2(args)
        return
    from slai_b200.replicas import ReplicaGroup
    group = ReplicaGroup(backend="nccl")
    if args.tp:
        run_tp(args, group)
        return

    from slai_b200 import synth
    from slai_b200.ops import Backend, LlmContext
    backend = Backend(local)
    ctx = LlmContext(backend)
    peak, peak_src = measured_peaks()
    cfg, m, mats, raw = build_model(backend, seed=rank)
    K, W = args.steps, args.warmup
    assert PROMPT_LEN + W + K + W + K < cfg.seq_len

    rng = np.random.default_rng(42 + rank)
    prompt = rng.integers(0, cfg.vocab_size, size=PROMPT_LEN).astype(np.int32)
    # warm-up, overwritten by the timed pass: the whole prompt, so that the prompt buffers (grown on demand and kept by the
    # library) have their size before the timed pass, as for every prompt after a server's first
    m.prefill(prompt[:-1], 0)
    backend.synchronize()
    t0 = time.perf_counter()
    m.prefill(prompt[:-1], 0)
    prefill_s = time.perf_counter() - t0
    pos = PROMPT_LEN - 1
    tok = int(prompt[-1])

    def barrier():
        group.barrier()
        backend.synchronize()

    # ---- device-resident decode: W warm-up tokens, then K timed tokens ----
    warm = m.generate(tok, pos, W)
    tok, pos = int(warm[-1]), pos + W
    sampler = ClockSampler(local)
    barrier()
    backend.timer_start()
    toks = m.generate(tok, pos, K)
    ms = backend.timer_stop()
    barrier()
    clocks = sampler.stop()
    pos_first, pos_last = pos, pos + K - 1
    tok, pos = int(toks[-1]), pos + K

    # ---- end to end through the per-token call: token id H2D, logits + greedy id D2H (pinned), every step ----
    pinned = C.c_void_p()
    backend.check(backend.lib.slai_malloc_host(backend.h, cfg.vocab_size * 4, C.byref(pinned)))
    for _ in range(W):
        tok = m.decode_into(tok, pos, pinned.value)
        pos += 1
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = m.decode_into(tok, pos, pinned.value)
        pos += 1
    backend.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()

    ms, e2e_s = group.max_over_ranks([ms, e2e_s])
    batch = None
    if rank == 0 and world == 1 and not args.no_batch:
        try:
            batch = measure_batch(m, cfg, 8, PROMPT_LEN, 32, 3, ms / K)
        except Exception as e:  # the headline line is still reported
            batch = {"error": f"{type(e).__name__}: {e}"}
    algo, per, nl = time_dominant_kernel(backend, ctx, cfg, mats) if rank == 0 else (0, 1.0, 0)
    launches_per_token = m.launches_per_token()
    backend.lib.slai_free_host(backend.h, pinned)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        nthreads = os.cpu_count() or 1
        layer = CpuLayer(cfg, {name: qm.raw.to_numpy() for name, qm in raw.items()})  # the very bytes the GPU model holds
        tl, to = layer.times(PROMPT_LEN, nthreads, reps=2)
        tl1, to1 = layer.times(PROMPT_LEN, 1, reps=1)
        cpu = {"value": 1.0 / (cfg.n_layers * tl + to), "unit": "tok/s", "cores": nthreads, "kind": "port",
               "single_thread_value": 1.0 / (cfg.n_layers * tl1 + to1),
               "sample": "one full layer (f32-dequantised weights, 7 dense gemvs, attention over 513 positions) "
                         "+ the logits gemv of the same model on the host; token time = 32 x layer + logits"}
        del layer
    gemv_table = gemv_microbench(backend, ctx, peak) if (rank == 0 and args.gemv) else None
    # The 7B path does not shard; the path that does (the 70B configuration) is measured next, over the same ranks, and
    # attached to the line: one model split over the GPUs, strong scaling.
    del m, mats, raw
    tp_rec = None
    if not args.no_tp:
        try:
            tp_rec = measure_tp(args, group)
        except Exception as e:  # the headline line is still reported
            tp_rec = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0:
        value = world * K / (ms * 1e-3)
        e2e = world * K / e2e_s
        wbytes = cfg.weight_bytes_per_token(synth.FMT_Q4_K, synth.FMT_Q6_K)
        kv_mean = float(np.mean([cfg.kv_bytes_at(p) for p in range(pos_first, pos_last + 1)]))
        small = (2 * cfg.n_layers + 1) * cfg.dim * 4 + cfg.dim * 4
        token_bytes = wbytes + kv_mean + small
        line = {
            "metric": "decode tok/s bs1 (Llama-2-7B Q4_K)", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(world, K, W),
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 16, "d2h_bytes_per_step": cfg.vocab_size * 4 + 4},
            "prefill": prefill_record(cfg, PROMPT_LEN - 1, prefill_s, ms / K),
            "gpu_launches": launches_per_token * K,
            "launches_per_token": launches_per_token,
            "token_roofline": {"bytes_per_token": token_bytes, "roofline_tok_s": peak * 1e9 / token_bytes,
                               "frac": (value / world) / (peak * 1e9 / token_bytes), "peak_source": peak_src},
            "roofline": {"bound": "hbm", "kernel": "gemv_kernel<Q4_K, gate/up pair, rmsnorm, silu> 2 x 11008x4096: the decode step's dominant kernel "
                                                   "(all 32 layers' pairs in turn, 1.6 GB > L2)",
                         "achieved": algo / per / 1e9, "peak": peak, "unit": "GB/s", "frac": algo / per / 1e9 / peak,
                         "traffic": DOMINANT_KERNEL_DRAM_BYTES, "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of this "
                         "kernel on this shape (captured launches of slai_b200.microbench --pair); algorithmic bytes %d" % algo,
                         "launches_timed": nl, "us_per_launch": per * 1e6, "peak_source": peak_src},
        }
        if gemv_table is not None:
            line["gemv_microbench"] = gemv_table
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if batch is not None:
            line["batch8"] = batch
        if tp_rec is not None:
            line["tp"] = tp_rec
        emit(line)
    group.close()


if __name__ == "__main__":
    main()
