"""Tensor-parallel decode.

CPU part (two `gloo` ranks): the sharding itself.  Each rank takes its shards with the product's own functions
(`slai_b200.tp.shard_llama_host`), runs the layer arithmetic on them with the oracle's operators, sums the two
exchange points over the ranks, and must reproduce the unsharded oracle model's logits.

GPU part (needs two GPUs; skipped otherwise): two processes, one context each, join a group through the C ABI and
decode with sharded weights; logits equal the oracle's within 1e-3 and are identical on both ranks.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _cfg():
    from slai_b200.models import Llama2Config
    from slai_b200 import _lib
    return Llama2Config(dim=512, hidden_dim=1024, n_layers=2, n_q_heads=8, n_kv_heads=4, vocab_size=640, seq_len=48, kv_dtype=_lib.KV_F32)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ---------------------------------------------------------------------------------------------------------------
# CPU: sharding arithmetic
# ---------------------------------------------------------------------------------------------------------------
class ShardedOracle:
    """One rank of a tensor-parallel Llama on the CPU, built from the oracle's operators."""

    def __init__(self, cfg, weights, fmt, rank, size, all_reduce, all_gather):
        from oracle import oracle as O
        from slai_b200 import tp
        self.O, self.cfg, self.size, self.all_reduce, self.all_gather = O, cfg, size, all_reduce, all_gather
        self.out_rows = tp.output_rows(cfg, size)
        shapes = tp.shard_shapes(cfg, size)
        sh = tp.shard_llama_host(cfg, weights, fmt, rank, size)
        self.w = {}
        for (name, l), val in sh.items():
            if name in shapes:
                self.w[(name, l)] = O.dequantize(fmt, val).reshape(shapes[name])
            elif name == "output":
                self.w[(name, l)] = O.dequantize(fmt, val).reshape(self.out_rows, cfg.dim)
            else:
                self.w[(name, l)] = np.asarray(val, dtype=np.float32)
        self.hs = cfg.head_size
        self.kv_local = cfg.kv_dim // size
        self.nq_local = cfg.n_q_heads // size
        self.kc = np.zeros((cfg.n_layers, cfg.seq_len, self.kv_local), dtype=np.float32)
        self.vc = np.zeros_like(self.kc)

    def forward(self, token, pos):
        O, c, w = self.O, self.cfg, self.w
        x = w[("token_embd", -1)].reshape(c.vocab_size, c.dim)[token].copy()
        for l in range(c.n_layers):
            xb = O.rms_norm(x, w[("attn_norm", l)], c.rms_norm_eps)
            q = O.gemv_f32(w[("wq", l)], xb)
            k = O.gemv_f32(w[("wk", l)], xb)
            v = O.gemv_f32(w[("wv", l)], xb)
            q, k = O.rope(q, k, self.hs, self.kv_local, pos, c.rope_base_freq)
            self.kc[l, pos], self.vc[l, pos] = k, v
            att, _ = O.attention(q, self.kc[l], self.vc[l], seq_len=c.seq_len, kv_dim=self.kv_local, kv_mul=c.n_q_heads // c.n_kv_heads,
                                 n_heads=self.nq_local, head_size=self.hs, pos=pos)
            x = x + self.all_reduce(O.gemv_f32(w[("wo", l)], att))          # exchange 1
            xb = O.rms_norm(x, w[("ffn_norm", l)], c.rms_norm_eps)
            hb = O.silu_gate(O.gemv_f32(w[("w_gate", l)], xb), O.gemv_f32(w[("w_up", l)], xb))
            x = x + self.all_reduce(O.gemv_f32(w[("w_down", l)], hb))       # exchange 2
        part = O.gemv_f32(w[("output", -1)], O.rms_norm(x, w[("out_norm", -1)], c.rms_norm_eps))
        return self.all_gather(part) if self.out_rows != c.vocab_size else part   # each rank holds vocab / size rows


def _cpu_rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    from slai_b200 import synth
    from slai_b200.models import synthetic_llama_host
    dist.init_process_group(backend="gloo")
    cfg = _cfg()
    weights = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=11, std=0.05, embd_std=1.0)

    def all_reduce(v):
        t = torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32).copy())
        dist.all_reduce(t)
        return t.numpy()

    def all_gather(v):
        parts = [torch.zeros(v.size, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32).copy()))
        return torch.cat(parts).numpy()

    m = ShardedOracle(cfg, weights, synth.FMT_Q4_K, rank, world, all_reduce, all_gather)
    outs = [m.forward(tok, pos) for pos, tok in enumerate([3, 17, 599, 42])]
    q.put((rank, np.stack(outs)))
    dist.barrier()
    dist.destroy_process_group()


def test_sharding_reproduces_the_unsharded_model_two_gloo_ranks():
    import torch.multiprocessing as mp
    from helpers import oracle_llama, rel_l2
    from slai_b200 import synth
    from slai_b200.models import synthetic_llama_host
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cpu_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cfg = _cfg()
    weights = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=11, std=0.05, embd_std=1.0)
    ref = oracle_llama(cfg, weights, synth.FMT_Q4_K, nthreads=2)
    want = np.stack([ref.forward(tok, pos) for pos, tok in enumerate([3, 17, 599, 42])])
    assert np.array_equal(got[0], got[1])              # the exchange leaves every rank with the same residual stream
    assert rel_l2(got[0], want) < 1e-5                 # summation order differs from the unsharded dot products only


def test_shard_shapes_and_divisibility():
    from slai_b200 import synth, tp
    from slai_b200.models import LLAMA2_70B, LLAMA2_7B
    for size in (2, 4, 8):
        tp.check_divisible(LLAMA2_70B, synth.FMT_Q4_K, size)
        sh = tp.shard_shapes(LLAMA2_70B, size)
        assert sh["wo"] == (8192, 8192 // size) and sh["w_down"] == (8192, 28672 // size) and sh["wk"] == (1024 // size, 8192)
        full = LLAMA2_70B.weight_bytes_per_token(synth.FMT_Q4_K, synth.FMT_Q6_K)
        per = tp.bytes_per_token_per_rank(LLAMA2_70B, synth.FMT_Q4_K, synth.FMT_Q6_K, size)
        assert tp.output_rows(LLAMA2_70B, size) == 32000 // size
        assert abs(per * size - full) < 1e-6 * full   # everything is sharded: the ranks' bytes add up to the model's
    with pytest.raises(ValueError):
        tp.check_divisible(LLAMA2_7B, synth.FMT_Q4_K, 8)  # 11008 / 8 = 1376 is not a multiple of 256
    rng = np.random.default_rng(0)
    blocks = synth.random_blocks(synth.FMT_Q8_0, 8, 128, rng)
    cols = tp.shard_blocks("wo", blocks, synth.FMT_Q8_0, 8, 128, 1, 2).reshape(8, 2, 34)
    assert np.array_equal(cols, blocks.reshape(8, 4, 34)[:, 2:4])
    rows = tp.shard_blocks("wq", blocks, synth.FMT_Q8_0, 8, 128, 1, 2).reshape(4, 4, 34)
    assert np.array_equal(rows, blocks.reshape(8, 4, 34)[4:])


# ---------------------------------------------------------------------------------------------------------------
# GPU: two ranks through the C ABI
# ---------------------------------------------------------------------------------------------------------------
def _gpu_rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from slai_b200 import synth, tp
    from slai_b200.models import synthetic_llama_host
    from slai_b200.ops import Backend
    dist.init_process_group(backend="gloo")  # host plumbing only: hands the group id around
    backend = Backend(rank)
    tp.join_group(backend, rank, world, tp.torch_broadcast)
    # the exchange operator on its own
    v = backend.vector(np.full(1000, rank + 1.0, dtype=np.float32))
    tp.all_reduce_sum(backend, v)
    s = v.to_numpy()
    cfg = _cfg()
    weights = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=11, std=0.05, embd_std=1.0)

    def run(m):
        outs, toks = [], []
        tok = 3
        for pos in range(8):
            lg, nxt = m.forward_logits(pos, tok)
            outs.append(lg.copy())
            toks.append(nxt)
            tok = [17, 599, 42, 5, 6, 7, 8, 9][pos]
        gen = m.generate(tok, 8, 24)
        backend.synchronize()  # raises if a bounded wait on a peer ran out
        return np.stack(outs), toks, list(gen), m.launches_per_token()

    # 1. the exchange as an NCCL all-reduce between the kernels
    m = tp.llama_from_host_tp(backend, cfg, weights, synth.FMT_Q4_K, None, rank, world)
    assert tp.output_rows(cfg, world) == cfg.vocab_size // world   # the logits matrix is sharded too
    tp.torch_barrier()   # the ranks start the first step together (peer polls are bounded)
    nccl = run(m)
    m.close()
    # 2. the exchange over peer memory, inside the GEMV kernels (same sums in the same order: identical bits)
    tp.enable_peer_exchange(backend, world, tp.torch_all_gather, tp.torch_barrier)
    m = tp.llama_from_host_tp(backend, cfg, weights, synth.FMT_Q4_K, None, rank, world)
    tp.torch_barrier()
    peer = run(m)
    # 3. a 20-token prompt through the tensor-core prompt pass on the shards (partial products summed with the group's
    #    all-reduce), then decoding continues on the peer exchange
    m3 = tp.llama_from_host_tp(backend, cfg, weights, synth.FMT_Q4_K, None, rank, world)
    tp.torch_barrier()
    prompt = np.random.default_rng(9).integers(0, cfg.vocab_size, size=20).astype(np.int32)
    pf_logits = m3.prefill(prompt, 0, want_logits=True)
    pf_gen = list(m3.generate(int(np.argmax(pf_logits)), 20, 12))
    backend.synchronize()
    dist.barrier()
    m3.close()
    q.put((rank, s, nccl[0], nccl[1], nccl[2], nccl[3], peer[0], peer[2], peer[3], pf_logits, pf_gen))
    dist.barrier()
    m.close()
    backend.check(backend.lib.slai_tp_shutdown(backend.h))
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_tensor_parallel_llama_matches_oracle():
    from slai_b200 import _lib
    lib = _lib.load()
    if lib.slai_device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from helpers import oracle_llama, rel_l2
    from oracle import oracle as O
    from slai_b200 import synth
    from slai_b200.models import synthetic_llama_host
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gpu_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=600) for _ in range(2))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg = _cfg()
    weights = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=11, std=0.05, embd_std=1.0)
    ref = oracle_llama(cfg, weights, synth.FMT_Q4_K, nthreads=4)
    tok = 3
    for pos in range(8):
        want = ref.forward(tok, pos)
        for r in range(2):
            assert rel_l2(got[r][2][pos], want) < 1e-3, (r, pos)
            assert got[r][3][pos] == int(np.argmax(got[r][2][pos]))
        tok = [17, 599, 42, 5, 6, 7, 8, 9][pos]
    assert np.array_equal(got[0][2], got[1][2])       # bitwise: both ranks hold the same residual stream
    assert got[0][4] == got[1][4]                     # and generate the same tokens
    assert np.allclose(got[0][1], 3.0) and np.allclose(got[1][1], 3.0)
    assert got[0][5] == 3 + cfg.n_layers * 7 + 1 + 1  # embed + (5 kernels + 2 exchanges) per layer + logits + gather + argmax + advance
    for r in range(2):                                # peer-memory exchange: no collective launches, identical results
        assert np.array_equal(got[r][6], got[r][2])
        assert got[r][7] == got[r][4]
        assert got[r][8] == 3 + cfg.n_layers * 5 + 1 + 1 + 1   # + the token tick, + the logits gather
    # sharded prompt pass: last logits against the oracle fed token by token, same continuation on both ranks
    ref2 = oracle_llama(cfg, weights, synth.FMT_Q4_K, nthreads=4)
    prompt = np.random.default_rng(9).integers(0, cfg.vocab_size, size=20).astype(np.int32)
    for pos, t in enumerate(prompt):
        want = ref2.forward(int(t), pos)
    for r in range(2):
        assert rel_l2(got[r][9], want) < 1e-3, r
    assert np.array_equal(got[0][9], got[1][9]) and got[0][10] == got[1][10]
    tok, want_gen = int(np.argmax(want)), []
    for i in range(12):
        rl = ref2.forward(tok, 20 + i)
        tok = O.argmax(rl)
        want_gen.append(tok)
    assert sum(1 for a, b in zip(got[0][10], want_gen) if a == b) >= 10, (got[0][10], want_gen)
