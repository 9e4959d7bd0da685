"""Tensor-parallel Llama decode: one process per GPU, weights sharded Megatron-style, one sum per half-layer.

Partition (per layer; `t` = group size, rank `r`):
  column-parallel (rows split, whole heads):  wq rows [r*dim/t, ...), wk / wv rows [r*kv_dim/t, ...),
                                              w_gate / w_up rows [r*hidden/t, ...)
  row-parallel (K split on block boundaries): wo columns [r*dim/t, ...), w_down columns [r*hidden/t, ...)
  output matrix: rows [r*vocab/t, ...) when vocab/t is a multiple of 16 (each rank computes its slice of the logits,
                 one all-gather puts the whole vector on every rank), else replicated
  replicated: norm weights, embedding, the residual stream x.
Each rank keeps the KV cache of its own KV heads; attention needs no exchange.  After wo and after w_down the
partial `dim`-vectors are summed over the ranks (`slai_tp_all_reduce_sum`: NCCL over NVLink, inside the decode graph).
The host program's own communication layer (torch.distributed here; anything else works) is used only to hand
the 128-byte group id to the ranks.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import synth
from .models import LLAMA_MATRICES, Llama2, Llama2Config
from .ops import Backend, GpuQuantMatrix, GpuVector

TP_ID_BYTES = 128
TP_HANDLE_BYTES = 64
ROW_PARALLEL = ("wo", "w_down")


def check_divisible(config: Llama2Config, fmt: int, size: int) -> None:
    be = synth.BLOCK_ELEMS[fmt]
    if config.n_kv_heads % size or config.n_q_heads % size:
        raise ValueError(f"{config.n_q_heads}/{config.n_kv_heads} heads do not split over {size} ranks")
    if (config.hidden_dim // size) % max(be, 16) or config.hidden_dim % size:
        raise ValueError(f"hidden_dim {config.hidden_dim} / {size} is not a multiple of the block size {be}")
    if (config.dim // size) % be:
        raise ValueError(f"dim {config.dim} / {size} is not a multiple of the block size {be}")


def shard_shapes(config: Llama2Config, size: int) -> dict:
    """(rows, cols) of one rank's shard of every layer matrix."""
    d, kv, h = config.dim, config.kv_dim, config.hidden_dim
    return dict(wq=(d // size, d), wk=(kv // size, d), wv=(kv // size, d), wo=(d, d // size),
                w_gate=(h // size, d), w_up=(h // size, d), w_down=(d, h // size))


def shard_blocks(name: str, blocks: np.ndarray, fmt: int, rows: int, cols: int, rank: int, size: int) -> np.ndarray:
    """Rank `rank`'s part of a matrix given as GGUF blocks (row-major: rows x cols/block_elems blocks)."""
    bb, be = synth.BLOCK_BYTES[fmt], synth.BLOCK_ELEMS[fmt]
    a = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(rows, cols // be, bb)
    if name in ROW_PARALLEL:
        n = (cols // size) // be
        part = a[:, rank * n:(rank + 1) * n, :]
    else:
        n = rows // size
        part = a[rank * n:(rank + 1) * n]
    return np.ascontiguousarray(part).reshape(-1)


def output_rows(config: Llama2Config, size: int) -> int:
    """Rows of the output matrix one rank holds: vocab / size when that is a whole number of 16-row tiles, else all."""
    return config.vocab_size // size if config.vocab_size % (16 * size) == 0 else config.vocab_size


def shard_llama_host(config: Llama2Config, weights: dict, fmt: int, rank: int, size: int, out_fmt: int | None = None) -> dict:
    """The weights dict of `synthetic_llama_host`, reduced to rank `rank`'s shards."""
    check_divisible(config, fmt, size)
    out_fmt = fmt if out_fmt is None else out_fmt
    full = config.matrix_shapes()
    out = {}
    for (name, l), val in weights.items():
        if name in LLAMA_MATRICES:
            r, c = full[name]
            out[(name, l)] = shard_blocks(name, val, fmt, r, c, rank, size)
        elif name == "output" and output_rows(config, size) != config.vocab_size:
            out[(name, l)] = shard_blocks(name, val, out_fmt, config.vocab_size, config.dim, rank, size)
        else:
            out[(name, l)] = val
    return out


def join_group(backend: Backend, rank: int, size: int, broadcast) -> None:
    """Collective.  `broadcast(obj_or_None)` returns rank 0's object on every rank (e.g. built on
    torch.distributed.broadcast_object_list)."""
    ident = None
    if rank == 0:
        buf = (C.c_ubyte * TP_ID_BYTES)()
        backend.check(backend.lib.slai_tp_unique_id(backend.h, buf))
        ident = bytes(buf)
    ident = broadcast(ident)
    buf = (C.c_ubyte * TP_ID_BYTES).from_buffer_copy(ident)
    backend.check(backend.lib.slai_tp_init(backend.h, buf, rank, size))


def enable_peer_exchange(backend: Backend, size: int, all_gather, barrier) -> None:
    """Collective.  Maps every rank's exchange region into every other rank (CUDA IPC over NVLink peer access): the
    per-half-layer sums then need no collective kernel.  `all_gather(obj)` returns the list of all ranks' objects in
    rank order; `barrier()` returns when every rank has called it.

    The kernels wait a bounded time (about a second) for a peer's partial sums, then raise the context's error flag:
    call a host barrier after loading the weights, before the first decode step, so that the ranks start together."""
    buf = (C.c_ubyte * TP_HANDLE_BYTES)()
    backend.check(backend.lib.slai_tp_peer_export(backend.h, buf))
    handles = all_gather(bytes(buf))
    blob = b"".join(handles)
    assert len(blob) == size * TP_HANDLE_BYTES
    backend.check(backend.lib.slai_tp_peer_attach(backend.h, (C.c_ubyte * len(blob)).from_buffer_copy(blob)))
    barrier()


def torch_all_gather(obj):
    import torch.distributed as dist
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def torch_barrier():
    import torch.distributed as dist
    dist.barrier()


def torch_broadcast(obj):
    import torch.distributed as dist
    box = [obj]
    dist.broadcast_object_list(box, src=0)
    return box[0]


def all_reduce_sum(backend: Backend, vec: GpuVector) -> None:
    backend.check(backend.lib.slai_tp_all_reduce_sum(backend.h, C.c_void_p(vec.ptr), C.c_void_p(vec.ptr), vec.n))


def llama_from_host_tp(backend: Backend, config: Llama2Config, weights: dict, fmt: int, out_fmt: int | None, rank: int, size: int) -> Llama2:
    """Sharded model from the full host weights (every rank holds the same dict and takes its part)."""
    out_fmt = fmt if out_fmt is None else out_fmt
    m = Llama2(backend, config, rank, size)
    shapes = shard_shapes(config, size)
    for (name, l), val in shard_llama_host(config, weights, fmt, rank, size, out_fmt).items():
        if name in LLAMA_MATRICES:
            r, c = shapes[name]
            m.set_matrix(name, l, GpuQuantMatrix(backend, fmt, r, c, val))
        elif name == "output":
            m.set_matrix(name, -1, GpuQuantMatrix(backend, out_fmt, output_rows(config, size), config.dim, val))
        else:
            m.set_f32(name, l, val)
    return m


def synthetic_llama_device_tp(backend: Backend, config: Llama2Config, fmt: int, out_fmt: int, rank: int, size: int, seed: int = 0,
                              std: float = 0.02) -> Llama2:
    """Benchmark-sized sharded model generated on the device.  Shards of different ranks are seeded independently
    (they are not slices of one global random matrix; throughput does not depend on that); everything replicated
    (embedding, norms) is seeded identically on all ranks, and every rank sees the gathered logits, so that the ranks
    decode the same tokens."""
    check_divisible(config, fmt, size)
    m = Llama2(backend, config, rank, size)
    sid = seed * 1_000_003
    for l in range(config.n_layers):
        for i, (name, (r, c)) in enumerate(shard_shapes(config, size).items()):
            m.set_matrix(name, l, GpuQuantMatrix.synthetic(backend, fmt, r, c, sid + 100_000 * (rank + 1) + 100 * l + i + 1, std))
        ones = np.ones(config.dim, dtype=np.float32)
        m.set_f32("attn_norm", l, ones)
        m.set_f32("ffn_norm", l, ones)
    emb = GpuVector(backend, config.vocab_size * config.dim)
    backend.check(backend.lib.slai_synth_normal_f32(backend.h, C.c_void_p(emb.ptr), emb.n, sid + 7_000_001, std))
    m.set_f32("token_embd", -1, emb)
    del emb
    m.set_f32("out_norm", -1, np.ones(config.dim, dtype=np.float32))
    vr = output_rows(config, size)
    m.set_matrix("output", -1, GpuQuantMatrix.synthetic(backend, out_fmt, vr, config.dim,
                                                        sid + 7_000_002 + (100_000 * (rank + 1) if vr != config.vocab_size else 0), std))
    return m


def bytes_per_token_per_rank(config: Llama2Config, fmt: int, out_fmt: int, size: int) -> int:
    """Packed weight bytes one rank streams per decoded token: its shard of every layer and of the output matrix."""
    per = sum(r * c for r, c in shard_shapes(config, size).values())
    return int(config.n_layers * per * synth.BITS_PER_WEIGHT[fmt] / 8 + output_rows(config, size) * config.dim * synth.BITS_PER_WEIGHT[out_fmt] / 8)
