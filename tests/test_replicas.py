"""Host logic of the N>1 path (independent replicas), run as two `gloo` ranks on the CPU.

Each rank decodes its share of a set of independent sequences with the CPU oracle standing in for the device
model (the plumbing under test never looks at the model).  Checked: the shares partition the sequences, the
gathered results equal a single-process run, and the job's throughput is all ranks' tokens over the slowest rank's
time.
"""
import os
import socket
import sys

import numpy as np
import pytest

from slai_b200.replicas import ReplicaGroup, sequence_share

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sequence_share_partitions():
    for n in (0, 1, 2, 7, 8, 9, 64):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                s = sequence_share(n, r, world)
                seen.extend(s)
                assert abs(len(s) - n / world) < 1
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        sequence_share(4, 2, 2)


def test_single_process_group_is_identity():
    os.environ.pop("WORLD_SIZE", None)
    os.environ.pop("RANK", None)
    g = ReplicaGroup(backend="gloo")
    assert g.world == 1 and g.rank == 0
    assert g.max_over_ranks([1.5, 2.0]) == [1.5, 2.0]
    assert g.job_throughput(10, 2.0) == 5.0
    assert g.gather_ids([1, 2]) == [[1, 2]]
    g.barrier()
    g.close()


def _decode_sequences(seq_ids, n_new):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import oracle_llama
    from slai_b200 import synth
    from slai_b200.models import TINY_LLAMA, synthetic_llama_host
    cfg = TINY_LLAMA
    weights = synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=4)
    out = {}
    for s in seq_ids:
        m = oracle_llama(cfg, weights, synth.FMT_Q8_0, nthreads=1)
        tok, ids = 1 + s, []
        for pos in range(n_new):
            logits = m.forward(tok, pos)
            tok = int(np.argmax(logits))
            ids.append(tok)
        out[s] = ids
    return out


def _rank_main(rank, world, port, n_seq, n_new, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    g = ReplicaGroup(backend="gloo")
    mine = g.my_sequences(n_seq)
    res = _decode_sequences(mine, n_new)
    g.barrier()
    # synthetic, unequal times: the slowest rank must define the job's time
    seconds = 1.0 + rank
    tput = g.job_throughput(len(mine) * n_new, seconds)
    mx = g.max_over_ranks([seconds, 10.0 - rank])
    flat = [t for s in mine for t in res[s]]
    gathered = g.gather_ids(flat)
    q.put((rank, list(mine), tput, mx, gathered))
    g.close()


def test_two_gloo_ranks_decode_their_shares():
    import torch.multiprocessing as mp
    world, n_seq, n_new = 2, 3, 6
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, n_seq, n_new, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    got.sort()
    single = _decode_sequences(range(n_seq), n_new)
    assert got[0][1] == [0, 1] and got[1][1] == [2]
    for rank, mine, tput, mx, gathered in got:
        assert tput == pytest.approx(n_seq * n_new / 2.0)  # slowest rank took 2 s
        assert mx == [2.0, 10.0]
        flat_all = [t for r in range(world) for t in gathered[r]]
        assert flat_all == [t for s in range(n_seq) for t in single[s]]
