"""Replica plumbing for models that do not shard (Llama-2-7B, GPT-2 XL at batch 1).

One process per GPU, each holding a full copy of the model and decoding its own sequences; no collective on the
data path.  `torch.distributed` is used only to divide the sequences, to fence the timed region and to take the
slowest rank's time.  The backend is "nccl" on GPUs and "gloo" in the CPU tests; everything here is backend-neutral.
"""
from __future__ import annotations

import os


class ReplicaGroup:
    """Rank/world bookkeeping read from the torchrun environment (RANK, LOCAL_RANK, WORLD_SIZE, MASTER_*)."""

    def __init__(self, backend: str = "nccl", init: bool = True):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.backend = backend
        self.dist = None
        self._device = "cpu"
        if self.world > 1 and init:
            import torch
            import torch.distributed as dist
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                dist.init_process_group(backend="nccl", device_id=torch.device("cuda", self.local_rank))
                self._device = "cuda"
            else:
                dist.init_process_group(backend=backend)
            self.dist = dist

    # ---- dividing independent sequences ----
    def my_sequences(self, n_total: int) -> range:
        """Contiguous, balanced share of `n_total` independent sequences (the first `n_total % world` ranks get one more)."""
        return sequence_share(n_total, self.rank, self.world)

    # ---- fencing and timing ----
    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, values):
        """Element-wise maximum over ranks of a list of floats (the slowest rank defines the job's time)."""
        vals = [float(v) for v in values]
        if self.dist is None:
            return vals
        import torch
        t = torch.tensor(vals, device=self._device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.cpu()]

    def sum_over_ranks(self, values):
        vals = [float(v) for v in values]
        if self.dist is None:
            return vals
        import torch
        t = torch.tensor(vals, device=self._device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return [float(x) for x in t.cpu()]

    def job_throughput(self, units_this_rank: float, seconds_this_rank: float) -> float:
        """Whole-job throughput: units of all ranks divided by the slowest rank's time."""
        total = self.sum_over_ranks([units_this_rank])[0]
        slowest = self.max_over_ranks([seconds_this_rank])[0]
        return total / slowest

    def gather_ids(self, ids):
        """All ranks' generated token ids, as a list indexed by rank (rank 0 uses it to report; no data-path role)."""
        if self.dist is None:
            return [list(ids)]
        out = [None] * self.world
        self.dist.all_gather_object(out, list(int(i) for i in ids))
        return out

    def close(self) -> None:
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()
            self.dist = None


def sequence_share(n_total: int, rank: int, world: int) -> range:
    if n_total < 0 or world < 1 or not (0 <= rank < world):
        raise ValueError("bad share request")
    base, extra = divmod(n_total, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))
