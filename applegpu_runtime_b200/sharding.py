"""Batch sharding over one process per GPU.

The reference is single-device and single-process (backend_cpp/applegpu_backend.cpp:1132-1134 reports
one device; python/applegpu_runtime/models/gpt2.py:47-91 has no batch dimension). Every op of the
forward path is independent across sequences and the weights are replicated, so the multi-GPU form
needs no exchange step: rank r of n owns sequences [r*B/n, (r+1)*B/n), results stay sharded, and the
only cross-rank traffic is host-side bookkeeping (a barrier around the timed region, a MAX over the
per-rank device times, an optional gather of the per-rank results). torch.distributed carries that
bookkeeping: NCCL when CUDA is present, gloo on CPU-only hosts.
"""
import os

import numpy as np


def shard_range(n_items, rank, world):
    """[lo, hi) of the items rank `rank` owns. Contiguous blocks; when `world` does not divide
    `n_items` the first `n_items % world` ranks hold one extra item (no rank differs by more than one)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(int(n_items), world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(array, rank, world, axis=0):
    """The slice of `array` (numpy, any rank) that `rank` owns along `axis`."""
    lo, hi = shard_range(array.shape[axis], rank, world)
    idx = [slice(None)] * array.ndim
    idx[axis] = slice(lo, hi)
    return array[tuple(idx)]


class RankGroup:
    """One process per GPU. `world == 1` (no launcher environment) is a no-op group."""

    def __init__(self, dist=None, rank=0, world=1):
        self.dist, self.rank, self.world = dist, rank, world

    @classmethod
    def from_env(cls, want_ranks=None, backend=None):
        """Join the group a launcher described in RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.
        Without those variables (or with want_ranks <= 1) the process is its own group."""
        if "RANK" not in os.environ or (want_ranks is not None and want_ranks <= 1):
            return cls()
        import torch
        import torch.distributed as dist
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        if not dist.is_initialized():
            dist.init_process_group(backend=backend, rank=rank, world_size=world)
        return cls(dist, rank, world)

    # ── bookkeeping collectives (host values only) ──
    def _device(self):
        return "cuda" if self.dist is not None and self.dist.get_backend() == "nccl" else "cpu"

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def _reduce(self, value, op_name):
        if self.dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self._device())
        self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, op_name))
        return float(t.item())

    def max(self, value):
        return self._reduce(value, "MAX")

    def sum(self, value):
        return self._reduce(value, "SUM")

    def gather_rows(self, local, n_total):
        """Concatenate per-rank int32/float32 row blocks (the shards of `shard_range`) on every rank.
        Used by tests and by callers that want the whole batch's next tokens in one place."""
        local = np.ascontiguousarray(local)
        if self.dist is None:
            return local
        import torch
        row_shape = local.shape[1:]
        sizes = [shard_range(n_total, r, self.world) for r in range(self.world)]
        longest = max(hi - lo for lo, hi in sizes)
        pad = np.zeros((longest,) + row_shape, local.dtype)
        pad[: local.shape[0]] = local
        mine = torch.from_numpy(pad).to(self._device())
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        self.dist.all_gather(parts, mine)
        return np.concatenate([p.cpu().numpy()[: hi - lo] for p, (lo, hi) in zip(parts, sizes)], axis=0)

    def throughput(self, units_local, ms_local):
        """Whole-job rate: the units every rank processed divided by the slowest rank's time."""
        total = self.sum(units_local)
        ms = self.max(ms_local)
        return total / (ms / 1e3), ms

    def close(self):
        if self.dist is not None and self.dist.is_initialized():
            self.dist.destroy_process_group()
        self.dist = None


def sharded_greedy_step(forward_last_logits, ids, group):
    """One data-parallel greedy step: each rank runs `forward_last_logits(ids_shard) -> [b, vocab]`
    on its own sequences and takes the row argmax (first maximum wins, as the reference's host
    np.argmax in models/generate.py:46-48 does); the shards are gathered so that every rank
    returns the next token of every sequence. No collective touches the data path itself."""
    lo, hi = shard_range(ids.shape[0], group.rank, group.world)
    if hi > lo:
        logits = np.asarray(forward_last_logits(ids[lo:hi]))
        nxt = np.argmax(logits, axis=-1).astype(np.int32).reshape(hi - lo, 1)
    else:
        nxt = np.zeros((0, 1), np.int32)
    return group.gather_rows(nxt, ids.shape[0]).reshape(-1)
