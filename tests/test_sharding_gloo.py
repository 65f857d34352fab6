"""Host-side multi-rank logic on CPU: world_size-2 (and 3) gloo groups as child processes.

The data path has no collective (sequences are independent, weights replicated); what is covered here
is the bookkeeping every multi-GPU run relies on: the shard partition, the barrier + MAX-over-ranks
timing, the summed throughput and the gather of per-rank results.
"""
import os
import socket
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from applegpu_runtime_b200.sharding import RankGroup, shard_batch, shard_range, sharded_greedy_step  # noqa: E402


def test_shard_range_partitions_every_size():
    for n in (0, 1, 7, 8, 32, 256, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (lo0, hi0), (lo1, hi1) in zip(spans, spans[1:]):
                assert hi0 == lo1
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
            assert sizes == sorted(sizes, reverse=True)


def test_shard_range_rejects_bad_rank():
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
    with pytest.raises(ValueError):
        shard_range(8, -1, 2)


def test_shard_batch_axis():
    x = np.arange(8 * 5).reshape(8, 5)
    assert np.array_equal(np.concatenate([shard_batch(x, r, 4) for r in range(4)]), x)
    assert np.array_equal(np.concatenate([shard_batch(x, r, 2, axis=1) for r in range(2)], axis=1), x)


def test_single_process_group_is_identity():
    g = RankGroup()
    g.barrier()
    assert g.max(3.5) == 3.5 and g.sum(2.0) == 2.0
    rate, ms = g.throughput(8192, 4.0)
    assert ms == 4.0 and rate == pytest.approx(8192 / 4e-3)
    rows = np.arange(6, dtype=np.int32).reshape(3, 2)
    assert np.array_equal(g.gather_rows(rows, 3), rows)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _toy_last_logits(ids):
    """A deterministic stand-in for the forward: logits depend on the sequence's ids only, so the
    sharded result must equal the unsharded one whatever the partition."""
    rng_free = (ids.astype(np.int64).sum(axis=1, keepdims=True) * 7919 + np.arange(97)[None, :] * 104729) % 1009
    return rng_free.astype(np.float32)


def _worker(rank, world, port, n_seq, out_dir):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                       "LOCAL_RANK": str(rank)})
    g = RankGroup.from_env(backend="gloo")
    assert (g.rank, g.world) == (rank, world)
    g.barrier()
    # timing: the job's time is the slowest rank's; the job's units are the sum over ranks
    lo, hi = shard_range(n_seq, rank, world)
    rate, ms = g.throughput((hi - lo) * 1024, 2.0 + rank)
    ids = np.random.default_rng(0).integers(0, 50257, (n_seq, 16))
    nxt = sharded_greedy_step(_toy_last_logits, ids, g)
    g.barrier()
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), rate=rate, ms=ms, nxt=nxt, mx=g.max(rank), sm=g.sum(rank + 1))
    g.close()


@pytest.mark.parametrize("world,n_seq", [(2, 8), (2, 5), (3, 8)])
def test_gloo_ranks_agree(tmp_path, world, n_seq):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n_seq, str(tmp_path)), nprocs=world, join=True)
    ids = np.random.default_rng(0).integers(0, 50257, (n_seq, 16))
    want = np.argmax(_toy_last_logits(ids), axis=-1).astype(np.int32)
    for r in range(world):
        z = np.load(tmp_path / f"r{r}.npz")
        assert float(z["ms"]) == 2.0 + (world - 1)
        assert float(z["rate"]) == pytest.approx(n_seq * 1024 / ((2.0 + world - 1) / 1e3))
        assert float(z["mx"]) == world - 1 and float(z["sm"]) == world * (world + 1) / 2
        assert np.array_equal(z["nxt"], want)
