"""Tensor-parallel BERT on two GPUs (one process per GPU, NCCL all-reduce on the runtime stream) against
the unsharded forward on one GPU. Skipped on a single-GPU box; the shard arithmetic itself is covered
on CPU in tests/test_host_logic.py and tests/test_sharding_gloo.py."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(n_layer=2, n_head=4, n_embd=256, d_ff=1024, vocab_size=1009, n_positions=128, type_vocab=2, eps=1e-12)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _state(seed):
    import torch  # noqa: F401
    from oracle import torch_ref
    w = {k: v.numpy() for k, v in torch_ref.init_bert_weights(CFG, seed=seed).items()}
    rng = np.random.default_rng(seed)
    for k in w:
        if k.endswith(".bias"):
            w[k] = (rng.standard_normal(w[k].shape) * 0.05).astype(np.float32)
    return w


def _worker(rank, world, port, out_dir):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port)})
    import applegpu_runtime_b200 as gpu
    from applegpu_runtime_b200.sharding import RankGroup
    from applegpu_runtime_b200.tp import TensorParallelGroup, load_bert_shard
    gpu.init_backend()
    group = RankGroup.from_env()
    tp = TensorParallelGroup(group)
    state = _state(21)
    ids = np.random.default_rng(21).integers(0, CFG["vocab_size"], (4, 128))
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 2e-2)):
        shard = load_bert_shard(state, CFG, group, dtype=dtype)
        got = gpu.bert_forward(shard, ids, all_reduce=tp.all_reduce).to_numpy()
        # the same forward as micro-batches in lock step with the collectives on the communication stream
        from applegpu_runtime_b200.bert import bert_forward_overlapped
        lapped = np.concatenate([o.to_numpy() for o in bert_forward_overlapped(shard, ids, tp, micro_batches=2)], axis=0)
        assert lapped.shape == got.shape and float(np.max(np.abs(lapped - got))) <= (1e-5 if dtype == "float32" else 2e-2) * float(np.max(np.abs(got)))
        if rank == 0:
            full = gpu.bert_forward(gpu.load_bert_state_dict(state, CFG, dtype="float32"), ids).to_numpy()
            err = float(np.max(np.abs(got - full)) / np.max(np.abs(full)))
            with open(os.path.join(out_dir, f"{dtype}.txt"), "w") as f:
                f.write(f"{err} {tol}")
        group.barrier()
    assert gpu.pipeline_status() == 0
    group.close()


def test_two_rank_tensor_parallel_bert_matches_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for dtype in ("float32", "bfloat16"):
        err, tol = map(float, open(tmp_path / f"{dtype}.txt").read().split())
        assert err <= tol, (dtype, err)
