"""BERT encoder forward (post-LN, erf-GELU, bidirectional attention) against the golden fixture made
from transformers' BertModel on CPU (tests/golden/bert_tiny.npz) and against the torch oracle at a
larger random-init config with head dimension 64 (the single-kernel attention path). Bars: fp32
hidden states atol 1e-3 (the reference's CPU-comparison tolerance, python/tests/test_cpp_backend.py:
311-371); bf16 within 2e-2 relative of fp32."""
import os

import numpy as np
import pytest
import torch

from oracle import torch_ref

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _fixture():
    z = np.load(os.path.join(HERE, "golden", "bert_tiny.npz"))
    c = z["config"].tolist()
    cfg = dict(n_layer=c[0], n_head=c[1], n_embd=c[2], d_ff=c[3], vocab_size=c[4], n_positions=c[5], type_vocab=c[6], eps=1e-12)
    weights = {k[2:]: z[k] for k in z.files if k.startswith("w:")}
    return cfg, weights, z


def test_tiny_bert_hidden_states_match_reference_cpu_path(gpu_dev):
    cfg, weights, z = _fixture()
    model = gpu_dev.load_bert_state_dict(weights, cfg)
    got = gpu_dev.bert_forward(model, z["ids"], z["types"]).to_numpy()
    assert got.shape == z["hidden"].shape
    np.testing.assert_allclose(got, z["hidden"], atol=1e-3)
    assert np.max(np.abs(got - z["hidden"])) < 5e-5


def test_bert_layer_collapses_to_seven_kernels(gpu_dev):
    cfg, weights, z = _fixture()
    model = gpu_dev.load_bert_state_dict(weights, cfg)
    plan = gpu_dev.bert_forward(model, z["ids"], z["types"]).plan()
    names = [l.split("_f32")[0] for l in plan.strip().splitlines()]
    assert names.count("fused_attention[full,merge_heads]") == 2
    assert names.count("fused_linear[bias,]") == 2                 # stacked Q/K/V projection
    assert names.count("fused_linear[bias,gelu_exact,]") == 2      # intermediate + erf-GELU
    assert names.count("fused_linear[bias,residual,]") == 4        # both output projections with their residual
    assert names.count("layer_norm") == 1 + 2 * 2
    assert "add_bias" not in names and "gelu_exact" not in names


CFG_MID = dict(n_layer=2, n_head=4, n_embd=256, d_ff=1024, vocab_size=1009, n_positions=192, type_vocab=2, eps=1e-12)


def test_mid_bert_fp32_and_bf16_against_torch_oracle(gpu_dev):
    w = torch_ref.init_bert_weights(CFG_MID, seed=5)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, CFG_MID["vocab_size"], (3, 192))
    types = rng.integers(0, 2, (3, 192))
    with torch.no_grad():
        ref = torch_ref.bert_forward(w, CFG_MID, torch.from_numpy(ids), torch.from_numpy(types)).numpy()
    m32 = gpu_dev.init_bert_weights(CFG_MID, seed=5, dtype="float32")       # same generator, same order
    got32 = gpu_dev.bert_forward(m32, ids, types).to_numpy()
    np.testing.assert_allclose(got32, ref, atol=1e-3)
    m16 = gpu_dev.init_bert_weights(CFG_MID, seed=5, dtype="bfloat16")
    got16 = gpu_dev.bert_forward(m16, ids, types).to_numpy()
    scale = float(np.max(np.abs(ref)))
    assert np.max(np.abs(got16 - ref)) <= 2e-2 * scale
    # the taped forward: the recording call and two replays (the second on other ids) give the untaped results
    for _ in range(2):
        assert np.array_equal(gpu_dev.bert_forward(m16, ids, types, compiled=True).to_numpy(), got16)
    ids2 = rng.integers(0, CFG_MID["vocab_size"], (3, 192))
    assert np.array_equal(gpu_dev.bert_forward(m16, ids2, types, compiled=True).to_numpy(), gpu_dev.bert_forward(m16, ids2, types).to_numpy())
    assert len(m16["_tapes"]) == 1
    assert gpu_dev.pipeline_status() == 0


def test_bert_head_and_ff_shards_sum_to_the_full_layer(gpu_dev):
    """Tensor-parallel shards (column-parallel Q/K/V and intermediate, row-parallel output projections)
    computed one after the other on one device: summing the row-parallel partial outputs where a
    collective would reproduces the unsharded forward."""
    w = {k: v.numpy() for k, v in torch_ref.init_bert_weights(CFG_MID, seed=6).items()}
    rng = np.random.default_rng(6)
    for k in w:
        if k.endswith(".bias"):
            w[k] = (rng.standard_normal(w[k].shape) * 0.05).astype(np.float32)
    ids = rng.integers(0, CFG_MID["vocab_size"], (2, 64))
    full = gpu_dev.bert_forward(gpu_dev.load_bert_state_dict(w, CFG_MID), ids).to_numpy()
    world = 2
    shards = [gpu_dev.load_bert_state_dict(w, CFG_MID, head_range=(r * 2, r * 2 + 2), ff_range=(r * 512, r * 512 + 512)) for r in range(world)]
    # emulate the group on one device: run the ranks in lockstep through a generator-free trick —
    # rank 1's partial outputs are recomputed inside rank 0's all_reduce hook from rank 0's inputs.
    from applegpu_runtime_b200 import bert as B

    def forward_lockstep():
        gpu = gpu_dev
        cfg = shards[0]["config"]
        d, heads, dh = cfg["n_embd"], cfg["local_heads"], cfg["n_embd"] // cfg["n_head"]
        dl = heads * dh
        Bsz, T = ids.shape
        rows = Bsz * T
        tok = gpu.from_numpy(np.ascontiguousarray(ids.reshape(-1), dtype=np.int32))
        pos = gpu.from_numpy(np.tile(np.arange(T, dtype=np.int32), Bsz))
        typ = gpu.from_numpy(np.zeros(rows, np.int32))
        w0 = shards[0]["weights"]
        x = gpu.embedding(w0["embeddings.word_embeddings.weight"], tok) + gpu.embedding(w0["embeddings.position_embeddings.weight"], pos)
        x = x + gpu.embedding(w0["embeddings.token_type_embeddings.weight"], typ)
        x = gpu.layer_norm(x, w0["embeddings.LayerNorm.weight"], w0["embeddings.LayerNorm.bias"], 1e-12)
        for i in range(cfg["n_layer"]):
            p = f"encoder.layer.{i}"
            parts = []
            for sh in shards:
                ws = sh["weights"]
                qkv = B._linear(x, ws, f"{p}.qkv")
                sp = [gpu.transpose_dims(gpu.reshape(gpu.slice(qkv, dim=1, start=j * dl, end=(j + 1) * dl), [Bsz, T, heads, dh]), 1, 2) for j in range(3)]
                a = gpu.reshape(gpu.transpose_dims(gpu.attention(*sp), 1, 2), [rows, dl])
                parts.append(B._linear(a, ws, f"{p}.attention.output.dense"))
            x = gpu.layer_norm(x + (parts[0] + parts[1]), w0[f"{p}.attention.output.LayerNorm.weight"], w0[f"{p}.attention.output.LayerNorm.bias"], 1e-12)
            parts = []
            for sh in shards:
                ws = sh["weights"]
                parts.append(B._linear(gpu.gelu_exact(B._linear(x, ws, f"{p}.intermediate.dense")), ws, f"{p}.output.dense"))
            x = gpu.layer_norm(x + (parts[0] + parts[1]), w0[f"{p}.output.LayerNorm.weight"], w0[f"{p}.output.LayerNorm.bias"], 1e-12)
        return gpu.reshape(x, [Bsz, T, d]).to_numpy()

    np.testing.assert_allclose(forward_lockstep(), full, atol=2e-4)


def test_segment_taped_micro_batched_forward_equals_the_plain_forward(gpu_dev):
    """bert_forward_overlapped (the tensor-parallel driver: micro-batches in lock step, segments between all-reduces
    recorded on tapes and replayed) on a single rank, where the collective is the identity. The plain forward adds
    the residual in the projection's epilogue (one rounding); here the projection is rounded to bf16 first because the
    all-reduce sits between the two, so the results agree to bf16 rounding, not bit for bit; the replayed passes must
    reproduce the recording pass's arithmetic exactly."""
    from applegpu_runtime_b200.bert import bert_forward_overlapped
    from applegpu_runtime_b200.sharding import RankGroup
    from applegpu_runtime_b200.tp import TensorParallelGroup
    import torch  # noqa: F401
    from oracle import torch_ref
    cfg = dict(n_layer=3, n_head=4, n_embd=256, d_ff=1024, vocab_size=1003, n_positions=128, type_vocab=2, eps=1e-12)
    state = {k: v.numpy() for k, v in torch_ref.init_bert_weights(cfg, seed=5).items()}
    model = gpu_dev.load_bert_state_dict(state, cfg, dtype="bfloat16")
    tp = TensorParallelGroup(RankGroup())
    rng = np.random.default_rng(5)
    for trial in range(3):                      # trial 0 records the tapes, 1 and 2 replay them on other ids
        ids = rng.integers(0, cfg["vocab_size"], (6, 64))
        want = gpu_dev.bert_forward(model, ids).to_numpy()
        parts = bert_forward_overlapped(model, ids, tp, micro_batches=3)
        got = np.concatenate([p.to_numpy() for p in parts], axis=0)
        assert got.shape == want.shape
        assert float(np.max(np.abs(got - want))) <= 2e-2 * float(np.max(np.abs(want))), (trial, float(np.max(np.abs(got - want))))
        again = np.concatenate([p.to_numpy() for p in bert_forward_overlapped(model, ids, tp, micro_batches=3)], axis=0)
        assert np.array_equal(again, got), trial
    assert len(model["_segment_tapes"]) == 2 * cfg["n_layer"] + 1
    assert gpu_dev.pipeline_status() == 0
