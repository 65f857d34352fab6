"""Host-side logic that needs no kernel launch: ids, shapes, dtype validation, error strings,
deferred frees, the fusion pass and its launch plan. Restates the host-only unit tests of the
reference (graph.rs:669-829, fusion.rs:291-483, ops.rs:2871-2998, tensor.rs:445-780) against
the C ABI. Runs in metadata-only mode when no GPU is present."""
import ctypes

import numpy as np
import pytest


def test_ids_are_monotonic_and_op_ids_start_at_100000(gpu):
    a = gpu.tensor([1.0, 2.0], shape=[2])
    b = gpu.tensor([1.0, 2.0], shape=[2])
    assert 0 < a.id < b.id < 100000          # tensor.rs:292-297
    c = a + b
    assert c.id >= 100000                    # ops.rs:165
    d = a + b
    assert d.id == c.id + 1 or d.id > c.id


def test_shape_and_dtype_queries(gpu):
    x = gpu.from_numpy(np.zeros((2, 3, 4), np.float32))
    assert x.shape == [2, 3, 4] and x.dtype == "float32"
    i = gpu.from_numpy(np.zeros((5,), np.int32))
    assert i.dtype == "int32"
    h = gpu.from_numpy(np.zeros((5,), np.float16))
    assert h.dtype == "float16"
    assert gpu.dtype_size("bfloat16") == 2 and gpu.dtype_size("int64") == 8


def test_matmul_shape_rules_and_errors(gpu):
    a = gpu.from_numpy(np.zeros((4, 2, 3), np.float32))
    b = gpu.from_numpy(np.zeros((3, 5), np.float32))
    assert (a @ b).shape == [4, 2, 5]                                   # broadcast batch (ops.rs:434-448)
    c = gpu.from_numpy(np.zeros((2, 1, 3, 5), np.float32))
    assert (a @ c).shape == [2, 4, 2, 5]
    with pytest.raises(ValueError, match=r"matmul inner dimensions mismatch: A\[\.\.\.,2,3\] \* B\[\.\.\.,5,3\]"):
        a @ gpu.from_numpy(np.zeros((5, 3), np.float32))
    with pytest.raises(ValueError, match="matmul requires at least 2D tensors"):
        gpu.from_numpy(np.zeros((3,), np.float32)) @ b
    with pytest.raises(ValueError, match="Dtype mismatch: Float32 vs Float16"):
        a @ gpu.from_numpy(np.zeros((3, 5), np.float16))
    with pytest.raises(ValueError, match="Matmul requires a float dtype, got int32"):
        gpu.from_numpy(np.zeros((2, 2), np.int32)) @ gpu.from_numpy(np.zeros((2, 2), np.int32))


def test_broadcast_rules(gpu):
    a = gpu.from_numpy(np.zeros((4, 1, 3), np.float32))
    b = gpu.from_numpy(np.zeros((5, 3), np.float32))
    assert (a + b).shape == [4, 5, 3]
    with pytest.raises(ValueError, match="Cannot broadcast shapes"):
        a + gpu.from_numpy(np.zeros((2, 2), np.float32))


def test_transformer_op_validation_messages(gpu):
    x = gpu.from_numpy(np.zeros((2, 4), np.float32))
    g3 = gpu.from_numpy(np.zeros((3,), np.float32))
    g4 = gpu.from_numpy(np.zeros((4,), np.float32))
    with pytest.raises(ValueError, match=r"gamma shape \[3\] must be \[4\]"):
        gpu.layer_norm(x, g3, g4)
    with pytest.raises(ValueError, match=r"beta shape \[3\] must be \[4\]"):
        gpu.layer_norm(x, g4, g3)
    w = gpu.from_numpy(np.zeros((5, 3), np.float32))
    with pytest.raises(ValueError, match="embedding indices must be Int32, got Float32"):
        gpu.embedding(w, gpu.from_numpy(np.zeros((2,), np.float32)))        # test_transformer_ops.py:139-144
    with pytest.raises(ValueError, match="embedding weights must be 2D"):
        gpu.embedding(g4, gpu.from_numpy(np.zeros((2,), np.int32)))
    idx = gpu.from_numpy(np.zeros((2, 3), np.int32))
    assert gpu.embedding(w, idx).shape == [2, 3, 3]                           # idx.shape + [D]
    with pytest.raises(ValueError, match=r"add_bias requires >= 2D input, got \[4\]"):
        gpu.add_bias(g4, g4)                                                  # ops.rs:3098-3111
    with pytest.raises(ValueError, match="add_bias bias length 3 != input dim 1 4"):
        gpu.add_bias(x, g3)
    with pytest.raises(ValueError, match="softmax_causal requires at least 2D tensor"):
        gpu.softmax_causal(g4)
    assert gpu.argmax(x).shape == [2] and gpu.argmax(x).dtype == "int32"
    assert gpu.argmax(g4).shape == [1]                                        # ops.rs:1400-1401
    with pytest.raises(ValueError, match="gather indices must be Int32"):
        gpu.gather(x, 1, gpu.from_numpy(np.zeros((2, 2), np.float32)))
    with pytest.raises(ValueError, match="gather currently supports only 2D tensors"):
        gpu.gather(g4, 0, gpu.from_numpy(np.zeros((2, 2), np.int32)))
    with pytest.raises(ValueError, match="index_select index must be 1D"):
        gpu.index_select(x, 0, gpu.from_numpy(np.zeros((2, 2), np.int32)))
    with pytest.raises(ValueError, match="Quantize scale must be non-zero"):
        gpu.quantize(x, "int8", scale=0.0)
    with pytest.raises(ValueError, match="Quantize target must be Int8 or UInt8"):
        gpu.quantize(x, "int32", scale=0.1)
    with pytest.raises(ValueError, match="Dequantize input must be Int8 or UInt8"):
        gpu.dequantize(x, "float32", scale=0.1)
    with pytest.raises(ValueError, match="Float64 is not supported"):
        gpu.from_numpy(np.zeros((2,), np.float64)) + gpu.from_numpy(np.zeros((2,), np.float64))


def test_layout_ops_shapes(gpu):
    x = gpu.from_numpy(np.zeros((6, 8), np.float32))
    assert gpu.slice(x, 1, 2, 5).shape == [6, 3]
    assert gpu.reshape(x, [2, 3, 8]).shape == [2, 3, 8]
    assert gpu.transpose(x).shape == [8, 6]
    assert gpu.transpose_dims(gpu.reshape(x, [2, 3, 8]), 0, 1).shape == [3, 2, 8]
    assert gpu.transpose_dims(x, 1, 1) is x                                   # no-op returns its input (ops.rs:522-524)
    assert gpu.concat(x, x, dim=0).shape == [12, 8]
    assert gpu.cast(x, "float32") is x                                        # ops.rs:2304-2307
    assert gpu.cast(x, "float16").dtype == "float16"
    with pytest.raises(ValueError, match=r"Cannot reshape: old shape \[6, 8\] has 48 elements, new shape \[5, 5\] has 25"):
        gpu.reshape(x, [5, 5])
    with pytest.raises(ValueError, match=r"slice end 9 > shape\[1\] = 8"):
        gpu.slice(x, 1, 0, 9)
    with pytest.raises(ValueError, match="slice start 3 >= end 3"):
        gpu.slice(x, 0, 3, 3)
    with pytest.raises(ValueError, match="concat shape mismatch on dim 1"):
        gpu.concat(x, gpu.from_numpy(np.zeros((6, 7), np.float32)), dim=0)
    with pytest.raises(ValueError, match="out of range for 2D tensor"):
        gpu.transpose_dims(x, 0, 2)


def test_attention_validation(gpu):
    q = gpu.from_numpy(np.zeros((2, 4, 8), np.float32))
    k = gpu.from_numpy(np.zeros((2, 6, 8), np.float32))
    v = gpu.from_numpy(np.zeros((2, 6, 5), np.float32))
    assert gpu.attention(q, k, v).shape == [2, 4, 5]
    assert gpu.attention_causal(q, k, v).shape == [2, 4, 5]
    with pytest.raises(ValueError, match="Q and K must have same d_k: 8 vs 5"):
        gpu.attention(q, v, v)
    with pytest.raises(ValueError, match="K and V must have same kv_len: 6 vs 4"):
        gpu.attention(q, k, gpu.from_numpy(np.zeros((2, 4, 5), np.float32)))


# ── fusion pass (fusion.rs:291-483, fusion_integration.rs:6-104, python/tests/test_fusion.py) ──
def test_elementwise_chain_add_relu_fuses_into_one_kernel(gpu):
    a = gpu.tensor([1.0, -2.0, 3.0, -4.0], shape=[4]); b = gpu.tensor([0.5, 0.5, 0.5, 0.5], shape=[4])
    y = (a + b).relu()
    plan = y.plan().strip().splitlines()
    assert len(plan) == 1 and plan[0].startswith("fused_") and "max((in0 + in1), 0.0f)" in plan[0]


def test_elementwise_chain_of_three_unaries(gpu):
    a = gpu.tensor([1.0, 4.0, 9.0], shape=[3])
    y = a.sqrt().__neg__().relu()
    plan = y.plan().strip().splitlines()
    assert len(plan) == 1 and "max((-sqrt(in0)), 0.0f)" in plan[0]


def test_chain_stops_at_a_node_with_two_consumers(gpu):
    a = gpu.tensor([1.0, 2.0], shape=[2]); b = gpu.tensor([1.0, 2.0], shape=[2])
    s = a + b               # consumed twice below: must stay its own kernel (ref_count != 1)
    y = s.relu() + s.exp()
    plan = y.plan().strip().splitlines()
    assert plan[0].startswith("elementwise_add")
    assert len(plan) >= 3


def test_single_elementwise_op_is_not_fused(gpu):
    a = gpu.tensor([1.0, 2.0], shape=[2])
    assert a.relu().plan().strip() == "elementwise_relu_f32 [2]"


def test_non_fusible_ops_break_chains(gpu):
    # GeluExact, ScalarMul and AddBias are not in the fusible set (graph.rs:273-280)
    a = gpu.tensor([1.0, 2.0], shape=[2])
    plan = gpu.gelu_exact(a.relu()).plan().strip().splitlines()
    assert [p.split("_f32")[0] for p in plan] == ["elementwise_relu", "gelu_exact"]


def _tiny_model(gpu):
    cfg = {"n_layer": 2, "n_head": 4, "n_embd": 64, "vocab_size": 100, "n_positions": 32}
    return gpu.init_gpt2_weights(cfg, seed=0)


def test_reference_chain_rule_never_fires_on_the_gpt2_graph(gpu):
    # every element-wise op of gpt2_forward sits alone between non-fusible ops, so the upstream
    # rule finds no chain of length 2
    gpu.set_fusion(elementwise_chains=True, patterns=False)
    try:
        logits, _ = gpu.gpt2_forward(_tiny_model(gpu), np.arange(16).reshape(2, 8))
        plan = logits.plan()
    finally:
        gpu.set_fusion(True, True)
    assert "fused_" not in plan
    names = [l.split("_f32")[0] for l in plan.strip().splitlines()]
    assert names.count("matmul") == 2 * (4 + 2) + 1          # 4 linears + QK^T + PV per layer, + LM head
    assert names.count("add_bias") == 8 and names.count("gelu") == 2 and names.count("softmax_causal") == 2


def test_graph_rewrites_collapse_the_gpt2_layer(gpu):
    logits, _ = gpu.gpt2_forward(_tiny_model(gpu), np.arange(16).reshape(2, 8))
    assert logits.shape == [2, 8, 100]
    names = [l.split("_f32")[0] for l in logits.plan().strip().splitlines()]
    assert names[0] == "fused_embed_add"
    assert names.count("fused_attention[causal,merge_heads]") == 2   # writes [B, T, h*d] directly: no head-merge copy
    assert names.count("fused_linear[bias,]") == 2                 # QKV projections
    assert names.count("fused_linear[bias,gelu,]") == 2            # FC1 + GELU
    assert names.count("fused_linear[bias,residual,]") == 4        # attention out-proj and FC2, with the residual add
    assert "add_bias" not in names and "gelu" not in names and "elementwise_add" not in names
    assert names.count("layer_norm") == 5
    compute = [n for n in names if n.split("[")[0] not in ("slice_dim1", "reshape", "transpose")]
    assert len(compute) == 1 + 2 * 7 + 2   # embed, 7 per layer, final LN, LM head


def test_kv_cache_step_uses_full_attention(gpu):
    m = _tiny_model(gpu)
    ids = np.arange(10).reshape(2, 5)
    logits, kv = gpu.gpt2_forward(m, ids)
    assert len(kv) == 2 and kv[0][0].shape == [2, 4, 5, 16]
    ids2 = np.concatenate([ids, np.zeros((2, 1), np.int64)], axis=1)
    logits2, kv2 = gpu.gpt2_forward(m, ids2, kv_cache=kv, last_only=True)
    assert logits2.shape == [2, 100] and kv2[0][0].shape == [2, 4, 6, 16]
    names = [l.split("_f32")[0] for l in logits2.plan().strip().splitlines()]
    assert names.count("fused_attention[full,merge_heads]") == 2 and names.count("concat_dim1") + names.count("concat_dim0") == 4


def test_free_is_deferred_while_pending_ops_use_a_tensor(gpu):
    lib = __import__("applegpu_runtime_b200")._lib.load()
    a = gpu.tensor([1.0, 2.0], shape=[2])
    y = a.relu()
    aid = a.id
    gpu.destroy(a)                              # lazy.rs:118-144: still referenced by the pending relu
    assert lib.applegpu_ffi_dtype(aid) == 0     # metadata still resolvable
    yid = y.id
    gpu.destroy(y)                              # dropping the consumer releases the input too
    assert lib.applegpu_ffi_dtype(yid) == -1 and lib.applegpu_ffi_dtype(aid) == -1


def test_zero_size_alloc_returns_null_with_a_valid_id(gpu):
    lib = __import__("applegpu_runtime_b200")._lib.load()
    tid = ctypes.c_uint64(0)
    p = lib.applegpu_ffi_alloc(0, 0, ctypes.byref(tid))
    assert p is None and tid.value > 0          # backend_ffi.rs:96-100
    lib.applegpu_ffi_free(tid.value)


def test_errors_are_thread_local_strings(gpu):
    lib = __import__("applegpu_runtime_b200")._lib.load()
    assert lib.applegpu_ffi_add(999999999, 999999998) == 0
    assert b"add failed" in lib.applegpu_ffi_last_error()
    dims = (ctypes.c_uint64 * 8)(); nd = ctypes.c_uint32()
    assert lib.applegpu_ffi_shape(123456789, dims, ctypes.byref(nd)) == -1
    assert b"shape failed" in lib.applegpu_ffi_last_error()
    assert lib.applegpu_ffi_dtype(123456789) == -1
    assert lib.applegpu_ffi_register_tensor(1, dims, 1, 42) == -1
    assert b"Invalid dtype wire value: 42" in lib.applegpu_ffi_last_error()


def test_kernel_registry_names(gpu):
    # compute.rs:1478-1567 resolve_kernel: base name + dtype suffix
    assert gpu.resolve_kernel("matmul", "bfloat16") == "matmul_bf16"
    assert gpu.resolve_kernel("layer_norm", "float16") == "layer_norm_f16"
    assert gpu.resolve_kernel("elementwise_add", "int32") == "elementwise_add_i32"
    assert gpu.resolve_kernel("softmax_causal", "int32") is None
    assert gpu.resolve_kernel("matmul", "float64") is None


def test_pool_size_classes_and_stats_api(gpu):
    s = gpu.pool_stats()
    for k in ("hits", "misses", "pooled_bytes", "bucket_count"):   # pool.rs:100-108
        assert k in s
    assert gpu.memory_usage() >= 0 and gpu.tensor_count() >= 0


def test_graph_rewrites_collapse_the_bert_layer(gpu):
    cfg = {"n_layer": 2, "n_head": 4, "n_embd": 64, "d_ff": 128, "vocab_size": 100, "n_positions": 32, "type_vocab": 2, "eps": 1e-12}
    model = gpu.init_bert_weights(cfg, seed=0)
    h = gpu.bert_forward(model, np.arange(16).reshape(2, 8))
    assert h.shape == [2, 8, 64]
    names = [l.split("_f32")[0] for l in h.plan().strip().splitlines()]
    assert names.count("fused_attention[full,merge_heads]") == 2
    assert names.count("fused_linear[bias,]") == 2 and names.count("fused_linear[bias,gelu_exact,]") == 2
    assert names.count("fused_linear[bias,residual,]") == 4 and names.count("layer_norm") == 5
    # a tensor-parallel shard keeps half of the heads and of the feed-forward units
    host = {k: np.zeros(v.shape, np.float32) for k, v in model["weights"].items() if "qkv" not in k}
    for i in range(2):
        for n in ("query", "key", "value"):
            host[f"encoder.layer.{i}.attention.self.{n}.weight"] = np.zeros((64, 64), np.float32)
            host[f"encoder.layer.{i}.attention.self.{n}.bias"] = np.zeros(64, np.float32)
    shard = gpu.load_bert_state_dict(host, cfg, head_range=(2, 4), ff_range=(64, 128))
    assert shard["config"]["local_heads"] == 2
    assert shard["weights"]["encoder.layer.0.qkv.weight"].shape == [96, 64]
    assert shard["weights"]["encoder.layer.0.attention.output.dense.weight"].shape == [64, 32]
    assert shard["weights"]["encoder.layer.0.intermediate.dense.weight"].shape == [64, 64]
    assert shard["weights"]["encoder.layer.0.output.dense.weight"].shape == [64, 64]
    assert gpu.bert_forward(shard, np.arange(16).reshape(2, 8), all_reduce=lambda t: t).shape == [2, 8, 64]


def test_tensor_parallel_head_and_ff_ranges():
    from applegpu_runtime_b200.tp import head_and_ff_ranges
    cfg = {"n_head": 12, "d_ff": 3072}
    spans = [head_and_ff_ranges(cfg, r, 8) for r in range(8)]
    assert [h1 - h0 for (h0, h1), _ in spans] == [2, 2, 2, 2, 1, 1, 1, 1]      # uneven head split at 8 ranks
    assert spans[0][0][0] == 0 and spans[-1][0][1] == 12
    assert all(f1 - f0 == 384 for _, (f0, f1) in spans)
    assert head_and_ff_ranges(cfg, 0, 1) == ((0, 12), (0, 3072))


def test_op_tape_replays_the_gpt2_forward_at_a_longer_kv_length(gpu):
    m = _tiny_model(gpu)
    ids = np.arange(10).reshape(2, 5)
    logits, kv = gpu.gpt2_forward(m, ids)
    plans = []
    for step in range(3):
        ids = np.concatenate([ids, np.zeros((2, 1), np.int64)], axis=1)
        logits, kv = gpu.gpt2_forward(m, ids, kv_cache=kv, last_only=True, compiled=True)   # step 0 records, 1 and 2 replay
        assert logits.shape == [2, 100] and kv[0][0].shape == [2, 4, 6 + step, 16]
        plans.append([l.split(" ")[0] for l in logits.plan().strip().splitlines()])
    # nothing is evaluated in this metadata-only mode, so each plan also holds the earlier steps' pending ops:
    # every replay must add exactly what the recorded step added
    per_step = len(plans[1]) - len(plans[0])
    assert per_step > 0 and len(plans[2]) - len(plans[1]) == per_step
    from collections import Counter
    assert Counter(plans[2]) - Counter(plans[1]) == Counter(plans[1]) - Counter(plans[0])
    assert len(m["_tapes"]) == 1
    # errors: wrong input count, unknown tape, nested recording
    tape = next(iter(m["_tapes"].values()))
    with pytest.raises(ValueError, match="takes"):
        tape.replay([kv[0][0]])
    gpu.tape_begin([])
    try:
        with pytest.raises(ValueError, match="already being recorded"):
            gpu.tape_begin([])
    finally:
        gpu.tape_abort()
    x = gpu.from_numpy(np.ones((2, 2), np.float32))
    n = gpu.tape_begin([x])
    y = gpu.relu(x + x)
    t = gpu.tape_end(n, [y])
    z = gpu.from_numpy(np.ones((3, 5), np.float32))
    (r,) = t.replay([z])
    assert r.shape == [3, 5] and "fused_" in r.plan()
    gpu.tape_begin([x])
    with pytest.raises(ValueError, match="not produced on the tape"):
        gpu.tape_end(1, [z])


def test_lm_head_argmax_fuses_only_after_the_logits_handle_is_dropped(gpu):
    x = gpu.cast(gpu.from_numpy(np.ones((8, 32), np.float32)), "bfloat16")
    wte = gpu.cast(gpu.from_numpy(np.ones((50, 32), np.float32)), "bfloat16")
    logits = gpu.reshape(x @ gpu.transpose(wte), [2, 4, 50])      # the tail of gpt2_forward
    nxt = gpu.argmax(logits)
    assert nxt.shape == [2, 4]
    held = [l.split(" ")[0] for l in nxt.plan().strip().splitlines()]
    assert held[-1].startswith("argmax")                           # logits still reachable: kept as a tensor
    assert not any(h.startswith("fused_linear[argmax") for h in held)
    del logits
    dropped = [l.split(" ")[0] for l in nxt.plan().strip().splitlines()]
    assert dropped[-1].startswith("fused_linear[argmax,]") and not any(h.startswith("argmax") for h in dropped)
    # fp32 products keep the two-kernel form (the tensor-core kernel is half precision only)
    x32 = gpu.from_numpy(np.ones((8, 32), np.float32)); w32 = gpu.from_numpy(np.ones((50, 32), np.float32))
    l32 = x32 @ gpu.transpose(w32)
    n32 = gpu.argmax(l32)
    del l32
    assert not any(l.startswith("fused_linear[argmax") for l in n32.plan().splitlines())


def test_interleave_advances_generators_in_lock_step():
    """bert.interleave drives the micro-batch forwards of the overlapped tensor-parallel path: one segment of each in
    turn, return values in order, exhausted generators dropped."""
    from applegpu_runtime_b200.bert import interleave
    log = []

    def steps(tag, n):
        for i in range(n):
            log.append((tag, i))
            yield
        return tag.upper()

    assert interleave([steps("a", 2), steps("b", 3), steps("c", 0)]) == ["A", "B", "C"]
    assert log == [("a", 0), ("b", 0), ("a", 1), ("b", 1), ("b", 2)]
