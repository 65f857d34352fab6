"""torch frontend (`applegpu_runtime_b200.torch_backend`): host-side logic, no device needed.

Mirrors what python/tests/test_torch_backend.py checks upstream at the recording level: tensors
wrap and keep shape / dtype, aten ops land in the op table, and a transformer written with plain
torch modules records the same fused plan as the hand-written forward.
"""
import copy

import pytest
import torch

from torch_models import TinyLM


@pytest.fixture()
def tb(gpu):
    import applegpu_runtime_b200.torch_backend as tb
    tb._enabled = True
    tb._strict = True
    tb.reset_fallback_stats()
    yield tb


def test_wrapper_keeps_shape_dtype_and_identity(tb):
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        t = tb.to_applegpu(torch.randn(3, 5).to(dt))
        assert isinstance(t, tb.ApplegpuTensor) and t.shape == (3, 5) and t.dtype == dt
        assert "applegpu" in repr(t)
        assert tb.to_applegpu(t) is t
    v = tb.to_applegpu(torch.randn(4, 6, 8))
    assert v.transpose(0, 2).shape == (8, 6, 4) and v.permute(2, 0, 1).shape == (8, 4, 6)
    assert v.reshape(24, 8).shape == (24, 8) and v[:, 1:3].shape == (4, 2, 8) and v[1].shape == (6, 8)
    assert v.unsqueeze(1).shape == (4, 1, 6, 8) and [s.shape for s in v.split(3, dim=1)] == [(4, 3, 8), (4, 3, 8)]
    assert torch.cat([v, v], dim=2).shape == (4, 6, 16)
    assert (v + v).shape == v.shape and (v * 2.0).dtype == torch.float32 and (1.0 - v).shape == v.shape


def test_ops_outside_the_table_raise_in_strict_mode(tb):
    t = tb.to_applegpu(torch.randn(4, 4))
    with pytest.raises(NotImplementedError, match="not in the op table"):
        torch.cumsum(t, 0)


def test_torch_transformer_records_the_fused_plan(tb, gpu):
    torch.manual_seed(0)
    model = tb.to_applegpu(TinyLM().eval(), torch.bfloat16)
    assert model.head.weight is model.wte.weight                      # tied weights stay one device tensor
    with torch.no_grad():
        logits = model(torch.randint(0, 128, (2, 16)))
    assert isinstance(logits, tb.ApplegpuTensor) and logits.shape == (2, 16, 128) and logits.dtype == torch.bfloat16
    if gpu.has_device:
        return                                                        # plans of evaluated graphs are empty
    kinds = [l.split(" ")[0] for l in logits._gpu.plan().strip().splitlines()]
    launched = [k for k in kinds if not k.startswith(("reshape", "transpose", "slice"))]
    assert tb.fallback_stats() == {}
    per_block = ["layer_norm_bf16", "fused_linear[bias,]_bf16", "fused_attention[causal,merge_heads]_bf16",
                 "fused_linear[bias,residual,]_bf16", "layer_norm_bf16", "fused_linear[bias,gelu,]_bf16", "fused_linear[bias,residual,]_bf16"]
    assert launched == ["embedding_bf16", "embedding_bf16", "elementwise_add_bf16"] + per_block * 2 + ["layer_norm_bf16", "matmul_bf16"]


def test_hf_gpt2_records_without_fallback(tb, gpu):
    transformers = pytest.importorskip("transformers")
    cfg = transformers.GPT2Config(n_layer=2, n_embd=128, n_head=2, vocab_size=96, n_positions=32, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = tb.to_applegpu(transformers.GPT2LMHeadModel(cfg).eval())
    assert type(model.transformer.h[0].mlp.act).__name__ == "GELU"     # gelu_new module -> aten gelu(tanh)
    with torch.no_grad():
        out = model(torch.randint(0, 96, (2, 12))).logits
    assert isinstance(out, tb.ApplegpuTensor) and out.shape == (2, 12, 96)
    assert tb.fallback_stats() == {}
    if not gpu.has_device:
        kinds = [l.split(" ")[0] for l in out._gpu.plan().strip().splitlines()]
        assert kinds.count("fused_attention[causal,merge_heads]_f32") == 2
        assert kinds.count("fused_linear[bias,gelu,]_f32") == 2 and kinds.count("fused_linear[bias,residual,]_f32") == 4


def test_compile_forward_replays_the_recorded_ops(tb, gpu):
    from collections import Counter
    torch.manual_seed(0)
    model = tb.to_applegpu(TinyLM().eval(), torch.bfloat16)
    run = tb.compile_forward(lambda ids: model(ids))
    with torch.no_grad():
        first = run(torch.randint(0, 128, (2, 16)))            # records
        second = run(torch.randint(0, 128, (2, 16)))           # replays
        other = run(torch.randint(0, 128, (2, 24)))            # new signature: records again
    assert len(run.cache) == 2
    assert first.shape == second.shape == (2, 16, 128) and other.shape == (2, 24, 128) and second.dtype == torch.bfloat16
    if not gpu.has_device:
        kinds = lambda t: Counter(l.split(" ")[0] for l in t._gpu.plan().strip().splitlines())
        a, b = kinds(first), kinds(second)
        # the replayed pass consists of the same kernels (the id upload / cast differs: it is outside the tape)
        for k in ("fused_linear[bias,gelu,]_bf16", "fused_linear[bias,residual,]_bf16", "fused_attention[causal,merge_heads]_bf16", "layer_norm_bf16"):
            assert a[k] == b[k] and a[k] > 0, k
    with pytest.raises(TypeError, match="device tensors"):
        tb.compile_forward(lambda ids: 3)(torch.zeros(2, 2))
    # the failed recording was aborted: a new one can start
    assert tb.compile_forward(lambda x: x + x)(torch.ones(2, 2)).shape == (2, 2)


def test_hf_bert_records_without_fallback(tb, gpu):
    transformers = pytest.importorskip("transformers")
    cfg = transformers.BertConfig(num_hidden_layers=2, hidden_size=128, num_attention_heads=2, intermediate_size=512, vocab_size=200,
                                  max_position_embeddings=64, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = tb.to_applegpu(transformers.BertModel(cfg, add_pooling_layer=False).eval())
    with torch.no_grad():
        out = model(torch.randint(0, 200, (2, 16))).last_hidden_state
    assert isinstance(out, tb.ApplegpuTensor) and out.shape == (2, 16, 128)
    assert tb.fallback_stats() == {}
    if not gpu.has_device:
        kinds = [l.split(" ")[0] for l in out._gpu.plan().strip().splitlines()]
        assert kinds.count("fused_attention[full,merge_heads]_f32") == 2            # bidirectional, head merge absorbed
        assert kinds.count("fused_linear[bias,gelu_exact,]_f32") == 2                # erf-GELU in the GEMM epilogue
        assert kinds.count("fused_linear[bias,residual,]_f32") == 4 and kinds.count("layer_norm_f32") == 5
