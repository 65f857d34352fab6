"""torch frontend on the device: the same torch module on PyTorch CPU and through
`applegpu_runtime_b200.torch_backend` (flows of python/tests/test_torch_backend.py and
test_gpt2.py upstream, with random-init weights standing in for the pretrained checkpoint)."""
import copy

import pytest
import torch

from torch_models import TinyLM

pytestmark = pytest.mark.gpu


@pytest.fixture()
def tb(gpu_dev):
    import applegpu_runtime_b200.torch_backend as tb
    tb.enable()                                  # strict: an op outside the table raises, nothing falls back to the host
    tb.reset_fallback_stats()
    return tb


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max())


def test_elementwise_and_layout_ops_match_torch(tb):
    torch.manual_seed(0)
    a, b = torch.randn(6, 10, 32), torch.randn(6, 10, 32)
    ga, gb = tb.to_applegpu(a), tb.to_applegpu(b)
    cases = {
        "add": (ga + gb, a + b), "sub_alpha": (torch.sub(ga, gb, alpha=2.0), torch.sub(a, b, alpha=2.0)), "mul": (ga * gb, a * b),
        "div": (ga / (gb.abs() + 1.0), a / (b.abs() + 1.0)), "scalar": (1.0 - ga * 0.5, 1.0 - a * 0.5), "neg_relu": (torch.relu(-ga), torch.relu(-a)),
        "tanh": (torch.tanh(ga), torch.tanh(a)), "gelu_tanh": (torch.nn.functional.gelu(ga, approximate="tanh"), torch.nn.functional.gelu(a, approximate="tanh")),
        "gelu_erf": (torch.nn.functional.gelu(ga), torch.nn.functional.gelu(a)), "pow3": (ga ** 3, a ** 3),
        "softmax": (torch.softmax(ga, -1), torch.softmax(a, -1)), "permute": (ga.permute(2, 0, 1).contiguous(), a.permute(2, 0, 1).contiguous()),
        "slice_cat": (torch.cat([ga[:, 2:5], gb[:, :3]], dim=1), torch.cat([a[:, 2:5], b[:, :3]], dim=1)),
        "select": (ga[3], a[3]),
        "bmm": (torch.bmm(ga, gb.transpose(1, 2)), torch.bmm(a, b.transpose(1, 2))),
        "layer_norm": (torch.nn.functional.layer_norm(ga, (32,)), torch.nn.functional.layer_norm(a, (32,))),
    }
    for name, (got, want) in cases.items():
        assert isinstance(got, tb.ApplegpuTensor), name
        assert got.shape == want.shape and _rel(got.to_torch_cpu(), want) < 2e-5, name
    assert tb.fallback_stats() == {}


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 2e-2)])
def test_torch_transformer_matches_cpu(tb, dtype, tol):
    torch.manual_seed(0)
    ref = TinyLM().eval()
    ids = torch.randint(0, 128, (3, 48))
    with torch.no_grad():
        want = ref(ids)
        import applegpu_runtime_b200 as gpu
        launches = gpu.launch_count()
        model = tb.to_applegpu(copy.deepcopy(ref), dtype)
        got = model(ids)                         # strict (the default): the whole forward stays in the op table
        out = got.to_torch_cpu()
    assert got.dtype == dtype and _rel(out.float(), want) < tol
    # 2 blocks: the fused plan launches ~20 kernels (+ uploads); the unfused composition would need > 60
    assert 15 <= gpu.launch_count() - launches <= 40
    assert gpu.pipeline_status() == 0
    # greedy next token identical (fp32)
    if dtype == torch.float32:
        assert torch.equal(torch.argmax(got[:, -1, :], dim=-1), want[:, -1, :].argmax(-1))


def test_hf_gpt2_random_init_logits_and_greedy_tokens(tb):
    transformers = pytest.importorskip("transformers")
    cfg = transformers.GPT2Config(n_layer=2, n_embd=128, n_head=2, vocab_size=96, n_positions=64, attn_implementation="sdpa")
    torch.manual_seed(0)
    ref = transformers.GPT2LMHeadModel(cfg).eval()
    ids = torch.randint(0, 96, (2, 12))
    with torch.no_grad():
        want = ref(ids).logits
        model = tb.to_applegpu(copy.deepcopy(ref))
        got = model(ids).logits
    assert isinstance(got, tb.ApplegpuTensor) and tb.fallback_stats() == {}
    assert _rel(got.to_torch_cpu(), want) < 2e-4
    # 6 greedy steps without a KV cache: same tokens as PyTorch CPU
    seq_ref, seq_dev = ids.clone(), ids.clone()
    with torch.no_grad():
        for _ in range(6):
            seq_ref = torch.cat([seq_ref, ref(seq_ref).logits[:, -1].argmax(-1, keepdim=True)], dim=1)
            nxt = torch.argmax(model(seq_dev).logits[:, -1, :], dim=-1)
            seq_dev = torch.cat([seq_dev, nxt.reshape(-1, 1)], dim=1)
    assert torch.equal(seq_ref, seq_dev)


def test_compile_forward_matches_the_uncompiled_forward(tb):
    torch.manual_seed(0)
    ref = TinyLM().eval()
    model = tb.to_applegpu(copy.deepcopy(ref))
    run = tb.compile_forward(lambda ids: model(ids))
    import applegpu_runtime_b200 as gpu
    with torch.no_grad():
        for seed in range(3):                                  # call 0 records, 1 and 2 replay
            ids = torch.randint(0, 128, (3, 40), generator=torch.Generator().manual_seed(seed))
            got = run(ids).to_torch_cpu()
            assert _rel(got, ref(ids)) < 2e-4
    assert len(run.cache) == 1 and gpu.pipeline_status() == 0


def test_hf_bert_random_init_matches_cpu(tb):
    transformers = pytest.importorskip("transformers")
    cfg = transformers.BertConfig(num_hidden_layers=2, hidden_size=128, num_attention_heads=2, intermediate_size=512, vocab_size=200,
                                  max_position_embeddings=64, attn_implementation="sdpa")
    torch.manual_seed(0)
    ref = transformers.BertModel(cfg, add_pooling_layer=False).eval()
    ids = torch.randint(0, 200, (3, 40))
    with torch.no_grad():
        want = ref(ids).last_hidden_state
        got = tb.to_applegpu(copy.deepcopy(ref))(ids).last_hidden_state
        got16 = tb.to_applegpu(copy.deepcopy(ref), torch.bfloat16)(ids).last_hidden_state
    assert tb.fallback_stats() == {}
    assert _rel(got.to_torch_cpu(), want) < 2e-4
    assert _rel(got16.to_torch_cpu().float(), want) < 3e-2     # 64-wide heads in bf16: tensor-core attention and linears
