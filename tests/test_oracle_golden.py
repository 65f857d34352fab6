"""Pins the CPU oracle: oracle/msl_ref.c against every known-answer vector the reference's
tests hold (tests/golden/known_answers.json), and oracle/torch_ref.py against logits and greedy
tokens produced by the reference's CPU path (transformers GPT2LMHeadModel on CPU, stored in
tests/golden/gpt2_tiny.npz by tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import msl_ref as R
from oracle import torch_ref

HERE = os.path.dirname(os.path.abspath(__file__))

with open(os.path.join(HERE, "golden", "known_answers.json")) as f:
    CASES = json.load(f)["cases"]


def run_oracle_case(c):
    f32 = lambda v: np.asarray(v, dtype=np.float32)
    op = c["op"]
    if op == "matmul": return R.matmul(f32(c["a"]), f32(c["b"]))
    if op == "softmax": return R.softmax(f32(c["x"]))
    if op == "softmax_causal": return R.softmax_causal(f32(c["x"]))
    if op == "layer_norm": return R.layer_norm(f32(c["x"]), f32(c["gamma"]), f32(c["beta"]), c["eps"])
    if op == "gelu": return R.gelu(f32(c["x"]))
    if op == "embedding": return R.embedding(f32(c["w"]), np.asarray(c["idx"], np.int32))
    if op == "add_bias": return R.add_bias(f32(c["x"]), f32(c["bias"]))
    if op == "argmax": return R.argmax(f32(c["x"]))
    if op == "gather": return R.gather(f32(c["x"]), c["dim"], np.asarray(c["idx"], np.int32))
    if op == "index_select": return R.index_select(f32(c["x"]), c["dim"], np.asarray(c["idx"], np.int32))
    raise AssertionError(op)


@pytest.mark.parametrize("case", CASES, ids=[f'{c["op"]}@{c["src"].split(" ")[0]}' for c in CASES])
def test_oracle_matches_reference_known_answers(case):
    got = run_oracle_case(case)
    exp = np.asarray(case["expect"])
    assert got.shape == exp.shape
    if case["tol"] == 0:
        assert np.array_equal(got.astype(np.float64), exp.astype(np.float64))
    else:
        assert np.max(np.abs(got.astype(np.float64) - exp)) <= case["tol"]


def test_oracle_matches_numpy_formulas():
    # the numpy formulations the reference's Python tests compare against
    rng = np.random.default_rng(0)
    x = rng.standard_normal((7, 33)).astype(np.float32)
    g = rng.standard_normal(33).astype(np.float32); b = rng.standard_normal(33).astype(np.float32)
    mean = x.mean(-1, keepdims=True); var = x.var(-1, keepdims=True)   # population variance (test_transformer_ops.py:44-83)
    np.testing.assert_allclose(R.layer_norm(x, g, b), g * (x - mean) / np.sqrt(var + 1e-5) + b, rtol=1e-4, atol=1e-5)
    e = np.exp(x - x.max(-1, keepdims=True))
    np.testing.assert_allclose(R.softmax(x), e / e.sum(-1, keepdims=True), rtol=1e-4)     # test_batched_ops.py:83-94
    a = rng.standard_normal((3, 5, 8)).astype(np.float32); w = rng.standard_normal((3, 8, 4)).astype(np.float32)
    np.testing.assert_allclose(R.matmul(a, w), np.matmul(a, w), rtol=1e-4, atol=1e-4)      # test_batched_ops.py:20-54
    np.testing.assert_allclose(R.matmul(a, w[0]), np.matmul(a, w[0]), rtol=1e-4, atol=1e-4)  # broadcast operand
    xs = torch.from_numpy(x)
    np.testing.assert_allclose(R.gelu(x), torch.nn.functional.gelu(xs, approximate="tanh").numpy(), atol=1e-5)  # test_gelu_exact.py:17-24
    np.testing.assert_allclose(R.gelu_exact(x), torch.nn.functional.gelu(xs).numpy(), atol=1e-5)               # test_gelu_exact.py:7-15


def test_oracle_quantize_round_half_away_and_clamp():
    # no upstream numeric test exists for quantize (parity unpinned); these are the rules of
    # kernel_templates.rs:2210-2211 checked on hand-computed values
    x = np.array([0.25, -0.25, 0.35, 0.05, -0.05, 100.0, -100.0, 0.0], np.float32)
    assert R.quantize(x, "int8", 0.1).tolist() == [3, -3, 4, 1, -1, 127, -128, 0]
    assert R.quantize(x, "uint8", 0.1, 10).tolist() == [13, 7, 14, 11, 9, 255, 0, 10]
    q = np.array([-128, -1, 0, 1, 127], np.int8)
    np.testing.assert_array_equal(R.dequantize(q, "float32", 0.5, 3), (q.astype(np.int32) - 3).astype(np.float32) * 0.5)


def test_oracle_causal_softmax_masking_and_bf16_store_rounding():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 5, 5)).astype(np.float32)
    y = R.softmax_causal(x)
    assert np.all(np.triu(y, 1) == 0)
    np.testing.assert_allclose(y.sum(-1), 1.0, rtol=1e-5)
    assert y[0, 0, 0] == 1.0
    yb = R.from_bf16(R.softmax_causal(R.to_bf16(x)))
    np.testing.assert_allclose(yb, y, atol=2e-2)


def _fixture():
    z = np.load(os.path.join(HERE, "golden", "gpt2_tiny.npz"))
    cfgv = z["config"].tolist()
    cfg = dict(n_layer=cfgv[0], n_head=cfgv[1], n_embd=cfgv[2], vocab_size=cfgv[3], n_positions=cfgv[4])
    weights = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("w:")}
    return cfg, weights, z


def test_torch_oracle_reproduces_reference_cpu_logits_and_greedy_tokens():
    cfg, weights, z = _fixture()
    ids = torch.from_numpy(z["ids"])
    logits, _ = torch_ref.gpt2_forward(weights, cfg, ids)
    np.testing.assert_allclose(logits.numpy(), z["logits"], atol=1e-5)
    assert logits.argmax(-1).tolist() == torch.from_numpy(z["logits"]).argmax(-1).tolist()
    greedy = torch_ref.gpt2_greedy(weights, cfg, ids, max_tokens=6)   # with KV cache
    assert greedy.tolist() == z["greedy"].tolist()


def test_msl_oracle_composes_to_the_same_gpt2_block():
    # The C restatement, chained like python/applegpu_runtime/models/gpt2.py:94-169, reproduces the
    # torch forward of one attention sub-block: pins matmul + add_bias + attention_causal together.
    cfg, weights, z = _fixture()
    d, h = cfg["n_embd"], cfg["n_head"]; dh = d // h
    rng = np.random.default_rng(2)
    T = 6
    x = rng.standard_normal((T, d)).astype(np.float32)
    W = weights["transformer.h.0.attn.c_attn.weight"].numpy(); bqkv = weights["transformer.h.0.attn.c_attn.bias"].numpy()
    qkv = R.add_bias(R.matmul(x, W), bqkv)
    q, k, v = [np.ascontiguousarray(qkv[:, i * d:(i + 1) * d].reshape(T, h, dh).transpose(1, 0, 2)) for i in range(3)]
    out = R.attention(q, k, v, causal=True)
    xt = torch.from_numpy(x)
    qkv_t = xt @ torch.from_numpy(W) + torch.from_numpy(bqkv)
    qt, kt, vt = [t.view(T, h, dh).transpose(0, 1) for t in qkv_t.split(d, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
    np.testing.assert_allclose(out, ref.numpy(), atol=1e-5)


def test_torch_oracle_reproduces_hf_bert_hidden_states():
    """oracle/torch_ref.bert_forward against transformers' BertModel on CPU (tests/golden/bert_tiny.npz)."""
    import torch
    from oracle import torch_ref
    z = np.load(os.path.join(HERE, "golden", "bert_tiny.npz"))
    c = z["config"].tolist()
    cfg = dict(n_layer=c[0], n_head=c[1], n_embd=c[2], d_ff=c[3], vocab_size=c[4], n_positions=c[5], type_vocab=c[6], eps=1e-12)
    w = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("w:")}
    with torch.no_grad():
        h = torch_ref.bert_forward(w, cfg, torch.from_numpy(z["ids"]), torch.from_numpy(z["types"])).numpy()
    np.testing.assert_allclose(h, z["hidden"], atol=1e-5)
