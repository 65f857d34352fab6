"""TEST INFRASTRUCTURE: PyTorch CPU eager restatement of the model forwards.

PyTorch CPU eager is the reference's own correctness oracle and benchmark baseline
(python/tests/test_cpp_backend.py:311-371 compares a GPT-2 against the same module on CPU;
python/tests/bench_comparison.py:23-50 and benchmarks/bench_mlp_cpp.py:30-79 time the CPU path).
`gpt2_forward` follows python/applegpu_runtime/models/gpt2.py:47-180 op for op on torch
tensors, with a batch dimension; tests pin it against transformers' GPT2LMHeadModel
(tests/golden/make_golden.py).
"""
import math

import torch
import torch.nn.functional as F


def gelu_tanh(x):
    # the reference clamps the tanh argument to [-10, 10] (kernel_templates.rs:301); tanh is
    # already +-1 in float32 there, so this equals torch's approximate='tanh' form.
    return F.gelu(x, approximate="tanh")


def gpt2_forward(weights, config, input_ids, kv_cache=None, dtype=torch.float32):
    """weights: {HF name: torch tensor}; input_ids: LongTensor [B, T]. Returns (logits [B,T,V], cache)."""
    n_layer, n_head, d = config["n_layer"], config["n_head"], config["n_embd"]
    dh = d // n_head
    ids = input_ids
    use_cache = kv_cache is not None
    if use_cache:
        tok = ids[:, -1:]
        pos0 = ids.shape[1] - 1
    else:
        tok = ids
        pos0 = 0
    B, T = tok.shape
    w = {k: v.to(dtype) for k, v in weights.items()}
    pos = torch.arange(pos0, pos0 + T)
    x = w["transformer.wte.weight"][tok] + w["transformer.wpe.weight"][pos][None]
    new_cache = []
    for i in range(n_layer):
        p = f"transformer.h.{i}"
        h = F.layer_norm(x, (d,), w[f"{p}.ln_1.weight"], w[f"{p}.ln_1.bias"], 1e-5)
        qkv = h @ w[f"{p}.attn.c_attn.weight"] + w[f"{p}.attn.c_attn.bias"]
        q, k, v = qkv.split(d, dim=-1)
        q = q.view(B, T, n_head, dh).transpose(1, 2)
        k = k.view(B, T, n_head, dh).transpose(1, 2)
        v = v.view(B, T, n_head, dh).transpose(1, 2)
        if use_cache:
            ck, cv = kv_cache[i]
            k = torch.cat([ck, k], dim=2)
            v = torch.cat([cv, v], dim=2)
        new_cache.append((k, v))
        scores = (q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(dh))
        if not use_cache:
            mask = torch.ones(T, T, dtype=torch.bool).tril()
            scores = scores.masked_fill(~mask, float("-inf"))
        att = torch.softmax(scores.float(), dim=-1).to(dtype)
        y = (att @ v).transpose(1, 2).reshape(B, T, d)
        x = x + (y @ w[f"{p}.attn.c_proj.weight"] + w[f"{p}.attn.c_proj.bias"])
        h2 = F.layer_norm(x, (d,), w[f"{p}.ln_2.weight"], w[f"{p}.ln_2.bias"], 1e-5)
        f = gelu_tanh(h2 @ w[f"{p}.mlp.c_fc.weight"] + w[f"{p}.mlp.c_fc.bias"])
        x = x + (f @ w[f"{p}.mlp.c_proj.weight"] + w[f"{p}.mlp.c_proj.bias"])
    x = F.layer_norm(x, (d,), w["transformer.ln_f.weight"], w["transformer.ln_f.bias"], 1e-5)
    logits = x @ w["transformer.wte.weight"].t()
    return logits, new_cache


def gpt2_greedy(weights, config, prompt_ids, max_tokens, dtype=torch.float32):
    """Greedy decode with KV cache; prompt_ids LongTensor [B, T]."""
    ids = prompt_ids.clone()
    cache = None
    for _ in range(max_tokens):
        logits, cache = gpt2_forward(weights, config, ids, kv_cache=cache, dtype=dtype)
        nxt = logits[:, -1, :].float().argmax(-1, keepdim=True)
        ids = torch.cat([ids, nxt], dim=1)
    return ids


def init_gpt2_weights(config, seed=0, std=0.02):
    """Same generator and order as applegpu_runtime_b200.gpt2.init_gpt2_weights (numpy default_rng)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    d, L = config["n_embd"], config["n_layer"]
    out = {}

    def normal(*shape):
        return torch.from_numpy((rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32))

    out["transformer.wte.weight"] = normal(config["vocab_size"], d)
    out["transformer.wpe.weight"] = normal(config["n_positions"], d)
    for i in range(L):
        p = f"transformer.h.{i}"
        out[f"{p}.ln_1.weight"] = torch.ones(d); out[f"{p}.ln_1.bias"] = torch.zeros(d)
        out[f"{p}.attn.c_attn.weight"] = normal(d, 3 * d); out[f"{p}.attn.c_attn.bias"] = torch.zeros(3 * d)
        out[f"{p}.attn.c_proj.weight"] = normal(d, d); out[f"{p}.attn.c_proj.bias"] = torch.zeros(d)
        out[f"{p}.ln_2.weight"] = torch.ones(d); out[f"{p}.ln_2.bias"] = torch.zeros(d)
        out[f"{p}.mlp.c_fc.weight"] = normal(d, 4 * d); out[f"{p}.mlp.c_fc.bias"] = torch.zeros(4 * d)
        out[f"{p}.mlp.c_proj.weight"] = normal(4 * d, d); out[f"{p}.mlp.c_proj.bias"] = torch.zeros(d)
    out["transformer.ln_f.weight"] = torch.ones(d); out["transformer.ln_f.bias"] = torch.zeros(d)
    return out


def mlp_forward(x, w1, b1, w2, b2):
    """Linear(64,128) -> ReLU -> Linear(128,10): the reference's CPU-runnable config
    (benchmarks/bench_mlp_cpp.py, python/tests/test_cpp_backend.py:121-133)."""
    return F.linear(F.relu(F.linear(x, w1, b1)), w2, b2)


def bert_forward(weights, config, input_ids, token_type_ids=None, dtype=torch.float32):
    """HF-architecture BERT encoder (post-LN, erf-GELU, bidirectional attention, no padding mask),
    the BERT-base benchmark configuration of the reference's torch backend
    (python/applegpu_runtime/torch_backend.py:246-1805 routes these ops one by one). weights:
    {BertModel state-dict name: tensor}; returns the last hidden state [B, T, d]. Pinned against
    transformers.BertModel through tests/golden/bert_tiny.npz (tests/golden/make_golden_bert.py)."""
    n_layer, n_head, d = config["n_layer"], config["n_head"], config["n_embd"]
    eps = config.get("eps", 1e-12)
    dh = d // n_head
    B, T = input_ids.shape
    if token_type_ids is None:
        token_type_ids = torch.zeros_like(input_ids)
    w = {k: v.to(dtype) for k, v in weights.items()}
    pos = torch.arange(T)
    x = w["embeddings.word_embeddings.weight"][input_ids] + w["embeddings.position_embeddings.weight"][pos][None] + \
        w["embeddings.token_type_embeddings.weight"][token_type_ids]
    x = F.layer_norm(x, (d,), w["embeddings.LayerNorm.weight"], w["embeddings.LayerNorm.bias"], eps)
    for i in range(n_layer):
        p = f"encoder.layer.{i}"

        def heads(t):
            return t.view(B, T, n_head, dh).transpose(1, 2)

        q = heads(F.linear(x, w[f"{p}.attention.self.query.weight"], w[f"{p}.attention.self.query.bias"]))
        k = heads(F.linear(x, w[f"{p}.attention.self.key.weight"], w[f"{p}.attention.self.key.bias"]))
        v = heads(F.linear(x, w[f"{p}.attention.self.value.weight"], w[f"{p}.attention.self.value.bias"]))
        scores = torch.matmul(q, k.transpose(-1, -2)) * (1.0 / math.sqrt(dh))
        attn = torch.matmul(torch.softmax(scores.float(), dim=-1).to(dtype), v)
        attn = attn.transpose(1, 2).reshape(B, T, d)
        attn = F.linear(attn, w[f"{p}.attention.output.dense.weight"], w[f"{p}.attention.output.dense.bias"])
        x = F.layer_norm(x + attn, (d,), w[f"{p}.attention.output.LayerNorm.weight"], w[f"{p}.attention.output.LayerNorm.bias"], eps)
        h = F.gelu(F.linear(x, w[f"{p}.intermediate.dense.weight"], w[f"{p}.intermediate.dense.bias"]))
        h = F.linear(h, w[f"{p}.output.dense.weight"], w[f"{p}.output.dense.bias"])
        x = F.layer_norm(x + h, (d,), w[f"{p}.output.LayerNorm.weight"], w[f"{p}.output.LayerNorm.bias"], eps)
    return x


def init_bert_weights(config, seed=0, std=0.02):
    """Seeded random BERT weights with the HF names and init (N(0, std) matrices and embeddings, zero
    biases, unit LayerNorm gains); same generator and draw order as applegpu_runtime_b200.bert."""
    import numpy as np
    rng = np.random.default_rng(seed)
    d, L, ff = config["n_embd"], config["n_layer"], config["d_ff"]
    out = {}

    def normal(*shape):
        return torch.from_numpy((rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32))

    out["embeddings.word_embeddings.weight"] = normal(config["vocab_size"], d)
    out["embeddings.position_embeddings.weight"] = normal(config["n_positions"], d)
    out["embeddings.token_type_embeddings.weight"] = normal(config.get("type_vocab", 2), d)
    out["embeddings.LayerNorm.weight"] = torch.ones(d); out["embeddings.LayerNorm.bias"] = torch.zeros(d)
    for i in range(L):
        p = f"encoder.layer.{i}"
        for name, shape in (("attention.self.query", (d, d)), ("attention.self.key", (d, d)), ("attention.self.value", (d, d)),
                            ("attention.output.dense", (d, d)), ("intermediate.dense", (ff, d)), ("output.dense", (d, ff))):
            out[f"{p}.{name}.weight"] = normal(*shape); out[f"{p}.{name}.bias"] = torch.zeros(shape[0])
        for name in ("attention.output.LayerNorm", "output.LayerNorm"):
            out[f"{p}.{name}.weight"] = torch.ones(d); out[f"{p}.{name}.bias"] = torch.zeros(d)
    return out
