"""Generates tests/golden/gpt2_tiny.npz from the reference's CPU path.

The reference validates its GPU forward against PyTorch CPU eager on a small GPT-2
(python/tests/test_cpp_backend.py:311-371) and against transformers' GPT2LMHeadModel
(:396-480, needs downloaded weights). This script builds a GPT2LMHeadModel from a GPT2Config
with seeded random init (no download), runs it on CPU in float32, and stores weights, token
ids, logits and greedy continuations. Run from the repo root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch
from transformers import GPT2Config, GPT2LMHeadModel

CFG = dict(n_layer=2, n_head=4, n_embd=32, vocab_size=96, n_positions=24)


def main():
    torch.manual_seed(1234)
    hf = GPT2LMHeadModel(GPT2Config(vocab_size=CFG["vocab_size"], n_positions=CFG["n_positions"], n_embd=CFG["n_embd"],
                                    n_layer=CFG["n_layer"], n_head=CFG["n_head"], resid_pdrop=0.0, embd_pdrop=0.0,
                                    attn_pdrop=0.0)).eval()
    # HF zero-initialises biases and sets LayerNorm to (1, 0); perturb them so the fixture exercises those terms.
    g = torch.Generator().manual_seed(99)
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if name.endswith(".bias") or "ln_" in name:
                p.add_(torch.randn(p.shape, generator=g) * 0.05)
    ids = torch.tensor([[1, 5, 10, 20, 50, 7, 3, 95], [3, 4, 5, 6, 7, 8, 9, 10]])
    with torch.no_grad():
        logits = hf(ids).logits.float()
        cur = ids.clone()
        for _ in range(6):
            nxt = hf(cur).logits[:, -1, :].argmax(-1, keepdim=True)
            cur = torch.cat([cur, nxt], dim=1)
    out = {"ids": ids.numpy().astype(np.int64), "logits": logits.numpy(), "greedy": cur.numpy().astype(np.int64),
           "config": np.array([CFG["n_layer"], CFG["n_head"], CFG["n_embd"], CFG["vocab_size"], CFG["n_positions"]], np.int64)}
    for k, v in hf.state_dict().items():
        if k.endswith(".attn.bias") or k.endswith(".attn.masked_bias") or k == "lm_head.weight":
            continue
        out["w:" + k] = v.float().numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gpt2_tiny.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
