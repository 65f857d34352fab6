"""Generates tests/golden/bert_tiny.npz from transformers' BertModel on CPU (float32).

The reference runs HF encoder models through its torch backend (python/applegpu_runtime/
torch_backend.py:246-1805) and checks them against PyTorch CPU eager; the BERT-base benchmark
config uses the HF architecture (post-LN, erf-GELU, eps 1e-12, bidirectional attention). This
script builds a tiny BertModel from a BertConfig with seeded random init (no download) and stores
weights, inputs and the last hidden state. Run from the repo root:
    python tests/golden/make_golden_bert.py
"""
import os

import numpy as np
import torch
from transformers import BertConfig, BertModel

CFG = dict(n_layer=2, n_head=4, n_embd=32, d_ff=64, vocab_size=80, n_positions=24, type_vocab=2, eps=1e-12)


def main():
    torch.manual_seed(4321)
    hf = BertModel(BertConfig(vocab_size=CFG["vocab_size"], hidden_size=CFG["n_embd"], num_hidden_layers=CFG["n_layer"],
                              num_attention_heads=CFG["n_head"], intermediate_size=CFG["d_ff"],
                              max_position_embeddings=CFG["n_positions"], type_vocab_size=CFG["type_vocab"],
                              hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=CFG["eps"],
                              hidden_act="gelu"), add_pooling_layer=False).eval()
    g = torch.Generator().manual_seed(7)
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if name.endswith(".bias") or "LayerNorm" in name:
                p.add_(torch.randn(p.shape, generator=g) * 0.05)
    ids = torch.tensor([[2, 5, 10, 20, 50, 7, 3, 79, 1, 0], [3, 4, 5, 6, 7, 8, 9, 10, 11, 12]])
    types = torch.tensor([[0, 0, 0, 0, 0, 1, 1, 1, 1, 1], [0, 0, 0, 1, 1, 1, 1, 1, 1, 1]])
    with torch.no_grad():
        hidden = hf(input_ids=ids, token_type_ids=types).last_hidden_state.float()
    out = {"ids": ids.numpy().astype(np.int64), "types": types.numpy().astype(np.int64), "hidden": hidden.numpy(),
           "config": np.array([CFG["n_layer"], CFG["n_head"], CFG["n_embd"], CFG["d_ff"], CFG["vocab_size"], CFG["n_positions"],
                               CFG["type_vocab"]], np.int64)}
    for k, v in hf.state_dict().items():
        if k.endswith("position_ids") or k.endswith("token_type_ids"):
            continue
        out["w:" + k] = v.float().numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bert_tiny.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
