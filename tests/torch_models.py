"""Small torch modules the torch-frontend tests run on both the CPU and the device."""
import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    """Pre-LN transformer block written the way torch users write it: nn.Linear on [B, T, D],
    split / view / transpose for the heads, scaled_dot_product_attention(is_causal=True)."""

    def __init__(self, d, heads):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc, self.out = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.heads = heads

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).split(D, dim=2)
        heads = lambda t: t.view(B, T, self.heads, D // self.heads).transpose(1, 2)
        a = F.scaled_dot_product_attention(heads(q), heads(k), heads(v), is_causal=True)
        x = x + self.proj(a.transpose(1, 2).contiguous().view(B, T, D))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class TinyLM(nn.Module):
    def __init__(self, vocab=128, d=256, heads=4, layers=2, ctx=64):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(ctx, d)
        self.blocks = nn.ModuleList(Block(d, heads) for _ in range(layers))
        self.lnf = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.head.weight = self.wte.weight          # tied, as in GPT-2
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02)

    def forward(self, ids):
        x = self.wte(ids) + self.wpe(torch.arange(ids.shape[1]))
        for b in self.blocks:
            x = b(x)
        return self.head(self.lnf(x))
