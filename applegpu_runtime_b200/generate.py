"""Autoregressive generation over gpt2_forward.

Reference: python/applegpu_runtime/models/generate.py — `_sample_token` (:34-80, temperature /
top-k / top-p on the host) and `generate` (:83-127, KV cache, full-logit readback each step).
Greedy decoding here takes argmax on the device (first index of the maximum, the same
tie-break as numpy's argmax that upstream uses) and reads back one int32 per sequence instead of
a [T, vocab] matrix.
"""
import numpy as np

from . import api as gpu
from .gpt2 import gpt2_forward


def _sample_token(logits_np, temperature=1.0, top_k=0, top_p=0.0, rng=None):
    if temperature <= 0:
        return int(np.argmax(logits_np))
    rng = rng or np.random
    logits_np = logits_np / temperature
    if top_k > 0:
        top_k = min(top_k, len(logits_np))
        keep = np.argpartition(logits_np, -top_k)[-top_k:]
        masked = np.full_like(logits_np, -np.inf)
        masked[keep] = logits_np[keep]
        logits_np = masked
    logits_np = logits_np - np.max(logits_np)
    probs = np.exp(logits_np)
    probs = probs / probs.sum()
    if top_p > 0.0:
        order = np.argsort(probs)[::-1]
        cum = np.cumsum(probs[order])
        cutoff = np.searchsorted(cum, top_p) + 1
        allowed = order[:cutoff]
        m = np.zeros_like(probs)
        m[allowed] = probs[allowed]
        probs = m / m.sum()
    return int(rng.choice(len(probs), p=probs))


def greedy_generate(model, input_ids, max_tokens=50, use_cache=True, compiled=True):
    """Greedy decode for a batch of equal-length prompts [B, T]; returns [B, T + max_tokens]. With
    `compiled` the decode steps (one new token against the KV cache) replay an op tape instead of
    re-issuing ~300 op calls each. With the cache, the token a step picks stays on the device and
    feeds the next step's embedding lookup directly (position ids come from one table uploaded up
    front), so the host never waits for the GPU inside the loop: it records step i+1 while step i
    runs, and the picked tokens are read back once at the end."""
    ids = np.asarray(input_ids, dtype=np.int64)
    if ids.ndim == 1:
        ids = ids.reshape(1, -1)
    if not use_cache:
        for _ in range(max_tokens):
            logits, _ = gpt2_forward(model, ids, kv_cache=None, last_only=True)
            nxt_t = gpu.argmax(logits)
            del logits
            ids = np.concatenate([ids, nxt_t.to_numpy().astype(np.int64).reshape(-1, 1)], axis=1)
        return ids
    B, T0 = ids.shape
    if max_tokens <= 0:
        return ids
    # positions of the decode steps: row s holds B copies of T0 + s (the step that consumes the token picked after
    # s + 1 forwards sits at position T0 + s)
    pos_table = gpu.from_numpy(np.repeat(np.arange(T0, T0 + max_tokens, dtype=np.int32)[:, None], B, axis=1))
    picked = []
    logits, kv = gpt2_forward(model, ids, kv_cache=None, last_only=True)          # prefill of the prompt
    for step in range(max_tokens):
        nxt_t = gpu.argmax(logits)
        del logits   # with the handle gone the LM head takes the row maximum in its own epilogue: no logits tensor
        nxt_t.eval()                                                              # launches only: no host wait
        picked.append(nxt_t)
        if step + 1 == max_tokens:
            break
        pos = gpu.reshape(gpu.slice(pos_table, 0, step, step + 1), [B])
        shape_only = np.empty((B, T0 + step + 1), dtype=np.int8)                  # gives the forward its [B, T] shape
        logits, kv = gpt2_forward(model, shape_only, kv_cache=kv, last_only=True, device_ids=(nxt_t, pos), compiled=compiled)
    new = np.stack([t.to_numpy().astype(np.int64).reshape(-1) for t in picked], axis=1)
    return np.concatenate([ids, new], axis=1)


def generate(model, input_ids, max_tokens=50, use_cache=True, temperature=1.0, top_k=50, top_p=0.9):
    """Same contract as the reference's `generate`: list of prompt ids in, prompt + generated out."""
    ids = list(input_ids)
    if temperature <= 0:
        return greedy_generate(model, ids, max_tokens, use_cache)[0].tolist()
    kv = None
    gpu.pool_drain()
    for _ in range(max_tokens):
        if use_cache:
            logits, kv = gpt2_forward(model, ids, kv_cache=kv, last_only=True)
        else:
            logits, _ = gpt2_forward(model, ids, kv_cache=None, last_only=True)
        last = logits.to_numpy().astype(np.float32)[0]
        ids.append(_sample_token(last, temperature=temperature, top_k=top_k, top_p=top_p))
    return ids
