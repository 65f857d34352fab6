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


_WEIGHT_ORDER = ("ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias", "attn.c_proj.weight", "attn.c_proj.bias",
                 "ln_2.weight", "ln_2.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias")


class Gpt2Decoder:
    """The library's static-shape decoder (include/applegpu_b200_ext.h, applegpu_gpt2_decoder_*): a preallocated
    [B, heads, max_len, 64] KV cache per layer appended in place, and a decode step captured once as a CUDA graph."""

    def __init__(self, model, batch, max_len):
        import ctypes
        from . import _lib
        self._lib = _lib.load()
        cfg, w = model["config"], model["weights"]
        names = ["transformer.wte.weight", "transformer.wpe.weight", "transformer.ln_f.weight", "transformer.ln_f.bias"]
        for i in range(cfg["n_layer"]):
            names += [f"transformer.h.{i}.{n}" for n in _WEIGHT_ORDER]
        ids = (ctypes.c_uint64 * len(names))(*[w[n].id for n in names])
        self.batch, self.max_len = int(batch), int(max_len)
        self.handle = int(self._lib.applegpu_gpt2_decoder_create(ids, len(names), cfg["n_layer"], cfg["n_head"], cfg["n_embd"], cfg["vocab_size"],
                                                                 cfg["n_positions"], self.batch, self.max_len))
        if not self.handle:
            raise ValueError(gpu._err())

    @staticmethod
    def supports(model, batch, total_len):
        cfg = model["config"]
        return ("int8" not in model and model.get("dtype", "float32") in ("float32", "float16", "bfloat16") and cfg["n_embd"] == 64 * cfg["n_head"]
                and 1 <= batch <= 16 and total_len <= cfg["n_positions"])

    def prefill(self, kv_cache, first_tokens, prompt_len):
        import ctypes
        flat = [t.id for kv in kv_cache for t in kv]
        arr = (ctypes.c_uint64 * len(flat))(*flat)
        if self._lib.applegpu_gpt2_decoder_prefill(self.handle, arr, len(flat), first_tokens.id, int(prompt_len)) != 0:
            raise ValueError(gpu._err())

    def steps(self, n, use_graph=True):
        """Runs n decode steps; returns the picked tokens as an int32 array [n, batch]."""
        import ctypes
        out = np.empty((int(n), self.batch), np.int32)
        if n > 0 and self._lib.applegpu_gpt2_decoder_steps(self.handle, int(n), out.ctypes.data_as(ctypes.c_void_p), bool(use_graph)) != 0:
            raise ValueError(gpu._err())
        return out

    def set_engine(self, persistent=False):
        """persistent=False (the default): one kernel per op, chained by programmatic dependent launches; True: the
        embeddings and all layers of a step run as one cooperative kernel with grid-wide barriers between phases (same
        arithmetic, same tokens; measured slower, kept as an option)."""
        if self._lib.applegpu_gpt2_decoder_set_engine(self.handle, 1 if persistent else 0) != 0:
            raise ValueError(gpu._err())

    @property
    def launches_per_step(self):
        return int(self._lib.applegpu_gpt2_decoder_launches_per_step(self.handle))

    @property
    def uses_graph(self):
        return int(self._lib.applegpu_gpt2_decoder_uses_graph(self.handle)) == 1

    def close(self):
        if self.handle:
            self._lib.applegpu_gpt2_decoder_destroy(self.handle)
            self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def greedy_generate(model, input_ids, max_tokens=50, use_cache=True, compiled=True, engine="auto"):
    """Greedy decode for a batch of equal-length prompts [B, T]; returns [B, T + max_tokens].

    With the cache and `engine` "auto" or "graph", the prompt runs through gpt2_forward and the decode steps through
    the library's decoder: a preallocated KV cache appended in place and one captured step replayed per token
    ("graph"; "direct" issues the same launches one by one; "persistent" and "persistent_direct" run the layers of a
    step as one cooperative kernel instead of one kernel per op). `engine="tape"` keeps the cache the reference's way
    (concatenation, models/gpt2.py:122-127) and replays an op tape per step (`compiled`), the picked token staying
    on the device between steps. Models the decoder does not take (int8 weights, head dimension other than 64,
    more than 16 sequences) use the tape engine."""
    ids = np.asarray(input_ids, dtype=np.int64)
    if ids.ndim == 1:
        ids = ids.reshape(1, -1)
    if use_cache and max_tokens > 1 and engine in ("auto", "graph", "direct", "persistent", "persistent_direct") and Gpt2Decoder.supports(model, ids.shape[0], ids.shape[1] + max_tokens):
        B, T0 = ids.shape
        logits, kv = gpt2_forward(model, ids, kv_cache=None, last_only=True)      # prefill of the prompt
        first = gpu.argmax(logits)
        del logits
        dec = Gpt2Decoder(model, B, T0 + max_tokens)
        try:
            dec.set_engine(persistent=engine.startswith("persistent"))
            dec.prefill(kv, first, T0)
            rest = dec.steps(max_tokens - 1, use_graph=engine in ("auto", "graph", "persistent"))
            model["_last_decoder_stats"] = {"launches_per_step": dec.launches_per_step, "graph": dec.uses_graph}
        finally:
            dec.close()
        new = np.concatenate([first.to_numpy().astype(np.int64).reshape(B, 1), rest.T.astype(np.int64)], axis=1)
        return np.concatenate([ids, new], axis=1)
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
