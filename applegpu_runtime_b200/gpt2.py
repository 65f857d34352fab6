"""GPT-2 forward as a sequence of hot-path ops, with a batch dimension.

Follows the reference's python/applegpu_runtime/models/gpt2.py:47-180 op for op (pre-LN blocks,
tanh-GELU, learned positions, tied LM head, KV cache by concatenation) and adds what the
reference lacks: a batch dimension ([B, T] token ids; linears run on [B*T, d], attention on
[B, heads, T, d_head]). The slice / reshape / transpose_dims calls below are views in this
runtime, and the fusion pass folds add_bias / gelu / residual into the GEMM epilogues and the
five attention ops into one node, so the kernel count per layer is far below the op count.
"""
import os

import numpy as np

from . import api as gpu

GPT2_SMALL = {"n_layer": 12, "n_head": 12, "n_embd": 768, "vocab_size": 50257, "n_positions": 1024}
GPT2_LARGE = {"n_layer": 36, "n_head": 20, "n_embd": 1280, "vocab_size": 50257, "n_positions": 1024}


def init_gpt2_weights(config=None, seed=0, dtype="float32", std=0.02):
    """Random-init weights with the HF GPT-2 layout and init (N(0, std) matrices and embeddings,
    zero biases, unit LayerNorm gains). Keys match `GPT2LMHeadModel.state_dict()`; Conv1D weights
    are [in, out] so `x @ W` needs no transpose (reference: models/gpt2.py:6-47)."""
    cfg = dict(GPT2_SMALL if config is None else config)
    rng = np.random.default_rng(seed)
    d, L = cfg["n_embd"], cfg["n_layer"]
    host = {}

    def normal(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32)

    host["transformer.wte.weight"] = normal(cfg["vocab_size"], d)
    host["transformer.wpe.weight"] = normal(cfg["n_positions"], d)
    for i in range(L):
        p = f"transformer.h.{i}"
        host[f"{p}.ln_1.weight"] = np.ones(d, np.float32)
        host[f"{p}.ln_1.bias"] = np.zeros(d, np.float32)
        host[f"{p}.attn.c_attn.weight"] = normal(d, 3 * d)
        host[f"{p}.attn.c_attn.bias"] = np.zeros(3 * d, np.float32)
        host[f"{p}.attn.c_proj.weight"] = normal(d, d)
        host[f"{p}.attn.c_proj.bias"] = np.zeros(d, np.float32)
        host[f"{p}.ln_2.weight"] = np.ones(d, np.float32)
        host[f"{p}.ln_2.bias"] = np.zeros(d, np.float32)
        host[f"{p}.mlp.c_fc.weight"] = normal(d, 4 * d)
        host[f"{p}.mlp.c_fc.bias"] = np.zeros(4 * d, np.float32)
        host[f"{p}.mlp.c_proj.weight"] = normal(4 * d, d)
        host[f"{p}.mlp.c_proj.bias"] = np.zeros(d, np.float32)
    host["transformer.ln_f.weight"] = np.ones(d, np.float32)
    host["transformer.ln_f.bias"] = np.zeros(d, np.float32)
    return load_gpt2_state_dict(host, cfg, dtype=dtype)


def load_gpt2_state_dict(state, config, dtype="float32", fold_layer_norms=True):
    """Uploads a {name: numpy / torch array} state dict (HF GPT-2 names). Returns the model dict
    the reference's `load_gpt2_weights` returns: {"weights": {...GpuTensor}, "config": {...}}. 16-bit models also get the
    layer_norm-folded copies of c_attn / c_fc that the prefill path uses (fold_gpt2_layer_norms; `fold_layer_norms=False`
    or APPLEGPU_LN_FOLD=0 keeps every layer_norm a kernel)."""
    weights = {}
    for name, arr in state.items():
        if name.endswith(".attn.bias") or name.endswith(".attn.masked_bias") or name == "lm_head.weight":
            continue  # causal-mask buffers and the tied head are not parameters of the forward
        if hasattr(arr, "detach"):
            arr = arr.detach().cpu().float().numpy()
        t = gpu.from_numpy(np.ascontiguousarray(arr, dtype=np.float32))
        if dtype != "float32":
            t = gpu.cast(t, dtype)
            t.eval()
        weights[name] = t
    model = {"weights": weights, "config": dict(config), "dtype": dtype}
    if fold_layer_norms and dtype != "float32" and "transformer.h.0.ln_1.weight" in weights and os.environ.get("APPLEGPU_LN_FOLD", "1") != "0":
        fold_gpt2_layer_norms(model)
    return model


def quantize_gpt2_linears(model):
    """Per-output-channel symmetric int8 for every linear weight (activations keep the model
    dtype). Weights are stored [N, K] (K-major) so the GEMM reads them as they lie."""
    w = model["weights"]
    q = {}
    for name, t in w.items():
        if name.endswith((".c_attn.weight", ".c_fc.weight", ".c_proj.weight")):
            wt = gpu.transpose(t)           # [out, in] view
            wt = gpu.reshape(wt, wt.shape)  # materialise [N, K] contiguous
            q[name] = gpu.quantize_weight(wt)
    model["int8"] = q
    model.pop("ln_fold", None)   # the folded copies are not quantised: the int8 path keeps its layer_norm kernels
    return model


def fold_gpt2_layer_norms(model):
    """Folds ln_1 / ln_2 of every block into the linear that follows it, for the prefill path of 16-bit models.

    layer_norm(x) @ W + b = rstd * (x @ W' - mean * s) + c with W' = gamma[:, None] * W, s = W'.sum(0) and
    c = beta @ W + b: the product runs on the un-normalised residual stream, the row statistics (sum and sum of squares
    over the 768 features, accumulated in fixed point with integer atomics so that the order of addition cannot change
    a bit) come from the epilogue of the GEMM that produced the stream (the attention output projection and the second
    feed-forward matrix, which add the residual), and the correction is two packed operations per two elements in the
    consumer's epilogue (api.linear_fused). 23 of the 25 layer_norm launches of a GPT-2-small forward disappear;
    block 0's ln_1 (its input comes from the embeddings) and ln_f stay kernels. s is summed from the rounded W' the GEMM
    multiplies with, so mean * s cancels exactly what the product accumulated."""
    if model.get("dtype", "float32") == "float32" or "int8" in model:
        return model
    w = model["weights"]
    cfg = model["config"]
    dtype = model["dtype"]
    fold = {}
    # Both layouts of the three weights whose best tile depends on it are kept (127 MB more for GPT-2-small): [K, N] for the
    # chained form (out-projection -> FC1 -> FC2 -> the next block's QKV as one launch, where tile shapes stop
    # mattering), and K-major copies for separate launches (see _kmajor_copy). The forward picks by its row count.
    for i in range(cfg["n_layer"]):
        p = f"transformer.h.{i}"
        for ln, lin in ((f"{p}.ln_1", f"{p}.attn.c_attn"), (f"{p}.ln_2", f"{p}.mlp.c_fc")):
            gamma = w[f"{ln}.weight"].to_numpy().astype(np.float32)
            beta = w[f"{ln}.bias"].to_numpy().astype(np.float32)
            w0 = w[f"{lin}.weight"].to_numpy().astype(np.float32)          # [K, N], the values the plain path multiplies with
            b0 = w[f"{lin}.bias"].to_numpy().astype(np.float32)
            wf = gpu.cast(gpu.from_numpy(np.ascontiguousarray(gamma[:, None] * w0)), dtype)
            wf.eval()
            colsum = gpu.from_numpy(wf.to_numpy().astype(np.float64).sum(0).astype(np.float32))
            cbias = gpu.cast(gpu.from_numpy((beta.astype(np.float64) @ w0.astype(np.float64) + b0).astype(np.float32)), dtype)
            cbias.eval()
            fold[lin] = (wf, colsum, cbias)
            if lin.endswith(".mlp.c_fc"):
                fold[lin + ".kmajor"] = _kmajor_copy(wf)          # stored [N, K]; the forward takes the transposed view
        # the two projections back to the 768-wide stream: N = 768 fills the 74 CTA pairs of the GEMM in 1.73 waves of
        # 256 x 192 tiles, a shape the kernel has for K-major weights only
        for lin in (f"{p}.attn.c_proj", f"{p}.mlp.c_proj"):
            fold[lin] = w[f"{lin}.weight"]
            fold[lin + ".kmajor"] = _kmajor_copy(w[f"{lin}.weight"])
    model["ln_fold"] = fold
    model["_ln_stats"] = {}
    return model


def _kmajor_copy(w):
    """A contiguous [N, K] copy of the [K, N] weight `w`: the same values stored K-major (what the tied LM head already
    is), for which the GEMM has its 256 x 192 CTA-pair tile. The forward multiplies with gpu.transpose(copy), a view."""
    wt = gpu.transpose(w)
    wt = gpu.reshape(wt, wt.shape)   # materialise [N, K] contiguous
    wt.eval()
    return wt


def _row_stats(model, rows):
    """Two zeroed [rows, 2] int64 tensors per row count: the running fixed-point (sum, sum of squares) of the residual
    stream's rows for ln_1 and ln_2. Each is cleared by the GEMM that runs before the one that fills it (stats_zero),
    and block 0 clears both, so a forward always starts from zeros whatever an interrupted one left behind."""
    pair = model["_ln_stats"].get(rows)
    if pair is None:
        pair = (gpu.from_numpy(np.zeros((rows, 2), np.int64)), gpu.from_numpy(np.zeros((rows, 2), np.int64)))
        model["_ln_stats"][rows] = pair
    return pair


def _linear(x, w, name, bias):
    q = w.get("__int8__", {}).get(name)
    if q is not None:
        y = gpu.matmul_int8(x, q[0], q[1])
    else:
        y = x @ w[name]
    return gpu.add_bias(y, bias)


def gpt2_forward(model, input_ids, kv_cache=None, last_only=False, device_ids=None, compiled=False):
    """GPT-2 forward with optional KV cache.

    input_ids: list of ints (the reference's form, batch 1) or an int array [B, T]. With a cache
    only the last token of each sequence is processed. Returns (logits, new_kv_cache); logits are
    [T, vocab] for list input (as upstream) or [B, T, vocab] for array input; with `last_only`
    only the final position goes through the LM head ([B, vocab]). `device_ids` = (token ids,
    position ids) as int32 GpuTensors of length B*T skips the host-to-device copy of the ids;
    `input_ids` then only supplies the [B, T] shape. `compiled=True` records the op sequence once per
    (batch, new tokens, cache / no cache) on an op tape and replays it on later calls: one library
    call per forward instead of one per op (shapes are re-inferred, so the tape taken at one KV length
    serves the next).
    """
    w = dict(model["weights"])
    if "int8" in model:
        w["__int8__"] = model["int8"]
    if "ln_fold" in model and kv_cache is None and np.asarray(input_ids).size >= 64 and "int8" not in model:
        w["__ln_fold__"] = model["ln_fold"]
        w["__ln_stats__"] = _row_stats(model, int(np.asarray(input_ids).size))
    cfg = model["config"]
    n_layer, n_head, n_embd = cfg["n_layer"], cfg["n_head"], cfg["n_embd"]
    d_head = n_embd // n_head

    ids = np.asarray(input_ids, dtype=np.int64)
    batched = ids.ndim == 2
    if not batched:
        ids = ids.reshape(1, -1)
    B = ids.shape[0]
    use_cache = kv_cache is not None
    if use_cache:
        tok = ids[:, -1:]
        pos_offset = ids.shape[1] - 1
    else:
        tok = ids
        pos_offset = 0
    T = tok.shape[1]
    rows = B * T

    if device_ids is not None:
        # token / position indices already resident on the device (int32 [B*T] each)
        indices, pos_indices = device_ids
    else:
        indices = gpu.from_numpy(np.ascontiguousarray(tok.reshape(-1), dtype=np.int32))
        pos = np.tile(np.arange(pos_offset, pos_offset + T, dtype=np.int32), B)
        pos_indices = gpu.from_numpy(pos)

    tape_key = tape_inputs = None
    if compiled:
        tape_key = ("gpt2", B, T, use_cache, bool(last_only), batched, "int8" in model, "__ln_fold__" in w, gpu.gemm_chain_applies(B * T))
        tape_inputs = [indices, pos_indices] + ([t for kv in kv_cache for t in kv] if use_cache else [])
        tape = model.setdefault("_tapes", {}).get(tape_key)
        if tape is not None:
            out = tape.replay(tape_inputs)
            return out[0], [(out[1 + 2 * i], out[2 + 2 * i]) for i in range(n_layer)]
        gpu.tape_begin(tape_inputs)
    try:
        logits, new_kv_cache = _record_forward(w, cfg, indices, pos_indices, kv_cache, B, T, last_only, batched)
    except Exception:
        if compiled:
            gpu.tape_abort()
        raise
    if compiled:
        model["_tapes"][tape_key] = gpu.tape_end(len(tape_inputs), [logits] + [t for kv in new_kv_cache for t in kv])
    return logits, new_kv_cache


def _record_forward(w, cfg, indices, pos_indices, kv_cache, B, T, last_only, batched):
    """Issues the ops of one forward (the body the reference's gpt2_forward runs per call)."""
    n_layer, n_head, n_embd = cfg["n_layer"], cfg["n_head"], cfg["n_embd"]
    d_head = n_embd // n_head
    rows = B * T
    use_cache = kv_cache is not None
    tok_emb = gpu.embedding(w["transformer.wte.weight"], indices)
    pos_emb = gpu.embedding(w["transformer.wpe.weight"], pos_indices)
    x = tok_emb + pos_emb  # [B*T, d]

    fold = w.get("__ln_fold__")
    chained = gpu.gemm_chain_applies(rows)                   # the block's linears will go out as one launch
    stats1, stats2 = w.get("__ln_stats__", (None, None))     # row statistics feeding ln_1 / ln_2
    new_kv_cache = []
    for i in range(n_layer):
        p = f"transformer.h.{i}"
        if fold is None:
            x_norm = gpu.layer_norm(x, w[f"{p}.ln_1.weight"], w[f"{p}.ln_1.bias"])
            qkv = _linear(x_norm, w, f"{p}.attn.c_attn.weight", w[f"{p}.attn.c_attn.bias"])
        elif i == 0:
            # the stream comes from the embeddings here: a layer_norm kernel, and the projection clears ln_2's statistics
            x_norm = gpu.layer_norm(x, w[f"{p}.ln_1.weight"], w[f"{p}.ln_1.bias"])
            qkv = gpu.linear_fused(x_norm, w[f"{p}.attn.c_attn.weight"], bias=w[f"{p}.attn.c_attn.bias"], stats_zero=stats2)
        else:
            wf, colsum, cbias = fold[f"{p}.attn.c_attn"]
            qkv = gpu.linear_fused(x, wf, bias=cbias, ln=(colsum, stats1, 1e-5))

        q_all = gpu.slice(qkv, dim=1, start=0, end=n_embd)
        k_new = gpu.slice(qkv, dim=1, start=n_embd, end=2 * n_embd)
        v_new = gpu.slice(qkv, dim=1, start=2 * n_embd, end=3 * n_embd)

        def heads(t):
            t = gpu.reshape(t, [B, T, n_head, d_head])
            return gpu.transpose_dims(t, 1, 2)  # [B, n_head, T, d_head]

        q, k, v = heads(q_all), heads(k_new), heads(v_new)
        if use_cache:
            ck, cv = kv_cache[i]
            k = gpu.concat(ck, k, dim=2)
            v = gpu.concat(cv, v, dim=2)
        new_kv_cache.append((k, v))

        attn = gpu.attention(q, k, v) if use_cache else gpu.attention_causal(q, k, v)
        attn = gpu.transpose_dims(attn, 1, 2)        # [B, T, n_head, d_head]
        attn = gpu.reshape(attn, [rows, n_embd])

        if fold is None:
            attn = _linear(attn, w, f"{p}.attn.c_proj.weight", w[f"{p}.attn.c_proj.bias"])
            x = x + attn

            x_norm2 = gpu.layer_norm(x, w[f"{p}.ln_2.weight"], w[f"{p}.ln_2.bias"])
            ffn = _linear(x_norm2, w, f"{p}.mlp.c_fc.weight", w[f"{p}.mlp.c_fc.bias"])
            ffn = gpu.gelu(ffn)
            ffn = _linear(ffn, w, f"{p}.mlp.c_proj.weight", w[f"{p}.mlp.c_proj.bias"])
            x = x + ffn
        else:
            # x += attn @ W + b, and ln_2's row statistics of the new x; ln_1's (already consumed) are cleared
            # chained (enough rows): the [K, N] weights; separate launches: the K-major copies through transposed views
            def weight(name):
                return fold[name] if chained else gpu.transpose(fold[name + ".kmajor"])
            x = gpu.linear_fused(attn, weight(f"{p}.attn.c_proj"), bias=w[f"{p}.attn.c_proj.bias"], residual=x, stats_out=stats2, stats_zero=stats1)
            _, colsum, cbias = fold[f"{p}.mlp.c_fc"]
            wf = fold[f"{p}.mlp.c_fc"][0] if chained else gpu.transpose(fold[f"{p}.mlp.c_fc.kmajor"])
            ffn = gpu.linear_fused(x, wf, bias=cbias, act="gelu", ln=(colsum, stats2, 1e-5))
            # x += ffn @ W + b, ln_1's statistics for the next block (none after the last: ln_f is a kernel), ln_2's cleared
            x = gpu.linear_fused(ffn, weight(f"{p}.mlp.c_proj"), bias=w[f"{p}.mlp.c_proj.bias"], residual=x,
                                 stats_out=stats1 if i + 1 < n_layer else None, stats_zero=stats2)

    x = gpu.layer_norm(x, w["transformer.ln_f.weight"], w["transformer.ln_f.bias"])
    if last_only:
        x = gpu.reshape(x, [B, T, n_embd])
        x = gpu.slice(x, dim=1, start=T - 1, end=T)
        x = gpu.reshape(x, [B, n_embd])
    lm_head_w = gpu.transpose(w["transformer.wte.weight"])  # a view; the GEMM reads wte K-major
    logits = x @ lm_head_w
    if last_only:
        return logits, new_kv_cache
    if batched:
        logits = gpu.reshape(logits, [B, T, cfg["vocab_size"]])
    return logits, new_kv_cache
