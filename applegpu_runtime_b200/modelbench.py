"""Whole-model timings for the benchmark configurations other than the headline one.

Counterpart of the reference's model-level benchmark scripts (python/tests/bench_comparison.py:23-50
times a forward against PyTorch CPU; benchmarks/bench_mlp_cpp.py:30-79 the MLP). Each line is one
configuration on synthetic seeded inputs (N(0, 0.02) weights, uniform token ids), timed with CUDA
events on the runtime stream after warm-up:

  gpt2_small_prefill   GPT-2-small forward, batch 8 x 128 and 8 x 1024 tokens (bf16 or fp32)
  gpt2_small_decode    8 prompts x 64 tokens, then 50 greedy steps with the KV cache (tokens/s = 8*50/time)
  gpt2_large_int8      GPT-2-large, per-output-channel int8 weights, bf16 activations, 32 x 512 tokens
  bert_base            BERT-base encoder, 256 x 512 tokens, bf16

  python -m applegpu_runtime_b200.modelbench --config all --dtype bfloat16
"""
import argparse
import json
import sys

import numpy as np

from . import _lib
from . import api as gpu
from .bert import BERT_BASE, bert_forward, init_bert_weights
from .generate import greedy_generate
from .gpt2 import GPT2_LARGE, GPT2_SMALL, gpt2_forward, init_gpt2_weights, quantize_gpt2_linears


def _time(fn, iters, warmup):
    lib = _lib.load()
    for _ in range(warmup):
        fn()
    gpu.synchronize()
    lib.applegpu_timer_start()
    for _ in range(iters):
        fn()
    return float(lib.applegpu_timer_stop_ms()) / iters


def _gemm_flops_per_token(cfg, d_ff=None, lm_head=True):
    d, L = cfg["n_embd"], cfg["n_layer"]
    ff = d_ff if d_ff is not None else 4 * d
    per_layer = 2 * (d * 3 * d + d * d + 2 * d * ff)
    return L * per_layer + (2 * d * cfg["vocab_size"] if lm_head else 0)


def bench_prefill(dtype, batch, seq, iters):
    model = init_gpt2_weights(GPT2_SMALL, seed=0, dtype=dtype)
    ids = np.random.default_rng(0).integers(0, GPT2_SMALL["vocab_size"], (batch, seq))

    def step():
        gpt2_forward(model, ids, compiled=True)[0].eval()   # op tape: recorded by the first warm-up call, replayed after

    ms = _time(step, iters, 3)
    flops = batch * seq * (_gemm_flops_per_token(GPT2_SMALL) + 4 * seq * GPT2_SMALL["n_embd"] * GPT2_SMALL["n_layer"])
    return {"config": "gpt2_small_prefill", "dtype": dtype, "batch": batch, "seq": seq, "ms": ms, "tokens_per_s": batch * seq / ms * 1e3,
            "tflops": flops / ms / 1e9}


def bench_decode(dtype, batch, prompt, steps, iters):
    model = init_gpt2_weights(GPT2_SMALL, seed=0, dtype=dtype)
    ids = np.random.default_rng(1).integers(0, GPT2_SMALL["vocab_size"], (batch, prompt))
    import time
    greedy_generate(model, ids, max_tokens=4, use_cache=True)      # warm-up: pool, tensor maps
    gpu.synchronize()
    best = None
    for _ in range(iters):
        t0 = time.perf_counter()
        out = greedy_generate(model, ids, max_tokens=steps, use_cache=True)   # reads every step's tokens on the host
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    assert out.shape == (batch, prompt + steps)
    weight_bytes = 124.4e6 * gpu.dtype_size(dtype)
    return {"config": "gpt2_small_decode", "dtype": dtype, "batch": batch, "prompt": prompt, "steps": steps, "ms": best * 1e3,
            "ms_per_step": best * 1e3 / steps, "tokens_per_s": batch * steps / best,
            "weight_stream_gbs": weight_bytes * steps / best / 1e9, "note": "wall clock: includes the prefill of the prompt, host sampling and graph recording"}


def bench_gpt2_large_int8(batch, seq, iters):
    model = quantize_gpt2_linears(init_gpt2_weights(GPT2_LARGE, seed=0, dtype="bfloat16"))
    # the 16-bit copies of the quantised matrices are not used by the forward any more
    for name in list(model["weights"]):
        if name.endswith((".c_attn.weight", ".c_fc.weight", ".c_proj.weight")):
            del model["weights"][name]
    ids = np.random.default_rng(2).integers(0, GPT2_LARGE["vocab_size"], (batch, seq))

    def step():
        gpt2_forward(model, ids)[0].eval()

    ms = _time(step, iters, 2)
    flops = batch * seq * (_gemm_flops_per_token(GPT2_LARGE) + 4 * seq * GPT2_LARGE["n_embd"] * GPT2_LARGE["n_layer"])
    return {"config": "gpt2_large_int8", "dtype": "bfloat16 activations, int8 weights", "batch": batch, "seq": seq, "ms": ms,
            "tokens_per_s": batch * seq / ms * 1e3, "tflops": flops / ms / 1e9}


def bench_bert_base(dtype, batch, seq, iters):
    model = init_bert_weights(BERT_BASE, seed=0, dtype=dtype)
    ids = np.random.default_rng(3).integers(0, BERT_BASE["vocab_size"], (batch, seq))

    def step():
        bert_forward(model, ids).eval()

    ms = _time(step, iters, 2)
    flops = batch * seq * (_gemm_flops_per_token(BERT_BASE, BERT_BASE["d_ff"], lm_head=False) + 4 * seq * BERT_BASE["n_embd"] * BERT_BASE["n_layer"])
    return {"config": "bert_base", "dtype": dtype, "batch": batch, "seq": seq, "ms": ms, "tokens_per_s": batch * seq / ms * 1e3,
            "tflops": flops / ms / 1e9}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all", choices=["all", "gpt2_small_prefill", "gpt2_small_decode", "gpt2_large_int8", "bert_base"])
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    gpu.init_backend()
    out = []

    def emit(r):
        out.append(r)
        print(json.dumps(r), flush=True)

    if args.config in ("all", "gpt2_small_prefill"):
        emit(bench_prefill(args.dtype, 8, 128, args.iters))
        emit(bench_prefill(args.dtype, 8, 1024, args.iters))
    if args.config in ("all", "gpt2_small_decode"):
        emit(bench_decode(args.dtype, 8, 64, 50, max(1, args.iters // 2)))
    if args.config in ("all", "gpt2_large_int8"):
        emit(bench_gpt2_large_int8(32, 512, max(1, args.iters // 2)))
    if args.config in ("all", "bert_base"):
        emit(bench_bert_base(args.dtype, 256, 512, max(1, args.iters // 2)))
    st = gpu.pipeline_status()
    if st:
        print(json.dumps({"pipeline_status": st}))
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
