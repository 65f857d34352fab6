"""Whole-model timings for the benchmark configurations other than the headline one.

Counterpart of the reference's model-level benchmark scripts (python/tests/bench_comparison.py:23-50
times a forward against PyTorch CPU; benchmarks/bench_mlp_cpp.py:30-79 the MLP). Each line is one
configuration on synthetic seeded inputs (N(0, 0.02) weights, uniform token ids), timed with CUDA
events on the runtime stream after warm-up:

  gpt2_small_prefill   GPT-2-small forward, batch 8 x 128 and 8 x 1024 tokens (bf16 or fp32)
  gpt2_small_decode    8 prompts x 64 tokens, then 50 greedy steps with the KV cache (tokens/s = 8*50/time)
  gpt2_large_int8      GPT-2-large, per-output-channel int8 weights, bf16 activations, 32 x 512 tokens
  bert_base            BERT-base encoder, 256 x 512 tokens, bf16
  bert_base_tp         the same, heads / feed-forward units sharded over the ranks of a torchrun launch (NCCL)
  gpt2_large_int8_sharded, bert_base_sharded   the batch of those configurations split over the ranks of a torchrun launch

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
        gpt2_forward(model, ids, compiled=True)[0].eval()   # op tape: recorded by the first warm-up call, replayed after

    ms = _time(step, iters, 2)
    flops = batch * seq * (_gemm_flops_per_token(GPT2_LARGE) + 4 * seq * GPT2_LARGE["n_embd"] * GPT2_LARGE["n_layer"])
    return {"config": "gpt2_large_int8", "dtype": "bfloat16 activations, int8 weights", "batch": batch, "seq": seq, "ms": ms,
            "tokens_per_s": batch * seq / ms * 1e3, "tflops": flops / ms / 1e9}


def bench_bert_base(dtype, batch, seq, iters):
    model = init_bert_weights(BERT_BASE, seed=0, dtype=dtype)
    ids = np.random.default_rng(3).integers(0, BERT_BASE["vocab_size"], (batch, seq))

    def step():
        bert_forward(model, ids, compiled=True).eval()   # op tape: recorded by the first warm-up call

    ms = _time(step, iters, 2)
    flops = batch * seq * (_gemm_flops_per_token(BERT_BASE, BERT_BASE["d_ff"], lm_head=False) + 4 * seq * BERT_BASE["n_embd"] * BERT_BASE["n_layer"])
    return {"config": "bert_base", "dtype": dtype, "batch": batch, "seq": seq, "ms": ms, "tokens_per_s": batch * seq / ms * 1e3,
            "tflops": flops / ms / 1e9}


def _bert_host_state(cfg, seed=0, std=0.02):
    rng = np.random.default_rng(seed)
    d, L, ff = cfg["n_embd"], cfg["n_layer"], cfg["d_ff"]
    st = {}

    def normal(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32)

    st["embeddings.word_embeddings.weight"] = normal(cfg["vocab_size"], d)
    st["embeddings.position_embeddings.weight"] = normal(cfg["n_positions"], d)
    st["embeddings.token_type_embeddings.weight"] = normal(cfg.get("type_vocab", 2), d)
    st["embeddings.LayerNorm.weight"] = np.ones(d, np.float32); st["embeddings.LayerNorm.bias"] = np.zeros(d, np.float32)
    for i in range(L):
        p = f"encoder.layer.{i}"
        for name, shape in (("attention.self.query", (d, d)), ("attention.self.key", (d, d)), ("attention.self.value", (d, d)),
                            ("attention.output.dense", (d, d)), ("intermediate.dense", (ff, d)), ("output.dense", (d, ff))):
            st[f"{p}.{name}.weight"] = normal(*shape); st[f"{p}.{name}.bias"] = np.zeros(shape[0], np.float32)
        for name in ("attention.output.LayerNorm", "output.LayerNorm"):
            st[f"{p}.{name}.weight"] = np.ones(d, np.float32); st[f"{p}.{name}.bias"] = np.zeros(d, np.float32)
    return st


def bench_bert_base_tp(dtype, batch, seq, iters):
    """BERT-base with heads and feed-forward units sharded over the launcher's ranks (torchrun, one rank per
    GPU): 2 NCCL all-reduces of [batch*seq, 768] per layer, timed both serialised on the runtime stream and overlapped
    with the next micro-batch's compute (bert_forward_overlapped). Rank 0 prints the line; times are the MAX over ranks
    of the CUDA-event time."""
    from .sharding import RankGroup
    from .tp import TensorParallelGroup, load_bert_shard
    group = RankGroup.from_env()
    tp = TensorParallelGroup(group)
    model = load_bert_shard(_bert_host_state(BERT_BASE), BERT_BASE, group, dtype=dtype)
    ids = np.random.default_rng(3).integers(0, BERT_BASE["vocab_size"], (batch, seq))

    from .bert import bert_forward_overlapped
    micro = 2

    def step_serial():
        bert_forward(model, ids, all_reduce=tp.all_reduce).eval()

    def step_overlapped():
        for out in bert_forward_overlapped(model, ids, tp, micro_batches=micro):
            out.eval()

    group.barrier()
    ms_serial = group.max(_time(step_serial, iters, 2))
    group.barrier()
    ms = group.max(_time(step_overlapped, iters, 2))
    group.barrier()
    payload = batch * seq * BERT_BASE["n_embd"] * gpu.dtype_size(dtype)
    r = {"config": "bert_base_tp", "dtype": dtype, "batch": batch, "seq": seq, "ranks": group.world, "ms": ms, "micro_batches": micro,
         "ms_all_reduce_on_runtime_stream": ms_serial,
         "tokens_per_s": batch * seq / ms * 1e3, "all_reduce_bytes": payload, "all_reduces_per_forward": 2 * BERT_BASE["n_layer"]}
    rank = group.rank
    group.close()
    return r if rank == 0 else None


def bench_batch_sharded(config, dtype, iters):
    """gpt2_large_int8 or bert_base with the batch split over the launcher's ranks (torchrun, one rank per GPU): no
    data-path collective, every rank runs the single-GPU forward on batch / world sequences. The time is the MAX
    over ranks of the CUDA-event time; tokens/s counts every rank's tokens. Rank 0 returns the line."""
    from .sharding import RankGroup, shard_range
    group = RankGroup.from_env()
    full = 32 if config == "gpt2_large_int8" else 256
    lo, hi = shard_range(full, group.rank, group.world)
    local = hi - lo
    group.barrier()
    r = bench_gpt2_large_int8(local, 512, iters) if config == "gpt2_large_int8" else bench_bert_base(dtype, local, 512, iters)
    ms = group.max(r["ms"])
    group.barrier()
    out = {"config": config + "_batch_sharded", "dtype": r["dtype"], "ranks": group.world, "global_batch": full, "batch_per_rank": local, "seq": 512,
           "ms": ms, "tokens_per_s": full * 512 / ms * 1e3, "tflops": r["tflops"] * r["ms"] / ms * full / local}
    rank = group.rank
    group.close()
    return out if rank == 0 else None


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all", choices=["all", "gpt2_small_prefill", "gpt2_small_decode", "gpt2_large_int8", "bert_base", "bert_base_tp", "gpt2_large_int8_sharded", "bert_base_sharded"])
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
    if args.config in ("gpt2_large_int8_sharded", "bert_base_sharded"):   # under torchrun: one rank per GPU
        r = bench_batch_sharded(args.config[:-len("_sharded")], args.dtype, max(1, args.iters // 2))
        if r is not None:
            emit(r)
    if args.config == "bert_base_tp":   # under torchrun: one rank per GPU
        r = bench_bert_base_tp(args.dtype, 256, 512, max(1, args.iters // 2))
        if r is not None:
            emit(r)
    st = gpu.pipeline_status()
    if st:
        print(json.dumps({"pipeline_status": st}))
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
