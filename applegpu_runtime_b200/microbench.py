"""Per-op microbenchmarks (the op microbench config of the headline benchmark, and the tool the
ncu captures under profiles/ are taken with).

Counterpart of the reference's benchmarks/bench_ops.py:23-39,122-142 (median of repeated launches
per op). Shapes default to the benchmark config: batched matmul B=8 with M=N=K in {1024, 2048, 4096};
layer_norm [8192, 768]; softmax_causal [96, 1024, 1024]; gelu+add_bias [8192, 3072]; plus the GEMM
and attention shapes of a GPT-2-small forward. Each line reports the CUDA-event time per launch,
the algorithmic work (flops for contractions, bytes otherwise) and the achieved rate. By default launches run back to back inside one event pair and cycle through
enough buffer sets (inputs and outputs) that no launch finds its data in the 126 MB L2.

  python -m applegpu_runtime_b200.microbench                      all ops, bf16 and fp32
  python -m applegpu_runtime_b200.microbench --op matmul --shape 8,4096,4096,4096 --dtype bfloat16 --iters 3
"""
import argparse
import ctypes
import json
import sys

import numpy as np

from . import _lib
from . import api as gpu


def _tensor(rng, shape, dtype, scale=1.0):
    t = gpu.from_numpy(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale))
    if dtype != "float32":
        t = gpu.cast(t, dtype)
        t.eval()
    return t


L2_BYTES = 126 << 20


def _nsets(footprint_bytes, rotate):
    """Buffer sets to cycle through so that consecutive launches never find their data in L2."""
    if not rotate:
        return 1
    return int(max(1, min(8, -(-2 * L2_BYTES // max(1, int(footprint_bytes))))))


def _time(fns, iters, warmup=3, single=False):
    """CUDA-event time per launch on the runtime stream. Default: one event pair around `iters`
    back-to-back launches cycling through the buffer sets in `fns` (outputs of the last len(fns)
    launches are kept alive so the pool rotates output buffers too). `single`: median of
    individually timed launches (includes launch latency)."""
    import collections
    lib = _lib.load()
    keep = collections.deque(maxlen=len(fns))
    for i in range(max(warmup, 2 * len(fns) + 2)):  # long enough for the pool to reach its steady set of buffers
        o = fns[i % len(fns)](); o.eval(); keep.append(o)
    gpu.synchronize()
    if single:
        times = []
        for i in range(iters):
            lib.applegpu_timer_start()
            o = fns[i % len(fns)](); o.eval(); keep.append(o)
            times.append(float(lib.applegpu_timer_stop_ms()))
        return float(np.median(times))
    # The timed loop replays each op from a tape (one library call instead of the Python-side recording), so that
    # the host keeps ahead of kernels of a few microseconds; ops that cannot be taped are issued as above.
    tapes = []
    for fn in fns:
        try:
            n = gpu.tape_begin([])
            try:
                out = fn()
                tape = gpu.tape_end(n, [out])
            except Exception:
                gpu.tape_abort()
                raise
            out.eval(); keep.append(out)
            tapes.append(tape)
        except Exception:
            tapes = None
            break
    if tapes:
        # the whole timed loop is one library call (applegpu_ffi_tape_replay_loop): the host cost per launch stays far
        # below the run time of even the smallest kernel here
        arr = (ctypes.c_uint64 * len(tapes))(*[t.handle for t in tapes])
        if lib.applegpu_ffi_tape_replay_loop(arr, len(tapes), 2 * len(tapes) + 2, len(tapes)) != 0:
            raise RuntimeError(lib.applegpu_ffi_last_error())
        gpu.synchronize()
        lib.applegpu_timer_start()
        if lib.applegpu_ffi_tape_replay_loop(arr, len(tapes), iters, len(tapes)) != 0:
            raise RuntimeError(lib.applegpu_ffi_last_error())
        return float(lib.applegpu_timer_stop_ms()) / iters
    gpu.synchronize()
    lib.applegpu_timer_start()
    for i in range(iters):
        o = fns[i % len(fns)](); o.eval(); keep.append(o)
    return float(lib.applegpu_timer_stop_ms()) / iters


def bench_matmul(rng, dtype, b, m, n, k, iters, opt):
    e = gpu.dtype_size(dtype)
    sets = []
    for _ in range(_nsets((b * m * k + b * k * n + b * m * n) * e, opt.rotate)):
        a = _tensor(rng, (b, m, k) if b > 1 else (m, k), dtype)
        w = _tensor(rng, (b, k, n) if b > 1 else (k, n), dtype)
        sets.append((a, w))
    ms = _time([lambda a=a, w=w: a @ w for a, w in sets], iters, single=opt.single)
    flops = 2.0 * b * m * n * k
    return {"op": "matmul", "dtype": dtype, "shape": [b, m, n, k], "ms": ms, "work": flops, "rate": flops / ms / 1e9, "unit": "TFLOP/s", "sets": len(sets)}


def bench_fused_linear(rng, dtype, m, n, k, act, residual, iters, opt, kmajor=False):
    """x @ W + b, then GELU or a residual add: one fused_linear launch (the four linears of a GPT-2 layer). `kmajor`:
    the weight is stored [n, k] and read through a transposed view."""
    e = gpu.dtype_size(dtype)
    sets = []
    for _ in range(_nsets((m * k + k * n + (2 if residual else 1) * m * n) * e, opt.rotate)):
        w = gpu.transpose(_tensor(rng, (n, k), dtype, 0.02)) if kmajor else _tensor(rng, (k, n), dtype, 0.02)
        sets.append((_tensor(rng, (m, k), dtype), w, _tensor(rng, (m, n), dtype) if residual else None))
    bias = _tensor(rng, (n,), dtype)

    def make(x, w, r):
        def fn():
            y = gpu.add_bias(x @ w, bias)
            if act:
                y = gpu.gelu_exact(y) if act == "erf" else gpu.gelu(y)
            return r + y if r is not None else y
        return fn

    ms = _time([make(*t) for t in sets], iters, single=opt.single)
    flops = 2.0 * m * n * k
    name = "fused_linear[bias" + (",gelu_erf" if act == "erf" else ",gelu" if act else "") + (",residual" if residual else "") + "]" + (" (B K-major)" if kmajor else "")
    return {"op": name, "dtype": dtype, "shape": [m, n, k], "ms": ms, "work": flops, "rate": flops / ms / 1e9, "unit": "TFLOP/s", "sets": len(sets)}


def bench_layer_linears(rng, dtype, rows, d, iters, opt, chained=True):
    """The four linears between two attention kernels of a GPT-2 block with folded layer_norms, as the model issues them
    (gpt2._record_forward): out-projection (+ residual, row statistics out), FC1 (folded ln_2, GELU), FC2 (+ residual,
    row statistics out) and the next block's QKV (folded ln_1), [K, N] weights, one evaluation. `chained`: one launch of
    the chained tensor-core kernel; otherwise four launches."""
    e = gpu.dtype_size(dtype)
    was = gpu.gemm_chain_enabled()
    gpu.set_gemm_chain(bool(chained))
    try:
        footprint = (rows * d * 4 + rows * 4 * d + rows * 3 * d + 12 * d * d) * e
        sets = []
        for _ in range(_nsets(footprint, opt.rotate)):
            attn, x = _tensor(rng, (rows, d), dtype), _tensor(rng, (rows, d), dtype)
            w = [_tensor(rng, (d, d), dtype, 0.02), _tensor(rng, (d, 4 * d), dtype, 0.02), _tensor(rng, (4 * d, d), dtype, 0.02), _tensor(rng, (d, 3 * d), dtype, 0.02)]
            b = [_tensor(rng, (n,), dtype) for n in (d, 4 * d, d, 3 * d)]
            cs = [gpu.from_numpy(np.zeros(n, np.float32)) for n in (4 * d, 3 * d)]
            st = [gpu.from_numpy(np.zeros((rows, 2), np.int64)) for _ in range(2)]
            for t in cs + st:
                t.eval()
            sets.append((attn, x, w, b, cs, st))

        def make(attn, x, w, b, cs, st):
            def fn():
                x2 = gpu.linear_fused(attn, w[0], bias=b[0], residual=x, stats_out=st[1], stats_zero=st[0])
                ff = gpu.linear_fused(x2, w[1], bias=b[1], act="gelu", ln=(cs[0], st[1], 1e-5))
                x3 = gpu.linear_fused(ff, w[2], bias=b[2], residual=x2, stats_out=st[0], stats_zero=st[1])
                return gpu.linear_fused(x3, w[3], bias=b[3], ln=(cs[1], st[0], 1e-5))
            return fn

        ms = _time([make(*t) for t in sets], iters, single=opt.single)
    finally:
        gpu.set_gemm_chain(was)
    flops = 2.0 * rows * d * d * 12
    name = "gpt2 block linears [out-proj, FC1, FC2, next QKV], " + ("chained: one launch" if chained else "four launches")
    return {"op": name, "dtype": dtype, "shape": [rows, d], "ms": ms, "work": flops, "rate": flops / ms / 1e9, "unit": "TFLOP/s", "sets": len(sets)}


def bench_w8_linear(rng, dtype, m, n, k, iters, opt):
    """x [m,k] (16-bit) @ int8 weights [n,k] with per-output-channel scales: matmul_int8, the linear of the int8 models."""
    e = gpu.dtype_size(dtype)
    sets = []
    for _ in range(_nsets(m * k * e + n * k + m * n * e, opt.rotate)):
        q, scales = gpu.quantize_weight(_tensor(rng, (n, k), "float32", 0.02))
        sets.append((_tensor(rng, (m, k), dtype), q, scales))
    ms = _time([lambda x=x, q=q, sc=sc: gpu.matmul_int8(x, q, sc) for x, q, sc in sets], iters, single=opt.single)
    flops = 2.0 * m * n * k
    return {"op": "matmul_int8", "dtype": dtype, "shape": [m, n, k], "ms": ms, "work": flops, "rate": flops / ms / 1e9, "unit": "TFLOP/s", "sets": len(sets)}


def bench_lm_head(rng, dtype, m, vocab, k, iters, opt):
    a = _tensor(rng, (m, k), dtype)
    wte = _tensor(rng, (vocab, k), dtype, 0.02)
    ms = _time([lambda: a @ gpu.transpose(wte)], iters, single=opt.single)
    flops = 2.0 * m * vocab * k
    return {"op": "matmul_kmajor_b", "dtype": dtype, "shape": [m, vocab, k], "ms": ms, "work": flops, "rate": flops / ms / 1e9, "unit": "TFLOP/s", "sets": 1}


def bench_layer_norm(rng, dtype, rows, cols, iters, opt):
    e = gpu.dtype_size(dtype)
    g = _tensor(rng, (cols,), dtype); b = _tensor(rng, (cols,), dtype)
    xs = [_tensor(rng, (rows, cols), dtype) for _ in range(_nsets(2 * rows * cols * e, opt.rotate))]
    ms = _time([lambda x=x: gpu.layer_norm(x, g, b, 1e-5) for x in xs], iters, single=opt.single)
    nbytes = 2.0 * rows * cols * e + 2 * cols * e
    return {"op": "layer_norm", "dtype": dtype, "shape": [rows, cols], "ms": ms, "work": nbytes, "rate": nbytes / ms / 1e6, "unit": "GB/s", "sets": len(xs)}


def bench_softmax_causal(rng, dtype, b, rows, cols, iters, opt):
    e = gpu.dtype_size(dtype)
    xs = [_tensor(rng, (b, rows, cols), dtype) for _ in range(_nsets(2 * b * rows * cols * e, opt.rotate))]
    ms = _time([lambda x=x: gpu.softmax_causal(x) for x in xs], iters, single=opt.single)
    tri = sum(min(r + 1, cols) for r in range(rows))
    nbytes = (b * tri + b * rows * cols) * float(e)   # lower-triangle read + full write
    return {"op": "softmax_causal", "dtype": dtype, "shape": [b, rows, cols], "ms": ms, "work": nbytes, "rate": nbytes / ms / 1e6, "unit": "GB/s", "sets": len(xs)}


def bench_gelu_add_bias(rng, dtype, rows, cols, iters, opt):
    e = gpu.dtype_size(dtype)
    bias = _tensor(rng, (cols,), dtype)
    xs = [_tensor(rng, (rows, cols), dtype) for _ in range(_nsets(2 * rows * cols * e, opt.rotate))]
    # the fusion pass turns add_bias -> gelu into one add_bias[gelu] kernel
    ms = _time([lambda x=x: gpu.gelu(gpu.add_bias(x, bias)) for x in xs], iters, single=opt.single)
    nbytes = 2.0 * rows * cols * e + cols * e
    return {"op": "gelu+add_bias", "dtype": dtype, "shape": [rows, cols], "ms": ms, "work": nbytes, "rate": nbytes / ms / 1e6, "unit": "GB/s", "sets": len(xs)}


def bench_attention(rng, dtype, b, h, t, d, causal, iters, opt):
    e = gpu.dtype_size(dtype)
    sets = []
    for _ in range(_nsets(4 * b * h * t * d * e, opt.rotate)):
        sets.append(tuple(_tensor(rng, (b, h, t, d), dtype) for _ in range(3)))
    fn = gpu.attention_causal if causal else gpu.attention
    ms = _time([lambda q=q, k=k, v=v: fn(q, k, v) for q, k, v in sets], iters, single=opt.single)
    flops = 4.0 * b * h * t * t * d * (0.5 if causal else 1.0)
    return {"op": "attention_causal" if causal else "attention", "dtype": dtype, "shape": [b, h, t, d], "ms": ms, "work": flops,
            "rate": flops / ms / 1e9, "unit": "TFLOP/s (causal-minimal flops)" if causal else "TFLOP/s", "sets": len(sets)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all")
    ap.add_argument("--shape", default="")
    ap.add_argument("--dtype", default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--act", default="", help="'erf' for the exact GELU in --op linears")
    ap.add_argument("--single", action="store_true", help="time every launch with its own event pair (includes launch latency)")
    ap.add_argument("--no-rotate", dest="rotate", action="store_false", help="one buffer set: inputs stay L2-warm between launches")
    args = ap.parse_args(argv)
    gpu.init_backend()
    rng = np.random.default_rng(0)
    dtypes = [args.dtype] if args.dtype else ["bfloat16", "float32"]
    shape = [int(x) for x in args.shape.split(",")] if args.shape else None
    out = []
    for dt in dtypes:
        if args.op in ("all", "matmul"):
            for s in ([shape] if shape else [[8, 1024, 1024, 1024], [8, 2048, 2048, 2048], [8, 4096, 4096, 4096]]):
                out.append(bench_matmul(rng, dt, *s, args.iters, args))
        if args.op in ("all", "gpt2_gemms") and dt != "float32":
            for (m, n, k) in [(8192, 2304, 768), (8192, 768, 768), (8192, 3072, 768), (8192, 768, 3072)]:
                out.append(bench_matmul(rng, dt, 1, m, n, k, args.iters, args))
            out.append(bench_lm_head(rng, dt, 8192, 50257, 768, args.iters, args))
        if args.op in ("all", "gpt2_linears") and dt != "float32":
            for (m, n, k, act, res) in [(8192, 2304, 768, False, False), (8192, 768, 768, False, True), (8192, 3072, 768, True, False),
                                        (8192, 768, 3072, False, True)]:
                out.append(bench_fused_linear(rng, dt, m, n, k, act, res, args.iters, args))
        if args.op == "gpt2_linears_kmajor" and dt != "float32":
            for (m, n, k, act, res) in [(8192, 2304, 768, False, False), (8192, 768, 768, False, True), (8192, 3072, 768, True, False),
                                        (8192, 768, 3072, False, True)]:
                out.append(bench_fused_linear(rng, dt, m, n, k, act, res, args.iters, args, kmajor=True))
        if args.op == "linears" and dt != "float32":
            # the four linears of a transformer layer at --shape rows,width (BERT-base: 131072,768 with --act erf)
            rows, d = shape or [131072, 768]
            for (n, k, act, res) in [(3 * d, d, False, False), (d, d, False, True), (4 * d, d, args.act or True, False), (d, 4 * d, False, True)]:
                out.append(bench_fused_linear(rng, dt, rows, n, k, act, res, args.iters, args))
        if args.op in ("all", "layer_linears") and dt != "float32":
            for chained in (True, False):
                out.append(bench_layer_linears(rng, dt, *(shape or [8192, 768]), args.iters, args, chained=chained))
        if args.op == "layer_linears_chained" and dt != "float32":
            out.append(bench_layer_linears(rng, dt, *(shape or [8192, 768]), args.iters, args, chained=True))
        if args.op == "w8_linear" and dt != "float32":
            out.append(bench_w8_linear(rng, dt, *(shape or [2048, 5120, 1280]), args.iters, args))
        if args.op == "lm_head":
            out.append(bench_lm_head(rng, dt, *(shape or [8192, 50257, 768]), args.iters, args))
        if args.op in ("all", "layer_norm"):
            out.append(bench_layer_norm(rng, dt, *(shape or [8192, 768]), args.iters, args))
        if args.op in ("all", "softmax_causal"):
            out.append(bench_softmax_causal(rng, dt, *(shape or [96, 1024, 1024]), args.iters, args))
        if args.op in ("all", "gelu_add_bias"):
            out.append(bench_gelu_add_bias(rng, dt, *(shape or [8192, 3072]), args.iters, args))
        if args.op in ("all", "attention"):
            out.append(bench_attention(rng, dt, *(shape or [8, 12, 1024, 64]), True, args.iters, args))
        for r in out:
            if not r.get("_printed"):
                r["_printed"] = True
                print(json.dumps({k: v for k, v in r.items() if k != "_printed"}), flush=True)
    st = gpu.pipeline_status()
    if st:
        print(json.dumps({"pipeline_status": st}))
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
