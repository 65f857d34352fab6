#!/usr/bin/env python
"""Headline benchmark: GPT-2-small-architecture forward tokens/s, and the per-op roofline rows.

  python bench.py --gpus N --steps K --warmup W              the B200 path (this library)
  python bench.py --impl reference --gpus N --steps K ...    the reference's CPU path (PyTorch CPU eager)

Workload at every N (both arms): GPT-2-small architecture (12 layers, d 768, 12 heads, MLP 3072, vocab
50257, ctx 1024), weights N(0, 0.02) seed 0, token ids uniform over the vocab, batch 8 x seq 1024 per
step. A step is one forward pass over one batch. The B200 arm computes in bf16 with fp32 accumulation;
with N > 1 (torchrun, one process per GPU) the batch dimension is sharded: every rank runs its own
8 x 1024 batch on replicated weights, no data-path collective, the aggregate is summed (weak scaling).
The reference arm runs the same 8 x 1024 batch per step in fp32 on the host cores (rank 0 only), one
forward per sequence, as the reference's own GPT-2 driver (which has no batch dimension) does.

One JSON line on rank 0:
  value         tokens/s with token ids already resident in HBM, CUDA events on the runtime's stream
  e2e           tokens/s through the public API with pinned HOST token ids: per step H2D of the ids,
                the forward, argmax of every position's logits on device, D2H of those int32 ids
  roofline      dominant kernel (the tcgen05 GEMM family): algorithmic FLOPs / CUDA-event time of
                those launches inside the forward, against the measured bf16 peaks (burst and sustained)
  sustained     the same step timed over a loop of at least two seconds (the power cap engages)
  cpu_baseline  PyTorch CPU eager fp32 on this host, bounded sample (rank 0, N = 1 only)
  parity        the bf16 forward of the sample sequence against the cpu_baseline leg's fp32 logits
  per_op        the op-microbenchmark rows (fp32 and bf16) with achieved rate and fraction of the measured peak
  fp32, decode  the same forward in float32; 50 greedy KV-cache steps at batch 8 (bf16)
  strong, tp    (N > 1) fixed global batch 8 split over the ranks; BERT-base tensor-parallel forward
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH, SEQ = 8, 1024
# kept here (not imported from the package) so that the reference arm never loads the CUDA library
GPT2_SMALL = {"n_layer": 12, "n_head": 12, "n_embd": 768, "vocab_size": 50257, "n_positions": 1024}
WORKLOAD = "gpt2-small forward, batch 8 x seq 1024 per step and per GPU, random init N(0,0.02), uniform token ids"


def workload_config(world):
    """The `config` object both arms print (identical, so the two lines are comparable key by key)."""
    return {"workload": WORKLOAD, "global_batch": BATCH * world, "seq_len": SEQ, "parallelism": f"batch-sharded x{world}, no collective",
            "l2": "4 rotating id buffers; the step's working set (249 MB of bf16 weights + activations) exceeds the 126 MB L2"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"bf16_tflops": d.get("bf16_tflops"), "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "hbm_gbs": d.get("hbm_gbs"),
                "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons from the moment it is started; `window()` summarises the
    samples that fall inside a host-time interval (the timed region)."""

    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, device_index):
        self.idx = device_index
        self.samples = []       # (host time, MHz, reason mask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._t = None
        self._nvml = None
        self._h = None

    def start(self):
        """NVML is initialised HERE, before the thread starts and before any timed region, so that the first
        sample does not wait for library start-up. Read-only queries: clocks and clock-event reasons."""
        try:
            import pynvml
            pynvml.nvmlInit()
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self._nvml = pynvml
        except Exception:
            self._nvml = None
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        if self._nvml is not None:
            nv = self._nvml
            while not self._stop.is_set():
                try:
                    self.samples.append((time.perf_counter(), float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)), int(self._reasons(self._h))))
                except Exception:
                    pass
                self._stop.wait(0.003)
            return
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        order = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.idx)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    f = [x.strip() for x in out[0].split(",")]
                    self.max_mhz = float(f[1])
                    mask = 0
                    for n, v in zip(order, f[2:6]):
                        if v.lower().startswith("active"):
                            mask |= self.BITS[n]
                    self.samples.append((time.perf_counter(), float(f[0]), mask))
            except Exception:
                pass
            self._stop.wait(0.1)

    def window(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        note = None
        if not inside and self.samples:
            # a region shorter than one sampling period: take the nearest samples on either side
            inside = sorted(self.samples, key=lambda s: min(abs(s[0] - t0), abs(s[0] - t1)))[:2]
            note = "region shorter than the sampling period: nearest samples"
        mask = 0
        for s in inside:
            mask |= s[2]
        out = {"sm_mhz": float(np.median([s[1] for s in inside])) if inside else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(n for n, b in self.BITS.items() if mask & b), "samples": len(inside)}
        if note:
            out["note"] = note
        return out

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        if self._nvml is not None:
            try:
                self._nvml.nvmlShutdown()
            except Exception:
                pass


# ── the reference's CPU path ────────────────────────────────────────────────
def cpu_forward(weights, ids_t):
    import torch
    from oracle import torch_ref
    with torch.no_grad():
        logits, _ = torch_ref.gpt2_forward(weights, GPT2_SMALL, ids_t)
    return logits


def cpu_baseline(sample_batch=1, repeats=2):
    """PyTorch CPU eager fp32 on all host cores, `sample_batch` sequences of 1024 tokens. Returns the baseline
    object and (ids, logits) of the sample for the parity check."""
    import torch
    from oracle import torch_ref
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = torch_ref.init_gpt2_weights(GPT2_SMALL, seed=0)
    rng = np.random.default_rng(0)
    ids = torch.from_numpy(rng.integers(0, GPT2_SMALL["vocab_size"], (sample_batch, SEQ)))
    cpu_forward(weights, ids[:1, :128])  # warm the thread pool
    times, logits = [], None
    for _ in range(repeats):
        t0 = time.perf_counter()
        logits = cpu_forward(weights, ids)
        times.append(time.perf_counter() - t0)
    best = min(times)
    base = {"value": sample_batch * SEQ / best, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{sample_batch} x {SEQ} tokens per forward, fp32, best of {repeats} (oracle/torch_ref.py, PyTorch CPU eager)",
            "seconds": best}
    return base, ids.numpy(), logits.numpy()


def run_reference(args):
    """The reference arm: its CPU path (PyTorch CPU eager, fp32) on the same 8 x 1024 batch per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return  # under torchrun rank 0 alone runs and prints the CPU arm
    import torch
    from oracle import torch_ref
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = torch_ref.init_gpt2_weights(GPT2_SMALL, seed=0)
    rng = np.random.default_rng(1000)
    ids = torch.from_numpy(rng.integers(0, GPT2_SMALL["vocab_size"], (BATCH, SEQ)))
    cpu_forward(weights, ids[:1, :128])

    def step():
        # one forward per sequence: the reference's gpt2_forward has no batch dimension (models/gpt2.py:47-91), and a
        # [1, 1024] forward keeps the attention scores and the logits of one sequence in cache. The step's result is
        # the next-token id of every position, as in the other arm's e2e leg.
        return [cpu_forward(weights, ids[b:b + 1]).argmax(-1) for b in range(BATCH)]

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    tps = BATCH * SEQ * args.steps / dt
    line = {"impl": "reference", "metric": "gpt2_small_forward_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
            "reference_path": "PyTorch CPU eager (the reference's own oracle and CPU baseline; its Metal path is unavailable on this box)",
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": f"{BATCH} x {SEQ} tokens per step (the full batch of one GPU's step, one forward per sequence), fp32, {args.steps} steps"},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ── per-op rows ─────────────────────────────────────────────────────────────
def per_op_rows(peaks, iters=20):
    """The op-microbenchmark configuration, fp32 and bf16, timed in-process by applegpu_runtime_b200.microbench
    (back-to-back launches inside one CUDA-event pair, buffer sets rotated so no launch finds its data in L2)."""
    from applegpu_runtime_b200 import microbench as mb
    opt = argparse.Namespace(rotate=True, single=False)
    rows = []
    rng = np.random.default_rng(0)
    for dt in ("bfloat16", "float32"):
        for s in (1024, 2048, 4096):
            rows.append(mb.bench_matmul(rng, dt, 8, s, s, s, max(3, iters // (1 if s < 4096 else 4)), opt))
        rows.append(mb.bench_layer_norm(rng, dt, 8192, 768, iters, opt))
        rows.append(mb.bench_softmax_causal(rng, dt, 96, 1024, 1024, iters, opt))
        rows.append(mb.bench_gelu_add_bias(rng, dt, 8192, 3072, iters, opt))
    out = []
    for r in rows:
        tensor = r["unit"].startswith("TFLOP")
        peak = peaks["bf16_tflops"] if tensor else peaks["hbm_gbs"]
        row = {"op": r["op"], "dtype": "bf16" if r["dtype"] == "bfloat16" else "f32", "shape": r["shape"], "us": round(r["ms"] * 1e3, 2),
               "achieved": round(r["rate"], 1), "unit": "TFLOP/s" if tensor else "GB/s", "peak": peak, "frac": round(r["rate"] / peak, 3)}
        if tensor and r["dtype"] == "float32":
            row["note"] = "fp32 product as a three-term bf16 split: 6x these flops run on the bf16 tensor pipe; frac is algorithmic flops over the bf16 burst peak"
        out.append(row)
    return out


def run_b200(args):
    from applegpu_runtime_b200.sharding import RankGroup
    group = RankGroup.from_env(args.gpus)  # bookkeeping only: barrier + MAX of the timings; no data-path collective
    rank, world = group.rank, group.world
    import applegpu_runtime_b200 as gpu
    from applegpu_runtime_b200 import _lib
    lib = _lib.load()
    gpu.init_backend()  # raises if the CUDA library or device is missing: no fallback
    import ctypes
    import torch  # pinned host buffers only

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", 0)))
    sampler.start()   # NVML comes up here, long before the first timed region

    cfg = GPT2_SMALL
    model = gpu.init_gpt2_weights(cfg, seed=0, dtype="bfloat16")
    rng = np.random.default_rng(1000 + rank)
    n_tok = BATCH * SEQ
    n_buf = 4
    host_ids = [torch.from_numpy(rng.integers(0, cfg["vocab_size"], n_tok).astype(np.int32)).pin_memory() for _ in range(n_buf)]
    host_pos = torch.from_numpy(np.tile(np.arange(SEQ, dtype=np.int32), BATCH)).pin_memory()
    host_out = torch.empty(n_tok, dtype=torch.int32).pin_memory()
    shape_ids = np.zeros((BATCH, SEQ), np.int64)

    dev_ids = [gpu.from_numpy(h.numpy()) for h in host_ids]
    dev_pos = gpu.from_numpy(host_pos.numpy())
    gpu.synchronize()

    def step_resident(i, m=model):
        # compiled=True: the forward's op list is recorded once on an op tape and replayed (one library call per step)
        logits, _ = gpu.gpt2_forward(m, shape_ids, device_ids=(dev_ids[i % n_buf], dev_pos), compiled=True)
        logits.eval()
        return logits

    def step_e2e(i):
        h = host_ids[i % n_buf]
        ids_t = gpu.GpuTensor(lib.applegpu_ffi_from_host(ctypes.c_void_p(h.data_ptr()), (ctypes.c_uint64 * 1)(n_tok), 1, 5))
        pos_t = gpu.GpuTensor(lib.applegpu_ffi_from_host(ctypes.c_void_p(host_pos.data_ptr()), (ctypes.c_uint64 * 1)(n_tok), 1, 5))
        logits, _ = gpu.gpt2_forward(model, shape_ids, device_ids=(ids_t, pos_t), compiled=True)   # op tape: one library call per forward
        nxt = gpu.argmax(logits)  # [B, T] int32: the step's result
        del logits
        if lib.applegpu_ffi_read_bytes(nxt.id, ctypes.c_void_p(host_out.data_ptr()), n_tok * 4) != 0:
            raise RuntimeError(lib.applegpu_ffi_last_error())
        return host_out

    # warm-up (also fills the buffer pool and the tensor-map cache)
    for i in range(max(args.warmup, 3)):
        step_resident(i)
    gpu.synchronize()

    # ── value: device-resident ids, CUDA events on the runtime stream, max over ranks ──
    launches0 = gpu.launch_count()
    group.barrier()
    gpu.synchronize()
    t_begin = time.perf_counter()
    lib.applegpu_timer_start()
    for i in range(args.steps):
        step_resident(i)
    ms = float(lib.applegpu_timer_stop_ms())
    gpu.synchronize()
    t_end = time.perf_counter()
    clocks = sampler.window(t_begin, t_end)
    group.barrier()
    launches = gpu.launch_count() - launches0
    ms = group.max(ms)
    tokens_total = n_tok * args.steps * world
    value = tokens_total / (ms / 1e3)

    # ── e2e: pinned host ids in, int32 next-token ids out, every step ──
    # Serving-loop form: step i's result is copied to pinned memory asynchronously and consumed while
    # step i+1 is already enqueued (one step in flight), so graph recording on the host overlaps the
    # GPU. Every step's H2D copy, forward, argmax and D2H copy sit inside the timed region, which ends
    # when the last result has landed. The blocking form (read every result before building the next
    # step) is timed too and reported beside it.
    host_outs = [torch.empty(n_tok, dtype=torch.int32).pin_memory() for _ in range(2)]

    def issue_e2e(i):
        h = host_ids[i % n_buf]
        ids_t = gpu.GpuTensor(lib.applegpu_ffi_from_host(ctypes.c_void_p(h.data_ptr()), (ctypes.c_uint64 * 1)(n_tok), 1, 5))
        pos_t = gpu.GpuTensor(lib.applegpu_ffi_from_host(ctypes.c_void_p(host_pos.data_ptr()), (ctypes.c_uint64 * 1)(n_tok), 1, 5))
        logits, _ = gpu.gpt2_forward(model, shape_ids, device_ids=(ids_t, pos_t), compiled=True)   # op tape: one library call per forward
        nxt = gpu.argmax(logits)
        del logits  # greedy serving keeps only the tokens: the LM head's epilogue then takes the row maximum itself
        if lib.applegpu_ffi_read_bytes_async(nxt.id, ctypes.c_void_p(host_outs[i % 2].data_ptr()), n_tok * 4) != 0:
            raise RuntimeError(lib.applegpu_ffi_last_error())
        return lib.applegpu_marker_record()

    def run_pipelined(steps):
        checksum, pending = 0, 0
        for i in range(steps):
            marker = issue_e2e(i)
            if pending:
                if lib.applegpu_marker_wait(pending) != 0:
                    raise RuntimeError("marker wait failed")
                checksum += int(host_outs[(i - 1) % 2][-1])  # the consumer reads step i-1's tokens
            pending = marker
        if lib.applegpu_marker_wait(pending) != 0:
            raise RuntimeError("marker wait failed")
        return checksum + int(host_outs[(steps - 1) % 2][-1])

    for i in range(3):
        step_e2e(i)
    group.barrier()
    gpu.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step_e2e(i)
    gpu.synchronize()
    ms_e2e_blocking = group.max((time.perf_counter() - t0) * 1e3)

    run_pipelined(3)
    group.barrier()
    gpu.synchronize()
    t0 = time.perf_counter()
    lib.applegpu_timer_start()
    run_pipelined(args.steps)
    ms_e2e_dev = float(lib.applegpu_timer_stop_ms())
    wall_e2e = (time.perf_counter() - t0) * 1e3
    ms_e2e = group.max(max(ms_e2e_dev, wall_e2e))
    e2e = {"value": tokens_total / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * n_tok * 4, "d2h_bytes_per_step": n_tok * 4,
           "ms_per_step": ms_e2e / args.steps, "mode": "one step in flight (async D2H to pinned memory, result consumed one step later)",
           "result": "argmax tokens [B, T] int32; the LM head runs in its argmax-epilogue form, so no logits tensor is written (the `value` leg writes 823 MB of logits per step)",
           "blocking_ms_per_step": ms_e2e_blocking / args.steps, "blocking_value": tokens_total / (ms_e2e_blocking / 1e3)}

    # ── sustained: the same resident-id step over a loop of at least two seconds ──
    group.barrier()
    gpu.synchronize()
    t_s0 = time.perf_counter()
    lib.applegpu_timer_start()
    n_sus = 0
    chunk = 50 if args.sustained_seconds > 0 else max(args.steps, 1)
    while True:
        for i in range(chunk):
            step_resident(n_sus + i)
        n_sus += chunk
        gpu.synchronize()
        if time.perf_counter() - t_s0 >= args.sustained_seconds or n_sus >= 5000:
            break
    ms_sus = float(lib.applegpu_timer_stop_ms())
    t_s1 = time.perf_counter()
    sus_clocks = sampler.window(t_s0, t_s1)
    ms_sus_step = group.max(ms_sus / n_sus)
    sustained = {"ms_per_step": ms_sus_step, "value": n_tok * world / (ms_sus_step / 1e3), "unit": "tokens/s", "steps": n_sus,
                 "seconds": (t_s1 - t_s0), "median_sm_mhz": sus_clocks["sm_mhz"], "reasons": sus_clocks["reasons"]}

    # ── roofline: per-kernel CUDA-event times inside the forward ──
    # pass 1: every kernel bracketed (the per-kernel table; with an event pair around each of ~90 launches the host
    # becomes the bottleneck, so these times are upper bounds). pass 2: only the GEMM family bracketed, the rest of the
    # step runs as it normally does: that pass gives the GEMM launch durations of the roofline.
    gpu.profile(True)
    prof_steps = min(args.steps, 5)
    for i in range(prof_steps):
        step_resident(i)
    rep = gpu.profile_report()
    gpu.profile(False)
    gpu.profile(True, only=["fused_linear", "matmul"])
    for i in range(prof_steps):
        step_resident(i)
    rep_gemm = gpu.profile_report()
    gpu.profile(False)
    status = gpu.pipeline_status()
    peaks = measured_peaks()
    gemm = {k: v for k, v in rep_gemm.items() if k.startswith(("fused_linear", "matmul"))}
    g_ms = sum(v["ms"] for v in gemm.values())
    g_flops = sum(v["work"] for v in gemm.values())
    g_launch = sum(v["launches"] for v in gemm.values())
    achieved = g_flops / (g_ms / 1e3) / 1e12 if g_ms > 0 else None
    total_ms = sum(v["ms"] for v in rep.values())
    # second reading: the untimed-by-events step minus the bracketed times of everything that is not a GEMM (attention,
    # layer_norm, embedding, argmax). Bracketing a launch exposes its launch latency and prologue, so this bound errs the
    # other way from `achieved`: the GEMM family's true in-pipeline rate lies between the two.
    other_ms = sum(v["ms"] for k, v in rep.items() if not k.startswith(("fused_linear", "matmul"))) / prof_steps
    step_ms = ms / args.steps
    by_sub = g_flops / prof_steps / ((step_ms - other_ms) / 1e3) / 1e12 if step_ms > other_ms > 0 else None
    roofline = {"bound": "tensor", "kernel": "gemm_tc_chain_kernel + gemm_tc_pair_kernel (tcgen05: per block one chained launch of out-proj, FC1, FC2 and the next QKV; block 0's QKV; LM head)",
                "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": (achieved / peaks["bf16_tflops"]) if achieved else None,
                "peak_source": peaks["source"] + " (burst: the timed region lasts tens of milliseconds at the full SM clock)",
                "frac_burst": (achieved / peaks["bf16_tflops"]) if achieved else None,
                "frac_sustained": (achieved / peaks["bf16_tflops_sustained"]) if achieved else None,
                "peak_sustained": peaks["bf16_tflops_sustained"],
                "traffic": gemm_traffic_bytes(), "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the GEMM launches of one forward; null = not captured for this revision)",
                "launches_per_step": g_launch / prof_steps, "avg_launch_ms": g_ms / max(g_launch, 1),
                "share_of_step": g_ms / prof_steps / (ms / args.steps),
                "achieved_by_subtraction": by_sub, "frac_by_subtraction": (by_sub / peaks["bf16_tflops"]) if by_sub else None,
                "by_subtraction": "GEMM flops / (device-timed step - event-bracketed time of every non-GEMM kernel): the GEMM launches keep their programmatic overlap, the others lose theirs, so this reads high where `achieved` reads low",
                "folded_layer_norm": "23 of the 25 layer_norm launches run inside these GEMMs' epilogues (row statistics out of out-proj / FC2, correction in QKV / FC1): their time is counted here, their flops are not",
                "timing": "CUDA events around every GEMM launch of the forward, in situ (other kernels not bracketed); an event pair costs each launch its programmatic-launch overlap with its neighbours",
                "per_kernel_ms_per_step": {k: round(v["ms"] / prof_steps, 4) for k, v in sorted(rep.items(), key=lambda kv: -kv[1]["ms"])}}

    line = {"metric": "gpt2_small_forward_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "sustained": sustained, "pipeline_status": status,
            "device": gpu.device_name()}

    # ── secondary figures (one GPU per rank; only rank 0's are printed) ──
    extras_ok = not args.quick
    if extras_ok and world > 1:
        line["strong"] = strong_scaling_leg(gpu, lib, group, model, cfg)
        line["tp"] = tensor_parallel_leg(gpu, lib, group)
    if rank == 0 and world == 1 and extras_ok:
        line["decode"] = decode_leg(gpu, model, cfg)
        if not args.no_cpu_baseline:
            base, s_ids, s_logits = cpu_baseline(sample_batch=1)
            line["cpu_baseline"] = base
            got = gpu.gpt2_forward(model, s_ids)[0].to_numpy().reshape(SEQ, -1)
            ref = s_logits.reshape(SEQ, -1)
            scale = float(np.max(np.abs(ref)))
            line["parity"] = {"max_rel_err": float(np.max(np.abs(got - ref)) / scale), "argmax_match": float(np.mean(got.argmax(-1) == ref.argmax(-1))),
                              "bar": "bf16 within 2e-2 relative of the fp32 oracle", "sample": "the cpu_baseline leg's 1 x 1024 sequence, all 1024 x 50257 logits"}
        else:
            s_ids = s_logits = None
        # float32 forward of the same batch (fp32 products run as a three-term bf16 split on the tensor cores)
        model32 = gpu.init_gpt2_weights(cfg, seed=0, dtype="float32")
        for i in range(3):
            step_resident(i, model32)
        gpu.synchronize()
        lib.applegpu_timer_start()
        n32 = max(3, min(args.steps, 10))
        for i in range(n32):
            step_resident(i, model32)
        ms32 = float(lib.applegpu_timer_stop_ms()) / n32
        line["fp32"] = {"ms_per_step": ms32, "value": n_tok / (ms32 / 1e3), "unit": "tokens/s"}
        if s_ids is not None:
            got32 = gpu.gpt2_forward(model32, s_ids)[0].to_numpy().reshape(SEQ, -1)
            line["fp32"]["max_abs_err_vs_oracle"] = float(np.max(np.abs(got32 - s_logits.reshape(SEQ, -1))))
            line["fp32"]["argmax_match"] = float(np.mean(got32.argmax(-1) == s_logits.reshape(SEQ, -1).argmax(-1)))
        del model32
        gpu.pool_drain()
        line["per_op"] = per_op_rows(peaks)
        line["pipeline_status"] = max(status, gpu.pipeline_status())
    sampler.stop()
    if rank == 0:
        print(json.dumps(line), flush=True)
    group.close()


def gemm_traffic_bytes():
    """Mean DRAM bytes per GEMM launch of one forward, read from the tracked record next to the ncu summaries
    (profiles/gemm_traffic.json: written from a capture, with the revision it was taken at); None if absent."""
    p = os.path.join(ROOT, "profiles", "gemm_traffic.json")
    try:
        with open(p) as f:
            return float(json.load(f)["mean_bytes_per_launch"])
    except Exception:
        return None


def decode_leg(gpu, model, cfg, steps=50, prompt=64):
    """50 greedy steps with the KV cache at batch 8 (bf16). `ms_per_step` is the wall clock of the whole generation
    (the prompt's prefill, creating the decoder, capturing its step, reading the tokens back) divided by the steps;
    `steady_ms_per_step` is the replayed step alone (wall clock of a run of graph launches, tokens read back at the end)."""
    from applegpu_runtime_b200.generate import Gpt2Decoder
    ids = np.random.default_rng(1).integers(0, cfg["vocab_size"], (BATCH, prompt))
    gpu.greedy_generate(model, ids, max_tokens=4, use_cache=True)
    gpu.synchronize()
    best, launches = None, 0
    for _ in range(2):
        l0 = gpu.launch_count()
        t0 = time.perf_counter()
        out = gpu.greedy_generate(model, ids, max_tokens=steps, use_cache=True)
        dt = time.perf_counter() - t0
        launches = gpu.launch_count() - l0
        best = dt if best is None or dt < best else best
    assert out.shape == (BATCH, prompt + steps)
    stats = dict(model.get("_last_decoder_stats", {}))
    logits, kv = gpu.gpt2_forward(model, ids, kv_cache=None, last_only=True)
    first = gpu.argmax(logits)
    del logits
    dec = Gpt2Decoder(model, BATCH, prompt + steps + 2)
    try:
        dec.prefill(kv, first, prompt)
        dec.steps(2)                       # the first step runs launch by launch, the second from the fresh capture
        t0 = time.perf_counter()
        dec.steps(steps - 2)
        steady = (time.perf_counter() - t0) / (steps - 2)
    finally:
        dec.close()
    weight_bytes = 124.4e6 * 2
    return {"ms_per_step": best * 1e3 / steps, "tokens_per_s": BATCH * steps / best, "steady_ms_per_step": steady * 1e3,
            "steady_tokens_per_s": BATCH / steady, "launches_per_step": stats.get("launches_per_step"), "cuda_graph": stats.get("graph"),
            "weight_stream_floor_ms": weight_bytes / (measured_peaks()["hbm_gbs"] * 1e9) * 1e3,
            "note": f"batch {BATCH}, prompt {prompt}, {steps} greedy steps; preallocated KV cache appended in place, one captured step replayed per token"}


def strong_scaling_leg(gpu, lib, group, model, cfg):
    """Fixed global batch of 8 sequences x 1024 split over the ranks (8 / world sequences each, no collective):
    the strong-scaling counterpart of the weak-scaling headline. MAX over ranks of the CUDA-event time."""
    from applegpu_runtime_b200.sharding import shard_range
    lo, hi = shard_range(BATCH, group.rank, group.world)
    local = hi - lo
    ms = 0.0
    if local > 0:
        rng = np.random.default_rng(2000 + group.rank)
        ids = gpu.from_numpy(rng.integers(0, cfg["vocab_size"], local * SEQ).astype(np.int32))
        pos = gpu.from_numpy(np.tile(np.arange(SEQ, dtype=np.int32), local))
        shape = np.zeros((local, SEQ), np.int64)

        def step():
            gpu.gpt2_forward(model, shape, device_ids=(ids, pos), compiled=True)[0].eval()
        for _ in range(3):
            step()
    group.barrier()
    gpu.synchronize()
    if local > 0:
        lib.applegpu_timer_start()
        for _ in range(10):
            step()
        ms = float(lib.applegpu_timer_stop_ms()) / 10
    ms = group.max(ms)
    return {"global_batch": BATCH, "seq_len": SEQ, "sequences_per_rank": local, "ms_per_step": ms, "value": BATCH * SEQ / (ms / 1e3), "unit": "tokens/s"}


def tensor_parallel_leg(gpu, lib, group):
    """BERT-base 256 x 512 bf16 with heads and feed-forward units sharded over the ranks (NCCL all-reduce over NVLink,
    two per layer, overlapped with the next micro-batch's compute): ms per forward (MAX over ranks), the same with the
    collectives serialised on the runtime stream, and, on a small batch, the relative error of the sharded bf16 forward
    against the unsharded float32 forward on the same GPU (bar: 2e-2, as for every bf16 path)."""
    try:
        from applegpu_runtime_b200 import modelbench as mbm
        from applegpu_runtime_b200.bert import BERT_BASE, bert_forward, bert_forward_overlapped, load_bert_state_dict
        from applegpu_runtime_b200.tp import TensorParallelGroup, load_bert_shard
        tp = TensorParallelGroup(group)
        state = mbm._bert_host_state(BERT_BASE)
        shard = load_bert_shard(state, BERT_BASE, group, dtype="bfloat16")
        rng = np.random.default_rng(3)
        small = rng.integers(0, BERT_BASE["vocab_size"], (4, 512))
        got = np.concatenate([o.to_numpy() for o in bert_forward_overlapped(shard, small, tp, micro_batches=2)], axis=0)
        full = load_bert_state_dict(state, BERT_BASE, dtype="float32")   # the unsharded forward in float32 is the reference
        want = bert_forward(full, small).to_numpy()
        del full
        err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
        rms = float(np.sqrt(np.mean((got - want) ** 2)) / np.sqrt(np.mean(want ** 2)))
        # for scale: the same error of the unsharded bf16 forward (what 16-bit storage costs without any sharding)
        full16 = load_bert_state_dict(state, BERT_BASE, dtype="bfloat16")
        got16 = bert_forward(full16, small).to_numpy()
        del full16
        err16 = float(np.max(np.abs(got16 - want)) / np.max(np.abs(want)))
        ids = rng.integers(0, BERT_BASE["vocab_size"], (256, 512))

        def timed(step):
            for _ in range(2):
                step()
            group.barrier()
            gpu.synchronize()
            lib.applegpu_timer_start()
            for _ in range(3):
                step()
            return group.max(float(lib.applegpu_timer_stop_ms()) / 3)

        def step_serial():
            bert_forward(shard, ids, all_reduce=tp.all_reduce).eval()

        def step_overlapped():
            for out in bert_forward_overlapped(shard, ids, tp, micro_batches=2):
                out.eval()
        ms_serial = timed(step_serial)
        ms = timed(step_overlapped)
        return {"workload": "bert-base encoder, batch 256 x seq 512, bf16, head / feed-forward split", "ranks": group.world, "ms_per_forward": ms,
                "ms_per_forward_all_reduce_on_runtime_stream": ms_serial, "micro_batches": 2,
                "tokens_per_s": 256 * 512 / (ms / 1e3), "max_rel_err_vs_unsharded": group.max(err), "rms_rel_err_vs_unsharded": group.max(rms),
                "max_rel_err_unsharded_bf16": err16, "error_reference": "unsharded float32 forward, 4 x 512 tokens; max |diff| / max |reference|",
                "all_reduces_per_forward": 24,
                "overlap": "each all-reduce runs on a communication stream while the runtime stream computes the next micro-batch's segment"}
    except Exception as e:   # the headline line must still be printed
        return {"error": f"{type(e).__name__}: {e}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="headline, e2e, sustained and roofline only (no per-op rows, fp32, decode, strong / tp legs)")
    ap.add_argument("--sustained-seconds", type=float, default=2.0, help="length of the sustained loop; 0 runs it for --steps steps only (launch lists under a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
