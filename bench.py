#!/usr/bin/env python
"""Headline benchmark: GPT-2-small-architecture forward tokens/s.

  python bench.py --gpus N --steps K --warmup W              the B200 path (this library)
  python bench.py --impl reference --gpus N --steps K ...    the reference's CPU path (PyTorch CPU eager)

Workload at every N: GPT-2-small architecture (12 layers, d 768, 12 heads, MLP 3072, vocab 50257,
ctx 1024), weights N(0, 0.02) seed 0, token ids uniform over the vocab, batch 8 x seq 1024 per GPU,
bf16 weights and activations with fp32 accumulation. A step is one forward pass over one batch.
With N > 1 (torchrun, one process per GPU) the batch dimension is sharded: every rank runs its
own 8 x 1024 batch on replicated weights, no data-path collective; the aggregate is summed
(weak scaling).

One JSON line on rank 0:
  value         tokens/s with token ids already resident in HBM, CUDA events on the runtime's stream
  e2e           tokens/s through the public API with pinned HOST token ids: per step H2D of the ids,
                the forward, argmax of every position's logits on device, D2H of those int32 ids
  roofline      dominant kernel (the tcgen05 GEMM family): algorithmic FLOPs / CUDA-event time of
                those launches inside the forward, against the measured bf16 peak
  cpu_baseline  PyTorch CPU eager fp32 on this host, bounded sample (rank 0, N = 1 only)
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
WORKLOAD = "gpt2-small forward, batch 8 x seq 1024 per GPU, bf16 (fp32 accumulate), random init N(0,0.02), uniform token ids"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"bf16_tflops": d.get("bf16_tflops"), "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "hbm_gbs": d.get("hbm_gbs"),
                "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    def __init__(self, device_index):
        self.idx = device_index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        """NVML in-process (a sample every few ms: the timed region lasts ~100 ms); nvidia-smi as a fallback.
        Read-only queries: clocks and the active clock-event reasons."""
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            bits = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop.is_set():
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                mask = int(get_reasons(h))
                for n, bit in bits.items():
                    if mask & bit:
                        self.reasons.add(n)
                self._stop.wait(0.004)
            pynvml.nvmlShutdown()
            return
        except Exception:
            pass
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.idx)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    f = [x.strip() for x in out[0].split(",")]
                    self.samples.append(float(f[0]))
                    self.max_mhz = float(f[1])
                    for n, v in zip(names, f[2:6]):
                        if v.lower().startswith("active"):
                            self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_reference_step(weights, cfg, ids_t):
    import torch
    from oracle import torch_ref
    with torch.no_grad():
        logits, _ = torch_ref.gpt2_forward(weights, cfg, ids_t)
        return logits[:, -1, :].argmax(-1)


def cpu_baseline(sample_batch, repeats=2):
    """PyTorch CPU eager fp32 on all host cores, `sample_batch` sequences of 1024 tokens."""
    import torch
    from oracle import torch_ref
    from applegpu_runtime_b200.gpt2 import GPT2_SMALL
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = torch_ref.init_gpt2_weights(GPT2_SMALL, seed=0)
    rng = np.random.default_rng(0)
    ids = torch.from_numpy(rng.integers(0, GPT2_SMALL["vocab_size"], (sample_batch, SEQ)))
    cpu_reference_step(weights, GPT2_SMALL, ids[:1, :128])  # warm the thread pool
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_reference_step(weights, GPT2_SMALL, ids)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": sample_batch * SEQ / best, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{sample_batch} x {SEQ} tokens per forward, fp32, best of {repeats} (oracle/torch_ref.py, PyTorch CPU eager)",
            "seconds": best}


def run_reference(args):
    """The reference arm: its CPU path (PyTorch CPU eager) on the same config, bounded sample."""
    if int(os.environ.get("RANK", "0")) != 0:
        return  # under torchrun rank 0 alone runs and prints the CPU arm
    import torch
    from oracle import torch_ref
    from applegpu_runtime_b200.gpt2 import GPT2_SMALL
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = torch_ref.init_gpt2_weights(GPT2_SMALL, seed=0)
    rng = np.random.default_rng(0)
    sample_batch = 1  # bounded sample of the 8 x 1024 workload: 1 sequence of 1024 tokens per step
    ids = torch.from_numpy(rng.integers(0, GPT2_SMALL["vocab_size"], (sample_batch, SEQ)))
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(weights, GPT2_SMALL, ids)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(weights, GPT2_SMALL, ids)
    dt = time.perf_counter() - t0
    tps = sample_batch * SEQ * args.steps / dt
    line = {"impl": "reference", "metric": "gpt2_small_forward_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "reference_path": "PyTorch CPU eager (the reference's own oracle and CPU baseline)"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": f"{sample_batch} x {SEQ} tokens per step, fp32 (the reference's Metal path is unavailable on this box)"},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_b200(args):
    from applegpu_runtime_b200.sharding import RankGroup
    group = RankGroup.from_env(args.gpus)  # bookkeeping only: barrier + MAX of the timings; no data-path collective
    rank, world = group.rank, group.world
    import applegpu_runtime_b200 as gpu
    from applegpu_runtime_b200 import _lib
    from applegpu_runtime_b200.gpt2 import GPT2_SMALL
    lib = _lib.load()
    gpu.init_backend()  # raises if the CUDA library or device is missing: no fallback
    import ctypes
    import torch  # pinned host buffers only

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

    def step_resident(i):
        # compiled=True: the forward's op list is recorded once on an op tape and replayed (one library call per step)
        logits, _ = gpu.gpt2_forward(model, shape_ids, device_ids=(dev_ids[i % n_buf], dev_pos), compiled=True)
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
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", 0)))
    launches0 = gpu.launch_count()
    group.barrier()
    gpu.synchronize()
    sampler.start()
    lib.applegpu_timer_start()
    for i in range(args.steps):
        step_resident(i)
    ms = float(lib.applegpu_timer_stop_ms())
    gpu.synchronize()
    clocks = sampler.stop()
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
           "blocking_ms_per_step": ms_e2e_blocking / args.steps, "blocking_value": tokens_total / (ms_e2e_blocking / 1e3)}

    # ── roofline: per-kernel CUDA-event times inside the forward ──
    gpu.profile(True)
    prof_steps = min(args.steps, 5)
    for i in range(prof_steps):
        step_resident(i)
    rep = gpu.profile_report()
    gpu.profile(False)
    status = gpu.pipeline_status()
    peaks = measured_peaks()
    gemm = {k: v for k, v in rep.items() if k.startswith(("fused_linear", "matmul"))}
    g_ms = sum(v["ms"] for v in gemm.values())
    g_flops = sum(v["work"] for v in gemm.values())
    g_launch = sum(v["launches"] for v in gemm.values())
    achieved = g_flops / (g_ms / 1e3) / 1e12 if g_ms > 0 else None
    total_ms = sum(v["ms"] for v in rep.values())
    roofline = {"bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05, all linear layers + LM head)",
                "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": (achieved / peaks["bf16_tflops_sustained"]) if achieved else None, "peak_source": peaks["source"] + " (sustained: timed inside a long step)",
                # mean DRAM bytes per GEMM launch of one forward, from the ncu captures summarised under profiles/
                # (gemm_tc_kernel__gpt2_small_linears_8192_bf16.md, gemm_tc_kernel__lm_head_8192x50257x768_bf16.md)
                "traffic": 49.2e6, "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum)", "launches_per_step": g_launch / prof_steps, "avg_launch_ms": g_ms / max(g_launch, 1),
                "share_of_step": g_ms / total_ms if total_ms else None,
                "per_kernel_ms_per_step": {k: round(v["ms"] / prof_steps, 4) for k, v in sorted(rep.items(), key=lambda kv: -kv[1]["ms"])}}

    line = {"metric": "gpt2_small_forward_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": BATCH * world, "seq_len": SEQ, "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "4 rotating id buffers; the step's working set (249 MB of bf16 weights + activations) exceeds the 126 MB L2"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "pipeline_status": status,
            "device": gpu.device_name()}
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_batch=1)
        print(json.dumps(line), flush=True)
    group.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
