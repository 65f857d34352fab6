"""Tensor parallelism over heads / feed-forward units for the encoder configuration that does not fit
the batch-sharded form (one process per GPU, NCCL over NVLink through torch.distributed).

The reference is single-device; this is the multi-GPU form of its op sequence for BERT-base
(python/applegpu_runtime/torch_backend.py:246-1805 routes the same ops on one device). Rank r holds
heads [r*h/n, (r+1)*h/n) of the stacked Q/K/V projection and the matching columns of the attention
output projection, and units [r*ff/n, (r+1)*ff/n) of the two feed-forward matrices
(`bert.load_bert_state_dict(..., head_range=, ff_range=)`). The two row-parallel projections of a
layer produce partial sums that are added over the group in place (NCCL all-reduce on the runtime's
own stream: the collective is ordered between the producing GEMM and the consuming layer_norm by
stream order, no host synchronisation); residual and layer_norm are computed redundantly by every
rank. Payload per all-reduce: B*T*d elements, 2 per layer.

`bert.bert_forward_overlapped` hides those collectives: the batch is cut into micro-batches whose forwards advance
in lock step, and each all-reduce runs on a communication stream (all_reduce_start / all_reduce_finish, ordered by
events) while the runtime stream computes the next micro-batch's segment.
"""
import ctypes
import os

import numpy as np

from . import _lib
from . import api as gpu
from .sharding import shard_range


class _DevMem:
    """Exposes a device range through __cuda_array_interface__ so torch can wrap it without a copy."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3, "strides": None}


_TYPESTR = {"float32": "<f4", "float16": "<f2", "bfloat16": "<i2", "int32": "<i4"}


def head_and_ff_ranges(config, rank, world):
    """The slice of attention heads and feed-forward units rank `rank` of `world` owns. Both are split
    into contiguous blocks that differ by at most one item (12 heads over 8 ranks: 2,2,2,2,1,1,1,1)."""
    return shard_range(config["n_head"], rank, world), shard_range(config["d_ff"], rank, world)


class TensorParallelGroup:
    """all_reduce(t) sums a materialised, contiguous GpuTensor over the ranks of a RankGroup, in place."""

    def __init__(self, group, sm_margin=None):
        self.group = group
        self._stream = None
        self._comm = None
        self._pg = None
        self._views = {}
        # SMs the compute kernels leave to the collective while the two overlap (all_reduce_start / _finish)
        self.sm_margin = int(os.environ.get("APPLEGPU_TP_SM_MARGIN", "16")) if sm_margin is None else int(sm_margin)

    def _process_group(self):
        """A group of its own for the data collectives, with NCCL's stream at high priority: its kernels then take
        the SMs that fall free between compute kernels instead of queueing behind them."""
        dist = self.group.dist
        if self._pg is None:
            try:
                opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
                self._pg = dist.new_group(ranks=list(range(self.group.world)), pg_options=opts)
            except Exception:
                self._pg = dist.group.WORLD
        return self._pg

    def _torch_stream(self):
        import torch
        if self._stream is None:
            handle = _lib.load().applegpu_stream()
            self._stream = torch.cuda.ExternalStream(int(handle or 0))
        return self._stream

    def _comm_stream(self):
        import torch
        if self._comm is None:
            self._comm = torch.cuda.Stream(priority=-1)
        return self._comm

    def _view(self, t):
        """The tensor's device memory as a flat torch tensor (evaluates `t`: its kernels are enqueued on the runtime stream)."""
        import torch
        lib = _lib.load()
        ptr = lib.applegpu_ffi_device_ptr(ctypes.c_uint64(t.id))
        if not ptr:
            raise ValueError(lib.applegpu_ffi_last_error().decode())
        dt = t.dtype
        key = (int(ptr), int(np.prod(t.shape)), dt)
        view = self._views.get(key)
        if view is None:
            # pool buffers recur from step to step: the wrapper (it owns nothing) is built once per address and size
            view = torch.as_tensor(_DevMem(ptr, [key[1]], _TYPESTR[dt]), device="cuda")
            if dt == "bfloat16":
                view = view.view(torch.bfloat16)   # the interface has no bfloat16 code: same bits, reinterpreted
            if len(self._views) >= 512:
                self._views.clear()
            self._views[key] = view
        return view

    def all_reduce(self, t):
        if self.group.world == 1 or self.group.dist is None:
            return t
        import torch
        view = self._view(t)
        with torch.cuda.stream(self._torch_stream()):
            self.group.dist.all_reduce(view, group=self._process_group())
        return t

    def all_reduce_start(self, t):
        """Starts the in-place sum of `t` over the ranks on the communication stream, ordered after the kernels that
        produce `t`; the runtime stream is not held up. Returns a handle for all_reduce_finish."""
        if self.group.world == 1 or self.group.dist is None:
            t.eval()
            return (t, None, None)
        import torch
        view = self._view(t)
        produced = torch.cuda.Event()
        produced.record(self._torch_stream())
        comm = self._comm_stream()
        comm.wait_event(produced)
        with torch.cuda.stream(comm):
            self.group.dist.all_reduce(view, group=self._process_group())
        done = torch.cuda.Event()
        done.record(comm)
        return (t, done, view)

    def all_reduce_finish(self, handle):
        """Orders the runtime stream after the collective started by all_reduce_start and returns the summed tensor."""
        t, done, _view = handle
        if done is not None:
            self._torch_stream().wait_event(done)
        return t


def load_bert_shard(state, config, group, dtype="bfloat16"):
    """This rank's shard of a BertModel state dict (see bert.load_bert_state_dict)."""
    from .bert import load_bert_state_dict
    heads, ff = head_and_ff_ranges(config, group.rank, group.world)
    return load_bert_state_dict(state, config, dtype=dtype, head_range=heads, ff_range=ff)
