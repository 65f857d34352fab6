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
"""
import ctypes

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

    def __init__(self, group):
        self.group = group
        self._stream = None

    def _torch_stream(self):
        import torch
        if self._stream is None:
            handle = _lib.load().applegpu_stream()
            self._stream = torch.cuda.ExternalStream(int(handle or 0))
        return self._stream

    def all_reduce(self, t):
        if self.group.world == 1 or self.group.dist is None:
            return t
        import torch
        lib = _lib.load()
        ptr = lib.applegpu_ffi_device_ptr(ctypes.c_uint64(t.id))
        if not ptr:
            raise ValueError(lib.applegpu_ffi_last_error().decode())
        dt = t.dtype
        view = torch.as_tensor(_DevMem(ptr, [int(np.prod(t.shape))], _TYPESTR[dt]), device="cuda")
        if dt == "bfloat16":
            view = view.view(torch.bfloat16)   # the interface has no bfloat16 code: same bits, reinterpreted
        with torch.cuda.stream(self._torch_stream()):
            self.group.dist.all_reduce(view)
        return t


def load_bert_shard(state, config, group, dtype="bfloat16"):
    """This rank's shard of a BertModel state dict (see bert.load_bert_state_dict)."""
    from .bert import load_bert_state_dict
    heads, ff = head_and_ff_ranges(config, group.rank, group.world)
    return load_bert_state_dict(state, config, dtype=dtype, head_range=heads, ff_range=ff)
