"""B200-native implementation of applegpu-runtime's transformer forward op set.

`import applegpu_runtime_b200 as gpu` exposes the same function names as the reference's
`import applegpu_runtime as gpu` for the ops on that path (python/applegpu_runtime/__init__.py:3-125);
everything executes in libapplegpu_b200.so (hand-written sm_100a CUDA behind the C ABI of
include/applegpu_b200_ffi.h). There is no CPU fallback: without the shared library the import fails.
"""
__version__ = "0.1.0"

from ._lib import load as _load, LIB_PATH  # noqa: E402

_load()  # fail loudly at import time if the native library is missing

from .api import (  # noqa: E402,F401
    GpuTensor, version, init_backend, device_name, dtype_size, from_numpy, from_numpy_shared, from_torch,
    from_torch_shared, from_bytes, aligned_numpy, tensor, eval, to_list, shape, destroy, memory_usage, tensor_count,
    add, sub, mul, div, neg, linear_fused, relu, exp, log, sqrt, scalar_mul, reshape, softmax, transpose, transpose_dims, tanh, sin,
    cos, gelu, gelu_exact, sigmoid, layer_norm, embedding, gather, index_select, attention, matmul, slice, concat,
    concat_all, add_bias, softmax_causal, argmax, cast, quantize, dequantize, sum, mean, attention_causal, abs, sign,
    pool_stats, pool_drain, set_pool_watermark, synchronize, quantize_weight, matmul_int8, set_fusion, set_matmul_path, matmul_path, set_f32_split, set_sm_margin, set_gemm_tile, set_gemm_chain, gemm_chain_enabled, gemm_chain_min_rows, gemm_chain_applies, set_attention_path,
    pipeline_status, launch_count, resolve_kernel, profile, profile_report, Tape, tape_begin, tape_end, tape_abort,
)
from .gpt2 import gpt2_forward, init_gpt2_weights, load_gpt2_state_dict, quantize_gpt2_linears, fold_gpt2_layer_norms, GPT2_SMALL, GPT2_LARGE  # noqa: E402,F401
from .bert import bert_forward, bert_forward_overlapped, init_bert_weights, load_bert_state_dict, BERT_BASE  # noqa: E402,F401
from .generate import generate, greedy_generate  # noqa: E402,F401
