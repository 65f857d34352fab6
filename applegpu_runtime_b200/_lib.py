"""ctypes binding of libapplegpu_b200.so (the C ABI in include/applegpu_b200_ffi.h and
include/applegpu_b200_ext.h).

This is the stub a maintainer of the reference would write to bind the library from Python;
the reference binds the same symbols in python/applegpu_runtime/cpp_backend.py:39-51 and
python/applegpu_runtime/compile_backend.py:41-60. Loading fails loudly when the shared
library is missing: there is no CPU fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libapplegpu_b200.so")

u8p = ctypes.POINTER(ctypes.c_uint8)
u64 = ctypes.c_uint64
u64p = ctypes.POINTER(ctypes.c_uint64)
u32 = ctypes.c_uint32
u32p = ctypes.POINTER(ctypes.c_uint32)
i8 = ctypes.c_int8
i32 = ctypes.c_int32
i64 = ctypes.c_int64
f32 = ctypes.c_float
vp = ctypes.c_void_p
cbool = ctypes.c_bool
cstr = ctypes.c_char_p

# name -> (restype, argtypes). The first block is the reference's header, the second the additive one.
REFERENCE_SYMBOLS = {
    "applegpu_ffi_init": (cbool, []),
    "applegpu_ffi_last_error": (cstr, []),
    "applegpu_ffi_alloc": (vp, [u64, i8, u64p]),
    "applegpu_ffi_free": (None, [u64]),
    "applegpu_ffi_register_tensor": (i32, [u64, u64p, u32, i8]),
    "applegpu_ffi_shape": (i32, [u64, u64p, u32p]),
    "applegpu_ffi_dtype": (i8, [u64]),
    "applegpu_ffi_add": (u64, [u64, u64]),
    "applegpu_ffi_matmul": (u64, [u64, u64]),
    "applegpu_ffi_relu": (u64, [u64]),
    "applegpu_ffi_mul": (u64, [u64, u64]),
    "applegpu_ffi_sub": (u64, [u64, u64]),
    "applegpu_ffi_neg": (u64, [u64]),
    "applegpu_ffi_copy": (i32, [u64, u64]),
    "applegpu_ffi_add_out": (vp, [u64, u64, u64p]),
    "applegpu_ffi_mul_out": (vp, [u64, u64, u64p]),
    "applegpu_ffi_sub_out": (vp, [u64, u64, u64p]),
    "applegpu_ffi_matmul_out": (vp, [u64, u64, u64p]),
    "applegpu_ffi_relu_out": (vp, [u64, u64p]),
    "applegpu_ffi_neg_out": (vp, [u64, u64p]),
    "applegpu_ffi_div_out": (vp, [u64, u64, u64p]),
    "applegpu_ffi_threshold_backward_out": (vp, [u64, u64, f32, u64p]),
    "applegpu_ffi_scalar_mul_out": (vp, [u64, f32, u64p]),
    "applegpu_ffi_mean_all_out": (vp, [u64, u64p]),
    "applegpu_ffi_eval": (i32, [u64]),
    "applegpu_ffi_synchronize": (None, []),
    "applegpu_ffi_read_f32": (i32, [u64, ctypes.POINTER(f32), u64]),
    "applegpu_eager_init": (cbool, []),
    "applegpu_eager_last_error": (cstr, []),
    "applegpu_eager_alloc": (vp, [u64p, u32, i8, u64p]),
    "applegpu_eager_free": (None, [u64]),
    "applegpu_eager_register_shape": (i32, [u64, u64p, u32]),
    "applegpu_eager_shape": (i32, [u64, u64p, u32p]),
    "applegpu_eager_dtype": (i8, [u64]),
    "applegpu_eager_add": (vp, [u64, u64, u64p]),
    "applegpu_eager_sub": (vp, [u64, u64, u64p]),
    "applegpu_eager_mul": (vp, [u64, u64, u64p]),
    "applegpu_eager_div": (vp, [u64, u64, u64p]),
    "applegpu_eager_relu": (vp, [u64, u64p]),
    "applegpu_eager_neg": (vp, [u64, u64p]),
    "applegpu_eager_matmul": (vp, [u64, u64, u64p]),
    "applegpu_eager_matmul_ex": (vp, [u64, u64, cbool, cbool, u64p]),
    "applegpu_eager_threshold_backward": (vp, [u64, u64, f32, u64p]),
    "applegpu_eager_scalar_mul": (vp, [u64, f32, u64p]),
    "applegpu_eager_mean_all": (vp, [u64, u64p]),
    "applegpu_eager_sum_dim": (vp, [u64, i64, cbool, u64p]),
    "applegpu_eager_create_view": (vp, [u64, u64p, u64p, u32, u64, u64p]),
    "applegpu_eager_add_inplace": (i32, [u64, u64]),
    "applegpu_eager_add_scaled_inplace": (i32, [u64, u64, f32]),
    "applegpu_eager_flush_and_wait": (None, []),
    "applegpu_eager_synchronize": (None, []),
    "applegpu_eager_embedding": (vp, [u64, u64, u64p]),
    "applegpu_eager_layer_norm": (vp, [u64, u64, u64, f32, u64p]),
    "applegpu_eager_gelu": (vp, [u64, u64p]),
    "applegpu_eager_softmax": (vp, [u64, u64p]),
    "applegpu_eager_find_by_data_ptr": (u64, [vp]),
}

EXT_SYMBOLS = {
    "applegpu_ffi_upload": (i32, [u64, vp, u64]),
    "applegpu_ffi_read_bytes": (i32, [u64, vp, u64]),
    "applegpu_ffi_read_bytes_async": (i32, [u64, vp, u64]),
    "applegpu_ffi_device_ptr": (vp, [u64]),
    "applegpu_ffi_tape_begin": (i32, [vp, u32]),
    "applegpu_ffi_tape_end": (u64, [vp, u32]),
    "applegpu_ffi_tape_abort": (None, []),
    "applegpu_ffi_tape_replay_loop": (i32, [u64p, u32, u32, u32]),
    "applegpu_ffi_tape_replay": (i32, [u64, vp, u32, vp, u32]),
    "applegpu_ffi_from_host": (u64, [vp, u64p, u32, i8]),
    "applegpu_eager_upload": (i32, [u64, vp, u64]),
    "applegpu_eager_download": (i32, [u64, vp, u64]),
    "applegpu_ffi_div": (u64, [u64, u64]),
    "applegpu_ffi_exp": (u64, [u64]),
    "applegpu_ffi_log": (u64, [u64]),
    "applegpu_ffi_sqrt": (u64, [u64]),
    "applegpu_ffi_tanh": (u64, [u64]),
    "applegpu_ffi_sin": (u64, [u64]),
    "applegpu_ffi_cos": (u64, [u64]),
    "applegpu_ffi_abs": (u64, [u64]),
    "applegpu_ffi_sign": (u64, [u64]),
    "applegpu_ffi_sigmoid": (u64, [u64]),
    "applegpu_ffi_gelu": (u64, [u64]),
    "applegpu_ffi_gelu_exact": (u64, [u64]),
    "applegpu_ffi_softmax": (u64, [u64]),
    "applegpu_ffi_softmax_causal": (u64, [u64]),
    "applegpu_ffi_layer_norm": (u64, [u64, u64, u64, f32]),
    "applegpu_ffi_embedding": (u64, [u64, u64]),
    "applegpu_ffi_add_bias": (u64, [u64, u64]),
    "applegpu_ffi_scalar_mul": (u64, [u64, f32]),
    "applegpu_ffi_argmax": (u64, [u64]),
    "applegpu_ffi_sum": (u64, [u64]),
    "applegpu_ffi_mean": (u64, [u64]),
    "applegpu_ffi_transpose": (u64, [u64]),
    "applegpu_ffi_transpose_dims": (u64, [u64, u32, u32]),
    "applegpu_ffi_reshape": (u64, [u64, u64p, u32]),
    "applegpu_ffi_slice": (u64, [u64, u32, u64, u64]),
    "applegpu_ffi_concat": (u64, [u64, u64, u32]),
    "applegpu_ffi_gather": (u64, [u64, u32, u64]),
    "applegpu_ffi_index_select": (u64, [u64, u32, u64]),
    "applegpu_ffi_cast": (u64, [u64, i8]),
    "applegpu_ffi_quantize": (u64, [u64, i8, f32, i32]),
    "applegpu_ffi_dequantize": (u64, [u64, i8, f32, i32]),
    "applegpu_ffi_attention": (u64, [u64, u64, u64]),
    "applegpu_ffi_attention_causal": (u64, [u64, u64, u64]),
    "applegpu_ffi_quantize_weight": (i32, [u64, u64p, u64p]),
    "applegpu_ffi_matmul_int8": (u64, [u64, u64, u64]),
    "applegpu_eager_gelu_exact": (vp, [u64, u64p]),
    "applegpu_eager_softmax_causal": (vp, [u64, u64p]),
    "applegpu_eager_add_bias": (vp, [u64, u64, u64p]),
    "applegpu_eager_argmax": (vp, [u64, u64p]),
    "applegpu_eager_gather": (vp, [u64, u32, u64, u64p]),
    "applegpu_eager_index_select": (vp, [u64, u32, u64, u64p]),
    "applegpu_eager_cast": (vp, [u64, i8, u64p]),
    "applegpu_eager_quantize": (vp, [u64, i8, f32, i32, u64p]),
    "applegpu_eager_dequantize": (vp, [u64, i8, f32, i32, u64p]),
    "applegpu_eager_attention": (vp, [u64, u64, u64, cbool, u64p]),
    "applegpu_eager_unary": (vp, [u64, cstr, u64p]),
    "applegpu_eager_view_as": (vp, [u64, i8, u64p, u64p, u32, u64, u64p]),
    "applegpu_eager_copy": (i32, [u64, u64]),
    "applegpu_eager_fill": (i32, [u64, u64]),
    "applegpu_eager_linear": (vp, [u64, u64, u64, u64, i32, cbool, u64p]),
    "applegpu_ffi_init_dry": (cbool, []),
    "applegpu_ffi_plan": (i64, [u64, ctypes.c_char_p, u64]),
    "applegpu_ffi_is_pending": (i32, [u64]),
    "applegpu_ffi_set_fusion": (None, [cbool, cbool]),
    "applegpu_pool_stats": (None, [u64p]),
    "applegpu_pool_drain": (None, []),
    "applegpu_pool_set_watermark": (None, [u64]),
    "applegpu_pool_prewarm": (i32, [u64p, u32]),
    "applegpu_pool_fail_next": (None, [i32]),
    "applegpu_memory_usage": (u64, []),
    "applegpu_tensor_count": (u64, []),
    "applegpu_stream": (vp, []),
    "applegpu_device": (i32, []),
    "applegpu_device_name": (cstr, []),
    "applegpu_launch_count": (u64, []),
    "applegpu_matmul_path": (cstr, [u64, u64, cbool]),
    "applegpu_set_matmul_path": (None, [i32]),
    "applegpu_set_gemm_tile": (None, [i32]),
    "applegpu_set_sm_margin": (None, [i32]),
    "applegpu_set_gemm_chain": (None, [ctypes.c_bool]),
    "applegpu_gemm_chain_enabled": (ctypes.c_bool, []),
    "applegpu_set_gemm_chain_min_rows": (None, [ctypes.c_int64]),
    "applegpu_gemm_chain_min_rows": (ctypes.c_int64, []),
    "applegpu_ffi_linear_fused": (u64, [u64, u64, u64, u64, i32, u64, u64, ctypes.c_float, u64, u64]),
    "applegpu_set_f32_split": (None, [ctypes.c_bool]),
    "applegpu_set_host_visible": (i32, [i32]),
    "applegpu_host_visible": (i32, []),
    "applegpu_set_attention_path": (None, [i32]),
    "applegpu_pipeline_status": (i32, []),
    "applegpu_eager_execute_graph": (i32, [vp, u32, vp, u32, vp, u32, vp, vp]),
    "applegpu_marker_record": (u64, []),
    "applegpu_marker_wait": (i32, [u64]),
    "applegpu_timer_start": (i32, []),
    "applegpu_timer_stop_ms": (f32, []),
    "applegpu_flush_l2": (i32, []),
    "applegpu_profile_enable": (None, [cbool]),
    "applegpu_profile_clear": (None, []),
    "applegpu_profile_filter": (None, [cstr]),
    "applegpu_profile_report": (i64, [ctypes.c_char_p, u64]),
    "applegpu_resolve_kernel": (cstr, [cstr, i8]),
    "applegpu_attention_noalloc": (i32, [vp, vp, vp, vp, i8, u64, u64, u64, u64, u64, cbool, vp]),
    "applegpu_attention_noalloc_status": (i32, [vp]),
    "applegpu_gpt2_decoder_create": (u64, [u64p, u32, u32, u32, u32, u32, u32, u32, u32]),
    "applegpu_gpt2_decoder_prefill": (i32, [u64, u64p, u32, u64, u32]),
    "applegpu_gpt2_decoder_steps": (i32, [u64, u32, vp, cbool]),
    "applegpu_gpt2_decoder_launches_per_step": (i32, [u64]),
    "applegpu_gpt2_decoder_uses_graph": (i32, [u64]),
    "applegpu_gpt2_decoder_set_engine": (i32, [u64, i32]),
    "applegpu_gpt2_decoder_destroy": (None, [u64]),
    "applegpu_test_wait_runs_out": (i32, [i32, u32]),
}

_lib = None


def load():
    """Load the shared library and declare every prototype. Raises if the library is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C applegpu_runtime_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). This package has no CPU fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for table in (REFERENCE_SYMBOLS, EXT_SYMBOLS):
        for name, (res, args) in table.items():
            fn = getattr(lib, name)  # AttributeError here means the .so and the headers disagree
            fn.restype = res
            fn.argtypes = args
    _lib = lib
    return lib
