/*
 * Additive entry points of the B200 build. None of these exist in the reference's
 * backend_cpp/applegpu_ffi.h: upstream reaches the same operations only through in-process Rust
 * calls from its PyO3 module (crates/python/src/metal_backend.rs -> crates/core/src/ops.rs), so
 * a C caller had no way to record them. Each function follows the conventions of
 * applegpu_b200_ffi.h and cites the Rust function whose behaviour it exposes.
 */
#ifndef APPLEGPU_B200_EXT_H
#define APPLEGPU_B200_EXT_H

#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>

#ifndef APPLEGPU_API
#  if defined(__GNUC__)
#    define APPLEGPU_API __attribute__((visibility("default")))
#  else
#    define APPLEGPU_API
#  endif
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ── host <-> device bytes (device pointers are not host-dereferenceable) ───── */
/* Stream-ordered copy into a tensor; the host buffer may be reused when the call returns
 * only if it is pageable (pinned buffers must outlive the next synchronize). */
APPLEGPU_API int32_t applegpu_ffi_upload(uint64_t tensor_id, const void* host_ptr, uint64_t nbytes);
/* Evaluates if pending, copies out, and waits. Reference: LazyRuntime::read_bytes, lazy.rs:2554-2560. */
APPLEGPU_API int32_t applegpu_ffi_read_bytes(uint64_t tensor_id, void* host_ptr, uint64_t nbytes);
/* Device address of a tensor's first element (evaluates it if pending; NULL for an unknown id or a
 * strided view). The memory stays valid while the tensor is alive; work enqueued on applegpu_stream()
 * is ordered with the runtime's own kernels, which is how a collective library reduces a tensor in
 * place between two ops. No counterpart in the reference (its buffers are host-visible). */
APPLEGPU_API void* applegpu_ffi_device_ptr(uint64_t tensor_id);
/* Same, but only enqueues the copy on the runtime stream: the bytes are defined after the next
 * applegpu_ffi_synchronize (or any blocking read). `host_ptr` should be pinned memory (a pageable
 * buffer makes the copy block) and must stay valid until then. Lets a caller issue the next forward
 * while the previous result is still in flight. No counterpart in the reference (its buffers are
 * host-visible unified memory, read in place). */
APPLEGPU_API int32_t applegpu_ffi_read_bytes_async(uint64_t tensor_id, void* host_ptr, uint64_t nbytes);
/* alloc + register_tensor + upload in one call; returns the id, 0 on failure. */
APPLEGPU_API uint64_t applegpu_ffi_from_host(const void* host_ptr, const uint64_t* dims, uint32_t ndim, int8_t dtype);
APPLEGPU_API int32_t applegpu_eager_upload(uint64_t id, const void* host_ptr, uint64_t nbytes);
APPLEGPU_API int32_t applegpu_eager_download(uint64_t id, void* host_ptr, uint64_t nbytes);

/* ── graph flavour: the rest of the transformer-forward op set ─────────────── */
/* Reference recorders: ops.rs div :364, unary ops :594-615, softmax :487-506, softmax_causal
 * :1367-1386, layer_norm :618-651, embedding :1194-1230, add_bias :1322-1361, scalar_mul :554-568,
 * argmax :1390-1413, sum / mean :1417-1470, transpose :540-552, transpose_dims :510-538, reshape
 * :570-592, slice :1234-1268, concat :1271-1316, gather :1729-1780, index_select :1784-1829, cast
 * :2299-2320, quantize :2250-2273, dequantize :2276-2296, attention :1531-1572, attention_causal
 * :1577-1618. All return the output id, 0 on failure. */
APPLEGPU_API uint64_t applegpu_ffi_div(uint64_t a_id, uint64_t b_id);
APPLEGPU_API uint64_t applegpu_ffi_exp(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_log(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_sqrt(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_tanh(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_sin(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_cos(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_abs(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_sign(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_sigmoid(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_gelu(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_gelu_exact(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_softmax(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_softmax_causal(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_layer_norm(uint64_t input_id, uint64_t gamma_id, uint64_t beta_id, float eps);
APPLEGPU_API uint64_t applegpu_ffi_embedding(uint64_t weight_id, uint64_t indices_id);
APPLEGPU_API uint64_t applegpu_ffi_add_bias(uint64_t input_id, uint64_t bias_id);
APPLEGPU_API uint64_t applegpu_ffi_scalar_mul(uint64_t input_id, float scale);
APPLEGPU_API uint64_t applegpu_ffi_argmax(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_sum(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_mean(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_transpose(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_transpose_dims(uint64_t input_id, uint32_t dim0, uint32_t dim1);
APPLEGPU_API uint64_t applegpu_ffi_reshape(uint64_t input_id, const uint64_t* dims, uint32_t ndim);
APPLEGPU_API uint64_t applegpu_ffi_slice(uint64_t input_id, uint32_t dim, uint64_t start, uint64_t end);
APPLEGPU_API uint64_t applegpu_ffi_concat(uint64_t a_id, uint64_t b_id, uint32_t dim);
APPLEGPU_API uint64_t applegpu_ffi_gather(uint64_t input_id, uint32_t dim, uint64_t index_id);
APPLEGPU_API uint64_t applegpu_ffi_index_select(uint64_t input_id, uint32_t dim, uint64_t index_id);
APPLEGPU_API uint64_t applegpu_ffi_cast(uint64_t input_id, int8_t target_dtype);
APPLEGPU_API uint64_t applegpu_ffi_quantize(uint64_t input_id, int8_t target_dtype, float scale, int32_t zero_point);
APPLEGPU_API uint64_t applegpu_ffi_dequantize(uint64_t input_id, int8_t target_dtype, float scale, int32_t zero_point);
APPLEGPU_API uint64_t applegpu_ffi_attention(uint64_t q_id, uint64_t k_id, uint64_t v_id);
APPLEGPU_API uint64_t applegpu_ffi_attention_causal(uint64_t q_id, uint64_t k_id, uint64_t v_id);

/* Per-output-channel symmetric int8 weights (no upstream counterpart; upstream lists
 * int8-weight matmul as backlog). quantize_weight: w [N,K] float -> *out_q [N,K] int8 and
 * *out_scales [N] f32 with scale[n] = max|w[n,:]|/127, evaluated immediately.
 * matmul_int8: x [..,M,K] @ (q * scale)^T -> [..,M,N], dequantisation fused into the GEMM. */
/* x [.., M, K] @ w [K, N] with the whole epilogue named up front (0 = absent): bias [N], residual [.., M, N], act
 * (0 none, 1 tanh-GELU, 2 erf-GELU, 3 ReLU), and layer_norm folded into the product. With ln_colsum [N] (float32) and
 * ln_stats [M, 2] (int64: sum and sum of squares of each row of x over K, in 2^-28 fixed point) the result is
 * act(rstd * (x @ w - mean * ln_colsum) + bias), i.e. layer_norm(x) @ w0 + b0 when w = gamma * w0 row-wise,
 * ln_colsum = column sums of w, bias = beta @ w0 + b0. With stats_out [M, 2] (int64) the (sum, sum of squares) of every
 * stored row are added into it (64-bit integer atomics on fixed-point values: associative, so the result does not depend
 * on the order in which CTAs finish; it must hold zeros), in the form a following call takes as ln_stats; with
 * stats_zero [M, 2] (int64) those rows of it are cleared. One kernel launch; tensor-core path only (16-bit dtypes,
 * TMA-compatible operands), an error otherwise. No counterpart in the reference. */
APPLEGPU_API uint64_t applegpu_ffi_linear_fused(uint64_t x_id, uint64_t w_id, uint64_t bias_id, uint64_t residual_id, int32_t act, uint64_t ln_colsum_id,
                                                uint64_t ln_stats_id, float ln_eps, uint64_t stats_out_id, uint64_t stats_zero_id);
APPLEGPU_API int32_t applegpu_ffi_quantize_weight(uint64_t weight_id, uint64_t* out_q_id, uint64_t* out_scales_id);
APPLEGPU_API uint64_t applegpu_ffi_matmul_int8(uint64_t x_id, uint64_t q_id, uint64_t scales_id);

/* ── eager flavour: the same ops, executed immediately ─────────────────────── */
APPLEGPU_API uint8_t* applegpu_eager_gelu_exact(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_softmax_causal(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_add_bias(uint64_t input_id, uint64_t bias_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_argmax(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_gather(uint64_t input_id, uint32_t dim, uint64_t index_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_index_select(uint64_t input_id, uint32_t dim, uint64_t index_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_cast(uint64_t input_id, int8_t target_dtype, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_quantize(uint64_t input_id, int8_t target_dtype, float scale, int32_t zero_point, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_dequantize(uint64_t input_id, int8_t target_dtype, float scale, int32_t zero_point, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_attention(uint64_t q_id, uint64_t k_id, uint64_t v_id, bool causal, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_unary(uint64_t input_id, const char* op_name, uint64_t* out_id);
/* Linear layer with its epilogue in the GEMM kernel: act(x @ w * 1 + bias) + residual.
 * bias_id / residual_id may be 0; act: 0 none, 1 tanh-GELU, 2 erf-GELU, 3 ReLU. w is [K,N], or
 * [N,K] when transpose_w. */
APPLEGPU_API uint8_t* applegpu_eager_linear(uint64_t x_id, uint64_t w_id, uint64_t bias_id, uint64_t residual_id, int32_t act, bool transpose_w, uint64_t* out_id);

/* What a frontend whose buffers live in DEVICE memory needs beside the reference's eager ABI (the reference's C++ shim
 * memcpy's and memsets through the returned pointers, backend_cpp/applegpu_backend.cpp:267-342, :691-749; these three
 * calls replace that):
 *   view_as  a typed, strided view over the buffer of `base` (any dtype, byte offset from the base's first byte);
 *            shares the buffer, is freed like any other id, fails if it would reach past the end of the buffer;
 *   copy     dst <- src on the device, both possibly strided, same shape (same dtype, or contiguous with conversion);
 *   fill     every element of the tensor (contiguous or a view) set to the low bytes of bit_pattern. */
APPLEGPU_API uint8_t* applegpu_eager_view_as(uint64_t base_id, int8_t dtype, const uint64_t* shape, const uint64_t* strides, uint32_t ndim, uint64_t byte_offset, uint64_t* out_id);
APPLEGPU_API int32_t applegpu_eager_copy(uint64_t dst_id, uint64_t src_id);
APPLEGPU_API int32_t applegpu_eager_fill(uint64_t id, uint64_t bit_pattern);

/* ── runtime services ──────────────────────────────────────────────────────── */
/* Metadata-only mode for hosts without a GPU: ids, shapes, validation, the fusion pass and
 * applegpu_ffi_plan work; anything that would launch a kernel fails. Must be the first init call. */
APPLEGPU_API bool applegpu_ffi_init_dry(void);
/* Writes the launch plan of eval(tensor_id) after the fusion pass, one kernel per line, without
 * running it. Returns the full length (may exceed cap), -1 on failure. */
APPLEGPU_API int64_t applegpu_ffi_plan(uint64_t tensor_id, char* buf, uint64_t cap);
APPLEGPU_API int32_t applegpu_ffi_is_pending(uint64_t tensor_id);
/* Toggle the reference's element-wise chain rule and this build's graph-level rewrites. */
APPLEGPU_API void applegpu_ffi_set_fusion(bool elementwise_chains, bool patterns);
/* out[0..6] = hits, misses, pooled_bytes, bucket_count, live_bytes, peak_live_bytes, live_buffers.
 * Reference: BufferPool::stats, pool.rs:100-108 (first four). */
APPLEGPU_API void applegpu_pool_stats(uint64_t* out7);
APPLEGPU_API void applegpu_pool_drain(void);
APPLEGPU_API void applegpu_pool_set_watermark(uint64_t max_pooled_bytes);
APPLEGPU_API int32_t applegpu_pool_prewarm(const uint64_t* sizes, uint32_t n);
/* Host-side fault injection for tests: the next n device allocations report failure. */
APPLEGPU_API void applegpu_pool_fail_next(int32_t n);
APPLEGPU_API uint64_t applegpu_memory_usage(void);
APPLEGPU_API uint64_t applegpu_tensor_count(void);
/* The CUDA stream (cudaStream_t) all work is enqueued on, and the device ordinal. */
APPLEGPU_API void* applegpu_stream(void);
APPLEGPU_API int32_t applegpu_device(void);
APPLEGPU_API const char* applegpu_device_name(void);
/* Kernel launches issued since process start. */
APPLEGPU_API uint64_t applegpu_launch_count(void);
/* Which kernel family a matmul of these tensors would take: "tcgen05", "simt", or NULL on error. */
APPLEGPU_API const char* applegpu_matmul_path(uint64_t a_id, uint64_t b_id, bool eager);
/* 0 auto, 1 force the CUDA-core kernel, 2 require a tcgen05 kernel, 3 tcgen05 with single-CTA
 * tiles only, 4 tcgen05 with CTA-pair 256 x 256 tiles (cta_group::2) where the shape is large enough. */
APPLEGPU_API void applegpu_set_matmul_path(int32_t mode);
/* Tuning override of the tensor-core kernel's tile shape: 0 = chosen per problem by the cost model (default);
 * 1256 / 1128 = CTA-pair tiles of 256 x 256 / 256 x 128; 256 / 192 / 128 = single-CTA tiles of 128 x that width. */
APPLEGPU_API void applegpu_set_gemm_tile(int32_t code);
/* Keeps `n` SMs out of the grids of the persistent kernels (GEMM, attention, row kernels), for a collective that runs
 * on another stream beside them. 0 (default) uses every SM. */
APPLEGPU_API void applegpu_set_sm_margin(int32_t n);
/* Chained linears (default on; APPLEGPU_GEMM_CHAIN=0 sets the initial value to off): inside one evaluation, consecutive
 * 16-bit fused linears with [K, N] weights where each reads the previous one's result (out-projection -> FC1 -> FC2 -> the
 * next block's QKV) are launched as ONE tensor-core kernel whose tiles wait, row block by row block, for the tiles that
 * produce their rows. Results are bit-identical to the separate launches. */
APPLEGPU_API void applegpu_set_gemm_chain(bool on);
APPLEGPU_API bool applegpu_gemm_chain_enabled(void);
/* Linears with fewer rows than this are never chained (default 4096, APPLEGPU_GEMM_CHAIN_MIN_ROWS: below about 16 row
 * blocks of 256 most tiles would wait for the tiles just before them and separate launches are faster). */
APPLEGPU_API void applegpu_set_gemm_chain_min_rows(int64_t rows);
APPLEGPU_API int64_t applegpu_gemm_chain_min_rows(void);
/* float32 matmuls of at least 2 GFLOP run on the tensor cores as a three-term bf16 split with float32
 * accumulation (error ~2^-22 relative); false keeps every float32 product on the CUDA-core kernel. */
APPLEGPU_API void applegpu_set_f32_split(bool on);
/* Host-visible mode. Upstream every returned `uint8_t*` is host-dereferenceable (shared Metal buffers;
 * backend_cpp/applegpu_backend.cpp:264-342 copies with memcpy, :691-749 builds CPU views over them). By
 * default this library returns plain device pointers. With APPLEGPU_HOST_VISIBLE=1 in the environment, or
 * applegpu_set_host_visible(1) before the first init call, the buffer pool is backed by CUDA managed memory:
 * the host may read and write a returned pointer once applegpu_eager_flush_and_wait / _synchronize /
 * applegpu_ffi_eval has returned, and every operand is moved back to the device ahead of the kernels that
 * use it. Returns 0, or -1 when the device context already exists in the other mode. */
APPLEGPU_API int32_t applegpu_set_host_visible(int32_t on);
APPLEGPU_API int32_t applegpu_host_visible(void);
/* 0 auto (single-kernel attention when head dim is 64 and dtype is f16/bf16), 1 always compose
 * attention from GEMM + softmax + GEMM with materialised scores. */
APPLEGPU_API void applegpu_set_attention_path(int32_t mode);
/* Reads and clears the pipeline status word of the tcgen05 kernels (0 = no bounded wait gave up). Every
 * blocking point of the library (read_bytes / read_f32 / eager_download, applegpu_ffi_synchronize,
 * applegpu_eager_flush_and_wait, applegpu_marker_wait) makes the same check once the stream is idle and
 * reports a non-zero word as an error ("tensor-core pipeline wait timed out (code N)"), so a caller of
 * the reference ABI alone cannot read an undefined result as success. Codes: 1 a TMA thread waiting for a free pipeline
 * stage, 2 the MMA thread waiting for a free accumulator, 3 for loaded operands, 4 an epilogue warp waiting for a full
 * accumulator, 5 an int8 converter warp waiting for raw weights, 6 a TMA thread of the chained kernel waiting for the row
 * block its tile reads, 8 that kernel's announcer waiting for a tile's stores, 31 the grid barrier of the persistent
 * decode kernel; the attention kernel uses 10 to 29. */
APPLEGPU_API int32_t applegpu_pipeline_status(void);
/* Test hook (no counterpart in the reference): launches one thread that waits, for at most `limit_us`
 * microseconds (capped at 50 ms), on a barrier nothing arrives at, then records `code` in the pipeline
 * status word and returns. It exercises the error path of the bounded waits without a fault or a hang. */
APPLEGPU_API int32_t applegpu_test_wait_runs_out(int32_t code, uint32_t limit_us);
/* CUDA-event stopwatch on the runtime stream. */
/* Op tapes: record the graph-flavour ops one pass of a host program issues, then re-record the same
 * ops on new inputs with one call (the per-op host cost of a Python driver is paid once). Between
 * tape_begin and tape_end every applegpu_ffi_* op call is noted; tensors in `var_inputs` become the
 * tape's parameters, any other tensor an op reads (weights) is reused by id and must stay alive.
 * tape_end returns a handle (0 on failure). tape_replay returns the number of ops recorded (-1 on
 * error) and writes the new ids of the tape's outputs; the caller owns those ids (free them as
 * usual), every other value is released as soon as its last consumer has run. Shapes are inferred
 * again on replay, so one tape serves inputs of different extents (a growing KV cache) as long as
 * the explicit shape arguments recorded on it still apply. The reference's counterpart is its
 * compiled-graph path (crates/core/src/compiled_graph.rs), which serialises the op list on the
 * Python side instead. */
APPLEGPU_API int32_t applegpu_ffi_tape_begin(const uint64_t* var_inputs, uint32_t n_var);
APPLEGPU_API uint64_t applegpu_ffi_tape_end(const uint64_t* outputs, uint32_t n_out);
APPLEGPU_API void applegpu_ffi_tape_abort(void);
APPLEGPU_API int32_t applegpu_ffi_tape_replay(uint64_t tape, const uint64_t* var_inputs, uint32_t n_var, uint64_t* out_ids, uint32_t n_out);
/* Benchmark helper: replays single-output tapes that take no variable inputs round robin `iters` times in one call,
 * evaluating each result and keeping the last `keep` (1..64) results alive. Returns 0, -1 on error. */
APPLEGPU_API int32_t applegpu_ffi_tape_replay_loop(const uint64_t* tapes, uint32_t n_tapes, uint32_t iters, uint32_t keep);
/* Compiled-graph executor: runs a serialized op list on the eager runtime in one call and returns the
 * number of outputs written (-1 on error, text in applegpu_eager_last_error). Replaces
 * applegpu_eager_execute_graph of the reference (crates/core/src/eager_ffi.rs:661-708; wire format and
 * op codes of crates/core/src/compiled_graph.rs:7-9,44-58), which its torch.compile backend calls
 * (python/applegpu_runtime/compile_backend.py). out_ptrs receive device pointers. */
APPLEGPU_API int32_t applegpu_eager_execute_graph(const uint8_t* ops_data, uint32_t ops_len, const uint64_t* input_tids, uint32_t n_inputs,
                                                  const uint16_t* output_indices, uint32_t n_outputs, uint64_t* out_tids, uint8_t** out_ptrs);
/* A marker is a point in the runtime stream; wait blocks the host until everything enqueued before
 * the marker (kernels, copies of applegpu_ffi_read_bytes_async) has completed. 0 = failure. Lets a
 * serving loop keep one step in flight: record after step i, build step i+1, then wait for i. */
APPLEGPU_API uint64_t applegpu_marker_record(void);
APPLEGPU_API int32_t applegpu_marker_wait(uint64_t marker);
APPLEGPU_API int32_t applegpu_timer_start(void);
APPLEGPU_API float applegpu_timer_stop_ms(void);
/* Evicts the L2 by streaming writes over a scratch buffer larger than the cache. */
APPLEGPU_API int32_t applegpu_flush_l2(void);
/* Per-kernel timing with CUDA events on the runtime stream. While enabled, every executed graph
 * node is bracketed by two events; the report (one line per kernel: "name launches total_ms work",
 * work = algorithmic flops for contractions, bytes otherwise) waits for the stream and resolves
 * them. Returns the full length of the report. */
APPLEGPU_API void applegpu_profile_enable(bool on);
APPLEGPU_API void applegpu_profile_clear(void);
/* Restricts the spans to nodes whose kernel name starts with one of the comma-separated prefixes ("" or NULL: all).
 * Timing one kernel family leaves the rest of the step running as it normally does (no event between its kernels). */
APPLEGPU_API void applegpu_profile_filter(const char* prefixes);
APPLEGPU_API int64_t applegpu_profile_report(char* buf, uint64_t cap);
/* Kernel name the registry resolves for (base name, dtype), e.g. ("matmul", 10) -> "matmul_bf16".
 * Reference: KernelRegistry::resolve_kernel, compute.rs:1478-1567. Returns NULL if unsupported. */
APPLEGPU_API const char* applegpu_resolve_kernel(const char* base_name, int8_t dtype);

/* ── GPT-2 greedy decoder: preallocated KV cache, one captured step ────────────
 * Counterpart of the reference's generate loop (python/applegpu_runtime/models/generate.py:83-127 over
 * models/gpt2.py:47-180), which re-records the forward for every token and grows its KV cache by concat
 * (gpt2.py:122-127). A decoder owns a [batch, heads, max_len, 64] key and value cache per layer; a step is a fixed
 * list of kernel launches (the current length and the picked tokens live in device memory), captured once as a
 * CUDA graph and replayed.
 *   create:  weight_ids = wte, wpe, ln_f.weight, ln_f.bias, then per layer ln_1.weight, ln_1.bias, c_attn.weight
 *            [d, 3d], c_attn.bias, attn c_proj.weight [d, d], its bias, ln_2.weight, ln_2.bias, c_fc.weight [d, 4d],
 *            its bias, mlp c_proj.weight [4d, d], its bias (graph-flavour tensor ids, one float dtype, head
 *            dimension 64, batch <= 16). Returns a handle, 0 on failure (applegpu_ffi_last_error).
 *   prefill: kv_ids = k0, v0, k1, v1, ... each [batch, heads, prompt_len, 64] (the cache a prompt forward returned),
 *            first_tokens_id = int32 [batch], the tokens picked from the prompt's last logits.
 *   steps:   runs n_steps steps (each consumes the previous token, appends to the cache, picks the next token as the
 *            first index of the row maximum of the logits) and writes the n_steps x batch picked tokens to
 *            host_tokens. use_graph = false issues the launches one by one instead of replaying the captured step. */
APPLEGPU_API uint64_t applegpu_gpt2_decoder_create(const uint64_t* weight_ids, uint32_t n_weights, uint32_t n_layer, uint32_t n_head, uint32_t n_embd,
                                                  uint32_t vocab, uint32_t n_positions, uint32_t batch, uint32_t max_len);
APPLEGPU_API int32_t applegpu_gpt2_decoder_prefill(uint64_t decoder, const uint64_t* kv_ids, uint32_t n_kv, uint64_t first_tokens_id, uint32_t prompt_len);
APPLEGPU_API int32_t applegpu_gpt2_decoder_steps(uint64_t decoder, uint32_t n_steps, int32_t* host_tokens, bool use_graph);
APPLEGPU_API int32_t applegpu_gpt2_decoder_launches_per_step(uint64_t decoder);
APPLEGPU_API int32_t applegpu_gpt2_decoder_uses_graph(uint64_t decoder);
/* engine 0 (default): one kernel per op, chained by programmatic dependent launches inside the captured step. engine 1:
 * embeddings and all layers of a step as one persistent cooperative kernel with grid-wide barriers between phases; the
 * same arithmetic in the same order, so the same tokens. Measured slower (0.65 against 0.50 ms per step for GPT-2-small at
 * batch 8: a software grid barrier costs about what a programmatic kernel boundary costs, and the per-op kernels keep
 * more CTAs resident); kept as an option. */
APPLEGPU_API int32_t applegpu_gpt2_decoder_set_engine(uint64_t decoder, int32_t engine);
APPLEGPU_API void applegpu_gpt2_decoder_destroy(uint64_t decoder);

/* ── attention without device allocation ───────────────────────────────────────
 * No counterpart in the reference.
 *
 * Every other attention entry point takes its score matrix from the buffer pool, which may call
 * cudaMallocAsync. This one is for callers that are not allowed to allocate device memory when
 * they need attention: a serving loop with a fixed memory budget, a plugin whose host
 * application owns every device buffer, code running between another framework's allocator
 * checkpoints. It computes softmax[_causal](Q K^T / sqrt(d_k)) V on caller-owned DEVICE pointers
 * and calls no cudaMalloc / cudaFree / pool routine; its scratch is a fixed array of
 * APPLEGPU_NOALLOC_SCRATCH_BYTES that is part of the library image (each GPU that loads the
 * library holds it until the process exits).
 *
 *   q [batch_heads, q_len, d_k], k [batch_heads, kv_len, d_k], v [batch_heads, kv_len, d_v],
 *   out [batch_heads, q_len, d_v]; all contiguous, all of `dtype` (0 f32, 1 f16, 10 bf16).
 *   cuda_stream: a cudaStream_t (NULL = the legacy default stream). Work is enqueued, not awaited.
 *
 * Limit: batch_heads * q_len * kv_len * sizeof(dtype) must not exceed
 * APPLEGPU_NOALLOC_SCRATCH_BYTES; larger problems are rejected with -1 and a message in
 * applegpu_ffi_last_error(). The first call on a device looks up the scratch address for that
 * device (with that device current); make that first call before any stream capture. All calls
 * share the one scratch array, which keeps the previous call's contents: calls whose GPU work
 * overlaps (different streams, different threads) race on it and must be serialised by the caller.
 * One process serves one GPU: a call made with another device current than the one the process's
 * kernels first ran on is rejected. Returns 0 on success.
 *
 * applegpu_attention_noalloc_status(stream): the tensor-core GEMMs inside bound every wait and record
 * a code in this entry point's own status word when one gives up (applegpu_pipeline_status does not
 * see that word). The status call waits for `cuda_stream`, copies the word to the host without
 * allocating, and returns it: 0 = the last call completed, > 0 = a wait timed out and `out` is
 * undefined, -1 = the query failed. */
#define APPLEGPU_NOALLOC_SCRATCH_BYTES (64ull << 20)
APPLEGPU_API int32_t applegpu_attention_noalloc(const void* q, const void* k, const void* v, void* out, int8_t dtype, uint64_t batch_heads, uint64_t q_len, uint64_t kv_len, uint64_t d_k, uint64_t d_v, bool causal, void* cuda_stream);
APPLEGPU_API int32_t applegpu_attention_noalloc_status(void* cuda_stream);

#ifdef __cplusplus
}
#endif

#endif /* APPLEGPU_B200_EXT_H */
