/*
 * C ABI of the transformer-forward op set, B200 build.
 *
 * Every prototype in this file has the same name, argument list and return convention as the
 * reference's backend_cpp/applegpu_ffi.h (lines cited per group), which is implemented there by
 * crates/core/src/backend_ffi.rs and crates/core/src/eager_ffi.rs. A caller written against the
 * reference header (the PrivateUse1 shim backend_cpp/applegpu_backend.cpp, the ctypes users in
 * python/applegpu_runtime/cpp_backend.py and compile_backend.py) links against
 * libapplegpu_b200.so without source changes, with one difference it must know about:
 *
 *   Returned `uint8_t*` data pointers are CUDA DEVICE pointers. The reference returns
 *   unified-memory pointers the CPU may dereference; here host code moves bytes with
 *   applegpu_eager_upload / applegpu_eager_download / applegpu_ffi_upload / applegpu_ffi_read_bytes
 *   (declared in applegpu_b200_ext.h). applegpu_ffi_read_f32 and applegpu_ffi_copy behave as upstream.
 *
 * Conventions (same as upstream): tensors are uint64_t ids from one process-wide counter starting
 * at 1; recorded-op ids start at 100000; dtype codes are int8_t wire codes (0 f32, 1 f16, 2 f64,
 * 3 i8, 4 i16, 5 i32, 6 i64, 7 u8, 8 u32, 9 bool, 10 bf16); dims are uint64_t arrays with
 * ndim <= 8; failures return NULL / 0 / -1 / false and leave a message for *_last_error(),
 * which is thread-local and stays valid until the next failure on that thread. Work is
 * asynchronous on one CUDA stream: results are defined after eval / synchronize /
 * flush_and_wait or a read-back call.
 */
#ifndef APPLEGPU_B200_FFI_H
#define APPLEGPU_B200_FFI_H

#include <stdint.h>
#include <stdbool.h>

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

/* ── graph (lazy) flavour ─────────────────────────────────────────────────── */

/* Lifecycle. Reference: applegpu_ffi.h:12-13, backend_ffi.rs:41-78. */
APPLEGPU_API bool applegpu_ffi_init(void);
APPLEGPU_API const char* applegpu_ffi_last_error(void);

/* Allocation. Reference: applegpu_ffi.h:16-17, backend_ffi.rs:87-123. A zero-byte request
 * returns NULL together with a valid id. free() is deferred while pending ops use the tensor. */
APPLEGPU_API uint8_t* applegpu_ffi_alloc(uint64_t size_bytes, int8_t dtype_i8, uint64_t* out_tensor_id);
APPLEGPU_API void applegpu_ffi_free(uint64_t tensor_id);

/* Tensor metadata. Reference: applegpu_ffi.h:20-22, backend_ffi.rs:150-222. */
APPLEGPU_API int32_t applegpu_ffi_register_tensor(uint64_t tensor_id, const uint64_t* dims, uint32_t ndim, int8_t dtype_i8);
APPLEGPU_API int32_t applegpu_ffi_shape(uint64_t tensor_id, uint64_t* out_dims, uint32_t* out_ndim);
APPLEGPU_API int8_t applegpu_ffi_dtype(uint64_t tensor_id);

/* Recorded ops: return the output tensor id, 0 on failure. Reference: applegpu_ffi.h:25-31,
 * backend_ffi.rs:226-334. */
APPLEGPU_API uint64_t applegpu_ffi_add(uint64_t a_id, uint64_t b_id);
APPLEGPU_API uint64_t applegpu_ffi_matmul(uint64_t a_id, uint64_t b_id);
APPLEGPU_API uint64_t applegpu_ffi_relu(uint64_t input_id);
APPLEGPU_API uint64_t applegpu_ffi_mul(uint64_t a_id, uint64_t b_id);
APPLEGPU_API uint64_t applegpu_ffi_sub(uint64_t a_id, uint64_t b_id);
APPLEGPU_API uint64_t applegpu_ffi_neg(uint64_t input_id);
APPLEGPU_API int32_t applegpu_ffi_copy(uint64_t src_id, uint64_t dst_id);

/* Recorded ops with the output buffer reserved up front: return its data pointer and write the
 * id to *out_id. Reference: applegpu_ffi.h:34-43, backend_ffi.rs:343-441. */
APPLEGPU_API uint8_t* applegpu_ffi_add_out(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_mul_out(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_sub_out(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_matmul_out(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_relu_out(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_neg_out(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_div_out(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_threshold_backward_out(uint64_t grad_id, uint64_t input_id, float threshold, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_scalar_mul_out(uint64_t input_id, float scale, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_ffi_mean_all_out(uint64_t input_id, uint64_t* out_id);

/* Evaluation and synchronisation. Reference: applegpu_ffi.h:46-47, backend_ffi.rs:130-146. */
APPLEGPU_API int32_t applegpu_ffi_eval(uint64_t tensor_id);
APPLEGPU_API void applegpu_ffi_synchronize(void);

/* Read-back as float32 (evaluates first if pending; other dtypes are widened).
 * Reference: applegpu_ffi.h:50, backend_ffi.rs:445-474. */
APPLEGPU_API int32_t applegpu_ffi_read_f32(uint64_t tensor_id, float* out_ptr, uint64_t max_elements);

/* ── eager flavour ────────────────────────────────────────────────────────── */

/* Reference: applegpu_ffi.h:53-54, eager_ffi.rs:69-101. */
APPLEGPU_API bool applegpu_eager_init(void);
APPLEGPU_API const char* applegpu_eager_last_error(void);

/* Reference: applegpu_ffi.h:56-60, eager_ffi.rs:105-215. Zero-element tensors still own a buffer. */
APPLEGPU_API uint8_t* applegpu_eager_alloc(const uint64_t* dims, uint32_t ndim, int8_t dtype, uint64_t* out_id);
APPLEGPU_API void applegpu_eager_free(uint64_t id);
APPLEGPU_API int32_t applegpu_eager_register_shape(uint64_t id, const uint64_t* dims, uint32_t ndim);
APPLEGPU_API int32_t applegpu_eager_shape(uint64_t id, uint64_t* out_dims, uint32_t* out_ndim);
APPLEGPU_API int8_t applegpu_eager_dtype(uint64_t id);

/* Element-wise and matmul. Binary ops broadcast and honour view strides and offsets; matmul
 * rejects non-contiguous inputs ("matmul requires contiguous inputs"); matmul_ex takes base
 * tensors plus transpose flags. Reference: applegpu_ffi.h:62-69, eager_ffi.rs:231-347,
 * eager.rs:246-342, :403-560. */
APPLEGPU_API uint8_t* applegpu_eager_add(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_sub(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_mul(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_div(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_relu(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_neg(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_matmul(uint64_t a_id, uint64_t b_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_matmul_ex(uint64_t a_id, uint64_t b_id, bool transpose_a, bool transpose_b, uint64_t* out_id);

/* Reference: applegpu_ffi.h:71-73. */
APPLEGPU_API uint8_t* applegpu_eager_threshold_backward(uint64_t grad_id, uint64_t input_id, float threshold, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_scalar_mul(uint64_t input_id, float scale, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_mean_all(uint64_t input_id, uint64_t* out_id);

/* Sum over one dimension (negative dims count from the end). Reference: applegpu_ffi.h:75, eager.rs:827-846. */
APPLEGPU_API uint8_t* applegpu_eager_sum_dim(uint64_t input_id, int64_t dim, bool keepdim, uint64_t* out_id);

/* A view shares the base buffer; strides and offset are in elements. Reference: applegpu_ffi.h:77, eager.rs:114-139. */
APPLEGPU_API uint8_t* applegpu_eager_create_view(uint64_t base_id, const uint64_t* shape, const uint64_t* strides, uint32_t ndim, uint64_t offset, uint64_t* out_id);

/* self += other, self += alpha * other. Reference: applegpu_ffi.h:79-80, eager.rs:1084-1096. */
APPLEGPU_API int32_t applegpu_eager_add_inplace(uint64_t self_id, uint64_t other_id);
APPLEGPU_API int32_t applegpu_eager_add_scaled_inplace(uint64_t self_id, uint64_t other_id, float alpha);

/* Both block until the stream is idle. Reference: applegpu_ffi.h:82-83, eager_ffi.rs:637-658. */
APPLEGPU_API void applegpu_eager_flush_and_wait(void);
APPLEGPU_API void applegpu_eager_synchronize(void);

/* GPT-2 ops: embedding (int32 indices, out shape = idx.shape + [D]), layer_norm and softmax over
 * the last dim, tanh-GELU. Reference: applegpu_ffi.h:86-89, eager.rs:957-1079. */
APPLEGPU_API uint8_t* applegpu_eager_embedding(uint64_t weight_id, uint64_t indices_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_layer_norm(uint64_t input_id, uint64_t gamma_id, uint64_t beta_id, float eps, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_gelu(uint64_t input_id, uint64_t* out_id);
APPLEGPU_API uint8_t* applegpu_eager_softmax(uint64_t input_id, uint64_t* out_id);

/* Reverse lookup by data pointer, preferring the owning tensor over views; 0 if unknown.
 * Reference: applegpu_ffi.h:92, eager_ffi.rs:611-633. */
APPLEGPU_API uint64_t applegpu_eager_find_by_data_ptr(const uint8_t* ptr);

#ifdef __cplusplus
}
#endif

#endif /* APPLEGPU_B200_FFI_H */
