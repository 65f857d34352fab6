// Index and conversion kernels: embedding, gather, index_select, quantize, dequantize, cast.
//
// Reference semantics: kernel_templates.rs:1119-1143 (embedding: out[i,:] = W[idx[i],:], int32
// indices, no bounds check), :870-975 (2-D gather / index_select), :2170-2187 (cast),
// :2193-2218 (quantize: round(x/scale)+zp with round-half-away-from-zero, clamp, cast),
// :2222-2240 (dequantize: float(q - zp) * scale, integer subtract first). These are
// bit-exact ops: IEEE divide (__fdiv_rn) and roundf, never a reciprocal multiply.
#include "common.cuh"

namespace ag { namespace k {

// ── embedding ───────────────────────────────────────────────────────────────
// One warp per output row, 16-byte packs. Out-of-range indices copy nothing useful upstream;
// here they are clamped into the table so a bad index can never fault the device.
template <int ESZ>
__global__ void __launch_bounds__(256) embedding_kernel(const uint8_t* __restrict__ w, const int32_t* __restrict__ idx, uint8_t* __restrict__ out,
                                                         int64_t n_idx, int64_t row_bytes, int64_t vocab) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int64_t i = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5); i < n_idx; i += (int64_t)gridDim.x * wpb) {
    int64_t r = idx[i];
    r = r < 0 ? 0 : (r >= vocab ? vocab - 1 : r);
    const uint8_t* src = w + r * row_bytes;
    uint8_t* dst = out + i * row_bytes;
    if (ESZ == 16) {
      int64_t packs = row_bytes / 16;
      for (int64_t p = lane; p < packs; p += 32)
        __stcs(reinterpret_cast<uint4*>(dst) + p, __ldg(reinterpret_cast<const uint4*>(src) + p));
    } else {
      for (int64_t b = lane; b < row_bytes / ESZ; b += 32) {
        if (ESZ == 4) reinterpret_cast<uint32_t*>(dst)[b] = reinterpret_cast<const uint32_t*>(src)[b];
        else if (ESZ == 2) reinterpret_cast<uint16_t*>(dst)[b] = reinterpret_cast<const uint16_t*>(src)[b];
        else dst[b] = src[b];
      }
    }
  }
}

Status embedding(cudaStream_t s, const TView& weight, const TView& idx, const TView& out) {
  if (!weight.contiguous() || !idx.contiguous() || !out.contiguous()) return Status::compute("embedding needs contiguous tensors");
  int64_t n_idx = idx.numel();
  int64_t vocab = weight.shape[0], dim = weight.shape[1];
  if (n_idx == 0 || dim == 0) return Status::OK();
  if (vocab == 0) return Status::compute("embedding from an empty table");
  int64_t row_bytes = dim * (int64_t)dtype_size(weight.dtype);
  int grid = grid_for(n_idx, 8, 8);
  const uint8_t* w = (const uint8_t*)weight.ptr; uint8_t* o = (uint8_t*)out.ptr; const int32_t* ix = (const int32_t*)idx.ptr;
  if (row_bytes % 16 == 0 && aligned16(w) && aligned16(o)) embedding_kernel<16><<<grid, 256, 0, s>>>(w, ix, o, n_idx, row_bytes, vocab);
  else if (row_bytes % 4 == 0) embedding_kernel<4><<<grid, 256, 0, s>>>(w, ix, o, n_idx, row_bytes, vocab);
  else if (row_bytes % 2 == 0) embedding_kernel<2><<<grid, 256, 0, s>>>(w, ix, o, n_idx, row_bytes, vocab);
  else embedding_kernel<1><<<grid, 256, 0, s>>>(w, ix, o, n_idx, row_bytes, vocab);
  AG_CHECK_LAUNCH("embedding");
  return Status::OK();
}

template <typename T>
__global__ void __launch_bounds__(256) embedding_add_kernel(const T* __restrict__ wte, const int32_t* __restrict__ tok, const T* __restrict__ wpe,
                                                             const int32_t* __restrict__ pos, T* __restrict__ out, int64_t n_idx, int dim,
                                                             int64_t vocab, int64_t n_pos) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger();
  for (int64_t i = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5); i < n_idx; i += (int64_t)gridDim.x * wpb) {
    int64_t r = tok[i]; r = r < 0 ? 0 : (r >= vocab ? vocab - 1 : r);
    int64_t q = pos[i]; q = q < 0 ? 0 : (q >= n_pos ? n_pos - 1 : q);
    const T* a = wte + r * dim; const T* b = wpe + q * dim; T* o = out + i * dim;
    for (int c = lane * N; c < dim; c += 32 * N) {
      Pack<T> x = ld16(a + c), y = ld16(b + c), z;
#pragma unroll
      for (int e = 0; e < N; e++) z.v[e] = Cvt<T>::from(Cvt<T>::to(x.v[e]) + Cvt<T>::to(y.v[e]));
      st16_stream(o + c, z);
    }
  }
}

Status embedding_add(cudaStream_t s, const TView& wte, const TView& tok, const TView& wpe, const TView& pos, const TView& out) {
  int64_t n_idx = tok.numel();
  int64_t dim = wte.shape[1];
  if (n_idx == 0 || dim == 0) return Status::OK();
  size_t esz = dtype_size(wte.dtype);
  if ((dim * esz) % 16 != 0 || !aligned16(wte.ptr) || !aligned16(wpe.ptr) || !aligned16(out.ptr))
    return Status::compute("embedding_add needs 16-byte aligned rows");
  int grid = grid_for(n_idx, 8, 8);
  cudaError_t le = cudaSuccess;
  AG_DISPATCH_FLOAT(wte.dtype, T, (le = launch_pdl(embedding_add_kernel<T>, dim3(grid), dim3(256), 0, s, (const T*)wte.ptr, (const int32_t*)tok.ptr,
      (const T*)wpe.ptr, (const int32_t*)pos.ptr, (T*)out.ptr, n_idx, (int)dim, wte.shape[0], wpe.shape[0])));
  if (le != cudaSuccess) return cuda_status(le, "embedding_add");
  return Status::OK();
}

// ── gather / index_select (2-D) ─────────────────────────────────────────────
template <typename E>
__global__ void gather2d_kernel(const E* __restrict__ in, const int32_t* __restrict__ idx, E* __restrict__ out,
                                int64_t out_rows, int64_t out_cols, int64_t in_rows, int64_t in_cols, int dim, int select) {
  int64_t n = out_rows * out_cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / out_cols, c = i % out_cols;
    int64_t sr, sc;
    if (select) {  // index_select: idx is 1-D
      if (dim == 0) { sr = idx[r]; sc = c; } else { sr = r; sc = idx[c]; }
    } else {       // gather: idx has the output's shape
      if (dim == 0) { sr = idx[i]; sc = c; } else { sr = r; sc = idx[i]; }
    }
    sr = sr < 0 ? 0 : (sr >= in_rows ? in_rows - 1 : sr);
    sc = sc < 0 ? 0 : (sc >= in_cols ? in_cols - 1 : sc);
    out[i] = in[sr * in_cols + sc];
  }
}
static Status gather_common(cudaStream_t s, const TView& in, int dim, const TView& idx, const TView& out, int select) {
  if (!in.contiguous() || !idx.contiguous() || !out.contiguous()) return Status::compute("gather needs contiguous tensors");
  int64_t n = out.numel();
  if (n == 0) return Status::OK();
  if (in.numel() == 0) return Status::compute("gather from an empty tensor");
  int grid = grid_for(n, 256, 8);
  int64_t orows = out.shape[0], ocols = out.shape[1], irows = in.shape[0], icols = in.shape[1];
  const int32_t* ix = (const int32_t*)idx.ptr;
  switch (dtype_size(in.dtype)) {
    case 1: gather2d_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)in.ptr, ix, (uint8_t*)out.ptr, orows, ocols, irows, icols, dim, select); break;
    case 2: gather2d_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)in.ptr, ix, (uint16_t*)out.ptr, orows, ocols, irows, icols, dim, select); break;
    case 4: gather2d_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)in.ptr, ix, (uint32_t*)out.ptr, orows, ocols, irows, icols, dim, select); break;
    default: gather2d_kernel<uint64_t><<<grid, 256, 0, s>>>((const uint64_t*)in.ptr, ix, (uint64_t*)out.ptr, orows, ocols, irows, icols, dim, select); break;
  }
  AG_CHECK_LAUNCH("gather");
  return Status::OK();
}
Status gather2d(cudaStream_t s, const TView& in, int dim, const TView& idx, const TView& out) { return gather_common(s, in, dim, idx, out, 0); }
Status index_select2d(cudaStream_t s, const TView& in, int dim, const TView& idx, const TView& out) { return gather_common(s, in, dim, idx, out, 1); }

// ── quantize / dequantize ───────────────────────────────────────────────────
template <bool SIGNED>
__device__ __forceinline__ uint8_t quant_one(float x, float scale, float zp) {
  float v = roundf(__fdiv_rn(x, scale)) + zp;
  if (SIGNED) { v = fminf(fmaxf(v, -128.0f), 127.0f); return (uint8_t)(int8_t)(int)v; }
  v = fminf(fmaxf(v, 0.0f), 255.0f);
  return (uint8_t)(int)v;
}
// 16 elements per thread: 16*sizeof(T) bytes in, one 16-byte store out.
template <typename T, bool SIGNED>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ in, uint8_t* __restrict__ out, int64_t n, float scale, float zp, int vec) {
  constexpr int N = Pack<T>::N;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t groups = vec ? n / 16 : 0;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    alignas(16) uint8_t q[16];
#pragma unroll
    for (int p = 0; p < 16 / N; p++) {
      Pack<T> x = ld16_stream(in + g * 16 + p * N);
#pragma unroll
      for (int e = 0; e < N; e++) q[p * N + e] = quant_one<SIGNED>(Cvt<T>::to(x.v[e]), scale, zp);
    }
    __stcs(reinterpret_cast<uint4*>(out + g * 16), *reinterpret_cast<const uint4*>(q));
  }
  for (int64_t i = groups * 16 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = quant_one<SIGNED>(Cvt<T>::to(in[i]), scale, zp);
}

Status quantize(cudaStream_t s, const TView& in, float scale, int zero_point, const TView& out) {
  if (!in.contiguous() || !out.contiguous()) return Status::compute("quantize needs contiguous tensors");
  int64_t n = in.numel();
  if (n == 0) return Status::OK();
  int vec = aligned16(in.ptr) && aligned16(out.ptr);
  int grid = grid_for((n + 15) / 16, 256, 8);
  bool is_signed = out.dtype == DType::I8;
  float zp = (float)zero_point;
  if (is_signed) { AG_DISPATCH_FLOAT(in.dtype, T, (quantize_kernel<T, true><<<grid, 256, 0, s>>>((const T*)in.ptr, (uint8_t*)out.ptr, n, scale, zp, vec))); }
  else { AG_DISPATCH_FLOAT(in.dtype, T, (quantize_kernel<T, false><<<grid, 256, 0, s>>>((const T*)in.ptr, (uint8_t*)out.ptr, n, scale, zp, vec))); }
  AG_CHECK_LAUNCH("quantize");
  return Status::OK();
}

template <typename T, bool SIGNED>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, int64_t n, float scale, int zp, int vec) {
  constexpr int N = Pack<T>::N;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t groups = vec ? n / 16 : 0;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    alignas(16) uint8_t q[16];
    *reinterpret_cast<uint4*>(q) = __ldcs(reinterpret_cast<const uint4*>(in + g * 16));
#pragma unroll
    for (int p = 0; p < 16 / N; p++) {
      Pack<T> o;
#pragma unroll
      for (int e = 0; e < N; e++) {
        int qi = SIGNED ? (int)(int8_t)q[p * N + e] : (int)q[p * N + e];
        o.v[e] = Cvt<T>::from((float)(qi - zp) * scale);
      }
      st16_stream(out + g * 16 + p * N, o);
    }
  }
  for (int64_t i = groups * 16 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int qi = SIGNED ? (int)(int8_t)in[i] : (int)in[i];
    out[i] = Cvt<T>::from((float)(qi - zp) * scale);
  }
}

Status dequantize(cudaStream_t s, const TView& in, float scale, int zero_point, const TView& out) {
  if (!in.contiguous() || !out.contiguous()) return Status::compute("dequantize needs contiguous tensors");
  int64_t n = in.numel();
  if (n == 0) return Status::OK();
  int vec = aligned16(in.ptr) && aligned16(out.ptr);
  int grid = grid_for((n + 15) / 16, 256, 8);
  if (in.dtype == DType::I8) { AG_DISPATCH_FLOAT(out.dtype, T, (dequantize_kernel<T, true><<<grid, 256, 0, s>>>((const uint8_t*)in.ptr, (T*)out.ptr, n, scale, zero_point, vec))); }
  else { AG_DISPATCH_FLOAT(out.dtype, T, (dequantize_kernel<T, false><<<grid, 256, 0, s>>>((const uint8_t*)in.ptr, (T*)out.ptr, n, scale, zero_point, vec))); }
  AG_CHECK_LAUNCH("dequantize");
  return Status::OK();
}

// Per-output-channel symmetric int8 for linear weights stored [N, K]:
// scale[n] = max|w[n,:]| / 127 (1 if the row is all zero), q = clamp(round(w/scale), -128, 127).
template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const T* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ scales, int64_t rows, int64_t cols) {
  __shared__ float red[33];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* x = w + r * cols;
    float m = 0.f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, fabsf(Cvt<T>::to(x[j])));
    m = block_max(m, red);
    float sc = m > 0.f ? __fdiv_rn(m, 127.0f) : 1.0f;
    if (threadIdx.x == 0) scales[r] = sc;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
      q[r * cols + j] = (int8_t)quant_one<true>(Cvt<T>::to(x[j]), sc, 0.f);
  }
}
Status quantize_rows(cudaStream_t s, const TView& w, const TView& q, const TView& scales) {
  if (!w.contiguous() || !q.contiguous() || w.nd() != 2) return Status::compute("quantize_rows needs a contiguous 2-D weight");
  int64_t rows = w.shape[0], cols = w.shape[1];
  if (rows == 0) return Status::OK();
  int grid = (int)(rows < (int64_t)sm_count() * 8 ? rows : (int64_t)sm_count() * 8);
  AG_DISPATCH_FLOAT(w.dtype, T, (quantize_rows_kernel<T><<<grid, 256, 0, s>>>((const T*)w.ptr, (int8_t*)q.ptr, (float*)scales.ptr, rows, cols)));
  AG_CHECK_LAUNCH("quantize_rows");
  return Status::OK();
}

// ── cast ────────────────────────────────────────────────────────────────────
template <typename S> struct CastLoad { static __device__ __forceinline__ S get(const S* p, int64_t i) { return p[i]; } };

template <typename S, typename D> struct CastOne {
  static __device__ __forceinline__ D run(S v) { return static_cast<D>(v); }
};
// half types go through float
template <typename D> struct CastOne<__half, D> { static __device__ __forceinline__ D run(__half v) { return static_cast<D>(__half2float(v)); } };
template <typename D> struct CastOne<__nv_bfloat16, D> { static __device__ __forceinline__ D run(__nv_bfloat16 v) { return static_cast<D>(__bfloat162float(v)); } };
template <typename S> struct CastOne<S, __half> { static __device__ __forceinline__ __half run(S v) { return __float2half_rn(static_cast<float>(v)); } };
template <typename S> struct CastOne<S, __nv_bfloat16> { static __device__ __forceinline__ __nv_bfloat16 run(S v) { return __float2bfloat16_rn(static_cast<float>(v)); } };
template <> struct CastOne<__half, __half> { static __device__ __forceinline__ __half run(__half v) { return v; } };
template <> struct CastOne<__nv_bfloat16, __nv_bfloat16> { static __device__ __forceinline__ __nv_bfloat16 run(__nv_bfloat16 v) { return v; } };
template <> struct CastOne<__half, __nv_bfloat16> { static __device__ __forceinline__ __nv_bfloat16 run(__half v) { return __float2bfloat16_rn(__half2float(v)); } };
template <> struct CastOne<__nv_bfloat16, __half> { static __device__ __forceinline__ __half run(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); } };
// bool target: non-zero -> 1
struct BoolT { uint8_t v; };

template <typename S, typename D, bool TO_BOOL>
__global__ void cast_kernel(const S* __restrict__ in, D* __restrict__ out, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (TO_BOOL) out[i] = (D)(CastOne<S, float>::run(in[i]) != 0.0f ? 1 : 0);
    else out[i] = CastOne<S, D>::run(in[i]);
  }
}

template <typename S>
static Status cast_from(cudaStream_t s, const S* in, const TView& out, int64_t n) {
  int grid = grid_for(n, 256, 8);
  switch (out.dtype) {
    case DType::F32: cast_kernel<S, float, false><<<grid, 256, 0, s>>>(in, (float*)out.ptr, n); break;
    case DType::F16: cast_kernel<S, __half, false><<<grid, 256, 0, s>>>(in, (__half*)out.ptr, n); break;
    case DType::BF16: cast_kernel<S, __nv_bfloat16, false><<<grid, 256, 0, s>>>(in, (__nv_bfloat16*)out.ptr, n); break;
    case DType::I8: cast_kernel<S, int8_t, false><<<grid, 256, 0, s>>>(in, (int8_t*)out.ptr, n); break;
    case DType::I16: cast_kernel<S, int16_t, false><<<grid, 256, 0, s>>>(in, (int16_t*)out.ptr, n); break;
    case DType::I32: cast_kernel<S, int32_t, false><<<grid, 256, 0, s>>>(in, (int32_t*)out.ptr, n); break;
    case DType::I64: cast_kernel<S, int64_t, false><<<grid, 256, 0, s>>>(in, (int64_t*)out.ptr, n); break;
    case DType::U8: cast_kernel<S, uint8_t, false><<<grid, 256, 0, s>>>(in, (uint8_t*)out.ptr, n); break;
    case DType::U32: cast_kernel<S, uint32_t, false><<<grid, 256, 0, s>>>(in, (uint32_t*)out.ptr, n); break;
    case DType::Bool: cast_kernel<S, uint8_t, true><<<grid, 256, 0, s>>>(in, (uint8_t*)out.ptr, n); break;
    default: return Status::unsupported("Float64 is not supported on this device path");
  }
  AG_CHECK_LAUNCH("cast");
  return Status::OK();
}

// int8 -> 16-bit float, 16 elements per thread (the widening of int8 weights ahead of a tensor-core GEMM: 1 byte
// read and 2 written per element, so it has to run at memory speed). A byte b = v ^ 0x80 placed in the low
// mantissa bits of 2^23 gives the float 8388608 + b exactly; subtracting 8388736 leaves v, which every 16-bit
// float format holds exactly: no integer-to-float conversion instruction (a quarter-rate pipe) is needed.
template <typename D>
__global__ void __launch_bounds__(256) widen_i8_kernel(const int8_t* __restrict__ in, D* __restrict__ out, int64_t n16) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n16; g += stride) {
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(in) + g);
    const uint32_t w[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
    Pack<D> o[2];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float f[4];
#pragma unroll
      for (int b = 0; b < 4; b++) f[b] = __uint_as_float(0x4B000000u | ((w[i] >> (8 * b)) & 0xffu)) - 8388736.0f;
      // elements 4*i .. 4*i+3 of the 16: the first 8 go to o[0], the rest to o[1]
      float r[4] = {f[0], f[1], f[2], f[3]};
      D* dst = &o[i >> 1].v[(i & 1) * 4];
#pragma unroll
      for (int b = 0; b < 4; b++) dst[b] = Cvt<D>::from(r[b]);
    }
    st16(out + g * 16, o[0]);          // the GEMM that follows reads these from L2: no evict-first hint
    st16(out + g * 16 + 8, o[1]);
  }
}

Status cast(cudaStream_t s, const TView& in, const TView& out) {
  if (!in.contiguous() || !out.contiguous()) return Status::compute("cast needs contiguous tensors");
  int64_t n = in.numel();
  if (n == 0) return Status::OK();
  if (in.dtype == DType::I8 && (out.dtype == DType::BF16 || out.dtype == DType::F16) && n % 16 == 0 && aligned16(in.ptr) && aligned16(out.ptr)) {
    const int64_t n16 = n / 16;
    int grid = grid_for(n16, 256, 8);
    if (out.dtype == DType::BF16) widen_i8_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const int8_t*)in.ptr, (__nv_bfloat16*)out.ptr, n16);
    else widen_i8_kernel<__half><<<grid, 256, 0, s>>>((const int8_t*)in.ptr, (__half*)out.ptr, n16);
    AG_CHECK_LAUNCH("cast (int8 widen)");
    return Status::OK();
  }
  switch (in.dtype) {
    case DType::F32: return cast_from<float>(s, (const float*)in.ptr, out, n);
    case DType::F16: return cast_from<__half>(s, (const __half*)in.ptr, out, n);
    case DType::BF16: return cast_from<__nv_bfloat16>(s, (const __nv_bfloat16*)in.ptr, out, n);
    case DType::I8: return cast_from<int8_t>(s, (const int8_t*)in.ptr, out, n);
    case DType::I16: return cast_from<int16_t>(s, (const int16_t*)in.ptr, out, n);
    case DType::I32: return cast_from<int32_t>(s, (const int32_t*)in.ptr, out, n);
    case DType::I64: return cast_from<int64_t>(s, (const int64_t*)in.ptr, out, n);
    case DType::U8: case DType::Bool: return cast_from<uint8_t>(s, (const uint8_t*)in.ptr, out, n);
    case DType::U32: return cast_from<uint32_t>(s, (const uint32_t*)in.ptr, out, n);
    default: return Status::unsupported("Float64 is not supported on this device path");
  }
}


// ── fp32 -> 3 x bf16 split (operands of the split-precision fp32 matmul) ─────
// A product of two split sums keeps the six largest cross terms:
//   a*b ~ a2*b0 + a1*b1 + a0*b2 + a1*b0 + a0*b1 + a0*b0      (smallest first)
// so the A side is laid out as terms {2,1,0,1,0,0} and the B side as {0,1,2,0,1,0}; one bf16 GEMM over
// the six-fold K extent with fp32 accumulation then yields the fp32 product to ~2^-22 relative.
__global__ void __launch_bounds__(256) split_bf16x3_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t rows, int64_t cols,
                                                            int64_t in_row_stride, int64_t in_batch_stride, int stack_rows, int b_side) {
  const int64_t packs_per_row = cols / 8;
  const int64_t total = rows * packs_per_row;
  const float* src = in + (int64_t)blockIdx.y * in_batch_stride;
  __nv_bfloat16* dst = out + (int64_t)blockIdx.y * rows * cols * 6;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / packs_per_row, c = (i % packs_per_row) * 8;
    const float4 x0 = *reinterpret_cast<const float4*>(src + r * in_row_stride + c);
    const float4 x1 = *reinterpret_cast<const float4*>(src + r * in_row_stride + c + 4);
    const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    Pack<__nv_bfloat16> t[3];
#pragma unroll
    for (int e = 0; e < 8; e++) {
      __nv_bfloat16 h0 = __float2bfloat16_rn(x[e]);
      float r1 = x[e] - __bfloat162float(h0);
      __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
      float r2 = r1 - __bfloat162float(h1);
      t[0].v[e] = h0; t[1].v[e] = h1; t[2].v[e] = __float2bfloat16_rn(r2);
    }
#pragma unroll
    for (int k = 0; k < 6; k++) {
      const int a_pat[6] = {2, 1, 0, 1, 0, 0}, b_pat[6] = {0, 1, 2, 0, 1, 0};
      const int term = b_side ? b_pat[k] : a_pat[k];
      __nv_bfloat16* o = stack_rows ? dst + ((int64_t)k * rows + r) * cols + c : dst + r * (cols * 6) + (int64_t)k * cols + c;
      st16(o, t[term]);
    }
  }
}

Status split_bf16x3(cudaStream_t s, const float* in, void* out_bf16, int64_t rows, int64_t cols, int64_t in_row_stride, int64_t batches,
                    int64_t in_batch_stride, bool stack_rows, bool b_side) {
  if (rows == 0 || cols == 0 || batches == 0) return Status::OK();
  if (cols % 8 != 0 || in_row_stride % 4 != 0 || in_batch_stride % 4 != 0 || !aligned16(in) || !aligned16(out_bf16))
    return Status::invalid("split_bf16x3 needs 16-byte aligned rows of a multiple of 8 columns");
  if (batches > 65535) return Status::invalid("split_bf16x3: too many batches");
  dim3 grid((unsigned)grid_for(rows * (cols / 8), 256, 8), (unsigned)batches, 1);
  split_bf16x3_kernel<<<grid, 256, 0, s>>>(in, static_cast<__nv_bfloat16*>(out_bf16), rows, cols, in_row_stride, in_batch_stride, stack_rows ? 1 : 0,
                                           b_side ? 1 : 0);
  AG_CHECK_LAUNCH("split_bf16x3");
  return Status::OK();
}

}}  // namespace ag::k
