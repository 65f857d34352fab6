// Device helpers shared by the bandwidth-bound kernels: 16-byte vector access,
// storage<->float conversion (half types compute in float and round once on store,
// as kernel_templates.rs:171-191 `needs_float_acc` does), warp/block reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <utility>
#include "kernels.h"

namespace ag { namespace k {

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to(float v) { return v; }
  static __device__ __forceinline__ float from(float v) { return v; }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16_rn(v); }
};

// A 16-byte pack of T.
template <typename T> struct alignas(16) Pack {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Pack<T> ld16(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
// Pack<T> from floats: 16-bit types convert two values per instruction.
template <typename T>
__device__ __forceinline__ void pack_from_floats(Pack<T>& o, const float* r) {
#pragma unroll
  for (int e = 0; e < Pack<T>::N; e++) o.v[e] = Cvt<T>::from(r[e]);
}
template <>
__device__ __forceinline__ void pack_from_floats<__nv_bfloat16>(Pack<__nv_bfloat16>& o, const float* r) {
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int q = 0; q < 4; q++) o2[q] = __floats2bfloat162_rn(r[2 * q], r[2 * q + 1]);
}
template <>
__device__ __forceinline__ void pack_from_floats<__half>(Pack<__half>& o, const float* r) {
  __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int q = 0; q < 4; q++) o2[q] = __floats2half2_rn(r[2 * q], r[2 * q + 1]);
}
// Streaming variants: data touched once should not displace reusable lines.
template <typename T>
__device__ __forceinline__ Pack<T> ld16_stream(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Pack<T>& v) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
}
template <typename T>
__device__ __forceinline__ void st16_stream(T* p, const Pack<T>& v) {
  __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions over up to 32 warps; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* smem /* >=33 floats */) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[w] = v;
  __syncthreads();
  float r = (lane < nw) ? smem[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* smem) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[w] = v;
  __syncthreads();
  float r = (lane < nw) ? smem[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// tanh-GELU with the reference's clamp (kernel_templates.rs:299-302).
// 0.5 * (1 + tanh(u)) = e^{2u} / (e^{2u} + 1), so gelu(x) = x * t / (t + 1) with t = exp(2u): one
// hardware exp2 and one fast divide, no cancellation for negative x (where 1 + tanh(u) is tiny),
// relative error ~|u| * 1e-6 — inside the 1e-5 bar at a quarter of the instructions of tanhf.
__device__ __forceinline__ float gelu_tanh_f(float x) {
  float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
  inner = fminf(fmaxf(inner, -10.0f), 10.0f);
  float t = __expf(2.0f * inner);
  return x * __fdividef(t, t + 1.0f);
}
// erf-GELU. The reference evaluates erf with the Abramowitz-Stegun 7.1.26 polynomial
// (kernel_templates.rs:312-323, max error 1.5e-7); erff is at least as close to the
// exact function, and both sit inside the 1e-5 tolerance of the reference's tests.
__device__ __forceinline__ float gelu_erf_f(float x) {
  return x * 0.5f * (1.0f + erff(x * 0.70710678118f));
}
// erf-GELU with the reference's own erf approximation (Abramowitz-Stegun 7.1.26,
// kernel_templates.rs:312-323) on the hardware reciprocal and exp2: a dozen instructions instead of
// erff's ~25. Absolute error about 1e-6 with the fast intrinsics: used where the result is stored in a
// 16-bit type (the GEMM epilogue), never for float32 outputs.
__device__ __forceinline__ float gelu_erf_fast_f(float x) {
  float z = x * 0.70710678118f;
  float a = fabsf(z);
  float t = __fdividef(1.0f, fmaf(0.3275911f, a, 1.0f));
  float p = fmaf(fmaf(fmaf(fmaf(1.061405429f, t, -1.453152027f), t, 1.421413741f), t, -0.284496736f), t, 0.254829592f) * t;
  float r = 1.0f - p * __expf(-a * a);
  float erf_z = copysignf(r, z);
  return 0.5f * x * (1.0f + erf_z);
}
// erf-GELU for results stored as bfloat16: 0.5 x (1 + tanh(x (c1 + c3 x^2 + c5 x^4))), the odd polynomial fitted so
// that the whole expression stays within 3e-5 absolute (2.5e-3 of the value) of 0.5 x (1 + erf(x / sqrt 2)) over the
// real line, below the 3.9e-3 rounding step of the stored value; the hardware tanh adds 2^-11 relative. One MUFU
// operation and eight others instead of two and twenty: this loop runs beside the next tile's main loop. The argument
// is clamped at |x| = 8, where tanh has long saturated, because the fitted polynomial turns over near |x| = 11.
__device__ __forceinline__ float gelu_erf_bf16_f(float x) {
  const float xc = fminf(fmaxf(x, -8.0f), 8.0f);
  const float x2 = xc * xc;
  const float u = xc * fmaf(fmaf(-3.58732362e-4f, x2, 3.70503451e-2f), x2, 7.97458471e-1f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}
__device__ __forceinline__ float apply_act(float x, Act a) {
  switch (a) {
    case Act::GeluTanh: return gelu_tanh_f(x);
    case Act::GeluErf: return gelu_erf_f(x);
    case Act::Relu: return fmaxf(x, 0.f);
    default: return x;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline Status cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return Status::OK();
  return Status::compute(std::string(what) + ": " + cudaGetErrorString(e));
}
#define AG_CHECK_LAUNCH(what) do { cudaError_t _e = cudaGetLastError(); if (_e != cudaSuccess) return cuda_status(_e, what); } while (0)

// ── programmatic dependent launch ───────────────────────────────────────────
// Kernels of the forward path are launched so that kernel N+1 may be scheduled while kernel N is
// still draining: its CTAs run their prologue (barrier init, TMEM allocation, descriptor prefetch)
// and then block in pdl_wait() until kernel N has completed and its writes are visible. Rules kept
// by every kernel launched through launch_pdl: all threads call pdl_wait() before the first access
// to global memory (so completion stays transitive along the stream), and pdl_trigger() follows
// it (the next kernel is released for scheduling once every CTA of this one has started).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();   // APPLEGPU_PDL=0 turns the launch attribute off (kernels then serialise as usual)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

// Grid sizing: a multiple of the SM count, capped by the work available.
int sm_count();
inline int grid_for(int64_t work_items, int per_block, int blocks_per_sm = 8) {
  int64_t need = (work_items + per_block - 1) / per_block;
  int64_t cap = (int64_t)sm_count() * blocks_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

#define AG_DISPATCH_FLOAT(dt, T, ...)                                              \
  switch (dt) {                                                                    \
    case DType::F32: { using T = float; __VA_ARGS__; break; }                      \
    case DType::F16: { using T = __half; __VA_ARGS__; break; }                     \
    case DType::BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    default: return Status::unsupported(std::string("kernel has no ") + dtype_name(dt) + " variant"); \
  }

}}  // namespace ag::k
