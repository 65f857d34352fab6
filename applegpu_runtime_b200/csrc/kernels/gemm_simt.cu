// Batched matmul, CUDA-core form: true-fp32 FMA accumulation in ascending k, any strides.
//
// Reference: kernel_templates.rs:987-1072 (`matmul{s}`: C[b,i,j] = sum_k A[b,i,k]*B[b,k,j],
// float accumulate, batch stride 0 = broadcast operand). This kernel serves fp32 inputs (whose
// reference tests demand rtol 1e-4, out of reach of single-pass TF32), operand layouts TMA
// cannot describe (rows not 16-byte aligned, transposed A), and int8 weights; half-precision
// inputs with TMA-compatible layouts go to the tcgen05 kernel in gemm_tc.cu.
#include "common.cuh"

namespace ag { namespace k {

template <typename T> struct LoadB { static __device__ __forceinline__ float get(const void* p, int64_t off) { return Cvt<T>::to(reinterpret_cast<const T*>(p)[off]); } };
struct LoadI8 { static __device__ __forceinline__ float get(const void* p, int64_t off) { return (float)reinterpret_cast<const int8_t*>(p)[off]; } };

struct SimtParams {
  const void* a; const void* b; void* c;
  int64_t m, n, k;
  int64_t a_row, a_col, a_batch, b_row, b_col, b_batch, c_row, c_batch;
  int64_t batch_inner, a_batch_inner, b_batch_inner, c_batch_inner;
  const void* bias; const void* residual; const float* b_scales;
  float alpha; int act;
};

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T, typename BL>
__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtParams p) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t bo = blockIdx.z / p.batch_inner, bi = blockIdx.z % p.batch_inner;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  const T* A = reinterpret_cast<const T*>(p.a) + bo * p.a_batch + bi * p.a_batch_inner;
  const char* Bbase = reinterpret_cast<const char*>(p.b);
  const int64_t b_off0 = bo * p.b_batch + bi * p.b_batch_inner;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
    // A tile: TM x TK, 1024 elements, 4 per thread. Consecutive threads walk the unit-stride dim.
#pragma unroll
    for (int l = 0; l < 4; l++) {
      int e = tid + l * 256;
      int mm, kk;
      if (p.a_col == 1) { kk = e % TK; mm = e / TK; } else { mm = e % TM; kk = e / TM; }
      int64_t gm = m0 + mm, gk = k0 + kk;
      float v = 0.f;
      if (gm < p.m && gk < p.k) v = Cvt<T>::to(A[gm * p.a_row + gk * p.a_col]);
      As[kk][mm] = v;
    }
#pragma unroll
    for (int l = 0; l < 4; l++) {
      int e = tid + l * 256;
      int nn, kk;
      if (p.b_col == 1) { nn = e % TN; kk = e / TN; } else { kk = e % TK; nn = e / TK; }
      int64_t gn = n0 + nn, gk = k0 + kk;
      float v = 0.f;
      if (gn < p.n && gk < p.k) v = BL::get(Bbase, b_off0 + gk * p.b_row + gn * p.b_col);
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  const int64_t c_off = bo * p.c_batch + bi * p.c_batch_inner;
  T* C = reinterpret_cast<T*>(p.c) + c_off;
  const T* R = p.residual ? reinterpret_cast<const T*>(p.residual) + c_off : nullptr;
  const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int64_t gm = m0 + ty * 4 + i;
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int64_t gn = n0 + tx * 4 + j;
      if (gn >= p.n) continue;
      float v = acc[i][j] * p.alpha;
      if (p.b_scales) v *= p.b_scales[gn];
      if (bias) v += Cvt<T>::to(bias[gn]);
      v = apply_act(v, (Act)p.act);
      if (R) v += Cvt<T>::to(R[gm * p.c_row + gn]);
      C[gm * p.c_row + gn] = Cvt<T>::from(v);
    }
  }
}

Status matmul_simt(cudaStream_t s, const GemmDesc& d) {
  if (d.m == 0 || d.n == 0 || d.batch == 0) return Status::OK();
  SimtParams p;
  p.a = d.a; p.b = d.b; p.c = d.c; p.m = d.m; p.n = d.n; p.k = d.k;
  p.a_row = d.a_row; p.a_col = d.a_col; p.a_batch = d.a_batch;
  p.b_row = d.b_row; p.b_col = d.b_col; p.b_batch = d.b_batch;
  p.c_row = d.c_row; p.c_batch = d.c_batch;
  p.batch_inner = d.batch_inner < 1 ? 1 : d.batch_inner;
  p.a_batch_inner = d.a_batch_inner; p.b_batch_inner = d.b_batch_inner; p.c_batch_inner = d.c_batch_inner;
  p.bias = d.ep.bias; p.residual = d.ep.residual; p.b_scales = d.ep.b_scales; p.alpha = d.ep.alpha; p.act = (int)d.ep.act;
  if (d.batch * p.batch_inner > 65535) return Status::compute("matmul batch too large for one launch");
  dim3 grid((unsigned)((d.n + TN - 1) / TN), (unsigned)((d.m + TM - 1) / TM), (unsigned)(d.batch * p.batch_inner));
  if (d.b_dtype == DType::I8) {
    AG_DISPATCH_FLOAT(d.dtype, T, (gemm_simt_kernel<T, LoadI8><<<grid, 256, 0, s>>>(p)));
  } else {
    if (d.b_dtype != d.dtype) return Status::invalid("matmul operand dtypes differ");
    AG_DISPATCH_FLOAT(d.dtype, T, (gemm_simt_kernel<T, LoadB<T>><<<grid, 256, 0, s>>>(p)));
  }
  AG_CHECK_LAUNCH("matmul (simt)");
  return Status::OK();
}

}}  // namespace ag::k
