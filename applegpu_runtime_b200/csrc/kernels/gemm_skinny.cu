// Skinny matmul: C[M, N] = A[M, K] * B[K, N] with M <= 16 (a decode step: one new token per sequence),
// 16-bit or float32 operands (float32: true fp32 multiply-adds, as kernel_templates.rs:987-1027 computes). The product is bound by reading B once (a weight matrix); the 128-row
// tensor-core tiles would leave it on N/256 CTAs (3..12 of 148 SMs) at one SM's share of HBM bandwidth
// each. Here the grid is (N / 64 column slabs) x (K / 128 row slabs): every CTA streams a 128 x 64 block
// of B with coalesced 128-byte (16-bit) or 256-byte (float32) rows, keeps its 16 x 128 block of A in shared memory, and writes an fp32
// partial [M, 64] to a workspace; the last CTA to finish a column slab (a counter per slab) adds the
// partials in K order (so the result does not depend on scheduling), applies the epilogue (alpha,
// bias, activation, residual) and stores the slab. Same arithmetic contract as the other matmul kernels
// (kernel_templates.rs:1029-1066): float accumulation, one rounding on store.
#include "common.cuh"
#include <mutex>

namespace ag { namespace k {

constexpr int kSkN = 64;      // columns per CTA
constexpr int kSkK = 128;     // K rows per CTA
constexpr int kSkMaxM = 16;
constexpr int kSkThreads = 256;
constexpr int64_t kSkMaxN = 65536;      // one counter per 64-column slab
constexpr int kSkMaxKSlabs = 64;
constexpr int64_t kSkMaxPartials = 1 << 18;   // k_slabs * n per launch: a 16 MB fp32 workspace

struct SkinnyParams {
  const void* a; const void* b; void* c;
  const void* bias; const void* residual;
  float alpha; int act;
  int m, n, k;
  long long a_row, b_row, c_row;
  int a_vec;                 // A rows are 16-byte aligned
  float* partial;            // [k_slabs][16][n]
  unsigned int* counters;    // one per column slab, zero between launches
  const void* ln_gamma;      // K-major kernel only: layer_norm of A's rows (gamma, beta of length k) before the product
  const void* ln_beta;
  float ln_eps;
};

// four consecutive elements of B as one load
template <typename T> struct BVec { using type = uint2; };
template <> struct BVec<float> { using type = uint4; };

template <typename T>
__global__ void __launch_bounds__(kSkThreads) gemm_skinny_kernel(const SkinnyParams p) {
  using V = typename BVec<T>::type;
  __shared__ float sA[kSkMaxM][kSkK];              // this CTA's block of A, as float
  __shared__ float sSum[kSkThreads / 32][kSkMaxM][kSkN];
  __shared__ unsigned int s_last;
  const int n0 = blockIdx.x * kSkN, k0 = blockIdx.y * kSkK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* A = reinterpret_cast<const T*>(p.a);
  const T* B = reinterpret_cast<const T*>(p.b);
  pdl_wait();
  pdl_trigger();
  // B first: every load of this CTA's 128 x 64 block is issued before anything waits on one. A warp owns
  // 16 consecutive K rows; per instruction its two half-warps read two rows, 16 lanes x 8 bytes each.
  const int half = lane >> 4, cl = lane & 15;
  const int col = n0 + cl * 4;
  V bv[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int kk = warp * 16 + i * 2 + half;
    bv[i] = V{};
    if (k0 + kk < p.k && col < p.n) bv[i] = __ldcs(reinterpret_cast<const V*>(B + (long long)(k0 + kk) * p.b_row + col));
  }
  // A block -> shared as float (M x 128, zero rows beyond M): one 16-byte load per thread
  {
    const int m = threadIdx.x >> 4, ch = threadIdx.x & 15;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = 0.f;
    if (m < p.m) {
      const T* src = A + (long long)m * p.a_row + k0 + ch * 8;
      if (p.a_vec && k0 + ch * 8 + 8 <= p.k) {
        if constexpr (sizeof(T) == 4) {
          const float4 q0 = *reinterpret_cast<const float4*>(src), q1 = *reinterpret_cast<const float4*>(src + 4);
          v[0] = q0.x; v[1] = q0.y; v[2] = q0.z; v[3] = q0.w; v[4] = q1.x; v[5] = q1.y; v[6] = q1.z; v[7] = q1.w;
        } else {
          Pack<T> q = ld16(src);
#pragma unroll
          for (int e = 0; e < 8; e++) v[e] = Cvt<T>::to(q.v[e]);
        }
      } else {
        for (int e = 0; e < 8; e++) if (k0 + ch * 8 + e < p.k) v[e] = Cvt<T>::to(src[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; e++) sA[m][ch * 8 + e] = v[e];
  }
  __syncthreads();
  float acc[kSkMaxM][4];
#pragma unroll
  for (int m = 0; m < kSkMaxM; m++) { acc[m][0] = 0.f; acc[m][1] = 0.f; acc[m][2] = 0.f; acc[m][3] = 0.f; }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int kk = warp * 16 + i * 2 + half;
    const T* pr = reinterpret_cast<const T*>(&bv[i]);
    const float b0 = Cvt<T>::to(pr[0]), b1 = Cvt<T>::to(pr[1]), b2 = Cvt<T>::to(pr[2]), b3 = Cvt<T>::to(pr[3]);
#pragma unroll
    for (int m = 0; m < kSkMaxM; m++) {
      const float a = sA[m][kk];           // two addresses per warp (one per half): broadcasts
      acc[m][0] = fmaf(a, b0, acc[m][0]); acc[m][1] = fmaf(a, b1, acc[m][1]);
      acc[m][2] = fmaf(a, b2, acc[m][2]); acc[m][3] = fmaf(a, b3, acc[m][3]);
    }
  }
  // the two half-warps hold different rows of the same columns
#pragma unroll
  for (int m = 0; m < kSkMaxM; m++) {
#pragma unroll
    for (int e = 0; e < 4; e++) acc[m][e] += __shfl_xor_sync(0xffffffffu, acc[m][e], 16);
  }
  if (half == 0) {
#pragma unroll
    for (int m = 0; m < kSkMaxM; m++) *reinterpret_cast<float4*>(&sSum[warp][m][cl * 4]) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  }
  __syncthreads();
  const int k_slabs = gridDim.y;
  float* my_partial = p.partial + ((long long)blockIdx.y * kSkMaxM) * p.n;
  for (int i = threadIdx.x; i < kSkMaxM * kSkN; i += kSkThreads) {
    int m = i / kSkN, c = i % kSkN;
    if (m < p.m && n0 + c < p.n) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kSkThreads / 32; w++) v += sSum[w][m][c];    // warp order = K order
      my_partial[(long long)m * p.n + n0 + c] = v;
    }
  }
  // the last CTA of this column slab finishes it
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int prev = atomicAdd(p.counters + blockIdx.x, 1u);
    s_last = (prev == (unsigned int)(k_slabs - 1)) ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  T* C = reinterpret_cast<T*>(p.c);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  const T* R = reinterpret_cast<const T*>(p.residual);
  for (int i = threadIdx.x; i < kSkMaxM * kSkN; i += kSkThreads) {
    int m = i / kSkN, c = i % kSkN;
    if (m < p.m && n0 + c < p.n) {
      float v = 0.f;
      for (int ks = 0; ks < k_slabs; ks++) v += __ldcg(p.partial + ((long long)ks * kSkMaxM + m) * p.n + n0 + c);   // K order: deterministic
      v *= p.alpha;
      if (bias) v += Cvt<T>::to(bias[n0 + c]);
      v = apply_act(v, (Act)p.act);
      if (R) v += Cvt<T>::to(R[(long long)m * p.c_row + n0 + c]);
      C[(long long)m * p.c_row + n0 + c] = Cvt<T>::from(v);
    }
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;   // ready for the next launch on this stream
}

// ── K-major B ───────────────────────────────────────────────────────────────
// The same problem with B stored [N, K] (rows along K: the tied LM head reads the embedding table this way).
// Every output column is a dot product of a B row with the M rows of A: a warp takes four B rows at a time,
// its lanes split K in 16-byte pieces (512 contiguous bytes per load instruction), A sits in shared memory as
// floats, the partial sums are combined with shuffles, and 2 x 32 lanes apply the epilogue to the 16 x 4
// results. No workspace, no cross-CTA step: the sum over K is in a fixed order.
constexpr int kSkR = 4;   // B rows per warp and pass

template <typename T, int MR>
__global__ void __launch_bounds__(kSkThreads) gemm_skinny_kmajor_kernel(const SkinnyParams p) {
  extern __shared__ __align__(16) float sAk[];     // [MR][K]
  constexpr int VEC = 16 / (int)sizeof(T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* A = reinterpret_cast<const T*>(p.a);
  const T* B = reinterpret_cast<const T*>(p.b);
  pdl_wait();
  pdl_trigger();
  for (int i = threadIdx.x; i < MR * p.k; i += kSkThreads) {
    const int m = i / p.k, kk = i - m * p.k;
    sAk[i] = m < p.m ? Cvt<T>::to(A[(long long)m * p.a_row + kk]) : 0.f;
  }
  __syncthreads();
  if (p.ln_gamma) {
    // layer_norm of the staged rows, in place (kernel_templates.rs:1097-1109: mean, population variance,
    // 1/sqrt(var + eps), gamma * (x - mean) * inv_std + beta): a warp per row, two passes over shared memory.
    const T* G = reinterpret_cast<const T*>(p.ln_gamma);
    const T* Bt = reinterpret_cast<const T*>(p.ln_beta);
    for (int m = warp; m < p.m; m += kSkThreads / 32) {
      float* row = sAk + m * p.k;
      float sum = 0.f;
      for (int kk = lane; kk < p.k; kk += 32) sum += row[kk];
      const float mean = warp_sum(sum) / (float)p.k;
      float sq = 0.f;
      for (int kk = lane; kk < p.k; kk += 32) { const float dlt = row[kk] - mean; sq += dlt * dlt; }
      const float inv_std = 1.0f / sqrtf(warp_sum(sq) / (float)p.k + p.ln_eps);
      for (int kk = lane; kk < p.k; kk += 32) row[kk] = Cvt<T>::to(G[kk]) * (row[kk] - mean) * inv_std + Cvt<T>::to(Bt[kk]);
    }
    __syncthreads();
  }
  const long long warps_total = (long long)gridDim.x * (kSkThreads / 32);
  for (long long n0 = ((long long)blockIdx.x * (kSkThreads / 32) + warp) * kSkR; n0 < p.n; n0 += warps_total * kSkR) {
    float acc[MR][kSkR];
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
      for (int r = 0; r < kSkR; r++) acc[m][r] = 0.f;
    for (int kc = lane * VEC; kc < p.k; kc += 32 * VEC) {
      float bf[kSkR][VEC];
#pragma unroll
      for (int r = 0; r < kSkR; r++) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (n0 + r < p.n) raw = __ldcs(reinterpret_cast<const uint4*>(B + (n0 + r) * p.b_row + kc));   // b_row: elements between B rows here
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int x = 0; x < VEC; x++) bf[r][x] = Cvt<T>::to(e[x]);
      }
#pragma unroll
      for (int m = 0; m < MR; m++) {
        float af[VEC];
#pragma unroll
        for (int q = 0; q < VEC / 4; q++) {
          const float4 a4 = *reinterpret_cast<const float4*>(sAk + m * p.k + kc + q * 4);
          af[q * 4] = a4.x; af[q * 4 + 1] = a4.y; af[q * 4 + 2] = a4.z; af[q * 4 + 3] = a4.w;
        }
#pragma unroll
        for (int r = 0; r < kSkR; r++)
#pragma unroll
          for (int x = 0; x < VEC; x++) acc[m][r] = fmaf(af[x], bf[r][x], acc[m][r]);
      }
    }
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
      for (int r = 0; r < kSkR; r++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[m][r] += __shfl_xor_sync(0xffffffffu, acc[m][r], o);
    // every lane holds all MR x 4 sums: lane l finishes (m, r) pairs l, l + 32, ...
    T* C = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const T* R = reinterpret_cast<const T*>(p.residual);
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
      for (int r = 0; r < kSkR; r++) {
        if (((m * kSkR + r) & 31) != lane) continue;
        const long long n = n0 + r;
        if (m >= p.m || n >= p.n) continue;
        float v = acc[m][r] * p.alpha;
        if (bias) v += Cvt<T>::to(bias[n]);
        v = apply_act(v, (Act)p.act);
        if (R) v += Cvt<T>::to(R[(long long)m * p.c_row + n]);
        C[(long long)m * p.c_row + n] = Cvt<T>::from(v);
      }
  }
}

constexpr int kSkKmMaxSmem = 96 * 1024;

bool skinny_kmajor_eligible(const GemmDesc& d) {
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16 || d.dtype == DType::F32) || d.b_dtype != d.dtype) return false;
  if (d.c_f32 || d.ep.argmax_keys || d.ep.b_scales) return false;
  if (d.batch != 1 || d.batch_inner != 1) return false;
  if (d.m < 1 || d.m > kSkMaxM || d.n < 256 || d.k < 64) return false;
  if (d.a_col != 1 || d.b_row != 1) return false;                       // A rows along K, B stored [N, K]
  const int vec = d.dtype == DType::F32 ? 4 : 8;
  if (d.k % vec != 0 || d.b_col % vec != 0 || (reinterpret_cast<uintptr_t>(d.b) & 15u) != 0) return false;   // 16-byte loads of B rows
  const int mr = d.m <= 8 ? 8 : 16;
  if ((int64_t)mr * d.k * (int64_t)sizeof(float) > kSkKmMaxSmem) return false;
  return true;
}

template <typename T>
static cudaError_t launch_kmajor(cudaStream_t s, const SkinnyParams& p, int mr, size_t smem, dim3 grid) {
  auto k8 = gemm_skinny_kmajor_kernel<T, 8>;
  auto k16 = gemm_skinny_kmajor_kernel<T, 16>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k8, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkKmMaxSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k16, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkKmMaxSmem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  return mr == 8 ? launch_pdl(k8, grid, dim3(kSkThreads), smem, s, p) : launch_pdl(k16, grid, dim3(kSkThreads), smem, s, p);
}

Status matmul_skinny_kmajor(cudaStream_t s, const GemmDesc& d) {
  SkinnyParams p;
  p.a = d.a; p.b = d.b; p.c = d.c; p.bias = d.ep.bias; p.residual = d.ep.residual; p.alpha = d.ep.alpha; p.act = (int)d.ep.act;
  p.m = (int)d.m; p.n = (int)d.n; p.k = (int)d.k; p.a_row = d.a_row; p.b_row = d.b_col; p.c_row = d.c_row;   // b_row: stride between B's [N, K] rows
  p.partial = nullptr; p.counters = nullptr; p.a_vec = 0;
  p.ln_gamma = d.ln_gamma; p.ln_beta = d.ln_beta; p.ln_eps = d.ln_eps;
  const int mr = d.m <= 8 ? 8 : 16;
  const size_t smem = (size_t)mr * d.k * sizeof(float);
  const long long groups = (d.n + kSkR - 1) / kSkR, per_block = kSkThreads / 32;
  long long blocks = (groups + per_block - 1) / per_block;
  const long long cap = (long long)sm_count() * (smem > 48 * 1024 ? 2 : 4);
  if (blocks > cap) blocks = cap;
  cudaError_t e = d.dtype == DType::F32 ? launch_kmajor<float>(s, p, mr, smem, dim3((unsigned)blocks))
                : d.dtype == DType::BF16 ? launch_kmajor<__nv_bfloat16>(s, p, mr, smem, dim3((unsigned)blocks))
                                         : launch_kmajor<__half>(s, p, mr, smem, dim3((unsigned)blocks));
  if (e != cudaSuccess) return cuda_status(e, "matmul (skinny, K-major B)");
  return Status::OK();
}

float* skinny_partials();            // workspace.cu: created with the device context
unsigned int* skinny_counters();

bool skinny_eligible(const GemmDesc& d) {
  if (d.ln_gamma) return false;
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16 || d.dtype == DType::F32) || d.b_dtype != d.dtype) return false;
  if (d.c_f32 || d.ep.argmax_keys || d.ep.b_scales) return false;
  if (d.batch != 1 || d.batch_inner != 1) return false;
  if (d.m < 1 || d.m > kSkMaxM || d.n < 256 || d.n > kSkMaxN || d.k < kSkK) return false;
  if (d.a_col != 1 || d.b_col != 1) return false;                       // A rows along K, B stored [K, N]
  const uintptr_t b_align = d.dtype == DType::F32 ? 15u : 7u;                                            // 4-element loads of B
  if (d.b_row % 4 != 0 || d.n % 4 != 0 || (reinterpret_cast<uintptr_t>(d.b) & b_align) != 0) return false;
  const int64_t ks = (d.k + kSkK - 1) / kSkK;
  if (ks > kSkMaxKSlabs || ks * d.n > kSkMaxPartials) return false;
  return true;
}

Status matmul_skinny(cudaStream_t s, const GemmDesc& d) {
  float* partial = skinny_partials();
  unsigned int* counters = skinny_counters();
  if (!partial || !counters) return Status::compute("matmul (skinny): the kernel workspace is not initialised");
  SkinnyParams p;
  p.a = d.a; p.b = d.b; p.c = d.c; p.bias = d.ep.bias; p.residual = d.ep.residual; p.alpha = d.ep.alpha; p.act = (int)d.ep.act;
  p.m = (int)d.m; p.n = (int)d.n; p.k = (int)d.k; p.a_row = d.a_row; p.b_row = d.b_row; p.c_row = d.c_row;
  p.partial = partial; p.counters = counters;
  p.ln_gamma = nullptr; p.ln_beta = nullptr; p.ln_eps = 0.f;
  p.a_vec = (d.a_row % (d.dtype == DType::F32 ? 4 : 8) == 0 && (reinterpret_cast<uintptr_t>(d.a) & 15u) == 0) ? 1 : 0;
  dim3 grid((unsigned)((d.n + kSkN - 1) / kSkN), (unsigned)((d.k + kSkK - 1) / kSkK), 1);
  cudaError_t e;
  if (d.dtype == DType::BF16) e = launch_pdl(gemm_skinny_kernel<__nv_bfloat16>, grid, dim3(kSkThreads), 0, s, p);
  else if (d.dtype == DType::F32) e = launch_pdl(gemm_skinny_kernel<float>, grid, dim3(kSkThreads), 0, s, p);
  else e = launch_pdl(gemm_skinny_kernel<__half>, grid, dim3(kSkThreads), 0, s, p);
  if (e != cudaSuccess) return cuda_status(e, "matmul (skinny)");
  return Status::OK();
}

}}  // namespace ag::k
