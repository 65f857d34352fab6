// Kernels of the static-shape decode step (one new token per sequence against a preallocated KV cache).
//
// The reference appends to its KV cache by concatenation and recomputes shapes every step
// (python/applegpu_runtime/models/gpt2.py:122-135: concat(dim=1) of the cached and the new keys / values, then the
// non-causal `attention` composition over the grown tensors). Here the cache is a fixed [B, heads, T_max, 64]
// buffer per layer, the current length lives in device memory, and one kernel per layer writes the new key / value
// row in place and attends over rows 0 .. len: the step has the same launch list at every length, so it can be
// captured once as a CUDA graph and replayed.
#include "common.cuh"

namespace ag { namespace k {

float* skinny_partials();            // workspace.cu: created with the device context (shared with the skinny matmul; launches of one
unsigned int* skinny_counters();     // stream never overlap past their dependency wait)

__device__ __forceinline__ unsigned long long globaltimer_ns_dec() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Geometry of a split-K linear work item of a decode step (see decode_linear_kernel below).
constexpr int kDlCols = 64;       // columns per CTA
constexpr int kDlRows = 128;      // K rows per CTA
constexpr int kDlThreads = 256;
constexpr int kDlMaxM = 16;

// One (sequence, head) of a decode step's attention, by the first 128 threads of the block (any others only join
// the barriers and contribute neutral elements to the block reductions, which leaves every sum bit-identical).
// s_qkv: this head's q | k | v of the new token as floats that hold storage-type values; kc / vc: the head's cache
// [t_max, 64]; out_row: 64 outputs; len = tokens already in the cache (the new token becomes row len).
struct AttnDecodeSmem {
  float s_q[64];
  float s_o[2][64];
  float s_red[33];
};
template <typename T>
__device__ __forceinline__ void attn_decode_item(const float* s_qkv, T* kc, T* vc, T* out_row, int len, int t_max, float scale, float* s_scores, AttnDecodeSmem& sm) {
  const int tid = threadIdx.x;
  if (len < 0) len = 0;
  if (len > t_max - 1) len = t_max - 1;      // a full cache overwrites its last row instead of writing past the end
  const int n_keys = len + 1;
  // append the new key / value row in place; stage q (pre-scaled) as floats
  if (tid < 64) { kc[(long long)len * 64 + tid] = Cvt<T>::from(s_qkv[64 + tid]); sm.s_q[tid] = s_qkv[tid] * scale; }
  else if (tid < 128) vc[(long long)len * 64 + (tid - 64)] = Cvt<T>::from(s_qkv[128 + (tid - 64)]);
  __syncthreads();                             // the block's own global writes are visible to it from here
  // scores: one key per thread and pass, the key row read as 16-byte packs
  constexpr int N = Pack<T>::N;                // elements per 16 bytes
  float m_local = -INFINITY;
  if (tid < 128) {
    for (int j = tid; j < n_keys; j += 128) {
      const T* kr = kc + (long long)j * 64;
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < 64 / N; c++) {
        Pack<T> pk = ld16(kr + c * N);
#pragma unroll
        for (int e = 0; e < N; e++) acc = fmaf(sm.s_q[c * N + e], Cvt<T>::to(pk.v[e]), acc);
      }
      s_scores[j] = acc;
      m_local = fmaxf(m_local, acc);
    }
  }
  const float m = block_max(m_local, sm.s_red);
  float l_local = 0.f;
  if (tid < 128) {
    for (int j = tid; j < n_keys; j += 128) { float p = __expf(s_scores[j] - m); s_scores[j] = p; l_local += p; }
  }
  const float l = block_sum(l_local, sm.s_red);
  __syncthreads();
  // output: thread (e, half) sums p_j * V[j][e] over its half of the keys; consecutive threads read consecutive elements
  if (tid < 128) {
    const int e = tid & 63, half = tid >> 6;
    float o = 0.f;
    for (int j = half; j < n_keys; j += 2) o = fmaf(s_scores[j], Cvt<T>::to(vc[(long long)j * 64 + e]), o);
    sm.s_o[half][e] = o;
  }
  __syncthreads();
  if (tid < 64) out_row[tid] = Cvt<T>::from((sm.s_o[0][tid] + sm.s_o[1][tid]) / l);
}

// grid = B * heads, 128 threads. qkv: [B, 3 * d] rows (q | k | v of the new token); caches: [B, heads, t_max, 64];
// out: [B, d] (heads merged). *len_ptr = tokens already in the cache; the new token becomes row *len_ptr.
// `part` non-null: qkv is not materialised; the projection left `slabs` (at most 8) float partials [slab][16][3 * d] and
// this kernel adds them in K order, adds `bias` and rounds to the storage type, exactly as the projection's own last CTA
// would have (all loads of a value in flight before the first addition).
template <typename T>
__global__ void __launch_bounds__(128) attention_decode_kernel(const T* __restrict__ qkv, T* __restrict__ kcache, T* __restrict__ vcache, T* __restrict__ out,
                                                               const int* __restrict__ len_ptr, int heads, int t_max, float scale,
                                                               const float* __restrict__ part, int slabs, const T* __restrict__ bias) {
  extern __shared__ float s_scores[];          // [t_max]
  __shared__ AttnDecodeSmem sm;
  __shared__ float s_qkv[192];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  const int d = heads * 64;
  if (part) {
    for (int i = threadIdx.x; i < 192; i += blockDim.x) {
      const int col = (i >> 6) * d + h * 64 + (i & 63);
      float v[8];
#pragma unroll
      for (int ks = 0; ks < 8; ks++) v[ks] = ks < slabs ? __ldcg(part + ((long long)ks * kDlMaxM + b) * 3 * d + col) : 0.f;
      float t = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ks++) if (ks < slabs) t += v[ks];
      if (bias) t += Cvt<T>::to(bias[col]);
      s_qkv[i] = Cvt<T>::to(Cvt<T>::from(t));
    }
  } else {
    const T* row = qkv + (long long)b * 3 * d;
    for (int i = threadIdx.x; i < 192; i += blockDim.x) s_qkv[i] = Cvt<T>::to(row[(i >> 6) * d + h * 64 + (i & 63)]);
  }
  __syncthreads();
  T* kc = kcache + ((long long)b * heads + h) * (long long)t_max * 64;
  T* vc = vcache + ((long long)b * heads + h) * (long long)t_max * 64;
  attn_decode_item<T>(s_qkv, kc, vc, out + (long long)b * d + h * 64, *len_ptr, t_max, scale, s_scores, sm);
}

Status attention_decode(cudaStream_t s, DType dt, const void* qkv, void* kcache, void* vcache, void* out, const int* len_ptr, int batch, int heads,
                        int t_max, float scale, const float* part, int slabs, const void* bias) {
  if (batch <= 0 || heads <= 0) return Status::OK();
  if (part && (slabs < 1 || slabs > 8 || batch > kDlMaxM)) return Status::invalid("attention_decode: 1..8 partial slabs of at most 16 rows");
  if (!part && !qkv) return Status::invalid("attention_decode: no q / k / v");
  if (t_max <= 0 || t_max > 8192) return Status::invalid("attention_decode: cache length must be in 1..8192");
  if (!aligned16(kcache) || !aligned16(vcache)) return Status::compute("attention_decode needs 16-byte aligned caches");
  const size_t smem = (size_t)t_max * sizeof(float);
  cudaError_t le = cudaSuccess;
  AG_DISPATCH_FLOAT(dt, T, (le = launch_pdl(attention_decode_kernel<T>, dim3((unsigned)(batch * heads)), dim3(128), smem, s, (const T*)qkv, (T*)kcache,
                                             (T*)vcache, (T*)out, len_ptr, heads, t_max, scale, part, slabs, (const T*)bias)));
  if (le != cudaSuccess) return cuda_status(le, "attention_decode");
  return Status::OK();
}

// ── linear layer of a decode step ───────────────────────────────────────────
// y[M, N] = act(layer_norm?(x)[M, K] @ W[K, N] + bias) + residual with M <= 16 and W as the reference stores its
// Conv1D weights ([in, out], rows along N). The product is bound by streaming W once, so the grid is
// (N / 64 column slabs) x (K / 128 row slabs) and every CTA has all its weight loads (8-byte loads, two 128-byte rows
// per warp instruction) in flight before it waits for anything. Three things set it apart from the general skinny
// matmul kernel:
//   * W is a model weight, never written by a kernel of the step, so its loads are issued BEFORE the programmatic
//     dependency wait: they overlap the previous kernel's tail, and x (which that kernel produces) is read after it;
//   * layer_norm of x runs in the prologue: every CTA takes the row statistics over the whole rows itself
//     (kernel_templates.rs:1097-1109: mean, population variance, 1/sqrt(var + eps)) and normalises its K slab on the
//     way into shared memory, which removes the separate layer_norm launches of the step;
//   * same deterministic reduction: fp32 partials per K slab in a workspace, the last CTA of a column slab (a
//     counter) adds them in K order and applies bias / activation / residual.


struct DecodeLinearParams {
  const void* x; const void* w; void* y;
  const void* bias; const void* residual; const void* ln_gamma; const void* ln_beta;
  float ln_eps; int act;
  int m, n, k;
  long long x_row, w_row, y_row;
  float* partial;            // [k_slabs][16][n]
  unsigned int* counters;    // one per column slab, zero between launches
  // x not materialised: it is act(sum over xp_slabs of xp[slab][m][.] + xp_bias) rounded to the storage type, i.e. the
  // unfinished result of the previous linear of the step (its row length is this linear's k)
  const float* xp = nullptr; int xp_slabs = 0; const void* xp_bias = nullptr; int xp_act = 0;
  // leave the result unfinished: only the partials are written, and the kernel that consumes them adds them up (no
  // fence, counter and reload by a last CTA on this launch's tail); y, bias, act and residual are then unused
  int partial_only = 0;
};

template <typename T> struct DlVec { using type = uint2; };      // four consecutive 16-bit weights
template <> struct DlVec<float> { using type = uint4; };

// Shared memory of one linear work item (a 64-column x 128-row slab of W against all rows of x).
struct DlSmem {
  float sX[kDlMaxM][kDlRows];                 // this item's slab of x (normalised if asked), as float
  float sSum[kDlThreads / 32][kDlMaxM][kDlCols];
  float s_mean[kDlMaxM], s_rstd[kDlMaxM];
};

// The item's weights: a warp owns 16 consecutive K rows, a lane four consecutive columns of two of them.
template <typename T>
__device__ __forceinline__ void dl_load_weights(const DecodeLinearParams& p, int n0, int k0, typename DlVec<T>::type (&wv)[8]) {
  using V = typename DlVec<T>::type;
  const T* W = reinterpret_cast<const T*>(p.w);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane >> 4, cl = lane & 15;
  const int col = n0 + cl * 4;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int kk = k0 + warp * 16 + i * 2 + half;
    wv[i] = V{};
    if (kk < p.k && col < p.n) wv[i] = __ldcs(reinterpret_cast<const V*>(W + (long long)kk * p.w_row + col));
  }
}

// Row statistics of layer_norm over the whole rows of x: a warp per row, the row in registers after one round of
// 16-byte loads (kernel_templates.rs:1097-1109: mean, population variance, 1/sqrt(var + eps)). Ends with a block barrier.
template <typename T>
__device__ __forceinline__ void dl_ln_stats(const DecodeLinearParams& p, DlSmem& sm) {
  constexpr int N16 = Pack<T>::N;
  const T* X = reinterpret_cast<const T*>(p.x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int m = warp; m < p.m; m += kDlThreads / 32) {
    const T* xr = X + (long long)m * p.x_row;
    const int packs = p.k / N16;
    float v[8][N16];                                   // up to 8 x 32 packs per row: k <= 256 * N16
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < 8; it++) {
      const int pk = lane + it * 32;
      if (pk < packs) {
        Pack<T> q = ld16(xr + pk * N16);
#pragma unroll
        for (int e = 0; e < N16; e++) { v[it][e] = Cvt<T>::to(q.v[e]); sum += v[it][e]; }
      } else {
#pragma unroll
        for (int e = 0; e < N16; e++) v[it][e] = 0.f;
      }
    }
    const float mean = warp_sum(sum) / (float)p.k;
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < 8; it++) {
      if (lane + it * 32 < packs) {
#pragma unroll
        for (int e = 0; e < N16; e++) { const float dlt = v[it][e] - mean; sq += dlt * dlt; }
      }
    }
    const float var = warp_sum(sq) / (float)p.k;
    if (lane == 0) { sm.s_mean[m] = mean; sm.s_rstd[m] = 1.0f / sqrtf(var + p.ln_eps); }
  }
  __syncthreads();
}

// The item's partial product into p.partial[k_slab][m][n0 ..]: x slab to shared memory (layer_norm applied on the way
// if asked; the statistics must be in sm), the products, the reduction over the CTA's warps in K order.
template <typename T>
__device__ __forceinline__ void dl_partial(const DecodeLinearParams& p, DlSmem& sm, int n0, int k0, int k_slab, const typename DlVec<T>::type (&wv)[8]) {
  const T* X = reinterpret_cast<const T*>(p.x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane >> 4, cl = lane & 15;
  // x slab -> shared as float (M x 128, zero beyond M and K): one 16-byte load per thread
  {
    const int m = threadIdx.x >> 4, ch = threadIdx.x & 15;
    constexpr int PER = kDlRows / 16;                    // 8 elements per thread
    float v[PER];
#pragma unroll
    for (int e = 0; e < PER; e++) v[e] = 0.f;
    const int kk = k0 + ch * PER;
    if (p.xp && m < p.m && kk + PER <= p.k && p.xp_slabs <= 8) {
      // the previous linear's partials, added in K order, + bias, activation, rounded as it would have been stored; all
      // loads of the (at most eight) slabs are in flight before the first addition
      float4 q[8][2];
#pragma unroll
      for (int ks = 0; ks < 8; ks++) {
        if (ks < p.xp_slabs) {
          const float4* src = reinterpret_cast<const float4*>(p.xp + ((long long)ks * kDlMaxM + m) * p.k + kk);
          q[ks][0] = __ldcg(src); q[ks][1] = __ldcg(src + 1);
        } else {
          q[ks][0] = make_float4(0.f, 0.f, 0.f, 0.f); q[ks][1] = q[ks][0];
        }
      }
      float t[PER];
#pragma unroll
      for (int e = 0; e < PER; e++) t[e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ks++) {
        if (ks < p.xp_slabs) {
          t[0] += q[ks][0].x; t[1] += q[ks][0].y; t[2] += q[ks][0].z; t[3] += q[ks][0].w;
          t[4] += q[ks][1].x; t[5] += q[ks][1].y; t[6] += q[ks][1].z; t[7] += q[ks][1].w;
        }
      }
#pragma unroll
      for (int e = 0; e < PER; e++) {
        if (p.xp_bias) t[e] += Cvt<T>::to(reinterpret_cast<const T*>(p.xp_bias)[kk + e]);
        v[e] = Cvt<T>::to(Cvt<T>::from(apply_act(t[e], (Act)p.xp_act)));
      }
    } else if (p.xp && m < p.m && kk < p.k) {
      for (int e = 0; e < PER; e++) {
        if (kk + e < p.k) {
          float t = 0.f;
          for (int ks = 0; ks < p.xp_slabs; ks++) t += __ldcg(p.xp + ((long long)ks * kDlMaxM + m) * p.k + kk + e);
          if (p.xp_bias) t += Cvt<T>::to(reinterpret_cast<const T*>(p.xp_bias)[kk + e]);
          v[e] = Cvt<T>::to(Cvt<T>::from(apply_act(t, (Act)p.xp_act)));
        }
      }
    } else if (m < p.m && kk < p.k) {
      const T* src = X + (long long)m * p.x_row + kk;
      if (kk + PER <= p.k) {
        if constexpr (sizeof(T) == 4) {
          const float4 q0 = *reinterpret_cast<const float4*>(src), q1 = *reinterpret_cast<const float4*>(src + 4);
          v[0] = q0.x; v[1] = q0.y; v[2] = q0.z; v[3] = q0.w; v[4] = q1.x; v[5] = q1.y; v[6] = q1.z; v[7] = q1.w;
        } else {
          Pack<T> q = ld16(src);
#pragma unroll
          for (int e = 0; e < PER; e++) v[e] = Cvt<T>::to(q.v[e]);
        }
      } else {
        for (int e = 0; e < PER; e++) if (kk + e < p.k) v[e] = Cvt<T>::to(src[e]);
      }
      if (p.ln_gamma) {
        const T* G = reinterpret_cast<const T*>(p.ln_gamma);
        const T* Bt = reinterpret_cast<const T*>(p.ln_beta);
        const float mean = sm.s_mean[m], rstd = sm.s_rstd[m];
        for (int e = 0; e < PER; e++) if (kk + e < p.k) v[e] = Cvt<T>::to(G[kk + e]) * (v[e] - mean) * rstd + Cvt<T>::to(Bt[kk + e]);
      }
    }
#pragma unroll
    for (int e = 0; e < PER; e++) sm.sX[m][ch * PER + e] = v[e];
  }
  __syncthreads();
  float acc[kDlMaxM][4];
#pragma unroll
  for (int m = 0; m < kDlMaxM; m++) { acc[m][0] = 0.f; acc[m][1] = 0.f; acc[m][2] = 0.f; acc[m][3] = 0.f; }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int kk = warp * 16 + i * 2 + half;
    const T* pr = reinterpret_cast<const T*>(&wv[i]);
    const float b0 = Cvt<T>::to(pr[0]), b1 = Cvt<T>::to(pr[1]), b2 = Cvt<T>::to(pr[2]), b3 = Cvt<T>::to(pr[3]);
#pragma unroll
    for (int m = 0; m < kDlMaxM; m++) {
      const float a = sm.sX[m][kk];                      // two addresses per warp (one per half): broadcasts
      acc[m][0] = fmaf(a, b0, acc[m][0]); acc[m][1] = fmaf(a, b1, acc[m][1]);
      acc[m][2] = fmaf(a, b2, acc[m][2]); acc[m][3] = fmaf(a, b3, acc[m][3]);
    }
  }
  // the two half-warps hold different rows of the same columns
#pragma unroll
  for (int m = 0; m < kDlMaxM; m++) {
#pragma unroll
    for (int e = 0; e < 4; e++) acc[m][e] += __shfl_xor_sync(0xffffffffu, acc[m][e], 16);
  }
  if (half == 0) {
#pragma unroll
    for (int m = 0; m < kDlMaxM; m++) *reinterpret_cast<float4*>(&sm.sSum[warp][m][cl * 4]) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  }
  __syncthreads();
  float* my_partial = p.partial + ((long long)k_slab * kDlMaxM) * p.n;
  for (int i = threadIdx.x; i < kDlMaxM * kDlCols; i += kDlThreads) {
    int m = i / kDlCols, c = i % kDlCols;
    if (m < p.m && n0 + c < p.n) {
      float v = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kDlThreads / 32; w8++) v += sm.sSum[w8][m][c];    // warp order = K order
      my_partial[(long long)m * p.n + n0 + c] = v;
    }
  }
}

// One finished element: the K slabs' partials added in K order (deterministic), bias, activation, residual.
template <typename T>
__device__ __forceinline__ float dl_finish_element(const DecodeLinearParams& p, int k_slabs, int m, int col) {
  float v = 0.f;
  for (int ks = 0; ks < k_slabs; ks++) v += __ldcg(p.partial + ((long long)ks * kDlMaxM + m) * p.n + col);
  if (p.bias) v += Cvt<T>::to(reinterpret_cast<const T*>(p.bias)[col]);
  v = apply_act(v, (Act)p.act);
  if (p.residual) v += Cvt<T>::to(reinterpret_cast<const T*>(p.residual)[(long long)m * p.y_row + col]);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kDlThreads) decode_linear_kernel(const DecodeLinearParams p) {
  using V = typename DlVec<T>::type;
  __shared__ DlSmem sm;
  __shared__ unsigned int s_last;
  const int n0 = blockIdx.x * kDlCols, k0 = blockIdx.y * kDlRows;
  // weights first, before the dependency wait (they are not produced by the step)
  V wv[8];
  dl_load_weights<T>(p, n0, k0, wv);
  pdl_wait();      // x, the residual and the workspace belong to the step: nothing of them is touched above this line
  pdl_trigger();
  if (p.ln_gamma) dl_ln_stats<T>(p, sm);
  dl_partial<T>(p, sm, n0, k0, (int)blockIdx.y, wv);
  if (p.partial_only) return;     // the consumer adds the partials up; the end of this grid orders them before its reads
  const int k_slabs = gridDim.y;
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
  T* Y = reinterpret_cast<T*>(p.y);
  for (int i = threadIdx.x; i < kDlMaxM * kDlCols; i += kDlThreads) {
    int m = i / kDlCols, c = i % kDlCols;
    if (m < p.m && n0 + c < p.n) Y[(long long)m * p.y_row + n0 + c] = Cvt<T>::from(dl_finish_element<T>(p, k_slabs, m, n0 + c));
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;   // ready for the next launch on this stream
}


bool decode_linear_eligible(const GemmDesc& d) {
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16 || d.dtype == DType::F32) || d.b_dtype != d.dtype) return false;
  if (d.c_f32 || d.ep.argmax_keys || d.ep.b_scales || d.ep.alpha != 1.0f) return false;
  if (d.batch != 1 || d.batch_inner != 1 || d.m < 1 || d.m > kDlMaxM || d.n < 64 || d.n > 65536 || d.k < 16) return false;
  if (d.a_col != 1 || d.b_col != 1 || d.b_row % 4 != 0 || d.n % 4 != 0) return false;      // W stored [K, N]; 4-element loads
  const uintptr_t align = d.dtype == DType::F32 ? 15u : 7u;
  if ((reinterpret_cast<uintptr_t>(d.b) & align) != 0) return false;
  const int n16 = d.dtype == DType::F32 ? 4 : 8;
  if (d.a_row % n16 != 0 || (reinterpret_cast<uintptr_t>(d.a) & 15u) != 0 || d.k % 8 != 0) return false;   // 16-byte loads of x
  if (d.ln_gamma && (d.k % n16 != 0 || d.k > 256 * n16)) return false;                                     // a row fits the registers of one warp
  const int64_t ks = (d.k + kDlRows - 1) / kDlRows;
  if (ks > 64 || ks * kDlMaxM * d.n > (int64_t)kDecodeRegionFloats) return false;                         // one workspace region: [k_slabs][16][n] floats
  return true;
}

float* decode_partial_region(int region) {
  float* base = skinny_partials();
  return base ? base + (size_t)region * kDecodeRegionFloats : nullptr;
}

Status decode_linear(cudaStream_t s, const GemmDesc& d, const DecodeLinearOpts& o) {
  if (!decode_linear_eligible(d)) return Status::invalid("decode_linear: shape or layout not supported");
  if (o.region < 0 || o.region >= kDecodeRegions) return Status::invalid("decode_linear: partial region");
  if (o.xp && (o.xp_slabs < 1 || o.xp_slabs > 64)) return Status::invalid("decode_linear: partial slabs of the input");
  if (((d.k + kDlRows - 1) / kDlRows) * kDlMaxM * d.n > (int64_t)kDecodeRegionFloats) return Status::invalid("decode_linear: partials exceed a workspace region");
  float* partial = decode_partial_region(o.region);
  unsigned int* counters = skinny_counters();
  if (!partial || !counters) return Status::compute("decode_linear: the kernel workspace is not initialised");
  DecodeLinearParams p;
  p.x = d.a; p.w = d.b; p.y = d.c; p.bias = d.ep.bias; p.residual = d.ep.residual; p.ln_gamma = d.ln_gamma; p.ln_beta = d.ln_beta; p.ln_eps = d.ln_eps;
  p.act = (int)d.ep.act; p.m = (int)d.m; p.n = (int)d.n; p.k = (int)d.k;
  p.x_row = d.a_row; p.w_row = d.b_row; p.y_row = d.c_row; p.partial = partial; p.counters = counters;
  p.partial_only = o.partial_only ? 1 : 0;
  p.xp = o.xp; p.xp_slabs = o.xp_slabs; p.xp_bias = o.xp_bias; p.xp_act = (int)o.xp_act;
  cudaError_t e;
  dim3 grid((unsigned)((d.n + kDlCols - 1) / kDlCols), (unsigned)((d.k + kDlRows - 1) / kDlRows), 1);
  if (d.dtype == DType::BF16) e = launch_pdl(decode_linear_kernel<__nv_bfloat16>, grid, dim3(kDlThreads), 0, s, p);
  else if (d.dtype == DType::F16) e = launch_pdl(decode_linear_kernel<__half>, grid, dim3(kDlThreads), 0, s, p);
  else e = launch_pdl(decode_linear_kernel<float>, grid, dim3(kDlThreads), 0, s, p);
  if (e != cudaSuccess) return cuda_status(e, "decode_linear");
  return Status::OK();
}

// ── the layers of a decode step as one persistent kernel ────────────────────
// Sixty dependent launches of a few microseconds each are bound by what lies between kernels (the drain of one grid,
// the dependency resolution and ramp of the next: ~8 µs per launch even inside a CUDA graph with programmatic edges).
// Here one cooperative grid walks all layers and separates the phases with a grid-wide barrier of its own (~1 µs):
//   E    x = wte[tok] + wpe[pos]
//   per layer:
//   P1   partial products of ln_1(x) @ W_qkv                      (36 x 6 items of 64 columns x 128 K rows)
//   P2   attention per (sequence, head): q, k, v summed from P1's partials, cache appended in place   (B x heads items)
//   P3   partial products of att @ W_proj                         (12 x 6 items)
//   P3b  x2 = x + sum of P3's partials + bias                     (element-wise)
//   P4   partial products of ln_2(x2) @ W_fc                      (48 x 6 items)
//   P5   partial products of gelu(P4 + bias) @ W_fc2, the operand summed from P4's partials on the way in   (12 x 24 items)
//   P5b  x = x2 + sum of P5's partials + bias                     (element-wise)
// Every item runs the same device functions, in the same order of additions, as the per-op kernels above, so the
// stream of tokens is the one the per-op engine produces. The barrier: one counter in global memory, cleared by a
// memset node before the launch; each CTA adds one and spins (bounded: 2 s, then an error word is set and every CTA
// leaves at its next barrier) until the count reaches phases-so-far x CTAs. The launch is cooperative, so all CTAs
// are resident and the spin cannot wait for a CTA that has not started.
struct MegaLayerW {
  const void *ln1_g, *ln1_b, *w_qkv, *b_qkv, *w_proj, *b_proj, *ln2_g, *ln2_b, *w_fc, *b_fc, *w_fc2, *b_fc2;
  void *kcache, *vcache;
};
struct MegaParams {
  const MegaLayerW* layers;
  int n_layer, heads, d, t_max, batch;
  const void *wte, *wpe;
  const int32_t *tok, *pos;
  const int* len_ptr;
  void *x, *x2, *att;             // [16][d] of the storage type
  float* partial;                 // four regions: qkv, proj, fc, fc2 partials
  unsigned int* bar;
  int* err;
  float scale;
};

#ifdef AG_DECODE_PROBE
__device__ unsigned long long g_mega_probe[2048];   // CTA 0: time after every barrier (ns)
__device__ int g_mega_probe_n;
#endif
__device__ __forceinline__ bool mega_barrier(const MegaParams& p, unsigned int& target) {
#ifdef AG_DECODE_PROBE
  if (blockIdx.x == 0 && threadIdx.x == 0 && g_mega_probe_n < 2046) g_mega_probe[g_mega_probe_n++] = globaltimer_ns_dec();   // arrival
#endif
  __syncthreads();
  if (threadIdx.x == 0) {
    target += gridDim.x;
    __threadfence();
    atomicAdd(p.bar, 1u);
    const unsigned long long t0 = globaltimer_ns_dec();
    unsigned int spins = 0;
    while (true) {
      unsigned int seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.bar) : "memory");
      if (seen >= target) break;
      if ((++spins & 0x3ffu) == 0) {
        if (*reinterpret_cast<volatile int*>(p.err) != 0) break;
        if (globaltimer_ns_dec() - t0 > 2000000000ull) { atomicCAS(p.err, 0, 31); break; }
      }
    }
    __threadfence();
  }
  __syncthreads();
#ifdef AG_DECODE_PROBE
  if (blockIdx.x == 0 && threadIdx.x == 0 && g_mega_probe_n < 2046) g_mega_probe[g_mega_probe_n++] = globaltimer_ns_dec();   // release
#endif
  return *reinterpret_cast<volatile int*>(p.err) == 0;
}

template <typename T>
__global__ void __launch_bounds__(kDlThreads, 2) decode_layers_kernel(const MegaParams p) {
  using V = typename DlVec<T>::type;
#ifdef AG_DECODE_PROBE
  if (blockIdx.x == 0 && threadIdx.x == 0) { g_mega_probe_n = 0; g_mega_probe[g_mega_probe_n++] = globaltimer_ns_dec(); }
#endif
  extern __shared__ float s_scores[];          // [t_max]
  __shared__ DlSmem sm;
  __shared__ AttnDecodeSmem asm_;
  __shared__ float s_qkv[192];
  const int D = p.d, B = p.batch;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  unsigned int target = 0;
  float* part_qkv = p.partial;
  float* part_proj = part_qkv + (long long)((D + kDlRows - 1) / kDlRows) * kDlMaxM * 3 * D;
  float* part_fc = part_proj + (long long)((D + kDlRows - 1) / kDlRows) * kDlMaxM * D;
  float* part_fc2 = part_fc + (long long)((D + kDlRows - 1) / kDlRows) * kDlMaxM * 4 * D;
  const int ks_d = (D + kDlRows - 1) / kDlRows, ks_4d = (4 * D + kDlRows - 1) / kDlRows;

  // The weights of this CTA's first item of the next linear phase are fetched as soon as the current linear phase is
  // done (they are constants of the model): the loads fly during the barriers and the phases in between, as the per-op
  // kernels fetch theirs ahead of the dependency wait.
  V wv_next[8];
  auto prefetch = [&](const void* wgt, int n, int k) {
    DecodeLinearParams lp{};
    lp.w = wgt; lp.n = n; lp.k = k; lp.w_row = n;
    const int n_slabs = (n + kDlCols - 1) / kDlCols, k_slabs = (k + kDlRows - 1) / kDlRows;
    if (cta < n_slabs * k_slabs) dl_load_weights<T>(lp, (cta % n_slabs) * kDlCols, (cta / n_slabs) * kDlRows, wv_next);
  };
  // one linear's partial products over the grid
  auto linear_partials = [&](DecodeLinearParams lp) {
    const int n_slabs = (lp.n + kDlCols - 1) / kDlCols, k_slabs = (lp.k + kDlRows - 1) / kDlRows;
    bool stats = false;
    for (int it = cta; it < n_slabs * k_slabs; it += G) {
      const int ns = it % n_slabs, ks = it / n_slabs;
      V wv[8];
      if (it == cta) {
#pragma unroll
        for (int i = 0; i < 8; i++) wv[i] = wv_next[i];
      } else {
        dl_load_weights<T>(lp, ns * kDlCols, ks * kDlRows, wv);
      }
      __syncthreads();                       // the previous item's shared-memory reads are done
      if (lp.ln_gamma && !stats) { dl_ln_stats<T>(lp, sm); stats = true; }
      dl_partial<T>(lp, sm, ns * kDlCols, ks * kDlRows, ks, wv);
    }
  };
  // y = round(sum of partials + bias + residual) over the grid
  auto finish_rows = [&](const DecodeLinearParams& lp, int k_slabs) {
    T* Y = reinterpret_cast<T*>(lp.y);
    for (int i = cta * kDlThreads + threadIdx.x; i < lp.m * lp.n; i += G * kDlThreads) {
      const int m = i / lp.n, c = i % lp.n;
      Y[(long long)m * lp.y_row + c] = Cvt<T>::from(dl_finish_element<T>(lp, k_slabs, m, c));
    }
  };

  // E: embeddings (a row per CTA; the sum rounded once, as the embedding kernel stores it)
  for (int b = cta; b < B; b += G) {
    const T* te = reinterpret_cast<const T*>(p.wte) + (long long)p.tok[b] * D;
    const T* pe = reinterpret_cast<const T*>(p.wpe) + (long long)p.pos[b] * D;
    T* xr = reinterpret_cast<T*>(p.x) + (long long)b * D;
    for (int i = threadIdx.x; i < D; i += kDlThreads) xr[i] = Cvt<T>::from(Cvt<T>::to(te[i]) + Cvt<T>::to(pe[i]));
  }
  prefetch(p.layers[0].w_qkv, 3 * D, D);
  if (!mega_barrier(p, target)) return;

  for (int l = 0; l < p.n_layer; l++) {
    const MegaLayerW& w = p.layers[l];
    DecodeLinearParams lp;
    // P1: ln_1(x) @ W_qkv
    lp = DecodeLinearParams{};
    lp.x = p.x; lp.w = w.w_qkv; lp.ln_gamma = w.ln1_g; lp.ln_beta = w.ln1_b; lp.ln_eps = 1e-5f;
    lp.m = B; lp.n = 3 * D; lp.k = D; lp.x_row = D; lp.w_row = 3 * D; lp.y_row = 3 * D; lp.partial = part_qkv;
    linear_partials(lp);
    prefetch(w.w_proj, D, D);
    if (!mega_barrier(p, target)) return;
    // P2: attention; q | k | v of the new token = P1's partials + bias, rounded as the projection would have stored them
    for (int it = cta; it < B * p.heads; it += G) {
      const int b = it / p.heads, h = it % p.heads;
      __syncthreads();
      for (int i = threadIdx.x; i < 192; i += kDlThreads) {
        const int col = (i >> 6) * D + h * 64 + (i & 63);
        float t = 0.f;
        for (int ks = 0; ks < ks_d; ks++) t += __ldcg(part_qkv + ((long long)ks * kDlMaxM + b) * 3 * D + col);
        t += Cvt<T>::to(reinterpret_cast<const T*>(w.b_qkv)[col]);
        s_qkv[i] = Cvt<T>::to(Cvt<T>::from(t));
      }
      __syncthreads();
      T* kc = reinterpret_cast<T*>(w.kcache) + ((long long)b * p.heads + h) * (long long)p.t_max * 64;
      T* vc = reinterpret_cast<T*>(w.vcache) + ((long long)b * p.heads + h) * (long long)p.t_max * 64;
      attn_decode_item<T>(s_qkv, kc, vc, reinterpret_cast<T*>(p.att) + (long long)b * D + h * 64, *p.len_ptr, p.t_max, p.scale, s_scores, asm_);
    }
    if (!mega_barrier(p, target)) return;
    // P3: att @ W_proj, then x2 = x + that + bias
    lp = DecodeLinearParams{};
    lp.x = p.att; lp.w = w.w_proj; lp.m = B; lp.n = D; lp.k = D; lp.x_row = D; lp.w_row = D; lp.y_row = D; lp.partial = part_proj;
    linear_partials(lp);
    prefetch(w.w_fc, 4 * D, D);
    if (!mega_barrier(p, target)) return;
    lp.y = p.x2; lp.bias = w.b_proj; lp.residual = p.x;
    finish_rows(lp, ks_d);
    if (!mega_barrier(p, target)) return;
    // P4: ln_2(x2) @ W_fc
    lp = DecodeLinearParams{};
    lp.x = p.x2; lp.w = w.w_fc; lp.ln_gamma = w.ln2_g; lp.ln_beta = w.ln2_b; lp.ln_eps = 1e-5f;
    lp.m = B; lp.n = 4 * D; lp.k = D; lp.x_row = D; lp.w_row = 4 * D; lp.y_row = 4 * D; lp.partial = part_fc;
    linear_partials(lp);
    prefetch(w.w_fc2, D, 4 * D);
    if (!mega_barrier(p, target)) return;
    // P5: gelu(P4 + bias) @ W_fc2, then x = x2 + that + bias
    lp = DecodeLinearParams{};
    lp.x = nullptr; lp.xp = part_fc; lp.xp_slabs = ks_d; lp.xp_bias = w.b_fc; lp.xp_act = (int)Act::GeluTanh;
    lp.w = w.w_fc2; lp.m = B; lp.n = D; lp.k = 4 * D; lp.x_row = 4 * D; lp.w_row = D; lp.y_row = D; lp.partial = part_fc2;
    linear_partials(lp);
    if (l + 1 < p.n_layer) prefetch(p.layers[l + 1].w_qkv, 3 * D, D);
    if (!mega_barrier(p, target)) return;
    lp.y = p.x; lp.bias = w.b_fc2; lp.residual = p.x2;
    finish_rows(lp, ks_4d);
    if (!mega_barrier(p, target)) return;
  }
}

// Enqueues the barrier reset and the cooperative launch. `layers` is a device array of n_layer entries.
Status decode_layers(cudaStream_t s, DType dt, const void* layers, int n_layer, int heads, int d, int t_max, int batch, const void* wte, const void* wpe,
                     const int32_t* tok, const int32_t* pos, const int* len_ptr, void* x, void* x2, void* att, unsigned int* bar, int* err) {
  if (batch < 1 || batch > kDlMaxM || d != heads * 64 || d % 8 != 0 || t_max < 1 || t_max > 8192) return Status::invalid("decode_layers: shape not supported");
  float* partial = skinny_partials();
  if (!partial) return Status::compute("decode_layers: the kernel workspace is not initialised");
  const long long ks_d = (d + kDlRows - 1) / kDlRows, ks_4d = (4 * d + kDlRows - 1) / kDlRows;
  const long long need = (ks_d * kDlMaxM * 3 * d) + (ks_d * kDlMaxM * d) + (ks_d * kDlMaxM * 4 * d) + (ks_4d * kDlMaxM * d);
  if (need > ((long long)1 << 18) * 16) return Status::invalid("decode_layers: the partial sums do not fit the workspace");
  MegaParams p;
  p.layers = static_cast<const MegaLayerW*>(layers); p.n_layer = n_layer; p.heads = heads; p.d = d; p.t_max = t_max; p.batch = batch;
  p.wte = wte; p.wpe = wpe; p.tok = tok; p.pos = pos; p.len_ptr = len_ptr; p.x = x; p.x2 = x2; p.att = att;
  p.partial = partial; p.bar = bar; p.err = err; p.scale = 1.0f / sqrtf(64.0f);
  // 42 KB of static shared memory leave ~5 KB of the default 48 KB for the scores: longer caches need the opt-in (set
  // on the first, uncaptured call)
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ae = cudaFuncSetAttribute(decode_layers_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * (int)sizeof(float));
    if (ae == cudaSuccess) ae = cudaFuncSetAttribute(decode_layers_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * (int)sizeof(float));
    if (ae == cudaSuccess) ae = cudaFuncSetAttribute(decode_layers_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * (int)sizeof(float));
    if (ae != cudaSuccess) return cuda_status(ae, "decode_layers shared-memory attribute");
    attr_set = true;
  }
  cudaError_t e = cudaMemsetAsync(bar, 0, sizeof(unsigned int), s);
  if (e != cudaSuccess) return cuda_status(e, "decode_layers barrier reset");
  cudaLaunchConfig_t cfg = {};
  // up to two CTAs per SM (every linear phase then has at most one item per CTA), as many as can be resident together
  int per_sm = 0;
  const size_t dyn = (size_t)t_max * sizeof(float);
  cudaError_t oe = dt == DType::BF16 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<__nv_bfloat16>, kDlThreads, dyn)
                   : dt == DType::F16 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<__half>, kDlThreads, dyn)
                                      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<float>, kDlThreads, dyn);
  if (oe != cudaSuccess || per_sm < 1) return Status::compute("decode_layers: the kernel does not fit an SM");
  if (per_sm > 2) per_sm = 2;
  cfg.gridDim = dim3((unsigned)(sm_count() * per_sm), 1, 1);
  cfg.blockDim = dim3(kDlThreads, 1, 1);
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeCooperative;
  attr.val.cooperative = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  if (dt == DType::BF16) e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<__nv_bfloat16>, p);
  else if (dt == DType::F16) e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<__half>, p);
  else e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<float>, p);
  if (e != cudaSuccess) return cuda_status(e, "decode_layers");
  return Status::OK();
}
#ifdef AG_DECODE_PROBE
extern "C" __attribute__((visibility("default"))) int applegpu_debug_decode_probe(unsigned long long* out, int cap) {
  int n = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&n, g_mega_probe_n, sizeof(int));
  if (n > cap) n = cap;
  if (n > 0) cudaMemcpyFromSymbol(out, g_mega_probe, sizeof(unsigned long long) * n);
  return n;
}
#endif
size_t decode_layers_table_bytes(int n_layer) { return sizeof(MegaLayerW) * (size_t)n_layer; }
void decode_layers_fill_entry(void* host_table, int l, const void* const* w12, void* kcache, void* vcache) {
  MegaLayerW& e = static_cast<MegaLayerW*>(host_table)[l];
  e.ln1_g = w12[0]; e.ln1_b = w12[1]; e.w_qkv = w12[2]; e.b_qkv = w12[3]; e.w_proj = w12[4]; e.b_proj = w12[5];
  e.ln2_g = w12[6]; e.ln2_b = w12[7]; e.w_fc = w12[8]; e.b_fc = w12[9]; e.w_fc2 = w12[10]; e.b_fc2 = w12[11];
  e.kcache = kcache; e.vcache = vcache;
}

// End of a decode step: the picked tokens go into the history, the next step's position ids are written, and the
// step and length counters advance. One block; every thread reads the counters before thread 0 changes them.
// `keys` non-null: the step's tokens are still the (value, column) keys the LM head's row-argmax epilogue merged; this
// kernel turns them into token ids itself (what argmax_finalize does: no key and the sticky-NaN key both mean column 0)
// and clears them for the next step, which saves the step a launch and a memset.
__global__ void decode_finish_kernel(int32_t* __restrict__ tok, int32_t* __restrict__ history, int32_t* __restrict__ pos_ids, int* step_ptr, int* len_ptr,
                                     int batch, int max_steps, unsigned long long* __restrict__ keys) {
  pdl_wait();
  pdl_trigger();
  const int step = *step_ptr, len = *len_ptr;
  __syncthreads();
  for (int t = threadIdx.x; t < batch; t += blockDim.x) {
    int32_t token;
    if (keys) {
      const unsigned long long k = keys[t];
      token = (k == 0ull || k == 0xffffffffffffffffull) ? 0 : (int32_t)(0xffffffffu - (uint32_t)(k & 0xffffffffu));
      keys[t] = 0ull;
      tok[t] = token;
    } else {
      token = tok[t];
    }
    if (step < max_steps) history[(long long)step * batch + t] = token;
    pos_ids[t] = len + 1;
  }
  if (threadIdx.x == 0) { *step_ptr = step + 1; *len_ptr = len + 1; }
}

Status decode_finish(cudaStream_t s, int32_t* tok, int32_t* history, int32_t* pos_ids, int* step_ptr, int* len_ptr, int batch, int max_steps,
                     unsigned long long* keys) {
  cudaError_t le = launch_pdl(decode_finish_kernel, dim3(1), dim3(128), 0, s, tok, history, pos_ids, step_ptr, len_ptr, batch, max_steps, keys);
  if (le != cudaSuccess) return cuda_status(le, "decode_finish");
  return Status::OK();
}

// counters[0] = step, counters[1] = len; pos_ids[0..batch) = len
__global__ void decode_reset_kernel(int* counters, int32_t* pos_ids, int batch, int len) {
  for (int t = threadIdx.x; t < batch; t += blockDim.x) pos_ids[t] = len;
  if (threadIdx.x == 0) { counters[0] = 0; counters[1] = len; }
}
Status decode_reset(cudaStream_t s, int* counters, int32_t* pos_ids, int batch, int len) {
  decode_reset_kernel<<<1, 128, 0, s>>>(counters, pos_ids, batch, len);
  AG_CHECK_LAUNCH("decode_reset");
  return Status::OK();
}

}}  // namespace ag::k
