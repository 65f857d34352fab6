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

// grid = B * heads, 128 threads. qkv: [B, 3 * d] rows (q | k | v of the new token); caches: [B, heads, t_max, 64];
// out: [B, d] (heads merged). *len_ptr = tokens already in the cache; the new token becomes row *len_ptr.
template <typename T>
__global__ void __launch_bounds__(128) attention_decode_kernel(const T* __restrict__ qkv, T* __restrict__ kcache, T* __restrict__ vcache, T* __restrict__ out,
                                                               const int* __restrict__ len_ptr, int heads, int t_max, float scale) {
  extern __shared__ float s_scores[];          // [t_max]
  __shared__ float s_q[64];
  __shared__ float s_o[2][64];
  __shared__ float s_red[33];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  const int d = heads * 64;
  const int tid = threadIdx.x;
  int len = *len_ptr;
  if (len < 0) len = 0;
  if (len > t_max - 1) len = t_max - 1;      // a full cache overwrites its last row instead of writing past the end
  const int n_keys = len + 1;
  const T* row = qkv + (long long)b * 3 * d;
  T* kc = kcache + ((long long)b * heads + h) * (long long)t_max * 64;
  T* vc = vcache + ((long long)b * heads + h) * (long long)t_max * 64;
  // append the new key / value row in place; stage q (pre-scaled) as floats
  if (tid < 64) { kc[(long long)len * 64 + tid] = row[d + h * 64 + tid]; s_q[tid] = Cvt<T>::to(row[h * 64 + tid]) * scale; }
  else vc[(long long)len * 64 + (tid - 64)] = row[2 * d + h * 64 + (tid - 64)];
  __syncthreads();                             // the block's own global writes are visible to it from here
  // scores: one key per thread and pass, the key row read as 16-byte packs
  constexpr int N = Pack<T>::N;                // elements per 16 bytes
  float m_local = -INFINITY;
  for (int j = tid; j < n_keys; j += 128) {
    const T* kr = kc + (long long)j * 64;
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < 64 / N; c++) {
      Pack<T> pk = ld16(kr + c * N);
#pragma unroll
      for (int e = 0; e < N; e++) acc = fmaf(s_q[c * N + e], Cvt<T>::to(pk.v[e]), acc);
    }
    s_scores[j] = acc;
    m_local = fmaxf(m_local, acc);
  }
  const float m = block_max(m_local, s_red);
  float l_local = 0.f;
  for (int j = tid; j < n_keys; j += 128) { float p = __expf(s_scores[j] - m); s_scores[j] = p; l_local += p; }
  const float l = block_sum(l_local, s_red);
  __syncthreads();
  // output: thread (e, half) sums p_j * V[j][e] over its half of the keys; consecutive threads read consecutive elements
  const int e = tid & 63, half = tid >> 6;
  float o = 0.f;
  for (int j = half; j < n_keys; j += 2) o = fmaf(s_scores[j], Cvt<T>::to(vc[(long long)j * 64 + e]), o);
  s_o[half][e] = o;
  __syncthreads();
  if (tid < 64) out[(long long)b * d + h * 64 + tid] = Cvt<T>::from((s_o[0][tid] + s_o[1][tid]) / l);
}

Status attention_decode(cudaStream_t s, DType dt, const void* qkv, void* kcache, void* vcache, void* out, const int* len_ptr, int batch, int heads,
                        int t_max, float scale) {
  if (batch <= 0 || heads <= 0) return Status::OK();
  if (t_max <= 0 || t_max > 8192) return Status::invalid("attention_decode: cache length must be in 1..8192");
  if (!aligned16(kcache) || !aligned16(vcache)) return Status::compute("attention_decode needs 16-byte aligned caches");
  const size_t smem = (size_t)t_max * sizeof(float);
  cudaError_t le = cudaSuccess;
  AG_DISPATCH_FLOAT(dt, T, (le = launch_pdl(attention_decode_kernel<T>, dim3((unsigned)(batch * heads)), dim3(128), smem, s, (const T*)qkv, (T*)kcache,
                                             (T*)vcache, (T*)out, len_ptr, heads, t_max, scale)));
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
constexpr int kDlCols = 64;       // columns per CTA
constexpr int kDlRows = 128;      // K rows per CTA
constexpr int kDlThreads = 256;
constexpr int kDlMaxM = 16;

struct DecodeLinearParams {
  const void* x; const void* w; void* y;
  const void* bias; const void* residual; const void* ln_gamma; const void* ln_beta;
  float ln_eps; int act;
  int m, n, k;
  long long x_row, w_row, y_row;
  float* partial;            // [k_slabs][16][n]
  unsigned int* counters;    // one per column slab, zero between launches
};

template <typename T> struct DlVec { using type = uint2; };      // four consecutive 16-bit weights
template <> struct DlVec<float> { using type = uint4; };

template <typename T>
__global__ void __launch_bounds__(kDlThreads) decode_linear_kernel(const DecodeLinearParams p) {
  using V = typename DlVec<T>::type;
  constexpr int N16 = Pack<T>::N;
  __shared__ float sX[kDlMaxM][kDlRows];                 // this CTA's slab of x (normalised if asked), as float
  __shared__ float sSum[kDlThreads / 32][kDlMaxM][kDlCols];
  __shared__ float s_mean[kDlMaxM], s_rstd[kDlMaxM];
  __shared__ unsigned int s_last;
  const int n0 = blockIdx.x * kDlCols, k0 = blockIdx.y * kDlRows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* X = reinterpret_cast<const T*>(p.x);
  const T* W = reinterpret_cast<const T*>(p.w);
  // weights first, before the dependency wait (they are not produced by the step): a warp owns 16 consecutive K rows
  const int half = lane >> 4, cl = lane & 15;
  const int col = n0 + cl * 4;
  V wv[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int kk = k0 + warp * 16 + i * 2 + half;
    wv[i] = V{};
    if (kk < p.k && col < p.n) wv[i] = __ldcs(reinterpret_cast<const V*>(W + (long long)kk * p.w_row + col));
  }
  pdl_wait();      // x, the residual and the workspace belong to the step: nothing of them is touched above this line
  pdl_trigger();
  if (p.ln_gamma) {
    // row statistics over the whole rows: a warp per row, the row in registers after one round of 16-byte loads
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
      if (lane == 0) { s_mean[m] = mean; s_rstd[m] = 1.0f / sqrtf(var + p.ln_eps); }
    }
    __syncthreads();
  }
  // x slab -> shared as float (M x 128, zero beyond M and K): one 16-byte load per thread
  {
    const int m = threadIdx.x >> 4, ch = threadIdx.x & 15;
    constexpr int PER = kDlRows / 16;                    // 8 elements per thread
    float v[PER];
#pragma unroll
    for (int e = 0; e < PER; e++) v[e] = 0.f;
    const int kk = k0 + ch * PER;
    if (m < p.m && kk < p.k) {
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
        const float mean = s_mean[m], rstd = s_rstd[m];
        for (int e = 0; e < PER; e++) if (kk + e < p.k) v[e] = Cvt<T>::to(G[kk + e]) * (v[e] - mean) * rstd + Cvt<T>::to(Bt[kk + e]);
      }
    }
#pragma unroll
    for (int e = 0; e < PER; e++) sX[m][ch * PER + e] = v[e];
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
      const float a = sX[m][kk];                         // two addresses per warp (one per half): broadcasts
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
    for (int m = 0; m < kDlMaxM; m++) *reinterpret_cast<float4*>(&sSum[warp][m][cl * 4]) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  }
  __syncthreads();
  const int k_slabs = gridDim.y;
  float* my_partial = p.partial + ((long long)blockIdx.y * kDlMaxM) * p.n;
  for (int i = threadIdx.x; i < kDlMaxM * kDlCols; i += kDlThreads) {
    int m = i / kDlCols, c = i % kDlCols;
    if (m < p.m && n0 + c < p.n) {
      float v = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kDlThreads / 32; w8++) v += sSum[w8][m][c];    // warp order = K order
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
  T* Y = reinterpret_cast<T*>(p.y);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  const T* R = reinterpret_cast<const T*>(p.residual);
  for (int i = threadIdx.x; i < kDlMaxM * kDlCols; i += kDlThreads) {
    int m = i / kDlCols, c = i % kDlCols;
    if (m < p.m && n0 + c < p.n) {
      float v = 0.f;
      for (int ks = 0; ks < k_slabs; ks++) v += __ldcg(p.partial + ((long long)ks * kDlMaxM + m) * p.n + n0 + c);   // K order: deterministic
      if (bias) v += Cvt<T>::to(bias[n0 + c]);
      v = apply_act(v, (Act)p.act);
      if (R) v += Cvt<T>::to(R[(long long)m * p.y_row + n0 + c]);
      Y[(long long)m * p.y_row + n0 + c] = Cvt<T>::from(v);
    }
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;   // ready for the next launch on this stream
}

float* skinny_partials();            // workspace.cu: created with the device context (shared with the skinny matmul; launches of one
unsigned int* skinny_counters();     // stream never overlap past their dependency wait)

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
  if (ks > 64 || ks * d.n > (1 << 18)) return false;                                                      // workspace: [k_slabs][16][n] floats
  return true;
}

Status decode_linear(cudaStream_t s, const GemmDesc& d) {
  if (!decode_linear_eligible(d)) return Status::invalid("decode_linear: shape or layout not supported");
  float* partial = skinny_partials();
  unsigned int* counters = skinny_counters();
  if (!partial || !counters) return Status::compute("decode_linear: the kernel workspace is not initialised");
  DecodeLinearParams p;
  p.x = d.a; p.w = d.b; p.y = d.c; p.bias = d.ep.bias; p.residual = d.ep.residual; p.ln_gamma = d.ln_gamma; p.ln_beta = d.ln_beta; p.ln_eps = d.ln_eps;
  p.act = (int)d.ep.act; p.m = (int)d.m; p.n = (int)d.n; p.k = (int)d.k;
  p.x_row = d.a_row; p.w_row = d.b_row; p.y_row = d.c_row; p.partial = partial; p.counters = counters;
  cudaError_t e;
  dim3 grid((unsigned)((d.n + kDlCols - 1) / kDlCols), (unsigned)((d.k + kDlRows - 1) / kDlRows), 1);
  if (d.dtype == DType::BF16) e = launch_pdl(decode_linear_kernel<__nv_bfloat16>, grid, dim3(kDlThreads), 0, s, p);
  else if (d.dtype == DType::F16) e = launch_pdl(decode_linear_kernel<__half>, grid, dim3(kDlThreads), 0, s, p);
  else e = launch_pdl(decode_linear_kernel<float>, grid, dim3(kDlThreads), 0, s, p);
  if (e != cudaSuccess) return cuda_status(e, "decode_linear");
  return Status::OK();
}

// End of a decode step: the picked tokens go into the history, the next step's position ids are written, and the
// step and length counters advance. One block; every thread reads the counters before thread 0 changes them.
__global__ void decode_finish_kernel(const int32_t* __restrict__ tok, int32_t* __restrict__ history, int32_t* __restrict__ pos_ids, int* step_ptr, int* len_ptr,
                                     int batch, int max_steps) {
  pdl_wait();
  pdl_trigger();
  const int step = *step_ptr, len = *len_ptr;
  __syncthreads();
  for (int t = threadIdx.x; t < batch; t += blockDim.x) {
    if (step < max_steps) history[(long long)step * batch + t] = tok[t];
    pos_ids[t] = len + 1;
  }
  if (threadIdx.x == 0) { *step_ptr = step + 1; *len_ptr = len + 1; }
}

Status decode_finish(cudaStream_t s, const int32_t* tok, int32_t* history, int32_t* pos_ids, int* step_ptr, int* len_ptr, int batch, int max_steps) {
  cudaError_t le = launch_pdl(decode_finish_kernel, dim3(1), dim3(128), 0, s, tok, history, pos_ids, step_ptr, len_ptr, batch, max_steps);
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
