// Row reductions: layer_norm, softmax / softmax_causal, argmax, sum/mean, sum_dim, mean_all.
//
// Reference semantics: kernel_templates.rs:1075-1116 (layer_norm: mean, population variance,
// 1/sqrt(var+eps)), :398-430 (softmax), :468-497 (softmax_causal: running max starts at -1e9,
// explicit zeros right of the diagonal, half types round exp() to storage before the divide),
// :500-520 (argmax: strict '>' scan from element 0, int32 result). The reference runs one
// thread per row over three serial passes; here a warp owns a row, keeps it in registers after
// a single 16-byte-vectorised read, reduces with shuffles, and writes once.
#include "common.cuh"
#include <cstdlib>

namespace ag { namespace k {

// ── layer_norm ──────────────────────────────────────────────────────────────
// Warp-per-row; ITERS packs per lane cover cols <= 32*ITERS*Pack::N. A persistent grid (a few CTAs per SM) walks the
// rows, and a warp keeps TWO rows in flight: the 16-byte loads of its next row are issued before the reductions of
// the current one, so loads, shuffles and stores of neighbouring rows overlap instead of every warp of the grid
// reading at the same time and then writing at the same time. Rows stay in registers as raw packs (converted
// where used), gamma / beta are fetched once per warp.
template <typename T, int ITERS>
__global__ void __launch_bounds__(256) layer_norm_warp_kernel(const T* __restrict__ in, const T* __restrict__ gamma, const T* __restrict__ beta,
                                                               T* __restrict__ out, int64_t rows, int cols, float eps) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int packs = cols / N;
  const float inv_cols = 1.0f / (float)cols;
  pdl_wait();
  pdl_trigger();
  constexpr bool kHoist = ITERS <= 4;
  Pack<T> gpk[kHoist ? ITERS : 1], bpk[kHoist ? ITERS : 1];
  if (kHoist) {
#pragma unroll
    for (int it = 0; it < (kHoist ? ITERS : 1); it++) {
      int pk = lane + it * 32;
      if (pk < packs) { gpk[it] = ld16(gamma + pk * N); bpk[it] = ld16(beta + pk * N); }
    }
  }
  const int64_t stride = (int64_t)gridDim.x * warps_per_block;
  int64_t row = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  Pack<T> cur[ITERS], nxt[ITERS];
  if (row < rows) {
#pragma unroll
    for (int it = 0; it < ITERS; it++) { int pk = lane + it * 32; if (pk < packs) cur[it] = ld16_stream(in + row * cols + pk * N); }
  }
  for (; row < rows; row += stride) {
    const int64_t next = row + stride;
    if (next < rows) {
#pragma unroll
      for (int it = 0; it < ITERS; it++) { int pk = lane + it * 32; if (pk < packs) nxt[it] = ld16_stream(in + next * cols + pk * N); }
    }
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      if (lane + it * 32 < packs) {
#pragma unroll
        for (int e = 0; e < N; e++) sum += Cvt<T>::to(cur[it].v[e]);
      }
    }
    const float mean = warp_sum(sum) * inv_cols;
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      if (lane + it * 32 < packs) {
#pragma unroll
        for (int e = 0; e < N; e++) { float d = Cvt<T>::to(cur[it].v[e]) - mean; sq += d * d; }
      }
    }
    const float var = warp_sum(sq) * inv_cols;
    const float inv_std = 1.0f / sqrtf(var + eps);
    T* y = out + row * cols;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      int pk = lane + it * 32;
      if (pk < packs) {
        Pack<T> g = kHoist ? gpk[kHoist ? it : 0] : ld16(gamma + pk * N);
        Pack<T> b = kHoist ? bpk[kHoist ? it : 0] : ld16(beta + pk * N);
        Pack<T> o;
        float r[N];
#pragma unroll
        for (int e = 0; e < N; e++) r[e] = Cvt<T>::to(g.v[e]) * (Cvt<T>::to(cur[it].v[e]) - mean) * inv_std + Cvt<T>::to(b.v[e]);
        pack_from_floats<T>(o, r);
        st16(y + pk * N, o);   // the next kernel (a GEMM) reads this from L2: no evict-first hint
      }
    }
#pragma unroll
    for (int it = 0; it < ITERS; it++) cur[it] = nxt[it];
  }
}

// Block-per-row, any cols / alignment: three passes over a row that stays in L1/L2.
template <typename T>
__global__ void __launch_bounds__(256) layer_norm_block_kernel(const T* __restrict__ in, const T* __restrict__ gamma, const T* __restrict__ beta,
                                                                T* __restrict__ out, int64_t rows, int64_t cols, float eps) {
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* x = in + row * cols;
    float s = 0.f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) s += Cvt<T>::to(x[j]);
    float mean = block_sum(s, red) / (float)cols;
    float q = 0.f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) { float d = Cvt<T>::to(x[j]) - mean; q += d * d; }
    float var = block_sum(q, red) / (float)cols;
    float inv_std = 1.0f / sqrtf(var + eps);
    T* y = out + row * cols;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
      y[j] = Cvt<T>::from(Cvt<T>::to(gamma[j]) * (Cvt<T>::to(x[j]) - mean) * inv_std + Cvt<T>::to(beta[j]));
  }
}

template <typename T>
static Status layer_norm_t(cudaStream_t s, const TView& in, const TView& gamma, const TView& beta, float eps, const TView& out) {
  constexpr int N = Pack<T>::N;
  int64_t cols = in.shape.back();
  int64_t rows = cols ? in.numel() / cols : 0;
  if (rows == 0 || cols == 0) return Status::OK();
  const T* x = (const T*)in.ptr; const T* g = (const T*)gamma.ptr; const T* b = (const T*)beta.ptr; T* y = (T*)out.ptr;
  bool vec = cols % N == 0 && aligned16(x) && aligned16(g) && aligned16(b) && aligned16(y);
  int64_t packs = cols / N;
  if (vec && packs <= 32 * 16) {
    // persistent: up to four CTAs of eight warps per SM, every warp walks rows with two in flight
    const int threads = 256, wpb = 8;
    // CTAs per SM (APPLEGPU_LN_BPS overrides): measured best on [8192, 768] at 2 for 16-bit rows and 4 for float32
    static const int bps_env = [] { const char* v = std::getenv("APPLEGPU_LN_BPS"); int n = v ? std::atoi(v) : 0; return n < 0 ? 0 : n > 8 ? 8 : n; }();
    const int bps = bps_env ? bps_env : (sizeof(T) == 4 ? 4 : 2);
    int grid = grid_for(rows, wpb, bps);
    int iters = (int)((packs + 31) / 32);
    cudaError_t le = cudaSuccess;
#define AG_LN(I) le = launch_pdl(layer_norm_warp_kernel<T, I>, dim3(grid), dim3(threads), 0, s, x, g, b, y, rows, (int)cols, eps)
    if (iters <= 1) AG_LN(1); else if (iters <= 2) AG_LN(2); else if (iters <= 3) AG_LN(3); else if (iters <= 4) AG_LN(4);
    else if (iters <= 6) AG_LN(6); else if (iters <= 8) AG_LN(8); else if (iters <= 12) AG_LN(12); else AG_LN(16);
#undef AG_LN
    if (le != cudaSuccess) return cuda_status(le, "layer_norm");
  } else {
    int grid = (int)(rows < (int64_t)sm_count() * 8 ? rows : (int64_t)sm_count() * 8);
    layer_norm_block_kernel<T><<<grid, 256, 0, s>>>(x, g, b, y, rows, cols, eps);
  }
  AG_CHECK_LAUNCH("layer_norm");
  return Status::OK();
}

Status layer_norm(cudaStream_t s, const TView& in, const TView& gamma, const TView& beta, float eps, const TView& out) {
  if (!in.contiguous() || !out.contiguous() || !gamma.contiguous() || !beta.contiguous())
    return Status::compute("layer_norm needs contiguous tensors");
  if (gamma.dtype != in.dtype || beta.dtype != in.dtype) return Status::invalid("layer_norm gamma/beta dtype must match input");
  AG_DISPATCH_FLOAT(in.dtype, T, return layer_norm_t<T>(s, in, gamma, beta, eps, out));
  return Status::OK();
}

// ── softmax / softmax_causal ────────────────────────────────────────────────
// Warp-per-row with the row in registers; `valid` = number of unmasked leading columns. A persistent grid walks the
// rows and a warp keeps two rows in flight: the 16-byte loads of its next row are issued before the reductions of the
// current one (a row's chain load -> max -> exp -> sum -> store is latency-bound on its own). Packs wholly left of the
// diagonal take a mask-free path, the one pack the diagonal crosses is masked per element, packs right of it are
// neither read nor computed: zeros are stored.
template <typename T, int ITERS, bool CAUSAL>
__global__ void __launch_bounds__(128, 4) softmax_warp_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t total_rows, int rows_per_mat, int cols) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int packs = cols / N;
  pdl_wait();
  pdl_trigger();
  auto valid_of = [&](int64_t row) -> int {
    if (!CAUSAL) return cols;
    // 32-bit remainder where the row count allows it: the 64-bit one costs about a fifth of a 1024-column row
    int r = total_rows <= 0x7fffffff ? (int)((unsigned int)row % (unsigned int)rows_per_mat) : (int)(row % rows_per_mat);
    return r + 1 < cols ? r + 1 : cols;
  };
  const int64_t stride = (int64_t)gridDim.x * wpb;
  int64_t row = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5);
  Pack<T> cur[ITERS], nxt[ITERS];
  int valid = 0;
  if (row < total_rows) {
    valid = valid_of(row);
#pragma unroll
    for (int it = 0; it < ITERS; it++) { int pk = lane + it * 32; if (pk < packs && pk * N < valid) cur[it] = ld16_stream(in + row * cols + pk * N); }
  }
  for (; row < total_rows; row += stride) {
    const int64_t next = row + stride;
    int next_valid = 0;
    if (next < total_rows) {
      next_valid = valid_of(next);
#pragma unroll
      for (int it = 0; it < ITERS; it++) { int pk = lane + it * 32; if (pk < packs && pk * N < next_valid) nxt[it] = ld16_stream(in + next * cols + pk * N); }
    }
    float v[ITERS][N];
    float m = CAUSAL ? -1e9f : -INFINITY;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      const int c0 = (lane + it * 32) * N;
      if (lane + it * 32 < packs && c0 < valid) {
        if (c0 + N <= valid) {
#pragma unroll
          for (int e = 0; e < N; e++) { v[it][e] = Cvt<T>::to(cur[it].v[e]); m = fmaxf(m, v[it][e]); }
        } else {
#pragma unroll
          for (int e = 0; e < N; e++) {
            const float f = Cvt<T>::to(cur[it].v[e]);
            const bool on = c0 + e < valid;
            v[it][e] = on ? f : -INFINITY;
            if (on) m = fmaxf(m, f);
          }
        }
      }
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      // packs entirely right of the diagonal (or past the row) hold only masked slots: skip their math
      if ((lane + it * 32) * N < valid && lane + it * 32 < packs) {
#pragma unroll
        for (int e = 0; e < N; e++) {
          // Masked slots hold -inf and contribute exp(-inf) = 0. __expf (hardware exp2) is within
          // 2 ulp plus the rounding of x*log2(e): well inside the 1e-5 bar.
          float ex = __expf(v[it][e] - m);
          sum += ex;
          // Half types: the reference stores exp() in the storage type and divides that value.
          v[it][e] = Cvt<T>::to(Cvt<T>::from(ex));
        }
      }
    }
    sum = warp_sum(sum);
    const float inv = __fdiv_rn(1.0f, sum);  // one division per row; e * (1/sum) is within 1 ulp of e / sum
    T* y = out + row * cols;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      int pk = lane + it * 32;
      int c0 = pk * N;
      if (pk < packs) {
        Pack<T> o;
        if (c0 < valid) {
          float r[N];
#pragma unroll
          for (int e = 0; e < N; e++) r[e] = v[it][e] * inv;     // masked slots hold exp(-inf) = 0: they store 0
          pack_from_floats<T>(o, r);
        } else {
#pragma unroll
          for (int e = 0; e < N; e++) o.v[e] = Cvt<T>::from(0.f);
        }
        st16_stream(y + c0, o);
      }
    }
#pragma unroll
    for (int it = 0; it < ITERS; it++) cur[it] = nxt[it];
    valid = next_valid;
  }
}

// Block-per-row for long or unaligned rows.
template <typename T, bool CAUSAL>
__global__ void __launch_bounds__(256) softmax_block_kernel(const T* in, T* out, int64_t total_rows, int64_t rows_per_mat, int64_t cols) {
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < total_rows; row += gridDim.x) {
    int64_t valid = cols;
    if (CAUSAL) { int64_t r = row % rows_per_mat; valid = r + 1 < cols ? r + 1 : cols; }
    const T* x = in + row * cols;
    float m = CAUSAL ? -1e9f : -INFINITY;
    for (int64_t j = threadIdx.x; j < valid; j += blockDim.x) m = fmaxf(m, Cvt<T>::to(x[j]));
    m = block_max(m, red);
    float sum = 0.f;
    for (int64_t j = threadIdx.x; j < valid; j += blockDim.x) sum += expf(Cvt<T>::to(x[j]) - m);
    sum = block_sum(sum, red);
    T* y = out + row * cols;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
      if (j < valid) {
        float e = Cvt<T>::to(Cvt<T>::from(expf(Cvt<T>::to(x[j]) - m)));
        y[j] = Cvt<T>::from(__fdiv_rn(e, sum));
      } else y[j] = Cvt<T>::from(0.f);
    }
  }
}

template <typename T, bool CAUSAL>
static Status softmax_t(cudaStream_t s, const TView& in, const TView& out) {
  constexpr int N = Pack<T>::N;
  int64_t cols = in.shape.back();
  if (cols == 0 || in.numel() == 0) return Status::OK();
  int64_t total_rows = in.numel() / cols;
  int64_t rows_per_mat = CAUSAL ? in.shape[in.nd() - 2] : 1;
  const T* x = (const T*)in.ptr; T* y = (T*)out.ptr;
  int64_t packs = cols / N;
  bool vec = cols % N == 0 && aligned16(x) && aligned16(y) && packs <= 32 * 16 && in.ptr != out.ptr;
  if (vec) {
    // persistent: four CTAs of four warps per SM (the kernel keeps two rows per warp in registers: ~128 registers)
    const int threads = 128, wpb = 4;
    int grid = grid_for(total_rows, wpb, 4);
    int iters = (int)((packs + 31) / 32);
    cudaError_t le = cudaSuccess;
#define AG_SM(I) le = launch_pdl(softmax_warp_kernel<T, I, CAUSAL>, dim3(grid), dim3(threads), 0, s, x, y, total_rows, (int)rows_per_mat, (int)cols)
    if (iters <= 1) AG_SM(1); else if (iters <= 2) AG_SM(2); else if (iters <= 4) AG_SM(4);
    else if (iters <= 8) AG_SM(8); else AG_SM(16);
#undef AG_SM
    if (le != cudaSuccess) return cuda_status(le, "softmax");
  } else {
    int grid = (int)(total_rows < (int64_t)sm_count() * 8 ? total_rows : (int64_t)sm_count() * 8);
    softmax_block_kernel<T, CAUSAL><<<grid, 256, 0, s>>>(x, y, total_rows, rows_per_mat, cols);
  }
  AG_CHECK_LAUNCH("softmax");
  return Status::OK();
}

Status softmax(cudaStream_t s, const TView& in, bool causal, const TView& out) {
  if (!in.contiguous() || !out.contiguous()) return Status::compute("softmax needs contiguous tensors");
  if (causal) { AG_DISPATCH_FLOAT(in.dtype, T, return (softmax_t<T, true>(s, in, out))); }
  else { AG_DISPATCH_FLOAT(in.dtype, T, return (softmax_t<T, false>(s, in, out))); }
  return Status::OK();
}

// ── argmax ──────────────────────────────────────────────────────────────────
// Serial-scan semantics: result = lowest index holding the maximum over non-NaN elements,
// except that a NaN in element 0 is never displaced (every '>' against NaN is false).
struct ArgPair { float v; int i; };
__device__ __forceinline__ ArgPair arg_better(ArgPair a, ArgPair b) {
  // a and b are both "valid" candidates (i >= 0); invalid carries i = INT_MAX and v = -inf.
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
template <typename T>
__global__ void __launch_bounds__(256) argmax_kernel(const T* __restrict__ in, int32_t* __restrict__ out, int64_t rows, int64_t cols, int64_t row_stride) {
  __shared__ float sv[32];
  __shared__ int si[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* x = in + row * row_stride;
    ArgPair best{-INFINITY, 0x7fffffff};
    // Each thread visits its elements in ascending index order, so a strict '>' keeps the first
    // maximum; NaNs never compare greater. Rows start on arbitrary element boundaries (a 50257-wide
    // row is only 2-byte aligned): scalar head up to the first 16-byte boundary, 16-byte packs, scalar tail.
    constexpr int N = Pack<T>::N;
    int64_t head = (int64_t)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(x) & 15u)) & 15u) / sizeof(T));
    if (head > cols) head = cols;
    for (int64_t j = threadIdx.x; j < head; j += blockDim.x) {
      float f = Cvt<T>::to(x[j]);
      if (f > best.v) best = ArgPair{f, (int)j};
    }
    const int64_t npacks = (cols - head) / N;
    const T* xv = x + head;
    int64_t pk = threadIdx.x;
    for (; pk + 3 * (int64_t)blockDim.x < npacks; pk += 4 * (int64_t)blockDim.x) {
      Pack<T> q[4];
#pragma unroll
      for (int u = 0; u < 4; u++) q[u] = ld16_stream(xv + (pk + u * (int64_t)blockDim.x) * N);
#pragma unroll
      for (int u = 0; u < 4; u++) {
#pragma unroll
        for (int e = 0; e < N; e++) {
          float f = Cvt<T>::to(q[u].v[e]);
          if (f > best.v) best = ArgPair{f, (int)(head + (pk + u * (int64_t)blockDim.x) * N + e)};
        }
      }
    }
    for (; pk < npacks; pk += blockDim.x) {
      Pack<T> q = ld16_stream(xv + pk * N);
#pragma unroll
      for (int e = 0; e < N; e++) {
        float f = Cvt<T>::to(q.v[e]);
        if (f > best.v) best = ArgPair{f, (int)(head + pk * N + e)};
      }
    }
    for (int64_t j = head + npacks * N + threadIdx.x; j < cols; j += blockDim.x) {
      float f = Cvt<T>::to(x[j]);
      if (f > best.v) best = ArgPair{f, (int)j};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = arg_better(best, other);
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[w] = best.v; si[w] = best.i; }
    __syncthreads();
    if (w == 0) {
      ArgPair b2 = lane < nw ? ArgPair{sv[lane], si[lane]} : ArgPair{-INFINITY, 0x7fffffff};
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ArgPair other{__shfl_xor_sync(0xffffffffu, b2.v, o), __shfl_xor_sync(0xffffffffu, b2.i, o)};
        b2 = arg_better(b2, other);
      }
      if (lane == 0) {
        float x0 = Cvt<T>::to(x[0]);
        int r = b2.i;
        if (x0 != x0 || r == 0x7fffffff) r = 0;  // NaN at 0 sticks; all-NaN row -> 0
        out[row] = r;
      }
    }
  }
}
// Integer rows (the reference allows every dtype but Bool): compare natively.
template <typename T>
__global__ void argmax_int_kernel(const T* __restrict__ in, int32_t* __restrict__ out, int64_t rows, int64_t cols) {
  int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const T* x = in + row * cols;
  T best = x[0]; int idx = 0;
  for (int64_t j = 1; j < cols; j++) if (x[j] > best) { best = x[j]; idx = (int)j; }
  out[row] = idx;
}

Status argmax(cudaStream_t s, const TView& in, const TView& out) {
  // rows dense, or all at one pitch (last stride 1, leading dims collapsing onto the row stride)
  int64_t cols = in.shape.back();
  if (cols == 0) return Status::compute("argmax over an empty row");
  int64_t rows = in.numel() / cols;
  int64_t row_stride = cols;
  if (!in.contiguous()) {
    if (in.shape.size() < 2 || in.strides.back() != 1) return Status::compute("argmax needs dense rows");
    row_stride = in.strides[in.shape.size() - 2];
    if (in.dtype != DType::F32 && in.dtype != DType::F16 && in.dtype != DType::BF16) return Status::compute("argmax needs a contiguous tensor");
  }
  if (rows == 0) return Status::OK();
  int grid = (int)(rows < (int64_t)sm_count() * 8 ? rows : (int64_t)sm_count() * 8);
  switch (in.dtype) {
    case DType::F32: argmax_kernel<float><<<grid, 256, 0, s>>>((const float*)in.ptr, (int32_t*)out.ptr, rows, cols, row_stride); break;
    case DType::F16: argmax_kernel<__half><<<grid, 256, 0, s>>>((const __half*)in.ptr, (int32_t*)out.ptr, rows, cols, row_stride); break;
    case DType::BF16: argmax_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in.ptr, (int32_t*)out.ptr, rows, cols, row_stride); break;
    case DType::I32: argmax_int_kernel<int32_t><<<(int)((rows + 127) / 128), 128, 0, s>>>((const int32_t*)in.ptr, (int32_t*)out.ptr, rows, cols); break;
    case DType::I64: argmax_int_kernel<int64_t><<<(int)((rows + 127) / 128), 128, 0, s>>>((const int64_t*)in.ptr, (int32_t*)out.ptr, rows, cols); break;
    case DType::U8: argmax_int_kernel<uint8_t><<<(int)((rows + 127) / 128), 128, 0, s>>>((const uint8_t*)in.ptr, (int32_t*)out.ptr, rows, cols); break;
    case DType::U32: argmax_int_kernel<uint32_t><<<(int)((rows + 127) / 128), 128, 0, s>>>((const uint32_t*)in.ptr, (int32_t*)out.ptr, rows, cols); break;
    case DType::I8: argmax_int_kernel<int8_t><<<(int)((rows + 127) / 128), 128, 0, s>>>((const int8_t*)in.ptr, (int32_t*)out.ptr, rows, cols); break;
    case DType::I16: argmax_int_kernel<int16_t><<<(int)((rows + 127) / 128), 128, 0, s>>>((const int16_t*)in.ptr, (int32_t*)out.ptr, rows, cols); break;
    default: return Status::unsupported("Argmax does not support bool dtype");
  }
  AG_CHECK_LAUNCH("argmax");
  return Status::OK();
}

// ── sums ────────────────────────────────────────────────────────────────────
// out[o, i] = sum_r in[o, r, i]   (outer, reduce, inner) — serves sum_dim and sum over last dim.
template <typename T>
__global__ void __launch_bounds__(256) sum_mid_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t outer, int64_t red, int64_t inner, float scale) {
  if (inner == 1) {
    __shared__ float sm[33];
    for (int64_t o = blockIdx.x; o < outer; o += gridDim.x) {
      float s = 0.f;
      for (int64_t r = threadIdx.x; r < red; r += blockDim.x) s += Cvt<T>::to(in[o * red + r]);
      s = block_sum(s, sm);
      if (threadIdx.x == 0) out[o] = Cvt<T>::from(s * scale);
    }
  } else {
    int64_t n = outer * inner;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
      int64_t o = i / inner, c = i % inner;
      float s = 0.f;
      for (int64_t r = 0; r < red; r++) s += Cvt<T>::to(in[(o * red + r) * inner + c]);
      out[i] = Cvt<T>::from(s * scale);
    }
  }
}
static Status sum_mid(cudaStream_t s, const TView& in, const TView& out, int64_t outer, int64_t red, int64_t inner, float scale) {
  if (!in.contiguous()) return Status::compute("sum needs a contiguous tensor");
  if (outer * inner == 0) return Status::OK();
  int grid = inner == 1 ? (int)(outer < (int64_t)sm_count() * 8 ? outer : (int64_t)sm_count() * 8) : grid_for(outer * inner, 256, 8);
  AG_DISPATCH_FLOAT(in.dtype, T, (sum_mid_kernel<T><<<grid, 256, 0, s>>>((const T*)in.ptr, (T*)out.ptr, outer, red, inner, scale)));
  AG_CHECK_LAUNCH("sum");
  return Status::OK();
}
Status sum_last(cudaStream_t s, const TView& in, const TView& out, bool mean) {
  int64_t cols = in.shape.empty() ? 1 : in.shape.back();
  int64_t rows = cols ? in.numel() / cols : 0;
  return sum_mid(s, in, out, rows, cols, 1, mean && cols ? 1.0f / (float)cols : 1.0f);
}
Status sum_dim(cudaStream_t s, const TView& in, int dim, const TView& out) {
  int64_t outer = 1, inner = 1;
  for (int d = 0; d < dim; d++) outer *= in.shape[d];
  for (int d = dim + 1; d < in.nd(); d++) inner *= in.shape[d];
  return sum_mid(s, in, out, outer, in.shape[dim], inner, 1.0f);
}
Status mean_all(cudaStream_t s, const TView& in, const TView& out) {
  int64_t n = in.numel();
  return sum_mid(s, in, out, 1, n, 1, n ? 1.0f / (float)n : 1.0f);
}

}}  // namespace ag::k
