// Batched matmul on the 5th-generation tensor cores: TMA -> shared-memory ring -> tcgen05.mma
// with fp32 accumulators in TMEM -> fused epilogue (alpha, per-channel scale, bias, activation,
// residual) -> global memory.
//
// Replaces the reference's 32x32 threadgroup-tile `matmul{s}` kernel (kernel_templates.rs:987-1072)
// and its MPSMatrixMultiplication call (swift/.../compute.swift:1584-1598) for f16/bf16 operands;
// the arithmetic contract is unchanged: C[b,i,j] = sum_k A[b,i,k] * B[b,k,j] with float
// accumulation and one rounding on store.
//
// One persistent CTA per SM walks output tiles of 128 x BN. Warp roles:
//   warp 0      TMA producer: fills a STAGES-deep ring of {A 128x64, B BNx64} tiles (128B swizzle)
//   warp 1      MMA issuer: one elected thread issues 4 x (128 x BN x 16) tcgen05.mma per stage,
//               commits the stage back to the producer, and owns the TMEM allocation
//   warps 2..9  epilogue: tcgen05.ld of the finished accumulator (two TMEM buffers, so the next
//               tile's main loop overlaps this tile's epilogue), epilogue math, stores
// B is taken either K-major ([N,K] rows, e.g. a tied embedding or K in Q.K^T) or N-major
// ([K,N] rows, the layout of every GPT-2 Conv1D weight and of V in P.V) through the
// descriptor's major bit, so no operand is ever transposed in memory.
#include "common.cuh"
#include "sm100.cuh"
#include <cuda.h>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace ag { namespace k {

using namespace ag::sm100;

constexpr int BM = 128;          // UMMA M (cta_group::1)
constexpr int BK = 64;           // 64 x 2 B = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kTcThreads = 64 + 8 * 32;   // TMA warp, MMA warp, eight epilogue warps

struct TcParams {
  void* c;
  const void* bias;
  const void* residual;
  const float* b_scales;
  float alpha;
  int act;
  int m, n, k, batch;          // batch = outer * inner
  int batch_inner;
  long long c_row, c_batch, c_batch_inner;
  int a_bcast, b_bcast;        // bit 0: outer index pinned to 0, bit 1: inner index pinned to 0
  int tiles_m, tiles_n;
  int vec_ok;                  // C (and residual) rows are 16-byte aligned: 16-byte global accesses
  int bias_vec;                // bias pointer is 16-byte aligned
  unsigned long long* argmax_keys;   // non-null: merge per-row (value, column) keys instead of storing C
  int c_f32;                         // C, bias and residual are float32 (operands are still 16-bit)
  const long long* ln_stats;         // folded layer_norm, consumer side: fixed-point (sum, sum of squares) per A row; the float slots hold ln_colsum
  const float* ln_colsum;
  float ln_inv_k, ln_eps;
  long long* stats_out;              // folded layer_norm, producer side: row sums of what is stored (fixed point, integer atomics)
  long long* stats_zero;             // rows of the other statistics tensor to clear
  int* status;
#ifdef AG_GEMM_PROBE
  long long* probe;   // per CTA: [0] cycles the MMA thread waited for a free accumulator, [1] cycles in the k loops, [2] k steps, [3] cycles epilogue warp 2 waited for a full accumulator, [4] cycles it spent in the epilogue, [5] tiles, [6] kernel cycles
#endif
};

constexpr int kEpiWarps = 8;                       // two warps per TMEM lane quarter, alternating column groups
constexpr int kStgBytesPerWarp = 32 * 64;           // a dense 32 x 32 tile of 2-byte elements, 64-byte swizzle
constexpr int kStgBytes = kEpiWarps * kStgBytesPerWarp;
// Byte offset of 16-byte chunk `chunk` (0..3) of row `row` inside a warp's staging tile. The tile is dense (64-byte
// rows) in the 64-byte swizzle of the TMA unit: the chunk index is XOR-ed with bits 7..8 of the address, i.e. with
// (row / 2) % 4, so a tiled bulk store can read it as it lies. Row-per-lane accesses (8 lanes per 128-bit phase: rows
// r..r+7 at one chunk) and 4-lanes-per-row accesses (2 rows x 4 chunks per phase) both touch 8 distinct bank groups.
__device__ __forceinline__ int stg_off(int row, int chunk) { return row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4); }
// Per tile an epilogue warp needs the bias values (2-byte) and, for int8 weights, the per-channel
// fp32 scales of its own column groups: half of the tile's columns.
constexpr int epi_slots(int bn) { return bn / 2; }
constexpr int bias_bytes(int bn) { return kEpiWarps * epi_slots(bn) * 2; }
constexpr int scale_bytes(int bn) { return kEpiWarps * epi_slots(bn) * 4; }

template <int BN> struct TcCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 192) ? 5 : 6;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStgBytes + bias_bytes(BN) + scale_bytes(BN) + 1024;  // ring + epilogue staging + bias / scale slices + alignment slack
  static_assert(kSmemBytes + 512 <= 232448, "dynamic + static shared memory must fit the 227 KB a CTA may use");
  static constexpr int kAccStride = (BN == 192) ? 256 : BN;        // column offset of the second accumulator
  static constexpr int kTmemCols = 2 * kAccStride;                 // two accumulator buffers (a power of two)
};

// Epilogue staging: each epilogue warp owns a [32 rows x 32 cols] 2-byte tile in shared memory (stg_off above).
// Results leave it through one tiled bulk store per 32 x 32 group (cp.async.bulk.tensor, issued by one lane and
// drained by the TMA unit while the warp computes the next group) when C's rows are 16-byte aligned; otherwise,
// and for float32 or argmax outputs, through plain global stores.

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 256-bit global accesses (sm_100): one lane moves 32 contiguous bytes, a whole L2 sector. With one output row per
// lane (the layout tcgen05.ld delivers) a lane's 32 columns of 16-bit results are two such stores, every sector is
// written in full, and nothing has to be transposed through shared memory first.
__device__ __forceinline__ void st_global_256(void* ptr, const uint32_t* r) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(ptr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void ld_global_256(const void* ptr, uint32_t* r) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "l"(ptr));
}

// This lane's residual row of one 32-column group (64 bytes) into registers; issued one group ahead of its use so
// that the load latency overlaps the previous group's math. Direct (32-byte aligned) layout only.
template <typename T>
__device__ __forceinline__ void load_residual_row(const TcParams& p, const T* R, long long gm, int col0, uint32_t (&rpre)[16]) {
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const int gc = col0 + 16 * j;
    if (gm < p.m && gc + 16 <= p.n) ld_global_256(R + gm * p.c_row + gc, &rpre[8 * j]);
    else {
      alignas(16) T tmp[16];
#pragma unroll
      for (int e = 0; e < 16; e++) tmp[e] = (gm < p.m && gc + e < p.n) ? R[gm * p.c_row + gc + e] : Cvt<T>::from(0.f);
#pragma unroll
      for (int w = 0; w < 8; w++) rpre[8 * j + w] = reinterpret_cast<const uint32_t*>(tmp)[w];
    }
  }
}

// One 32-column group of one warp's 32 rows: TMEM -> registers -> epilogue math -> global memory.
// Every epilogue option is tested once per group (uniform branches around 32-element loops).
//   p.vec_ok == 2  rows of C (and of the residual) are 32-byte aligned: each lane stores its own row's 64 bytes with
//                  two 256-bit stores and reads its residual row the same way; no shared memory on the path
//   p.vec_ok == 1  rows are 16-byte aligned: results are transposed through the warp's staging tile and stored with
//                  4 lanes per row (64 contiguous bytes per row per instruction)
//   p.vec_ok == 0  unaligned rows (a dense 50257-wide LM head): staged, 32 consecutive elements per instruction
// Two 16-bit floats in one register, for the epilogue paths that work on rounded values pairwise.
template <typename T> struct Packed2;
template <> struct Packed2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ type from_floats(float lo, float hi) { return __floats2bfloat162_rn(lo, hi); }
  static __device__ __forceinline__ float low_to_float(type v) { return __low2float(v); }
};
template <> struct Packed2<__half> {
  using type = __half2;
  static __device__ __forceinline__ type from_floats(float lo, float hi) { return __floats2half2_rn(lo, hi); }
  static __device__ __forceinline__ float low_to_float(type v) { return __low2float(v); }
};

// Packed fp32 pipe: two independent operations per instruction on a 64-bit register pair.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Two packed 16-bit floats (one 32-bit word, element 0 in the low half) -> two floats in a 64-bit pair, exactly.
template <typename T> __device__ __forceinline__ uint64_t widen2(uint32_t w);
template <> __device__ __forceinline__ uint64_t widen2<__nv_bfloat16>(uint32_t w) {
  return pack_f32x2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));   // bf16 is the upper half of a float
}
template <> __device__ __forceinline__ uint64_t widen2<__half>(uint32_t w) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  return pack_f32x2(f.x, f.y);
}

constexpr float kStatsScale = 268435456.0f;          // 2^28: row statistics travel as fixed-point int64 (see emit_row_stats)
constexpr float kStatsUnscale = 1.0f / 268435456.0f;

// Folded layer_norm, consumer side: mean and 1/std of A row `gm` from the (sum, sum of squares) its producer left.
__device__ __forceinline__ longlong2 ln_stats_fetch(const TcParams& p, long long gm) {
  if (!p.ln_stats || gm < 0 || gm >= p.m) return make_longlong2(0, 0);
  return __ldg(reinterpret_cast<const longlong2*>(p.ln_stats) + gm);
}
__device__ __forceinline__ void ln_stats_finish(const TcParams& p, const longlong2 raw, float& mean, float& rstd) {
  if (!p.ln_stats) return;
  const float2 st = make_float2(__ll2float_rn(raw.x) * kStatsUnscale, __ll2float_rn(raw.y) * kStatsUnscale);
  const float mu = st.x * p.ln_inv_k;
  const float var = fmaxf(fmaf(-mu, mu, st.y * p.ln_inv_k), 0.f);
  rstd = 1.0f / sqrtf(var + p.ln_eps);
  mean = -mu * rstd;     // handed on as the shift factor: result = acc * rstd + colsum * (-mean * rstd)
}
__device__ __forceinline__ void ln_row_stats(const TcParams& p, long long gm, float& mean, float& rstd) {
  if (!p.ln_stats || gm >= p.m) return;
  ln_stats_finish(p, ln_stats_fetch(p, gm), mean, rstd);
}
// Folded layer_norm, producer side. A row's (sum, sum of squares) is accumulated from the partial sums of the CTAs
// that store pieces of it. The partials are converted to 2^-28 fixed point and added with 64-bit integer atomics:
// integer addition is associative, so the statistics (and everything computed from them) do not depend on the order in
// which CTAs finish. Range: |sum|, sum of squares < 2^35 per row; resolution 4e-9.
__device__ __forceinline__ void group_stats(const TcParams& p, const float (&v)[32], int col0, float& row_sum, float& row_sq) {
  float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
  if (col0 + 32 <= p.n) {   // uniform: the whole group lies inside the matrix
#pragma unroll
    for (int e = 0; e < 32; e += 2) { s0 += v[e]; s1 += v[e + 1]; q0 = fmaf(v[e], v[e], q0); q1 = fmaf(v[e + 1], v[e + 1], q1); }
  } else {
#pragma unroll
    for (int e = 0; e < 32; e++) {
      if (col0 + e < p.n) { s0 += v[e]; q0 = fmaf(v[e], v[e], q0); }
    }
  }
  row_sum += s0 + s1; row_sq += q0 + q1;
}
// This thread's share of row `gm` (its column groups of one tile) goes into the row's running sums; the rows of the
// other statistics tensor are cleared by the tile that holds column 0.
__device__ __forceinline__ void emit_row_stats(const TcParams& p, long long gm, bool clears, float row_sum, float row_sq) {
  if (gm >= p.m) return;
  if (p.stats_out) {
    atomicAdd(reinterpret_cast<unsigned long long*>(p.stats_out) + 2 * gm, (unsigned long long)__float2ll_rn(row_sum * kStatsScale));
    atomicAdd(reinterpret_cast<unsigned long long*>(p.stats_out) + 2 * gm + 1, (unsigned long long)__float2ll_rn(row_sq * kStatsScale));
  }
  if (p.stats_zero && clears) *reinterpret_cast<longlong2*>(p.stats_zero + 2 * gm) = make_longlong2(0, 0);
}

#ifdef AG_CHAIN_PROBE
__device__ long long g_epi_probe[8];   // [0] tmem load + wait, [1] math, [2] stores, [3] groups, [4] residual prologue (CTA 0, warp 2, lane 0)
#define AG_EPI_T(var) long long var = clock64()
#define AG_EPI_ADD(slot, a, b) do { if (blockIdx.x == 0 && (threadIdx.x >> 5) == 2 && lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(&g_epi_probe[slot]), (unsigned long long)((b) - (a))); } while (0)
#else
#define AG_EPI_T(var)
#define AG_EPI_ADD(slot, a, b)
#endif
template <typename T>
__device__ __forceinline__ void epilogue_group(const TcParams& p, uint32_t taddr, uint8_t* stg, const T* bias_s, const float* scale_s, uint32_t (&rpre)[16],
                                               long long row0, int col0, int next_col0, long long c_off, int lane, unsigned long long& best_key,
                                               float ln_mean, float ln_rstd, float& row_sum, float& row_sq, const float* bias_f = nullptr) {
  T* C = reinterpret_cast<T*>(p.c) + c_off;
  const T* R = p.residual ? reinterpret_cast<const T*>(p.residual) + c_off : nullptr;
  const int sub_row = lane >> 2, sub_chunk = lane & 3;
  const bool direct = p.vec_ok == 2;

  // 1. residual. Direct layout: this group's row was fetched one group ahead; the next group's fetch is issued here
  //    and lands while this group is computed. Staged layouts: the tile goes to shared memory (coalesced reads).
  uint32_t rcur[16];
  if (R && !p.c_f32) {
    if (direct) {
#pragma unroll
      for (int w = 0; w < 16; w++) rcur[w] = rpre[w];
      if (next_col0 >= 0) load_residual_row<T>(p, R, row0 + lane, next_col0, rpre);
    } else {
      if (p.vec_ok) {
#pragma unroll
        for (int it = 0; it < 4; it++) {
          long long gm = row0 + it * 8 + sub_row;
          int gc = col0 + sub_chunk * 8;
          uint4 v4 = make_uint4(0, 0, 0, 0);
          if (gm < p.m && gc + 8 <= p.n) v4 = *reinterpret_cast<const uint4*>(R + gm * p.c_row + gc);
          else if (gm < p.m && gc < p.n) {
            alignas(16) T tmp[8];
#pragma unroll
            for (int e = 0; e < 8; e++) tmp[e] = gc + e < p.n ? R[gm * p.c_row + gc + e] : Cvt<T>::from(0.f);
            v4 = *reinterpret_cast<uint4*>(tmp);
          }
          *reinterpret_cast<uint4*>(stg + stg_off(it * 8 + sub_row, sub_chunk)) = v4;
        }
      } else {
        for (int r = 0; r < 32; r++) {
          long long gm = row0 + r;
          T v = (gm < p.m && col0 + lane < p.n) ? R[gm * p.c_row + col0 + lane] : Cvt<T>::from(0.f);
          *reinterpret_cast<T*>(stg + stg_off(r, lane >> 3) + (lane & 7) * 2) = v;
        }
      }
      __syncwarp();
    }
  }

  // 2. accumulators -> registers
  uint32_t acc[32];
  AG_EPI_T(t_a);
  tmem_ld_32x32(taddr, acc);
  tmem_ld_wait();
  AG_EPI_T(t_b);
  AG_EPI_ADD(0, t_a, t_b);
  float v[32];
#pragma unroll
  for (int e = 0; e < 32; e++) v[e] = __uint_as_float(acc[e]);

  if (p.c_f32) {
    // float32 output (split-precision fp32 product): bias (staged as floats where the int8 scales
    // would be) and residual are float32; each lane stores its own row's 32 columns, 128 contiguous bytes.
    float* Cf = reinterpret_cast<float*>(p.c) + c_off;
    const float* Rf = p.residual ? reinterpret_cast<const float*>(p.residual) + c_off : nullptr;
    if (p.alpha != 1.0f) {
#pragma unroll
      for (int e = 0; e < 32; e++) v[e] *= p.alpha;
    }
    if (scale_s) {
#pragma unroll
      for (int g = 0; g < 8; g++) {
        float4 b4 = *reinterpret_cast<const float4*>(scale_s + g * 4);
        v[g * 4 + 0] += b4.x; v[g * 4 + 1] += b4.y; v[g * 4 + 2] += b4.z; v[g * 4 + 3] += b4.w;
      }
    }
    switch ((Act)p.act) {
      case Act::GeluTanh:
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = gelu_tanh_f(v[e]);
        break;
      case Act::GeluErf:
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = gelu_erf_f(v[e]);
        break;
      case Act::Relu:
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = fmaxf(v[e], 0.f);
        break;
      default: break;
    }
    const long long gm = row0 + lane;
    if (gm < p.m) {
      float* crow = Cf + gm * p.c_row + col0;
      const float* rrow = Rf ? Rf + gm * p.c_row + col0 : nullptr;
      if (p.vec_ok && col0 + 32 <= p.n) {
#pragma unroll
        for (int g = 0; g < 8; g++) {
          float4 o = make_float4(v[g * 4 + 0], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          if (rrow) { float4 r4 = *reinterpret_cast<const float4*>(rrow + g * 4); o.x += r4.x; o.y += r4.y; o.z += r4.z; o.w += r4.w; }
          *reinterpret_cast<float4*>(crow + g * 4) = o;
        }
      } else {
        for (int e = 0; e < 32 && col0 + e < p.n; e++) crow[e] = v[e] + (rrow ? rrow[e] : 0.f);
      }
    }
    return;
  }

  // 3a. The common case (16-bit C with 32-byte aligned rows, results stored): the whole chain on the packed fp32 pipe,
  //     two columns per instruction. The epilogue warps share their schedulers' issue slots with the next tile's main
  //     loop bookkeeping and with each other, and the K = 768 products of a transformer block are bound by exactly
  //     these instructions, so every one that goes counts. Same operations in the same order as the scalar code below
  //     (fma.rn / add.rn / mul.rn on each half), except that the bias rides in the folded layer_norm's FMA and the
  //     tanh-GELU polynomial is factored as x * (c0 + c1 * x^2).
  if (direct && !p.argmax_keys && bias_f) {
    uint64_t vp[16];
#pragma unroll
    for (int w = 0; w < 16; w++) vp[w] = pack_f32x2(v[2 * w], v[2 * w + 1]);
    if (p.alpha != 1.0f) {
      const uint64_t a2 = pack_f32x2(p.alpha, p.alpha);
#pragma unroll
      for (int w = 0; w < 16; w++) vp[w] = mul_f32x2(vp[w], a2);
    }
    if (p.ln_stats) {
      // acc * rstd + (colsum * shift + bias)
      const uint64_t r2 = pack_f32x2(ln_rstd, ln_rstd), sh2 = pack_f32x2(ln_mean, ln_mean);
#pragma unroll
      for (int g = 0; g < 8; g++) {
        const ulonglong2 cs = *reinterpret_cast<const ulonglong2*>(scale_s + g * 4);   // same address in every lane: a broadcast
        const ulonglong2 bb = *reinterpret_cast<const ulonglong2*>(bias_f + g * 4);
        vp[2 * g] = fma_f32x2(vp[2 * g], r2, fma_f32x2(cs.x, sh2, bb.x));
        vp[2 * g + 1] = fma_f32x2(vp[2 * g + 1], r2, fma_f32x2(cs.y, sh2, bb.y));
      }
    } else {
#pragma unroll
      for (int g = 0; g < 8; g++) {
        const ulonglong2 bb = *reinterpret_cast<const ulonglong2*>(bias_f + g * 4);
        if (scale_s) {
          const ulonglong2 sc = *reinterpret_cast<const ulonglong2*>(scale_s + g * 4);
          vp[2 * g] = fma_f32x2(vp[2 * g], sc.x, bb.x);
          vp[2 * g + 1] = fma_f32x2(vp[2 * g + 1], sc.y, bb.y);
        } else {
          vp[2 * g] = add_f32x2(vp[2 * g], bb.x);
          vp[2 * g + 1] = add_f32x2(vp[2 * g + 1], bb.y);
        }
      }
    }
    if ((Act)p.act == Act::GeluTanh && std::is_same<T, __nv_bfloat16>::value) {
      // 0.5 x (1 + tanh(x (c0 + c1 x^2))) with the hardware tanh (relative error about 2^-11, a quarter of a bf16 step)
      const uint64_t c0 = pack_f32x2(0.7978845608f, 0.7978845608f), c1 = pack_f32x2(0.0356774081f, 0.0356774081f), half2v = pack_f32x2(0.5f, 0.5f);
#pragma unroll
      for (int w = 0; w < 16; w++) {
        const uint64_t x = vp[w];
        const uint64_t u = mul_f32x2(x, fma_f32x2(mul_f32x2(x, x), c1, c0));
        float u0, u1, t0, t1;
        unpack_f32x2(u, u0, u1);
        asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(u0));
        asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(u1));
        const uint64_t hx = mul_f32x2(x, half2v);
        vp[w] = fma_f32x2(hx, pack_f32x2(t0, t1), hx);
      }
    } else if ((Act)p.act == Act::GeluErf && std::is_same<T, __nv_bfloat16>::value) {
      // the erf form for bf16 results (common.cuh gelu_erf_bf16_f: an odd polynomial fitted to erf inside one tanh),
      // clamped per element, the rest two at a time
      const uint64_t c1 = pack_f32x2(7.97458471e-1f, 7.97458471e-1f), c3 = pack_f32x2(3.70503451e-2f, 3.70503451e-2f),
                     c5 = pack_f32x2(-3.58732362e-4f, -3.58732362e-4f), half2v = pack_f32x2(0.5f, 0.5f);
#pragma unroll
      for (int w = 0; w < 16; w++) {
        const uint64_t x = vp[w];
        float a, b;
        unpack_f32x2(x, a, b);
        const uint64_t xc = pack_f32x2(fminf(fmaxf(a, -8.0f), 8.0f), fminf(fmaxf(b, -8.0f), 8.0f));
        const uint64_t x2 = mul_f32x2(xc, xc);
        const uint64_t u = mul_f32x2(xc, fma_f32x2(fma_f32x2(c5, x2, c3), x2, c1));
        float u0, u1, t0, t1;
        unpack_f32x2(u, u0, u1);
        asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(u0));
        asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(u1));
        const uint64_t hx = mul_f32x2(x, half2v);
        vp[w] = fma_f32x2(hx, pack_f32x2(t0, t1), hx);
      }
    } else if ((Act)p.act != Act::None) {
      // the other activations element by element: one uniform test, then a straight loop (as in the scalar path)
#pragma unroll
      for (int w = 0; w < 16; w++) unpack_f32x2(vp[w], v[2 * w], v[2 * w + 1]);
      switch ((Act)p.act) {
        case Act::GeluTanh:
#pragma unroll
          for (int e = 0; e < 32; e++) v[e] = gelu_tanh_f(v[e]);
          break;
        case Act::GeluErf:
          if (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
            for (int e = 0; e < 32; e++) v[e] = gelu_erf_bf16_f(v[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 32; e++) v[e] = gelu_erf_fast_f(v[e]);
          }
          break;
        case Act::Relu:
#pragma unroll
          for (int e = 0; e < 32; e++) v[e] = fmaxf(v[e], 0.f);
          break;
        default: break;
      }
#pragma unroll
      for (int w = 0; w < 16; w++) vp[w] = pack_f32x2(v[2 * w], v[2 * w + 1]);
    }
    if (R) {
#pragma unroll
      for (int w = 0; w < 16; w++) vp[w] = add_f32x2(vp[w], widen2<T>(rcur[w]));
    }
    if (p.stats_out) {
      if (col0 + 32 <= p.n) {
        uint64_t s2 = 0, q2 = 0;    // the bit pattern of (0.f, 0.f)
#pragma unroll
        for (int w = 0; w < 16; w++) { s2 = add_f32x2(s2, vp[w]); q2 = fma_f32x2(vp[w], vp[w], q2); }
        float s0, s1, q0, q1;
        unpack_f32x2(s2, s0, s1); unpack_f32x2(q2, q0, q1);
        row_sum += s0 + s1; row_sq += q0 + q1;
      } else {
#pragma unroll
        for (int w = 0; w < 16; w++) unpack_f32x2(vp[w], v[2 * w], v[2 * w + 1]);
        group_stats(p, v, col0, row_sum, row_sq);
      }
    }
    uint32_t o[16];
#pragma unroll
    for (int w = 0; w < 16; w++) {
      float a, b;
      unpack_f32x2(vp[w], a, b);
      o[w] = pack2<T>(a, b);
    }
    const long long gm = row0 + lane;
    AG_EPI_T(t_c2);
    AG_EPI_ADD(1, t_b, t_c2);
    if (gm < p.m) {
      T* crow = C + gm * p.c_row + col0;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        if (col0 + 16 * j + 16 <= p.n) st_global_256(crow + 16 * j, &o[8 * j]);
        else {
          const T* tv = reinterpret_cast<const T*>(&o[8 * j]);
          for (int e = 0; e < 16 && col0 + 16 * j + e < p.n; e++) crow[16 * j + e] = tv[e];
        }
      }
    }
    AG_EPI_T(t_d2);
    AG_EPI_ADD(2, t_c2, t_d2);
    AG_EPI_ADD(3, 0, 1);
    return;
  }

  // 3. epilogue math: one uniform test per option, then a straight 32-element loop
  if (p.alpha != 1.0f) {
#pragma unroll
    for (int e = 0; e < 32; e++) v[e] *= p.alpha;
  }
  if (p.ln_stats) {
    // folded layer_norm: the product ran on the raw rows; this row's mean times the weight's column sums comes off,
    // then its 1/std scales the rest (the float slots hold the column sums)
    // two elements per instruction on the packed fp32 pipe: acc * rstd + colsum * shift
    const uint64_t r2 = pack_f32x2(ln_rstd, ln_rstd), sh2 = pack_f32x2(ln_mean, ln_mean);
#pragma unroll
    for (int g = 0; g < 8; g++) {
      const ulonglong2 cs = *reinterpret_cast<const ulonglong2*>(scale_s + g * 4);   // same address in every lane: a broadcast
      unpack_f32x2(fma_f32x2(pack_f32x2(v[g * 4 + 0], v[g * 4 + 1]), r2, mul_f32x2(cs.x, sh2)), v[g * 4 + 0], v[g * 4 + 1]);
      unpack_f32x2(fma_f32x2(pack_f32x2(v[g * 4 + 2], v[g * 4 + 3]), r2, mul_f32x2(cs.y, sh2)), v[g * 4 + 2], v[g * 4 + 3]);
    }
  } else if (scale_s) {
#pragma unroll
    for (int g = 0; g < 8; g++) {
      float4 sc = *reinterpret_cast<const float4*>(scale_s + g * 4);   // same address in every lane: a broadcast
      v[g * 4 + 0] *= sc.x; v[g * 4 + 1] *= sc.y; v[g * 4 + 2] *= sc.z; v[g * 4 + 3] *= sc.w;
    }
  }
  if (bias_s) {
    // this group's 32 bias values were staged in shared memory before the accumulator wait:
    // every lane reads the same 16 bytes (a broadcast)
#pragma unroll
    for (int g = 0; g < 4; g++) {
      Pack<T> b = *reinterpret_cast<const Pack<T>*>(bias_s + g * 8);
#pragma unroll
      for (int e = 0; e < 8; e++) v[g * 8 + e] += Cvt<T>::to(b.v[e]);
    }
  }
  switch ((Act)p.act) {
    case Act::GeluTanh:
      if (std::is_same<T, __nv_bfloat16>::value) {
        // bf16 results: the hardware tanh (relative error about 2^-11) stays four times below the
        // rounding step of the stored value and needs one MUFU operation instead of two (exp and
        // reciprocal), which matters because this loop runs beside the next tile's main loop.
#pragma unroll
        for (int e = 0; e < 32; e++) {
          float x = v[e];
          float u = 0.7978845608f * fmaf(0.044715f * x, x * x, x);
          float t;
          asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
          float hx = 0.5f * x;
          v[e] = fmaf(hx, t, hx);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = gelu_tanh_f(v[e]);
      }
      break;
    case Act::GeluErf:
      if (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = gelu_erf_bf16_f(v[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = gelu_erf_fast_f(v[e]);
      }
      break;
    case Act::Relu:
#pragma unroll
      for (int e = 0; e < 32; e++) v[e] = fmaxf(v[e], 0.f);
      break;
    default: break;
  }
  if (p.argmax_keys) {
    // Row argmax over this group's columns of the value as it would have been stored (rounded to T).
    // Key = order-preserving bits of the value in the high word, inverted column in the low word: the
    // larger key is the larger value, or the lower column among equals. NaNs are never selected,
    // except in column 0, which then keeps the row (the serial scan's behaviour).
    if (col0 > 0 && col0 + 32 <= p.n) {
      // Whole group inside the matrix and away from column 0: work on the rounded values two at a time. Packed
      // converts, a tree of packed maxima (a NaN operand loses to a number, as in the scan), then the lowest column
      // whose rounded value equals the maximum (compared as numbers: +0 and -0 tie, as in the scan): ~90
      // instructions for 32 columns instead of ~350.
      using T2 = typename Packed2<T>::type;
      T2 pk[16];
#pragma unroll
      for (int w = 0; w < 16; w++) pk[w] = Packed2<T>::from_floats(v[2 * w], v[2 * w + 1]);
      T2 mx[8];
#pragma unroll
      for (int w = 0; w < 8; w++) mx[w] = __hmax2(pk[w], pk[w + 8]);
#pragma unroll
      for (int w = 0; w < 4; w++) mx[w] = __hmax2(mx[w], mx[w + 4]);
      mx[0] = __hmax2(__hmax2(mx[0], mx[2]), __hmax2(mx[1], mx[3]));
      const T2 top = __hmax2(mx[0], __lowhigh2highlow(mx[0]));     // both halves: the group's maximum
      int first = -1;
#pragma unroll
      for (int w = 15; w >= 0; w--) {
        const unsigned eq = __heq2_mask(pk[w], top);                // 0xFFFF per half that equals the maximum
        if (eq & 0xffff0000u) first = 2 * w + 1;
        if (eq & 0x0000ffffu) first = 2 * w;
      }
      if (first >= 0) {                                             // an all-NaN group has no candidate
        const float r = Packed2<T>::low_to_float(top);
        const uint32_t b = __float_as_uint(r);
        const uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
        const unsigned long long key = ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - (uint32_t)(col0 + first));
        if (key > best_key) best_key = key;
      }
      return;
    }
#pragma unroll
    for (int e = 0; e < 32; e++) {
      int col = col0 + e;
      float r = Cvt<T>::to(Cvt<T>::from(v[e]));
      uint32_t b = __float_as_uint(r);
      uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
      unsigned long long key = ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - (uint32_t)col);
      if (r != r) key = (col == 0) ? 0xffffffffffffffffull : 0ull;
      if (col < p.n && key > best_key) best_key = key;
    }
    return;
  }

  if (direct) {
    // 4a. residual from registers, then two 256-bit stores of this lane's own row
    if (R) {
#pragma unroll
      for (int w = 0; w < 16; w++) {
        const T* rv = reinterpret_cast<const T*>(&rcur[w]);
        v[2 * w] += Cvt<T>::to(rv[0]); v[2 * w + 1] += Cvt<T>::to(rv[1]);
      }
    }
    if (p.stats_out) group_stats(p, v, col0, row_sum, row_sq);
    uint32_t o[16];
#pragma unroll
    for (int w = 0; w < 16; w++) o[w] = pack2<T>(v[2 * w], v[2 * w + 1]);
    const long long gm = row0 + lane;
    AG_EPI_T(t_c);
    AG_EPI_ADD(1, t_b, t_c);
    if (gm < p.m) {
      T* crow = C + gm * p.c_row + col0;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        if (col0 + 16 * j + 16 <= p.n) st_global_256(crow + 16 * j, &o[8 * j]);
        else {
          const T* tv = reinterpret_cast<const T*>(&o[8 * j]);
          for (int e = 0; e < 16 && col0 + 16 * j + e < p.n; e++) crow[16 * j + e] = tv[e];
        }
      }
    }
    AG_EPI_T(t_d);
    AG_EPI_ADD(2, t_c, t_d);
    AG_EPI_ADD(3, 0, 1);
    return;
  }

  // 4b. staged layouts: residual from the staging tile, results back into it, then coalesced stores
  if (R) {
#pragma unroll
    for (int g = 0; g < 4; g++) {
      Pack<T> r = *reinterpret_cast<const Pack<T>*>(stg + stg_off(lane, g));
#pragma unroll
      for (int e = 0; e < 8; e++) v[g * 8 + e] += Cvt<T>::to(r.v[e]);
    }
  }
  if (p.stats_out) group_stats(p, v, col0, row_sum, row_sq);
#pragma unroll
  for (int g = 0; g < 4; g++) {
    uint4 o;
    o.x = pack2<T>(v[g * 8 + 0], v[g * 8 + 1]); o.y = pack2<T>(v[g * 8 + 2], v[g * 8 + 3]);
    o.z = pack2<T>(v[g * 8 + 4], v[g * 8 + 5]); o.w = pack2<T>(v[g * 8 + 6], v[g * 8 + 7]);
    *reinterpret_cast<uint4*>(stg + stg_off(lane, g)) = o;
  }
  __syncwarp();
  if (p.vec_ok) {
#pragma unroll
    for (int it = 0; it < 4; it++) {
      int r = it * 8 + sub_row;
      long long gm = row0 + r;
      int gc = col0 + sub_chunk * 8;
      if (gm < p.m && gc < p.n) {
        uint4 o = *reinterpret_cast<const uint4*>(stg + stg_off(r, sub_chunk));
        if (gc + 8 <= p.n) *reinterpret_cast<uint4*>(C + gm * p.c_row + gc) = o;
        else {
          const T* tv = reinterpret_cast<const T*>(&o);
          for (int e = 0; e < 8 && gc + e < p.n; e++) C[gm * p.c_row + gc + e] = tv[e];
        }
      }
    }
  } else if (col0 + lane < p.n) {
    for (int r = 0; r < 32; r++) {
      long long gm = row0 + r;
      if (gm >= p.m) break;
      C[gm * p.c_row + col0 + lane] = *reinterpret_cast<const T*>(stg + stg_off(r, lane >> 3) + (lane & 7) * 2);
    }
  }
  __syncwarp();
}

template <int BN, bool B_MN, typename T>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TcParams p) {
  using Cfg = TcCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.k + BK - 1) / BK;
  const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;
  const long long num_tiles = tiles_per_batch * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], kEpiWarps); }
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();      // everything above overlapped the previous kernel's tail; operands are final from here
  pdl_trigger();

  if (warp == 0) {
    // ── TMA producer ──
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int batch = (int)(t / tiles_per_batch);
        int rem = (int)(t % tiles_per_batch);
        int m0 = (rem % p.tiles_m) * BM;
        int n0 = (rem / p.tiles_m) * BN;
        int bo = batch / p.batch_inner, bi = batch % p.batch_inner;
        int a_bo = (p.a_bcast & 1) ? 0 : bo, a_bi = (p.a_bcast & 2) ? 0 : bi;
        int b_bo = (p.b_bcast & 1) ? 0 : bo, b_bi = (p.b_bcast & 2) ? 0 : bi;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_4d(sa, &tmap_a, &full_bar[stage], kb * BK, m0, a_bi, a_bo);
          if (B_MN) {
            // [K,N] rows: one 64(n) x 64(k) box per 64-wide slice of the tile's N extent.
#pragma unroll
            for (int j = 0; j < BN / 64; j++)
              tma_load_4d(sb + j * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + j * 64, kb * BK, b_bi, b_bo);
          } else {
            tma_load_4d(sb, &tmap_b, &full_bar[stage], kb * BK, n0, b_bi, b_bo);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer ──
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 0, B_MN ? 1 : 0, BM, BN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
#ifdef AG_GEMM_PROBE
      long long pr_wait = 0, pr_main = 0, pr_steps = 0, pr_t0 = clock64();
#endif
      for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
#ifdef AG_GEMM_PROBE
        long long pc0 = clock64();
#endif
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, p.status, 2)) { ok = false; break; }
        tc_fence_after_sync();
#ifdef AG_GEMM_PROBE
        long long pc1 = clock64(); pr_wait += pc1 - pc0;
#endif
        uint32_t tmem_d = tmem_base + (uint32_t)(acc * Cfg::kAccStride);
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, 3)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; kk++) {
            // A, K-major: 8-row groups 1024 B apart; a K step of 16 elements is 32 B inside the swizzle row.
            uint64_t da = make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            uint64_t db;
            if (B_MN) {
              // B, N-major: rows are k (128 B = 64 n); 8-k groups 1024 B apart (SBO); 64-n slices
              // 64*128 B apart (LBO); a K step of 16 rows is 2048 B.
              db = make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * 128, 1024);
            } else {
              db = make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            }
            mma_f16_ss(tmem_d, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&tmem_full_bar[acc]);  // accumulator complete
#ifdef AG_GEMM_PROBE
        pr_main += clock64() - pc1; pr_steps += num_kb;
#endif
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
#ifdef AG_GEMM_PROBE
      if (p.probe) { p.probe[blockIdx.x * 16 + 0] = pr_wait; p.probe[blockIdx.x * 16 + 1] = pr_main; p.probe[blockIdx.x * 16 + 2] = pr_steps; p.probe[blockIdx.x * 16 + 6] = pr_t0; }
#endif
    }
  } else {
    // ── epilogue warps ──
    const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter .. +31
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int batch = (int)(t / tiles_per_batch);
      int rem = (int)(t % tiles_per_batch);
      int m0 = (rem % p.tiles_m) * BM;
      int n0 = (rem / p.tiles_m) * BN;
      // Everything that does not depend on the accumulator is fetched before waiting for it: this
      // warp's bias slice (into warp-private shared memory) and the first group's residual rows.
      const int pair = (warp - 2) >> 2;  // the two warps of a lane quarter alternate 32-column groups
      long long row0 = (long long)m0 + quarter * 32;
      long long c_off = (long long)(batch / p.batch_inner) * p.c_batch + (long long)(batch % p.batch_inner) * p.c_batch_inner;
      T* bias_s = reinterpret_cast<T*>(smem + STAGES * Cfg::kStageBytes + kStgBytes) + (warp - 2) * epi_slots(BN);
      // 16-bit C with 32-byte aligned rows: the packed epilogue takes the bias as floats; they wait in the warp's staging
      // tile, which that layout leaves unused (zeros when there is no bias)
      const bool packed_epi = p.vec_ok == 2 && !p.c_f32 && !p.argmax_keys;
      float* bias_f = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes + (warp - 2) * kStgBytesPerWarp);
      if (packed_epi) {
        const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
        for (int gi = 0; gi < BN / 64; gi++) {
          int ci = n0 + (pair + 2 * gi) * 32 + lane;
          bias_f[gi * 32 + lane] = (bias && ci < p.n) ? Cvt<T>::to(__ldg(bias + ci)) : 0.f;
        }
      } else if (p.bias && !p.c_f32) {
        const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
        for (int gi = 0; gi < BN / 64; gi++) {
          int ci = n0 + (pair + 2 * gi) * 32 + lane;
          bias_s[gi * 32 + lane] = ci < p.n ? __ldg(bias + ci) : Cvt<T>::from(0.f);
        }
      }
      float* scale_s = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes + kStgBytes + bias_bytes(BN)) + (warp - 2) * epi_slots(BN);
      // the float slots hold the int8 per-channel scales, or the float32 bias of a float32-output product
      const float* fsrc = p.c_f32 ? reinterpret_cast<const float*>(p.bias) : (p.ln_stats ? p.ln_colsum : p.b_scales);
      if (fsrc) {
#pragma unroll
        for (int gi = 0; gi < BN / 64; gi++) {
          int ci = n0 + (pair + 2 * gi) * 32 + lane;
          scale_s[gi * 32 + lane] = ci < p.n ? __ldg(fsrc + ci) : 0.f;
        }
      }
      uint32_t rpre[16];
      if (p.residual && p.vec_ok == 2 && !p.c_f32 && n0 + pair * 32 < p.n)
        load_residual_row<T>(p, reinterpret_cast<const T*>(p.residual) + c_off, row0 + lane, n0 + pair * 32, rpre);
      // folded layer_norm: this row's statistics are fetched (and turned into scale and shift) before the accumulator wait too
      float ln_mean = 0.f, ln_rstd = 1.f;
      ln_row_stats(p, row0 + lane, ln_mean, ln_rstd);
      __syncwarp();
#ifdef AG_GEMM_PROBE
      long long pe0 = clock64();
#endif
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], acc_phase, p.status, 4))) { ok = false; break; }  // warp-uniform
      tc_fence_after_sync();
#ifdef AG_GEMM_PROBE
      long long pe1 = clock64();
#endif
      uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * Cfg::kAccStride);
      uint8_t* stg = smem + STAGES * Cfg::kStageBytes + (warp - 2) * kStgBytesPerWarp;
      unsigned long long best_key = 0;   // argmax mode: this row's best over the warp's column groups of the tile
      float row_sum = 0.f, row_sq = 0.f;
#pragma unroll 1
      for (int g = pair, gi = 0; g < BN / 32; g += 2, gi++) {
        if (n0 + g * 32 >= p.n) break;  // uniform across the warp
        int next_col0 = (g + 2 < BN / 32 && n0 + (g + 2) * 32 < p.n) ? n0 + (g + 2) * 32 : -1;
        epilogue_group<T>(p, taddr + (uint32_t)(g * 32), stg, (p.bias && !p.c_f32) ? bias_s + gi * 32 : nullptr, fsrc ? scale_s + gi * 32 : nullptr, rpre, row0, n0 + g * 32, next_col0,
                          c_off, lane, best_key, ln_mean, ln_rstd, row_sum, row_sq, packed_epi ? bias_f + gi * 32 : nullptr);
      }
      if (p.argmax_keys && best_key != 0 && row0 + lane < p.m) atomicMax(p.argmax_keys + row0 + lane, best_key);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      emit_row_stats(p, row0 + lane, n0 == 0 && pair == 0, row_sum, row_sq);   // after the accumulator is handed back
#ifdef AG_GEMM_PROBE
      if (p.probe && warp == 2 && lane == 0) {
        long long pe2 = clock64();
        p.probe[blockIdx.x * 16 + 3] += pe1 - pe0; p.probe[blockIdx.x * 16 + 4] += pe2 - pe1; p.probe[blockIdx.x * 16 + 5] += 1; p.probe[blockIdx.x * 16 + 7] = pe2;
      }
#endif
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ── CTA-pair variant ────────────────────────────────────────────────────────
// Two CTAs of a cluster compute one 256 x BN tile with cta_group::2 MMAs. Each CTA loads its own
// 128 rows of A and only HALF of the B tile (BN / 2 columns); the tensor cores of the pair
// exchange the halves. Per CTA and 64-deep K step that is 32 KB (BN = 256) fetched from L2 instead
// of the 48 KB a single-CTA 128 x 256 tile needs, and the L2 -> shared-memory feed is what bounds
// the single-CTA main loop (measured: about 100 bytes per clock per SM at best, against the 96 the
// tensor pipe consumes at full rate for that tile). A pipeline stage holds TWO k-blocks (BK = 128 per
// barrier round trip): a barrier in the peer CTA is a cluster-level arrive, and with one k-block per
// stage that latency is paid every 512 tensor cycles and shows (650 cycles per step measured);
// with two per stage the main loop runs at the tensor rate (517 cycles per step).
//   full barriers     live in the even CTA; both CTAs' TMA loads credit their bytes there
//   empty/tmem_full   one copy per CTA; the even CTA's MMA thread commits to both
//   tmem_empty        lives in the even CTA; the epilogue warps of both CTAs arrive there
// Everything else (warp roles, epilogue, bounded waits) is as in the single-CTA kernel.
constexpr int kPairKbPerStage = 2;
template <int BN> struct PairCfg {
  static constexpr int kABytes = BM * BK * 2;               // this CTA's 128 rows of A, one k-block
  static constexpr int kBBytes = (BN / 2) * BK * 2;         // this CTA's half of B, one k-block
  static constexpr int kKbBytes = kABytes + kBBytes;
  static constexpr int kStageBytes = kPairKbPerStage * kKbBytes;
  static constexpr int kStages = (BN == 128) ? 4 : 3;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStgBytes + bias_bytes(BN) + scale_bytes(BN) + 1024;
  static_assert(kSmemBytes + 512 <= 232448, "dynamic + static shared memory must fit the 227 KB a CTA may use");
  static constexpr int kAccStride = (BN == 192) ? 256 : BN; // column distance between the two accumulator buffers
  static constexpr int kTmemCols = 2 * kAccStride;          // two accumulator buffers (a power of two)
};

// W8 = the B operand is an int8 [N, K] weight (per-output-channel symmetric quantisation): the dequantisation
// happens inside this kernel's prologue. TMA brings each CTA's half of the weight tile in as raw bytes (64-byte
// swizzle) into the upper half of the stage's B area; four converter warps read their rows into registers, meet
// at a named barrier (the raw bytes lie where widened rows will be written), widen the integers exactly to the
// activation type in the 128-byte-swizzled K-major layout the MMA descriptor expects, and arrive on the stage's
// full barrier in the even CTA, which therefore counts the A bytes of both CTAs plus eight converter warps. The
// per-channel scales multiply the accumulator in the epilogue (exact for per-output-channel scaling), so the
// only copy of the weights in global memory is the int8 one and no widened copy is ever written there.
constexpr int kConvWarps = 4;
constexpr int kTcThreadsW8 = kTcThreads + kConvWarps * 32;
// Four int8 values (one 32-bit word) -> two words of packed 16-bit floats, exactly. Each byte is biased to
// unsigned (u = v + 128), dropped into the mantissa of 2^23 (0x4B000000 | u = 8388608 + u), and the float
// subtraction of 8388736 leaves v; values of at most 8 significant bits survive the narrowing unchanged.
template <typename T>
__device__ __forceinline__ void widen_s8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.0f;
  float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.0f;
  float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.0f;
  float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.0f;
  if (std::is_same<T, __nv_bfloat16>::value) {
    lo = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);   // upper halves: bf16 is a truncated float
    hi = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
  } else {
    lo = pack2<T>(f0, f1);
    hi = pack2<T>(f2, f3);
  }
}

template <int BN, bool B_MN, typename T, bool W8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(W8 ? kTcThreadsW8 : kTcThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TcParams p) {
  using Cfg = PairCfg<BN>;
  static_assert(!W8 || (BN == 256 && !B_MN), "the int8-weight form takes a K-major [N, K] weight and 256-wide tiles");
  constexpr int STAGES = Cfg::kStages;
  constexpr int KBS = kPairKbPerStage;
  constexpr int kRawBytes = (BN / 2) * BK;                  // this CTA's half of the int8 weight tile, one k-block
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t raw_bar[STAGES];                      // W8: the raw int8 bytes of a stage have landed (per CTA)
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = even CTA (issues the MMAs), 1 = its peer
  const int num_kb = (p.k + BK - 1) / BK;
  const int rounds = (num_kb + KBS - 1) / KBS;   // a k-block past the end of K is fetched as zeros (TMA out-of-range fill)
  const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;   // tiles of 256 x BN
  const long long num_tiles = tiles_per_batch * p.batch;
  const long long first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], W8 ? 1 + 2 * kConvWarps : 1); mbar_init(&empty_bar[s], 1); mbar_init(&raw_bar[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 2 * kEpiWarps); }
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is signalled on them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ── TMA producer (both CTAs) ──
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (long long t = first_tile; t < num_tiles && ok; t += tile_step) {
        int batch = (int)(t / tiles_per_batch);
        int rem = (int)(t % tiles_per_batch);
        int m0 = (rem % p.tiles_m) * (2 * BM) + (int)rank * BM;
        int n0 = (rem / p.tiles_m) * BN + (int)rank * (BN / 2);
        int bo = batch / p.batch_inner, bi = batch % p.batch_inner;
        int a_bo = (p.a_bcast & 1) ? 0 : bo, a_bi = (p.a_bcast & 2) ? 0 : bi;
        int b_bo = (p.b_bcast & 1) ? 0 : bo, b_bi = (p.b_bcast & 2) ? 0 : bi;
        for (int r = 0; r < rounds; r++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(&full_bar[stage], W8 ? 2 * KBS * Cfg::kABytes : 2 * Cfg::kStageBytes);   // both CTAs' bytes
          if (W8) mbar_expect_tx(&raw_bar[stage], KBS * kRawBytes);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
#pragma unroll
          for (int j = 0; j < KBS; j++) {
            const int kc = (r * KBS + j) * BK;
            uint8_t* sa = smem + stage * Cfg::kStageBytes + j * Cfg::kKbBytes;
            uint8_t* sb = sa + Cfg::kABytes;
            tma_load_4d_pair(sa, &tmap_a, bar, kc, m0, a_bi, a_bo);
            if (W8) {
              // raw bytes into the upper half of the B area (the lower half is written first by the converters)
              tma_load_4d(sb + Cfg::kBBytes - kRawBytes, &tmap_b, &raw_bar[stage], kc, n0, 0, 0);
            } else if (B_MN) {
#pragma unroll
              for (int q = 0; q < BN / 128; q++)
                tma_load_4d_pair(sb + q * (64 * BK * 2), &tmap_b, bar, n0 + q * 64, kc, b_bi, b_bo);
            } else {
              tma_load_4d_pair(sb, &tmap_b, bar, kc, n0, b_bi, b_bo);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer (even CTA only) ──
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 0, B_MN ? 1 : 0, 2 * BM, BN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
#ifdef AG_GEMM_PROBE
      long long pr_wait = 0, pr_main = 0, pr_steps = 0, pr_t0 = clock64();
#endif
      for (long long t = first_tile; t < num_tiles && ok; t += tile_step) {
#ifdef AG_GEMM_PROBE
        long long pc0 = clock64();
#endif
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, p.status, 2)) { ok = false; break; }
        tc_fence_after_sync();
#ifdef AG_GEMM_PROBE
        long long pc1 = clock64(); pr_wait += pc1 - pc0;
#endif
        uint32_t tmem_d = tmem_base + (uint32_t)(acc * Cfg::kAccStride);
        for (int r = 0; r < rounds; r++) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, 3)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int j = 0; j < KBS; j++) {
            uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes + j * Cfg::kKbBytes);
            uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; kk++) {
              uint64_t da = make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
              uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * 128, 1024)
                                 : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
              mma_f16_ss_pair(tmem_d, da, db, idesc, (r > 0 || j > 0 || kk > 0) ? 1u : 0u);
            }
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          mma_commit_pair(mapa_u32(eb, 0));
          mma_commit_pair(mapa_u32(eb, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t fb = smem_u32(&tmem_full_bar[acc]);
        mma_commit_pair(mapa_u32(fb, 0));
        mma_commit_pair(mapa_u32(fb, 1));
#ifdef AG_GEMM_PROBE
        pr_main += clock64() - pc1; pr_steps += num_kb;
#endif
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
#ifdef AG_GEMM_PROBE
      if (p.probe) { p.probe[blockIdx.x * 16 + 0] = pr_wait; p.probe[blockIdx.x * 16 + 1] = pr_main; p.probe[blockIdx.x * 16 + 2] = pr_steps; p.probe[blockIdx.x * 16 + 6] = pr_t0; }
#endif
    }
  } else if (W8 && warp >= 2 + kEpiWarps) {
    // ── converter warps (both CTAs): int8 rows -> 16-bit rows of this CTA's half of the B tile ──
    const int row = (warp - 2 - kEpiWarps) * 32 + lane;       // 0 .. BN/2 - 1: one weight row per thread
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (long long t = first_tile; t < num_tiles && ok; t += tile_step) {
      for (int r = 0; r < rounds; r++) {
        const bool landed = mbar_wait(&raw_bar[stage], phase, p.status, 5);
        uint4 q[KBS][4];
#pragma unroll
        for (int j = 0; j < KBS; j++) {
          const uint8_t* raw = smem + stage * Cfg::kStageBytes + j * Cfg::kKbBytes + Cfg::kABytes + Cfg::kBBytes - kRawBytes;
#pragma unroll
          for (int c = 0; c < 4; c++) q[j][c] = *reinterpret_cast<const uint4*>(raw + stg_off(row, c));   // 64-byte rows, 64-byte swizzle
        }
        // Every converter thread of this CTA holds its raw rows: the widened rows may now overwrite them. The same
        // barrier carries the AND of `landed`, so that after a wait that gave up all four warps leave together
        // (a warp that went on alone would wait at this barrier for ever).
        uint32_t all_landed;
        asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 q, %1, 0;\n bar.red.and.pred p, 1, %2, q;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(all_landed) : "r"((uint32_t)landed), "n"(kConvWarps * 32) : "memory");
        if (!all_landed) { ok = false; break; }
#pragma unroll
        for (int j = 0; j < KBS; j++) {
          uint8_t* dst = smem + stage * Cfg::kStageBytes + j * Cfg::kKbBytes + Cfg::kABytes + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
          for (int c = 0; c < 4; c++) {
            // 16 int8 = words x, y, z, w -> two 16-byte chunks (2c, 2c + 1) of the 128-byte row, chunk index XOR (row % 8)
            uint4 lo4, hi4;
            widen_s8x4<T>(q[j][c].x, lo4.x, lo4.y); widen_s8x4<T>(q[j][c].y, lo4.z, lo4.w);
            widen_s8x4<T>(q[j][c].z, hi4.x, hi4.y); widen_s8x4<T>(q[j][c].w, hi4.z, hi4.w);
            *reinterpret_cast<uint4*>(dst + (((2 * c) ^ (row & 7)) << 4)) = lo4;
            *reinterpret_cast<uint4*>(dst + (((2 * c + 1) ^ (row & 7)) << 4)) = hi4;
          }
        }
        fence_proxy_async_smem();   // the MMA reads these rows through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&full_bar[stage]), 0));
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ── epilogue warps (both CTAs; each reads its own 128 accumulator lanes) ──
    const int quarter = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    // folded layer_norm: a row's statistics are fetched one tile ahead (the load of the next tile's row is in flight
    // during this tile's epilogue), so their latency is never on the path between two tiles
    auto tile_row = [&](long long tt) -> long long {
      if (tt >= num_tiles) return -1;
      const int rem_ = (int)(tt % tiles_per_batch);
      return (long long)((rem_ % p.tiles_m) * (2 * BM) + (int)rank * BM) + quarter * 32 + lane;
    };
    longlong2 stats_next = ln_stats_fetch(p, tile_row(first_tile));
    for (long long t = first_tile; t < num_tiles && ok; t += tile_step) {
      int batch = (int)(t / tiles_per_batch);
      int rem = (int)(t % tiles_per_batch);
      int m0 = (rem % p.tiles_m) * (2 * BM) + (int)rank * BM;
      int n0 = (rem / p.tiles_m) * BN;
      const int pair = (warp - 2) >> 2;
      long long row0 = (long long)m0 + quarter * 32;
      const longlong2 stats_cur = stats_next;
      stats_next = ln_stats_fetch(p, tile_row(t + tile_step));
      long long c_off = (long long)(batch / p.batch_inner) * p.c_batch + (long long)(batch % p.batch_inner) * p.c_batch_inner;
      T* bias_s = reinterpret_cast<T*>(smem + STAGES * Cfg::kStageBytes + kStgBytes) + (warp - 2) * epi_slots(BN);
      // 16-bit C with 32-byte aligned rows: the packed epilogue takes the bias as floats; they wait in the warp's staging
      // tile, which that layout leaves unused (zeros when there is no bias)
      const bool packed_epi = p.vec_ok == 2 && !p.c_f32 && !p.argmax_keys;
      float* bias_f = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes + (warp - 2) * kStgBytesPerWarp);
      if (packed_epi) {
        const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
        for (int gi = 0; gi < BN / 64; gi++) {
          int ci = n0 + (pair + 2 * gi) * 32 + lane;
          bias_f[gi * 32 + lane] = (bias && ci < p.n) ? Cvt<T>::to(__ldg(bias + ci)) : 0.f;
        }
      } else if (p.bias && !p.c_f32) {
        const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
        for (int gi = 0; gi < BN / 64; gi++) {
          int ci = n0 + (pair + 2 * gi) * 32 + lane;
          bias_s[gi * 32 + lane] = ci < p.n ? __ldg(bias + ci) : Cvt<T>::from(0.f);
        }
      }
      float* scale_s = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes + kStgBytes + bias_bytes(BN)) + (warp - 2) * epi_slots(BN);
      // the float slots hold the int8 per-channel scales, or the float32 bias of a float32-output product
      const float* fsrc = p.c_f32 ? reinterpret_cast<const float*>(p.bias) : (p.ln_stats ? p.ln_colsum : p.b_scales);
      if (fsrc) {
#pragma unroll
        for (int gi = 0; gi < BN / 64; gi++) {
          int ci = n0 + (pair + 2 * gi) * 32 + lane;
          scale_s[gi * 32 + lane] = ci < p.n ? __ldg(fsrc + ci) : 0.f;
        }
      }
      uint32_t rpre[16];
      if (p.residual && p.vec_ok == 2 && !p.c_f32 && n0 + pair * 32 < p.n)
        load_residual_row<T>(p, reinterpret_cast<const T*>(p.residual) + c_off, row0 + lane, n0 + pair * 32, rpre);
      // folded layer_norm: this row's statistics are fetched (and turned into scale and shift) before the accumulator wait too
      float ln_mean = 0.f, ln_rstd = 1.f;
      if (row0 + lane < p.m) ln_stats_finish(p, stats_cur, ln_mean, ln_rstd);
      __syncwarp();
#ifdef AG_GEMM_PROBE
      long long pe0 = clock64();
#endif
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], acc_phase, p.status, 4))) { ok = false; break; }
      tc_fence_after_sync();
#ifdef AG_GEMM_PROBE
      long long pe1 = clock64();
#endif
      uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * Cfg::kAccStride);
      uint8_t* stg = smem + STAGES * Cfg::kStageBytes + (warp - 2) * kStgBytesPerWarp;
      unsigned long long best_key = 0;
      float row_sum = 0.f, row_sq = 0.f;
      if (row0 < p.m) {   // a peer CTA whose rows lie past M has nothing to store
#pragma unroll 1
        for (int g = pair, gi = 0; g < BN / 32; g += 2, gi++) {
          if (n0 + g * 32 >= p.n) break;
          int next_col0 = (g + 2 < BN / 32 && n0 + (g + 2) * 32 < p.n) ? n0 + (g + 2) * 32 : -1;
          epilogue_group<T>(p, taddr + (uint32_t)(g * 32), stg, (p.bias && !p.c_f32) ? bias_s + gi * 32 : nullptr, fsrc ? scale_s + gi * 32 : nullptr, rpre, row0, n0 + g * 32, next_col0,
                            c_off, lane, best_key, ln_mean, ln_rstd, row_sum, row_sq, packed_epi ? bias_f + gi * 32 : nullptr);
        }
        }
      if (p.argmax_keys && best_key != 0 && row0 + lane < p.m) atomicMax(p.argmax_keys + row0 + lane, best_key);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty_bar[acc]), 0));
      if (row0 < p.m) emit_row_stats(p, row0 + lane, n0 == 0 && pair == 0, row_sum, row_sq);   // after the accumulator is handed back
#ifdef AG_GEMM_PROBE
      if (p.probe && warp == 2 && lane == 0 && rank == 0) {
        long long pe2 = clock64();
        p.probe[blockIdx.x * 16 + 3] += pe1 - pe0; p.probe[blockIdx.x * 16 + 4] += pe2 - pe1; { long long ti = p.probe[blockIdx.x * 16 + 5]; if (ti < 6) p.probe[blockIdx.x * 16 + 8 + ti] = pe2 - pe1; } p.probe[blockIdx.x * 16 + 5] += 1; p.probe[blockIdx.x * 16 + 7] = pe2;
      }
#endif
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // Neither CTA may leave (or free TMEM) while its peer can still signal its barriers or run
  // MMAs against its shared memory.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
}

// ── chained products ────────────────────────────────────────────────────────
// Up to kChainMax products in ONE launch of the CTA-pair kernel's pipeline, where product g + 1 reads product g's result
// as its A operand (a transformer block's out-projection -> FC1 -> FC2 -> the next block's QKV). Run one after the
// other, each of these short products pays its own pipeline fill, the exposed epilogue of its last tiles and a partly
// filled last wave; chained, the tensor pipe only drains once. What makes it possible is that a 256-row block of
// product g + 1 needs nothing but the same 256 rows of product g:
//   tiles         every product is cut into 256 x 256 tiles, row block by row block; the host deals the tiles of all
//                 products, in that order, to the CTA pairs (each tile to the pair with the least work so far) and
//                 every pair walks its own list, so the roles of a pair need no run-time scheduler
//   dependencies  when the eight epilogue warps of a CTA have stored their parts of a tile they arrive on a shared-memory
//                 barrier; the CTA's announcer warp (one thread) waits for it, fences (proxy fence, __threadfence: the
//                 stores it has observed through the barrier become visible GPU-wide first) and adds 8 to the counter of
//                 (product, row block), so the fence's latency is not on the epilogue warps' path. The TMA thread of a
//                 consumer tile waits (bounded) until the producer's row block has all its arrivals (16 per tile), then
//                 fences the async proxy and loads. A tile only ever waits for tiles earlier in the global order, and every pair takes its
//                 tiles in that order, so the earliest unfinished tile can always run: no cycle
//   epilogue      row statistics and residual rows of the next tile are fetched ahead only when its row block is
//                 already complete (its counter is read one tile earlier); otherwise after the accumulator wait
//   counters      zero on entry; the last CTA to leave zeroes them again
// N-major B ([K, N] weights), 16-bit types, unbatched; the epilogue is the pair kernel's (bias, activation, residual,
// folded layer_norm on either side).
constexpr int kChainFlagInts = kChainMax * kChainFlagStride;   // + 1 exit counter behind them
struct ChainParams {
  TcParams prob[kChainMax];
  int need[kChainMax];          // arrivals of the previous product's row block a tile of product g waits for (0: none)
  int count;
  const int* list_off;          // [clusters + 1] into `list`
  const int* list;              // product << 24 | tile index within the product (row-block major), in execution order
  int* flags;                   // [kChainFlagInts + 1]
#ifdef AG_CHAIN_PROBE
  long long* probe;             // per CTA, 16 slots: where the roles' cycles go (compile-time diagnostic only)
#endif
};
struct alignas(64) ChainMaps { CUtensorMap a[kChainMax]; CUtensorMap b[kChainMax]; };

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// A look at a counter that orders nothing by itself (an acquire load holds the warp's later memory operations back until
// it has returned, a full L2 round trip in the middle of an epilogue): only used as a hint, see the epilogue warps.
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
// Bounded like every other wait of these kernels: gives up (recording `code`) after the limit or when another role has.
__device__ __forceinline__ bool flag_wait(const int* f, int need, int* status, int code) {
  if (ld_acquire_gpu(f) >= need) return true;
  unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_gpu(f) >= need) return true;
    if ((++spins & 0x3f) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) { atomicCAS(status, 0, code); return false; }
    }
  }
}
// Row statistics written earlier in the same launch: read past L1 (the non-coherent path of ln_stats_fetch is for
// data that is constant for the whole launch).
__device__ __forceinline__ longlong2 ln_stats_fetch_cg(const TcParams& p, long long gm) {
  if (!p.ln_stats || gm < 0 || gm >= p.m) return make_longlong2(0, 0);
  return __ldcg(reinterpret_cast<const longlong2*>(p.ln_stats) + gm);
}

// Epilogue warps: 8 (two per TMEM lane quarter, alternating column groups, 168 registers each). 4 (one per quarter, every
// group, 220 registers) was measured at 146 against 112 us per GPT-2-small block: eight groups per tile in series
// (121 us with its 255-register budget spent on accumulator loads issued a group ahead).
constexpr int kChainEpiWarps = 8;
constexpr int kChainGroupStep = kChainEpiWarps / 4;           // column groups between two groups of one warp
constexpr int kChainGroups = 8 / kChainGroupStep;             // 32-column groups of a 256-wide tile per warp
constexpr int kChainThreads = 64 + kChainEpiWarps * 32 + 32;  // TMA warp, MMA warp, epilogue warps, announcer warp
template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kChainThreads, 1)
gemm_tc_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams cp) {
  constexpr int BN = 256;
  using Cfg = PairCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int KBS = kPairKbPerStage;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint64_t stored_bar[2];        // a tile's results are stored (eight epilogue warps arrive; the announcer waits)
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_last;
  __shared__ TcParams s_prob[kChainMax];

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = blockIdx.x >> 1;

  {
    const int* src = reinterpret_cast<const int*>(cp.prob);
    int* dst = reinterpret_cast<int*>(s_prob);
    for (int i = threadIdx.x; i < (int)(sizeof(TcParams) / 4) * cp.count; i += blockDim.x) dst[i] = src[i];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 2 * kChainEpiWarps); mbar_init(&stored_bar[a], kChainEpiWarps); }
    mbar_fence_init();
    for (int g = 0; g < cp.count; g++) { prefetch_tmap(&maps.a[g]); prefetch_tmap(&maps.b[g]); }
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();
  pdl_trigger();
  const int li0 = __ldg(cp.list_off + cluster), li1 = __ldg(cp.list_off + cluster + 1);
  int* const status = s_prob[0].status;
#ifdef AG_CHAIN_PROBE
  const long long probe_t0 = clock64();
#endif

  if (warp == 0) {
    // ── TMA producer (both CTAs) ──
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int li = li0; li < li1 && ok; li++) {
        const int e = __ldg(cp.list + li);
        const int g = e >> 24, lt = e & 0xffffff;
        const TcParams& p = s_prob[g];
        const int mi = lt / p.tiles_n, ni = lt - mi * p.tiles_n;
        const int m0 = mi * (2 * BM) + (int)rank * BM;
        const int n0 = ni * BN + (int)rank * (BN / 2);
        const int rounds = ((p.k + BK - 1) / BK + KBS - 1) / KBS;
        const CUtensorMap* ta = &maps.a[g];
        const CUtensorMap* tb = &maps.b[g];
#ifdef AG_CHAIN_PROBE
        long long q0 = clock64();
#endif
        if (cp.need[g] > 0) {
          // the rows this tile reads are another tile's results: wait for them, then order the generic-proxy view this
          // thread has just acquired before the async-proxy reads it is about to issue
          if (!flag_wait(cp.flags + (g - 1) * kChainFlagStride + mi, cp.need[g], status, 6)) { ok = false; break; }
          fence_proxy_async_global();
        }
#ifdef AG_CHAIN_PROBE
        if (cp.probe) { cp.probe[blockIdx.x * 16 + 0] += clock64() - q0; cp.probe[blockIdx.x * 16 + 8 + g] += clock64() - q0; }
#endif
        for (int r = 0; r < rounds; r++) {
#ifdef AG_CHAIN_PROBE
          long long q1 = clock64();
#endif
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, status, 1)) { ok = false; break; }
#ifdef AG_CHAIN_PROBE
          if (cp.probe) cp.probe[blockIdx.x * 16 + 1] += clock64() - q1;
#endif
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
#pragma unroll
          for (int j = 0; j < KBS; j++) {
            const int kc = (r * KBS + j) * BK;
            uint8_t* sa = smem + stage * Cfg::kStageBytes + j * Cfg::kKbBytes;
            uint8_t* sb = sa + Cfg::kABytes;
            tma_load_4d_pair(sa, ta, bar, kc, m0, 0, 0);
#pragma unroll
            for (int q = 0; q < BN / 128; q++)
              tma_load_4d_pair(sb + q * (64 * BK * 2), tb, bar, n0 + q * 64, kc, 0, 0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer (even CTA only) ──
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 0, 1, 2 * BM, BN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int li = li0; li < li1 && ok; li++) {
        const int g = __ldg(cp.list + li) >> 24;
        const int rounds = ((s_prob[g].k + BK - 1) / BK + KBS - 1) / KBS;
#ifdef AG_CHAIN_PROBE
        long long q0 = clock64();
#endif
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, status, 2)) { ok = false; break; }
        tc_fence_after_sync();
#ifdef AG_CHAIN_PROBE
        if (cp.probe) { cp.probe[blockIdx.x * 16 + 2] += clock64() - q0; cp.probe[blockIdx.x * 16 + 4] += rounds; }
#endif
        uint32_t tmem_d = tmem_base + (uint32_t)(acc * Cfg::kAccStride);
        for (int r = 0; r < rounds; r++) {
#ifdef AG_CHAIN_PROBE
          long long q1 = clock64();
#endif
          if (!mbar_wait(&full_bar[stage], phase, status, 3)) { ok = false; break; }
          tc_fence_after_sync();
#ifdef AG_CHAIN_PROBE
          if (cp.probe) cp.probe[blockIdx.x * 16 + 3] += clock64() - q1;
#endif
#pragma unroll
          for (int j = 0; j < KBS; j++) {
            uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes + j * Cfg::kKbBytes);
            uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; kk++) {
              uint64_t da = make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
              uint64_t db = make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * 128, 1024);
              mma_f16_ss_pair(tmem_d, da, db, idesc, (r > 0 || j > 0 || kk > 0) ? 1u : 0u);
            }
          }
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          mma_commit_pair(mapa_u32(eb, 0));
          mma_commit_pair(mapa_u32(eb, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t fb = smem_u32(&tmem_full_bar[acc]);
        mma_commit_pair(mapa_u32(fb, 0));
        mma_commit_pair(mapa_u32(fb, 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp == 2 + kChainEpiWarps) {
    // ── announcer (both CTAs): tile by tile, "this CTA's rows of the tile are stored" -> the row block's counter ──
    if (lane == 0) {
      int slot = 0; uint32_t parity = 0;
      for (int li = li0; li < li1; li++) {
        const int e = __ldg(cp.list + li);
        const int g = e >> 24, lt = e & 0xffffff;
        if (!mbar_wait(&stored_bar[slot], parity, status, 8)) break;
        fence_proxy_async_global();
        __threadfence();
        atomicAdd(cp.flags + g * kChainFlagStride + lt / s_prob[g].tiles_n, kChainEpiWarps);
        if (++slot == 2) { slot = 0; parity ^= 1; }
      }
    }
  } else {
    // ── epilogue warps (both CTAs; each reads its own 128 accumulator lanes) ──
    const int quarter = warp & 3;
    const int pair = (warp - 2) >> 2;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    bool fetched = false;            // this tile's row statistics and first residual group are already in registers
    longlong2 stats_raw = make_longlong2(0, 0);
    uint32_t rpre[16];
    int e_next = li0 < li1 ? __ldg(cp.list + li0) : -1;
    int e_next2 = li0 + 1 < li1 ? __ldg(cp.list + li0 + 1) : -1;   // list entries are read two tiles ahead: nothing waits for them
    T col_bias[kChainGroups];                         // the next tile's bias and column sums of this lane's columns, one tile ahead
    float col_sum[kChainGroups];                      // (as loaded: a conversion here would wait for the load)
    auto fetch_cols = [&](int e_) {
      const int g_ = e_ >> 24, lt_ = e_ & 0xffffff;
      const TcParams& q = s_prob[g_];
      const int n0_ = (lt_ % q.tiles_n) * BN;
      const T* bias = reinterpret_cast<const T*>(q.bias);
      const float* cs = q.ln_stats ? q.ln_colsum : nullptr;
#pragma unroll
      for (int gi = 0; gi < kChainGroups; gi++) {
        const int ci = n0_ + (pair + kChainGroupStep * gi) * 32 + lane;
        col_bias[gi] = (bias && ci < q.n) ? __ldg(bias + ci) : Cvt<T>::from(0.f);
        col_sum[gi] = (cs && ci < q.n) ? __ldg(cs + ci) : 0.f;
      }
    };
    if (e_next >= 0) fetch_cols(e_next);
    int fv_next = 0;                 // the dependency counter of the next tile, read one tile ahead
    if (e_next >= 0 && cp.need[e_next >> 24] > 0) {
      const int g_ = e_next >> 24, lt_ = e_next & 0xffffff;
      fv_next = ld_relaxed_gpu(cp.flags + (g_ - 1) * kChainFlagStride + lt_ / s_prob[g_].tiles_n);
    }
    for (int li = li0; li < li1 && ok; li++) {
#ifdef AG_CHAIN_PROBE
      const long long q_top = clock64();
#endif
      const int e = e_next;
      const int fv = fv_next;
      const int g = e >> 24, lt = e & 0xffffff;
      // a copy in registers: fields read through a pointer into shared memory would be loaded again after every
      // store and tensor-memory load of the epilogue (their asm statements clobber memory)
      TcParams p;
      {
        const TcParams& sp = s_prob[g];
        p.c = sp.c; p.bias = sp.bias; p.residual = sp.residual; p.b_scales = nullptr; p.alpha = sp.alpha; p.act = sp.act;
        p.m = sp.m; p.n = sp.n; p.k = sp.k; p.batch = 1; p.batch_inner = 1; p.c_row = sp.c_row; p.c_batch = 0; p.c_batch_inner = 0;
        p.a_bcast = 0; p.b_bcast = 0; p.tiles_m = sp.tiles_m; p.tiles_n = sp.tiles_n; p.vec_ok = 2 /* the only layout a link may have: the others compile out */; p.bias_vec = 0;
        p.argmax_keys = nullptr; p.c_f32 = 0; p.ln_stats = sp.ln_stats; p.ln_colsum = sp.ln_colsum; p.ln_inv_k = sp.ln_inv_k; p.ln_eps = sp.ln_eps;
        p.stats_out = sp.stats_out; p.stats_zero = sp.stats_zero; p.status = status;
      }
      const int mi = lt / p.tiles_n, ni = lt - mi * p.tiles_n;
      const int need = cp.need[g];
      e_next = e_next2;
      e_next2 = li + 2 < li1 ? __ldg(cp.list + li + 2) : -1;
      fv_next = 0;
      if (e_next >= 0 && cp.need[e_next >> 24] > 0) {
        const int g_ = e_next >> 24, lt_ = e_next & 0xffffff;
        fv_next = ld_relaxed_gpu(cp.flags + (g_ - 1) * kChainFlagStride + lt_ / s_prob[g_].tiles_n);
      }
      const int m0 = mi * (2 * BM) + (int)rank * BM;
      const int n0 = ni * BN;
      const long long row0 = (long long)m0 + quarter * 32;
      // this tile's bias and column sums were fetched into registers one tile ago; they go to shared memory as floats (the
      // packed epilogue reads them as broadcasts; the staging tile is unused with 32-byte aligned rows)
      float* bias_f = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes) + (warp - 2) * (kChainGroups * 32);
      float* scale_s = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes + kStgBytes + bias_bytes(BN)) + (warp - 2) * (kChainGroups * 32);
      const float* fsrc = p.ln_stats ? p.ln_colsum : nullptr;
#pragma unroll
      for (int gi = 0; gi < kChainGroups; gi++) { bias_f[gi * 32 + lane] = Cvt<T>::to(col_bias[gi]); scale_s[gi * 32 + lane] = col_sum[gi]; }
      if (e_next >= 0) fetch_cols(e_next);
      const bool res_ahead = p.residual && p.vec_ok == 2 && n0 + pair * 32 < p.n;
      // `fv` is a relaxed look at the counter taken one tile ago. Seeing it complete, the loads below are issued after
      // it (they depend on the branch), go to L2 (the statistics) or to lines this SM has not touched in this launch (the
      // residual rows), and the producer's stores were GPU-visible before the counter moved: they read the final values.
      if (!fetched && (need == 0 || fv >= need)) {
        stats_raw = ln_stats_fetch_cg(p, row0 + lane);
        if (res_ahead) load_residual_row<T>(p, reinterpret_cast<const T*>(p.residual), row0 + lane, n0 + pair * 32, rpre);
        fetched = true;
      }
      __syncwarp();
#ifdef AG_CHAIN_PROBE
      long long q0 = clock64();
      long long q1 = q0;
#endif
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], acc_phase, status, 4))) { ok = false; break; }
      tc_fence_after_sync();
#ifdef AG_CHAIN_PROBE
      long long q2 = clock64();
      if (cp.probe && warp == 2 && lane == 0) { cp.probe[blockIdx.x * 16 + 15] += q0 - q_top; cp.probe[blockIdx.x * 16 + 5] += q1 - q0; cp.probe[blockIdx.x * 16 + 6] += q2 - q1; cp.probe[blockIdx.x * 16 + 12] += fetched ? 0 : 1; }
#endif
      if (!fetched) {
        // This pair's TMA thread acquired the row block's counter before it loaded the tile's operands, and the full
        // accumulator this warp has just waited for follows those loads through the pipeline's barriers: the producer's
        // stores are ordered before these reads without another look at the counter.
        stats_raw = ln_stats_fetch_cg(p, row0 + lane);
        if (res_ahead) load_residual_row<T>(p, reinterpret_cast<const T*>(p.residual), row0 + lane, n0 + pair * 32, rpre);
      }
      fetched = false;
      float ln_mean = 0.f, ln_rstd = 1.f;
      if (row0 + lane < p.m) ln_stats_finish(p, stats_raw, ln_mean, ln_rstd);
      uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * Cfg::kAccStride);
      uint8_t* stg = nullptr;   // the staged layouts are not used here (rows are 32-byte aligned)
      unsigned long long best_key = 0;
      float row_sum = 0.f, row_sq = 0.f;
      if (row0 < p.m) {
#pragma unroll 1
        for (int gg = pair, gi = 0; gg < BN / 32; gg += kChainGroupStep, gi++) {
          if (n0 + gg * 32 >= p.n) break;
          int next_col0 = (gg + kChainGroupStep < BN / 32 && n0 + (gg + kChainGroupStep) * 32 < p.n) ? n0 + (gg + kChainGroupStep) * 32 : -1;
          epilogue_group<T>(p, taddr + (uint32_t)(gg * 32), stg, nullptr, fsrc ? scale_s + gi * 32 : nullptr, rpre, row0, n0 + gg * 32, next_col0,
                            0, lane, best_key, ln_mean, ln_rstd, row_sum, row_sq, bias_f + gi * 32);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty_bar[acc]), 0));
      if (row0 < p.m) emit_row_stats(p, row0 + lane, n0 == 0 && pair == 0, row_sum, row_sq);
      __syncwarp();                                   // every lane's stores and atomics are issued: the announcer takes over
      if (lane == 0) mbar_arrive(&stored_bar[acc]);
      // the next tile's statistics and first residual rows, if its row block is known to be complete
      if (e_next >= 0) {
        const int gn = e_next >> 24, ltn = e_next & 0xffffff;
        const TcParams& pn = s_prob[gn];
        if (cp.need[gn] == 0 || fv_next >= cp.need[gn]) {
          const int min_ = ltn / pn.tiles_n, nin = ltn - min_ * pn.tiles_n;
          const long long rown = (long long)(min_ * (2 * BM) + (int)rank * BM) + quarter * 32;
          stats_raw = ln_stats_fetch_cg(pn, rown + lane);
          if (pn.residual && pn.vec_ok == 2 && nin * BN + pair * 32 < pn.n)
            load_residual_row<T>(pn, reinterpret_cast<const T*>(pn.residual), rown + lane, nin * BN + pair * 32, rpre);
          fetched = true;
        }
      }
#ifdef AG_CHAIN_PROBE
      if (cp.probe && warp == 2 && lane == 0) { cp.probe[blockIdx.x * 16 + 7] += clock64() - q2; cp.probe[blockIdx.x * 16 + 13] += 1; }
#endif
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
#ifdef AG_CHAIN_PROBE
  if (cp.probe && threadIdx.x == 0) cp.probe[blockIdx.x * 16 + 14] += clock64() - probe_t0;
#endif
  // the last CTA to get here has seen every other one finish with the counters: it zeroes them for the next launch
  if (threadIdx.x == 0) { __threadfence(); s_last = atomicAdd(cp.flags + kChainFlagInts, 1) == (int)gridDim.x - 1 ? 1 : 0; }
  __syncthreads();
  if (s_last) {
    for (int i = threadIdx.x; i < cp.count * kChainFlagStride; i += blockDim.x) cp.flags[i] = 0;
    if (threadIdx.x == 0) cp.flags[kChainFlagInts] = 0;
  }
}

// ── host side ───────────────────────────────────────────────────────────────
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// APPLEGPU_W8_FUSED: 'auto' (default) widens int8 weights inside the GEMM for up to kW8FusedMaxRows activation rows and by one
// separate pass per call above that; '1' always inside the GEMM; '0' always by the separate pass.
static int g_w8_fused = [] { const char* v = std::getenv("APPLEGPU_W8_FUSED"); return !v ? 2 : v[0] == '0' ? 0 : v[0] == '1' ? 1 : 2; }();
// Measured on a B200 (GPT-2-large linears, bf16 activations): at 2048 rows both forms take the same time; at 16384 rows the
// prologue form is 6-20 % slower, because it widens the same weight tile again for every 256-row block of the activations
// and those instructions compete with the epilogue for issue slots and with the tensor pipe for power.
constexpr int64_t kW8FusedMaxRows = 2048;
struct MapKey {
  const void* ptr; uint64_t d[4]; uint64_t s[3]; uint32_t b0, b1; int dt; int pad;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; i++) { h ^= w[i]; h *= 1099511628211ull; }
    return (size_t)h;
  }
};
static std::mutex g_map_mu;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

// 4-D map over (inner, rows, batch_inner, batch_outer) of 2-byte elements with a 128B-swizzled
// box {b0, b1, 1, 1}. Strides are in elements; a dimension of extent 1 may carry any stride.
Status make_map(CUtensorMap* out, DType dt, const void* ptr, uint64_t inner, uint64_t rows, uint64_t nbi, uint64_t nbo,
                uint64_t row_stride, uint64_t bi_stride, uint64_t bo_stride, uint32_t b0, uint32_t b1) {
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr; key.d[0] = inner; key.d[1] = rows; key.d[2] = nbi; key.d[3] = nbo;
  key.s[0] = row_stride; key.s[1] = bi_stride; key.s[2] = bo_stride; key.b0 = b0; key.b1 = b1; key.dt = (int)dt;
  {
    std::lock_guard<std::mutex> g(g_map_mu);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) { *out = it->second; return Status::OK(); }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return Status::compute("cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[4] = {inner, rows, nbi, nbo};
  uint64_t s1 = row_stride * 2;
  uint64_t s2 = (nbi > 1 ? bi_stride : rows * row_stride) * 2;
  uint64_t s3 = (nbo > 1 ? bo_stride : (nbi > 1 ? nbi * bi_stride : rows * row_stride)) * 2;
  cuuint64_t gstride[3] = {s1, s2, s3};
  cuuint32_t box[4] = {b0, b1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType cdt = dt == DType::BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(out, cdt, 4, const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Status::compute("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  {
    std::lock_guard<std::mutex> g(g_map_mu);
    if (g_map_cache.size() > 4096) g_map_cache.clear();
    g_map_cache.emplace(key, *out);
  }
  return Status::OK();
}

// Map over an int8 [rows, inner] matrix (bytes; 64-byte swizzle, box {b0 bytes, b1 rows}): the raw weight tiles of
// the int8-weight kernel.
static Status make_map_u8(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t rows, uint64_t row_stride, uint32_t b0, uint32_t b1) {
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr; key.d[0] = inner; key.d[1] = rows; key.s[0] = row_stride; key.b0 = b0; key.b1 = b1; key.dt = (int)DType::I8;
  {
    std::lock_guard<std::mutex> g(g_map_mu);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) { *out = it->second; return Status::OK(); }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return Status::compute("cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[4] = {inner, rows, 1, 1};
  cuuint64_t gstride[3] = {row_stride, rows * row_stride, rows * row_stride};
  cuuint32_t box[4] = {b0, b1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Status::compute("cuTensorMapEncodeTiled (int8) failed with code " + std::to_string((int)r));
  {
    std::lock_guard<std::mutex> g(g_map_mu);
    g_map_cache.emplace(key, *out);
  }
  return Status::OK();
}

// 0 = not expressible, 1 = K-major ([N,K] rows), 2 = N-major ([K,N] rows).
static int classify_b(const GemmDesc& d) {
  if (d.b_row == 1 && d.b_col % 8 == 0 && d.b_col >= d.k) return 1;
  if (d.b_col == 1 && d.b_row % 8 == 0 && d.b_row >= d.n) return 2;
  return 0;
}

// int8 weights [N, K] (contiguous rows of K bytes, K a multiple of 16, 16-byte aligned) against 16-bit activations with
// more than one row block: the CTA-pair kernel widens them in its prologue.
bool matmul_w8_fused_eligible(const GemmDesc& d) {
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16) || d.b_dtype != DType::I8) return false;
  if (d.batch != 1 || d.batch_inner != 1 || d.c_f32 || d.ep.argmax_keys || !d.ep.b_scales) return false;
  if (d.m <= BM || d.n < 1 || d.k < 16 || d.k % 16 != 0) return false;
  if (d.m > 0x7fffffff || d.n > 0x7fffffff || d.k > 0x7fffffff) return false;
  if (d.b_row != 1 || d.b_col != d.k) return false;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(d.a) || !al16(d.b)) return false;
  if (d.a_col != 1 || d.a_row % 8 != 0 || d.a_row < d.k) return false;
  return g_w8_fused == 1 || (g_w8_fused == 2 && d.m <= kW8FusedMaxRows);
}

static bool tc_eligible(const GemmDesc& d) {
  if (matmul_w8_fused_eligible(d)) return true;
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16) || d.b_dtype != d.dtype) return false;
  if (d.m < 1 || d.n < 1 || d.k < 1 || d.batch < 1 || d.batch_inner < 1) return false;
  if (d.m > 0x7fffffff || d.n > 0x7fffffff || d.k > 0x7fffffff || d.batch * d.batch_inner > 0x7fffffff) return false;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(d.a) || !al16(d.b)) return false;
  // A must be K-major with 16-byte aligned rows; batch strides 16-byte aligned (0 = broadcast).
  if (d.a_col != 1 || d.a_row % 8 != 0 || d.a_row < d.k) return false;
  if (d.batch > 1 && d.a_batch % 8 != 0) return false;
  if (d.batch_inner > 1 && d.a_batch_inner % 8 != 0) return false;
  if (classify_b(d) == 0) return false;
  if (d.batch > 1 && d.b_batch % 8 != 0) return false;
  if (d.batch_inner > 1 && d.b_batch_inner % 8 != 0) return false;
  return true;
}

Status matmul_simt(cudaStream_t s, const GemmDesc& d);
bool skinny_eligible(const GemmDesc& d);
Status matmul_skinny(cudaStream_t s, const GemmDesc& d);
bool skinny_kmajor_eligible(const GemmDesc& d);
Status matmul_skinny_kmajor(cudaStream_t s, const GemmDesc& d);

int* matmul_status_word();            // workspace.cu: created with the device context

template <int BN, bool B_MN, typename T>
static Status launch_tc(cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, long long num_tiles) {
  using Cfg = TcCfg<BN>;
  static bool attr_set = false;
  auto kern = gemm_tc_kernel<BN, B_MN, T>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return cuda_status(e, "matmul (tcgen05) smem attribute");
    attr_set = true;
  }
  int grid = (int)(num_tiles < sm_count() ? num_tiles : sm_count());
  cudaError_t le = launch_pdl(kern, dim3(grid), dim3(kTcThreads), Cfg::kSmemBytes, s, ma, mb, p);
  if (le != cudaSuccess) return cuda_status(le, "matmul (tcgen05)");
  return Status::OK();
}

// Clusters of two CTAs (one CTA per SM) that can be resident at once; 0 if the query fails.
template <int BN, bool B_MN, typename T>
static int pair_clusters() {
  static int cached = -1;
  if (cached >= 0) return cached;
  using Cfg = PairCfg<BN>;
  auto kern = gemm_tc_pair_kernel<BN, B_MN, T>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) { cudaGetLastError(); return cached = 0; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * (sm_count() / 2)), 1, 1);
  cfg.blockDim = dim3(kTcThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  if (n > sm_count() / 2) n = sm_count() / 2;
  return cached = n;
}

template <int BN, bool B_MN, typename T>
static Status launch_tc_pair(cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, long long num_tiles) {
  int clusters = pair_clusters<BN, B_MN, T>();
  if (clusters <= 0) return Status::compute("matmul (tcgen05, CTA pairs): no resident cluster available");
  int grid = 2 * (int)(num_tiles < clusters ? num_tiles : clusters);
  cudaError_t le = launch_pdl(gemm_tc_pair_kernel<BN, B_MN, T>, dim3(grid), dim3(kTcThreads), PairCfg<BN>::kSmemBytes, s, ma, mb, p);
  if (le != cudaSuccess) return cuda_status(le, "matmul (tcgen05, CTA pairs)");
  return Status::OK();
}

template <typename T>
static Status launch_tc_pair_w8(cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, long long num_tiles) {
  static int clusters = -1;
  auto kern = gemm_tc_pair_kernel<256, false, T, true>;
  if (clusters < 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<256>::kSmemBytes) != cudaSuccess) { cudaGetLastError(); clusters = 0; }
    else {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(2 * (sm_count() / 2)), 1, 1);
      cfg.blockDim = dim3(kTcThreadsW8, 1, 1);
      cfg.dynamicSmemBytes = PairCfg<256>::kSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
      cfg.attrs = &attr; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
      clusters = n > sm_count() / 2 ? sm_count() / 2 : n;
    }
  }
  if (clusters <= 0) return Status::compute("matmul (tcgen05, int8 weights): no resident cluster available");
  int grid = 2 * (int)(num_tiles < clusters ? num_tiles : clusters);
  cudaError_t le = launch_pdl(kern, dim3(grid), dim3(kTcThreadsW8), PairCfg<256>::kSmemBytes, s, ma, mb, p);
  if (le != cudaSuccess) return cuda_status(le, "matmul (tcgen05, int8 weights)");
  return Status::OK();
}

#ifdef AG_GEMM_PROBE
long long* g_tc_probe = nullptr;   // set by the probe harness; the kernel then records where its cycles go
#endif
static int g_force_path = 0;   // 0 auto, 1 simt, 2 tcgen05 (error if not eligible), 3 single-CTA tiles only, 4 CTA-pair tiles where they apply

// Tile shape by modelled cost. A candidate is a CTA-pair tile (256 x 256 or 256 x 128, one tile per two SMs) or a
// single-CTA tile (128 x 256 / 192 / 128). Cost = full waves of the persistent grid x k-steps x the measured
// main-loop cycles per 64-deep k-step of that shape, plus the exposed epilogue of a CTA's last tile. The pair
// tiles run their main loop at the tensor rate (they fetch a third less operand data per flop from L2) and win
// wherever they fill their waves; the single-CTA tiles win where the coarser pair grid would leave a mostly idle last
// wave (N = 768 with M = 8192).
struct TileChoice { bool pair; int bn; };
static bool g_direct_store = [] { const char* v = std::getenv("APPLEGPU_GEMM_DIRECT_STORE"); return !(v && v[0] == '0'); }();   // APPLEGPU_GEMM_DIRECT_STORE=0: always transpose results through shared memory
static int g_tile_override = 0;   // APPLEGPU_GEMM_TILE / set_gemm_tile: 0 auto, else pair*1000 + bn
static TileChoice choose_tile(const GemmDesc& d, long long nb, int force_path) {
  struct Cand { bool pair; int bn; int step; };
  // cycles per k-step (64 deep) of one CTA's tile, measured on a B200 with the kernel's own cycle probes (pair 192:
  // interpolated). The 256 x 192 pair tile exists for K-major B only: each CTA loads half of the B tile, and 96 columns
  // are not a whole number of 64-column swizzle atoms of an N-major operand.
  static const Cand cands[6] = {{true, 256, 530}, {true, 192, 465}, {true, 128, 400}, {false, 256, 780}, {false, 192, 640}, {false, 128, 590}};
  const bool b_kmajor = classify_b(d) != 2;
  const long long num_kb = (d.k + BK - 1) / BK;
  const bool pair_ok = d.m > BM && force_path != 3;
  if (g_tile_override) {
    TileChoice t{g_tile_override >= 1000, g_tile_override % 1000};
    if ((!t.pair || pair_ok) && !(t.pair && t.bn == 192 && !b_kmajor)) return t;
  }
  TileChoice best{false, 128};
  long long best_cost = -1;
  for (const Cand& c : cands) {
    if (c.pair && !pair_ok) continue;
    if (c.pair && c.bn == 192 && !b_kmajor) continue;
    if (!c.pair && force_path == 4 && pair_ok) continue;
    if (c.bn != 128 && d.n <= 128) continue;
    const long long bm = c.pair ? 2 * BM : BM;
    const long long units = c.pair ? sm_count() / 2 : sm_count();
    const long long tiles = ((d.m + bm - 1) / bm) * ((d.n + c.bn - 1) / c.bn) * nb;
    const long long waves = (tiles + units - 1) / units;
    const long long cost = waves * num_kb * c.step + 1500 + 26 * c.bn;   // fill + the last tile's exposed epilogue
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = TileChoice{c.pair, c.bn}; }
  }
  return best;
}

Status matmul_tc(cudaStream_t s, const GemmDesc& d, int* status_word) {
  const bool w8 = d.b_dtype == DType::I8;
  const bool b_mn = !w8 && classify_b(d) == 2;
  const long long nb = d.batch * d.batch_inner;
  const TileChoice tile = w8 ? TileChoice{true, 256} : choose_tile(d, nb, g_force_path);
  const bool use_pair = tile.pair;
  const int bn = tile.bn;
  long long tiles_m = use_pair ? (d.m + 2 * BM - 1) / (2 * BM) : (d.m + BM - 1) / BM;
  long long tiles_n = (d.n + bn - 1) / bn;
  CUtensorMap ma, mb;
  // A broadcast (stride-0) batch level is mapped as extent 1 and its coordinate pinned to 0.
  int a_bcast = ((d.batch > 1 && d.a_batch == 0) ? 1 : 0) | ((d.batch_inner > 1 && d.a_batch_inner == 0) ? 2 : 0);
  int b_bcast = ((d.batch > 1 && d.b_batch == 0) ? 1 : 0) | ((d.batch_inner > 1 && d.b_batch_inner == 0) ? 2 : 0);
  uint64_t a_nbo = (a_bcast & 1) ? 1 : (uint64_t)d.batch, a_nbi = (a_bcast & 2) ? 1 : (uint64_t)d.batch_inner;
  uint64_t b_nbo = (b_bcast & 1) ? 1 : (uint64_t)d.batch, b_nbi = (b_bcast & 2) ? 1 : (uint64_t)d.batch_inner;
  AG_RETURN_IF_ERROR(make_map(&ma, d.dtype, d.a, (uint64_t)d.k, (uint64_t)d.m, a_nbi, a_nbo, (uint64_t)d.a_row,
                              (uint64_t)d.a_batch_inner, (uint64_t)d.a_batch, BK, BM));
  if (w8) {
    AG_RETURN_IF_ERROR(make_map_u8(&mb, d.b, (uint64_t)d.k, (uint64_t)d.n, (uint64_t)d.b_col, BK, (uint32_t)(bn / 2)));
  } else if (!b_mn) {
    AG_RETURN_IF_ERROR(make_map(&mb, d.dtype, d.b, (uint64_t)d.k, (uint64_t)d.n, b_nbi, b_nbo, (uint64_t)d.b_col,
                                (uint64_t)d.b_batch_inner, (uint64_t)d.b_batch, BK, (uint32_t)(use_pair ? bn / 2 : bn)));
  } else {
    AG_RETURN_IF_ERROR(make_map(&mb, d.dtype, d.b, (uint64_t)d.n, (uint64_t)d.k, b_nbi, b_nbo, (uint64_t)d.b_row,
                                (uint64_t)d.b_batch_inner, (uint64_t)d.b_batch, 64, BK));
  }
  TcParams p;
  p.c = d.c; p.bias = d.ep.bias; p.residual = d.ep.residual; p.b_scales = d.ep.b_scales; p.alpha = d.ep.alpha; p.act = (int)d.ep.act;
  p.m = (int)d.m; p.n = (int)d.n; p.k = (int)d.k; p.batch = (int)nb; p.batch_inner = (int)d.batch_inner;
  p.c_row = d.c_row; p.c_batch = d.c_batch; p.c_batch_inner = d.c_batch_inner; p.a_bcast = a_bcast; p.b_bcast = b_bcast;
  p.tiles_m = (int)tiles_m; p.tiles_n = (int)tiles_n; p.status = status_word;
  p.argmax_keys = d.ep.argmax_keys;
  p.c_f32 = d.c_f32 ? 1 : 0;
  p.ln_stats = d.ep.ln_stats; p.ln_colsum = d.ep.ln_colsum; p.ln_inv_k = d.k ? 1.0f / (float)d.k : 0.f; p.ln_eps = d.ep.ln_eps;
  p.stats_out = d.ep.stats_out; p.stats_zero = d.ep.stats_zero;
#ifdef AG_GEMM_PROBE
  p.probe = g_tc_probe;
#endif
  if (p.argmax_keys && nb != 1) return Status::invalid("matmul: the row-argmax epilogue takes an unbatched product");
  auto al16p = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  const int64_t cvec = d.c_f32 ? 4 : 8;   // elements per 16 bytes of C
  p.vec_ok = (al16p(d.c) && d.c_row % cvec == 0 && d.c_batch % cvec == 0 && d.c_batch_inner % cvec == 0 &&
              (!d.ep.residual || al16p(d.ep.residual))) ? 1 : 0;
  // 16-bit C whose rows (and batch strides, and residual) are 32-byte aligned: one row per lane, 256-bit accesses
  auto al32p = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31u) == 0; };
  if (p.vec_ok && !d.c_f32 && g_direct_store && al32p(d.c) && d.c_row % 16 == 0 && d.c_batch % 16 == 0 && d.c_batch_inner % 16 == 0 &&
      (!d.ep.residual || al32p(d.ep.residual)))
    p.vec_ok = 2;
  p.bias_vec = (d.ep.bias && al16p(d.ep.bias)) ? 1 : 0;
  long long num_tiles = tiles_m * tiles_n * nb;
  if (w8) return d.dtype == DType::BF16 ? launch_tc_pair_w8<__nv_bfloat16>(s, ma, mb, p, num_tiles) : launch_tc_pair_w8<__half>(s, ma, mb, p, num_tiles);
#define AG_TCP(BNV, MN) \
  (d.dtype == DType::BF16 ? launch_tc_pair<BNV, MN, __nv_bfloat16>(s, ma, mb, p, num_tiles) : launch_tc_pair<BNV, MN, __half>(s, ma, mb, p, num_tiles))
  if (use_pair) {
    if (bn == 256) return b_mn ? AG_TCP(256, true) : AG_TCP(256, false);
    if (bn == 192 && !b_mn) return AG_TCP(192, false);
    return b_mn ? AG_TCP(128, true) : AG_TCP(128, false);
  }
#undef AG_TCP
#define AG_TC(BNV, MN) \
  (d.dtype == DType::BF16 ? launch_tc<BNV, MN, __nv_bfloat16>(s, ma, mb, p, num_tiles) : launch_tc<BNV, MN, __half>(s, ma, mb, p, num_tiles))
  if (bn == 256) return b_mn ? AG_TC(256, true) : AG_TC(256, false);
  if (bn == 192) return b_mn ? AG_TC(192, true) : AG_TC(192, false);
  return b_mn ? AG_TC(128, true) : AG_TC(128, false);
#undef AG_TC
}

// ── chained products, host side ─────────────────────────────────────────────
#ifdef AG_CHAIN_PROBE
long long* g_chain_probe = nullptr;   // set by a probe harness
void chain_epi_probe(long long* out) { cudaMemcpyFromSymbol(out, g_epi_probe, sizeof(long long) * 8); }
#endif
// Fewer rows than this and the products go out one by one: with a handful of 256-row blocks most tiles wait for the
// tiles just before them (measured on GPT-2-small's block: chained 66 / 76 / 83 / 114 us against 54 / 72 / 86 / 145 us
// for four launches at 1024 / 3072 / 4096 / 8192 rows).
static int64_t g_chain_min_rows = [] { const char* v = std::getenv("APPLEGPU_GEMM_CHAIN_MIN_ROWS"); return v ? (int64_t)std::atoll(v) : (int64_t)4096; }();
void set_gemm_chain_min_rows(int64_t rows) { g_chain_min_rows = rows < 0 ? 0 : rows; }
int64_t gemm_chain_min_rows() { return g_chain_min_rows; }

bool matmul_chain_candidate(const GemmDesc& d) {
  if (g_force_path == 1 || g_force_path == 3 || g_tile_override) return false;
  if (d.m < g_chain_min_rows) return false;
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16) || d.b_dtype != d.dtype) return false;
  if (!tc_eligible(d) || classify_b(d) != 2) return false;
  if (d.batch != 1 || d.batch_inner != 1 || d.c_f32 || d.ep.argmax_keys || d.ep.b_scales || d.ln_gamma) return false;
  if (d.ep.ln_stats && !d.ep.ln_colsum) return false;
  if (d.m <= BM || !d.c) return false;
  // C (and residual) rows 32-byte aligned: the epilogue's one-row-per-lane layout, the only one the chained kernel has
  auto al32 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31u) == 0; };
  if (!g_direct_store || !al32(d.c) || d.c_row % 16 != 0 || (d.ep.residual && !al32(d.ep.residual))) return false;
  const long long tiles_m = (d.m + 2 * BM - 1) / (2 * BM), tiles_n = (d.n + 255) / 256;
  return tiles_m <= kChainFlagStride && tiles_m * tiles_n < (1 << 24);
}

namespace {
// What a product reads and writes, as byte ranges. Row-wise buffers (activations, statistics) may be shared between the
// products of a chain when they are the SAME rows (same base, pitch and width): row block m of a later product only
// runs after row block m of every earlier one. Anything else that overlaps a written buffer is refused.
enum ChainBufKind { kBufA, kBufB, kBufBias, kBufResidual, kBufColsum, kBufLnStats, kBufC, kBufStatsOut, kBufStatsZero };
struct ChainBuf { const uint8_t* lo; const uint8_t* hi; ChainBufKind kind; int64_t pitch, width; bool written, rowwise; };
int chain_bufs(const GemmDesc& d, ChainBuf* out) {
  int n = 0;
  auto add = [&](const void* p, int64_t bytes, ChainBufKind kind, int64_t pitch, int64_t width, bool written, bool rowwise) {
    if (!p) return;
    const uint8_t* lo = static_cast<const uint8_t*>(p);
    out[n++] = ChainBuf{lo, lo + bytes, kind, pitch, width, written, rowwise};
  };
  add(d.a, ((d.m - 1) * d.a_row + d.k) * 2, kBufA, d.a_row, d.k, false, true);
  add(d.b, ((d.k - 1) * d.b_row + d.n) * 2, kBufB, d.b_row, d.n, false, false);
  add(d.ep.bias, d.n * 2, kBufBias, 0, d.n, false, false);
  add(d.ep.residual, ((d.m - 1) * d.c_row + d.n) * 2, kBufResidual, d.c_row, d.n, false, true);
  add(d.ep.ln_colsum, d.n * 4, kBufColsum, 0, d.n, false, false);
  add(d.ep.ln_stats, d.m * 16, kBufLnStats, 2, 2, false, true);
  add(d.c, ((d.m - 1) * d.c_row + d.n) * 2, kBufC, d.c_row, d.n, true, true);
  add(d.ep.stats_out, d.m * 16, kBufStatsOut, 2, 2, true, true);
  add(d.ep.stats_zero, d.m * 16, kBufStatsZero, 2, 2, true, true);
  return n;
}
bool chain_same_rows(const ChainBuf& x, const ChainBuf& y) {
  return x.rowwise && y.rowwise && x.lo == y.lo && x.pitch == y.pitch && x.width == y.width;
}
}  // namespace

bool matmul_chain_can_append(const GemmDesc* chain, int count, const GemmDesc& next) {
  if (count < 1 || count >= kChainMax || !matmul_chain_candidate(next)) return false;
  const GemmDesc& prev = chain[count - 1];
  if (next.dtype != chain[0].dtype || next.m != chain[0].m) return false;
  if (next.a != prev.c || next.a_row != prev.c_row || next.k != prev.n) return false;
  ChainBuf nb[9], hb[9];
  const int nn = chain_bufs(next, nb);
  for (int h = 0; h < count; h++) {
    const int hn = chain_bufs(chain[h], hb);
    for (int i = 0; i < nn; i++) {
      for (int j = 0; j < hn; j++) {
        const ChainBuf& x = nb[i];
        const ChainBuf& y = hb[j];
        if (!(x.written || y.written) || x.hi <= y.lo || y.hi <= x.lo) continue;
        if (!chain_same_rows(x, y)) return false;
        if (x.kind == kBufA && !(h == count - 1 && y.kind == kBufC)) return false;   // A is the previous result and nothing else
        if (x.kind == kBufC && y.kind == kBufC) return false;
        if (x.kind == kBufStatsOut && (y.kind == kBufStatsOut || y.kind == kBufLnStats)) return false;
      }
    }
  }
  return true;
}

namespace {
struct ChainListKey {
  int64_t m; int count, clusters; int64_t n[kChainMax], k[kChainMax]; int cost[kChainMax];
  bool operator==(const ChainListKey& o) const { return std::memcmp(this, &o, sizeof(ChainListKey)) == 0; }
};
struct ChainList { ChainListKey key; int off_ints; int total; std::vector<int> host; };
std::mutex g_chain_mu;
std::deque<ChainList> g_chain_lists;     // deque: the host copies stay where they are while an upload may still read them
int g_chain_arena_used = 0;

const int g_chain_kstep = [] { const char* v = std::getenv("APPLEGPU_CHAIN_KSTEP"); return v ? std::atoi(v) : 520; }();
const int g_chain_epi_base = [] { const char* v = std::getenv("APPLEGPU_CHAIN_EPI_BASE"); return v ? std::atoi(v) : 11000; }();
// Modelled cycles of one tile, for dealing the tiles out evenly: the main loop at the tensor rate, or the epilogue where
// that is longer (K = 768). Measured on a GPT-2-small block: 123.7 / 121.4 / 117.4 / 117.2 us with an epilogue base of
// 5 200 / 8 000 / 11 000 / 15 000 cycles (what matters is the weight of the 48-step FC2 tiles against the 12-step ones:
// about 2 : 1, the epilogue being what bounds the short ones); the k-step cost makes no difference between 420 and 620.
// APPLEGPU_CHAIN_EPI_BASE / APPLEGPU_CHAIN_KSTEP override the two for tuning.
int chain_tile_cost(const GemmDesc& d) {
  const int num_kb = (int)((d.k + BK - 1) / BK);
  int epi = g_chain_epi_base;
  if (d.ep.act != Act::None) epi += 1500;
  if (d.ep.residual) epi += 800;
  if (d.ep.ln_stats) epi += 300;
  if (d.ep.stats_out) epi += 400;
  const int main_loop = num_kb * g_chain_kstep;
  return main_loop > epi ? main_loop : epi;
}

// The tiles of all products in dependency order (product by product, row block by row block), each given to the pair
// that has the least modelled work so far. Returns the device address of [offsets (clusters + 1) | entries].
Status chain_list_for(cudaStream_t s, const GemmDesc* chain, int count, int clusters, const int** d_off, const int** d_list) {
  ChainListKey key;
  std::memset(&key, 0, sizeof(key));
  key.m = chain[0].m; key.count = count; key.clusters = clusters;
  for (int g = 0; g < count; g++) { key.n[g] = chain[g].n; key.k[g] = chain[g].k; key.cost[g] = chain_tile_cost(chain[g]); }
  int* arena = chain_arena();
  if (!arena) return Status::compute("matmul: the kernel workspace is not initialised");
  std::lock_guard<std::mutex> lock(g_chain_mu);
  for (const ChainList& l : g_chain_lists) {
    if (l.key == key) { *d_off = arena + l.off_ints; *d_list = arena + l.off_ints + clusters + 1; return Status::OK(); }
  }
  const int64_t tiles_m = (chain[0].m + 2 * BM - 1) / (2 * BM);
  int64_t total = 0;
  for (int g = 0; g < count; g++) total += tiles_m * ((chain[g].n + 255) / 256);
  const int64_t ints = clusters + 1 + total;
  if (ints > kChainArenaInts) return Status::unsupported("matmul: chained products with too many tiles");
  if (g_chain_arena_used + ints > kChainArenaInts) {
    // start over; launches that read the old lists are ahead of the upload below in stream order
    g_chain_lists.clear();
    g_chain_arena_used = 0;
  }
  // Global order = product after product, row block after row block. (A wavefront over groups of row blocks, so that
  // consumers trail their producers by a step, was measured slower: 123 us per GPT-2-small layer with one group, 141 /
  // 177 / 258 us with 4 / 8 / 16: with a few tiles per pair and step every step boundary becomes a dependency stall.)
  std::vector<std::vector<int>> per(clusters);
  std::vector<long long> load(clusters, 0);
  for (int g = 0; g < count; g++) {
    const int64_t tn = (chain[g].n + 255) / 256;
    for (int64_t t = 0; t < tiles_m * tn; t++) {
      int best = 0;
      for (int c = 1; c < clusters; c++) if (load[c] < load[best]) best = c;
      per[best].push_back((g << 24) | (int)t);
      load[best] += key.cost[g];
    }
  }
  g_chain_lists.emplace_back();
  ChainList& l = g_chain_lists.back();
  l.key = key; l.off_ints = g_chain_arena_used; l.total = (int)total;
  l.host.reserve((size_t)ints);
  int run = 0;
  for (int c = 0; c < clusters; c++) { l.host.push_back(run); run += (int)per[c].size(); }
  l.host.push_back(run);
  for (int c = 0; c < clusters; c++) l.host.insert(l.host.end(), per[c].begin(), per[c].end());
  cudaError_t e = cudaMemcpyAsync(arena + l.off_ints, l.host.data(), (size_t)ints * sizeof(int), cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) { g_chain_lists.pop_back(); return cuda_status(e, "matmul (chained): tile list upload"); }
  g_chain_arena_used += (int)ints;
  *d_off = arena + l.off_ints; *d_list = arena + l.off_ints + clusters + 1;
  return Status::OK();
}

template <typename T>
int chain_clusters() {
  static int cached = -1;
  if (cached >= 0) return cached;
  auto kern = gemm_tc_chain_kernel<T>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<256>::kSmemBytes) != cudaSuccess) { cudaGetLastError(); return cached = 0; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * (sm_count() / 2)), 1, 1);
  cfg.blockDim = dim3(kChainThreads, 1, 1);
  cfg.dynamicSmemBytes = PairCfg<256>::kSmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  return cached = n;
}
}  // namespace

Status matmul_chain(cudaStream_t s, const GemmDesc* chain, int count) {
  if (count < 2 || count > kChainMax) return Status::invalid("matmul (chained): 2.." + std::to_string(kChainMax) + " products");
  for (int g = 0; g < count; g++) {
    if (!matmul_chain_candidate(chain[g])) return Status::invalid("matmul (chained): product " + std::to_string(g) + " cannot be chained");
    if (g > 0 && !matmul_chain_can_append(chain, g, chain[g])) return Status::invalid("matmul (chained): product " + std::to_string(g) + " does not follow the one before");
  }
  int* st = matmul_status_word();
  int* flags = chain_flags();
  if (!st || !flags) return Status::compute("matmul: the kernel workspace is not initialised");
  const bool bf16 = chain[0].dtype == DType::BF16;
  int clusters = bf16 ? chain_clusters<__nv_bfloat16>() : chain_clusters<__half>();
  if (clusters > sm_count() / 2) clusters = sm_count() / 2;   // sm_count() leaves out the SMs kept free for a collective
  if (clusters <= 0) return Status::compute("matmul (chained): no resident cluster available");
  ChainMaps maps;
  ChainParams cp;
  std::memset(&cp, 0, sizeof(cp));
  cp.count = count;
  cp.flags = flags;
#ifdef AG_CHAIN_PROBE
  cp.probe = g_chain_probe;
#endif
  const int64_t tiles_m = (chain[0].m + 2 * BM - 1) / (2 * BM);
  auto al16p = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  auto al32p = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31u) == 0; };
  for (int g = 0; g < count; g++) {
    const GemmDesc& d = chain[g];
    AG_RETURN_IF_ERROR(make_map(&maps.a[g], d.dtype, d.a, (uint64_t)d.k, (uint64_t)d.m, 1, 1, (uint64_t)d.a_row, 0, 0, BK, BM));
    AG_RETURN_IF_ERROR(make_map(&maps.b[g], d.dtype, d.b, (uint64_t)d.n, (uint64_t)d.k, 1, 1, (uint64_t)d.b_row, 0, 0, 64, BK));
    TcParams& p = cp.prob[g];
    p.c = d.c; p.bias = d.ep.bias; p.residual = d.ep.residual; p.b_scales = nullptr; p.alpha = d.ep.alpha; p.act = (int)d.ep.act;
    p.m = (int)d.m; p.n = (int)d.n; p.k = (int)d.k; p.batch = 1; p.batch_inner = 1;
    p.c_row = d.c_row; p.c_batch = 0; p.c_batch_inner = 0; p.a_bcast = 0; p.b_bcast = 0;
    p.tiles_m = (int)tiles_m; p.tiles_n = (int)((d.n + 255) / 256); p.status = st;
    p.argmax_keys = nullptr; p.c_f32 = 0;
    p.ln_stats = d.ep.ln_stats; p.ln_colsum = d.ep.ln_colsum; p.ln_inv_k = d.k ? 1.0f / (float)d.k : 0.f; p.ln_eps = d.ep.ln_eps;
    p.stats_out = d.ep.stats_out; p.stats_zero = d.ep.stats_zero;
#ifdef AG_GEMM_PROBE
    p.probe = nullptr;
#endif
    p.vec_ok = (al16p(d.c) && d.c_row % 8 == 0 && (!d.ep.residual || al16p(d.ep.residual))) ? 1 : 0;
    if (p.vec_ok && g_direct_store && al32p(d.c) && d.c_row % 16 == 0 && (!d.ep.residual || al32p(d.ep.residual))) p.vec_ok = 2;
    p.bias_vec = (d.ep.bias && al16p(d.ep.bias)) ? 1 : 0;
    cp.need[g] = g == 0 ? 0 : 2 * kChainEpiWarps * cp.prob[g - 1].tiles_n;   // every epilogue warp of both CTAs, every tile of the row block
  }
  AG_RETURN_IF_ERROR(chain_list_for(s, chain, count, clusters, &cp.list_off, &cp.list));
  cudaError_t le = bf16 ? launch_pdl(gemm_tc_chain_kernel<__nv_bfloat16>, dim3(2 * clusters), dim3(kChainThreads), PairCfg<256>::kSmemBytes, s, maps, cp)
                        : launch_pdl(gemm_tc_chain_kernel<__half>, dim3(2 * clusters), dim3(kChainThreads), PairCfg<256>::kSmemBytes, s, maps, cp);
  if (le != cudaSuccess) return cuda_status(le, "matmul (tcgen05, chained)");
  return Status::OK();
}

// APPLEGPU_MATMUL_PATH=simt|tcgen05|tcgen05_1cta|tcgen05_pair sets the initial value of the path switch.
static int initial_force_path() {
  const char* v = std::getenv("APPLEGPU_MATMUL_PATH");
  if (!v) return 0;
  if (std::strcmp(v, "simt") == 0) return 1;
  if (std::strcmp(v, "tcgen05") == 0) return 2;
  if (std::strcmp(v, "tcgen05_1cta") == 0) return 3;
  if (std::strcmp(v, "tcgen05_pair") == 0) return 4;
  return 0;
}
static const int g_force_path_init = (g_force_path = initial_force_path());
void set_matmul_path(int mode) { g_force_path = mode; }
// APPLEGPU_GEMM_TILE=pair256|pair192|pair128|s256|s192|s128 pins the tile shape of the tensor-core kernel (a tuning override).
static int initial_tile_override() {
  const char* v = std::getenv("APPLEGPU_GEMM_TILE");
  if (!v) return 0;
  if (std::strcmp(v, "pair256") == 0) return 1256;
  if (std::strcmp(v, "pair192") == 0) return 1192;   // K-major B only
  if (std::strcmp(v, "pair128") == 0) return 1128;
  if (std::strcmp(v, "s256") == 0) return 256;
  if (std::strcmp(v, "s192") == 0) return 192;
  if (std::strcmp(v, "s128") == 0) return 128;
  return 0;
}
static const int g_tile_override_init = (g_tile_override = initial_tile_override());
void set_gemm_tile(int code) { g_tile_override = code; }

const char* matmul_path(const GemmDesc& d) {
  if (g_force_path == 1) return "simt";
  return tc_eligible(d) ? "tcgen05" : "simt";
}

__global__ void argmax_finalize_kernel(const unsigned long long* __restrict__ keys, int32_t* __restrict__ out, int64_t rows) {
  pdl_wait();
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  unsigned long long k = keys[i];
  // no key (an all-NaN row) and the sticky-NaN key both mean column 0
  out[i] = (k == 0ull || k == 0xffffffffffffffffull) ? 0 : (int32_t)(0xffffffffu - (uint32_t)(k & 0xffffffffu));
}
Status argmax_finalize(cudaStream_t s, const unsigned long long* keys, int32_t* out, int64_t rows) {
  if (rows == 0) return Status::OK();
  cudaError_t e = launch_pdl(argmax_finalize_kernel, dim3((unsigned)((rows + 255) / 256)), dim3(256), 0, s, keys, out, rows);
  if (e != cudaSuccess) return cuda_status(e, "argmax_finalize");
  return Status::OK();
}

Status matmul(cudaStream_t s, const GemmDesc& d) {
  if (d.m == 0 || d.n == 0 || d.batch == 0) return Status::OK();
  if (d.ln_gamma) {
    if (!skinny_kmajor_eligible(d)) return Status::invalid("matmul: the layer_norm prologue needs at most 16 rows against a [N, K] weight");
    return matmul_skinny_kmajor(s, d);
  }
  bool elig = tc_eligible(d);
  if (d.ep.argmax_keys && (!elig || g_force_path == 1)) return Status::invalid("matmul: the row-argmax epilogue needs the tensor-core kernel");
  if (d.ep.ln_stats || d.ep.stats_out || d.ep.stats_zero) {
    if (!elig || g_force_path == 1 || d.batch != 1 || d.batch_inner != 1 || d.c_f32 || d.ep.argmax_keys || d.ep.b_scales || (d.ep.ln_stats && !d.ep.ln_colsum))
      return Status::invalid("matmul: the folded layer_norm epilogue needs an unbatched 16-bit product on the tensor-core kernel");
    int* st = matmul_status_word();
    if (!st) return Status::compute("matmul: the kernel workspace is not initialised");
    return matmul_tc(s, d, st);
  }
  // a handful of rows against a [K, N] weight: bound by streaming B, spread over every SM
  if (g_force_path == 0 && skinny_eligible(d)) return matmul_skinny(s, d);
  // the same against a [N, K] weight; 16-bit products that large keep the tensor-core kernel (it is as fast there and
  // feeds the fused argmax), float32 ones would otherwise fall to the CUDA-core tile kernel
  if (g_force_path == 0 && d.dtype == DType::F32 && skinny_kmajor_eligible(d)) return matmul_skinny_kmajor(s, d);
  if (g_force_path == 2 && !elig) return Status::compute("matmul: tcgen05 path forced but operands are not TMA-compatible");
  if (elig && g_force_path != 1) {
    int* st = matmul_status_word();
    if (!st) return Status::compute("matmul: the kernel workspace is not initialised");
    return matmul_tc(s, d, st);
  }
  return matmul_simt(s, d);
}

// Same dispatch with a caller-provided status word: performs no device allocation.
Status matmul_with_status(cudaStream_t s, const GemmDesc& d, int* status_word) {
  if (d.m == 0 || d.n == 0 || d.batch == 0) return Status::OK();
  bool elig = tc_eligible(d);
  if (g_force_path == 2 && !elig) return Status::compute("matmul: tcgen05 path forced but operands are not TMA-compatible");
  if (elig && g_force_path != 1) return matmul_tc(s, d, status_word);
  return matmul_simt(s, d);
}

}}  // namespace ag::k
