// Fused scaled-dot-product attention for head dimension 64 (bf16 / f16): softmax[_causal](Q K^T /
// sqrt(d)) V in one kernel, scores never leave the SM.
//
// Replaces the reference's 5-launch composition (ops.rs:1531-1618: transpose(K), matmul,
// scalar_mul, softmax[_causal], matmul, with [.., Tq, Tk] score tensors materialised three times)
// for the shapes every model on the path uses (GPT-2 small / large and BERT-base all have
// d_head = 64). Semantics kept: mask is `col > row` with rows counted from 0, probabilities are
// rounded to the storage type before the P.V product (the reference stores softmax output in
// the storage type), the row sum is accumulated unrounded in float.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key/value sequence in blocks of
// 128:  S = Q K_j^T (tcgen05, fp32 in TMEM) -> online softmax by 128 threads, one query row each
// (running max / sum in registers, exp2 with the 1/sqrt(d) scale folded in) -> P_j as bf16 into
// shared memory in the 128B-swizzled K-major layout the tensor core reads -> O_j = P_j V_j
// (tcgen05, V read N-major in place) -> O = O * alpha + O_j in registers. Warp roles: warp 0
// TMA producer (Q once, K double-buffered, V single-buffered), warp 1 MMA issuer and TMEM owner,
// warps 2..5 softmax / output. Two CTAs fit per SM (96 KB shared memory, 256 TMEM columns each),
// so one CTA's softmax overlaps the other's MMAs. All waits are bounded.
#include "common.cuh"
#include "sm100.cuh"
#include <cuda.h>
#include <cstdlib>
#include <type_traits>

namespace ag { namespace k {

using namespace ag::sm100;

Status make_map(CUtensorMap* out, DType dt, const void* ptr, uint64_t inner, uint64_t rows, uint64_t nbi, uint64_t nbo,
                uint64_t row_stride, uint64_t bi_stride, uint64_t bo_stride, uint32_t b0, uint32_t b1);
int* matmul_status_word();

constexpr int kAttnThreads = 192;
constexpr int kQ = 128;    // query rows per CTA
constexpr int kKV = 64;    // keys per block
constexpr int kD = 64;     // head dimension
constexpr int kQBytes = kQ * kD * 2;                     // 16 KB
constexpr int kKVBytes = kKV * kD * 2;                   // 8 KB: one K or V block
constexpr int kAttnSmem = kQBytes + 2 * kKVBytes /*K*/ + 2 * kKVBytes /*V*/ + 1024;
constexpr int kAttnTmemCols = 256;                       // S: 2 x 64 (P over the head of each), O: 64

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T> __device__ __forceinline__ uint32_t pack2_t(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2_t<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2_t<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnParams {
  void* o;
  long long o_b, o_h, o_t;   // element strides of the output
  int heads, tq, tk;
  int causal;
  int o_vec;                 // output rows are 16-byte aligned
  float scale_log2;          // (1/sqrt(d)) * log2(e)
  int* status;
};

// How far (in log2 units) the running row maximum may grow before the accumulated output is rescaled.
// Until then probabilities are taken relative to the older, smaller maximum and may reach 2^kRescaleLog2:
// exact in the arithmetic of softmax (numerator and denominator carry the same factor), harmless in
// range (bf16 / f16 probabilities up to 256, fp32 sums), and it keeps the output accumulator in tensor
// memory untouched for almost every block.
constexpr float kRescaleLog2 = 8.0f;

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_full[2];
  __shared__ uint32_t tmem_base_slot;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;            // two stages
  uint8_t* sV = sK + 2 * kKVBytes;       // two stages

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (p.tq + kQ - 1) / kQ;
  // blockIdx.x (the index CTAs are launched along first) runs over (batch, head); blockIdx.y over query
  // tiles, longest causal prefix first: every heavy tile of every head starts before any light one, which
  // is the longest-processing-time order and keeps the last wave short.
  const int qt = q_tiles - 1 - (int)blockIdx.y;
  const int bh = (int)blockIdx.x;
  const int b = bh / p.heads, h = bh % p.heads;
  const int q0 = qt * kQ;
  int n_blocks = (p.tk + kKV - 1) / kKV;
  if (p.causal) {
    int last_col = q0 + kQ - 1;  // the largest column any row of this tile may see
    int nb = last_col / kKV + 1;
    if (nb < n_blocks) n_blocks = nb;
  }

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4);
    }
    mbar_init(&o_full[0], 1); mbar_init(&o_full[1], 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, kAttnTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  // columns 0..127: two S buffers of 64 fp32 columns; P_j (64 keys as 32 packed columns) overwrites the
  // head of the S buffer it was computed from. Columns 128..191: the output accumulator.
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * kKV;
  pdl_wait();      // the prologue above may overlap the tail of the kernel that produces Q, K and V
  pdl_trigger();

  if (warp == 0) {
    // ── TMA producer: Q once, then K and V blocks through two-deep rings ──
    if (lane == 0) {
      mbar_expect_tx(&q_full, kQBytes);
      tma_load_4d(sQ, &tmap_q, &q_full, 0, q0, h, b);
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; j++) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(&k_empty[st], ph ^ 1, p.status, 11)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], kKVBytes);
        tma_load_4d(sK + st * kKVBytes, &tmap_k, &k_full[st], 0, j * kKV, h, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, p.status, 12)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], kKVBytes);
        tma_load_4d(sV + st * kKVBytes, &tmap_v, &v_full[st], 0, j * kKV, h, b);
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer. S_j = Q K_j^T runs two blocks ahead of the softmax (two S buffers); O += P_j V_j
    //    reads P_j from tensor memory and accumulates in tensor memory. MMAs execute in issue order,
    //    so S_{j+2} (issued after P_j V_j) cannot overwrite P_j before that product has read it. ──
    if (lane == 0) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, kQ, kKV);   // S = Q K^T: both K-major, N = 64
      constexpr uint32_t idesc_o = make_idesc_f16(fmt, 0, 1, kQ, kD);    // O = P V: V is N-major, N = 64
      bool ok = mbar_wait(&q_full, 0, p.status, 13);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (uint32_t)((j >> 1) & 1), p.status, 14)) return false;
        tc_fence_after_sync();
        const uint32_t a = smem_u32(sQ), bb = smem_u32(sK + st * kKVBytes);
#pragma unroll
        for (int kk = 0; kk < kD / 16; kk++)
          mma_f16_ss(tmem_s + (uint32_t)(st * kKV), make_smem_desc_sw128(a + kk * 32, 16, 1024), make_smem_desc_sw128(bb + kk * 32, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(&k_empty[st]);
        mma_commit(&s_full[st]);
        return true;
      };
      if (ok && n_blocks > 0) ok = issue_s(0);
      if (ok && n_blocks > 1) ok = issue_s(1);
      for (int j = 0; j < n_blocks && ok; j++) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(&v_full[st], ph, p.status, 16)) { ok = false; break; }
        if (!mbar_wait(&p_full[st], ph, p.status, 17)) { ok = false; break; }   // P_j stored, O rescaled if it had to be
        tc_fence_after_sync();
        const uint32_t bb = smem_u32(sV + st * kKVBytes);
#pragma unroll
        for (int kk = 0; kk < kKV / 16; kk++) {
          // P: 16 keys = 8 packed columns. V: rows are keys (128 B = 64 head dims); 16 keys = 2048 B.
          mma_f16_ts(tmem_o, tmem_s + (uint32_t)(st * kKV + kk * 8), make_smem_desc_sw128(bb + kk * 2048, 64 * 128, 1024), idesc_o,
                     (j > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(&v_empty[st]);
        // Even and odd blocks signal different barriers: a waiter can then be at most one phase behind
        // (P_{j-2} V_{j-2} is always complete before S_j is), so its parity test cannot alias.
        mma_commit(&o_full[st]);
        if (j + 2 < n_blocks) { if (!issue_s(j + 2)) { ok = false; break; } }
      }
    }
  } else {
    // ── softmax / output: thread = query row ──
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;          // row inside the tile = TMEM lane
    const int row = q0 + r;                     // row inside the sequence
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float m_ref = -INFINITY;   // the maximum the stored probabilities and sums are relative to
    float l_run = 0.f;
    const float sc = p.scale_log2;
    bool ok = true;

    for (int j = 0; j < n_blocks && ok; j++) {
      const int st = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[st], ph, p.status, 19))) { ok = false; break; }  // warp-uniform exits
      tc_fence_after_sync();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(tmem_s + lane_addr + (uint32_t)(st * kKV), s0);
      tmem_ld_32x32(tmem_s + lane_addr + (uint32_t)(st * kKV + 32), s1);
      tmem_ld_wait();

      const int col_base = j * kKV;
      // columns this row may see inside the block: [0, lim)
      int lim = p.tk - col_base;
      if (p.causal) { int c = row - col_base + 1; if (c < lim) lim = c; }
      if (lim > kKV) lim = kKV;
      // warp-uniform: selects the mask-free arithmetic below
      const bool full = __all_sync(0xffffffffu, lim >= kKV);
      float m_blk;
      if (!full) {
        // masked columns become -inf once, so both paths share the four-chain maximum below
#pragma unroll
        for (int e = 0; e < 32; e++) {
          if (e >= lim) s0[e] = 0xff800000u;
          if (32 + e >= lim) s1[e] = 0xff800000u;
        }
      }
      {
        float m0 = __uint_as_float(s0[0]), m1 = __uint_as_float(s0[1]), m2 = __uint_as_float(s0[2]), m3 = __uint_as_float(s0[3]);
#pragma unroll
        for (int e = 4; e < 32; e += 4) {
          m0 = fmaxf(m0, __uint_as_float(s0[e])); m1 = fmaxf(m1, __uint_as_float(s0[e + 1]));
          m2 = fmaxf(m2, __uint_as_float(s0[e + 2])); m3 = fmaxf(m3, __uint_as_float(s0[e + 3]));
        }
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          m0 = fmaxf(m0, __uint_as_float(s1[e])); m1 = fmaxf(m1, __uint_as_float(s1[e + 1]));
          m2 = fmaxf(m2, __uint_as_float(s1[e + 2])); m3 = fmaxf(m3, __uint_as_float(s1[e + 3]));
        }
        m_blk = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      // Move the reference maximum only when this row's maximum outgrew it by more than the margin (or
      // when the row sees its first scores); the accumulated output and sum are then rescaled.
      const float m_cand = fmaxf(m_ref, m_blk * sc);
      const bool moves = (m_cand - m_ref > kRescaleLog2) || (m_ref == -INFINITY && m_cand != -INFINITY);
      const float alpha = moves ? ex2_approx(m_ref - m_cand) : 1.0f;      // exp2(-inf) = 0 for a first block
      if (moves) m_ref = m_cand;
      if (j > 0 && __any_sync(0xffffffffu, moves)) {
        // O holds the products up to block j-1: wait for the last of them, scale this row, write it back
        if (!__all_sync(0xffffffffu, mbar_wait(&o_full[(j - 1) & 1], (uint32_t)(((j - 1) >> 1) & 1), p.status, 21))) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < kD / 32; c++) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_o + lane_addr + (uint32_t)(c * 32), ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
          tmem_st_32x32(tmem_o + lane_addr + (uint32_t)(c * 32), ov);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

      // probabilities = exp2(s * scale - m_ref): one FFMA, one MUFU, one add per element, in place
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      // masked columns hold -inf: exp2(-inf) = 0, no separate path (the scale is positive)
#pragma unroll
      for (int e = 0; e < 32; e++) {
        s0[e] = __float_as_uint(ex2_approx(fmaf(__uint_as_float(s0[e]), sc, -m_use)));
        s1[e] = __float_as_uint(ex2_approx(fmaf(__uint_as_float(s1[e]), sc, -m_use)));
      }
#pragma unroll
      for (int e = 0; e < 32; e += 4) {
        l0 += __uint_as_float(s0[e]) + __uint_as_float(s1[e]);         l1 += __uint_as_float(s0[e + 1]) + __uint_as_float(s1[e + 1]);
        l2 += __uint_as_float(s0[e + 2]) + __uint_as_float(s1[e + 2]); l3 += __uint_as_float(s0[e + 3]) + __uint_as_float(s1[e + 3]);
      }
      l_run += (l0 + l1) + (l2 + l3);
      // P_j: keys 2c and 2c+1 of this row packed into column c, over the head of the S buffer just read
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 16; c++) {
        pk[c] = pack2_t<T>(__uint_as_float(s0[2 * c]), __uint_as_float(s0[2 * c + 1]));
        pk[16 + c] = pack2_t<T>(__uint_as_float(s1[2 * c]), __uint_as_float(s1[2 * c + 1]));
      }
      tmem_st_32x32(tmem_s + lane_addr + (uint32_t)(st * kKV), pk);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[st]);
    }
    // the last product
    if (ok && n_blocks > 0) ok = __all_sync(0xffffffffu, mbar_wait(&o_full[(n_blocks - 1) & 1], (uint32_t)(((n_blocks - 1) >> 1) & 1), p.status, 22));
    if (ok && n_blocks > 0) {
      tc_fence_after_sync();
      const float inv = 1.0f / l_run;
      T* dst = reinterpret_cast<T*>(p.o) + (long long)b * p.o_b + (long long)h * p.o_h + (long long)row * p.o_t;
#pragma unroll
      for (int c = 0; c < kD / 32; c++) {
        uint32_t ov[32];
        tmem_ld_32x32(tmem_o + lane_addr + (uint32_t)(c * 32), ov);
        tmem_ld_wait();
        if (row < p.tq) {
          if (p.o_vec) {
#pragma unroll
            for (int g = 0; g < 4; g++) {
              uint4 o;
              o.x = pack2_t<T>(__uint_as_float(ov[g * 8 + 0]) * inv, __uint_as_float(ov[g * 8 + 1]) * inv);
              o.y = pack2_t<T>(__uint_as_float(ov[g * 8 + 2]) * inv, __uint_as_float(ov[g * 8 + 3]) * inv);
              o.z = pack2_t<T>(__uint_as_float(ov[g * 8 + 4]) * inv, __uint_as_float(ov[g * 8 + 5]) * inv);
              o.w = pack2_t<T>(__uint_as_float(ov[g * 8 + 6]) * inv, __uint_as_float(ov[g * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e++) dst[c * 32 + e] = Cvt<T>::from(__uint_as_float(ov[e]) * inv);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kAttnTmemCols);
}

static bool attn_view_ok(const void* ptr, int64_t sb, int64_t sh, int64_t st, int64_t batch, int64_t heads) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return false;
  if (st % 8 != 0 || st < kD) return false;
  if (heads > 1 && sh % 8 != 0) return false;
  if (batch > 1 && sb % 8 != 0) return false;
  return true;
}

bool attention_fused_eligible(const AttnDesc& d) {
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16)) return false;
  if (d.d != kD || d.dv != kD) return false;
  if (d.tq < 1 || d.tk < 1 || d.batch < 1 || d.heads < 1) return false;
  if (d.tq > 0x3fffffff || d.tk > 0x3fffffff || d.batch * d.heads > 0x7fffffff || (d.tq + kQ - 1) / kQ > 65535) return false;
  return attn_view_ok(d.q, d.q_b, d.q_h, d.q_t, d.batch, d.heads) && attn_view_ok(d.k, d.k_b, d.k_h, d.k_t, d.batch, d.heads) &&
         attn_view_ok(d.v, d.v_b, d.v_h, d.v_t, d.batch, d.heads);
}

template <typename T>
static Status launch_attention(cudaStream_t s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p,
                               dim3 grid) {
  static bool attr_set = false;
  auto kern = attention_tc_kernel<T>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
    if (e != cudaSuccess) return cuda_status(e, "attention smem attribute");
    attr_set = true;
  }
  cudaError_t le = launch_pdl(kern, dim3(grid), dim3(kAttnThreads), kAttnSmem, s, mq, mk, mv, p);
  if (le != cudaSuccess) return cuda_status(le, "attention (tcgen05)");
  return Status::OK();
}

Status attention(cudaStream_t s, const AttnDesc& d) {
  if (!attention_fused_eligible(d)) return Status::compute("attention: operands are not eligible for the fused kernel");
  int* st = matmul_status_word();
  if (!st) return Status::compute("attention: cannot allocate status word");
  CUtensorMap mq, mk, mv;
  AG_RETURN_IF_ERROR(make_map(&mq, d.dtype, d.q, kD, (uint64_t)d.tq, (uint64_t)d.heads, (uint64_t)d.batch, (uint64_t)d.q_t, (uint64_t)d.q_h, (uint64_t)d.q_b, kD, kQ));
  AG_RETURN_IF_ERROR(make_map(&mk, d.dtype, d.k, kD, (uint64_t)d.tk, (uint64_t)d.heads, (uint64_t)d.batch, (uint64_t)d.k_t, (uint64_t)d.k_h, (uint64_t)d.k_b, kD, kKV));
  AG_RETURN_IF_ERROR(make_map(&mv, d.dtype, d.v, kD, (uint64_t)d.tk, (uint64_t)d.heads, (uint64_t)d.batch, (uint64_t)d.v_t, (uint64_t)d.v_h, (uint64_t)d.v_b, kD, kKV));
  AttnParams p;
  p.o = d.o; p.o_b = d.o_b; p.o_h = d.o_h; p.o_t = d.o_t;
  p.heads = (int)d.heads; p.tq = (int)d.tq; p.tk = (int)d.tk; p.causal = d.causal ? 1 : 0;
  p.o_vec = ((reinterpret_cast<uintptr_t>(d.o) & 15u) == 0 && d.o_t % 8 == 0 && d.o_h % 8 == 0 && d.o_b % 8 == 0) ? 1 : 0;
  p.scale_log2 = d.scale * 1.4426950408889634f;
  p.status = st;
  dim3 grid((unsigned)(d.batch * d.heads), (unsigned)((d.tq + kQ - 1) / kQ), 1);
  if (d.dtype == DType::BF16) return launch_attention<__nv_bfloat16>(s, mq, mk, mv, p, grid);
  return launch_attention<__half>(s, mq, mk, mv, p, grid);
}

}}  // namespace ag::k
