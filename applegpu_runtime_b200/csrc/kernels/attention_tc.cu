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
// A tile is 128 query rows of one (batch, head); its key/value sequence is walked in blocks of 64:
// S = Q K_j^T (tcgen05, fp32 in tensor memory) -> online softmax by 128 threads, one query row each (running max /
// sum in registers, exp2 with the 1/sqrt(d) scale folded in, packed fp32 arithmetic) -> P_j in the storage type
// written over the S buffer it came from -> O += P_j V_j (tcgen05 with the P operand read from tensor memory, V read
// N-major in place), O staying in tensor memory until the tile ends. CTAs are persistent, two per SM (97 KB of shared
// memory, 256 tensor-memory columns and 166 registers per thread each), and each walks a fixed list of tiles,
// heaviest first. Warp roles: warp 0 TMA producer (Q double-buffered per tile, K and V through four-stage rings that
// run on across tile boundaries), warp 1 MMA issuer and tensor-memory owner, warps 2..5 softmax / output. The next
// tile's Q, K, V loads and first two score blocks are issued while the softmax warps finish the current tile, and a
// finished tile's output is normalised and stored after the first block of the next one, so neither the load
// latency nor the last product's latency leaves the softmax warps idle. All waits are bounded.
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
constexpr int kKVStages = 4;                             // K and V rings: loads run up to four blocks ahead of the MMAs
constexpr int kAttnSmem = 2 * kQBytes /*Q, two tiles*/ + kKVStages * kKVBytes /*K*/ + kKVStages * kKVBytes /*V*/ + 1024;
constexpr int kAttnTmemCols = 256;                       // S: 2 x 64 (P over the head of each), O: 64

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Blackwell's packed fp32 pipe: two independent fp32 operations per instruction on a 64-bit register pair, and the
// three-input maximum. The softmax below is bound by instruction issue and the MUFU pipe, not by arithmetic.
__device__ __forceinline__ float max3_f32(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
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
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
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
  int bh;                    // batch * heads
  int q_tiles;               // query tiles of kQ rows per (batch, head)
  int total_tiles;           // bh * q_tiles
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

#ifdef AG_ATTN_PROBE
// Timeline probe (compile-time only): per CTA start / end time, SM and key blocks processed.
__device__ unsigned long long g_attn_cta[4096][4];
#endif

// The tiles one CTA works through, the same sequence for each of its warp roles. Tiles are ranked heaviest first
// (under a causal mask the last query tile of a head sees the most keys; every head has the same tiles) and dealt
// to the CTAs in passes that alternate direction, so the CTA that got the heaviest tile of one pass gets the
// lightest of the next: a fixed schedule (no counter in global memory) within ~10 % of an even split.
struct TileWalk {
  int pass, cta, n_cta;
  int t;            // tiles this CTA has started so far (selects the Q buffer and barrier phases)
  int qt, b, h, q0, n_blocks;
  bool valid;
  __device__ void start(const AttnParams& p, int cta_, int n_cta_) { pass = 0; cta = cta_; n_cta = n_cta_; t = -1; next(p); }
  __device__ void next(const AttnParams& p) {
    const int r = pass * n_cta + ((pass & 1) ? (n_cta - 1 - cta) : cta);
    pass++; t++;
    valid = r < p.total_tiles;
    if (!valid) return;
    qt = p.q_tiles - 1 - r / p.bh;
    const int bh = r % p.bh;
    b = bh / p.heads; h = bh % p.heads;
    q0 = qt * kQ;
    n_blocks = (p.tk + kKV - 1) / kKV;
    if (p.causal) {
      const int nb = (q0 + kQ - 1) / kKV + 1;   // through the largest column any row of this tile may see
      if (nb < n_blocks) n_blocks = nb;
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full[2], q_empty[2], k_full[kKVStages], k_empty[kKVStages], v_full[kKVStages], v_empty[kKVStages], s_full[2], p_full[2], o_full[2], o_empty;
  __shared__ uint32_t tmem_base_slot;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                            // two buffers: the next tile's Q arrives while this tile runs
  uint8_t* sK = sQ + 2 * kQBytes;                // kKVStages stages
  uint8_t* sV = sK + kKVStages * kKVBytes;       // kKVStages stages

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef AG_ATTN_PROBE
  const unsigned long long cta_t0 = globaltimer_ns();
  int probe_blocks = 0;
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < kKVStages; s++) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4); mbar_init(&o_full[s], 1);
    }
    mbar_init(&o_empty, 4);
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

  // Every role walks the same tiles and numbers their key blocks g = 0, 1, 2, ... across tile boundaries: g picks
  // the K / V stage (g % kKVStages), the S buffer (g & 1) and the barrier phases, so the pipeline never drains
  // between tiles: the next tile's Q, K and V are in flight and its first scores computed while the softmax
  // warps finish the current one.
  if (warp == 0) {
    // ── TMA producer ──
    if (lane == 0) {
      TileWalk w; w.start(p, (int)blockIdx.x, (int)gridDim.x);
      int g = 0;
      bool ok = true;
      for (; w.valid && ok; w.next(p)) {
        const int qb = w.t & 1;
        if (!mbar_wait(&q_empty[qb], (uint32_t)(((w.t >> 1) & 1) ^ 1), p.status, 10)) { ok = false; break; }
        mbar_expect_tx(&q_full[qb], kQBytes);
        tma_load_4d(sQ + qb * kQBytes, &tmap_q, &q_full[qb], 0, w.q0, w.h, w.b);
        for (int j = 0; j < w.n_blocks; j++, g++) {
          const int st = g % kKVStages;
          const uint32_t ph = (uint32_t)((g / kKVStages) & 1);
          if (!mbar_wait(&k_empty[st], ph ^ 1, p.status, 11)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], kKVBytes);
          tma_load_4d(sK + st * kKVBytes, &tmap_k, &k_full[st], 0, j * kKV, w.h, w.b);
          if (!mbar_wait(&v_empty[st], ph ^ 1, p.status, 12)) { ok = false; break; }
          mbar_expect_tx(&v_full[st], kKVBytes);
          tma_load_4d(sV + st * kKVBytes, &tmap_v, &v_full[st], 0, j * kKV, w.h, w.b);
        }
      }
    }
  } else if (warp == 1) {
    // ── MMA issuer. S = Q K^T runs two blocks ahead of the softmax (two S buffers), across tile boundaries;
    //    O += P V reads P from tensor memory and accumulates in tensor memory. MMAs execute in issue order,
    //    so S_{g+2} (issued after P_g V_g) cannot overwrite P_g before that product has read it. ──
    if (lane == 0) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, kQ, kKV);   // S = Q K^T: both K-major, N = 64
      constexpr uint32_t idesc_o = make_idesc_f16(fmt, 0, 1, kQ, kD);    // O = P V: V is N-major, N = 64
      TileWalk ws; ws.start(p, (int)blockIdx.x, (int)gridDim.x);   // the tile whose scores are issued next
      int js = 0, gs = 0;
      bool ok = true;
      auto issue_s = [&]() -> bool {
        if (!ws.valid) return true;
        const int qb = ws.t & 1, sb = gs & 1, kst = gs % kKVStages;
        if (js == 0 && !mbar_wait(&q_full[qb], (uint32_t)((ws.t >> 1) & 1), p.status, 13)) return false;
        if (!mbar_wait(&k_full[kst], (uint32_t)((gs / kKVStages) & 1), p.status, 14)) return false;
        tc_fence_after_sync();
        const uint32_t a = smem_u32(sQ + qb * kQBytes), bb = smem_u32(sK + kst * kKVBytes);
#pragma unroll
        for (int kk = 0; kk < kD / 16; kk++)
          mma_f16_ss(tmem_s + (uint32_t)(sb * kKV), make_smem_desc_sw128(a + kk * 32, 16, 1024), make_smem_desc_sw128(bb + kk * 32, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(&k_empty[kst]);
        mma_commit(&s_full[sb]);
        gs++;
        if (++js == ws.n_blocks) { mma_commit(&q_empty[qb]); js = 0; ws.next(p); }
        return true;
      };
      ok = issue_s();
      if (ok) ok = issue_s();
      TileWalk wp; wp.start(p, (int)blockIdx.x, (int)gridDim.x);   // the tile whose products are issued
      int gp = 0;
      for (; wp.valid && ok; wp.next(p)) {
        for (int j = 0; j < wp.n_blocks; j++, gp++) {
          const int sb = gp & 1, vst = gp % kKVStages;
          if (!mbar_wait(&v_full[vst], (uint32_t)((gp / kKVStages) & 1), p.status, 16)) { ok = false; break; }
          if (!mbar_wait(&p_full[sb], (uint32_t)((gp >> 1) & 1), p.status, 17)) { ok = false; break; }   // P stored, O rescaled if it had to be
          // the first product of a tile overwrites O: the softmax warps must have read the previous tile's out
          if (j == 0 && wp.t > 0 && !mbar_wait(&o_empty, (uint32_t)((wp.t - 1) & 1), p.status, 18)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t bb = smem_u32(sV + vst * kKVBytes);
#pragma unroll
          for (int kk = 0; kk < kKV / 16; kk++) {
            // P: 16 keys = 8 packed columns. V: rows are keys (128 B = 64 head dims); 16 keys = 2048 B.
            mma_f16_ts(tmem_o, tmem_s + (uint32_t)(sb * kKV + kk * 8), make_smem_desc_sw128(bb + kk * 2048, 64 * 128, 1024), idesc_o,
                       (j > 0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(&v_empty[vst]);
          // Even and odd blocks signal different barriers: a waiter can then be at most one phase behind
          // (P_{g-2} V_{g-2} is always complete before S_g is), so its parity test cannot alias.
          mma_commit(&o_full[sb]);
          if (!issue_s()) { ok = false; break; }
        }
      }
    }
  } else {
    // ── softmax / output: thread = query row ──
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;          // row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sc = p.scale_log2;
    bool ok = true;
    int g = 0;
    // the finished tile whose output is still in tensor memory: normalised and stored after the first block of the
    // next tile, so the wait for its last product hides behind that block's arithmetic
    bool have_prev = false;
    float prev_l = 1.f;
    T* prev_dst = nullptr;
    bool prev_row_ok = false;
    int prev_g = 0;

    auto store_prev = [&]() -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(&o_full[prev_g & 1], (uint32_t)((prev_g >> 1) & 1), p.status, 22))) return false;
      tc_fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld_32x32(tmem_o + lane_addr, o0);
      tmem_ld_32x32(tmem_o + lane_addr + 32u, o1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty);       // the accumulator may be overwritten by the next tile's first product
      const float inv = 1.0f / prev_l;
      if (prev_row_ok) {
        if (p.o_vec) {
#pragma unroll
          for (int gq = 0; gq < 4; gq++) {
            uint4 o;
            o.x = pack2_t<T>(__uint_as_float(o0[gq * 8 + 0]) * inv, __uint_as_float(o0[gq * 8 + 1]) * inv);
            o.y = pack2_t<T>(__uint_as_float(o0[gq * 8 + 2]) * inv, __uint_as_float(o0[gq * 8 + 3]) * inv);
            o.z = pack2_t<T>(__uint_as_float(o0[gq * 8 + 4]) * inv, __uint_as_float(o0[gq * 8 + 5]) * inv);
            o.w = pack2_t<T>(__uint_as_float(o0[gq * 8 + 6]) * inv, __uint_as_float(o0[gq * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(prev_dst + gq * 8) = o;
          }
#pragma unroll
          for (int gq = 0; gq < 4; gq++) {
            uint4 o;
            o.x = pack2_t<T>(__uint_as_float(o1[gq * 8 + 0]) * inv, __uint_as_float(o1[gq * 8 + 1]) * inv);
            o.y = pack2_t<T>(__uint_as_float(o1[gq * 8 + 2]) * inv, __uint_as_float(o1[gq * 8 + 3]) * inv);
            o.z = pack2_t<T>(__uint_as_float(o1[gq * 8 + 4]) * inv, __uint_as_float(o1[gq * 8 + 5]) * inv);
            o.w = pack2_t<T>(__uint_as_float(o1[gq * 8 + 6]) * inv, __uint_as_float(o1[gq * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(prev_dst + 32 + gq * 8) = o;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e++) {
            prev_dst[e] = Cvt<T>::from(__uint_as_float(o0[e]) * inv);
            prev_dst[32 + e] = Cvt<T>::from(__uint_as_float(o1[e]) * inv);
          }
        }
      }
      return true;
    };

    TileWalk w; w.start(p, (int)blockIdx.x, (int)gridDim.x);
    for (; w.valid && ok; w.next(p)) {
      const int row = w.q0 + r;                   // row inside the sequence
      float m_ref = -INFINITY;   // the maximum the stored probabilities and sums are relative to
      float l_run = 0.f;
      for (int j = 0; j < w.n_blocks && ok; j++, g++) {
        const int st = g & 1;
        const uint32_t ph = (uint32_t)((g >> 1) & 1);
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
          // masked columns become -inf once, so both paths share the maximum below
#pragma unroll
          for (int e = 0; e < 32; e++) {
            if (e >= lim) s0[e] = 0xff800000u;
            if (32 + e >= lim) s1[e] = 0xff800000u;
          }
        }
        {
          // four chains of three-input maxima: two new scores per instruction
          auto sv = [&](int i) { return __uint_as_float(i < 32 ? s0[i] : s1[i - 32]); };
          float mc[4] = {sv(0), sv(1), sv(2), sv(3)};
#pragma unroll
          for (int i = 0; i < 30; i++) mc[i & 3] = max3_f32(mc[i & 3], sv(4 + 2 * i), sv(5 + 2 * i));
          m_blk = fmaxf(max3_f32(mc[0], mc[1], mc[2]), mc[3]);
        }
        // Move the reference maximum only when this row's maximum outgrew it by more than the margin (or
        // when the row sees its first scores); the accumulated output and sum are then rescaled.
        const float m_cand = fmaxf(m_ref, m_blk * sc);
        const bool moves = (m_cand - m_ref > kRescaleLog2) || (m_ref == -INFINITY && m_cand != -INFINITY);
        // the rescale factor goes through the MUFU pipe, behind whatever the SM's other warps queued there: only the
        // warps that have a row to rescale compute it
        float alpha = 1.0f;
        const bool any_moves = __any_sync(0xffffffffu, moves);
        if (any_moves) {
          if (moves) { alpha = ex2_approx(m_ref - m_cand); m_ref = m_cand; }      // exp2(-inf) = 0 for a first block
        }
        if (j > 0 && any_moves) {
          // O holds the products up to block j-1: wait for the last of them, scale this row, write it back
          if (!__all_sync(0xffffffffu, mbar_wait(&o_full[(g - 1) & 1], (uint32_t)(((g - 1) >> 1) & 1), p.status, 21))) { ok = false; break; }
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

        // probabilities = exp2(s * scale - m_ref), in place: one packed FMA per two scores, one MUFU each, packed sums.
        // Masked columns hold -inf: exp2(-inf) = 0, no separate path (the scale is positive).
        const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(-m_use, -m_use);
        uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};   // (0.f, 0.f) pairs
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float a0, a1, b0, b1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s0[e]), __uint_as_float(s0[e + 1])), sc2, nm2), a0, a1);
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s1[e]), __uint_as_float(s1[e + 1])), sc2, nm2), b0, b1);
          a0 = ex2_approx(a0); a1 = ex2_approx(a1); b0 = ex2_approx(b0); b1 = ex2_approx(b1);
          s0[e] = __float_as_uint(a0); s0[e + 1] = __float_as_uint(a1); s1[e] = __float_as_uint(b0); s1[e + 1] = __float_as_uint(b1);
          acc[(e >> 1) & 1] = add_f32x2(acc[(e >> 1) & 1], pack_f32x2(a0, a1));
          acc[2 + ((e >> 1) & 1)] = add_f32x2(acc[2 + ((e >> 1) & 1)], pack_f32x2(b0, b1));
        }
        {
          float x0, x1;
          unpack_f32x2(add_f32x2(add_f32x2(acc[0], acc[1]), add_f32x2(acc[2], acc[3])), x0, x1);
          l_run += x0 + x1;
        }
        // P: keys 2c and 2c+1 of this row packed into column c, over the head of the S buffer just read
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
        if (j == 0 && have_prev) {
          if (!store_prev()) { ok = false; break; }
          have_prev = false;
        }
      }
      if (!ok) break;
      have_prev = true;
      prev_l = l_run; prev_g = g - 1; prev_row_ok = row < p.tq;
      prev_dst = reinterpret_cast<T*>(p.o) + (long long)w.b * p.o_b + (long long)w.h * p.o_h + (long long)row * p.o_t;
#ifdef AG_ATTN_PROBE
      probe_blocks += w.n_blocks;
#endif
    }
    if (ok && have_prev) ok = store_prev();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kAttnTmemCols);
#ifdef AG_ATTN_PROBE
  if (threadIdx.x == 64 && blockIdx.x < 4096) {
    unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    g_attn_cta[blockIdx.x][0] = cta_t0; g_attn_cta[blockIdx.x][1] = globaltimer_ns(); g_attn_cta[blockIdx.x][2] = smid; g_attn_cta[blockIdx.x][3] = (unsigned long long)probe_blocks;
  }
#endif
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
  if (d.tq > 0x3fffffff || d.tk > 0x3fffffff || d.batch * d.heads * ((d.tq + kQ - 1) / kQ) > 0x3fffffff) return false;
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
  p.bh = (int)(d.batch * d.heads); p.q_tiles = (int)((d.tq + kQ - 1) / kQ); p.total_tiles = p.bh * p.q_tiles;
  // persistent CTAs: two per SM (registers and tensor-memory columns allow two), each walking its share of the tiles
  const int resident = 2 * sm_count();
  dim3 grid((unsigned)(p.total_tiles < resident ? p.total_tiles : resident), 1, 1);
  if (d.dtype == DType::BF16) return launch_attention<__nv_bfloat16>(s, mq, mk, mv, p, grid);
  return launch_attention<__half>(s, mq, mk, mv, p, grid);
}

#ifdef AG_ATTN_PROBE
void attn_probe_read_ctas(unsigned long long* out, int n) { cudaMemcpyFromSymbol(out, g_attn_cta, sizeof(unsigned long long) * 4 * n); }
#endif

}}  // namespace ag::k
