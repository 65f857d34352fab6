// float32 attention in one kernel: softmax[_causal]((Q K^T) * scale) V with head dim 64, true fp32
// multiply-adds on the CUDA cores and an online softmax, so the [Tq, Tk] score matrix never exists.
//
// The reference composes attention from five ops with materialised scores (ops.rs:1531-1618:
// transpose, matmul, scalar_mul, softmax / softmax_causal, matmul); at GPT-2-small's 8 x 12 x 1024 x 1024
// that is 403 MB per score tensor and layer. Same arithmetic here per element (fp32 products summed in
// fp32, scores scaled as fp32 before the softmax, kernel_templates.rs:398-430 / :468-497 for the softmax
// itself), in a different summation order: the row maximum and sum are carried across 64-key blocks.
// 16-bit inputs take the tensor-core kernel (attention_tc.cu); other head dims are composed from GEMMs.
//
// One CTA = 64 query rows of one (batch, head); 256 threads as 16 x 16: thread (ty, tx) owns rows
// ty*4..+3 and, of each 64-key block, score columns tx, tx+16, tx+32, tx+48 and output columns
// tx*4..+3. Q, K, P tiles sit in shared memory with a row pitch of 68 floats (16-byte reads by the 16
// lanes of a half-warp then fall in 8 bank groups, the minimum for 256 bytes), V unpadded.
#include "common.cuh"

namespace ag { namespace k {

constexpr int kAfQ = 64, kAfK = 64, kAfD = 64, kAfPitch = 68;
constexpr int kAfSmem = (3 * kAfQ * kAfPitch + kAfK * kAfD) * (int)sizeof(float);   // Q, K, P, V tiles

struct AttnF32Params {
  const float* q; const float* k; const float* v; float* o;
  long long q_b, q_h, q_t, k_b, k_h, k_t, v_b, v_h, v_t, o_b, o_h, o_t;
  int heads, tq, tk;
  float scale;
};

template <bool CAUSAL>
__global__ void __launch_bounds__(256, 3) attention_f32_kernel(const AttnF32Params p) {
  extern __shared__ __align__(16) float af_smem[];
  float* Qs = af_smem;
  float* Ks = Qs + kAfQ * kAfPitch;
  float* Ps = Ks + kAfK * kAfPitch;
  float* Vs = Ps + kAfQ * kAfPitch;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int bh = blockIdx.x;
  // causal tiles differ in work (1 .. Tq/64 key blocks): the heaviest are launched first
  const int qt = CAUSAL ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int q0 = qt * kAfQ;
  const float* Q = p.q + (long long)b * p.q_b + (long long)h * p.q_h;
  const float* K = p.k + (long long)b * p.k_b + (long long)h * p.k_h;
  const float* V = p.v + (long long)b * p.v_b + (long long)h * p.v_h;
  float* O = p.o + (long long)b * p.o_b + (long long)h * p.o_h;
  pdl_wait();
  pdl_trigger();

  for (int idx = t; idx < kAfQ * (kAfD / 4); idx += 256) {
    const int r = idx >> 4, c4 = idx & 15;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + r < p.tq) v = *reinterpret_cast<const float4*>(Q + (long long)(q0 + r) * p.q_t + c4 * 4);
    *reinterpret_cast<float4*>(Qs + r * kAfPitch + c4 * 4) = v;
  }
  float o[4][4], m[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < 4; c++) o[i][c] = 0.f;
  }
  const int kend = CAUSAL ? min(p.tk, q0 + kAfQ) : p.tk;
  for (int k0 = 0; k0 < kend; k0 += kAfK) {
    __syncthreads();   // the previous block's reads of K, V and P are done (and Q is in place)
    for (int idx = t; idx < kAfK * (kAfD / 4); idx += 256) {
      const int r = idx >> 4, c4 = idx & 15;
      float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
      if (k0 + r < p.tk) {
        kv = *reinterpret_cast<const float4*>(K + (long long)(k0 + r) * p.k_t + c4 * 4);
        vv = *reinterpret_cast<const float4*>(V + (long long)(k0 + r) * p.v_t + c4 * 4);
      }
      *reinterpret_cast<float4*>(Ks + r * kAfPitch + c4 * 4) = kv;
      *reinterpret_cast<float4*>(Vs + r * kAfD + c4 * 4) = vv;
    }
    __syncthreads();
    // scores of this block: rows ty*4+i, columns tx+16*jj
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int jj = 0; jj < 4; jj++) s[i][jj] = 0.f;
#pragma unroll 4
    for (int d4 = 0; d4 < kAfD / 4; d4++) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty * 4 + i) * kAfPitch + d4 * 4);
#pragma unroll
      for (int jj = 0; jj < 4; jj++) kv[jj] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * jj) * kAfPitch + d4 * 4);
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          s[i][jj] = fmaf(qv[i].x, kv[jj].x, s[i][jj]); s[i][jj] = fmaf(qv[i].y, kv[jj].y, s[i][jj]);
          s[i][jj] = fmaf(qv[i].z, kv[jj].z, s[i][jj]); s[i][jj] = fmaf(qv[i].w, kv[jj].w, s[i][jj]);
        }
    }
    // scale, mask, online softmax update (the 16 lanes that share ty hold one row's 64 columns)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int row = q0 + ty * 4 + i;
      float mx = -INFINITY;
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int col = k0 + tx + 16 * jj;
        float x = s[i][jj] * p.scale;
        if (col >= p.tk || (CAUSAL && col > row)) x = -INFINITY;
        s[i][jj] = x;
        mx = fmaxf(mx, x);
      }
#pragma unroll
      for (int sh = 1; sh < 16; sh <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
      const float m_new = fmaxf(m[i], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // a row with nothing visible yet: every term is exp(-inf) = 0
      const float corr = __expf(m[i] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const float pe = __expf(s[i][jj] - m_use);
        sum += pe;
        Ps[(ty * 4 + i) * kAfPitch + tx + 16 * jj] = pe;
      }
#pragma unroll
      for (int sh = 1; sh < 16; sh <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sh);
      l[i] = l[i] * corr + sum;
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < 4; c++) o[i][c] *= corr;
    }
    __syncthreads();
    // O += P V: rows ty*4+i, output columns tx*4..+3
#pragma unroll 4
    for (int j4 = 0; j4 < kAfK / 4; j4++) {
      float4 pv[4], vv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty * 4 + i) * kAfPitch + j4 * 4);
#pragma unroll
      for (int jj = 0; jj < 4; jj++) vv[jj] = *reinterpret_cast<const float4*>(Vs + (j4 * 4 + jj) * kAfD + tx * 4);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float pj[4] = {pv[i].x, pv[i].y, pv[i].z, pv[i].w};
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          o[i][0] = fmaf(pj[jj], vv[jj].x, o[i][0]); o[i][1] = fmaf(pj[jj], vv[jj].y, o[i][1]);
          o[i][2] = fmaf(pj[jj], vv[jj].z, o[i][2]); o[i][3] = fmaf(pj[jj], vv[jj].w, o[i][3]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = q0 + ty * 4 + i;
    if (row >= p.tq) continue;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
    *reinterpret_cast<float4*>(O + (long long)row * p.o_t + tx * 4) = make_float4(o[i][0] * inv, o[i][1] * inv, o[i][2] * inv, o[i][3] * inv);
  }
}

static bool af_view_ok(const void* ptr, int64_t sb, int64_t sh, int64_t st, int64_t batch, int64_t heads) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return false;      // 16-byte row accesses
  if (st % 4 != 0 || st < kAfD) return false;
  if (heads > 1 && sh % 4 != 0) return false;
  if (batch > 1 && sb % 4 != 0) return false;
  return true;
}

bool attention_f32_eligible(const AttnDesc& d) {
  if (d.dtype != DType::F32 || d.d != kAfD || d.dv != kAfD) return false;
  if (d.tq < 1 || d.tk < 1 || d.batch < 1 || d.heads < 1) return false;
  if (d.tq > 0x3fffffff || d.tk > 0x3fffffff || d.batch * d.heads > 0x7fffffff || (d.tq + kAfQ - 1) / kAfQ > 65535) return false;
  return af_view_ok(d.q, d.q_b, d.q_h, d.q_t, d.batch, d.heads) && af_view_ok(d.k, d.k_b, d.k_h, d.k_t, d.batch, d.heads) &&
         af_view_ok(d.v, d.v_b, d.v_h, d.v_t, d.batch, d.heads) && af_view_ok(d.o, d.o_b, d.o_h, d.o_t, d.batch, d.heads);
}

Status attention_f32(cudaStream_t s, const AttnDesc& d) {
  if (!attention_f32_eligible(d)) return Status::compute("attention (float32): operands are not eligible for the single-kernel form");
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_f32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAfSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_f32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAfSmem);
    if (e != cudaSuccess) return cuda_status(e, "attention (float32) smem attribute");
    attr_set = true;
  }
  AttnF32Params p;
  p.q = static_cast<const float*>(d.q); p.k = static_cast<const float*>(d.k); p.v = static_cast<const float*>(d.v); p.o = static_cast<float*>(d.o);
  p.q_b = d.q_b; p.q_h = d.q_h; p.q_t = d.q_t; p.k_b = d.k_b; p.k_h = d.k_h; p.k_t = d.k_t;
  p.v_b = d.v_b; p.v_h = d.v_h; p.v_t = d.v_t; p.o_b = d.o_b; p.o_h = d.o_h; p.o_t = d.o_t;
  p.heads = (int)d.heads; p.tq = (int)d.tq; p.tk = (int)d.tk; p.scale = d.scale;
  dim3 grid((unsigned)(d.batch * d.heads), (unsigned)((d.tq + kAfQ - 1) / kAfQ), 1);
  cudaError_t e = d.causal ? launch_pdl(attention_f32_kernel<true>, grid, dim3(256), (size_t)kAfSmem, s, p)
                           : launch_pdl(attention_f32_kernel<false>, grid, dim3(256), (size_t)kAfSmem, s, p);
  if (e != cudaSuccess) return cuda_status(e, "attention (float32)");
  return Status::OK();
}

}}  // namespace ag::k
