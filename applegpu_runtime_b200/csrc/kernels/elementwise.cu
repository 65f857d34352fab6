// Element-wise kernels: binary / unary / scalar_mul / fused chains / add_bias (+activation) /
// threshold_backward / in-place axpy / strided copy.
//
// Reference semantics: kernel_templates.rs:54-88 (binary, N-D strided), :91-168 (unary),
// :197-221 (scalar_mul), :272-307 (gelu), :311-360 (gelu_exact), :747-762 (add_bias),
// :1146-1169 (copy_strided); fusion.rs:167-238 (fused chains). The reference launches one
// thread per element with div/mod index math even for contiguous data; here contiguous data
// moves as 16-byte packs through a grid sized from the SM count, and the strided form is
// kept for views and broadcasts.
#include "common.cuh"
#include <cstdlib>
#include <type_traits>

namespace ag { namespace k {

static int g_sm_count = 0;
static int g_sm_margin = 0;   // SMs left free for kernels of other streams (a collective running beside the compute)
int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) g_sm_count = n;
    else g_sm_count = 148;
  }
  const int usable = g_sm_count - g_sm_margin;
  return usable < 8 ? 8 : usable;
}
// Persistent kernels size their grids from sm_count(): a margin keeps that many SMs out of them, so the CTAs of a
// collective on another stream find room at once instead of waiting for a persistent kernel to end (and a persistent
// kernel is not left with fewer SMs than the CTAs it launched).
void set_sm_margin(int n) { g_sm_margin = n < 0 ? 0 : n; }

static int g_pdl_override = -1;
void set_pdl_override(int on) { g_pdl_override = on; }
bool pdl_enabled() {
  static const bool on = [] { const char* v = std::getenv("APPLEGPU_PDL"); return !(v && v[0] == '0'); }();
  return g_pdl_override < 0 ? on : g_pdl_override != 0;
}

// ── index helpers ───────────────────────────────────────────────────────────
struct NdIndex {
  int nd;
  int64_t shape[kMaxDims];
};
template <int MAXOPS>
struct NdStrides {
  int64_t s[MAXOPS][kMaxDims];
};

// Collapse adjacent dims when every operand's strides allow it; returns new nd.
static int collapse(int nd, int64_t* shape, int64_t (*strides)[kMaxDims], int nops) {
  // drop size-1 dims
  int w = 0;
  for (int i = 0; i < nd; i++) {
    if (shape[i] == 1) continue;
    shape[w] = shape[i];
    for (int o = 0; o < nops; o++) strides[o][w] = strides[o][i];
    w++;
  }
  nd = w;
  if (nd == 0) { shape[0] = 1; for (int o = 0; o < nops; o++) strides[o][0] = 1; return 1; }
  int out = 0;
  for (int i = 1; i < nd; i++) {
    bool can = true;
    for (int o = 0; o < nops; o++) if (strides[o][out] != strides[o][i] * shape[i]) { can = false; break; }
    if (can) {
      shape[out] *= shape[i];
      for (int o = 0; o < nops; o++) strides[o][out] = strides[o][i];
    } else {
      out++;
      shape[out] = shape[i];
      for (int o = 0; o < nops; o++) strides[o][out] = strides[o][i];
    }
  }
  return out + 1;
}

// ── fused / unary / binary float program ────────────────────────────────────
__device__ __forceinline__ float apply_unary(int op, float x) {
  switch (op) {
    case (int)UnOp::Neg: return -x;
    case (int)UnOp::Relu: return fmaxf(x, 0.0f);
    case (int)UnOp::Exp: return expf(x);
    case (int)UnOp::Log: return logf(x);
    case (int)UnOp::Sqrt: return sqrtf(x);
    case (int)UnOp::Tanh: return tanhf(x);
    case (int)UnOp::Sin: return sinf(x);
    case (int)UnOp::Cos: return cosf(x);
    case (int)UnOp::Gelu: return gelu_tanh_f(x);
    case (int)UnOp::GeluExact: return gelu_erf_f(x);
    case (int)UnOp::Sigmoid: return 1.0f / (1.0f + expf(-x));
    case (int)UnOp::Abs: return fabsf(x);
    case (int)UnOp::Sign: return (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : 0.f);
    default: return x;
  }
}
__device__ __forceinline__ float apply_binary(int op, float a, float b) {
  switch (op) {
    case (int)BinOp::Add: return a + b;
    case (int)BinOp::Sub: return a - b;
    case (int)BinOp::Mul: return a * b;
    default: return __fdiv_rn(a, b);
  }
}

// Block forms: the op is tested once, then a straight loop runs over the thread's elements.
template <int M>
__device__ __forceinline__ void unary_block(int op, const float (&x)[M], float (&y)[M]) {
#define AG_UN(CASE, EXPR) case (int)UnOp::CASE: _Pragma("unroll") for (int i = 0; i < M; i++) { float v = x[i]; y[i] = (EXPR); } break;
  switch (op) {
    AG_UN(Neg, -v) AG_UN(Relu, fmaxf(v, 0.0f)) AG_UN(Exp, expf(v)) AG_UN(Log, logf(v)) AG_UN(Sqrt, sqrtf(v)) AG_UN(Tanh, tanhf(v))
    AG_UN(Sin, sinf(v)) AG_UN(Cos, cosf(v)) AG_UN(Gelu, gelu_tanh_f(v)) AG_UN(GeluExact, gelu_erf_f(v))
    AG_UN(Sigmoid, 1.0f / (1.0f + expf(-v))) AG_UN(Abs, fabsf(v)) AG_UN(Sign, (v > 0.f) ? 1.f : ((v < 0.f) ? -1.f : 0.f))
    default:
#pragma unroll
      for (int i = 0; i < M; i++) y[i] = x[i];
  }
#undef AG_UN
}
template <int M>
__device__ __forceinline__ void binary_block(int op, const float (&a)[M], const float (&b)[M], float (&y)[M]) {
  switch (op) {
    case (int)BinOp::Add:
#pragma unroll
      for (int i = 0; i < M; i++) y[i] = a[i] + b[i];
      break;
    case (int)BinOp::Sub:
#pragma unroll
      for (int i = 0; i < M; i++) y[i] = a[i] - b[i];
      break;
    case (int)BinOp::Mul:
#pragma unroll
      for (int i = 0; i < M; i++) y[i] = a[i] * b[i];
      break;
    default:
#pragma unroll
      for (int i = 0; i < M; i++) y[i] = __fdiv_rn(a[i], b[i]);
  }
}

struct ProgParams {
  FusedProgram prog;
  const void* in[kFusedMaxInputs];
  float scalar;  // multiplies the result when use_scalar (scalar_mul)
  int use_scalar;
};

// Contiguous form: every leaf has the output's shape (or is a single element, bcast[j]=1).
template <typename T>
__global__ void __launch_bounds__(256) program_vec_kernel(ProgParams p, uint32_t bcast_mask, T* __restrict__ out, int64_t n_packs, int64_t n) {
  constexpr int N = Pack<T>::N;
  constexpr int U = 16 / N;  // 16 elements per thread per trip: 4 (fp32) or 2 (half types) independent 16-byte loads in flight per leaf
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t pk0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; pk0 < n_packs; pk0 += stride * U) {
    float acc[U * N];
    const int ni = p.prog.n_instrs;
    for (int it = 0; it < ni; it++) {
      FusedInstr ins = p.prog.instrs[it];
      float a[U * N], b[U * N];
      if (ins.a < 0) {
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
          for (int e = 0; e < N; e++) a[u * N + e] = acc[u * N + e];
      } else {
        const T* src = reinterpret_cast<const T*>(p.in[ins.a]);
        if (bcast_mask & (1u << ins.a)) {
          float s = Cvt<T>::to(src[0]);
#pragma unroll
          for (int u = 0; u < U; u++)
#pragma unroll
            for (int e = 0; e < N; e++) a[u * N + e] = s;
        } else {
          Pack<T> v[U];
#pragma unroll
          for (int u = 0; u < U; u++) { int64_t pk = pk0 + u * stride; if (pk < n_packs) v[u] = ld16_stream(src + pk * N); }
#pragma unroll
          for (int u = 0; u < U; u++)
#pragma unroll
            for (int e = 0; e < N; e++) a[u * N + e] = Cvt<T>::to(v[u].v[e]);
        }
      }
      if (ins.is_binary) {
        if (ins.b < 0) {
#pragma unroll
          for (int u = 0; u < U; u++)
#pragma unroll
            for (int e = 0; e < N; e++) b[u * N + e] = acc[u * N + e];
        } else {
          const T* src = reinterpret_cast<const T*>(p.in[ins.b]);
          if (bcast_mask & (1u << ins.b)) {
            float s = Cvt<T>::to(src[0]);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
              for (int e = 0; e < N; e++) b[u * N + e] = s;
          } else {
            Pack<T> v[U];
#pragma unroll
            for (int u = 0; u < U; u++) { int64_t pk = pk0 + u * stride; if (pk < n_packs) v[u] = ld16_stream(src + pk * N); }
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
              for (int e = 0; e < N; e++) b[u * N + e] = Cvt<T>::to(v[u].v[e]);
          }
        }
        binary_block<U * N>(ins.op, a, b, acc);
      } else {
        unary_block<U * N>(ins.op, a, acc);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      int64_t pk = pk0 + u * stride;
      if (pk >= n_packs) break;
      Pack<T> o;
#pragma unroll
      for (int e = 0; e < N; e++) o.v[e] = Cvt<T>::from(p.use_scalar ? acc[u * N + e] * p.scalar : acc[u * N + e]);
      st16_stream(out + pk * N, o);
    }
  }
  // tail (n not a multiple of the pack width)
  int64_t tail0 = n_packs * N;
  for (int64_t i = tail0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float acc = 0.f;
    for (int it = 0; it < p.prog.n_instrs; it++) {
      FusedInstr ins = p.prog.instrs[it];
      float a = ins.a < 0 ? acc : Cvt<T>::to(reinterpret_cast<const T*>(p.in[ins.a])[(bcast_mask & (1u << ins.a)) ? 0 : i]);
      if (ins.is_binary) {
        float b = ins.b < 0 ? acc : Cvt<T>::to(reinterpret_cast<const T*>(p.in[ins.b])[(bcast_mask & (1u << ins.b)) ? 0 : i]);
        acc = apply_binary(ins.op, a, b);
      } else acc = apply_unary(ins.op, a);
    }
    if (p.use_scalar) acc *= p.scalar;
    out[i] = Cvt<T>::from(acc);
  }
}

// Strided form: output contiguous over `idx.shape`, each leaf with its own element strides.
template <typename T>
__global__ void __launch_bounds__(256) program_strided_kernel(ProgParams p, NdIndex idx, NdStrides<kFusedMaxInputs> st, T* __restrict__ out, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t coord[kMaxDims];
    int64_t r = i;
#pragma unroll
    for (int d = kMaxDims - 1; d >= 0; d--) {
      if (d < idx.nd) { coord[d] = r % idx.shape[d]; r /= idx.shape[d]; } else coord[d] = 0;
    }
    auto load = [&](int j) -> float {
      int64_t off = 0;
#pragma unroll
      for (int d = 0; d < kMaxDims; d++) if (d < idx.nd) off += coord[d] * st.s[j][d];
      return Cvt<T>::to(reinterpret_cast<const T*>(p.in[j])[off]);
    };
    float acc = 0.f;
    for (int it = 0; it < p.prog.n_instrs; it++) {
      FusedInstr ins = p.prog.instrs[it];
      float a = ins.a < 0 ? acc : load(ins.a);
      if (ins.is_binary) {
        float b = ins.b < 0 ? acc : load(ins.b);
        acc = apply_binary(ins.op, a, b);
      } else acc = apply_unary(ins.op, a);
    }
    if (p.use_scalar) acc *= p.scalar;
    out[i] = Cvt<T>::from(acc);
  }
}

static Status run_program(cudaStream_t s, const FusedProgram& prog, const TView* ins, const TView& out, float scalar, bool use_scalar) {
  if (prog.n_inputs < 1 || prog.n_inputs > kFusedMaxInputs || prog.n_instrs < 1 || prog.n_instrs > kFusedMaxInstrs)
    return Status::compute("fused program out of range");
  if (!out.contiguous()) return Status::compute("element-wise output must be contiguous");
  int64_t n = out.numel();
  if (n == 0) return Status::OK();
  ProgParams p;
  p.prog = prog; p.scalar = scalar; p.use_scalar = use_scalar ? 1 : 0;
  for (int j = 0; j < kFusedMaxInputs; j++) p.in[j] = nullptr;
  // classify leaves
  bool vec_ok = true;
  uint32_t bmask = 0;
  size_t esz = dtype_size(out.dtype);
  for (int j = 0; j < prog.n_inputs; j++) {
    if (ins[j].dtype != out.dtype) return Status::invalid(std::string("dtype mismatch: ") + dtype_debug(ins[j].dtype) + " vs " + dtype_debug(out.dtype));
    p.in[j] = ins[j].ptr;
    if (ins[j].numel() == 1) { bmask |= 1u << j; continue; }
    if (!(ins[j].contiguous() && ins[j].numel() == n)) vec_ok = false;
    if (!aligned16(ins[j].ptr)) vec_ok = false;
  }
  if (!aligned16(out.ptr)) vec_ok = false;
  const int threads = 256;
  if (vec_ok) {
    int64_t per = 16 / esz;
    int64_t n_packs = n / per;
    int grid = grid_for(n_packs > 0 ? n_packs : 1, threads, 8);
    AG_DISPATCH_FLOAT(out.dtype, T, (program_vec_kernel<T><<<grid, threads, 0, s>>>(p, bmask, (T*)out.ptr, n_packs, n)));
    AG_CHECK_LAUNCH("fused elementwise");
    return Status::OK();
  }
  NdIndex idx; NdStrides<kFusedMaxInputs> st;
  int64_t strides_tmp[kFusedMaxInputs][kMaxDims];
  int nd = out.nd();
  if (nd > kMaxDims) return Status::invalid("too many dims");
  int64_t shape_tmp[kMaxDims];
  for (int d = 0; d < nd; d++) shape_tmp[d] = out.shape[d];
  for (int j = 0; j < prog.n_inputs; j++) {
    Dims bs = broadcast_strides(ins[j].shape, ins[j].strides, out.shape);
    for (int d = 0; d < nd; d++) strides_tmp[j][d] = bs[d];
  }
  nd = collapse(nd, shape_tmp, strides_tmp, prog.n_inputs);
  idx.nd = nd;
  for (int d = 0; d < kMaxDims; d++) idx.shape[d] = d < nd ? shape_tmp[d] : 1;
  for (int j = 0; j < kFusedMaxInputs; j++)
    for (int d = 0; d < kMaxDims; d++) st.s[j][d] = (j < prog.n_inputs && d < nd) ? strides_tmp[j][d] : 0;
  int grid = grid_for(n, threads, 8);
  AG_DISPATCH_FLOAT(out.dtype, T, (program_strided_kernel<T><<<grid, threads, 0, s>>>(p, idx, st, (T*)out.ptr, n)));
  AG_CHECK_LAUNCH("fused elementwise (strided)");
  return Status::OK();
}

// ── integer binary (Add/Sub/Mul/Div on i32/i64/u8/u32) ──────────────────────
template <typename T>
__global__ void binary_int_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                  NdIndex idx, NdStrides<2> st, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t r = i, oa = 0, ob = 0;
    for (int d = idx.nd - 1; d >= 0; d--) {
      int64_t c = r % idx.shape[d]; r /= idx.shape[d];
      oa += c * st.s[0][d]; ob += c * st.s[1][d];
    }
    T x = a[oa], y = b[ob], z;
    switch (op) {
      case (int)BinOp::Add: z = x + y; break;
      case (int)BinOp::Sub: z = x - y; break;
      case (int)BinOp::Mul: z = x * y; break;
      default: z = (y == 0) ? (T)0 : (T)(x / y); break;
    }
    out[i] = z;
  }
}

Status binary(cudaStream_t s, BinOp op, const TView& a, const TView& b, const TView& out) {
  if (a.dtype != b.dtype) return Status::invalid(std::string("dtype mismatch: ") + dtype_debug(a.dtype) + " vs " + dtype_debug(b.dtype));
  if (out.dtype == DType::F32 || out.dtype == DType::F16 || out.dtype == DType::BF16) {
    FusedProgram prog; prog.n_inputs = 2; prog.n_instrs = 1;
    prog.instrs[0] = FusedInstr{(int8_t)op, 1, 0, 1};
    TView ins[2] = {a, b};
    return run_program(s, prog, ins, out, 1.f, false);
  }
  int64_t n = out.numel();
  if (n == 0) return Status::OK();
  NdIndex idx; NdStrides<2> st;
  int64_t shape_tmp[kMaxDims], strides_tmp[2][kMaxDims];
  int nd = out.nd();
  Dims sa = broadcast_strides(a.shape, a.strides, out.shape), sb = broadcast_strides(b.shape, b.strides, out.shape);
  for (int d = 0; d < nd; d++) { shape_tmp[d] = out.shape[d]; strides_tmp[0][d] = sa[d]; strides_tmp[1][d] = sb[d]; }
  nd = collapse(nd, shape_tmp, strides_tmp, 2);
  idx.nd = nd;
  for (int d = 0; d < kMaxDims; d++) { idx.shape[d] = d < nd ? shape_tmp[d] : 1; st.s[0][d] = d < nd ? strides_tmp[0][d] : 0; st.s[1][d] = d < nd ? strides_tmp[1][d] : 0; }
  int grid = grid_for(n, 256, 8);
  switch (out.dtype) {
    case DType::I32: binary_int_kernel<int32_t><<<grid, 256, 0, s>>>((int)op, (const int32_t*)a.ptr, (const int32_t*)b.ptr, (int32_t*)out.ptr, idx, st, n); break;
    case DType::I64: binary_int_kernel<int64_t><<<grid, 256, 0, s>>>((int)op, (const int64_t*)a.ptr, (const int64_t*)b.ptr, (int64_t*)out.ptr, idx, st, n); break;
    case DType::U8: binary_int_kernel<uint8_t><<<grid, 256, 0, s>>>((int)op, (const uint8_t*)a.ptr, (const uint8_t*)b.ptr, (uint8_t*)out.ptr, idx, st, n); break;
    case DType::U32: binary_int_kernel<uint32_t><<<grid, 256, 0, s>>>((int)op, (const uint32_t*)a.ptr, (const uint32_t*)b.ptr, (uint32_t*)out.ptr, idx, st, n); break;
    default: return Status::unsupported(std::string("binary op does not support ") + dtype_name(out.dtype));
  }
  AG_CHECK_LAUNCH("binary (int)");
  return Status::OK();
}

Status unary(cudaStream_t s, UnOp op, const TView& in, const TView& out) {
  FusedProgram prog; prog.n_inputs = 1; prog.n_instrs = 1;
  prog.instrs[0] = FusedInstr{(int8_t)op, 0, 0, 0};
  return run_program(s, prog, &in, out, 1.f, false);
}

Status scalar_mul(cudaStream_t s, const TView& in, float scale, const TView& out) {
  FusedProgram prog; prog.n_inputs = 1; prog.n_instrs = 1;
  prog.instrs[0] = FusedInstr{(int8_t)UnOp::Copy, 0, 0, 0};
  return run_program(s, prog, &in, out, scale, true);
}

Status fused_elementwise(cudaStream_t s, const FusedProgram& prog, const TView* ins, const TView& out) {
  return run_program(s, prog, ins, out, 1.f, false);
}

// ── add_bias (+ activation) ─────────────────────────────────────────────────
// 2-D form [rows, C]: bias index is the column; C % pack == 0 so a pack never straddles rows.
template <typename T>
__global__ void __launch_bounds__(256) add_bias_rows_kernel(const T* __restrict__ in, const T* __restrict__ bias, T* __restrict__ out,
                                                             int64_t n_packs, int packs_per_row, Act act) {
  constexpr int N = Pack<T>::N;
  constexpr int U = 4;       // independent 16-byte loads in flight per thread and trip
  pdl_wait();
  pdl_trigger();
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // the pack's column is tracked incrementally: a 64-bit modulo per pack costs more than the activation
  const int step = (int)(stride % packs_per_row);
  int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int col = (int)(first % packs_per_row);
  for (int64_t pk0 = first; pk0 < n_packs; pk0 += stride * U) {
    Pack<T> x[U], b[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      int64_t pk = pk0 + u * stride;
      if (pk < n_packs) { x[u] = ld16_stream(in + pk * N); b[u] = ld16(bias + col * N); }
      col += step;
      if (col >= packs_per_row) col -= packs_per_row;
    }
    float v[U * N];
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      // packed bf16 add: two sums per instruction, each rounded once to bf16 (what the separate add_bias kernel
      // of the reference stores), then widened for the activation
#pragma unroll
      for (int u = 0; u < U; u++) {
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x[u]);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
#pragma unroll
        for (int q = 0; q < N / 2; q++) {
          const float2 f = __bfloat1622float2(__hadd2(x2[q], b2[q]));
          v[u * N + 2 * q] = f.x; v[u * N + 2 * q + 1] = f.y;
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; u++)
#pragma unroll
        for (int e = 0; e < N; e++) {
          // The sum is rounded to the storage type before the activation, as two separate
          // reference kernels (add_bias then gelu) would do.
          v[u * N + e] = Cvt<T>::to(Cvt<T>::from(Cvt<T>::to(x[u].v[e]) + Cvt<T>::to(b[u].v[e])));
        }
    }
    switch (act) {  // tested once per trip, not per element
      case Act::GeluTanh:
        if (std::is_same<T, __nv_bfloat16>::value) {
          // bf16 results: the hardware tanh (relative error about 2^-11, a quarter of the rounding step of the
          // stored value) is what the GEMM epilogue uses for the same function, so the fused and the unfused
          // linear layer agree; one MUFU operation per element instead of two
#pragma unroll
          for (int i = 0; i < U * N; i++) {
            const float x = v[i];
            const float u = 0.7978845608f * fmaf(0.044715f * x, x * x, x);
            float t;
            asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
            const float hx = 0.5f * x;
            v[i] = fmaf(hx, t, hx);
          }
        } else {
#pragma unroll
          for (int i = 0; i < U * N; i++) v[i] = gelu_tanh_f(v[i]);
        }
        break;
      case Act::GeluErf:
        if (std::is_same<T, __nv_bfloat16>::value) {
          // the same function as the GEMM epilogue's, so the fused and the unfused linear layer agree
#pragma unroll
          for (int i = 0; i < U * N; i++) v[i] = gelu_erf_bf16_f(v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < U * N; i++) v[i] = gelu_erf_f(v[i]);
        }
        break;
      case Act::Relu:
#pragma unroll
        for (int i = 0; i < U * N; i++) v[i] = fmaxf(v[i], 0.f);
        break;
      default: break;
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      int64_t pk = pk0 + u * stride;
      if (pk >= n_packs) break;
      Pack<T> o;
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int q = 0; q < N / 2; q++) o2[q] = __floats2bfloat162_rn(v[u * N + 2 * q], v[u * N + 2 * q + 1]);
      } else {
#pragma unroll
        for (int e = 0; e < N; e++) o.v[e] = Cvt<T>::from(v[u * N + e]);
      }
      st16_stream(out + pk * N, o);
    }
  }
}
template <typename T>
__global__ void add_bias_generic_kernel(const T* __restrict__ in, const T* __restrict__ bias, T* __restrict__ out,
                                        int64_t n, int64_t inner, int64_t channels, Act act) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t ch = (i / inner) % channels;
    float v = Cvt<T>::to(Cvt<T>::from(Cvt<T>::to(in[i]) + Cvt<T>::to(bias[ch])));
    out[i] = Cvt<T>::from(apply_act(v, act));
  }
}

Status add_bias(cudaStream_t s, const TView& in, const TView& bias, Act act, const TView& out) {
  if (!in.contiguous() || !out.contiguous() || !bias.contiguous()) return Status::compute("add_bias needs contiguous tensors");
  int64_t n = in.numel();
  if (n == 0) return Status::OK();
  int64_t channels = in.shape[1];
  int64_t inner = 1;
  for (int d = 2; d < in.nd(); d++) inner *= in.shape[d];
  size_t esz = dtype_size(in.dtype);
  int64_t per = 16 / esz;
  if (inner == 1 && channels % per == 0 && aligned16(in.ptr) && aligned16(out.ptr) && aligned16(bias.ptr)) {
    int64_t n_packs = n / per;
    int grid = grid_for(n_packs, 256, 8);
    cudaError_t le = cudaSuccess;
    AG_DISPATCH_FLOAT(in.dtype, T, (le = launch_pdl(add_bias_rows_kernel<T>, dim3(grid), dim3(256), 0, s, (const T*)in.ptr, (const T*)bias.ptr, (T*)out.ptr, n_packs, (int)(channels / per), act)));
    if (le != cudaSuccess) return cuda_status(le, "add_bias");
  } else {
    int grid = grid_for(n, 256, 8);
    AG_DISPATCH_FLOAT(in.dtype, T, (add_bias_generic_kernel<T><<<grid, 256, 0, s>>>((const T*)in.ptr, (const T*)bias.ptr, (T*)out.ptr, n, inner, channels, act)));
  }
  AG_CHECK_LAUNCH("add_bias");
  return Status::OK();
}

// ── threshold_backward, in-place axpy ───────────────────────────────────────
template <typename T>
__global__ void threshold_backward_kernel(const T* __restrict__ g, const T* __restrict__ x, T* __restrict__ out, float thr, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = (Cvt<T>::to(x[i]) > thr) ? g[i] : Cvt<T>::from(0.f);
}
Status threshold_backward(cudaStream_t s, const TView& grad, const TView& in, float threshold, const TView& out) {
  if (!grad.contiguous() || !in.contiguous()) return Status::compute("threshold_backward needs contiguous tensors");
  int64_t n = out.numel();
  if (n == 0) return Status::OK();
  int grid = grid_for(n, 256, 8);
  AG_DISPATCH_FLOAT(out.dtype, T, (threshold_backward_kernel<T><<<grid, 256, 0, s>>>((const T*)grad.ptr, (const T*)in.ptr, (T*)out.ptr, threshold, n)));
  AG_CHECK_LAUNCH("threshold_backward");
  return Status::OK();
}

template <typename T>
__global__ void axpy_inplace_kernel(T* __restrict__ self, const T* __restrict__ other, float alpha, NdIndex idx, NdStrides<2> st, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t r = i, oa = 0, ob = 0;
    for (int d = idx.nd - 1; d >= 0; d--) {
      int64_t c = r % idx.shape[d]; r /= idx.shape[d];
      oa += c * st.s[0][d]; ob += c * st.s[1][d];
    }
    self[oa] = Cvt<T>::from(Cvt<T>::to(self[oa]) + alpha * Cvt<T>::to(other[ob]));
  }
}
Status add_scaled_inplace(cudaStream_t s, const TView& self, const TView& other, float alpha) {
  if (self.dtype != other.dtype) return Status::invalid(std::string("dtype mismatch: ") + dtype_debug(self.dtype) + " vs " + dtype_debug(other.dtype));
  int64_t n = self.numel();
  if (n == 0) return Status::OK();
  NdIndex idx; NdStrides<2> st;
  int64_t shape_tmp[kMaxDims], strides_tmp[2][kMaxDims];
  int nd = self.nd();
  Dims sb = broadcast_strides(other.shape, other.strides, self.shape);
  for (int d = 0; d < nd; d++) { shape_tmp[d] = self.shape[d]; strides_tmp[0][d] = self.strides[d]; strides_tmp[1][d] = sb[d]; }
  nd = collapse(nd, shape_tmp, strides_tmp, 2);
  idx.nd = nd;
  for (int d = 0; d < kMaxDims; d++) { idx.shape[d] = d < nd ? shape_tmp[d] : 1; st.s[0][d] = d < nd ? strides_tmp[0][d] : 0; st.s[1][d] = d < nd ? strides_tmp[1][d] : 0; }
  int grid = grid_for(n, 256, 8);
  AG_DISPATCH_FLOAT(self.dtype, T, (axpy_inplace_kernel<T><<<grid, 256, 0, s>>>((T*)self.ptr, (const T*)other.ptr, alpha, idx, st, n)));
  AG_CHECK_LAUNCH("add_scaled_inplace");
  return Status::OK();
}

// ── strided copy ────────────────────────────────────────────────────────────
template <typename E>
__global__ void __launch_bounds__(256) copy_strided_kernel(const E* __restrict__ src, E* __restrict__ dst, NdIndex idx, NdStrides<2> st, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t r = i, oa = 0, ob = 0;
    for (int d = idx.nd - 1; d >= 0; d--) {
      int64_t c = r % idx.shape[d]; r /= idx.shape[d];
      oa += c * st.s[0][d]; ob += c * st.s[1][d];
    }
    dst[ob] = src[oa];
  }
}

// One strided copy, prepared for launch: collapsed shape / strides in units of `w` bytes.
struct CopyJob {
  const void* src; void* dst;
  NdIndex idx; NdStrides<2> st;
  int64_t n;          // elements of width w
  bool flat;          // both sides are one contiguous run
};

static Status prepare_copy(const TView& src, const TView& dst, size_t max_w, CopyJob* job, size_t* width) {
  if (src.shape != dst.shape) return Status::compute("copy_strided shape mismatch " + dims_str(src.shape) + " vs " + dims_str(dst.shape));
  size_t esz = dtype_size(src.dtype);
  if (esz != dtype_size(dst.dtype)) return Status::compute("copy_strided element size mismatch");
  int64_t n = src.numel();
  if (n == 0) { job->src = src.ptr; job->dst = dst.ptr; job->n = 0; job->flat = true; job->idx.nd = 0; *width = esz; return Status::OK(); }
  int64_t shape_tmp[kMaxDims], strides_tmp[2][kMaxDims];
  int nd = src.nd();
  for (int d = 0; d < nd; d++) { shape_tmp[d] = src.shape[d]; strides_tmp[0][d] = src.strides[d]; strides_tmp[1][d] = dst.strides[d]; }
  nd = collapse(nd, shape_tmp, strides_tmp, 2);
  job->flat = nd == 1 && strides_tmp[0][0] == 1 && strides_tmp[1][0] == 1;
  // Widen the element to 16 bytes when the innermost runs allow it.
  size_t w = esz;
  int last = nd - 1;
  if (n > 0 && strides_tmp[0][last] == 1 && strides_tmp[1][last] == 1) {
    for (size_t cand : {16, 8, 4, 2}) {
      if (cand <= esz) break;
      if (cand > max_w) continue;
      int64_t ratio = (int64_t)(cand / esz);
      bool ok = shape_tmp[last] % ratio == 0 &&
                (reinterpret_cast<uintptr_t>(src.ptr) % cand) == 0 && (reinterpret_cast<uintptr_t>(dst.ptr) % cand) == 0;
      for (int d = 0; d < last && ok; d++) ok = strides_tmp[0][d] % ratio == 0 && strides_tmp[1][d] % ratio == 0;
      if (ok) {
        shape_tmp[last] /= ratio;
        for (int d = 0; d < last; d++) { strides_tmp[0][d] /= ratio; strides_tmp[1][d] /= ratio; }
        w = cand; n /= ratio;
        break;
      }
    }
  }
  job->src = src.ptr; job->dst = dst.ptr; job->n = n;
  job->idx.nd = nd;
  for (int d = 0; d < kMaxDims; d++) {
    job->idx.shape[d] = d < nd ? shape_tmp[d] : 1;
    job->st.s[0][d] = d < nd ? strides_tmp[0][d] : 0; job->st.s[1][d] = d < nd ? strides_tmp[1][d] : 0;
  }
  *width = w;
  return Status::OK();
}

Status copy_strided(cudaStream_t s, const TView& src, const TView& dst) {
  CopyJob job; size_t w;
  AG_RETURN_IF_ERROR(prepare_copy(src, dst, 16, &job, &w));
  if (src.numel() == 0) return Status::OK();
  if (job.flat) {
    cudaError_t e = cudaMemcpyAsync(dst.ptr, src.ptr, (size_t)src.numel() * dtype_size(src.dtype), cudaMemcpyDeviceToDevice, s);
    return cuda_status(e, "copy");
  }
  const NdIndex& idx = job.idx; const NdStrides<2>& st = job.st; const int64_t n = job.n;
  int grid = grid_for(n, 256, 8);
  switch (w) {
    case 16: copy_strided_kernel<uint4><<<grid, 256, 0, s>>>((const uint4*)src.ptr, (uint4*)dst.ptr, idx, st, n); break;
    case 8: copy_strided_kernel<uint64_t><<<grid, 256, 0, s>>>((const uint64_t*)src.ptr, (uint64_t*)dst.ptr, idx, st, n); break;
    case 4: copy_strided_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)src.ptr, (uint32_t*)dst.ptr, idx, st, n); break;
    case 2: copy_strided_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)src.ptr, (uint16_t*)dst.ptr, idx, st, n); break;
    default: copy_strided_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)src.ptr, (uint8_t*)dst.ptr, idx, st, n); break;
  }
  AG_CHECK_LAUNCH("copy_strided");
  return Status::OK();
}

// Two strided copies in one launch (the two halves of a concat): blocks [0, blocks_a) run the first job,
// the rest the second; both use the widest element both allow.
template <typename E>
__global__ void __launch_bounds__(256) copy_strided_pair_kernel(CopyJob a, CopyJob b, int blocks_a) {
  const bool second = (int)blockIdx.x >= blocks_a;
  const CopyJob& j = second ? b : a;
  const int64_t nblocks = second ? (int64_t)gridDim.x - blocks_a : blocks_a;
  const int64_t first = second ? (int64_t)blockIdx.x - blocks_a : blockIdx.x;
  const E* __restrict__ src = reinterpret_cast<const E*>(j.src);
  E* __restrict__ dst = reinterpret_cast<E*>(j.dst);
  const int64_t stride = nblocks * blockDim.x;
  for (int64_t i = first * blockDim.x + threadIdx.x; i < j.n; i += stride) {
    int64_t r = i, oa = 0, ob = 0;
    for (int d = j.idx.nd - 1; d >= 0; d--) {
      int64_t c = r % j.idx.shape[d]; r /= j.idx.shape[d];
      oa += c * j.st.s[0][d]; ob += c * j.st.s[1][d];
    }
    dst[ob] = src[oa];
  }
}

Status copy_strided_pair(cudaStream_t s, const TView& src_a, const TView& dst_a, const TView& src_b, const TView& dst_b) {
  if (src_a.numel() == 0) return copy_strided(s, src_b, dst_b);
  if (src_b.numel() == 0) return copy_strided(s, src_a, dst_a);
  CopyJob ja, jb; size_t wa, wb;
  AG_RETURN_IF_ERROR(prepare_copy(src_a, dst_a, 16, &ja, &wa));
  AG_RETURN_IF_ERROR(prepare_copy(src_b, dst_b, 16, &jb, &wb));
  if (wa != wb) {
    const size_t w = wa < wb ? wa : wb;
    AG_RETURN_IF_ERROR(prepare_copy(src_a, dst_a, w, &ja, &wa));
    AG_RETURN_IF_ERROR(prepare_copy(src_b, dst_b, w, &jb, &wb));
    if (wa != wb) {   // one side cannot reach the common width (alignment): fall back to two launches
      AG_RETURN_IF_ERROR(copy_strided(s, src_a, dst_a));
      return copy_strided(s, src_b, dst_b);
    }
  }
  const int ga = grid_for(ja.n, 256, 8), gb = grid_for(jb.n, 256, 8);
  switch (wa) {
    case 16: copy_strided_pair_kernel<uint4><<<ga + gb, 256, 0, s>>>(ja, jb, ga); break;
    case 8: copy_strided_pair_kernel<uint64_t><<<ga + gb, 256, 0, s>>>(ja, jb, ga); break;
    case 4: copy_strided_pair_kernel<uint32_t><<<ga + gb, 256, 0, s>>>(ja, jb, ga); break;
    case 2: copy_strided_pair_kernel<uint16_t><<<ga + gb, 256, 0, s>>>(ja, jb, ga); break;
    default: copy_strided_pair_kernel<uint8_t><<<ga + gb, 256, 0, s>>>(ja, jb, ga); break;
  }
  AG_CHECK_LAUNCH("copy_strided_pair");
  return Status::OK();
}

// ── L2 flush ────────────────────────────────────────────────────────────────
__global__ void flush_kernel(uint4* p, int64_t n, uint32_t v) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = make_uint4(v, v, v, v);
}
Status flush_l2(cudaStream_t s, void* scratch, size_t bytes) {
  int64_t n = (int64_t)(bytes / 16);
  if (n == 0) return Status::OK();
  flush_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>((uint4*)scratch, n, 0u);
  AG_CHECK_LAUNCH("flush_l2");
  return Status::OK();
}

// ── fill ────────────────────────────────────────────────────────────────────
// out[i] = pattern for a contiguous run of n elements of 1, 2, 4 or 8 bytes (the bit pattern of the value in the
// tensor's own dtype, prepared by the caller): zero_ / fill_ of a frontend whose buffers live in device memory.
template <typename E>
__global__ void __launch_bounds__(256) fill_kernel(E* __restrict__ out, E value, int64_t n) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = value;
}
Status fill(cudaStream_t s, void* out, int elem_size, uint64_t pattern, int64_t n) {
  if (n <= 0) return Status::OK();
  int grid = grid_for(n, 256 * 4, 8);
  cudaError_t e;
  switch (elem_size) {
    case 1: e = launch_pdl(fill_kernel<uint8_t>, dim3(grid), dim3(256), 0, s, (uint8_t*)out, (uint8_t)pattern, n); break;
    case 2: e = launch_pdl(fill_kernel<uint16_t>, dim3(grid), dim3(256), 0, s, (uint16_t*)out, (uint16_t)pattern, n); break;
    case 4: e = launch_pdl(fill_kernel<uint32_t>, dim3(grid), dim3(256), 0, s, (uint32_t*)out, (uint32_t)pattern, n); break;
    case 8: e = launch_pdl(fill_kernel<unsigned long long>, dim3(grid), dim3(256), 0, s, (unsigned long long*)out, (unsigned long long)pattern, n); break;
    default: return Status::invalid("fill: element size must be 1, 2, 4 or 8 bytes");
  }
  if (e != cudaSuccess) return cuda_status(e, "fill");
  return Status::OK();
}

}}  // namespace ag::k
