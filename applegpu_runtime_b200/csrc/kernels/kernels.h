// Host-side launchers for the sm_100a kernels. One entry per kernel family of the
// reference's crates/core/src/kernel_templates.rs; each launcher validates what the
// kernel needs (alignment, dtype) and enqueues on the given stream. Nothing here
// allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include "../core/types.h"

namespace ag { namespace k {

enum class BinOp : int { Add = 0, Sub, Mul, Div };
enum class UnOp : int {
  Neg = 0, Relu, Exp, Log, Sqrt, Tanh, Sin, Cos, Gelu, GeluExact, Sigmoid, Abs, Sign, Copy
};
enum class Act : int { None = 0, GeluTanh = 1, GeluErf = 2, Relu = 3 };

// Fused element-wise chain (reference: fusion.rs:167-238 emits MSL text; here the chain
// is a register program interpreted per element). Registers 0..n_inputs-1 hold the loaded
// leaf inputs; instruction i writes register n_inputs+i; the last register is stored.
struct FusedInstr { int8_t op; int8_t is_binary; int8_t a; int8_t b; };
constexpr int kFusedMaxInputs = 8;
constexpr int kFusedMaxInstrs = 24;
struct FusedProgram {
  int n_inputs = 0;
  int n_instrs = 0;
  FusedInstr instrs[kFusedMaxInstrs];
};

Status binary(cudaStream_t s, BinOp op, const TView& a, const TView& b, const TView& out);
Status unary(cudaStream_t s, UnOp op, const TView& in, const TView& out);
Status scalar_mul(cudaStream_t s, const TView& in, float scale, const TView& out);
Status fused_elementwise(cudaStream_t s, const FusedProgram& prog, const TView* ins, const TView& out);
// out[i] = act(in[i] + bias[(i / inner) % channels]); channels = dims[1], inner = prod(dims[2:]).
Status add_bias(cudaStream_t s, const TView& in, const TView& bias, Act act, const TView& out);
Status threshold_backward(cudaStream_t s, const TView& grad, const TView& in, float threshold, const TView& out);
// self += alpha * other (both contiguous or same-strided views).
Status add_scaled_inplace(cudaStream_t s, const TView& self, const TView& other, float alpha);

Status layer_norm(cudaStream_t s, const TView& in, const TView& gamma, const TView& beta, float eps, const TView& out);
// Row softmax over the last dim. causal: rows are the second-to-last dim, mask col > row.
Status softmax(cudaStream_t s, const TView& in, bool causal, const TView& out);
Status argmax(cudaStream_t s, const TView& in, const TView& out_i32);
Status sum_last(cudaStream_t s, const TView& in, const TView& out, bool mean);
Status sum_dim(cudaStream_t s, const TView& in, int dim, const TView& out);
Status mean_all(cudaStream_t s, const TView& in, const TView& out);

Status embedding(cudaStream_t s, const TView& weight, const TView& idx, const TView& out);
// out[i,:] = wte[tok[i],:] + wpe[pos[i],:] in one pass (token + position embedding).
Status embedding_add(cudaStream_t s, const TView& wte, const TView& tok, const TView& wpe, const TView& pos, const TView& out);
Status gather2d(cudaStream_t s, const TView& in, int dim, const TView& idx, const TView& out);
Status index_select2d(cudaStream_t s, const TView& in, int dim, const TView& idx, const TView& out);

Status quantize(cudaStream_t s, const TView& in, float scale, int zero_point, const TView& out);
Status dequantize(cudaStream_t s, const TView& in, float scale, int zero_point, const TView& out);
// Per-output-channel symmetric int8: w [N,K] float -> q [N,K] int8, scale[n] = max|w[n,:]|/127.
Status quantize_rows(cudaStream_t s, const TView& w, const TView& q, const TView& scales);
Status cast(cudaStream_t s, const TView& in, const TView& out);
// Strided gather-copy: dst (any strides) <- src (any strides), same shape and dtype size.
Status copy_strided(cudaStream_t s, const TView& src, const TView& dst);
// n contiguous elements of elem_size bytes set to the low bytes of `pattern`
Status fill(cudaStream_t s, void* out, int elem_size, uint64_t pattern, int64_t n);
// two strided copies in one launch (the halves of a concat)
Status copy_strided_pair(cudaStream_t s, const TView& src_a, const TView& dst_a, const TView& src_b, const TView& dst_b);

struct GemmEpilogue {
  const void* bias = nullptr;      // [N], same dtype as C
  const void* residual = nullptr;  // same layout as C
  Act act = Act::None;
  float alpha = 1.0f;              // applied to the accumulator before bias
  const float* b_scales = nullptr; // int8-weight path: per-output-channel scales [N]
  // Row argmax instead of a stored product (tensor-core kernels, unbatched): each row's best
  // (value rounded to the storage type, lowest column on ties) is merged into keys[row] with a 64-bit
  // atomic max; C is not written. keys must be zeroed first; argmax_finalize turns them into int32.
  unsigned long long* argmax_keys = nullptr;
  // layer_norm folded into the product (tensor-core kernels, unbatched, 16-bit C). A consumer whose A rows are the
  // un-normalised x computes rstd[i] * (acc[i][n] - mean[i] * ln_colsum[n]) before bias / activation, with mean and
  // rstd from ln_stats[i] = (sum, sum of squares) of row i over K in 2^-28 fixed point (int64); the weight must carry
  // gamma (W'[k][n] = gamma[k] * W[k][n], ln_colsum[n] = sum_k W'[k][n], bias[n] = sum_k beta[k] * W[k][n] + b[n]).
  // A producer adds the (sum, sum of squares) of every row it stores into stats_out with 64-bit integer atomics
  // (associative: the result does not depend on the order in which CTAs finish) and clears the same rows of stats_zero.
  const long long* ln_stats = nullptr;
  const float* ln_colsum = nullptr;
  float ln_eps = 1e-5f;
  long long* stats_out = nullptr;
  long long* stats_zero = nullptr;
};
struct GemmDesc {
  DType dtype;            // dtype of A and C (f32/f16/bf16)
  DType b_dtype;          // = dtype, or I8 for the weight-quantised path
  const void* a; const void* b; void* c;
  int64_t m, n, k;
  // Batch index = (outer, inner): `batch` outer entries, each with `batch_inner` inner entries,
  // so that a [B, heads, T, d] view with unrelated B and head strides needs no copy.
  int64_t batch, batch_inner = 1;
  // Element strides. a: [batch, m, k]; b: logical [batch, k, n]; c: [batch, m, n] with ldc.
  int64_t a_row, a_col, a_batch, a_batch_inner = 0;
  int64_t b_row, b_col, b_batch, b_batch_inner = 0;  // b_row = stride along k, b_col = stride along n
  int64_t c_row, c_batch, c_batch_inner = 0;
  // Operands are f16/bf16 but C, bias and residual are float32 (the split-precision fp32 product).
  bool c_f32 = false;
  // Prologue: layer_norm over A's rows (gamma, beta of length k, same dtype as A) before the product. Taken only by
  // the K-major skinny kernel (at most 16 rows against a [N, K] weight: a decode step), which stages A's rows whole.
  const void* ln_gamma = nullptr;
  const void* ln_beta = nullptr;
  float ln_eps = 1e-5f;
  GemmEpilogue ep;
};
Status matmul(cudaStream_t s, const GemmDesc& d);
// Chained products: up to kChainMax unbatched 16-bit products with [K, N] weights, each reading the previous one's
// result as its A operand, as ONE launch of the tensor-core kernel (a 256-row block of product g + 1 only needs the same
// rows of product g, so tiles of consecutive products overlap and the pipeline fills and drains once).
//   matmul_chain_candidate   d could be a link of a chain
//   matmul_chain_can_append  `next` may follow chain[0 .. count): it reads chain[count - 1]'s result, and no buffer of
//                            one product overlaps a buffer another one writes except row block by row block
//   matmul_chain             launches them (count >= 2; results are those of `matmul` on each in turn, bit for bit)
constexpr int kChainMax = 4;
constexpr int kChainFlagStride = 1024;       // row blocks of 256 rows per product
constexpr int kChainArenaInts = 1 << 18;     // tile lists kept on the device
void set_gemm_chain_min_rows(int64_t rows);   // products with fewer rows are never chained (default 4096; APPLEGPU_GEMM_CHAIN_MIN_ROWS)
int64_t gemm_chain_min_rows();
bool matmul_chain_candidate(const GemmDesc& d);
bool matmul_chain_can_append(const GemmDesc* chain, int count, const GemmDesc& next);
Status matmul_chain(cudaStream_t s, const GemmDesc* chain, int count);
int* chain_flags();
int* chain_arena();
// int8 [N, K] weights against f16 / bf16 activations: true when the tensor-core kernel takes the int8 operand as it
// lies and widens it in its own prologue (per-channel scales in the epilogue); false when the caller has to hand the
// kernel a 16-bit copy instead (a single row block, K not a multiple of 16, unaligned operands).
bool matmul_w8_fused_eligible(const GemmDesc& d);
// At most 16 rows against a weight stored [N, K] (rows along K): each warp streams four weight rows at a time, A's rows
// wait in shared memory as floats, no workspace, fixed summation order. Takes the layer_norm prologue of GemmDesc.
bool skinny_kmajor_eligible(const GemmDesc& d);
Status matmul_skinny_kmajor(cudaStream_t s, const GemmDesc& d);
// Reports which kernel family `matmul` would choose: "tcgen05" or "simt".
const char* matmul_path(const GemmDesc& d);
// fp32 -> three bf16 terms x = x0 + x1 + x2 (each the bf16 rounding of what the previous ones left), written
// six times in the order a product of two such sums is accumulated: out holds, for t = 0..5, term pattern[t]
// of the input, either side by side along the columns (stack_rows = false: out[r, t*cols + c], row pitch
// 6*cols) or block over block (stack_rows = true: out[t*rows + r, c]). `batches` matrices, strides in elements.
Status split_bf16x3(cudaStream_t s, const float* in, void* out_bf16, int64_t rows, int64_t cols, int64_t in_row_stride, int64_t batches,
                    int64_t in_batch_stride, bool stack_rows, bool b_side);
Status argmax_finalize(cudaStream_t s, const unsigned long long* keys, int32_t* out, int64_t rows);

struct AttnDesc {
  DType dtype;
  const void* q; const void* k; const void* v; void* o;
  int64_t batch, heads, tq, tk, d, dv; // leading dims = (batch, heads)
  int64_t q_b, q_h, q_t;               // element strides (last dim contiguous)
  int64_t k_b, k_h, k_t;
  int64_t v_b, v_h, v_t;
  int64_t o_b, o_h, o_t;
  float scale;
  bool causal;
};
// Single-kernel attention (tcgen05, d = dv = 64, f16/bf16, TMA-compatible views); `attention_fused_eligible`
// tells whether `attention` accepts the problem, otherwise the caller composes it from GEMMs.
bool attention_fused_eligible(const AttnDesc& d);
Status attention(cudaStream_t s, const AttnDesc& d);
// float32 form (CUDA-core multiply-adds, online softmax, d = dv = 64, 16-byte aligned rows; `o` and its strides
// take part in the eligibility test).
bool attention_f32_eligible(const AttnDesc& d);
Status attention_f32(cudaStream_t s, const AttnDesc& d);

// Fixed workspace of the kernel layer (pipeline status word + pinned mirror, skinny-GEMM partials):
// created once, when the device context is set up, so that no op call allocates.
Status init_device_workspace(cudaStream_t s);
int* matmul_status_word();          // the pipeline status word (a bounded wait that gives up records its code there)
// The layers of a GPT-2 decode step as one cooperative persistent kernel (decode.cu); `layers` is a device table built with
// decode_layers_fill_entry on the host (12 weight pointers per layer in the decoder's order, then the layer's caches).
Status decode_layers(cudaStream_t s, DType dt, const void* layers, int n_layer, int heads, int d, int t_max, int batch, const void* wte, const void* wpe,
                     const int32_t* tok, const int32_t* pos, const int* len_ptr, void* x, void* x2, void* att, unsigned int* bar, int* err);
size_t decode_layers_table_bytes(int n_layer);
void decode_layers_fill_entry(void* host_table, int l, const void* const* w12, void* kcache, void* vcache);
// Pipeline status word of the tcgen05 kernels: a bounded wait that gives up records a code there.
// status_snapshot enqueues a copy into pinned slot `slot` (0 .. status_slots()-1); once the stream, or
// an event recorded after the snapshot, has been waited for, status_take returns the value and, when
// it is non-zero, clears the device word. matmul_take_status does snapshot + wait + take on slot 0.
int status_slots();
Status status_snapshot(cudaStream_t s, int slot);
int status_take(cudaStream_t s, int slot);
int matmul_take_status(cudaStream_t s);
// Test hook: one thread waits (for at most limit_ns, capped at 50 ms) on a barrier nothing arrives at,
// records `code` in the status word and returns.
Status launch_wait_runs_out(cudaStream_t s, int code, unsigned long long limit_ns);

// Decode step against a preallocated KV cache [B, heads, t_max, 64]: writes the new token's key / value row at index
// *len_ptr and attends over rows 0 .. *len_ptr (q, k, v of the new token are the thirds of qkv's [B, 3 * heads * 64] rows).
// `part` non-null: q / k / v arrive as the `slabs` float partials [slab][16][3 * heads * 64] an unfinished projection left
// (decode_linear with partial_only); the kernel adds them, adds `bias` and rounds as the projection would have.
Status attention_decode(cudaStream_t s, DType dt, const void* qkv, void* kcache, void* vcache, void* out, const int* len_ptr, int batch, int heads,
                        int t_max, float scale, const float* part = nullptr, int slabs = 0, const void* bias = nullptr);
// Linear layer of a decode step (at most 16 rows against a [K, N] MODEL WEIGHT, i.e. a matrix no kernel of the step
// writes: its loads are issued ahead of the programmatic dependency wait); takes the layer_norm prologue of GemmDesc
// and the bias / activation / residual epilogue.
bool decode_linear_eligible(const GemmDesc& d);
// The split-K partials live in one of kDecodeRegions regions of the workspace, so that an unfinished result
// (partial_only: no last-CTA reduction; the consumer adds the partials up) survives until its consumer has run while
// other linears use another region. xp: the A operand is such an unfinished result, act(sum of xp_slabs partials +
// xp_bias) rounded to the storage type (d.a is then unused, d.k is the producer's n).
constexpr int kDecodeRegions = 3;
constexpr size_t kDecodeRegionFloats = (size_t)1 << 20;     // 4 MB each
struct DecodeLinearOpts {
  int region = 0;
  bool partial_only = false;
  const float* xp = nullptr; int xp_slabs = 0; const void* xp_bias = nullptr; Act xp_act = Act::None;
};
float* decode_partial_region(int region);
Status decode_linear(cudaStream_t s, const GemmDesc& d, const DecodeLinearOpts& o = DecodeLinearOpts());
// End of a decode step: history[step] = tok, pos_ids = len + 1, step and len advance (all in device memory).
// `keys` non-null: tok is first filled from the row-argmax keys of the LM head (and the keys cleared for the next step).
Status decode_finish(cudaStream_t s, int32_t* tok, int32_t* history, int32_t* pos_ids, int* step_ptr, int* len_ptr, int batch, int max_steps,
                     unsigned long long* keys = nullptr);
Status decode_reset(cudaStream_t s, int* counters, int32_t* pos_ids, int batch, int len);
// Programmatic dependent launch can be switched off for a region of host code (stream capture of a decode step).
void set_pdl_override(int on);   // -1 follow the environment, 0 off, 1 on
void set_sm_margin(int n);       // SMs kept out of the persistent kernels' grids

// Writes more than the L2 capacity so the next timed kernel starts cold.
Status flush_l2(cudaStream_t s, void* scratch, size_t bytes);

}}  // namespace ag::k
