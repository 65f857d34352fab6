// The op enum and the lazy DAG.
//
// Mirrors crates/core/src/graph.rs: `OpKind` (:42-163, same variant set and names),
// `kernel_name` (:168-255), `is_elementwise` (:273-280), `OpNode` (:485-498), and `Graph`
// with `topo_sort` (:541-579), `ref_count` (:582-586), `parallel_levels` (:595-620).
// Three variants at the end (FusedLinear, FusedAttention, FusedEmbedAdd) do not exist
// upstream: only the fusion pass creates them, they never cross the API.
#pragma once
#include <unordered_map>
#include <unordered_set>
#include <string>
#include <vector>
#include "types.h"
#include "../kernels/kernels.h"

namespace ag {

enum class Op : uint8_t {
  Add, Sub, Mul, Div, Neg, Relu, Exp, Log, Sqrt, Matmul, FusedElementwise, Softmax, LogSoftmax,
  Transpose, ScalarMul, Tanh, Sin, Cos, Gelu, Sigmoid, LayerNorm, Embedding, Reshape, Slice, Concat,
  AddBias, SoftmaxCausal, Argmax, Sum, Mean, Var, Abs, Sign, Pow, Clamp, Where, MaskedFill, Triu, Tril,
  Gather, IndexSelect, Conv1d, Conv2d, BatchNorm, MaxPool2d, MaxPool2dWithIndices, AvgPool2d,
  SoftmaxBackward, LayerNormBackward, Conv2dBackwardInput, Conv2dBackwardWeight, Conv1dBackwardInput,
  EmbeddingBackward, BatchNormBackward, ThresholdBackward, TanhBackward, SigmoidBackward, GeluBackward,
  GeluExact, GeluExactBackward, GeluTanhBackward, MaxPool2dBackward, Lt, Gt, Le, Ge, Eq, Ne,
  BitwiseAnd, BitwiseOr, BitwiseXor, BitwiseNot, Shl, Shr, Mod, ElemMin, ElemMax, LogicalNot,
  Cast, Quantize, Dequantize, ScatterWrite, ScatterAdd, Amax,
  // produced by the fusion pass only
  FusedLinear, FusedAttention, FusedEmbedAdd,
  // additive: int8-weight linear (per-output-channel scales), no upstream counterpart
  MatmulInt8,
  Count_
};

const char* op_debug_name(Op op);    // variant name, e.g. "SoftmaxCausal"
bool op_in_hot_path(Op op);          // has a CUDA kernel in this build

struct OpKind {
  Op op = Op::Add;
  // parameters (meaning depends on op)
  int64_t i0 = 0, i1 = 0, i2 = 0;    // Transpose{dim0,dim1}; Slice{dim,start,end}; Concat{dim}; Gather{dim}; Quantize{zero_point}
  float f0 = 0.f, f1 = 0.f;          // ScalarMul value; LayerNorm eps; Quantize scale; ThresholdBackward threshold
  DType dt = DType::F32;             // Cast/Quantize/Dequantize target
  Dims shape;                        // Reshape new_shape
  // FusedElementwise
  k::FusedProgram prog;
  std::string function_name;         // "fused_<n>" like the reference
  std::string expr;                  // human-readable expression of the chain
  // FusedLinear epilogue: inputs = [a, b, (bias), (residual), (ln_colsum, ln_stats), (stats_out), (stats_zero)]
  bool has_bias = false, has_residual = false, trans_b = false, causal = false;
  // layer_norm folded into the product (f1 = eps): has_ln reads per-row (sum, sum of squares) ([rows, 2] int64, fixed
  // point) and the weight's column sums; has_stats_out adds the stored rows' sums into such a tensor, has_stats_zero
  // clears another
  bool has_ln = false, has_stats_out = false, has_stats_zero = false;
  k::Act act = k::Act::None;

  // Base kernel name without dtype suffix (graph.rs:168-255).
  std::string kernel_name() const;
  bool is_elementwise() const;  // the fusible set (graph.rs:273-280)
  bool is_unary() const;
};

struct OpNode {
  uint64_t id = 0;
  OpKind op;
  std::vector<uint64_t> inputs;
  Dims out_shape;
  DType out_dtype = DType::F32;
};

class Graph {
 public:
  void add_node(OpNode n);
  bool has_node(uint64_t id) const { return nodes_.count(id) != 0; }
  const OpNode* get_node(uint64_t id) const;
  OpNode* get_node_mut(uint64_t id);
  bool remove_node(uint64_t id, OpNode* out = nullptr);
  size_t len() const { return nodes_.size(); }
  // Number of nodes that list `id` among their inputs.
  size_t ref_count(uint64_t id) const;
  // Post-order DFS from `target`: every pending ancestor before its consumers.
  Status topo_sort(uint64_t target, std::vector<uint64_t>* order) const;
  // Groups of mutually independent nodes, in dependency order.
  std::vector<std::vector<uint64_t>> parallel_levels(const std::vector<uint64_t>& order) const;
  const std::unordered_map<uint64_t, OpNode>& nodes() const { return nodes_; }

 private:
  std::unordered_map<uint64_t, OpNode> nodes_;
  // consumer counts kept incrementally so ref_count is O(1) (upstream scans every node)
  std::unordered_map<uint64_t, size_t> refs_;
};

}  // namespace ag
