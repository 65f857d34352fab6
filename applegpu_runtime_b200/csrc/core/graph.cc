#include "graph.h"
#include <algorithm>

namespace ag {

static const char* kOpNames[] = {
  "Add", "Sub", "Mul", "Div", "Neg", "Relu", "Exp", "Log", "Sqrt", "Matmul", "FusedElementwise", "Softmax", "LogSoftmax",
  "Transpose", "ScalarMul", "Tanh", "Sin", "Cos", "Gelu", "Sigmoid", "LayerNorm", "Embedding", "Reshape", "Slice", "Concat",
  "AddBias", "SoftmaxCausal", "Argmax", "Sum", "Mean", "Var", "Abs", "Sign", "Pow", "Clamp", "Where", "MaskedFill", "Triu", "Tril",
  "Gather", "IndexSelect", "Conv1d", "Conv2d", "BatchNorm", "MaxPool2d", "MaxPool2dWithIndices", "AvgPool2d",
  "SoftmaxBackward", "LayerNormBackward", "Conv2dBackwardInput", "Conv2dBackwardWeight", "Conv1dBackwardInput",
  "EmbeddingBackward", "BatchNormBackward", "ThresholdBackward", "TanhBackward", "SigmoidBackward", "GeluBackward",
  "GeluExact", "GeluExactBackward", "GeluTanhBackward", "MaxPool2dBackward", "Lt", "Gt", "Le", "Ge", "Eq", "Ne",
  "BitwiseAnd", "BitwiseOr", "BitwiseXor", "BitwiseNot", "Shl", "Shr", "Mod", "ElemMin", "ElemMax", "LogicalNot",
  "Cast", "Quantize", "Dequantize", "ScatterWrite", "ScatterAdd", "Amax",
  "FusedLinear", "FusedAttention", "FusedEmbedAdd", "MatmulInt8",
};
static_assert(sizeof(kOpNames) / sizeof(kOpNames[0]) == (size_t)Op::Count_, "op name table out of sync");

const char* op_debug_name(Op op) { return kOpNames[(size_t)op]; }

bool op_in_hot_path(Op op) {
  switch (op) {
    case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: case Op::Neg: case Op::Relu: case Op::Exp: case Op::Log:
    case Op::Sqrt: case Op::Matmul: case Op::FusedElementwise: case Op::Softmax: case Op::Transpose: case Op::ScalarMul:
    case Op::Tanh: case Op::Sin: case Op::Cos: case Op::Gelu: case Op::Sigmoid: case Op::LayerNorm: case Op::Embedding:
    case Op::Reshape: case Op::Slice: case Op::Concat: case Op::AddBias: case Op::SoftmaxCausal: case Op::Argmax:
    case Op::Sum: case Op::Mean: case Op::Abs: case Op::Sign: case Op::Gather: case Op::IndexSelect:
    case Op::ThresholdBackward: case Op::GeluExact: case Op::Cast: case Op::Quantize: case Op::Dequantize:
    case Op::FusedLinear: case Op::FusedAttention: case Op::FusedEmbedAdd: case Op::MatmulInt8:
      return true;
    default:
      return false;
  }
}

std::string OpKind::kernel_name() const {
  switch (op) {
    case Op::Add: return "elementwise_add"; case Op::Sub: return "elementwise_sub";
    case Op::Mul: return "elementwise_mul"; case Op::Div: return "elementwise_div";
    case Op::Neg: return "elementwise_neg"; case Op::Relu: return "elementwise_relu";
    case Op::Exp: return "elementwise_exp"; case Op::Log: return "elementwise_log";
    case Op::Sqrt: return "elementwise_sqrt"; case Op::Matmul: return "matmul";
    case Op::FusedElementwise: return function_name;
    case Op::Softmax: return "softmax"; case Op::LogSoftmax: return "log_softmax";
    case Op::Transpose: return "transpose"; case Op::ScalarMul: return "scalar_mul";
    case Op::Tanh: return "elementwise_tanh"; case Op::Sin: return "elementwise_sin"; case Op::Cos: return "elementwise_cos";
    case Op::Gelu: return "gelu"; case Op::Sigmoid: return "sigmoid"; case Op::LayerNorm: return "layer_norm";
    case Op::Embedding: return "embedding"; case Op::Reshape: return "reshape";
    case Op::Slice: return i0 == 0 ? "slice_dim0" : "slice_dim1";
    case Op::Concat: return i0 == 0 ? "concat_dim0" : "concat_dim1";
    case Op::AddBias: return "add_bias"; case Op::SoftmaxCausal: return "softmax_causal"; case Op::Argmax: return "argmax";
    case Op::Sum: return "sum"; case Op::Mean: return "mean"; case Op::Var: return "var";
    case Op::Abs: return "elementwise_abs"; case Op::Sign: return "elementwise_sign";
    case Op::Pow: return "pow"; case Op::Clamp: return "clamp"; case Op::Where: return "where";
    case Op::MaskedFill: return "masked_fill"; case Op::Triu: return "triu"; case Op::Tril: return "tril";
    case Op::Gather: return i0 == 0 ? "gather_dim0" : "gather_dim1";
    case Op::IndexSelect: return i0 == 0 ? "index_select_dim0" : "index_select_dim1";
    case Op::Conv1d: return "conv1d"; case Op::Conv2d: return "conv2d"; case Op::BatchNorm: return "batch_norm";
    case Op::MaxPool2d: return "max_pool2d"; case Op::MaxPool2dWithIndices: return "max_pool2d_idx";
    case Op::AvgPool2d: return "avg_pool2d"; case Op::SoftmaxBackward: return "softmax_backward";
    case Op::LayerNormBackward: return "layer_norm_backward"; case Op::Conv2dBackwardInput: return "conv2d_backward_input";
    case Op::Conv2dBackwardWeight: return "conv2d_backward_weight"; case Op::Conv1dBackwardInput: return "conv1d_backward_input";
    case Op::EmbeddingBackward: return "embedding_backward"; case Op::BatchNormBackward: return "batch_norm_backward";
    case Op::ThresholdBackward: return "threshold_backward"; case Op::TanhBackward: return "tanh_backward";
    case Op::SigmoidBackward: return "sigmoid_backward"; case Op::GeluBackward: return "gelu_backward";
    case Op::GeluExact: return "gelu_exact"; case Op::GeluExactBackward: return "gelu_exact_backward";
    case Op::GeluTanhBackward: return "gelu_tanh_backward"; case Op::MaxPool2dBackward: return "max_pool2d_backward";
    case Op::Lt: return "lt"; case Op::Gt: return "gt"; case Op::Le: return "le"; case Op::Ge: return "ge";
    case Op::Eq: return "eq"; case Op::Ne: return "ne";
    case Op::BitwiseAnd: return "bitwise_and"; case Op::BitwiseOr: return "bitwise_or"; case Op::BitwiseXor: return "bitwise_xor";
    case Op::BitwiseNot: return "bitwise_not"; case Op::Shl: return "shl"; case Op::Shr: return "shr"; case Op::Mod: return "mod";
    case Op::ElemMin: return "elem_min"; case Op::ElemMax: return "elem_max"; case Op::LogicalNot: return "logical_not";
    case Op::Cast: return "cast"; case Op::Quantize: return "quantize"; case Op::Dequantize: return "dequantize";
    case Op::ScatterWrite: return "scatter_write"; case Op::ScatterAdd: return "scatter_add"; case Op::Amax: return "amax";
    case Op::FusedLinear: return "fused_linear"; case Op::FusedAttention: return "fused_attention";
    case Op::FusedEmbedAdd: return "fused_embed_add"; case Op::MatmulInt8: return "matmul_int8";
    default: return "unknown";
  }
}

bool OpKind::is_elementwise() const {
  switch (op) {
    case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: case Op::Neg: case Op::Relu: case Op::Exp: case Op::Log:
    case Op::Sqrt: case Op::Tanh: case Op::Sin: case Op::Cos: case Op::Gelu: case Op::Sigmoid: case Op::Abs: case Op::Sign:
      return true;
    default: return false;
  }
}
bool OpKind::is_unary() const {
  switch (op) {
    case Op::Neg: case Op::Relu: case Op::Exp: case Op::Log: case Op::Sqrt: case Op::Tanh: case Op::Sin: case Op::Cos:
    case Op::Gelu: case Op::GeluExact: case Op::Sigmoid: case Op::Abs: case Op::Sign: case Op::BitwiseNot: case Op::LogicalNot:
      return true;
    default: return false;
  }
}

static void unique_inputs(const OpNode& n, std::vector<uint64_t>* out) {
  out->clear();
  for (uint64_t i : n.inputs) if (std::find(out->begin(), out->end(), i) == out->end()) out->push_back(i);
}

void Graph::add_node(OpNode n) {
  std::vector<uint64_t> u;
  unique_inputs(n, &u);
  for (uint64_t i : u) refs_[i]++;
  uint64_t id = n.id;
  nodes_[id] = std::move(n);
}
const OpNode* Graph::get_node(uint64_t id) const {
  auto it = nodes_.find(id);
  return it == nodes_.end() ? nullptr : &it->second;
}
OpNode* Graph::get_node_mut(uint64_t id) {
  auto it = nodes_.find(id);
  return it == nodes_.end() ? nullptr : &it->second;
}
bool Graph::remove_node(uint64_t id, OpNode* out) {
  auto it = nodes_.find(id);
  if (it == nodes_.end()) return false;
  std::vector<uint64_t> u;
  unique_inputs(it->second, &u);
  for (uint64_t i : u) {
    auto r = refs_.find(i);
    if (r != refs_.end()) { if (--r->second == 0) refs_.erase(r); }
  }
  if (out) *out = std::move(it->second);
  nodes_.erase(it);
  return true;
}
size_t Graph::ref_count(uint64_t id) const {
  auto r = refs_.find(id);
  return r == refs_.end() ? 0 : r->second;
}

Status Graph::topo_sort(uint64_t target, std::vector<uint64_t>* order) const {
  order->clear();
  if (!has_node(target)) return Status::graph("Node " + std::to_string(target) + " not found in graph");
  std::unordered_set<uint64_t> visited;
  // iterative post-order DFS (a 36-layer model records thousands of nodes; no recursion)
  struct Frame { uint64_t id; size_t next; };
  std::vector<Frame> stack;
  stack.push_back({target, 0});
  visited.insert(target);
  while (!stack.empty()) {
    Frame& f = stack.back();
    const OpNode* n = get_node(f.id);
    if (n && f.next < n->inputs.size()) {
      uint64_t in = n->inputs[f.next++];
      if (has_node(in) && !visited.count(in)) { visited.insert(in); stack.push_back({in, 0}); }
    } else {
      order->push_back(f.id);
      stack.pop_back();
    }
  }
  return Status::OK();
}

std::vector<std::vector<uint64_t>> Graph::parallel_levels(const std::vector<uint64_t>& order) const {
  std::unordered_map<uint64_t, size_t> level;
  size_t max_level = 0;
  for (uint64_t id : order) {
    const OpNode* n = get_node(id);
    size_t l = 0;
    if (n) for (uint64_t in : n->inputs) {
      auto it = level.find(in);
      if (it != level.end() && it->second + 1 > l) l = it->second + 1;
    }
    level[id] = l;
    if (l > max_level) max_level = l;
  }
  std::vector<std::vector<uint64_t>> out(order.empty() ? 0 : max_level + 1);
  for (uint64_t id : order) out[level[id]].push_back(id);
  return out;
}

}  // namespace ag
