// Shape / dtype validation and output inference for every op on the hot path.
//
// Restates crates/core/src/ops.rs: validate_op_dtype (:29-163), binary/unary recorders
// (:171-216), matmul (:390-460), softmax (:487-506), transpose_dims (:510-552), scalar_mul,
// reshape (:570-592), layer_norm (:618-651), embedding (:1194-1230), slice / concat
// (:1234-1316), add_bias (:1322-1361), softmax_causal (:1367-1386), argmax (:1390-1413),
// gather / index_select (:1729-1829), quantize / dequantize / cast (:2250-2320).
// Error texts follow the reference so its tests' message checks carry over.
#include "runtime.h"

namespace ag {

static Status validate_compute_dtype(DType dt) {
  if (dt == DType::F64) return Status::unsupported("Float64 is not supported for GPU compute. Cast to Float32 first.");
  return Status::OK();
}

Status validate_op_dtype(const OpKind& kind, DType dt) {
  AG_RETURN_IF_ERROR(validate_compute_dtype(dt));
  const char* nm = op_debug_name(kind.op);
  auto is_int4 = [&] { return dt == DType::I32 || dt == DType::I64 || dt == DType::U8 || dt == DType::U32; };
  switch (kind.op) {
    case Op::Exp: case Op::Log: case Op::Sqrt: case Op::Tanh: case Op::Sin: case Op::Cos: case Op::Relu: case Op::Gelu:
    case Op::GeluExact: case Op::Sigmoid: case Op::Softmax: case Op::LogSoftmax: case Op::SoftmaxCausal: case Op::Matmul:
    case Op::LayerNorm: case Op::BatchNorm: case Op::Conv1d: case Op::Conv2d: case Op::MaxPool2d: case Op::MaxPool2dWithIndices:
    case Op::AvgPool2d: case Op::AddBias: case Op::Embedding: case Op::Mean: case Op::Var: case Op::Amax:
    case Op::SoftmaxBackward: case Op::LayerNormBackward: case Op::Conv2dBackwardInput: case Op::Conv2dBackwardWeight:
    case Op::Conv1dBackwardInput: case Op::EmbeddingBackward: case Op::ScatterWrite: case Op::ScatterAdd:
    case Op::BatchNormBackward: case Op::ThresholdBackward: case Op::TanhBackward: case Op::SigmoidBackward:
    case Op::GeluBackward: case Op::GeluTanhBackward: case Op::GeluExactBackward: case Op::MaxPool2dBackward:
    case Op::FusedLinear: case Op::FusedAttention: case Op::FusedEmbedAdd: case Op::MatmulInt8:
      if (!dtype_is_float(dt)) return Status::unsupported(std::string(nm) + " requires a float dtype, got " + dtype_name(dt));
      return Status::OK();
    case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: case Op::Neg: case Op::Abs: case Op::Sign: case Op::Clamp:
    case Op::ScalarMul: case Op::Pow:
      if (dt == DType::Bool || dt == DType::I8 || dt == DType::I16)
        return Status::unsupported(std::string(nm) + " does not support " + dtype_name(dt));
      return Status::OK();
    case Op::Cast: case Op::Reshape: case Op::Transpose: case Op::Slice: case Op::Concat: case Op::Where: case Op::MaskedFill:
    case Op::Triu: case Op::Tril:
      return Status::OK();
    case Op::Gather: case Op::IndexSelect: case Op::Sum: case Op::Argmax:
      if (dt == DType::Bool) return Status::unsupported(std::string(nm) + " does not support bool dtype");
      return Status::OK();
    case Op::Lt: case Op::Gt: case Op::Le: case Op::Ge: case Op::ElemMin: case Op::ElemMax:
      if (!(dtype_is_float(dt) || is_int4())) return Status::unsupported(std::string(nm) + " does not support " + dtype_name(dt));
      return Status::OK();
    case Op::Eq: case Op::Ne:
      if (!(dtype_is_float(dt) || is_int4() || dt == DType::Bool)) return Status::unsupported(std::string(nm) + " does not support " + dtype_name(dt));
      return Status::OK();
    case Op::BitwiseAnd: case Op::BitwiseOr: case Op::BitwiseXor: case Op::BitwiseNot:
      if (!(is_int4() || dt == DType::Bool)) return Status::unsupported(std::string(nm) + " requires an integer or Bool dtype, got " + dtype_name(dt));
      return Status::OK();
    case Op::Shl: case Op::Shr: case Op::Mod:
      if (!is_int4()) return Status::unsupported(std::string(nm) + " requires an integer dtype, got " + dtype_name(dt));
      return Status::OK();
    case Op::LogicalNot:
      if (dt != DType::Bool) return Status::unsupported(std::string("LogicalNot requires Bool dtype, got ") + dtype_name(dt));
      return Status::OK();
    default:
      return Status::OK();
  }
}

static Status need_inputs(const OpNode& n, size_t k) {
  if (n.inputs.size() != k)
    return Status::invalid(std::string(op_debug_name(n.op.op)) + " expects " + std::to_string(k) + " inputs, got " + std::to_string(n.inputs.size()));
  return Status::OK();
}

Status infer_node(const MetaSource& src, OpNode* node) {
  OpKind& k = node->op;
  const std::vector<uint64_t>& in = node->inputs;
  auto shp = [&](size_t i, Dims* d) { return src.shape(in[i], d); };
  auto dty = [&](size_t i, DType* d) { return src.dtype(in[i], d); };

  if (!op_in_hot_path(k.op))
    return Status::compute(std::string(op_debug_name(k.op)) + " is unsupported on this backend (outside the transformer forward op set)");

  switch (k.op) {
    case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      DType a, b; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(dty(1, &b));
      if (a != b) return Status::invalid(std::string("Dtype mismatch: ") + dtype_debug(a) + " vs " + dtype_debug(b));
      AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      Dims sa, sb; AG_RETURN_IF_ERROR(shp(0, &sa)); AG_RETURN_IF_ERROR(shp(1, &sb));
      AG_RETURN_IF_ERROR(check_ndim(sa)); AG_RETURN_IF_ERROR(check_ndim(sb));
      AG_RETURN_IF_ERROR(broadcast_shapes(sa, sb, &node->out_shape));
      node->out_dtype = a;
      return Status::OK();
    }
    case Op::Neg: case Op::Relu: case Op::Exp: case Op::Log: case Op::Sqrt: case Op::Tanh: case Op::Sin: case Op::Cos:
    case Op::Gelu: case Op::GeluExact: case Op::Sigmoid: case Op::Abs: case Op::Sign: case Op::ScalarMul: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a));
      AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      AG_RETURN_IF_ERROR(shp(0, &node->out_shape));
      AG_RETURN_IF_ERROR(check_ndim(node->out_shape));
      node->out_dtype = a;
      return Status::OK();
    }
    case Op::Matmul: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      DType a, b; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      AG_RETURN_IF_ERROR(dty(1, &b)); AG_RETURN_IF_ERROR(validate_op_dtype(k, b));
      Dims sa, sb; AG_RETURN_IF_ERROR(shp(0, &sa)); AG_RETURN_IF_ERROR(shp(1, &sb));
      if (sa.size() < 2) return Status::invalid("matmul requires at least 2D tensors, got " + dims_str(sa));
      if (sb.size() < 2) return Status::invalid("matmul requires at least 2D tensors, got " + dims_str(sb));
      if (a != b) return Status::invalid(std::string("Dtype mismatch: ") + dtype_debug(a) + " vs " + dtype_debug(b));
      int64_t m = sa[sa.size() - 2], k1 = sa[sa.size() - 1], k2 = sb[sb.size() - 2], n = sb[sb.size() - 1];
      if (k1 != k2)
        return Status::invalid("matmul inner dimensions mismatch: A[...," + std::to_string(m) + "," + std::to_string(k1) + "] * B[...," +
                               std::to_string(k2) + "," + std::to_string(n) + "]");
      Dims ba(sa.begin(), sa.end() - 2), bb(sb.begin(), sb.end() - 2), bo;
      bool both2d = ba.empty() && bb.empty();
      if (ba.empty()) ba = {1};
      if (bb.empty()) bb = {1};
      AG_RETURN_IF_ERROR(broadcast_shapes(ba, bb, &bo));
      if (both2d) bo.clear();
      bo.push_back(m); bo.push_back(n);
      AG_RETURN_IF_ERROR(check_ndim(bo));
      node->out_shape = bo; node->out_dtype = a;
      return Status::OK();
    }
    case Op::FusedLinear: {
      // recorded directly (applegpu_ffi_linear_fused): x [.., M, K] @ w [K, N] with the epilogue inputs that follow
      size_t want = 2 + (k.has_bias ? 1 : 0) + (k.has_residual ? 1 : 0) + (k.has_ln ? 2 : 0) + (k.has_stats_out ? 1 : 0) + (k.has_stats_zero ? 1 : 0);
      AG_RETURN_IF_ERROR(need_inputs(*node, want));
      DType a, w; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(dty(1, &w));
      AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      if (w != a) return Status::invalid(std::string("dtype mismatch: ") + dtype_debug(a) + " vs " + dtype_debug(w));
      Dims sa, sw; AG_RETURN_IF_ERROR(shp(0, &sa)); AG_RETURN_IF_ERROR(shp(1, &sw));
      if (sa.size() < 2 || sw.size() != 2) return Status::invalid("linear_fused requires x >= 2D and a 2D [K,N] weight");
      if (sa.back() != sw[0]) return Status::invalid("matmul inner dim mismatch: " + std::to_string(sa.back()) + " vs " + std::to_string(sw[0]));
      Dims so = sa; so.back() = sw[1];
      const int64_t rows = numel_of(so) / (sw[1] ? sw[1] : 1);
      size_t idx = 2;
      if (k.has_bias) { Dims sb; AG_RETURN_IF_ERROR(shp(idx++, &sb)); if (sb.size() != 1 || sb[0] != sw[1]) return Status::invalid("linear_fused bias must be [" + std::to_string(sw[1]) + "]"); }
      if (k.has_residual) { Dims sr; AG_RETURN_IF_ERROR(shp(idx++, &sr)); if (sr != so) return Status::invalid("linear_fused residual shape " + dims_str(sr) + " must be " + dims_str(so)); }
      auto stats_ok = [&](size_t i, int64_t r) -> Status {
        Dims ss; DType sd; AG_RETURN_IF_ERROR(shp(i, &ss)); AG_RETURN_IF_ERROR(dty(i, &sd));
        if (sd != DType::I64 || ss.size() != 2 || ss[0] != r || ss[1] != 2) return Status::invalid("linear_fused row statistics must be Int64 [" + std::to_string(r) + ", 2], got " + dims_str(ss));
        return Status::OK();
      };
      if (k.has_ln) {
        Dims sc; DType cd; AG_RETURN_IF_ERROR(shp(idx, &sc)); AG_RETURN_IF_ERROR(dty(idx, &cd)); idx++;
        if (cd != DType::F32 || sc.size() != 1 || sc[0] != sw[1]) return Status::invalid("linear_fused column sums must be Float32 [" + std::to_string(sw[1]) + "]");
        AG_RETURN_IF_ERROR(stats_ok(idx++, numel_of(sa) / (sa.back() ? sa.back() : 1)));
      }
      if (k.has_stats_out) AG_RETURN_IF_ERROR(stats_ok(idx++, rows));
      if (k.has_stats_zero) AG_RETURN_IF_ERROR(stats_ok(idx++, rows));
      node->out_shape = so; node->out_dtype = a;
      return Status::OK();
    }
    case Op::MatmulInt8: {
      // x [.., M, K] (float) @ dequant(w_q [N, K] int8, scales [N] f32)^T -> [.., M, N]
      AG_RETURN_IF_ERROR(need_inputs(*node, 3));
      DType a, w, sc; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(dty(1, &w)); AG_RETURN_IF_ERROR(dty(2, &sc));
      AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      if (w != DType::I8) return Status::unsupported("matmul_int8 weight must be Int8");
      if (sc != DType::F32) return Status::unsupported("matmul_int8 scales must be Float32");
      Dims sa, sw, ss; AG_RETURN_IF_ERROR(shp(0, &sa)); AG_RETURN_IF_ERROR(shp(1, &sw)); AG_RETURN_IF_ERROR(shp(2, &ss));
      if (sa.size() < 2 || sw.size() != 2) return Status::invalid("matmul_int8 requires x >= 2D and a 2D [N,K] weight");
      if (sa.back() != sw[1]) return Status::invalid("matmul_int8 inner dimensions mismatch: " + std::to_string(sa.back()) + " vs " + std::to_string(sw[1]));
      if (ss.size() != 1 || ss[0] != sw[0]) return Status::invalid("matmul_int8 scales shape " + dims_str(ss) + " must be [" + std::to_string(sw[0]) + "]");
      node->out_shape = sa; node->out_shape.back() = sw[0]; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Softmax: case Op::SoftmaxCausal: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      Dims s; AG_RETURN_IF_ERROR(shp(0, &s));
      if (k.op == Op::Softmax && s.empty()) return Status::invalid("softmax requires at least 1D tensor");
      if (k.op == Op::SoftmaxCausal && s.size() < 2) return Status::invalid("softmax_causal requires at least 2D tensor, got " + dims_str(s));
      node->out_shape = s; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Transpose: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      Dims s; AG_RETURN_IF_ERROR(shp(0, &s));
      int64_t nd = (int64_t)s.size();
      if (k.i0 >= nd || k.i1 >= nd || k.i0 < 0 || k.i1 < 0)
        return Status::invalid("transpose dims (" + std::to_string(k.i0) + ", " + std::to_string(k.i1) + ") out of range for " + std::to_string(nd) + "D tensor");
      std::swap(s[k.i0], s[k.i1]);
      node->out_shape = s; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Reshape: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      Dims s; AG_RETURN_IF_ERROR(shp(0, &s));
      int64_t on = numel_of(s), nn = numel_of(k.shape);
      if (on != nn)
        return Status::invalid("Cannot reshape: old shape " + dims_str(s) + " has " + std::to_string(on) + " elements, new shape " +
                               dims_str(k.shape) + " has " + std::to_string(nn));
      AG_RETURN_IF_ERROR(check_ndim(k.shape));
      AG_RETURN_IF_ERROR(dty(0, &node->out_dtype));
      node->out_shape = k.shape;
      return Status::OK();
    }
    case Op::Slice: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      Dims s; AG_RETURN_IF_ERROR(shp(0, &s));
      if (k.i0 < 0 || k.i0 >= (int64_t)s.size()) return Status::invalid("slice dim " + std::to_string(k.i0) + " >= ndim " + std::to_string(s.size()));
      if (k.i1 >= k.i2) return Status::invalid("slice start " + std::to_string(k.i1) + " >= end " + std::to_string(k.i2));
      if (k.i2 > s[k.i0]) return Status::invalid("slice end " + std::to_string(k.i2) + " > shape[" + std::to_string(k.i0) + "] = " + std::to_string(s[k.i0]));
      s[k.i0] = k.i2 - k.i1;
      node->out_shape = s; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Concat: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      DType a, b; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a)); AG_RETURN_IF_ERROR(dty(1, &b));
      if (a != b) return Status::invalid(std::string("concat dtype mismatch: ") + dtype_debug(a) + " vs " + dtype_debug(b));
      Dims sa, sb; AG_RETURN_IF_ERROR(shp(0, &sa)); AG_RETURN_IF_ERROR(shp(1, &sb));
      if (sa.size() != sb.size()) return Status::invalid("concat ndim mismatch: " + dims_str(sa) + " vs " + dims_str(sb));
      if (k.i0 < 0 || k.i0 >= (int64_t)sa.size()) return Status::invalid("concat dim " + std::to_string(k.i0) + " >= ndim " + std::to_string(sa.size()));
      for (size_t i = 0; i < sa.size(); i++)
        if ((int64_t)i != k.i0 && sa[i] != sb[i])
          return Status::invalid("concat shape mismatch on dim " + std::to_string(i) + ": " + std::to_string(sa[i]) + " vs " + std::to_string(sb[i]));
      sa[k.i0] += sb[k.i0];
      node->out_shape = sa; node->out_dtype = a;
      return Status::OK();
    }
    case Op::LayerNorm: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 3));
      Dims s; AG_RETURN_IF_ERROR(shp(0, &s));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      if (s.empty()) return Status::invalid("layer_norm requires at least 1D input");
      int64_t cols = s.back();
      Dims g, b; AG_RETURN_IF_ERROR(shp(1, &g));
      if (!(g.size() == 1 && g[0] == cols)) return Status::invalid("gamma shape " + dims_str(g) + " must be [" + std::to_string(cols) + "]");
      AG_RETURN_IF_ERROR(shp(2, &b));
      if (!(b.size() == 1 && b[0] == cols)) return Status::invalid("beta shape " + dims_str(b) + " must be [" + std::to_string(cols) + "]");
      node->out_shape = s; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Embedding: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      Dims w, ix; DType wd, id;
      AG_RETURN_IF_ERROR(shp(0, &w)); AG_RETURN_IF_ERROR(dty(0, &wd)); AG_RETURN_IF_ERROR(shp(1, &ix)); AG_RETURN_IF_ERROR(dty(1, &id));
      AG_RETURN_IF_ERROR(validate_op_dtype(k, wd));
      if (w.size() != 2) return Status::invalid("embedding weights must be 2D [vocab_size, embed_dim]");
      if (ix.empty()) return Status::invalid("embedding indices must have at least 1 dimension");
      if (id != DType::I32) return Status::invalid(std::string("embedding indices must be Int32, got ") + dtype_debug(id));
      ix.push_back(w[1]);
      AG_RETURN_IF_ERROR(check_ndim(ix));
      node->out_shape = ix; node->out_dtype = wd;
      return Status::OK();
    }
    case Op::AddBias: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      DType a, b; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a)); AG_RETURN_IF_ERROR(dty(1, &b));
      if (a != b) return Status::invalid(std::string("add_bias dtype mismatch: ") + dtype_debug(a) + " vs " + dtype_debug(b));
      Dims s, bs; AG_RETURN_IF_ERROR(shp(0, &s)); AG_RETURN_IF_ERROR(shp(1, &bs));
      if (s.size() < 2) return Status::invalid("add_bias requires >= 2D input, got " + dims_str(s));
      if (bs.size() != 1) return Status::invalid("add_bias requires 1D bias, got " + dims_str(bs));
      if (bs[0] != s[1]) return Status::invalid("add_bias bias length " + std::to_string(bs[0]) + " != input dim 1 " + std::to_string(s[1]));
      node->out_shape = s; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Argmax: case Op::Sum: case Op::Mean: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      Dims s; AG_RETURN_IF_ERROR(shp(0, &s));
      const char* nm = k.op == Op::Argmax ? "argmax" : (k.op == Op::Sum ? "sum" : "mean");
      if (s.empty()) return Status::invalid(std::string(nm) + " requires at least 1D tensor");
      s.pop_back();
      if (s.empty()) s = {1};
      node->out_shape = s; node->out_dtype = k.op == Op::Argmax ? DType::I32 : a;
      return Status::OK();
    }
    case Op::Gather: case Op::IndexSelect: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      const bool g = k.op == Op::Gather;
      const std::string nm = g ? "gather" : "index_select";
      DType a, id; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      Dims s, ix; AG_RETURN_IF_ERROR(shp(0, &s)); AG_RETURN_IF_ERROR(shp(1, &ix)); AG_RETURN_IF_ERROR(dty(1, &id));
      if (id != DType::I32) return Status::invalid(nm + " indices must be Int32, got " + dtype_debug(id));
      if (s.size() != 2) return Status::invalid(nm + " currently supports only 2D tensors");
      if (g && ix.size() != 2) return Status::invalid("gather index must be 2D (same ndim as input)");
      if (!g && ix.size() != 1) return Status::invalid("index_select index must be 1D");
      if (k.i0 > 1 || k.i0 < 0) return Status::invalid(nm + " dim " + std::to_string(k.i0) + " not supported for 2D tensors (must be 0 or 1)");
      if (g) {
        if (k.i0 == 0 && ix[1] != s[1]) return Status::invalid("gather dim=0: index cols " + std::to_string(ix[1]) + " must match input cols " + std::to_string(s[1]));
        if (k.i0 == 1 && ix[0] != s[0]) return Status::invalid("gather dim=1: index rows " + std::to_string(ix[0]) + " must match input rows " + std::to_string(s[0]));
        node->out_shape = ix;
      } else {
        node->out_shape = k.i0 == 0 ? Dims{ix[0], s[1]} : Dims{s[0], ix[0]};
      }
      node->out_dtype = a;
      return Status::OK();
    }
    case Op::ThresholdBackward: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 2));
      DType a, b; AG_RETURN_IF_ERROR(dty(0, &a)); AG_RETURN_IF_ERROR(dty(1, &b)); AG_RETURN_IF_ERROR(validate_op_dtype(k, a));
      if (a != b) return Status::invalid(std::string("Dtype mismatch: ") + dtype_debug(a) + " vs " + dtype_debug(b));
      Dims sa, sb; AG_RETURN_IF_ERROR(shp(0, &sa)); AG_RETURN_IF_ERROR(shp(1, &sb));
      if (sa != sb) return Status::invalid("threshold_backward shape mismatch: " + dims_str(sa) + " vs " + dims_str(sb));
      node->out_shape = sa; node->out_dtype = a;
      return Status::OK();
    }
    case Op::Cast: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a));
      AG_RETURN_IF_ERROR(validate_op_dtype(k, a)); AG_RETURN_IF_ERROR(validate_op_dtype(k, k.dt));
      AG_RETURN_IF_ERROR(shp(0, &node->out_shape));
      node->out_dtype = k.dt;
      return Status::OK();
    }
    case Op::Quantize: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a));
      if (!dtype_is_float(a)) return Status::unsupported("Quantize input must be a float dtype");
      if (!(k.dt == DType::I8 || k.dt == DType::U8)) return Status::unsupported("Quantize target must be Int8 or UInt8");
      if (k.f0 == 0.0f) return Status::invalid("Quantize scale must be non-zero");
      AG_RETURN_IF_ERROR(validate_compute_dtype(a));
      AG_RETURN_IF_ERROR(shp(0, &node->out_shape));
      node->out_dtype = k.dt;
      return Status::OK();
    }
    case Op::Dequantize: {
      AG_RETURN_IF_ERROR(need_inputs(*node, 1));
      DType a; AG_RETURN_IF_ERROR(dty(0, &a));
      if (!(a == DType::I8 || a == DType::U8)) return Status::unsupported("Dequantize input must be Int8 or UInt8");
      if (!dtype_is_float(k.dt)) return Status::unsupported("Dequantize target must be a float dtype");
      AG_RETURN_IF_ERROR(validate_compute_dtype(k.dt));
      AG_RETURN_IF_ERROR(shp(0, &node->out_shape));
      node->out_dtype = k.dt;
      return Status::OK();
    }
    default:
      return Status::compute(std::string(op_debug_name(k.op)) + " cannot be recorded directly");
  }
}

}  // namespace ag
