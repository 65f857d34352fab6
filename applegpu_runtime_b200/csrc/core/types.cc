#include "types.h"

namespace ag {

bool dtype_from_name(const std::string& n, DType* out) {
  struct E { const char* a; const char* b; DType d; };
  static const E table[] = {
    {"float16", "f16", DType::F16}, {"float32", "f32", DType::F32}, {"float64", "f64", DType::F64},
    {"int8", "i8", DType::I8}, {"int16", "i16", DType::I16}, {"int32", "i32", DType::I32},
    {"int64", "i64", DType::I64}, {"uint8", "u8", DType::U8}, {"uint32", "u32", DType::U32},
    {"bool", "bool_", DType::Bool}, {"bfloat16", "bf16", DType::BF16},
  };
  for (auto& e : table) if (n == e.a || n == e.b) { *out = e.d; return true; }
  return false;
}

std::string Status::to_string() const {
  switch (kind) {
    case ErrKind::Ok: return "";
    case ErrKind::DeviceNotAvailable: return msg.empty() ? "CUDA GPU device not available" : msg;
    case ErrKind::BackendNotInitialized: return "Backend not initialized, call init_backend() first";
    case ErrKind::InvalidTensor: return "Invalid tensor: " + msg;
    case ErrKind::BufferAllocationFailed: return "Failed to allocate GPU buffer of " + msg + " bytes";
    case ErrKind::ComputeFailed: return "Compute failed: " + msg;
    case ErrKind::GraphError: return "Graph error: " + msg;
    case ErrKind::ResourceLimitExceeded: return "Resource limit exceeded: " + msg;
    case ErrKind::UnsupportedDtype: return "Unsupported dtype: " + msg;
    case ErrKind::ImmutableBuffer: return "Tensor " + msg + " has a borrowed (immutable) buffer and cannot be used as output";
  }
  return msg;
}

std::string dims_str(const Dims& d) {
  std::ostringstream os;
  os << "[";
  for (size_t i = 0; i < d.size(); i++) { if (i) os << ", "; os << d[i]; }
  os << "]";
  return os.str();
}

Dims contiguous_strides(const Dims& shape) {
  Dims s(shape.size(), 0);
  int64_t acc = 1;
  for (int i = (int)shape.size() - 1; i >= 0; i--) { s[i] = acc; acc *= shape[i]; }
  return s;
}

bool is_contiguous(const Dims& shape, const Dims& strides) {
  int64_t expected = 1;
  for (int i = (int)shape.size() - 1; i >= 0; i--) {
    if (shape[i] != 1 && strides[i] != expected) return false;
    expected *= shape[i];
  }
  return true;
}

Status check_ndim(const Dims& d) {
  if ((int)d.size() > kMaxDims) {
    return Status::invalid("Shape has " + std::to_string(d.size()) + " dimensions, maximum is " + std::to_string(kMaxDims));
  }
  return Status::OK();
}

Status broadcast_shapes(const Dims& a, const Dims& b, Dims* out) {
  size_t n = a.size() > b.size() ? a.size() : b.size();
  Dims o(n, 1);
  for (size_t i = 0; i < n; i++) {
    int64_t x = i < a.size() ? a[a.size() - 1 - i] : 1;
    int64_t y = i < b.size() ? b[b.size() - 1 - i] : 1;
    int64_t r;
    if (x == y) r = x; else if (x == 1) r = y; else if (y == 1) r = x;
    else {
      return Status::invalid("Cannot broadcast shapes " + dims_str(a) + " and " + dims_str(b) + ": dim " +
                             std::to_string(n - 1 - i) + " is " + std::to_string(x) + " vs " + std::to_string(y));
    }
    o[n - 1 - i] = r;
  }
  *out = o;
  return Status::OK();
}

Dims broadcast_strides(const Dims& src_shape, const Dims& src_strides, const Dims& target) {
  Dims s(target.size(), 0);
  size_t off = target.size() - src_shape.size();
  for (size_t i = 0; i < src_shape.size(); i++) {
    s[i + off] = (src_shape[i] == target[i + off]) ? src_strides[i] : 0;
  }
  return s;
}

}  // namespace ag
