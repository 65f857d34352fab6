// Tensor metadata shared by the host runtime and the kernel launchers.
//
// Mirrors the reference's crates/core/src/tensor.rs (DType :5-17, wire codes :59-91,
// MAX_DIMS :113, Shape :117-168, TensorLayout :189-246) and error.rs (Display strings
// :36-53), restated as plain C++ value types.
#pragma once
#include <cstdint>
#include <cstddef>
#include <string>
#include <vector>
#include <sstream>

namespace ag {

constexpr int kMaxDims = 8;

// Values are the wire codes of the reference (tensor.rs:59-73): they cross the C ABI as int8_t.
enum class DType : int8_t {
  F32 = 0, F16 = 1, F64 = 2, I8 = 3, I16 = 4, I32 = 5, I64 = 6, U8 = 7, U32 = 8, Bool = 9, BF16 = 10,
  Invalid = -1
};

inline bool dtype_from_wire(int v, DType* out) {
  if (v < 0 || v > 10) return false;
  *out = static_cast<DType>(v);
  return true;
}
inline size_t dtype_size(DType d) {
  switch (d) {
    case DType::Bool: case DType::I8: case DType::U8: return 1;
    case DType::F16: case DType::BF16: case DType::I16: return 2;
    case DType::F32: case DType::I32: case DType::U32: return 4;
    case DType::F64: case DType::I64: return 8;
    default: return 0;
  }
}
inline bool dtype_is_float(DType d) {
  return d == DType::F32 || d == DType::F16 || d == DType::BF16 || d == DType::F64;
}
// Lower-case name (tensor.rs `name()`), used in UnsupportedDtype messages.
inline const char* dtype_name(DType d) {
  switch (d) {
    case DType::F16: return "float16"; case DType::F32: return "float32"; case DType::F64: return "float64";
    case DType::I8: return "int8"; case DType::I16: return "int16"; case DType::I32: return "int32";
    case DType::I64: return "int64"; case DType::U8: return "uint8"; case DType::U32: return "uint32";
    case DType::Bool: return "bool"; case DType::BF16: return "bfloat16"; default: return "invalid";
  }
}
// Variant name as the reference's `{:?}` prints it, used in InvalidTensor messages.
inline const char* dtype_debug(DType d) {
  switch (d) {
    case DType::F16: return "Float16"; case DType::F32: return "Float32"; case DType::F64: return "Float64";
    case DType::I8: return "Int8"; case DType::I16: return "Int16"; case DType::I32: return "Int32";
    case DType::I64: return "Int64"; case DType::U8: return "UInt8"; case DType::U32: return "UInt32";
    case DType::Bool: return "Bool"; case DType::BF16: return "BFloat16"; default: return "Invalid";
  }
}
// Kernel-name suffix (kernel_templates.rs:24-38).
inline const char* dtype_suffix(DType d) {
  switch (d) {
    case DType::F32: return "_f32"; case DType::F16: return "_f16"; case DType::BF16: return "_bf16";
    case DType::I8: return "_i8"; case DType::I16: return "_i16"; case DType::I32: return "_i32";
    case DType::I64: return "_i64"; case DType::U8: return "_u8"; case DType::U32: return "_u32";
    case DType::Bool: return "_bool"; default: return "_f64";
  }
}
bool dtype_from_name(const std::string& n, DType* out);

// ── errors ──────────────────────────────────────────────────────────────────
enum class ErrKind {
  Ok, DeviceNotAvailable, BackendNotInitialized, InvalidTensor, BufferAllocationFailed, ComputeFailed,
  GraphError, ResourceLimitExceeded, UnsupportedDtype, ImmutableBuffer
};

struct Status {
  ErrKind kind = ErrKind::Ok;
  std::string msg;
  bool ok() const { return kind == ErrKind::Ok; }
  explicit operator bool() const { return ok(); }
  // Same text as the reference's `impl Display for GpuError` (error.rs:36-53).
  std::string to_string() const;
  static Status OK() { return Status(); }
  static Status invalid(std::string m) { return Status{ErrKind::InvalidTensor, std::move(m)}; }
  static Status unsupported(std::string m) { return Status{ErrKind::UnsupportedDtype, std::move(m)}; }
  static Status compute(std::string m) { return Status{ErrKind::ComputeFailed, std::move(m)}; }
  static Status graph(std::string m) { return Status{ErrKind::GraphError, std::move(m)}; }
  static Status limit(std::string m) { return Status{ErrKind::ResourceLimitExceeded, std::move(m)}; }
  static Status alloc_failed(size_t n) { return Status{ErrKind::BufferAllocationFailed, std::to_string(n)}; }
  static Status no_device(std::string m) { return Status{ErrKind::DeviceNotAvailable, std::move(m)}; }
};

#define AG_RETURN_IF_ERROR(expr) do { ::ag::Status _s = (expr); if (!_s.ok()) return _s; } while (0)

// ── shape / layout ──────────────────────────────────────────────────────────
using Dims = std::vector<int64_t>;

// `[a, b, c]` — the reference formats shapes with `{:?}` of a Vec<usize>.
std::string dims_str(const Dims& d);
inline int64_t numel_of(const Dims& d) { int64_t n = 1; for (auto x : d) n *= x; return n; }
Dims contiguous_strides(const Dims& shape);
bool is_contiguous(const Dims& shape, const Dims& strides);
// NumPy-style broadcast, right-aligned (tensor.rs:148-168). Error text matches the reference.
Status broadcast_shapes(const Dims& a, const Dims& b, Dims* out);
// Strides of `src` (given its real strides) viewed in `target`; 0 on broadcast dims.
Dims broadcast_strides(const Dims& src_shape, const Dims& src_strides, const Dims& target);
Status check_ndim(const Dims& d);

// What a kernel launcher sees: a device pointer plus element strides.
struct TView {
  void* ptr = nullptr;
  DType dtype = DType::F32;
  Dims shape;
  Dims strides;  // elements
  int64_t numel() const { return numel_of(shape); }
  bool contiguous() const { return is_contiguous(shape, strides); }
  int nd() const { return (int)shape.size(); }
  size_t nbytes() const { return (size_t)numel() * dtype_size(dtype); }
  static TView make(void* p, DType dt, const Dims& shape) {
    TView v; v.ptr = p; v.dtype = dt; v.shape = shape; v.strides = contiguous_strides(shape); return v;
  }
};

}  // namespace ag
