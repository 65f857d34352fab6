// PrivateUse1 ("applegpu") backend for PyTorch over the C ABI of this library, for buffers that live in DEVICE memory.
//
// Plays the role of the reference's backend_cpp/applegpu_backend.cpp (allocator :139-169, copies :267-342, 39 aten
// registrations :1055-1096, CPU fallback :754-764, guard / hooks :1104-1150): torch tensors on device "applegpu" whose
// storage is a buffer of the eager runtime, aten ops routed to applegpu_eager_* calls, everything else through
// PyTorch's CPU fallback. The reference can memcpy / memset / from_blob through the pointers the ABI returns because
// its buffers are unified memory; here the pointers are CUDA device pointers and never dereferenced on the host:
//   * host <-> device bytes move with applegpu_eager_upload / applegpu_eager_download,
//   * device <-> device copies, zero_ and fill_ are kernels (applegpu_eager_copy / applegpu_eager_fill),
//   * a torch tensor (any dtype, sizes, strides, storage offset) is presented to the runtime as a typed view over its
//     storage's buffer (applegpu_eager_view_as) for the duration of one call.
// Written against include/applegpu_b200_ffi.h and include/applegpu_b200_ext.h only; links libapplegpu_b200.so.
#include <ATen/ATen.h>
#include <ATen/EmptyTensor.h>
#include <ATen/InferSize.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <ATen/native/CPUFallback.h>
#include <ATen/native/Resize.h>
#include <ATen/native/TensorShape.h>
#include <ATen/native/transformers/attention.h>
#include <c10/core/Allocator.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <torch/library.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "../../../include/applegpu_b200_ext.h"
#include "../../../include/applegpu_b200_ffi.h"

namespace {

const c10::Device kDev(c10::DeviceType::PrivateUse1, 0);

const char* last_error() {
  const char* m = applegpu_eager_last_error();
  return m ? m : "unknown error";
}

// ── storage: one runtime buffer per torch storage ────────────────────────────
struct Slot { uint64_t id; };
void release_slot(void* ctx) {
  auto* s = static_cast<Slot*>(ctx);
  if (s) { applegpu_eager_free(s->id); delete s; }
}

// Both runtimes of the library come up with the first allocation (not at load time: loading the extension on a
// machine without a GPU must not abort the process, the first tensor raises instead).
void ensure_runtime() {
  static const bool ready = [] {
    TORCH_CHECK(applegpu_ffi_init(), "applegpu: runtime init failed: ", applegpu_ffi_last_error() ? applegpu_ffi_last_error() : "unknown error");
    TORCH_CHECK(applegpu_eager_init(), "applegpu: eager runtime init failed: ", last_error());
    TORCH_CHECK(applegpu_host_visible() == 0, "applegpu: this backend keeps its buffers in device memory; unset APPLEGPU_HOST_VISIBLE");
    return true;
  }();
  (void)ready;
}

struct DeviceAllocator final : c10::Allocator {
  c10::DataPtr allocate(size_t nbytes) override {
    ensure_runtime();
    uint64_t dims[1] = {nbytes ? nbytes : 1};
    uint64_t id = 0;
    uint8_t* p = applegpu_eager_alloc(dims, 1, /*uint8*/ 7, &id);
    TORCH_CHECK(p != nullptr, "applegpu: allocation of ", nbytes, " bytes failed: ", last_error());
    return {p, new Slot{id}, &release_slot, kDev};
  }
  c10::DeleterFnPtr raw_deleter() const override { return nullptr; }
  void copy_data(void* dest, const void* src, std::size_t count) const override {
    // both pointers are starts of runtime buffers
    uint64_t d = applegpu_eager_find_by_data_ptr(static_cast<const uint8_t*>(dest));
    uint64_t s = applegpu_eager_find_by_data_ptr(static_cast<const uint8_t*>(src));
    TORCH_CHECK(d && s, "applegpu: copy_data between pointers the runtime does not own");
    copy_bytes(d, s, count);
  }
  // The first `count` bytes of buffer `src` into buffer `dst`, on the device.
  static void copy_bytes(uint64_t dst, uint64_t src, size_t count) {
    if (count == 0) return;
    uint64_t shape[1] = {count}, stride[1] = {1}, vd = 0, vs = 0;
    bool ok = applegpu_eager_view_as(dst, 7, shape, stride, 1, 0, &vd) != nullptr && applegpu_eager_view_as(src, 7, shape, stride, 1, 0, &vs) != nullptr;
    int32_t rc = ok ? applegpu_eager_copy(vd, vs) : -1;
    if (vd) applegpu_eager_free(vd);
    if (vs) applegpu_eager_free(vs);
    TORCH_CHECK(rc == 0, "applegpu: copy failed: ", last_error());
  }
};
DeviceAllocator g_allocator;

int8_t wire_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return 0; case at::kHalf: return 1; case at::kDouble: return 2; case at::kChar: return 3; case at::kShort: return 4;
    case at::kInt: return 5; case at::kLong: return 6; case at::kByte: return 7; case at::kBool: return 9; case at::kBFloat16: return 10;
    default: TORCH_CHECK(false, "applegpu: dtype ", t, " has no runtime code");
  }
}
bool is_float16_32(at::ScalarType t) { return t == at::kFloat || t == at::kHalf || t == at::kBFloat16; }
bool on_device(const at::Tensor& t) { return t.defined() && t.device().type() == c10::DeviceType::PrivateUse1; }
bool host_scalar(const at::Tensor& t) { return t.defined() && !on_device(t) && t.dim() == 0; }

// A tensor as the runtime sees it for one call: a typed strided view over the storage's buffer.
struct Handle {
  uint64_t id = 0;
  explicit Handle(const at::Tensor& t) {
    TORCH_CHECK(on_device(t), "applegpu: expected a tensor on device applegpu");
    auto* slot = static_cast<Slot*>(t.storage().data_ptr().get_context());
    TORCH_CHECK(slot != nullptr, "applegpu: tensor storage was not allocated by this backend");
    std::vector<uint64_t> shape(t.sizes().begin(), t.sizes().end()), strides(t.dim());
    if (t.is_contiguous()) {
      // torch calls a tensor contiguous whatever the strides of its size-1 dims are: hand over the canonical ones
      uint64_t run = 1;
      for (int64_t i = t.dim() - 1; i >= 0; i--) { strides[i] = run; run *= shape[i] ? shape[i] : 1; }
    } else {
      for (int64_t i = 0; i < t.dim(); i++) {
        TORCH_CHECK(t.stride(i) >= 0, "applegpu: negative strides are not supported");
        strides[i] = (uint64_t)t.stride(i);
      }
    }
    uint64_t one = 1;
    uint8_t* p = applegpu_eager_view_as(slot->id, wire_dtype(t.scalar_type()), shape.empty() ? &one : shape.data(), strides.empty() ? &one : strides.data(),
                                        (uint32_t)t.dim(), (uint64_t)t.storage_offset() * t.element_size(), &id);
    TORCH_CHECK(p != nullptr || t.numel() == 0, "applegpu: cannot view tensor: ", last_error());
  }
  ~Handle() { if (id) applegpu_eager_free(id); }
  Handle(const Handle&) = delete;
  Handle& operator=(const Handle&) = delete;
};

// A fresh contiguous runtime tensor (id, device pointer) as a torch tensor that owns it.
at::Tensor adopt(uint64_t id, uint8_t* ptr, at::IntArrayRef sizes, at::ScalarType dt) {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  size_t nbytes = (size_t)numel * c10::elementSize(dt);
  c10::DataPtr dp(ptr, new Slot{id}, &release_slot, kDev);
  c10::Storage storage(c10::Storage::use_byte_size_t(), nbytes, std::move(dp), &g_allocator, /*resizable=*/false);
  auto t = at::detail::make_tensor<c10::TensorImpl>(std::move(storage), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), c10::scalarTypeToTypeMeta(dt));
  t.unsafeGetTensorImpl()->set_sizes_contiguous(sizes);
  return t;
}

at::Tensor new_empty(at::IntArrayRef sizes, at::ScalarType dt) {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  size_t nbytes = (size_t)numel * c10::elementSize(dt);
  c10::Storage storage(c10::Storage::use_byte_size_t(), nbytes, g_allocator.allocate(nbytes), &g_allocator, /*resizable=*/true);
  auto t = at::detail::make_tensor<c10::TensorImpl>(std::move(storage), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), c10::scalarTypeToTypeMeta(dt));
  t.unsafeGetTensorImpl()->set_sizes_contiguous(sizes);
  return t;
}

// ── factories ────────────────────────────────────────────────────────────────
at::Tensor op_empty(c10::SymIntArrayRef size, std::optional<at::ScalarType> dtype, std::optional<at::Layout>, std::optional<at::Device>,
                    std::optional<bool>, std::optional<at::MemoryFormat>) {
  return new_empty(C10_AS_INTARRAYREF_SLOW(size), dtype.value_or(at::get_default_dtype_as_scalartype()));
}
at::Tensor op_empty_strided(c10::SymIntArrayRef size, c10::SymIntArrayRef stride, std::optional<at::ScalarType> dtype, std::optional<at::Layout>,
                            std::optional<at::Device>, std::optional<bool>) {
  auto sizes = C10_AS_INTARRAYREF_SLOW(size);
  auto strides = C10_AS_INTARRAYREF_SLOW(stride);
  at::ScalarType dt = dtype.value_or(at::get_default_dtype_as_scalartype());
  size_t nbytes = at::detail::computeStorageNbytes(sizes, strides, c10::elementSize(dt));
  c10::Storage storage(c10::Storage::use_byte_size_t(), nbytes, g_allocator.allocate(nbytes), &g_allocator, /*resizable=*/true);
  auto t = at::detail::make_tensor<c10::TensorImpl>(std::move(storage), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), c10::scalarTypeToTypeMeta(dt));
  t.unsafeGetTensorImpl()->set_sizes_and_strides(sizes, strides);
  return t;
}

// ── copies ───────────────────────────────────────────────────────────────────
at::Tensor device_contiguous(const at::Tensor& t) {
  if (t.is_contiguous()) return t;
  at::Tensor c = new_empty(t.sizes(), t.scalar_type());
  Handle hd(c), hs(t);
  TORCH_CHECK(applegpu_eager_copy(hd.id, hs.id) == 0, "applegpu: copy failed: ", last_error());
  return c;
}

void copy_into(const at::Tensor& dst, const at::Tensor& src) {
  if (dst.numel() == 0) return;
  if (on_device(dst) && !on_device(src)) {
    // host -> device: a contiguous host tensor of the destination's dtype and shape, uploaded in one piece
    at::Tensor host = src.to(dst.scalar_type()).expand_as(dst).contiguous();
    if (dst.is_contiguous()) {
      Handle hd(dst);
      TORCH_CHECK(applegpu_eager_upload(hd.id, host.data_ptr(), host.nbytes()) == 0, "applegpu: upload failed: ", last_error());
      applegpu_eager_synchronize();   // the host tensor may be a temporary
    } else {
      at::Tensor stage = new_empty(dst.sizes(), dst.scalar_type());
      { Handle hs(stage); TORCH_CHECK(applegpu_eager_upload(hs.id, host.data_ptr(), host.nbytes()) == 0, "applegpu: upload failed: ", last_error()); }
      applegpu_eager_synchronize();
      Handle hd(dst), hs(stage);
      TORCH_CHECK(applegpu_eager_copy(hd.id, hs.id) == 0, "applegpu: copy failed: ", last_error());
    }
    return;
  }
  if (!on_device(dst) && on_device(src)) {
    // device -> host: gather on the device if needed, one download (it waits for the stream), convert on the host
    at::Tensor dev = device_contiguous(src);
    at::Tensor host = at::empty(dev.sizes(), dst.options().dtype(dev.scalar_type()).device(at::kCPU));
    {
      Handle hs(dev);
      TORCH_CHECK(applegpu_eager_download(hs.id, host.data_ptr(), host.nbytes()) == 0, "applegpu: download failed: ", last_error());
    }
    dst.copy_(host);
    return;
  }
  // device -> device
  at::Tensor s = src;
  if (s.sizes() != dst.sizes()) s = s.expand_as(dst);
  if (s.scalar_type() != dst.scalar_type() && !(s.is_contiguous() && dst.is_contiguous())) {
    // converting copy of strided tensors: through the host (rare)
    at::Tensor h = at::empty(s.sizes(), s.options().device(at::kCPU));
    copy_into(h, s);
    copy_into(dst, h.to(dst.scalar_type()));
    return;
  }
  Handle hd(dst), hs(s);
  TORCH_CHECK(applegpu_eager_copy(hd.id, hs.id) == 0, "applegpu: copy failed: ", last_error());
}

at::Tensor& op_copy_(at::Tensor& self, const at::Tensor& src, bool) { copy_into(self, src); return self; }
at::Tensor op_copy_from(const at::Tensor& self, const at::Tensor& dst, bool) { copy_into(dst, self); return dst; }
// torch's resize_: the storage grows when the new extent does not fit (old bytes are kept), never shrinks.
void resize_to(const at::Tensor& self, at::IntArrayRef sizes) {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  size_t need = ((size_t)self.storage_offset() + (size_t)numel) * self.element_size();
  if (need > self.storage().nbytes()) {
    c10::DataPtr fresh = g_allocator.allocate(need);
    size_t old = self.storage().nbytes();
    auto* was = static_cast<Slot*>(self.storage().data_ptr().get_context());
    if (old > 0 && was) DeviceAllocator::copy_bytes(static_cast<Slot*>(fresh.get_context())->id, was->id, old);
    self.storage().set_data_ptr_noswap(std::move(fresh));
    self.storage().set_nbytes(need);
  }
  self.unsafeGetTensorImpl()->set_sizes_contiguous(sizes);
}
const at::Tensor& op_resize_(const at::Tensor& self, c10::SymIntArrayRef size, std::optional<at::MemoryFormat>) {
  resize_to(self, C10_AS_INTARRAYREF_SLOW(size));
  return self;
}
at::Tensor op_copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  if (dst.sizes() != self.sizes()) {
    if (on_device(dst)) resize_to(dst, self.sizes()); else dst.resize_(self.sizes());
  }
  copy_into(dst, self);
  return dst;
}

uint64_t bits_of(const at::Scalar& v, at::ScalarType dt) {
  uint64_t out = 0;
  switch (dt) {
    case at::kFloat: { float f = v.toFloat(); std::memcpy(&out, &f, 4); break; }
    case at::kDouble: { double d = v.toDouble(); std::memcpy(&out, &d, 8); break; }
    case at::kHalf: { at::Half h = v.toHalf(); std::memcpy(&out, &h, 2); break; }
    case at::kBFloat16: { at::BFloat16 h = v.toBFloat16(); std::memcpy(&out, &h, 2); break; }
    case at::kLong: { int64_t i = v.toLong(); std::memcpy(&out, &i, 8); break; }
    case at::kInt: { int32_t i = v.toInt(); std::memcpy(&out, &i, 4); break; }
    case at::kShort: { int16_t i = v.toShort(); std::memcpy(&out, &i, 2); break; }
    case at::kChar: { int8_t i = v.toChar(); std::memcpy(&out, &i, 1); break; }
    case at::kByte: { uint8_t i = v.toByte(); std::memcpy(&out, &i, 1); break; }
    case at::kBool: { uint8_t i = v.toBool() ? 1 : 0; std::memcpy(&out, &i, 1); break; }
    default: TORCH_CHECK(false, "applegpu: fill_ of dtype ", dt);
  }
  return out;
}
at::Tensor& op_fill_(at::Tensor& self, const at::Scalar& value) {
  if (self.numel() == 0) return self;
  Handle h(self);
  TORCH_CHECK(applegpu_eager_fill(h.id, bits_of(value, self.scalar_type())) == 0, "applegpu: fill failed: ", last_error());
  return self;
}
at::Tensor& op_zero_(at::Tensor& self) { return op_fill_(self, 0); }

// ── CPU fallback for everything the table below does not route ──────────────
void cpu_fallback(const c10::OperatorHandle& op, torch::jit::Stack* stack) { at::native::cpu_fallback(op, stack); }

template <typename... Args>
at::Tensor via_fallback(const char* name, const char* overload, Args&&... args) {
  auto op = c10::Dispatcher::singleton().findSchemaOrThrow(name, overload);
  torch::jit::Stack stack;
  torch::jit::push(stack, std::forward<Args>(args)...);
  at::native::cpu_fallback(op, &stack);
  return torch::jit::pop(stack).toTensor();
}

// ── element-wise and linear algebra ─────────────────────────────────────────
using BinaryFn = uint8_t* (*)(uint64_t, uint64_t, uint64_t*);
at::Tensor run_binary(BinaryFn fn, const at::Tensor& a, const at::Tensor& b) {
  Handle ha(a), hb(b);
  uint64_t out = 0;
  uint8_t* p = fn(ha.id, hb.id, &out);
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  return adopt(out, p, at::infer_size(a.sizes(), b.sizes()), a.scalar_type());
}
at::Tensor scaled(const at::Tensor& a, double factor) {
  Handle ha(a);
  uint64_t out = 0;
  uint8_t* p = applegpu_eager_scalar_mul(ha.id, (float)factor, &out);
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  return adopt(out, p, a.sizes(), a.scalar_type());
}
// A Python number on either side arrives as a 0-dim CPU tensor: it becomes a one-element device tensor (a fill
// kernel, no host copy) that the binary kernel broadcasts.
at::Tensor device_scalar(const at::Scalar& v, at::ScalarType dt) {
  at::Tensor t = new_empty({}, dt);
  Handle h(t);
  TORCH_CHECK(applegpu_eager_fill(h.id, bits_of(v, dt)) == 0, "applegpu: fill failed: ", last_error());
  return t;
}
bool float_on_device(const at::Tensor& t) { return on_device(t) && is_float16_32(t.scalar_type()) && t.numel() > 0; }
// Both operands as device tensors of one float dtype, or false (the caller falls back to the CPU kernel).
bool binary_operands(const at::Tensor& a, const at::Tensor& b, at::Tensor* oa, at::Tensor* ob) {
  if (float_on_device(a) && float_on_device(b) && a.scalar_type() == b.scalar_type()) { *oa = a; *ob = b; return true; }
  if (float_on_device(a) && host_scalar(b) && (b.is_floating_point() || isIntegralType(b.scalar_type(), true))) { *oa = a; *ob = device_scalar(b.item(), a.scalar_type()); return true; }
  if (float_on_device(b) && host_scalar(a) && (a.is_floating_point() || isIntegralType(a.scalar_type(), true))) { *oa = device_scalar(a.item(), b.scalar_type()); *ob = b; return true; }
  return false;
}

at::Tensor op_add(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) {
  at::Tensor x, y;
  if (binary_operands(a, b, &x, &y)) return run_binary(applegpu_eager_add, x, alpha.toDouble() == 1.0 ? y : scaled(y, alpha.toDouble()));
  return via_fallback("aten::add", "Tensor", a, b, alpha);
}
at::Tensor op_sub(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) {
  at::Tensor x, y;
  if (binary_operands(a, b, &x, &y)) return run_binary(applegpu_eager_sub, x, alpha.toDouble() == 1.0 ? y : scaled(y, alpha.toDouble()));
  return via_fallback("aten::sub", "Tensor", a, b, alpha);
}
at::Tensor op_mul(const at::Tensor& a, const at::Tensor& b) {
  if (float_on_device(a) && host_scalar(b)) return scaled(a, b.item<double>());
  if (float_on_device(b) && host_scalar(a)) return scaled(b, a.item<double>());
  at::Tensor x, y;
  if (binary_operands(a, b, &x, &y)) return run_binary(applegpu_eager_mul, x, y);
  return via_fallback("aten::mul", "Tensor", a, b);
}
at::Tensor op_div(const at::Tensor& a, const at::Tensor& b) {
  if (float_on_device(a) && host_scalar(b) && b.item<double>() != 0.0) return scaled(a, 1.0 / b.item<double>());
  at::Tensor x, y;
  if (binary_operands(a, b, &x, &y)) return run_binary(applegpu_eager_div, x, y);
  return via_fallback("aten::div", "Tensor", a, b);
}
at::Tensor op_add_scalar(const at::Tensor& a, const at::Scalar& v, const at::Scalar& alpha) {
  if (float_on_device(a)) return run_binary(applegpu_eager_add, a, device_scalar(v.toDouble() * alpha.toDouble(), a.scalar_type()));
  return via_fallback("aten::add", "Scalar", a, v, alpha);
}
at::Tensor op_mul_scalar(const at::Tensor& a, const at::Scalar& s) {
  if (float_on_device(a)) return scaled(a, s.toDouble());
  return via_fallback("aten::mul", "Scalar", a, s);
}
at::Tensor op_pow_scalar(const at::Tensor& a, const at::Scalar& e) {
  // small whole exponents as repeated products (the tanh form of GELU written out in Python uses x**3)
  double ev = e.toDouble();
  if (float_on_device(a) && (ev == 2.0 || ev == 3.0)) {
    at::Tensor sq = run_binary(applegpu_eager_mul, a, a);
    return ev == 2.0 ? sq : run_binary(applegpu_eager_mul, sq, a);
  }
  return via_fallback("aten::pow", "Tensor_Scalar", a, e);
}
at::Tensor& op_add_(at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha) {
  at::Tensor r = op_add(self, other, alpha);
  copy_into(self, r);
  return self;
}
at::Tensor& op_mul_(at::Tensor& self, const at::Tensor& other) {
  at::Tensor r = op_mul(self, other);
  copy_into(self, r);
  return self;
}

using UnaryFn = uint8_t* (*)(uint64_t, uint64_t*);
at::Tensor run_unary(UnaryFn fn, const at::Tensor& a) {
  Handle ha(a);
  uint64_t out = 0;
  uint8_t* p = fn(ha.id, &out);
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  return adopt(out, p, a.sizes(), a.scalar_type());
}
at::Tensor run_named(const char* name, const char* aten_name, const at::Tensor& a) {
  if (!float_on_device(a)) return via_fallback(aten_name, "", a);
  Handle ha(a);
  uint64_t out = 0;
  uint8_t* p = applegpu_eager_unary(ha.id, name, &out);
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  return adopt(out, p, a.sizes(), a.scalar_type());
}
at::Tensor op_relu(const at::Tensor& a) { return run_named("relu", "aten::relu", a); }
at::Tensor op_neg(const at::Tensor& a) { return run_named("neg", "aten::neg", a); }
at::Tensor op_tanh(const at::Tensor& a) { return run_named("tanh", "aten::tanh", a); }
at::Tensor op_exp(const at::Tensor& a) { return run_named("exp", "aten::exp", a); }
at::Tensor op_log(const at::Tensor& a) { return run_named("log", "aten::log", a); }
at::Tensor op_sqrt(const at::Tensor& a) { return run_named("sqrt", "aten::sqrt", a); }
at::Tensor op_sigmoid(const at::Tensor& a) { return run_named("sigmoid", "aten::sigmoid", a); }
at::Tensor op_abs(const at::Tensor& a) { return run_named("abs", "aten::abs", a); }
at::Tensor op_gelu(const at::Tensor& a, c10::string_view approximate) {
  if (float_on_device(a)) return run_unary(approximate == "tanh" ? applegpu_eager_gelu : applegpu_eager_gelu_exact, a);
  return via_fallback("aten::gelu", "", a, std::string(approximate));
}

// [.., M, K] @ [.., K, N]: the runtime's matmul takes contiguous operands and broadcasts leading dims
at::Tensor run_matmul(const at::Tensor& a, const at::Tensor& b) {
  at::Tensor ac = device_contiguous(a), bc = device_contiguous(b);
  Handle ha(ac), hb(bc);
  uint64_t out = 0;
  uint8_t* p = applegpu_eager_matmul(ha.id, hb.id, &out);
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  std::vector<int64_t> batch = at::infer_size(at::IntArrayRef(ac.sizes().data(), ac.dim() - 2), at::IntArrayRef(bc.sizes().data(), bc.dim() - 2));
  batch.push_back(ac.size(-2));
  batch.push_back(bc.size(-1));
  return adopt(out, p, batch, a.scalar_type());
}
// x [M,K] @ w [K,N] (+ bias [N]) in one GEMM launch: the bias is added in the epilogue and a transposed view of a
// contiguous [N,K] weight (nn.Linear's weight.t()) is read in place through its strides.
bool plain_or_transposed(const at::Tensor& w) { return w.dim() == 2 && (w.is_contiguous() || (w.stride(0) == 1 && w.stride(1) == w.size(0))); }
at::Tensor run_linear(const at::Tensor& x, const at::Tensor& w, const at::Tensor* bias) {
  at::Tensor xc = device_contiguous(x), wc = plain_or_transposed(w) ? w : device_contiguous(w);
  Handle hx(xc), hw(wc);
  uint64_t out = 0;
  uint8_t* p;
  if (bias) {
    at::Tensor bc = device_contiguous(*bias);
    Handle hb(bc);
    p = applegpu_eager_linear(hx.id, hw.id, hb.id, 0, 0, false, &out);
  } else {
    p = applegpu_eager_linear(hx.id, hw.id, 0, 0, 0, false, &out);
  }
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  return adopt(out, p, {x.size(0), w.size(1)}, x.scalar_type());
}
bool matmul_operands(const at::Tensor& a, const at::Tensor& b) {
  return float_on_device(a) && float_on_device(b) && a.scalar_type() == b.scalar_type();
}
at::Tensor op_mm(const at::Tensor& a, const at::Tensor& b) {
  if (matmul_operands(a, b) && a.dim() == 2 && b.dim() == 2) return run_linear(a, b, nullptr);
  return via_fallback("aten::mm", "", a, b);
}
at::Tensor op_bmm(const at::Tensor& a, const at::Tensor& b) {
  if (matmul_operands(a, b) && a.dim() == 3 && b.dim() == 3) return run_matmul(a, b);
  return via_fallback("aten::bmm", "", a, b);
}
at::Tensor op_addmm(const at::Tensor& bias, const at::Tensor& a, const at::Tensor& b, const at::Scalar& beta, const at::Scalar& alpha) {
  if (matmul_operands(a, b) && a.dim() == 2 && b.dim() == 2 && float_on_device(bias) && bias.scalar_type() == a.scalar_type() && beta.toDouble() == 1.0 &&
      alpha.toDouble() == 1.0) {
    if (bias.dim() == 1 && bias.size(0) == b.size(1)) return run_linear(a, b, &bias);
    return run_binary(applegpu_eager_add, run_linear(a, b, nullptr), bias);
  }
  return via_fallback("aten::addmm", "", bias, a, b, beta, alpha);
}

// Fused attention (softmax(Q K^T / sqrt(d)) V in one kernel) behind torch's scaled_dot_product_attention: the backend
// choice says "overrideable" for the calls the kernel covers and "math" (decomposed into the ops above) otherwise.
bool attention_covered(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const std::optional<at::Tensor>& mask, double dropout, bool causal,
                       std::optional<double> scale) {
  if (!(float_on_device(q) && float_on_device(k) && float_on_device(v))) return false;
  if (q.scalar_type() != k.scalar_type() || q.scalar_type() != v.scalar_type()) return false;
  if (mask.has_value() && mask->defined()) return false;
  if (dropout != 0.0 || q.dim() < 3 || q.dim() != k.dim() || q.dim() != v.dim()) return false;
  for (int64_t i = 0; i + 2 < q.dim(); i++) if (q.size(i) != k.size(i) || q.size(i) != v.size(i)) return false;
  if (k.size(-1) != q.size(-1) || k.size(-2) != v.size(-2)) return false;
  if (causal && q.size(-2) != k.size(-2)) return false;   // torch aligns the causal mask top-left when the lengths differ
  if (scale.has_value() && std::abs(*scale - 1.0 / std::sqrt((double)q.size(-1))) > 1e-12) return false;
  return true;
}
int64_t op_fused_sdp_choice(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const std::optional<at::Tensor>& mask, double dropout, bool causal,
                            std::optional<double> scale, bool enable_gqa) {
  constexpr int64_t kMath = 0, kOverrideable = 4;   // sdp::SDPBackend
  return (!enable_gqa && attention_covered(q, k, v, mask, dropout, causal, scale)) ? kOverrideable : kMath;
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor, at::Tensor, at::Tensor> op_sdp_overrideable(
    const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const std::optional<at::Tensor>& bias, double dropout, bool causal, bool, std::optional<double> scale) {
  TORCH_CHECK(attention_covered(q, k, v, bias, dropout, causal, scale), "applegpu: fused attention does not cover this call (mask, dropout, custom scale or unequal causal lengths)");
  at::Tensor qc = device_contiguous(q), kc = device_contiguous(k), vc = device_contiguous(v);
  Handle hq(qc), hk(kc), hv(vc);
  uint64_t out = 0;
  uint8_t* p = applegpu_eager_attention(hq.id, hk.id, hv.id, causal, &out);
  TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
  std::vector<int64_t> shape(q.sizes().begin(), q.sizes().end());
  shape.back() = v.size(-1);
  at::Tensor none = at::empty({0}, at::TensorOptions().dtype(at::kLong));
  // inference only: no log-sum-exp is kept for a backward pass
  return {adopt(out, p, shape, q.scalar_type()), new_empty({0}, at::kFloat), none, none, c10::SymInt(q.size(-2)), c10::SymInt(k.size(-2)), none, none, none};
}

at::Tensor op_softmax(const at::Tensor& a, int64_t dim, bool half_to_float) {
  int64_t d = dim < 0 ? dim + a.dim() : dim;
  if (on_device(a) && is_float16_32(a.scalar_type()) && !half_to_float && a.dim() >= 1 && d == a.dim() - 1 && a.numel() > 0) {
    at::Tensor c = device_contiguous(a);
    return run_unary(applegpu_eager_softmax, c);
  }
  return via_fallback("aten::_softmax", "", a, dim, half_to_float);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> op_native_layer_norm(const at::Tensor& x, c10::SymIntArrayRef normalized_shape, const std::optional<at::Tensor>& w,
                                                                   const std::optional<at::Tensor>& b, double eps) {
  auto ns = C10_AS_INTARRAYREF_SLOW(normalized_shape);
  if (on_device(x) && is_float16_32(x.scalar_type()) && ns.size() == 1 && x.dim() >= 1 && ns[0] == x.size(-1) && w.has_value() && b.has_value() &&
      w->defined() && b->defined() && on_device(*w) && on_device(*b) && w->scalar_type() == x.scalar_type() && b->scalar_type() == x.scalar_type() && x.numel() > 0) {
    at::Tensor xc = device_contiguous(x), wc = device_contiguous(*w), bc = device_contiguous(*b);
    Handle hx(xc), hw(wc), hb(bc);
    uint64_t out = 0;
    uint8_t* p = applegpu_eager_layer_norm(hx.id, hw.id, hb.id, (float)eps, &out);
    TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
    // inference only: the statistics outputs are not produced (the reference returns placeholders too, torch_backend.py:1392-1420)
    std::vector<int64_t> stat(x.sizes().begin(), x.sizes().end());
    stat.back() = 1;
    return {adopt(out, p, x.sizes(), x.scalar_type()), new_empty(stat, at::kFloat), new_empty(stat, at::kFloat)};
  }
  auto op = c10::Dispatcher::singleton().findSchemaOrThrow("aten::native_layer_norm", "");
  torch::jit::Stack stack;
  torch::jit::push(stack, x, normalized_shape, w, b, eps);
  at::native::cpu_fallback(op, &stack);
  auto r2 = torch::jit::pop(stack).toTensor(); auto r1 = torch::jit::pop(stack).toTensor(); auto r0 = torch::jit::pop(stack).toTensor();
  return {r0, r1, r2};
}

at::Tensor op_embedding(const at::Tensor& weight, const at::Tensor& indices, c10::SymInt padding_idx, bool scale_grad, bool sparse) {
  if (on_device(weight) && is_float16_32(weight.scalar_type()) && weight.dim() == 2 && indices.numel() > 0 &&
      (indices.scalar_type() == at::kLong || indices.scalar_type() == at::kInt)) {
    // the runtime gathers with int32 indices (kernel_templates.rs:1119-1143): int64 ids are narrowed by a cast kernel
    at::Tensor dev_idx;
    if (on_device(indices)) {
      at::Tensor ic = device_contiguous(indices);
      if (ic.scalar_type() == at::kInt) dev_idx = ic;
      else {
        Handle hi64(ic);
        uint64_t cid = 0;
        uint8_t* cp = applegpu_eager_cast(hi64.id, /*int32*/ 5, &cid);
        TORCH_CHECK(cp != nullptr, "applegpu: ", last_error());
        dev_idx = adopt(cid, cp, ic.sizes(), at::kInt);
      }
    } else {
      at::Tensor idx32 = indices.to(at::kInt).contiguous();
      dev_idx = new_empty(idx32.sizes(), at::kInt);
      copy_into(dev_idx, idx32);
    }
    at::Tensor wc = device_contiguous(weight);
    Handle hw(wc), hi(dev_idx);
    uint64_t out = 0;
    uint8_t* p = applegpu_eager_embedding(hw.id, hi.id, &out);
    TORCH_CHECK(p != nullptr, "applegpu: ", last_error());
    std::vector<int64_t> shape(indices.sizes().begin(), indices.sizes().end());
    shape.push_back(weight.size(1));
    return adopt(out, p, shape, weight.scalar_type());
  }
  return via_fallback("aten::embedding", "", weight, indices, padding_idx, scale_grad, sparse);
}

// cat: one strided copy kernel per input into its slice of the result (a KV cache append is a cat along the sequence)
at::Tensor op_cat(const at::ITensorListRef& tensors, int64_t dim) {
  std::vector<at::Tensor> parts;
  bool device_only = true;
  for (const at::Tensor& t : tensors) {
    if (t.dim() == 1 && t.numel() == 0) continue;      // the legacy "empty" operand of cat
    if (!on_device(t) || (!parts.empty() && (t.scalar_type() != parts[0].scalar_type() || t.dim() != parts[0].dim()))) device_only = false;
    parts.push_back(t);
  }
  if (!device_only || parts.empty()) {
    auto op = c10::Dispatcher::singleton().findSchemaOrThrow("aten::cat", "");
    torch::jit::Stack stack;
    torch::jit::push(stack, std::vector<at::Tensor>(tensors.begin(), tensors.end()), dim);
    at::native::cpu_fallback(op, &stack);
    return torch::jit::pop(stack).toTensor();
  }
  int64_t d = dim < 0 ? dim + parts[0].dim() : dim;
  TORCH_CHECK(d >= 0 && d < parts[0].dim(), "applegpu: cat dimension out of range");
  std::vector<int64_t> shape(parts[0].sizes().begin(), parts[0].sizes().end());
  shape[d] = 0;
  for (auto& t : parts) {
    for (int64_t i = 0; i < t.dim(); i++) TORCH_CHECK(i == d || t.size(i) == shape[i], "applegpu: cat operands differ outside the cat dimension");
    shape[d] += t.size(d);
  }
  at::Tensor out = new_empty(shape, parts[0].scalar_type());
  int64_t at_row = 0;
  for (auto& t : parts) {
    if (t.size(d) == 0) continue;
    copy_into(out.narrow(d, at_row, t.size(d)), t);
    at_row += t.size(d);
  }
  return out;
}

// ── views: metadata only, the storage is shared ─────────────────────────────
at::Tensor op_view(const at::Tensor& self, c10::SymIntArrayRef size) { return at::native::view(self, C10_AS_INTARRAYREF_SLOW(size)); }
at::Tensor op_as_strided(const at::Tensor& self, c10::SymIntArrayRef size, c10::SymIntArrayRef stride, std::optional<c10::SymInt> offset) {
  std::optional<int64_t> off;
  if (offset.has_value()) off = offset->expect_int();
  return at::native::as_strided_tensorimpl(self, C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride), off);
}
at::Tensor op_reshape_alias(const at::Tensor& self, c10::SymIntArrayRef size, c10::SymIntArrayRef stride) {
  return at::native::_reshape_alias(self, C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride));
}
at::Tensor& op_set_source_storage(at::Tensor& self, at::Storage source, c10::SymInt offset, c10::SymIntArrayRef size, c10::SymIntArrayRef stride) {
  return at::native::set_storage_cpu_(self, std::move(source), offset.expect_int(), C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride));
}
at::Scalar op_local_scalar_dense(const at::Tensor& self) {
  at::Tensor host = at::empty({}, self.options().device(at::kCPU));
  copy_into(host, self.reshape({}));
  return host.item();
}

// ── device guard and hooks: one device, one stream (the runtime's own) ───────
struct GuardImpl final : c10::impl::DeviceGuardImplInterface {
  c10::DeviceType type() const override { return c10::DeviceType::PrivateUse1; }
  c10::Device exchangeDevice(c10::Device) const override { return kDev; }
  c10::Device getDevice() const override { return kDev; }
  void setDevice(c10::Device) const override {}
  void uncheckedSetDevice(c10::Device) const noexcept override {}
  c10::Stream getStream(c10::Device) const noexcept override { return c10::Stream(c10::Stream::DEFAULT, kDev); }
  c10::Stream getDefaultStream(c10::Device) const override { return c10::Stream(c10::Stream::DEFAULT, kDev); }
  c10::Stream exchangeStream(c10::Stream) const noexcept override { return c10::Stream(c10::Stream::DEFAULT, kDev); }
  c10::DeviceIndex deviceCount() const noexcept override { return 1; }
};
C10_REGISTER_GUARD_IMPL(PrivateUse1, GuardImpl);

struct Hooks final : at::PrivateUse1HooksInterface {
  bool hasPrimaryContext(c10::DeviceIndex) const override { return true; }
};

const bool g_registered = [] {
  c10::SetAllocator(c10::DeviceType::PrivateUse1, &g_allocator);
  at::RegisterPrivateUse1HooksInterface(new Hooks());
  return true;
}();

}  // namespace

// scaled_dot_product_attention asks this stub (not the dispatcher) which backend serves a PrivateUse1 call
namespace at::native {
REGISTER_PRIVATEUSE1_DISPATCH(_fused_sdp_choice_stub, &op_fused_sdp_choice)
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("empty.memory_format", op_empty);
  m.impl("empty_strided", op_empty_strided);
  m.impl("copy_", op_copy_);
  m.impl("_copy_from", op_copy_from);
  m.impl("_copy_from_and_resize", op_copy_from_and_resize);
  m.impl("resize_", op_resize_);
  m.impl("fill_.Scalar", op_fill_);
  m.impl("zero_", op_zero_);
  m.impl("_local_scalar_dense", op_local_scalar_dense);
  m.impl("view", op_view);
  m.impl("as_strided", op_as_strided);
  m.impl("_reshape_alias", op_reshape_alias);
  m.impl("set_.source_Storage_storage_offset", op_set_source_storage);
  m.impl("add.Tensor", op_add);
  m.impl("sub.Tensor", op_sub);
  m.impl("mul.Tensor", op_mul);
  m.impl("div.Tensor", op_div);
  m.impl("mul.Scalar", op_mul_scalar);
  m.impl("add.Scalar", op_add_scalar);
  m.impl("pow.Tensor_Scalar", op_pow_scalar);
  m.impl("tanh", op_tanh);
  m.impl("exp", op_exp);
  m.impl("log", op_log);
  m.impl("sqrt", op_sqrt);
  m.impl("sigmoid", op_sigmoid);
  m.impl("abs", op_abs);
  m.impl("_fused_sdp_choice", op_fused_sdp_choice);
  m.impl("_scaled_dot_product_fused_attention_overrideable", op_sdp_overrideable);
  m.impl("add_.Tensor", op_add_);
  m.impl("mul_.Tensor", op_mul_);
  m.impl("relu", op_relu);
  m.impl("neg", op_neg);
  m.impl("gelu", op_gelu);
  m.impl("mm", op_mm);
  m.impl("bmm", op_bmm);
  m.impl("addmm", op_addmm);
  m.impl("_softmax", op_softmax);
  m.impl("native_layer_norm", op_native_layer_norm);
  m.impl("embedding", op_embedding);
  m.impl("cat", op_cat);
}

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) { m.fallback(torch::CppFunction::makeFromBoxedFunction<&cpu_fallback>()); }
