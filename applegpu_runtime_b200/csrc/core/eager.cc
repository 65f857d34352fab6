// EagerRuntime: stride-aware tensors, views, one kernel launch per op call.
//
// Reference: eager.rs — EagerTensor {buffer, layout, dtype, byte offset} (:13-64), alloc
// (:90-110, zero-byte tensors still get a 4-byte buffer), create_view (:114-139), free (:143-149),
// binary_op with broadcast + view strides (:246-342), matmul (:403-479, contiguous inputs only),
// matmul_ex (:485-560, transpose flags on base tensors), embedding / layer_norm / gelu / softmax
// (:957-1079), add_scaled_inplace (:1084-1096), sum_dim (:827-846). Ops are asynchronous: results
// are valid after flush_and_wait / synchronize or a download.
#include "runtime.h"

namespace ag {

struct EagerMeta : MetaSource {
  const EagerRuntime* rt;
  explicit EagerMeta(const EagerRuntime* r) : rt(r) {}
  Status shape(uint64_t id, Dims* out) const override { return rt->shape(id, out); }
  Status dtype(uint64_t id, DType* out) const override { return rt->dtype(id, out); }
};

Status EagerRuntime::get(uint64_t id, const TensorRec** out) const {
  auto it = tensors_.find(id);
  if (it == tensors_.end()) return Status::invalid("tensor " + std::to_string(id) + " not found");
  *out = &it->second;
  return Status::OK();
}
const TensorRec* EagerRuntime::tensor(uint64_t id) const {
  auto it = tensors_.find(id);
  return it == tensors_.end() ? nullptr : &it->second;
}
Status EagerRuntime::shape(uint64_t id, Dims* out) const {
  const TensorRec* t; AG_RETURN_IF_ERROR(get(id, &t)); *out = t->shape; return Status::OK();
}
Status EagerRuntime::dtype(uint64_t id, DType* out) const {
  const TensorRec* t; AG_RETURN_IF_ERROR(get(id, &t)); *out = t->dtype; return Status::OK();
}

Status EagerRuntime::alloc(const Dims& shape, DType dt, uint64_t* id, void** ptr) {
  AG_RETURN_IF_ERROR(check_ndim(shape));
  TensorRec r;
  r.shape = shape; r.strides = contiguous_strides(shape); r.dtype = dt; r.has_meta = true;
  size_t nbytes = (size_t)numel_of(shape) * dtype_size(dt);
  AG_RETURN_IF_ERROR(Shared::get().pool.acquire(nbytes == 0 ? 4 : nbytes, &r.buf));
  *id = next_tensor_id();
  *ptr = r.buf->ptr;
  tensors_[*id] = std::move(r);
  return Status::OK();
}

void EagerRuntime::free_tensor(uint64_t id) { tensors_.erase(id); }

Status EagerRuntime::register_shape(uint64_t id, const Dims& shape) {
  auto it = tensors_.find(id);
  if (it == tensors_.end()) return Status::invalid("tensor " + std::to_string(id) + " not found");
  AG_RETURN_IF_ERROR(check_ndim(shape));
  it->second.shape = shape; it->second.strides = contiguous_strides(shape);
  return Status::OK();
}

Status EagerRuntime::create_view(uint64_t base, const Dims& shape, const Dims& strides, uint64_t offset_elems, uint64_t* id, void** ptr) {
  const TensorRec* b; AG_RETURN_IF_ERROR(get(base, &b));
  AG_RETURN_IF_ERROR(check_ndim(shape));
  TensorRec v = *b;
  v.shape = shape;
  v.strides = contiguous_strides(shape);
  for (size_t i = 0; i < strides.size() && i < shape.size(); i++) v.strides[i] = strides[i];
  v.byte_offset = b->byte_offset + (size_t)offset_elems * dtype_size(b->dtype);
  *id = next_tensor_id();
  *ptr = v.data();
  tensors_[*id] = std::move(v);
  return Status::OK();
}

Status EagerRuntime::run(OpKind kind, const std::vector<uint64_t>& inputs, uint64_t* out_id, void** out_ptr) {
  OpNode node;
  node.op = std::move(kind);
  node.inputs = inputs;
  EagerMeta meta(this);
  AG_RETURN_IF_ERROR(infer_node(meta, &node));
  std::vector<const TensorRec*> ins;
  for (uint64_t in : inputs) { const TensorRec* t; AG_RETURN_IF_ERROR(get(in, &t)); ins.push_back(t); }
  TensorRec out;
  // Eager results always own a fresh contiguous buffer (views come only from create_view).
  std::shared_ptr<Buffer> ob;
  size_t nbytes = (size_t)numel_of(node.out_shape) * dtype_size(node.out_dtype);
  AG_RETURN_IF_ERROR(Shared::get().pool.acquire(nbytes == 0 ? 4 : nbytes, &ob));
  AG_RETURN_IF_ERROR(execute_node(node, ins, &out, ob));
  node.id = next_tensor_id();
  *out_id = node.id;
  *out_ptr = out.data();
  out.has_meta = true;
  tensors_[node.id] = std::move(out);
  return Status::OK();
}

Status EagerRuntime::add_scaled_inplace(uint64_t self, uint64_t other, float alpha) {
  const TensorRec *a, *b;
  AG_RETURN_IF_ERROR(get(self, &a)); AG_RETURN_IF_ERROR(get(other, &b));
  DeviceCtx& ctx = DeviceCtx::get();
  AG_RETURN_IF_ERROR(ctx.make_current());
  if (ctx.dry) return Status::compute("no CUDA device (dry-run mode)");
  Dims bs;
  AG_RETURN_IF_ERROR(broadcast_shapes(a->shape, b->shape, &bs));
  if (bs != a->shape) return Status::invalid("in-place add cannot broadcast self from " + dims_str(a->shape) + " to " + dims_str(bs));
  if (a->buf) ctx.prefetch(a->buf->ptr, a->buf->capacity);
  if (b->buf) ctx.prefetch(b->buf->ptr, b->buf->capacity);
  return k::add_scaled_inplace(ctx.stream, a->view(), b->view(), alpha);
}

uint64_t EagerRuntime::adopt(TensorRec rec) {
  uint64_t id = next_tensor_id();
  rec.has_meta = true;
  tensors_[id] = std::move(rec);
  return id;
}

uint64_t EagerRuntime::find_by_data_ptr(const void* p) const {
  uint64_t view_match = 0;
  for (auto& kv : tensors_) {
    if (kv.second.data() == p) {
      if (kv.second.byte_offset == 0) return kv.first;  // prefer the owner over views (eager_ffi.rs:611-633)
      if (!view_match) view_match = kv.first;
    }
  }
  return view_match;
}

}  // namespace ag
