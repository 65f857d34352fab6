// LazyRuntime: materialised tensors + a pending graph, evaluated on demand.
//
// Reference: lazy.rs — `eval` (:208-365) = topo-sort -> fusion::optimize -> execute in order on
// one command buffer -> wait; pre-allocated outputs (:437-442); deferred frees while pending
// nodes still reference a tensor (:118-144); read_bytes / read_f32 (:2554-2560). Here the
// command buffer is the runtime's CUDA stream: eval only enqueues, and the host waits when it
// reads data back.
#include "runtime.h"
#include <cstring>
#include <sstream>

namespace ag {

struct LazyMeta : MetaSource {
  const LazyRuntime* rt;
  explicit LazyMeta(const LazyRuntime* r) : rt(r) {}
  Status shape(uint64_t id, Dims* out) const override { return rt->shape(id, out); }
  Status dtype(uint64_t id, DType* out) const override { return rt->dtype(id, out); }
};

Status LazyRuntime::shape(uint64_t id, Dims* out) const {
  auto t = tensors_.find(id);
  if (t != tensors_.end() && t->second.has_meta) { *out = t->second.shape; return Status::OK(); }
  const OpNode* n = graph_.get_node(id);
  if (n) { *out = n->out_shape; return Status::OK(); }
  return Status::invalid("Tensor " + std::to_string(id) + " not found");
}
Status LazyRuntime::dtype(uint64_t id, DType* out) const {
  auto t = tensors_.find(id);
  if (t != tensors_.end() && t->second.has_meta) { *out = t->second.dtype; return Status::OK(); }
  const OpNode* n = graph_.get_node(id);
  if (n) { *out = n->out_dtype; return Status::OK(); }
  return Status::invalid("Tensor " + std::to_string(id) + " not found");
}
const TensorRec* LazyRuntime::tensor(uint64_t id) const {
  auto t = tensors_.find(id);
  return t == tensors_.end() ? nullptr : &t->second;
}
size_t LazyRuntime::memory_usage() const {
  size_t n = 0;
  std::unordered_set<const Buffer*> seen;
  for (auto& kv : tensors_) if (kv.second.buf && seen.insert(kv.second.buf.get()).second) n += kv.second.buf->capacity;
  return n;
}

void LazyRuntime::record_op(OpNode n) { graph_.add_node(std::move(n)); }

Status LazyRuntime::alloc_raw(size_t bytes, uint64_t* id, void** ptr) {
  *id = next_tensor_id();
  if (bytes == 0) { *ptr = nullptr; TensorRec r; r.has_meta = false; tensors_[*id] = r; return Status::OK(); }
  TensorRec r;
  AG_RETURN_IF_ERROR(Shared::get().pool.acquire(bytes, &r.buf));
  r.has_meta = false;
  *ptr = r.buf->ptr;
  tensors_[*id] = r;
  return Status::OK();
}

Status LazyRuntime::register_tensor(uint64_t id, const Dims& dims, DType dt) {
  auto it = tensors_.find(id);
  if (it == tensors_.end()) return Status::invalid("No pre-allocated buffer for tensor " + std::to_string(id));
  AG_RETURN_IF_ERROR(check_ndim(dims));
  size_t need = (size_t)numel_of(dims) * dtype_size(dt);
  size_t have = it->second.buf ? it->second.buf->capacity : 0;
  if (need > have) return Status::invalid("tensor " + std::to_string(id) + " needs " + std::to_string(need) + " bytes but its buffer holds " + std::to_string(have));
  it->second.shape = dims; it->second.strides = contiguous_strides(dims); it->second.dtype = dt; it->second.has_meta = true;
  return Status::OK();
}

Status LazyRuntime::insert_tensor(uint64_t id, TensorRec rec) {
  rec.has_meta = true;
  tensors_[id] = std::move(rec);
  return Status::OK();
}

Status LazyRuntime::preallocate_output(uint64_t node_id, void** ptr) {
  const OpNode* n = graph_.get_node(node_id);
  if (!n) {
    // The recorder may have returned an existing tensor (e.g. a same-dtype cast).
    const TensorRec* t = tensor(node_id);
    if (t) { *ptr = t->data(); return Status::OK(); }
    return Status::invalid("cannot determine output shape");
  }
  size_t bytes = (size_t)numel_of(n->out_shape) * dtype_size(n->out_dtype);
  if (bytes == 0) { *ptr = nullptr; return Status::OK(); }
  std::shared_ptr<Buffer> b;
  AG_RETURN_IF_ERROR(Shared::get().pool.acquire(bytes, &b));
  *ptr = b->ptr;
  prealloc_[node_id] = b;
  return Status::OK();
}

void LazyRuntime::free_tensor(uint64_t id) {
  if (graph_.ref_count(id) > 0) { deferred_free_.insert(id); return; }
  // A pending node nobody consumes can simply be dropped.
  if (graph_.has_node(id)) {
    OpNode n;
    graph_.remove_node(id, &n);
    prealloc_.erase(id);
    // its inputs may have been waiting on it
    for (uint64_t in : n.inputs) if (deferred_free_.count(in) && graph_.ref_count(in) == 0) { deferred_free_.erase(in); free_tensor(in); }
    return;
  }
  tensors_.erase(id);
}

Status LazyRuntime::eval(uint64_t id) {
  if (tensors_.count(id) && !graph_.has_node(id)) return Status::OK();
  if (!graph_.has_node(id)) return Status::graph("Tensor " + std::to_string(id) + " not found in graph or materialized tensors");
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) return Status::compute("no CUDA device (dry-run mode): eval is unavailable");
  std::vector<uint64_t> order;
  AG_RETURN_IF_ERROR(graph_.topo_sort(id, &order));
  std::unordered_set<uint64_t> keep{id};
  for (auto& kv : prealloc_) keep.insert(kv.first);  // outputs the caller already holds pointers to
  std::vector<uint64_t> minted;
  order = fusion::optimize(graph_, order, keep, &deferred_free_, &minted);
  for (uint64_t m : minted) deferred_free_.insert(m);   // nobody holds a handle: dropped after the last consumer ran

  ChainScope chain_scope;   // consecutive fused linears of this evaluation may go out as one chained launch
  // remaining uses inside this evaluation, to drop dead intermediates early
  for (uint64_t nid : order) {
    const OpNode* np = graph_.get_node(nid);
    if (!np) return Status::graph("node " + std::to_string(nid) + " vanished during evaluation");
    const OpNode& node_ref = *np;   // executed in place; moved out of the graph afterwards (no deep copy per node)
    std::vector<const TensorRec*> ins;
    ins.reserve(node_ref.inputs.size());
    for (uint64_t in : node_ref.inputs) {
      auto t = tensors_.find(in);
      if (t == tensors_.end() || !t->second.has_meta)
        return Status::graph("Input tensor " + std::to_string(in) + " for op " + std::to_string(nid) + " is not materialized");
      ins.push_back(&t->second);
    }
    std::shared_ptr<Buffer> ob;
    auto pa = prealloc_.find(nid);
    if (pa != prealloc_.end()) { ob = pa->second; }
    TensorRec out;
    Status st = execute_node(node_ref, ins, &out, ob);
    if (!st.ok()) return st;  // the graph keeps the unevaluated remainder, like abort_batch upstream
    if (pa != prealloc_.end()) prealloc_.erase(pa);
    OpNode node;
    graph_.remove_node(nid, &node);
    out.has_meta = true;
    tensors_[nid] = std::move(out);
    kernels_launched++;
    // inputs whose last consumer just ran and that the caller already freed
    for (uint64_t in : node.inputs) {
      if (deferred_free_.count(in) && graph_.ref_count(in) == 0) { deferred_free_.erase(in); tensors_.erase(in); }
    }
    if (nid != id && deferred_free_.count(nid) && graph_.ref_count(nid) == 0) { deferred_free_.erase(nid); tensors_.erase(nid); }
  }
  AG_RETURN_IF_ERROR(chain_scope.finish());
  // ids absorbed by the fusion pass no longer exist anywhere
  for (auto it = deferred_free_.begin(); it != deferred_free_.end();) {
    if (!graph_.has_node(*it) && !tensors_.count(*it)) it = deferred_free_.erase(it); else ++it;
  }
  return Status::OK();
}

Status LazyRuntime::plan(uint64_t id, std::string* out) {
  std::ostringstream os;
  if (!graph_.has_node(id)) { *out = ""; return tensors_.count(id) ? Status::OK() : Status::graph("Tensor " + std::to_string(id) + " not found"); }
  // Work on a copy so planning does not consume the pending graph.
  Graph copy = graph_;
  std::vector<uint64_t> order;
  AG_RETURN_IF_ERROR(copy.topo_sort(id, &order));
  std::unordered_set<uint64_t> keep{id};
  for (auto& kv : prealloc_) keep.insert(kv.first);
  std::vector<uint64_t> minted;
  order = fusion::optimize(copy, order, keep, &deferred_free_, &minted);
  for (uint64_t nid : order) {
    const OpNode* n = copy.get_node(nid);
    if (!n) continue;
    os << n->op.kernel_name();
    if (n->op.op == Op::FusedLinear) {
      os << "[";
      if (n->op.i1 == 1) os << "int8,";
      if (n->op.i2 == 1) os << "argmax,";
      if (n->op.f0 != 1.0f) os << "scale,";
      if (n->op.has_bias) os << "bias,";
      if (n->op.act == k::Act::GeluTanh) os << "gelu,"; else if (n->op.act == k::Act::GeluErf) os << "gelu_exact,"; else if (n->op.act == k::Act::Relu) os << "relu,";
      if (n->op.has_residual) os << "residual,";
      if (n->op.has_ln) os << "layer_norm_in,";
      if (n->op.has_stats_out) os << "row_stats,";
      os << "]";
    }
    if (n->op.op == Op::FusedAttention) os << (n->op.causal ? "[causal" : "[full") << (n->op.i0 == 1 ? ",merge_heads]" : "]");
    if (n->op.op == Op::AddBias && n->op.act != k::Act::None) os << (n->op.act == k::Act::GeluTanh ? "[gelu]" : n->op.act == k::Act::GeluErf ? "[gelu_exact]" : "[relu]");
    if (n->op.op == Op::FusedElementwise) os << "{" << n->op.expr << "}";
    os << dtype_suffix(n->out_dtype) << " " << dims_str(n->out_shape) << "\n";
  }
  *out = os.str();
  return Status::OK();
}

Status LazyRuntime::get_ptr(uint64_t id, void** ptr) {
  const TensorRec* t = tensor(id);
  if (!t) return Status::invalid("Tensor " + std::to_string(id) + " not found");
  *ptr = t->data();
  return Status::OK();
}

Status LazyRuntime::read_bytes(uint64_t id, void* host, size_t nbytes, bool wait) {
  if (is_pending(id)) AG_RETURN_IF_ERROR(eval(id));
  const TensorRec* t = tensor(id);
  if (!t || !t->has_meta) return Status::invalid("Tensor " + std::to_string(id) + " not found");
  return download(*t, host, nbytes, wait);
}

Status LazyRuntime::write_bytes(uint64_t id, const void* host, size_t nbytes) {
  const TensorRec* t = tensor(id);
  if (!t) return Status::invalid("Tensor " + std::to_string(id) + " not found");
  if (!t->has_meta) {
    // raw allocation not yet registered: bound by capacity
    if (!t->buf || nbytes > t->buf->capacity) return Status::invalid("write exceeds buffer capacity");
    DeviceCtx& ctx = DeviceCtx::get();
    if (ctx.dry) return Status::compute("no CUDA device (dry-run mode)");
    cudaError_t e = cudaMemcpyAsync(t->buf->ptr, host, nbytes, cudaMemcpyHostToDevice, ctx.stream);
    if (e != cudaSuccess) return Status::compute(std::string("upload: ") + cudaGetErrorString(e));
    return Status::OK();
  }
  return upload(*t, host, nbytes);
}

// Host-side widening for read_f32 (reference: lazy.rs read_f32 converts per dtype).
static float half_to_float(uint16_t h) {
  uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
  uint32_t f;
  if (exp == 0) {
    if (man == 0) f = sign << 31;
    else { int e = -1; do { man <<= 1; e++; } while (!(man & 0x400)); man &= 0x3ff; f = (sign << 31) | ((uint32_t)(127 - 15 - e) << 23) | (man << 13); }
  } else if (exp == 31) f = (sign << 31) | 0x7f800000u | (man << 13);
  else f = (sign << 31) | ((exp + 112) << 23) | (man << 13);
  float r; std::memcpy(&r, &f, 4); return r;
}

Status LazyRuntime::read_f32(uint64_t id, float* out, uint64_t max_elements) {
  if (is_pending(id)) AG_RETURN_IF_ERROR(eval(id));
  const TensorRec* t = tensor(id);
  if (!t || !t->has_meta) return Status::invalid("Tensor " + std::to_string(id) + " not found");
  uint64_t n = (uint64_t)numel_of(t->shape);
  if (n > max_elements) n = max_elements;
  size_t esz = dtype_size(t->dtype);
  if (t->dtype == DType::F32) return download(*t, out, n * 4);
  std::vector<uint8_t> tmp(n * esz);
  AG_RETURN_IF_ERROR(download(*t, tmp.data(), n * esz));
  for (uint64_t i = 0; i < n; i++) {
    const uint8_t* p = tmp.data() + i * esz;
    switch (t->dtype) {
      case DType::F16: { uint16_t h; std::memcpy(&h, p, 2); out[i] = half_to_float(h); break; }
      case DType::BF16: { uint16_t h; std::memcpy(&h, p, 2); uint32_t f = (uint32_t)h << 16; std::memcpy(&out[i], &f, 4); break; }
      case DType::I8: out[i] = (float)*(const int8_t*)p; break;
      case DType::U8: case DType::Bool: out[i] = (float)*p; break;
      case DType::I16: { int16_t v; std::memcpy(&v, p, 2); out[i] = (float)v; break; }
      case DType::I32: { int32_t v; std::memcpy(&v, p, 4); out[i] = (float)v; break; }
      case DType::U32: { uint32_t v; std::memcpy(&v, p, 4); out[i] = (float)v; break; }
      case DType::I64: { int64_t v; std::memcpy(&v, p, 8); out[i] = (float)v; break; }
      case DType::F64: { double v; std::memcpy(&v, p, 8); out[i] = (float)v; break; }
      default: out[i] = 0.f;
    }
  }
  return Status::OK();
}

}  // namespace ag
