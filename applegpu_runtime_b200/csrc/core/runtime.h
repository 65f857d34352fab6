// Device context, buffer pool, tensor records, and the two runtimes behind the C ABI.
//
// Reference counterparts: pool.rs / buffer.rs (BufferPool: bucketed reuse, hit/miss stats,
// watermark, drain), lazy.rs (LazyRuntime: materialised tensors + pending graph, eval =
// topo-sort -> fusion -> execute), eager.rs (EagerRuntime: stride-aware tensors, views,
// per-op immediate dispatch). The Metal command buffer becomes one CUDA stream; buffers come
// from a stream-ordered cudaMallocAsync pool, so a buffer released on the host can be handed
// to the next op without a device synchronisation.
#pragma once
#include <cuda_runtime.h>
#include <memory>
#include <mutex>
#include <map>
#include <unordered_map>
#include <unordered_set>
#include <vector>
#include "types.h"
#include "graph.h"

namespace ag {

struct DeviceCtx {
  int device = -1;
  cudaStream_t stream = nullptr;
  bool dry = false;       // metadata-only mode: no device, nothing executes
  bool ready = false;
  // Host-visible mode: pool buffers are CUDA managed memory, so the pointers the C-ABI returns can be read and
  // written by the host after a flush, as the reference's shared Metal buffers can (the PrivateUse1 shim does
  // memcpy on them). Chosen before the context is created (APPLEGPU_HOST_VISIBLE=1 or request_host_visible).
  bool host_visible = false;
  static void request_host_visible(bool on);
  // Moves a managed range to the device ahead of the kernels that use it (no-op outside host-visible mode).
  void prefetch(const void* ptr, size_t bytes) const;
  int sm_count = 0;
  size_t total_mem = 0;
  std::string name;
  // One context per process (one process per GPU).
  static DeviceCtx& get();
  Status init(bool allow_dry);
  Status make_current() const;
};

struct Buffer {
  void* ptr = nullptr;
  size_t capacity = 0;
  bool borrowed = false;  // memory owned by the caller (register_external)
};

struct PoolStats {
  uint64_t hits = 0, misses = 0, pooled_bytes = 0, bucket_count = 0;
  uint64_t live_bytes = 0, peak_live_bytes = 0, live_buffers = 0;
};

class BufferPool {
 public:
  explicit BufferPool(size_t max_pooled_bytes);
  ~BufferPool();
  // Returns a buffer of at least `size` bytes whose deleter hands it back to the pool.
  Status acquire(size_t size, std::shared_ptr<Buffer>* out);
  PoolStats stats() const;
  void drain();
  void set_max_pooled_bytes(size_t n);
  size_t max_pooled_bytes() const { return max_pooled_; }
  Status prewarm(const std::vector<size_t>& sizes);
  // Size class for a request: powers of two with four steps per octave above 4 KiB.
  static size_t size_class(size_t n);
  // Test hook: make the next `n` device allocations fail (host-side fault injection).
  void fail_next_allocs(int n) { fail_next_ = n; }
  void set_memory_limit(size_t bytes) { memory_limit_ = bytes; }

 private:
  void release(Buffer* b);
  mutable std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_;
  size_t max_pooled_;
  size_t pooled_bytes_ = 0;
  uint64_t hits_ = 0, misses_ = 0;
  size_t live_bytes_ = 0, peak_live_ = 0, live_buffers_ = 0;
  size_t memory_limit_ = 0;  // 0 = none
  int fail_next_ = 0;
  uint64_t fake_ptr_ = 0x1000;  // dry mode addresses
};

struct TensorRec {
  std::shared_ptr<Buffer> buf;
  Dims shape;
  Dims strides;        // elements
  DType dtype = DType::F32;
  size_t byte_offset = 0;
  bool has_meta = false;  // graph flavour: alloc() precedes register_tensor()
  void* data() const { return buf ? static_cast<uint8_t*>(buf->ptr) + byte_offset : nullptr; }
  TView view() const { TView v; v.ptr = data(); v.dtype = dtype; v.shape = shape; v.strides = strides; return v; }
  bool contiguous() const { return is_contiguous(shape, strides); }
  size_t nbytes() const { return (size_t)numel_of(shape) * dtype_size(dtype); }
};

uint64_t next_tensor_id();  // process-global, starts at 1 (tensor.rs:292-297)
uint64_t next_op_id();      // starts at 100000 (ops.rs:165)
uint64_t next_fused_id();   // starts at 200000 (fusion.rs:7)

// Shared state: one pool and one stream serve both flavours.
struct Shared {
  BufferPool pool;
  Shared();
  static Shared& get();
};

// Executes one node: inputs are materialised records, `out` receives the result (a fresh
// buffer, or a view of an input for layout-only ops). `out_buf`, if set, is a caller-provided
// destination (the *_out ABI variants).
// While one is alive on this thread, execute_node may hold fused linears back to launch consecutive ones as one chained
// kernel (exec.cc). finish() launches what is still held; a scope destroyed without it (an evaluation that failed) drops it.
void set_gemm_chain(bool on);
bool gemm_chain_enabled();
struct ChainScope {
  ChainScope();
  ~ChainScope();
  Status finish();
  ChainScope(const ChainScope&) = delete;
  ChainScope& operator=(const ChainScope&) = delete;
};
Status execute_node(const OpNode& node, const std::vector<const TensorRec*>& inputs, TensorRec* out,
                    std::shared_ptr<Buffer> out_buf = nullptr);
Status make_contiguous(const TensorRec& in, TensorRec* out);
Status upload(const TensorRec& t, const void* host, size_t nbytes);
Status download(const TensorRec& t, void* host, size_t nbytes, bool wait = true);

class LazyRuntime {
 public:
  Status shape(uint64_t id, Dims* out) const;
  Status dtype(uint64_t id, DType* out) const;
  bool is_pending(uint64_t id) const { return graph_.has_node(id); }
  bool is_materialized(uint64_t id) const { return tensors_.count(id) != 0; }
  void record_op(OpNode n);
  Status eval(uint64_t id);
  // alloc + register (backend_ffi.rs:87-115, :195-222)
  Status alloc_raw(size_t bytes, uint64_t* id, void** ptr);
  Status register_tensor(uint64_t id, const Dims& dims, DType dt);
  Status preallocate_output(uint64_t node_id, void** ptr);
  Status insert_tensor(uint64_t id, TensorRec rec);
  void free_tensor(uint64_t id);  // deferred while pending nodes reference it (lazy.rs:118-144)
  Status read_bytes(uint64_t id, void* host, size_t nbytes, bool wait = true);
  Status read_f32(uint64_t id, float* out, uint64_t max_elements);
  Status write_bytes(uint64_t id, const void* host, size_t nbytes);
  Status get_ptr(uint64_t id, void** ptr);
  const TensorRec* tensor(uint64_t id) const;
  size_t tensor_count() const { return tensors_.size(); }
  size_t memory_usage() const;
  // Text description of what eval(id) would launch after the fusion pass.
  Status plan(uint64_t id, std::string* out);
  Graph& graph() { return graph_; }
  // counters
  uint64_t kernels_launched = 0;

 private:
  std::unordered_map<uint64_t, TensorRec> tensors_;
  std::unordered_map<uint64_t, std::shared_ptr<Buffer>> prealloc_;  // outputs reserved by *_out calls
  std::unordered_set<uint64_t> deferred_free_;
  Graph graph_;
};

class EagerRuntime {
 public:
  Status alloc(const Dims& shape, DType dt, uint64_t* id, void** ptr);
  void free_tensor(uint64_t id);
  Status register_shape(uint64_t id, const Dims& shape);
  Status shape(uint64_t id, Dims* out) const;
  Status dtype(uint64_t id, DType* out) const;
  Status create_view(uint64_t base, const Dims& shape, const Dims& strides, uint64_t offset_elems, uint64_t* id, void** ptr);
  // Runs `kind` on `inputs` now; the result is a new contiguous tensor.
  Status run(OpKind kind, const std::vector<uint64_t>& inputs, uint64_t* out_id, void** out_ptr);
  Status add_scaled_inplace(uint64_t self, uint64_t other, float alpha);
  // Registers an already-computed record under a fresh id.
  uint64_t adopt(TensorRec rec);
  uint64_t find_by_data_ptr(const void* p) const;
  const TensorRec* tensor(uint64_t id) const;
  Status get(uint64_t id, const TensorRec** out) const;
  size_t tensor_count() const { return tensors_.size(); }

 private:
  std::unordered_map<uint64_t, TensorRec> tensors_;
};

// Shape/dtype inference + validation shared by both flavours (the bodies of ops.rs).
struct MetaSource {
  virtual ~MetaSource() {}
  virtual Status shape(uint64_t id, Dims* out) const = 0;
  virtual Status dtype(uint64_t id, DType* out) const = 0;
};
Status validate_op_dtype(const OpKind& op, DType dt);  // ops.rs:29-163
// Fills node->out_shape / out_dtype or returns the reference's validation error.
Status infer_node(const MetaSource& src, OpNode* node);

namespace fusion {
// Reference rule (fusion.rs:243-285): linear element-wise chains -> FusedElementwise, plus the
// graph-level rewrites of this build (linear epilogues, attention, embedding sum, layout sinks).
// `released`: ids whose caller-side handle has been freed while ops still consume them.
// `minted`: receives the ids of nodes the pass created that no caller knows (to be freed after their last use).
std::vector<uint64_t> optimize(Graph& g, const std::vector<uint64_t>& order, const std::unordered_set<uint64_t>& keep,
                               const std::unordered_set<uint64_t>* released = nullptr, std::vector<uint64_t>* minted = nullptr);
void set_enabled(bool elementwise, bool patterns);
void get_enabled(bool* elementwise, bool* patterns);
}

}  // namespace ag
