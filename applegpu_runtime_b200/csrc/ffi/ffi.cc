// extern "C" surface: include/applegpu_b200_ffi.h (the reference's symbols) and
// include/applegpu_b200_ext.h (additive). Mirrors backend_ffi.rs and eager_ffi.rs: one global
// runtime per flavour behind a mutex, idempotent init, thread-local last-error strings, no
// exceptions across the boundary.
#include "../../../include/applegpu_b200_ffi.h"
#include "../../../include/applegpu_b200_ext.h"
#include "../core/runtime.h"
#include "../kernels/kernels.h"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <unordered_set>

namespace ag {
extern bool g_fused_attention;
void set_f32_split(bool on);
uint64_t launch_count();
void note_launches(uint64_t n);
namespace profile { void enable(bool on); void clear(); std::string report(); void set_filter(const std::string& csv); }
struct Gpt2DecoderCfg { int n_layer, n_head, n_embd, vocab, n_positions, batch, max_len; };
Status decoder_create(const std::vector<TensorRec>& weights, const Gpt2DecoderCfg& cfg, uint64_t* handle);
Status decoder_prefill(uint64_t handle, const std::vector<TensorRec>& kvs, const TensorRec& first_tokens, int prompt_len);
Status decoder_steps(uint64_t handle, int n_steps, int32_t* host_tokens, bool use_graph);
int decoder_launches_per_step(uint64_t handle);
int decoder_uses_graph(uint64_t handle);
Status decoder_set_engine(uint64_t handle, int engine);
void decoder_destroy(uint64_t handle);
namespace k {
void set_matmul_path(int mode);
void set_gemm_tile(int code);
}
}
using namespace ag;

namespace {

struct LazyState { std::mutex mu; LazyRuntime rt; bool ready = false; };
struct EagerState { std::mutex mu; EagerRuntime rt; bool ready = false; };
// Leaked on purpose: buffers held by the runtimes return to the pool from their deleters, so
// neither may be destroyed before the other at process exit; the CUDA context reclaims the memory.
LazyState& lazy_state() { static LazyState* s = new LazyState(); return *s; }
EagerState& eager_state() { static EagerState* s = new EagerState(); return *s; }

thread_local std::string t_ffi_error; thread_local bool t_ffi_has_error = false;
thread_local std::string t_eager_error; thread_local bool t_eager_has_error = false;
void set_ffi_error(const std::string& m) { t_ffi_error = m; t_ffi_has_error = true; }
void set_eager_error(const std::string& m) { t_eager_error = m; t_eager_has_error = true; }
}  // namespace
namespace ag {
// Lets entry points defined in other translation units report through applegpu_ffi_last_error().
void set_ffi_error_text(const std::string& m) { set_ffi_error(m); }
}
namespace {

Dims to_dims(const uint64_t* d, uint32_t n) { Dims v(n); for (uint32_t i = 0; i < n; i++) v[i] = (int64_t)d[i]; return v; }

struct LazyMetaSrc : MetaSource {
  const LazyRuntime* rt;
  explicit LazyMetaSrc(const LazyRuntime* r) : rt(r) {}
  Status shape(uint64_t id, Dims* out) const override { return rt->shape(id, out); }
  Status dtype(uint64_t id, DType* out) const override { return rt->dtype(id, out); }
};

bool ffi_ready(const char* what) {
  if (lazy_state().ready) return true;
  set_ffi_error(std::string(what) + " failed: applegpu FFI not initialized - call applegpu_ffi_init() first");
  return false;
}
bool eager_ready() {
  if (eager_state().ready) return true;
  set_eager_error("applegpu eager FFI not initialized - call applegpu_eager_init() first");
  return false;
}

// Validate + record one node; returns its id or 0 (message prefixed "<name> failed: ").
// ── op tapes ────────────────────────────────────────────────────────────────
// A tape is the op list one pass of a host program recorded (kinds, parameters, and which earlier
// value or external tensor each input is). Replaying it re-records the same ops on new inputs in one
// call: shapes are inferred again, so a tape taken at one KV length replays at another. Values are
// numbered in recording order; inputs < 0 name external slots: the first n_var are the variable
// inputs named at tape_begin, the rest are tensors that were simply alive during recording (weights)
// and are reused by id. Guarded by the graph-flavour mutex.
struct TapeOp { OpKind kind; std::vector<int64_t> in; };
struct Tape {
  std::vector<TapeOp> ops;
  std::vector<uint64_t> ext;      // external slots; the first n_var entries are placeholders
  uint32_t n_var = 0;
  std::vector<int64_t> outputs;
};
static std::vector<std::unique_ptr<Tape>> g_tapes;
static std::unique_ptr<Tape> g_rec;                              // tape being recorded, if any
static std::unordered_map<uint64_t, int64_t> g_rec_slot;         // tensor id -> value index or -(slot+1)

static int64_t tape_slot_of(uint64_t id) {
  auto it = g_rec_slot.find(id);
  if (it != g_rec_slot.end()) return it->second;
  g_rec->ext.push_back(id);                                      // a constant of the tape
  int64_t s = -(int64_t)g_rec->ext.size();
  g_rec_slot[id] = s;
  return s;
}

uint64_t record(const char* name, OpKind kind, std::vector<uint64_t> inputs) {
  if (!ffi_ready(name)) return 0;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  OpNode node;
  node.op = std::move(kind);
  node.inputs = std::move(inputs);
  LazyMetaSrc src(&st.rt);
  Status s = infer_node(src, &node);
  if (!s.ok()) { set_ffi_error(std::string(name) + " failed: " + s.to_string()); return 0; }
  node.id = next_op_id();
  uint64_t id = node.id;
  if (g_rec) {
    TapeOp t;
    t.kind = node.op;
    for (uint64_t in : node.inputs) t.in.push_back(tape_slot_of(in));
    g_rec_slot[id] = (int64_t)g_rec->ops.size();
    g_rec->ops.push_back(std::move(t));
  }
  st.rt.record_op(std::move(node));
  return id;
}
OpKind mk(Op op) { OpKind k; k.op = op; return k; }

uint8_t* record_out(const char* name, OpKind kind, std::vector<uint64_t> inputs, uint64_t* out_id) {
  uint64_t id = record(name, std::move(kind), std::move(inputs));
  if (!id) return nullptr;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  void* ptr = nullptr;
  Status s = st.rt.preallocate_output(id, &ptr);
  if (!s.ok()) { set_ffi_error("alloc output failed: " + s.to_string()); return nullptr; }
  if (out_id) *out_id = id;
  return static_cast<uint8_t*>(ptr);
}

uint8_t* eager_run(OpKind kind, std::vector<uint64_t> inputs, uint64_t* out_id) {
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  uint64_t id = 0; void* ptr = nullptr;
  Status s = st.rt.run(std::move(kind), inputs, &id, &ptr);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  if (out_id) *out_id = id;
  return static_cast<uint8_t*>(ptr);
}

Status init_device(bool dry) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.ready) return Status::OK();
  if (dry) { ctx.dry = true; ctx.ready = true; ctx.name = "dry-run (no device)"; return Status::OK(); }
  return ctx.init(true);
}

cudaEvent_t g_ev0 = nullptr, g_ev1 = nullptr;
std::shared_ptr<Buffer> g_flush_buf;   // taken from the stream-ordered pool on first use, kept
constexpr size_t kFlushBytes = (size_t)256 << 20;  // 2x the 126 MB L2

}  // namespace

extern "C" {

// ── graph flavour ───────────────────────────────────────────────────────────
bool applegpu_ffi_init(void) {
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (st.ready) return true;
  Status s = init_device(false);
  if (!s.ok()) { set_ffi_error(s.to_string()); return false; }
  Shared::get();
  st.ready = true;
  return true;
}
bool applegpu_ffi_init_dry(void) {
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (st.ready) return DeviceCtx::get().dry;
  Status s = init_device(true);
  if (!s.ok()) { set_ffi_error(s.to_string()); return false; }
  Shared::get();
  st.ready = true;
  return DeviceCtx::get().dry;
}
const char* applegpu_ffi_last_error(void) { return t_ffi_has_error ? t_ffi_error.c_str() : nullptr; }

uint8_t* applegpu_ffi_alloc(uint64_t size_bytes, int8_t, uint64_t* out_tensor_id) {
  if (!ffi_ready("alloc")) return nullptr;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  uint64_t id = 0; void* ptr = nullptr;
  Status s = st.rt.alloc_raw((size_t)size_bytes, &id, &ptr);
  if (!s.ok()) { set_ffi_error("alloc failed: " + s.to_string()); return nullptr; }
  if (out_tensor_id) *out_tensor_id = id;
  return static_cast<uint8_t*>(ptr);
}
void applegpu_ffi_free(uint64_t tensor_id) {
  if (!lazy_state().ready) return;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  st.rt.free_tensor(tensor_id);
}
int32_t applegpu_ffi_register_tensor(uint64_t tensor_id, const uint64_t* dims, uint32_t ndim, int8_t dtype_i8) {
  if (!ffi_ready("register_tensor")) return -1;
  DType dt;
  if (!dtype_from_wire(dtype_i8, &dt)) { set_ffi_error("Invalid dtype wire value: " + std::to_string((int)dtype_i8)); return -1; }
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.register_tensor(tensor_id, to_dims(dims, ndim), dt);
  if (!s.ok()) { set_ffi_error("register_tensor failed: " + s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_ffi_shape(uint64_t tensor_id, uint64_t* out_dims, uint32_t* out_ndim) {
  if (!ffi_ready("shape")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Dims d;
  Status s = st.rt.shape(tensor_id, &d);
  if (!s.ok()) { set_ffi_error("shape failed: " + s.to_string()); return -1; }
  *out_ndim = (uint32_t)d.size();
  for (size_t i = 0; i < d.size(); i++) out_dims[i] = (uint64_t)d[i];
  return 0;
}
int8_t applegpu_ffi_dtype(uint64_t tensor_id) {
  if (!lazy_state().ready) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  DType dt;
  if (!st.rt.dtype(tensor_id, &dt).ok()) return -1;
  return (int8_t)dt;
}

uint64_t applegpu_ffi_add(uint64_t a, uint64_t b) { return record("add", mk(Op::Add), {a, b}); }
uint64_t applegpu_ffi_sub(uint64_t a, uint64_t b) { return record("sub", mk(Op::Sub), {a, b}); }
uint64_t applegpu_ffi_mul(uint64_t a, uint64_t b) { return record("mul", mk(Op::Mul), {a, b}); }
uint64_t applegpu_ffi_div(uint64_t a, uint64_t b) { return record("div", mk(Op::Div), {a, b}); }
uint64_t applegpu_ffi_matmul(uint64_t a, uint64_t b) { return record("matmul", mk(Op::Matmul), {a, b}); }
uint64_t applegpu_ffi_relu(uint64_t x) { return record("relu", mk(Op::Relu), {x}); }
uint64_t applegpu_ffi_neg(uint64_t x) { return record("neg", mk(Op::Neg), {x}); }
uint64_t applegpu_ffi_exp(uint64_t x) { return record("exp", mk(Op::Exp), {x}); }
uint64_t applegpu_ffi_log(uint64_t x) { return record("log", mk(Op::Log), {x}); }
uint64_t applegpu_ffi_sqrt(uint64_t x) { return record("sqrt", mk(Op::Sqrt), {x}); }
uint64_t applegpu_ffi_tanh(uint64_t x) { return record("tanh", mk(Op::Tanh), {x}); }
uint64_t applegpu_ffi_sin(uint64_t x) { return record("sin", mk(Op::Sin), {x}); }
uint64_t applegpu_ffi_cos(uint64_t x) { return record("cos", mk(Op::Cos), {x}); }
uint64_t applegpu_ffi_abs(uint64_t x) { return record("abs", mk(Op::Abs), {x}); }
uint64_t applegpu_ffi_sign(uint64_t x) { return record("sign", mk(Op::Sign), {x}); }
uint64_t applegpu_ffi_sigmoid(uint64_t x) { return record("sigmoid", mk(Op::Sigmoid), {x}); }
uint64_t applegpu_ffi_gelu(uint64_t x) { return record("gelu", mk(Op::Gelu), {x}); }
uint64_t applegpu_ffi_gelu_exact(uint64_t x) { return record("gelu_exact", mk(Op::GeluExact), {x}); }
uint64_t applegpu_ffi_softmax(uint64_t x) { return record("softmax", mk(Op::Softmax), {x}); }
uint64_t applegpu_ffi_softmax_causal(uint64_t x) { return record("softmax_causal", mk(Op::SoftmaxCausal), {x}); }
uint64_t applegpu_ffi_layer_norm(uint64_t x, uint64_t gamma, uint64_t beta, float eps) {
  OpKind k = mk(Op::LayerNorm); k.f0 = eps;
  return record("layer_norm", k, {x, gamma, beta});
}
uint64_t applegpu_ffi_embedding(uint64_t w, uint64_t idx) { return record("embedding", mk(Op::Embedding), {w, idx}); }
uint64_t applegpu_ffi_add_bias(uint64_t x, uint64_t b) { return record("add_bias", mk(Op::AddBias), {x, b}); }
uint64_t applegpu_ffi_scalar_mul(uint64_t x, float scale) { OpKind k = mk(Op::ScalarMul); k.f0 = scale; return record("scalar_mul", k, {x}); }
uint64_t applegpu_ffi_argmax(uint64_t x) { return record("argmax", mk(Op::Argmax), {x}); }
uint64_t applegpu_ffi_sum(uint64_t x) { return record("sum", mk(Op::Sum), {x}); }
uint64_t applegpu_ffi_mean(uint64_t x) { return record("mean", mk(Op::Mean), {x}); }
uint64_t applegpu_ffi_transpose_dims(uint64_t x, uint32_t d0, uint32_t d1) {
  if (d0 == d1) {
    // the reference returns the input id itself for a no-op transpose (ops.rs:522-524), after range checks
    if (!ffi_ready("transpose")) return 0;
    LazyState& st = lazy_state();
    std::lock_guard<std::mutex> g(st.mu);
    Dims s;
    Status r = st.rt.shape(x, &s);
    if (!r.ok()) { set_ffi_error("transpose failed: " + r.to_string()); return 0; }
    if (d0 >= s.size()) {
      set_ffi_error("transpose failed: Invalid tensor: transpose dims (" + std::to_string(d0) + ", " + std::to_string(d1) + ") out of range for " + std::to_string(s.size()) + "D tensor");
      return 0;
    }
    return x;
  }
  OpKind k = mk(Op::Transpose); k.i0 = d0; k.i1 = d1;
  return record("transpose", k, {x});
}
uint64_t applegpu_ffi_transpose(uint64_t x) {
  if (!ffi_ready("transpose")) return 0;
  Dims s;
  {
    LazyState& st = lazy_state();
    std::lock_guard<std::mutex> g(st.mu);
    Status r = st.rt.shape(x, &s);
    if (!r.ok()) { set_ffi_error("transpose failed: " + r.to_string()); return 0; }
  }
  if (s.size() < 2) { set_ffi_error("transpose failed: Invalid tensor: transpose requires at least 2D tensor, got " + dims_str(s)); return 0; }
  return applegpu_ffi_transpose_dims(x, (uint32_t)s.size() - 2, (uint32_t)s.size() - 1);
}
uint64_t applegpu_ffi_reshape(uint64_t x, const uint64_t* dims, uint32_t ndim) {
  OpKind k = mk(Op::Reshape); k.shape = to_dims(dims, ndim);
  return record("reshape", k, {x});
}
uint64_t applegpu_ffi_slice(uint64_t x, uint32_t dim, uint64_t start, uint64_t end) {
  OpKind k = mk(Op::Slice); k.i0 = dim; k.i1 = (int64_t)start; k.i2 = (int64_t)end;
  return record("slice", k, {x});
}
uint64_t applegpu_ffi_concat(uint64_t a, uint64_t b, uint32_t dim) { OpKind k = mk(Op::Concat); k.i0 = dim; return record("concat", k, {a, b}); }
uint64_t applegpu_ffi_gather(uint64_t x, uint32_t dim, uint64_t idx) { OpKind k = mk(Op::Gather); k.i0 = dim; return record("gather", k, {x, idx}); }
uint64_t applegpu_ffi_index_select(uint64_t x, uint32_t dim, uint64_t idx) { OpKind k = mk(Op::IndexSelect); k.i0 = dim; return record("index_select", k, {x, idx}); }
uint64_t applegpu_ffi_cast(uint64_t x, int8_t target) {
  DType dt;
  if (!dtype_from_wire(target, &dt)) { set_ffi_error("cast failed: Invalid dtype wire value: " + std::to_string((int)target)); return 0; }
  if (!ffi_ready("cast")) return 0;
  {
    LazyState& st = lazy_state();
    std::lock_guard<std::mutex> g(st.mu);
    DType cur;
    if (st.rt.dtype(x, &cur).ok() && cur == dt && cur != DType::F64) return x;  // no-op cast returns its input (ops.rs:2304-2307)
  }
  OpKind k = mk(Op::Cast); k.dt = dt;
  return record("cast", k, {x});
}
uint64_t applegpu_ffi_quantize(uint64_t x, int8_t target, float scale, int32_t zp) {
  DType dt;
  if (!dtype_from_wire(target, &dt)) { set_ffi_error("quantize failed: Invalid dtype wire value: " + std::to_string((int)target)); return 0; }
  OpKind k = mk(Op::Quantize); k.dt = dt; k.f0 = scale; k.i0 = zp;
  return record("quantize", k, {x});
}
uint64_t applegpu_ffi_dequantize(uint64_t x, int8_t target, float scale, int32_t zp) {
  DType dt;
  if (!dtype_from_wire(target, &dt)) { set_ffi_error("dequantize failed: Invalid dtype wire value: " + std::to_string((int)target)); return 0; }
  OpKind k = mk(Op::Dequantize); k.dt = dt; k.f0 = scale; k.i0 = zp;
  return record("dequantize", k, {x});
}

static uint64_t attention_impl(const char* name, uint64_t q, uint64_t kk, uint64_t v, bool causal) {
  // The 5-op composition of ops.rs:1531-1618; the fusion pass may later collapse it.
  if (!ffi_ready(name)) return 0;
  Dims qs, ks, vs;
  {
    LazyState& st = lazy_state();
    std::lock_guard<std::mutex> g(st.mu);
    Status s = st.rt.shape(q, &qs);
    if (s.ok()) s = st.rt.shape(kk, &ks);
    if (s.ok()) s = st.rt.shape(v, &vs);
    if (!s.ok()) { set_ffi_error(std::string(name) + " failed: " + s.to_string()); return 0; }
  }
  if (qs.size() < 2 || ks.size() < 2 || vs.size() < 2) {
    set_ffi_error(std::string(name) + (causal ? " failed: Invalid tensor: attention_causal requires at least 2D tensors"
                                              : " failed: Invalid tensor: attention requires at least 2D tensors for Q, K, V"));
    return 0;
  }
  int64_t dk = qs.back();
  if (ks.back() != dk) { set_ffi_error(std::string(name) + " failed: Invalid tensor: Q and K must have same d_k: " + std::to_string(dk) + " vs " + std::to_string(ks.back())); return 0; }
  int64_t kv = ks[ks.size() - 2];
  if (vs[vs.size() - 2] != kv) { set_ffi_error(std::string(name) + " failed: Invalid tensor: K and V must have same kv_len: " + std::to_string(kv) + " vs " + std::to_string(vs[vs.size() - 2])); return 0; }
  uint64_t kt = applegpu_ffi_transpose(kk);
  if (!kt) return 0;
  uint64_t scores = applegpu_ffi_matmul(q, kt);
  if (!scores) return 0;
  uint64_t scaled = applegpu_ffi_scalar_mul(scores, 1.0f / std::sqrt((float)dk));
  if (!scaled) return 0;
  uint64_t w = causal ? applegpu_ffi_softmax_causal(scaled) : applegpu_ffi_softmax(scaled);
  if (!w) return 0;
  uint64_t out = applegpu_ffi_matmul(w, v);
  // The intermediates belong to this call: release them so only the graph holds them.
  applegpu_ffi_free(kt); applegpu_ffi_free(scores); applegpu_ffi_free(scaled); applegpu_ffi_free(w);
  return out;
}
uint64_t applegpu_ffi_attention(uint64_t q, uint64_t k, uint64_t v) { return attention_impl("attention", q, k, v, false); }
uint64_t applegpu_ffi_attention_causal(uint64_t q, uint64_t k, uint64_t v) { return attention_impl("attention_causal", q, k, v, true); }

uint64_t applegpu_ffi_matmul_int8(uint64_t x, uint64_t q, uint64_t scales) { return record("matmul_int8", mk(Op::MatmulInt8), {x, q, scales}); }

uint64_t applegpu_ffi_linear_fused(uint64_t x, uint64_t w, uint64_t bias, uint64_t residual, int32_t act, uint64_t ln_colsum, uint64_t ln_stats, float ln_eps,
                                   uint64_t stats_out, uint64_t stats_zero) {
  OpKind k = mk(Op::FusedLinear);
  k.f0 = 1.0f; k.f1 = ln_eps;
  k.act = act == 1 ? k::Act::GeluTanh : act == 2 ? k::Act::GeluErf : act == 3 ? k::Act::Relu : k::Act::None;
  std::vector<uint64_t> in{x, w};
  if (bias) { k.has_bias = true; in.push_back(bias); }
  if (residual) { k.has_residual = true; in.push_back(residual); }
  if (ln_colsum || ln_stats) {
    if (!ln_colsum || !ln_stats) { set_ffi_error("linear_fused failed: the folded layer_norm needs both the column sums and the row statistics"); return 0; }
    k.has_ln = true; in.push_back(ln_colsum); in.push_back(ln_stats);
  }
  if (stats_out) { k.has_stats_out = true; in.push_back(stats_out); }
  if (stats_zero) { k.has_stats_zero = true; in.push_back(stats_zero); }
  return record("linear_fused", std::move(k), std::move(in));
}

int32_t applegpu_ffi_quantize_weight(uint64_t weight_id, uint64_t* out_q_id, uint64_t* out_scales_id) {
  if (!ffi_ready("quantize_weight")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (st.rt.is_pending(weight_id)) { Status s = st.rt.eval(weight_id); if (!s.ok()) { set_ffi_error("quantize_weight failed: " + s.to_string()); return -1; } }
  const TensorRec* w = st.rt.tensor(weight_id);
  if (!w || !w->has_meta) { set_ffi_error("quantize_weight failed: Invalid tensor: Tensor " + std::to_string(weight_id) + " not found"); return -1; }
  if (w->shape.size() != 2 || !dtype_is_float(w->dtype) || w->dtype == DType::F64) { set_ffi_error("quantize_weight failed: Invalid tensor: weight must be a 2D float tensor [N,K]"); return -1; }
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) { set_ffi_error("quantize_weight failed: no CUDA device (dry-run mode)"); return -1; }
  TensorRec wc, q, sc;
  Status s = make_contiguous(*w, &wc);
  if (s.ok()) { q.shape = w->shape; q.strides = contiguous_strides(q.shape); q.dtype = DType::I8; q.has_meta = true; s = Shared::get().pool.acquire(q.nbytes() ? q.nbytes() : 4, &q.buf); }
  if (s.ok()) { sc.shape = {w->shape[0]}; sc.strides = {1}; sc.dtype = DType::F32; sc.has_meta = true; s = Shared::get().pool.acquire(sc.nbytes() ? sc.nbytes() : 4, &sc.buf); }
  if (s.ok()) s = ctx.make_current();
  if (s.ok()) s = k::quantize_rows(ctx.stream, wc.view(), q.view(), sc.view());
  if (!s.ok()) { set_ffi_error("quantize_weight failed: " + s.to_string()); return -1; }
  uint64_t qid = next_tensor_id(), sid = next_tensor_id();
  st.rt.insert_tensor(qid, q); st.rt.insert_tensor(sid, sc);
  *out_q_id = qid; *out_scales_id = sid;
  return 0;
}

int32_t applegpu_ffi_copy(uint64_t src_id, uint64_t dst_id) {
  if (!ffi_ready("copy")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (st.rt.is_pending(src_id)) { Status s = st.rt.eval(src_id); if (!s.ok()) { set_ffi_error("copy: eval src failed: " + s.to_string()); return -1; } }
  const TensorRec* src = st.rt.tensor(src_id);
  if (!src || !src->has_meta) { set_ffi_error("copy failed: Invalid tensor: Tensor " + std::to_string(src_id) + " not found"); return -1; }
  const TensorRec* dst = st.rt.tensor(dst_id);
  if (!dst || !dst->buf) { set_ffi_error("copy: dst tensor " + std::to_string(dst_id) + " not found"); return -1; }
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) { set_ffi_error("copy failed: no CUDA device (dry-run mode)"); return -1; }
  TensorRec c;
  Status s = make_contiguous(*src, &c);
  if (!s.ok()) { set_ffi_error("copy failed: " + s.to_string()); return -1; }
  size_t n = c.nbytes();
  if (n > dst->buf->capacity - dst->byte_offset) { set_ffi_error("copy failed: destination buffer is smaller than the source"); return -1; }
  if (n) {
    cudaError_t e = cudaMemcpyAsync(dst->data(), c.data(), n, cudaMemcpyDeviceToDevice, ctx.stream);
    if (e != cudaSuccess) { set_ffi_error(std::string("copy failed: ") + cudaGetErrorString(e)); return -1; }
  }
  return 0;
}

uint8_t* applegpu_ffi_add_out(uint64_t a, uint64_t b, uint64_t* o) { return record_out("add", mk(Op::Add), {a, b}, o); }
uint8_t* applegpu_ffi_mul_out(uint64_t a, uint64_t b, uint64_t* o) { return record_out("mul", mk(Op::Mul), {a, b}, o); }
uint8_t* applegpu_ffi_sub_out(uint64_t a, uint64_t b, uint64_t* o) { return record_out("sub", mk(Op::Sub), {a, b}, o); }
uint8_t* applegpu_ffi_div_out(uint64_t a, uint64_t b, uint64_t* o) { return record_out("div", mk(Op::Div), {a, b}, o); }
uint8_t* applegpu_ffi_matmul_out(uint64_t a, uint64_t b, uint64_t* o) { return record_out("matmul", mk(Op::Matmul), {a, b}, o); }
uint8_t* applegpu_ffi_relu_out(uint64_t x, uint64_t* o) { return record_out("relu", mk(Op::Relu), {x}, o); }
uint8_t* applegpu_ffi_neg_out(uint64_t x, uint64_t* o) { return record_out("neg", mk(Op::Neg), {x}, o); }
uint8_t* applegpu_ffi_threshold_backward_out(uint64_t grad, uint64_t x, float thr, uint64_t* o) {
  OpKind k = mk(Op::ThresholdBackward); k.f0 = thr;
  return record_out("threshold_backward", k, {grad, x}, o);
}
uint8_t* applegpu_ffi_scalar_mul_out(uint64_t x, float scale, uint64_t* o) { OpKind k = mk(Op::ScalarMul); k.f0 = scale; return record_out("scalar_mul", k, {x}, o); }
uint8_t* applegpu_ffi_mean_all_out(uint64_t x, uint64_t* o) {
  // mean_all = reshape to [1, numel] then mean over the last dim -> [1] (ops.rs mean_all composition).
  if (!ffi_ready("mean_all")) return nullptr;
  Dims s;
  {
    LazyState& st = lazy_state();
    std::lock_guard<std::mutex> g(st.mu);
    Status r = st.rt.shape(x, &s);
    if (!r.ok()) { set_ffi_error("mean_all failed: " + r.to_string()); return nullptr; }
  }
  uint64_t n = (uint64_t)numel_of(s);
  uint64_t flat = applegpu_ffi_reshape(x, &n, 1);
  if (!flat) return nullptr;
  uint8_t* p = record_out("mean_all", mk(Op::Mean), {flat}, o);
  applegpu_ffi_free(flat);
  return p;
}

int32_t applegpu_ffi_eval(uint64_t tensor_id) {
  if (!ffi_ready("eval")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.eval(tensor_id);
  if (!s.ok()) { set_ffi_error("eval failed: " + s.to_string()); return -1; }
  return 0;
}
// Waits for the runtime stream. A tcgen05 kernel whose bounded wait gave up leaves its code in the
// pipeline status word; every blocking point of the library reads that word once the stream is idle
// and turns a non-zero value into an error (here, where the signature returns nothing, into the
// last-error text of both flavours), so a timed-out pipeline cannot pass for a result.
void applegpu_ffi_synchronize(void) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry) return;
  k::status_snapshot(ctx.stream, 0);
  cudaStreamSynchronize(ctx.stream);
  int code = k::status_take(ctx.stream, 0);
  if (code != 0) {
    std::string m = "synchronize failed: tensor-core pipeline wait timed out (code " + std::to_string(code) + "); results since the last synchronisation are undefined";
    set_ffi_error(m); set_eager_error(m);
  }
}
int32_t applegpu_ffi_read_f32(uint64_t tensor_id, float* out_ptr, uint64_t max_elements) {
  if (!ffi_ready("read_f32")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.read_f32(tensor_id, out_ptr, max_elements);
  if (!s.ok()) { set_ffi_error("read_f32 failed: " + s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_ffi_upload(uint64_t tensor_id, const void* host_ptr, uint64_t nbytes) {
  if (!ffi_ready("upload")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.write_bytes(tensor_id, host_ptr, (size_t)nbytes);
  if (!s.ok()) { set_ffi_error("upload failed: " + s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_ffi_read_bytes(uint64_t tensor_id, void* host_ptr, uint64_t nbytes) {
  if (!ffi_ready("read_bytes")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.read_bytes(tensor_id, host_ptr, (size_t)nbytes);
  if (!s.ok()) { set_ffi_error("read_bytes failed: " + s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_ffi_tape_begin(const uint64_t* var_inputs, uint32_t n_var) {
  if (!ffi_ready("tape_begin")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (g_rec) { set_ffi_error("tape_begin failed: a tape is already being recorded"); return -1; }
  g_rec.reset(new Tape());
  g_rec_slot.clear();
  g_rec->n_var = n_var;
  for (uint32_t k = 0; k < n_var; k++) { g_rec->ext.push_back(0); g_rec_slot[var_inputs[k]] = -(int64_t)(k + 1); }
  return 0;
}
uint64_t applegpu_ffi_tape_end(const uint64_t* outputs, uint32_t n_out) {
  if (!ffi_ready("tape_end")) return 0;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (!g_rec) { set_ffi_error("tape_end failed: no tape is being recorded"); return 0; }
  std::unique_ptr<Tape> t = std::move(g_rec);
  for (uint32_t k = 0; k < n_out; k++) {
    auto it = g_rec_slot.find(outputs[k]);
    if (it == g_rec_slot.end()) { g_rec_slot.clear(); set_ffi_error("tape_end failed: output " + std::to_string(outputs[k]) + " was not produced on the tape"); return 0; }
    if (it->second < 0 && (uint64_t)(-it->second - 1) >= t->n_var) { g_rec_slot.clear(); set_ffi_error("tape_end failed: output " + std::to_string(outputs[k]) + " is a constant of the tape"); return 0; }
    t->outputs.push_back(it->second);
  }
  g_rec_slot.clear();
  g_tapes.push_back(std::move(t));
  return (uint64_t)g_tapes.size();   // handles start at 1
}
void applegpu_ffi_tape_abort(void) {
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  g_rec.reset();
  g_rec_slot.clear();
}
int32_t applegpu_ffi_tape_replay(uint64_t tape, const uint64_t* var_inputs, uint32_t n_var, uint64_t* out_ids, uint32_t n_out) {
  if (!ffi_ready("tape_replay")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (tape == 0 || tape > g_tapes.size()) { set_ffi_error("tape_replay failed: unknown tape " + std::to_string(tape)); return -1; }
  const Tape& t = *g_tapes[tape - 1];
  if (n_var != t.n_var || n_out != t.outputs.size()) { set_ffi_error("tape_replay failed: the tape takes " + std::to_string(t.n_var) + " inputs and gives " + std::to_string(t.outputs.size()) + " outputs"); return -1; }
  if (g_rec) { set_ffi_error("tape_replay failed: a tape is being recorded"); return -1; }
  std::vector<uint64_t> vals;
  vals.reserve(t.ops.size());
  auto resolve = [&](int64_t s) -> uint64_t {
    if (s >= 0) return vals[(size_t)s];
    size_t k = (size_t)(-s - 1);
    return k < t.n_var ? var_inputs[k] : t.ext[k];
  };
  LazyMetaSrc src(&st.rt);
  for (const TapeOp& op : t.ops) {
    OpNode node;
    node.op = op.kind;
    for (int64_t s : op.in) node.inputs.push_back(resolve(s));
    Status s = infer_node(src, &node);
    if (!s.ok()) {
      // drop what this replay recorded so far
      for (uint64_t v : vals) st.rt.free_tensor(v);
      set_ffi_error("tape_replay failed: " + s.to_string());
      return -1;
    }
    node.id = next_op_id();
    vals.push_back(node.id);
    st.rt.record_op(std::move(node));
  }
  std::unordered_set<uint64_t> kept;
  for (uint32_t k = 0; k < n_out; k++) { out_ids[k] = resolve(t.outputs[k]); kept.insert(out_ids[k]); }
  // values nobody holds a handle to are released as soon as their last consumer has run
  for (uint64_t v : vals) if (!kept.count(v)) st.rt.free_tensor(v);
  return (int32_t)t.ops.size();
}
int32_t applegpu_ffi_tape_replay_loop(const uint64_t* tapes, uint32_t n_tapes, uint32_t iters, uint32_t keep) {
  // Replays single-output tapes without variable inputs round robin, evaluates every result, and keeps the last
  // `keep` results alive (so the pool rotates output buffers too). One library call for the whole loop: the host
  // cost per launch is a few hundred nanoseconds instead of a Python round trip, which is what a kernel of a few
  // microseconds needs to be timed back to back.
  if (!ffi_ready("tape_replay_loop")) return -1;
  if (n_tapes == 0 || keep == 0 || keep > 64) { set_ffi_error("tape_replay_loop failed: need at least one tape and 1..64 kept results"); return -1; }
  std::vector<uint64_t> ring(keep, 0);
  int32_t rc = 0;
  for (uint32_t i = 0; i < iters; i++) {
    uint64_t out = 0;
    if (applegpu_ffi_tape_replay(tapes[i % n_tapes], nullptr, 0, &out, 1) < 0 || applegpu_ffi_eval(out) != 0) { rc = -1; if (out) applegpu_ffi_free(out); break; }
    uint64_t& slot = ring[i % keep];
    if (slot) applegpu_ffi_free(slot);
    slot = out;
  }
  for (uint64_t id : ring) if (id) applegpu_ffi_free(id);
  return rc;
}
void* applegpu_ffi_device_ptr(uint64_t tensor_id) {
  if (!ffi_ready("device_ptr")) return nullptr;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (st.rt.is_pending(tensor_id)) {
    Status s = st.rt.eval(tensor_id);
    if (!s.ok()) { set_ffi_error("device_ptr failed: " + s.to_string()); return nullptr; }
  }
  const TensorRec* t = st.rt.tensor(tensor_id);
  if (!t || !t->has_meta) { set_ffi_error("device_ptr failed: Tensor " + std::to_string(tensor_id) + " not found"); return nullptr; }
  if (!t->contiguous()) { set_ffi_error("device_ptr failed: tensor is a strided view"); return nullptr; }
  return t->data();
}
int32_t applegpu_ffi_read_bytes_async(uint64_t tensor_id, void* host_ptr, uint64_t nbytes) {
  if (!ffi_ready("read_bytes_async")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.read_bytes(tensor_id, host_ptr, (size_t)nbytes, /*wait=*/false);
  if (!s.ok()) { set_ffi_error("read_bytes_async failed: " + s.to_string()); return -1; }
  return 0;
}
uint64_t applegpu_ffi_from_host(const void* host_ptr, const uint64_t* dims, uint32_t ndim, int8_t dtype) {
  DType dt;
  if (!dtype_from_wire(dtype, &dt)) { set_ffi_error("Invalid dtype wire value: " + std::to_string((int)dtype)); return 0; }
  Dims d = to_dims(dims, ndim);
  uint64_t bytes = (uint64_t)numel_of(d) * dtype_size(dt);
  uint64_t id = 0;
  uint8_t* p = applegpu_ffi_alloc(bytes == 0 ? 4 : bytes, dtype, &id);
  if (!p && !DeviceCtx::get().dry) return 0;
  if (!id) return 0;
  if (applegpu_ffi_register_tensor(id, dims, ndim, dtype) != 0) { applegpu_ffi_free(id); return 0; }
  if (host_ptr && bytes && !DeviceCtx::get().dry) {
    if (applegpu_ffi_upload(id, host_ptr, bytes) != 0) { applegpu_ffi_free(id); return 0; }
  }
  return id;
}
int64_t applegpu_ffi_plan(uint64_t tensor_id, char* buf, uint64_t cap) {
  if (!ffi_ready("plan")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  std::string out;
  Status s = st.rt.plan(tensor_id, &out);
  if (!s.ok()) { set_ffi_error("plan failed: " + s.to_string()); return -1; }
  if (buf && cap) { size_t n = out.size() < cap - 1 ? out.size() : (size_t)cap - 1; std::memcpy(buf, out.data(), n); buf[n] = 0; }
  return (int64_t)out.size();
}
int32_t applegpu_ffi_is_pending(uint64_t tensor_id) {
  if (!lazy_state().ready) return 0;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  return st.rt.is_pending(tensor_id) ? 1 : 0;
}
void applegpu_ffi_set_fusion(bool elementwise_chains, bool patterns) { fusion::set_enabled(elementwise_chains, patterns); }

// ── eager flavour ───────────────────────────────────────────────────────────
bool applegpu_eager_init(void) {
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  if (st.ready) return true;
  Status s = init_device(false);
  if (!s.ok()) { set_eager_error(s.to_string()); return false; }
  Shared::get();
  st.ready = true;
  return true;
}
const char* applegpu_eager_last_error(void) { return t_eager_has_error ? t_eager_error.c_str() : nullptr; }

uint8_t* applegpu_eager_alloc(const uint64_t* dims, uint32_t ndim, int8_t dtype, uint64_t* out_id) {
  if (!eager_ready()) return nullptr;
  DType dt;
  if (!dtype_from_wire(dtype, &dt)) { set_eager_error("invalid dtype wire value: " + std::to_string((int)dtype)); return nullptr; }
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  uint64_t id = 0; void* ptr = nullptr;
  Status s = st.rt.alloc(to_dims(dims, ndim), dt, &id, &ptr);
  if (!s.ok()) { set_eager_error("alloc failed: " + s.to_string()); return nullptr; }
  if (out_id) *out_id = id;
  return static_cast<uint8_t*>(ptr);
}
void applegpu_eager_free(uint64_t id) {
  if (!eager_state().ready) return;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  st.rt.free_tensor(id);
}
int32_t applegpu_eager_register_shape(uint64_t id, const uint64_t* dims, uint32_t ndim) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.register_shape(id, to_dims(dims, ndim));
  if (!s.ok()) { set_eager_error(s.kind == ErrKind::InvalidTensor && s.msg.rfind("tensor ", 0) == 0 ? s.msg : s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_eager_shape(uint64_t id, uint64_t* out_dims, uint32_t* out_ndim) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  Dims d;
  Status s = st.rt.shape(id, &d);
  if (!s.ok()) { set_eager_error(s.to_string()); return -1; }
  *out_ndim = (uint32_t)d.size();
  for (size_t i = 0; i < d.size(); i++) out_dims[i] = (uint64_t)d[i];
  return 0;
}
int8_t applegpu_eager_dtype(uint64_t id) {
  if (!eager_state().ready) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  DType dt;
  if (!st.rt.dtype(id, &dt).ok()) return -1;
  return (int8_t)dt;
}

uint8_t* applegpu_eager_add(uint64_t a, uint64_t b, uint64_t* o) { return eager_run(mk(Op::Add), {a, b}, o); }
uint8_t* applegpu_eager_sub(uint64_t a, uint64_t b, uint64_t* o) { return eager_run(mk(Op::Sub), {a, b}, o); }
uint8_t* applegpu_eager_mul(uint64_t a, uint64_t b, uint64_t* o) { return eager_run(mk(Op::Mul), {a, b}, o); }
uint8_t* applegpu_eager_div(uint64_t a, uint64_t b, uint64_t* o) { return eager_run(mk(Op::Div), {a, b}, o); }
uint8_t* applegpu_eager_relu(uint64_t x, uint64_t* o) { return eager_run(mk(Op::Relu), {x}, o); }
uint8_t* applegpu_eager_neg(uint64_t x, uint64_t* o) { return eager_run(mk(Op::Neg), {x}, o); }

uint8_t* applegpu_eager_matmul(uint64_t a, uint64_t b, uint64_t* o) {
  if (!eager_ready()) return nullptr;
  {
    EagerState& st = eager_state();
    std::lock_guard<std::mutex> g(st.mu);
    const TensorRec *ta, *tb;
    Status s = st.rt.get(a, &ta);
    if (s.ok()) s = st.rt.get(b, &tb);
    if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
    if (!ta->contiguous() || !tb->contiguous()) { set_eager_error("Invalid tensor: matmul requires contiguous inputs"); return nullptr; }
  }
  return eager_run(mk(Op::Matmul), {a, b}, o);
}

uint8_t* applegpu_eager_matmul_ex(uint64_t a, uint64_t b, bool ta, bool tb, uint64_t* o) {
  // Transposes are stride swaps on temporary views of the base tensors; the GEMM reads them in place.
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  uint64_t va = a, vb = b;
  auto make_t = [&](uint64_t id, uint64_t* out) -> bool {
    std::lock_guard<std::mutex> g(st.mu);
    const TensorRec* t;
    Status s = st.rt.get(id, &t);
    if (!s.ok()) { set_eager_error(s.to_string()); return false; }
    if (t->shape.size() < 2) { set_eager_error("Invalid tensor: matmul requires 2D+ tensors"); return false; }
    Dims sh = t->shape, stv = t->strides;
    size_t n = sh.size();
    std::swap(sh[n - 1], sh[n - 2]); std::swap(stv[n - 1], stv[n - 2]);
    void* p;
    s = st.rt.create_view(id, sh, stv, 0, out, &p);
    if (!s.ok()) { set_eager_error(s.to_string()); return false; }
    return true;
  };
  if (ta && !make_t(a, &va)) return nullptr;
  if (tb && !make_t(b, &vb)) { if (ta) applegpu_eager_free(va); return nullptr; }
  uint8_t* r = eager_run(mk(Op::Matmul), {va, vb}, o);
  if (ta) applegpu_eager_free(va);
  if (tb) applegpu_eager_free(vb);
  return r;
}

uint8_t* applegpu_eager_threshold_backward(uint64_t grad, uint64_t x, float thr, uint64_t* o) {
  OpKind k = mk(Op::ThresholdBackward); k.f0 = thr;
  return eager_run(k, {grad, x}, o);
}
uint8_t* applegpu_eager_scalar_mul(uint64_t x, float scale, uint64_t* o) { OpKind k = mk(Op::ScalarMul); k.f0 = scale; return eager_run(k, {x}, o); }

static uint8_t* eager_reduce(uint64_t x, int mode, int64_t dim, bool keepdim, uint64_t* o) {
  // mode 0: mean over all elements -> [1]; mode 1: sum over `dim`.
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec* t;
  Status s = st.rt.get(x, &t);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  if (!dtype_is_float(t->dtype) || t->dtype == DType::F64) { set_eager_error(std::string("Unsupported dtype: reduction requires a float dtype, got ") + dtype_name(t->dtype)); return nullptr; }
  Dims out_shape;
  int64_t nd = (int64_t)t->shape.size();
  if (mode == 1) {
    if (dim < 0) dim += nd;
    if (dim < 0 || dim >= nd) { set_eager_error("Invalid tensor: sum_dim: dim out of range for " + std::to_string(nd) + "D tensor"); return nullptr; }
    for (int64_t i = 0; i < nd; i++) { if (i == dim) { if (keepdim) out_shape.push_back(1); } else out_shape.push_back(t->shape[i]); }
  } else out_shape = {1};
  DeviceCtx& ctx = DeviceCtx::get();
  TensorRec c, out;
  s = make_contiguous(*t, &c);
  if (s.ok()) {
    out.shape = out_shape; out.strides = contiguous_strides(out_shape); out.dtype = t->dtype; out.has_meta = true;
    s = Shared::get().pool.acquire(out.nbytes() ? out.nbytes() : 4, &out.buf);
  }
  if (s.ok()) s = ctx.make_current();
  if (s.ok() && ctx.dry) s = Status::compute("no CUDA device (dry-run mode)");
  if (s.ok()) s = mode == 1 ? k::sum_dim(ctx.stream, c.view(), (int)dim, out.view()) : k::mean_all(ctx.stream, c.view(), out.view());
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  uint64_t id = st.rt.adopt(out);
  if (o) *o = id;
  return static_cast<uint8_t*>(out.data());
}
uint8_t* applegpu_eager_mean_all(uint64_t x, uint64_t* o) { return eager_reduce(x, 0, 0, false, o); }
uint8_t* applegpu_eager_sum_dim(uint64_t x, int64_t dim, bool keepdim, uint64_t* o) { return eager_reduce(x, 1, dim, keepdim, o); }

uint8_t* applegpu_eager_create_view(uint64_t base, const uint64_t* shape, const uint64_t* strides, uint32_t ndim, uint64_t offset, uint64_t* out_id) {
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  uint64_t id = 0; void* p = nullptr;
  Status s = st.rt.create_view(base, to_dims(shape, ndim), to_dims(strides, ndim), offset, &id, &p);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  if (out_id) *out_id = id;
  return static_cast<uint8_t*>(p);
}
// ── what a frontend with device-resident buffers needs beside the reference's eager ABI ──
uint8_t* applegpu_eager_view_as(uint64_t base, int8_t dtype, const uint64_t* shape, const uint64_t* strides, uint32_t ndim, uint64_t byte_offset, uint64_t* out_id) {
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  DType dt;
  if (!dtype_from_wire(dtype, &dt)) { set_eager_error("view_as: unknown dtype code " + std::to_string((int)dtype)); return nullptr; }
  const TensorRec* b = st.rt.tensor(base);
  if (!b) { set_eager_error("tensor " + std::to_string(base) + " not found"); return nullptr; }
  if (ndim > (uint32_t)kMaxDims) { set_eager_error("view_as: too many dimensions"); return nullptr; }
  TensorRec v = *b;
  v.dtype = dt; v.shape = to_dims(shape, ndim); v.strides = to_dims(strides, ndim);
  v.byte_offset = b->byte_offset + (size_t)byte_offset;
  // the furthest element the view can reach must lie inside the buffer
  size_t reach = 0;
  bool empty = false;
  for (uint32_t i = 0; i < ndim; i++) { if (v.shape[i] == 0) empty = true; else reach += (size_t)(v.shape[i] - 1) * (size_t)v.strides[i]; }
  if (!empty && b->buf && v.byte_offset + (reach + 1) * dtype_size(dt) > b->buf->capacity) { set_eager_error("view_as: the view reaches past the end of the buffer"); return nullptr; }
  uint64_t id = st.rt.adopt(v);
  if (out_id) *out_id = id;
  return static_cast<uint8_t*>(v.data());
}
int32_t applegpu_eager_copy(uint64_t dst, uint64_t src) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec *d, *s0;
  Status s = st.rt.get(dst, &d);
  if (s.ok()) s = st.rt.get(src, &s0);
  if (s.ok() && d->shape != s0->shape) s = Status::invalid("copy: shape mismatch " + dims_str(d->shape) + " vs " + dims_str(s0->shape));
  DeviceCtx& ctx = DeviceCtx::get();
  if (s.ok() && ctx.dry) s = Status::compute("no CUDA device (dry-run mode)");
  if (s.ok() && numel_of(d->shape) > 0) {
    if (d->dtype == s0->dtype) s = k::copy_strided(ctx.stream, s0->view(), d->view());
    else if (d->contiguous() && s0->contiguous()) s = k::cast(ctx.stream, s0->view(), d->view());
    else s = Status::invalid("copy: a converting copy needs contiguous tensors");
    if (s.ok()) note_launches(1);
  }
  if (!s.ok()) { set_eager_error(s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_eager_fill(uint64_t id, uint64_t bit_pattern) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec* t;
  Status s = st.rt.get(id, &t);
  DeviceCtx& ctx = DeviceCtx::get();
  if (s.ok() && ctx.dry) s = Status::compute("no CUDA device (dry-run mode)");
  if (s.ok() && numel_of(t->shape) > 0) {
    if (t->contiguous()) { s = k::fill(ctx.stream, t->data(), (int)dtype_size(t->dtype), bit_pattern, numel_of(t->shape)); if (s.ok()) note_launches(1); }
    else {
      // a strided view: fill a one-element source and broadcast it through the strided copy
      TensorRec one;
      one.dtype = t->dtype; one.shape = t->shape; one.strides.assign(t->shape.size(), 0); one.has_meta = true;
      s = Shared::get().pool.acquire(256, &one.buf);
      if (s.ok()) s = k::fill(ctx.stream, one.data(), (int)dtype_size(t->dtype), bit_pattern, 1);
      if (s.ok()) s = k::copy_strided(ctx.stream, one.view(), t->view());
      if (s.ok()) note_launches(2);
    }
  }
  if (!s.ok()) { set_eager_error(s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_eager_add_scaled_inplace(uint64_t self, uint64_t other, float alpha) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = st.rt.add_scaled_inplace(self, other, alpha);
  if (!s.ok()) { set_eager_error(s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_eager_add_inplace(uint64_t self, uint64_t other) { return applegpu_eager_add_scaled_inplace(self, other, 1.0f); }
void applegpu_eager_flush_and_wait(void) { applegpu_ffi_synchronize(); }
void applegpu_eager_synchronize(void) { applegpu_ffi_synchronize(); }

uint8_t* applegpu_eager_embedding(uint64_t w, uint64_t idx, uint64_t* o) { return eager_run(mk(Op::Embedding), {w, idx}, o); }
uint8_t* applegpu_eager_layer_norm(uint64_t x, uint64_t gamma, uint64_t beta, float eps, uint64_t* o) {
  OpKind k = mk(Op::LayerNorm); k.f0 = eps;
  return eager_run(k, {x, gamma, beta}, o);
}
uint8_t* applegpu_eager_gelu(uint64_t x, uint64_t* o) { return eager_run(mk(Op::Gelu), {x}, o); }
uint8_t* applegpu_eager_softmax(uint64_t x, uint64_t* o) { return eager_run(mk(Op::Softmax), {x}, o); }
uint64_t applegpu_eager_find_by_data_ptr(const uint8_t* ptr) {
  if (!eager_state().ready) return 0;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  return st.rt.find_by_data_ptr(ptr);
}

// ── compiled-graph executor ─────────────────────────────────────────────────
// One call runs a whole serialized op list on the eager runtime (reference: eager_ffi.rs:661-708,
// compiled_graph.rs:7-9,44-58,65-199). Wire format per op, little-endian:
//   op_code u8, n_inputs u8, inputs [u16; n] (indices into the node table: graph inputs first, then
//   one entry per executed op), out_ndim u8, out_dims [u64; ndim], out_dtype u8, params_len u8,
//   params [f32; plen].
// Op codes as upstream: 0 add, 1 sub, 2 mul, 3 div, 4 matmul, 5 relu, 6 neg, 7 threshold_backward
// (param 0 = threshold), 8 scalar_mul (param 0 = scale), 9 mean_all, 10 sum_dim (params dim,
// keepdim), 11 transpose (last two dims, a view), 12 view (contiguous strides of out_dims), 13 addmm
// (bias, m1, m2), 255 identity. Non-contiguous matmul operands are first copied, as upstream does
// with scalar_mul(x, 1.0). Unlike upstream every read of the byte stream is bounds-checked.
namespace {
struct GraphCursor {
  const uint8_t* p; size_t n; size_t i = 0; bool ok = true;
  bool need(size_t k) { if (i + k > n) { ok = false; return false; } return true; }
  uint8_t u8() { if (!need(1)) return 0; return p[i++]; }
  uint16_t u16() { if (!need(2)) return 0; uint16_t v; std::memcpy(&v, p + i, 2); i += 2; return v; }
  uint64_t u64() { if (!need(8)) return 0; uint64_t v; std::memcpy(&v, p + i, 8); i += 8; return v; }
  float f32() { if (!need(4)) return 0.f; float v; std::memcpy(&v, p + i, 4); i += 4; return v; }
};
struct GraphSlot { uint64_t id; uint8_t* ptr; bool contiguous; };
}  // namespace

int32_t applegpu_eager_execute_graph(const uint8_t* ops_data, uint32_t ops_len, const uint64_t* input_tids, uint32_t n_inputs,
                                     const uint16_t* output_indices, uint32_t n_outputs, uint64_t* out_tids, uint8_t** out_ptrs) {
  if (!eager_ready()) return -1;
  std::vector<GraphSlot> nodes;
  {
    EagerState& st = eager_state();
    std::lock_guard<std::mutex> g(st.mu);
    for (uint32_t k = 0; k < n_inputs; k++) {
      const TensorRec* t = st.rt.tensor(input_tids[k]);
      nodes.push_back({input_tids[k], t ? static_cast<uint8_t*>(t->data()) : nullptr, t ? t->contiguous() : true});
    }
  }
  auto fail = [](const std::string& m) { set_eager_error("compiled graph failed: " + m); return -1; };
  GraphCursor c{ops_data, ops_len};
  while (c.i < c.n) {
    uint8_t code = c.u8();
    uint8_t nin = c.u8();
    std::vector<size_t> idx;
    for (int k = 0; k < nin; k++) idx.push_back(c.u16());
    uint8_t ondim = c.u8();
    std::vector<uint64_t> odims;
    for (int k = 0; k < ondim; k++) odims.push_back(c.u64());
    (void)c.u8();  // out_dtype: informational, results take their dtype from the operands
    uint8_t plen = c.u8();
    std::vector<float> params;
    for (int k = 0; k < plen; k++) params.push_back(c.f32());
    if (!c.ok) return fail("truncated op stream");
    for (size_t ix : idx) if (ix >= nodes.size()) return fail("input index " + std::to_string(ix) + " out of range");
    auto need_inputs = [&](size_t k) { return idx.size() >= k; };
    auto in = [&](size_t k) -> GraphSlot { return nodes[idx[k]]; };
    // a contiguous copy of a strided operand (upstream: scalar_mul(x, 1.0))
    auto contiguous_id = [&](GraphSlot s, uint64_t* id) -> bool {
      if (s.contiguous) { *id = s.id; return true; }
      uint64_t cid = 0;
      if (!applegpu_eager_scalar_mul(s.id, 1.0f, &cid) && cid == 0) return false;
      *id = cid; return true;
    };
    if (code == 255) { if (!need_inputs(1)) return fail("identity needs one input"); nodes.push_back(in(0)); continue; }
    uint64_t oid = 0; uint8_t* optr = nullptr; bool ocontig = true;
    switch (code) {
      case 0: case 1: case 2: case 3: {
        if (!need_inputs(2)) return fail("binary op needs two inputs");
        uint64_t a = in(0).id, b = in(1).id;
        optr = code == 0 ? applegpu_eager_add(a, b, &oid) : code == 1 ? applegpu_eager_sub(a, b, &oid)
             : code == 2 ? applegpu_eager_mul(a, b, &oid) : applegpu_eager_div(a, b, &oid);
        break;
      }
      case 4: {
        if (!need_inputs(2)) return fail("matmul needs two inputs");
        uint64_t a, b;
        if (!contiguous_id(in(0), &a) || !contiguous_id(in(1), &b)) return -1;
        optr = applegpu_eager_matmul(a, b, &oid);
        break;
      }
      case 13: {
        if (!need_inputs(3)) return fail("addmm needs three inputs");
        uint64_t m1, m2, mm = 0;
        if (!contiguous_id(in(1), &m1) || !contiguous_id(in(2), &m2)) return -1;
        if (!applegpu_eager_matmul(m1, m2, &mm) && mm == 0) return -1;
        optr = applegpu_eager_add(mm, in(0).id, &oid);
        break;
      }
      case 5: if (!need_inputs(1)) return fail("relu needs one input"); optr = applegpu_eager_relu(in(0).id, &oid); break;
      case 6: if (!need_inputs(1)) return fail("neg needs one input"); optr = applegpu_eager_neg(in(0).id, &oid); break;
      case 7:
        if (!need_inputs(2)) return fail("threshold_backward needs two inputs");
        optr = applegpu_eager_threshold_backward(in(0).id, in(1).id, params.empty() ? 0.f : params[0], &oid);
        break;
      case 8: if (!need_inputs(1)) return fail("scalar_mul needs one input"); optr = applegpu_eager_scalar_mul(in(0).id, params.empty() ? 1.f : params[0], &oid); break;
      case 9: if (!need_inputs(1)) return fail("mean_all needs one input"); optr = applegpu_eager_mean_all(in(0).id, &oid); break;
      case 10:
        if (!need_inputs(1)) return fail("sum_dim needs one input");
        optr = applegpu_eager_sum_dim(in(0).id, params.empty() ? 0 : (int64_t)params[0], params.size() > 1 && params[1] != 0.f, &oid);
        break;
      case 11: case 12: {
        if (!need_inputs(1)) return fail("view needs one input");
        std::vector<uint64_t> shape, strides;
        if (code == 11) {
          EagerState& st = eager_state();
          std::lock_guard<std::mutex> g(st.mu);
          const TensorRec* t = st.rt.tensor(in(0).id);
          if (!t) return fail("Tensor " + std::to_string(in(0).id) + " not found");
          if (t->shape.size() < 2) return fail("Invalid tensor: transpose requires 2D+");
          for (int64_t d : t->shape) shape.push_back((uint64_t)d);
          for (int64_t s : t->strides) strides.push_back((uint64_t)s);
          std::swap(shape[shape.size() - 2], shape[shape.size() - 1]);
          std::swap(strides[strides.size() - 2], strides[strides.size() - 1]);
          ocontig = false;
        } else {
          shape = odims;
          strides.assign(shape.size(), 1);
          for (int k = (int)shape.size() - 2; k >= 0; k--) strides[k] = strides[k + 1] * shape[k + 1];
        }
        optr = applegpu_eager_create_view(in(0).id, shape.data(), strides.data(), (uint32_t)shape.size(), 0, &oid);
        break;
      }
      default: return fail("unsupported op: " + std::to_string((int)code));
    }
    if (oid == 0) return -1;  // the op recorded its own error text
    nodes.push_back({oid, optr, ocontig});
  }
  uint32_t done = 0;
  for (; done < n_outputs; done++) {
    size_t ix = output_indices[done];
    if (ix >= nodes.size()) return fail("output " + std::to_string(ix) + " out of range");
    if (out_tids) out_tids[done] = nodes[ix].id;
    if (out_ptrs) out_ptrs[done] = nodes[ix].ptr;
  }
  return (int32_t)done;
}

uint8_t* applegpu_eager_gelu_exact(uint64_t x, uint64_t* o) { return eager_run(mk(Op::GeluExact), {x}, o); }
uint8_t* applegpu_eager_softmax_causal(uint64_t x, uint64_t* o) { return eager_run(mk(Op::SoftmaxCausal), {x}, o); }
uint8_t* applegpu_eager_add_bias(uint64_t x, uint64_t b, uint64_t* o) { return eager_run(mk(Op::AddBias), {x, b}, o); }
uint8_t* applegpu_eager_argmax(uint64_t x, uint64_t* o) { return eager_run(mk(Op::Argmax), {x}, o); }
uint8_t* applegpu_eager_gather(uint64_t x, uint32_t dim, uint64_t idx, uint64_t* o) { OpKind k = mk(Op::Gather); k.i0 = dim; return eager_run(k, {x, idx}, o); }
uint8_t* applegpu_eager_index_select(uint64_t x, uint32_t dim, uint64_t idx, uint64_t* o) { OpKind k = mk(Op::IndexSelect); k.i0 = dim; return eager_run(k, {x, idx}, o); }
uint8_t* applegpu_eager_cast(uint64_t x, int8_t target, uint64_t* o) {
  DType dt;
  if (!dtype_from_wire(target, &dt)) { set_eager_error("invalid dtype wire value: " + std::to_string((int)target)); return nullptr; }
  OpKind k = mk(Op::Cast); k.dt = dt;
  return eager_run(k, {x}, o);
}
uint8_t* applegpu_eager_quantize(uint64_t x, int8_t target, float scale, int32_t zp, uint64_t* o) {
  DType dt;
  if (!dtype_from_wire(target, &dt)) { set_eager_error("invalid dtype wire value: " + std::to_string((int)target)); return nullptr; }
  OpKind k = mk(Op::Quantize); k.dt = dt; k.f0 = scale; k.i0 = zp;
  return eager_run(k, {x}, o);
}
uint8_t* applegpu_eager_dequantize(uint64_t x, int8_t target, float scale, int32_t zp, uint64_t* o) {
  DType dt;
  if (!dtype_from_wire(target, &dt)) { set_eager_error("invalid dtype wire value: " + std::to_string((int)target)); return nullptr; }
  OpKind k = mk(Op::Dequantize); k.dt = dt; k.f0 = scale; k.i0 = zp;
  return eager_run(k, {x}, o);
}
uint8_t* applegpu_eager_unary(uint64_t x, const char* name, uint64_t* o) {
  struct E { const char* n; Op op; };
  static const E table[] = {{"neg", Op::Neg}, {"relu", Op::Relu}, {"exp", Op::Exp}, {"log", Op::Log}, {"sqrt", Op::Sqrt}, {"tanh", Op::Tanh},
                            {"sin", Op::Sin}, {"cos", Op::Cos}, {"gelu", Op::Gelu}, {"gelu_exact", Op::GeluExact}, {"sigmoid", Op::Sigmoid},
                            {"abs", Op::Abs}, {"sign", Op::Sign}};
  for (auto& e : table) if (name && std::strcmp(name, e.n) == 0) return eager_run(mk(e.op), {x}, o);
  set_eager_error(std::string("unknown unary op: ") + (name ? name : "(null)"));
  return nullptr;
}

// Shape inference for the two ops below reuses matmul's rules through a scratch node.
uint8_t* applegpu_eager_linear(uint64_t x, uint64_t w, uint64_t bias, uint64_t residual, int32_t act, bool transpose_w, uint64_t* o) {
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec *tx, *tw, *tb = nullptr, *tr = nullptr;
  Status s = st.rt.get(x, &tx);
  if (s.ok()) s = st.rt.get(w, &tw);
  if (s.ok() && bias) s = st.rt.get(bias, &tb);
  if (s.ok() && residual) s = st.rt.get(residual, &tr);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  if (tx->shape.size() < 2 || tw->shape.size() != 2) { set_eager_error("Invalid tensor: linear requires x >= 2D and a 2D weight"); return nullptr; }
  if (tx->dtype != tw->dtype) { set_eager_error(std::string("Invalid tensor: dtype mismatch: ") + dtype_debug(tx->dtype) + " vs " + dtype_debug(tw->dtype)); return nullptr; }
  TensorRec wv = *tw;
  if (transpose_w) { std::swap(wv.shape[0], wv.shape[1]); std::swap(wv.strides[0], wv.strides[1]); }
  if (tx->shape.back() != wv.shape[0]) {
    set_eager_error("Invalid tensor: matmul inner dim mismatch: " + std::to_string(tx->shape.back()) + " vs " + std::to_string(wv.shape[0]));
    return nullptr;
  }
  OpNode node;
  node.op.op = Op::FusedLinear; node.op.f0 = 1.0f;
  node.op.act = act == 1 ? k::Act::GeluTanh : act == 2 ? k::Act::GeluErf : act == 3 ? k::Act::Relu : k::Act::None;
  node.out_shape = tx->shape; node.out_shape.back() = wv.shape[1]; node.out_dtype = tx->dtype;
  // collapse x to 2-D so the bias lands on the last dim
  TensorRec xc;
  s = make_contiguous(*tx, &xc);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  Dims full = node.out_shape;
  int64_t rows = numel_of(xc.shape) / (xc.shape.back() ? xc.shape.back() : 1);
  xc.shape = {rows, xc.shape.back()}; xc.strides = contiguous_strides(xc.shape);
  node.out_shape = {rows, wv.shape[1]};
  std::vector<const TensorRec*> ins{&xc, &wv};
  TensorRec rc;
  if (tb) {
    if (!(tb->shape.size() == 1 && tb->shape[0] == wv.shape[1])) { set_eager_error("Invalid tensor: linear bias must be [" + std::to_string(wv.shape[1]) + "]"); return nullptr; }
    node.op.has_bias = true; ins.push_back(tb);
  }
  if (tr) {
    if (tr->shape != full) { set_eager_error("Invalid tensor: linear residual shape " + dims_str(tr->shape) + " must be " + dims_str(full)); return nullptr; }
    s = make_contiguous(*tr, &rc);
    if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
    rc.shape = node.out_shape; rc.strides = contiguous_strides(rc.shape);
    node.op.has_residual = true; ins.push_back(&rc);
  }
  TensorRec out;
  s = execute_node(node, ins, &out, nullptr);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  out.shape = full; out.strides = contiguous_strides(full);
  uint64_t id = st.rt.adopt(out);
  if (o) *o = id;
  return static_cast<uint8_t*>(out.data());
}

uint8_t* applegpu_eager_attention(uint64_t q, uint64_t kk, uint64_t v, bool causal, uint64_t* o) {
  if (!eager_ready()) return nullptr;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec *tq, *tk, *tv;
  Status s = st.rt.get(q, &tq);
  if (s.ok()) s = st.rt.get(kk, &tk);
  if (s.ok()) s = st.rt.get(v, &tv);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  if (tq->shape.size() < 2 || tk->shape.size() < 2 || tv->shape.size() < 2) { set_eager_error("Invalid tensor: attention requires at least 2D tensors for Q, K, V"); return nullptr; }
  if (!(tq->dtype == tk->dtype && tk->dtype == tv->dtype) || !dtype_is_float(tq->dtype) || tq->dtype == DType::F64) { set_eager_error("Invalid tensor: attention requires Q, K, V of one float dtype"); return nullptr; }
  if (tk->shape.back() != tq->shape.back()) { set_eager_error("Invalid tensor: Q and K must have same d_k: " + std::to_string(tq->shape.back()) + " vs " + std::to_string(tk->shape.back())); return nullptr; }
  if (tk->shape[tk->shape.size() - 2] != tv->shape[tv->shape.size() - 2]) { set_eager_error("Invalid tensor: K and V must have same kv_len: " + std::to_string(tk->shape[tk->shape.size() - 2]) + " vs " + std::to_string(tv->shape[tv->shape.size() - 2])); return nullptr; }
  if (tq->shape.size() != tk->shape.size() || tq->shape.size() != tv->shape.size() ||
      !std::equal(tq->shape.begin(), tq->shape.end() - 2, tk->shape.begin()) || !std::equal(tq->shape.begin(), tq->shape.end() - 2, tv->shape.begin())) {
    set_eager_error("Invalid tensor: attention requires matching leading dims on Q, K, V"); return nullptr;
  }
  OpNode node;
  node.op.op = Op::FusedAttention; node.op.causal = causal;
  node.out_shape = tq->shape; node.out_shape.back() = tv->shape.back(); node.out_dtype = tq->dtype;
  TensorRec out;
  s = execute_node(node, {tq, tk, tv}, &out, nullptr);
  if (!s.ok()) { set_eager_error(s.to_string()); return nullptr; }
  uint64_t id = st.rt.adopt(out);
  if (o) *o = id;
  return static_cast<uint8_t*>(out.data());
}

int32_t applegpu_eager_upload(uint64_t id, const void* host_ptr, uint64_t nbytes) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec* t;
  Status s = st.rt.get(id, &t);
  if (s.ok()) s = upload(*t, host_ptr, (size_t)nbytes);
  if (!s.ok()) { set_eager_error(s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_eager_download(uint64_t id, void* host_ptr, uint64_t nbytes) {
  if (!eager_ready()) return -1;
  EagerState& st = eager_state();
  std::lock_guard<std::mutex> g(st.mu);
  const TensorRec* t;
  Status s = st.rt.get(id, &t);
  if (s.ok()) s = download(*t, host_ptr, (size_t)nbytes);
  if (!s.ok()) { set_eager_error(s.to_string()); return -1; }
  return 0;
}

// ── runtime services ────────────────────────────────────────────────────────
void applegpu_pool_stats(uint64_t* out7) {
  PoolStats s = Shared::get().pool.stats();
  out7[0] = s.hits; out7[1] = s.misses; out7[2] = s.pooled_bytes; out7[3] = s.bucket_count;
  out7[4] = s.live_bytes; out7[5] = s.peak_live_bytes; out7[6] = s.live_buffers;
}
void applegpu_pool_drain(void) { Shared::get().pool.drain(); }
void applegpu_pool_set_watermark(uint64_t n) { Shared::get().pool.set_max_pooled_bytes((size_t)n); }
int32_t applegpu_pool_prewarm(const uint64_t* sizes, uint32_t n) {
  std::vector<size_t> v(sizes, sizes + n);
  Status s = Shared::get().pool.prewarm(v);
  if (!s.ok()) { set_ffi_error(s.to_string()); return -1; }
  return 0;
}
void applegpu_pool_fail_next(int32_t n) { Shared::get().pool.fail_next_allocs(n); }
uint64_t applegpu_memory_usage(void) { return Shared::get().pool.stats().live_bytes; }
uint64_t applegpu_tensor_count(void) {
  uint64_t n = 0;
  { LazyState& st = lazy_state(); std::lock_guard<std::mutex> g(st.mu); n += st.rt.tensor_count(); }
  { EagerState& st = eager_state(); std::lock_guard<std::mutex> g(st.mu); n += st.rt.tensor_count(); }
  return n;
}
void* applegpu_stream(void) { return (void*)DeviceCtx::get().stream; }
int32_t applegpu_device(void) { return DeviceCtx::get().device; }
const char* applegpu_device_name(void) { return DeviceCtx::get().name.c_str(); }
uint64_t applegpu_launch_count(void) { return ag::launch_count(); }
void applegpu_set_matmul_path(int32_t mode) { k::set_matmul_path(mode); }
void applegpu_set_f32_split(bool on) { ag::set_f32_split(on); }
int32_t applegpu_set_host_visible(int32_t on) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.ready) return (ctx.host_visible == (on != 0)) ? 0 : -1;   // buffers of the other kind may already be out
  DeviceCtx::request_host_visible(on != 0);
  return 0;
}
int32_t applegpu_host_visible(void) { return DeviceCtx::get().host_visible ? 1 : 0; }
void applegpu_set_attention_path(int32_t mode) { ag::g_fused_attention = (mode != 1); }
void applegpu_set_gemm_tile(int32_t code) { k::set_gemm_tile(code); }
void applegpu_set_sm_margin(int32_t n) { k::set_sm_margin(n); }
void applegpu_set_gemm_chain(bool on) { ag::set_gemm_chain(on); }
bool applegpu_gemm_chain_enabled(void) { return ag::gemm_chain_enabled(); }
void applegpu_set_gemm_chain_min_rows(int64_t rows) { k::set_gemm_chain_min_rows(rows); }
int64_t applegpu_gemm_chain_min_rows(void) { return k::gemm_chain_min_rows(); }
int32_t applegpu_pipeline_status(void) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry) return 0;
  return k::matmul_take_status(ctx.stream);
}
const char* applegpu_matmul_path(uint64_t a, uint64_t b, bool eager) {
  TensorRec ta, tb;
  if (eager) {
    EagerState& st = eager_state(); std::lock_guard<std::mutex> g(st.mu);
    const TensorRec *pa, *pb;
    if (!st.rt.get(a, &pa).ok() || !st.rt.get(b, &pb).ok()) return nullptr;
    ta = *pa; tb = *pb;
  } else {
    LazyState& st = lazy_state(); std::lock_guard<std::mutex> g(st.mu);
    const TensorRec *pa = st.rt.tensor(a), *pb = st.rt.tensor(b);
    if (!pa || !pb || !pa->has_meta || !pb->has_meta) return nullptr;
    ta = *pa; tb = *pb;
  }
  if (ta.shape.size() < 2 || tb.shape.size() < 2) return nullptr;
  k::GemmDesc d;
  size_t an = ta.shape.size(), bn = tb.shape.size();
  d.dtype = ta.dtype; d.b_dtype = tb.dtype; d.a = ta.data(); d.b = tb.data(); d.c = nullptr;
  d.m = ta.shape[an - 2]; d.k = ta.shape[an - 1]; d.n = tb.shape[bn - 1];
  d.a_row = ta.strides[an - 2]; d.a_col = ta.strides[an - 1]; d.b_row = tb.strides[bn - 2]; d.b_col = tb.strides[bn - 1];
  d.batch = 1; d.a_batch = d.b_batch = d.c_batch = 0; d.c_row = d.n;
  return k::matmul_path(d);
}
int32_t applegpu_timer_start(void) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry) return -1;
  if (!g_ev0) { cudaEventCreate(&g_ev0); cudaEventCreate(&g_ev1); }
  return cudaEventRecord(g_ev0, ctx.stream) == cudaSuccess ? 0 : -1;
}
float applegpu_timer_stop_ms(void) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry || !g_ev0) return -1.f;
  if (cudaEventRecord(g_ev1, ctx.stream) != cudaSuccess) return -1.f;
  if (cudaEventSynchronize(g_ev1) != cudaSuccess) return -1.f;
  float ms = -1.f;
  cudaEventElapsedTime(&ms, g_ev0, g_ev1);
  return ms;
}
// Completion markers: a small ring of reusable events (timing disabled: cheaper to record).
static constexpr int kMarkerSlots = 64;
static cudaEvent_t g_markers[kMarkerSlots];
static uint64_t g_marker_seq = 0;
static std::mutex g_marker_mu;
uint64_t applegpu_marker_record(void) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry) return 0;
  std::lock_guard<std::mutex> g(g_marker_mu);
  uint64_t seq = ++g_marker_seq;
  cudaEvent_t& ev = g_markers[seq % kMarkerSlots];
  if (!ev && cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) { ev = nullptr; return 0; }
  k::status_snapshot(ctx.stream, 1 + (int)(seq % kMarkerSlots));   // read back by marker_wait
  if (cudaEventRecord(ev, ctx.stream) != cudaSuccess) return 0;
  return seq;
}
int32_t applegpu_marker_wait(uint64_t marker) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry || marker == 0) return -1;
  cudaEvent_t ev;
  {
    std::lock_guard<std::mutex> g(g_marker_mu);
    if (marker > g_marker_seq) return -1;
    // a slot that has been re-recorded since marks a later point of the same stream: waiting on it
    // still implies that `marker` completed
    ev = g_markers[marker % kMarkerSlots];
  }
  if (!ev) return -1;
  if (cudaEventSynchronize(ev) != cudaSuccess) return -1;
  int code = k::status_take(ctx.stream, 1 + (int)(marker % kMarkerSlots));
  if (code != 0) {
    set_ffi_error("marker_wait failed: tensor-core pipeline wait timed out (code " + std::to_string(code) + ")");
    return -1;
  }
  return 0;
}
int32_t applegpu_flush_l2(void) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry) return -1;
  if (!g_flush_buf && !Shared::get().pool.acquire(kFlushBytes, &g_flush_buf).ok()) { g_flush_buf.reset(); return -1; }
  return k::flush_l2(ctx.stream, g_flush_buf->ptr, kFlushBytes).ok() ? 0 : -1;
}
// ── GPT-2 greedy decoder (preallocated KV cache, captured step) ─────────────
static Status materialised(LazyRuntime& rt, uint64_t id, TensorRec* out) {
  if (rt.is_pending(id)) AG_RETURN_IF_ERROR(rt.eval(id));
  const TensorRec* t = rt.tensor(id);
  if (!t || !t->has_meta || !t->buf) return Status::invalid("Tensor " + std::to_string(id) + " not found");
  *out = *t;
  return Status::OK();
}
uint64_t applegpu_gpt2_decoder_create(const uint64_t* weight_ids, uint32_t n_weights, uint32_t n_layer, uint32_t n_head, uint32_t n_embd, uint32_t vocab,
                                      uint32_t n_positions, uint32_t batch, uint32_t max_len) {
  if (!ffi_ready("gpt2_decoder_create")) return 0;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  std::vector<TensorRec> w(n_weights);
  for (uint32_t i = 0; i < n_weights; i++) {
    Status s = materialised(st.rt, weight_ids[i], &w[i]);
    if (!s.ok()) { set_ffi_error("gpt2_decoder_create failed: " + s.to_string()); return 0; }
  }
  Gpt2DecoderCfg cfg{(int)n_layer, (int)n_head, (int)n_embd, (int)vocab, (int)n_positions, (int)batch, (int)max_len};
  uint64_t h = 0;
  Status s = decoder_create(w, cfg, &h);
  if (!s.ok()) { set_ffi_error("gpt2_decoder_create failed: " + s.to_string()); return 0; }
  return h;
}
int32_t applegpu_gpt2_decoder_prefill(uint64_t decoder, const uint64_t* kv_ids, uint32_t n_kv, uint64_t first_tokens_id, uint32_t prompt_len) {
  if (!ffi_ready("gpt2_decoder_prefill")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  std::vector<TensorRec> kv(n_kv);
  TensorRec tok;
  Status s = Status::OK();
  for (uint32_t i = 0; i < n_kv && s.ok(); i++) s = materialised(st.rt, kv_ids[i], &kv[i]);
  if (s.ok()) s = materialised(st.rt, first_tokens_id, &tok);
  if (s.ok()) s = decoder_prefill(decoder, kv, tok, (int)prompt_len);
  if (!s.ok()) { set_ffi_error("gpt2_decoder_prefill failed: " + s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_gpt2_decoder_steps(uint64_t decoder, uint32_t n_steps, int32_t* host_tokens, bool use_graph) {
  if (!ffi_ready("gpt2_decoder_steps")) return -1;
  LazyState& st = lazy_state();
  std::lock_guard<std::mutex> g(st.mu);
  Status s = decoder_steps(decoder, (int)n_steps, host_tokens, use_graph);
  if (!s.ok()) { set_ffi_error("gpt2_decoder_steps failed: " + s.to_string()); return -1; }
  return 0;
}
int32_t applegpu_gpt2_decoder_launches_per_step(uint64_t decoder) { return decoder_launches_per_step(decoder); }
int32_t applegpu_gpt2_decoder_uses_graph(uint64_t decoder) { return decoder_uses_graph(decoder); }
int32_t applegpu_gpt2_decoder_set_engine(uint64_t decoder, int32_t engine) {
  Status s = decoder_set_engine(decoder, engine);
  if (!s.ok()) { set_ffi_error("gpt2_decoder_set_engine failed: " + s.to_string()); return -1; }
  return 0;
}
void applegpu_gpt2_decoder_destroy(uint64_t decoder) { decoder_destroy(decoder); }

int32_t applegpu_test_wait_runs_out(int32_t code, uint32_t limit_us) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.ready || ctx.dry) return -1;
  Status s = k::launch_wait_runs_out(ctx.stream, code, (unsigned long long)limit_us * 1000ull);
  if (!s.ok()) { set_ffi_error("test_wait_runs_out failed: " + s.to_string()); return -1; }
  return 0;
}
void applegpu_profile_enable(bool on) { ag::profile::enable(on); }
void applegpu_profile_clear(void) { ag::profile::clear(); }
void applegpu_profile_filter(const char* prefixes) { ag::profile::set_filter(prefixes ? prefixes : ""); }
int64_t applegpu_profile_report(char* buf, uint64_t cap) {
  std::string out = ag::profile::report();
  if (buf && cap) { size_t n = out.size() < cap - 1 ? out.size() : (size_t)cap - 1; std::memcpy(buf, out.data(), n); buf[n] = 0; }
  return (int64_t)out.size();
}
const char* applegpu_resolve_kernel(const char* base_name, int8_t dtype) {
  thread_local std::string out;
  DType dt;
  if (!base_name || !dtype_from_wire(dtype, &dt) || dt == DType::F64) return nullptr;
  std::string b(base_name);
  static const char* float_only[] = {"matmul", "softmax", "softmax_causal", "layer_norm", "gelu", "gelu_exact", "add_bias", "embedding",
                                     "elementwise_exp", "elementwise_log", "elementwise_sqrt", "elementwise_tanh", "elementwise_relu", "sigmoid"};
  for (const char* f : float_only) if (b == f && !dtype_is_float(dt)) return nullptr;
  out = b + dtype_suffix(dt);
  return out.c_str();
}

}  // extern "C"
