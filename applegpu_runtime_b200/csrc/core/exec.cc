// Node executor: turns one graph node plus materialised inputs into kernel launches.
//
// Plays the role of LazyRuntime::execute_node_nb (lazy.rs:1571-2429) and of the per-op bodies
// of EagerRuntime (eager.rs:246-1172). Layout-only ops (transpose, slice, reshape) return
// views that share the input buffer whenever the strides allow it — upstream materialises each
// of them with a copy kernel (lazy.rs:1891-1917, :2246-2262) — and consumers either read the
// strided view directly (matmul, element-wise, copy) or make it contiguous first.
#include "runtime.h"
#include <algorithm>
#include <array>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <map>
#include <mutex>
#include <sstream>

namespace ag {

std::atomic<uint64_t> g_launch_count{0};
uint64_t launch_count() { return g_launch_count.load(); }
void note_launches(uint64_t n) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }

// Optional per-kernel timing: CUDA events bracket each launch on the runtime stream and are
// resolved when the report is read. Off by default (events cost host time, not kernel time).
namespace profile {
struct Span { std::string name; cudaEvent_t a, b; double work; };
static bool g_on = false;
static std::vector<Span> g_spans;
static std::vector<cudaEvent_t> g_free_events;   // events are reused: creating one costs more host time than a small kernel runs
static std::mutex g_mu;
void enable(bool on) { std::lock_guard<std::mutex> g(g_mu); g_on = on; }
bool enabled() { return g_on; }
void clear() {
  std::lock_guard<std::mutex> g(g_mu);
  for (auto& s : g_spans) { g_free_events.push_back(s.a); g_free_events.push_back(s.b); }
  g_spans.clear();
}
// Only nodes whose kernel name starts with one of these prefixes get a span (empty: every node). Bracketing every
// kernel of a forward makes the host the bottleneck and breaks every programmatic-launch overlap; bracketing one
// kernel family keeps the rest of the step as it normally runs.
static std::vector<std::string> g_filter;
void set_filter(const std::string& csv) {
  std::lock_guard<std::mutex> g(g_mu);
  g_filter.clear();
  size_t i = 0;
  while (i < csv.size()) {
    size_t j = csv.find(',', i);
    if (j == std::string::npos) j = csv.size();
    if (j > i) g_filter.push_back(csv.substr(i, j - i));
    i = j + 1;
  }
}
static bool wanted(const std::string& name) {
  if (g_filter.empty()) return true;
  for (const std::string& p : g_filter) if (name.compare(0, p.size(), p) == 0) return true;
  return false;
}
static bool take_event(cudaEvent_t* e) {
  if (!g_free_events.empty()) { *e = g_free_events.back(); g_free_events.pop_back(); return true; }
  return cudaEventCreate(e) == cudaSuccess;
}
struct Scope {
  bool live = false; size_t idx = 0;
  Scope(const std::string& name, double work) {
    if (!g_on) return;
    DeviceCtx& ctx = DeviceCtx::get();
    if (ctx.dry) return;
    Span sp; sp.name = name; sp.work = work;
    std::lock_guard<std::mutex> g(g_mu);
    if (!take_event(&sp.a) || !take_event(&sp.b)) return;
    cudaEventRecord(sp.a, ctx.stream);
    g_spans.push_back(sp); idx = g_spans.size() - 1; live = true;
  }
  ~Scope() {
    if (!live) return;
    std::lock_guard<std::mutex> g(g_mu);
    cudaEventRecord(g_spans[idx].b, DeviceCtx::get().stream);
  }
};
// "name count total_ms work" per line; work = algorithmic flops (GEMM, attention) or bytes (the rest).
std::string report() {
  DeviceCtx& ctx = DeviceCtx::get();
  if (!ctx.dry && ctx.ready) cudaStreamSynchronize(ctx.stream);
  std::lock_guard<std::mutex> g(g_mu);
  std::map<std::string, std::array<double, 3>> agg;
  for (auto& s : g_spans) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, s.a, s.b) != cudaSuccess) continue;
    auto& a = agg[s.name]; a[0] += 1; a[1] += ms; a[2] += s.work;
  }
  std::ostringstream os;
  for (auto& kv : agg) os << kv.first << " " << (long long)kv.second[0] << " " << kv.second[1] << " " << kv.second[2] << "\n";
  return os.str();
}
}  // namespace profile

#define AG_LAUNCH(expr) do { AG_RETURN_IF_ERROR(expr); g_launch_count.fetch_add(1, std::memory_order_relaxed); } while (0)

// ── chained linears ──────────────────────────────────────────────────────────
// Inside one evaluation (LazyRuntime::eval opens a ChainScope) a fused linear that the chained tensor-core kernel can take
// is not launched at once but held back; while the next node is again such a linear that reads the held one's result, it
// joins. Anything else (another kind of node, a linear that does not follow, four links, the end of the evaluation)
// launches what is held: one product through k::matmul, several as ONE k::matmul_chain launch. The held products keep
// their operands and results alive, so the pool cannot hand one of those buffers to a later link.
namespace chain {
struct Pending { k::GemmDesc g; std::vector<TensorRec> keep; std::string span; double work; };
static thread_local int t_scope_depth = 0;
static thread_local std::vector<Pending> t_pending;
static thread_local std::string t_span;     // the profile span of the linear being executed (set by execute_node)
static thread_local double t_work = 0;
static bool g_enabled = [] { const char* v = std::getenv("APPLEGPU_GEMM_CHAIN"); return !(v && v[0] == '0'); }();   // APPLEGPU_GEMM_CHAIN=0 / set_gemm_chain(false): every linear is its own launch
static bool active() { return g_enabled && t_scope_depth > 0; }

static Status flush() {
  if (t_pending.empty()) return Status::OK();
  std::vector<Pending> p;
  p.swap(t_pending);
  cudaStream_t s = DeviceCtx::get().stream;
  if (p.size() == 1) {
    if (profile::enabled() && profile::wanted(p[0].span)) {
      profile::Scope scope(p[0].span, p[0].work);
      AG_LAUNCH(k::matmul(s, p[0].g));
    } else {
      AG_LAUNCH(k::matmul(s, p[0].g));
    }
    return Status::OK();
  }
  std::vector<k::GemmDesc> descs;
  double work = 0;
  for (const Pending& q : p) { descs.push_back(q.g); work += q.work; }
  // one span for the launch, under the links' own name: a chain of n links counts as one launch doing their work
  if (profile::enabled() && profile::wanted(p[0].span)) {
    profile::Scope scope(p[0].span, work);
    AG_LAUNCH(k::matmul_chain(s, descs.data(), (int)descs.size()));
  } else {
    AG_LAUNCH(k::matmul_chain(s, descs.data(), (int)descs.size()));
  }
  return Status::OK();
}

// Holds `g` back, or launches it, as described above. `keep` = every tensor the product touches.
static Status submit(const k::GemmDesc& g, std::vector<TensorRec> keep) {
  std::vector<k::GemmDesc> held;
  for (const Pending& q : t_pending) held.push_back(q.g);
  if (!t_pending.empty() && !k::matmul_chain_can_append(held.data(), (int)held.size(), g)) AG_RETURN_IF_ERROR(flush());
  if (!k::matmul_chain_candidate(g)) {
    AG_RETURN_IF_ERROR(flush());
    cudaStream_t s = DeviceCtx::get().stream;
    if (profile::enabled() && profile::wanted(t_span)) {
      profile::Scope scope(t_span, t_work);
      AG_LAUNCH(k::matmul(s, g));
    } else {
      AG_LAUNCH(k::matmul(s, g));
    }
    return Status::OK();
  }
  t_pending.push_back(Pending{g, std::move(keep), t_span, t_work});
  if ((int)t_pending.size() == k::kChainMax) return flush();
  return Status::OK();
}
}  // namespace chain

void set_gemm_chain(bool on) { chain::g_enabled = on; }
bool gemm_chain_enabled() { return chain::g_enabled; }
ChainScope::ChainScope() { chain::t_scope_depth++; }
ChainScope::~ChainScope() {
  // only non-empty after an error ended the evaluation early: the held products' results are already handed out as
  // materialised tensors, so they are still launched (best effort)
  if (--chain::t_scope_depth == 0 && !chain::t_pending.empty()) (void)chain::flush();
}
Status ChainScope::finish() { return chain::flush(); }

static Status alloc_out(const Dims& shape, DType dt, TensorRec* out, std::shared_ptr<Buffer> out_buf) {
  out->shape = shape; out->strides = contiguous_strides(shape); out->dtype = dt; out->byte_offset = 0; out->has_meta = true;
  size_t nbytes = (size_t)numel_of(shape) * dtype_size(dt);
  if (out_buf) {
    if (out_buf->capacity < nbytes) return Status::compute("pre-allocated output is too small");
    out->buf = out_buf;
    return Status::OK();
  }
  return Shared::get().pool.acquire(nbytes == 0 ? 4 : nbytes, &out->buf);
}

Status make_contiguous(const TensorRec& in, TensorRec* out) {
  if (in.contiguous()) { *out = in; return Status::OK(); }
  AG_RETURN_IF_ERROR(alloc_out(in.shape, in.dtype, out, nullptr));
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) return Status::OK();
  AG_LAUNCH(k::copy_strided(ctx.stream, in.view(), out->view()));
  return Status::OK();
}

Status upload(const TensorRec& t, const void* host, size_t nbytes) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) return Status::compute("no CUDA device (dry-run mode)");
  if (!t.contiguous()) return Status::invalid("upload needs a contiguous tensor");
  if (nbytes > t.nbytes()) return Status::invalid("upload of " + std::to_string(nbytes) + " bytes exceeds tensor size " + std::to_string(t.nbytes()));
  if (nbytes == 0) return Status::OK();
  cudaError_t e = cudaMemcpyAsync(t.data(), host, nbytes, cudaMemcpyHostToDevice, ctx.stream);
  if (e != cudaSuccess) return Status::compute(std::string("upload: ") + cudaGetErrorString(e));
  return Status::OK();
}

Status download(const TensorRec& t, void* host, size_t nbytes, bool wait) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) return Status::compute("no CUDA device (dry-run mode)");
  TensorRec c;
  AG_RETURN_IF_ERROR(make_contiguous(t, &c));
  if (nbytes > c.nbytes()) nbytes = c.nbytes();
  if (nbytes) {
    cudaError_t e = cudaMemcpyAsync(host, c.data(), nbytes, cudaMemcpyDeviceToHost, ctx.stream);
    if (e != cudaSuccess) return Status::compute(std::string("download: ") + cudaGetErrorString(e));
  }
  if (!wait) return Status::OK();  // stream-ordered: the bytes are defined after the next synchronize
  k::status_snapshot(ctx.stream, 0);
  cudaError_t e = cudaStreamSynchronize(ctx.stream);
  if (e != cudaSuccess) return Status::compute(std::string("synchronize: ") + cudaGetErrorString(e));
  // a tcgen05 kernel whose bounded wait gave up left its code in the pipeline status word: the bytes are not a result
  int code = k::status_take(ctx.stream, 0);
  if (code != 0) return Status::compute("tensor-core pipeline wait timed out (code " + std::to_string(code) + ")");
  return Status::OK();
}

// Strides that present `old` (shape, strides) as `new_shape` without moving data, if any.
static bool view_strides(const Dims& old_shape, const Dims& old_strides, const Dims& new_shape, Dims* out) {
  int64_t numel = numel_of(old_shape);
  out->assign(new_shape.size(), 0);
  if (numel == 0) { *out = contiguous_strides(new_shape); return true; }
  int vd = (int)new_shape.size() - 1;
  if (old_shape.empty()) { for (auto& s : *out) s = 1; return true; }
  int64_t chunk_base = old_strides.back();
  int64_t t_numel = 1, v_numel = 1;
  for (int td = (int)old_shape.size() - 1; td >= 0; td--) {
    t_numel *= old_shape[td];
    if (td == 0 || (old_shape[td - 1] != 1 && old_strides[td - 1] != t_numel * chunk_base)) {
      while (vd >= 0 && (v_numel < t_numel || new_shape[vd] == 1)) {
        (*out)[vd] = v_numel * chunk_base;
        v_numel *= new_shape[vd];
        vd--;
      }
      if (v_numel != t_numel) return false;
      if (td > 0) { chunk_base = old_strides[td - 1]; t_numel = 1; v_numel = 1; }
    }
  }
  return vd == -1;
}

// Describe a (possibly strided, possibly broadcast) batched matmul for the GEMM launchers.
static Status build_gemm(const TensorRec& a, const TensorRec& b, const TensorRec& c, k::GemmDesc* d,
                         std::vector<TensorRec>* keep_alive) {
  TensorRec A = a, B = b;
  auto fill = [&](const TensorRec& A2, const TensorRec& B2) -> bool {
    int an = (int)A2.shape.size(), bn = (int)B2.shape.size(), cn = (int)c.shape.size();
    d->m = A2.shape[an - 2]; d->k = A2.shape[an - 1]; d->n = B2.shape[bn - 1];
    d->a_row = A2.strides[an - 2]; d->a_col = A2.strides[an - 1];
    d->b_row = B2.strides[bn - 2]; d->b_col = B2.strides[bn - 1];
    d->c_row = c.strides[cn - 2];
    // batch dims of C with per-operand strides (0 where the operand broadcasts)
    int nb = cn - 2;
    std::vector<int64_t> bs(nb), sa(nb, 0), sb(nb, 0), sc(nb);
    for (int i = 0; i < nb; i++) {
      bs[i] = c.shape[i]; sc[i] = c.strides[i];
      int ai = i - (nb - (an - 2)), bi = i - (nb - (bn - 2));
      if (ai >= 0 && A2.shape[ai] != 1) sa[i] = A2.strides[ai];
      if (bi >= 0 && B2.shape[bi] != 1) sb[i] = B2.strides[bi];
    }
    // drop size-1 dims, merge neighbours that are jointly collapsible
    std::vector<int64_t> ms, ma, mb, mc;
    for (int i = 0; i < nb; i++) {
      if (bs[i] == 1) continue;
      if (!ms.empty() && ma.back() == sa[i] * bs[i] && mb.back() == sb[i] * bs[i] && mc.back() == sc[i] * bs[i]) {
        ms.back() *= bs[i]; ma.back() = sa[i]; mb.back() = sb[i]; mc.back() = sc[i];
      } else { ms.push_back(bs[i]); ma.push_back(sa[i]); mb.push_back(sb[i]); mc.push_back(sc[i]); }
    }
    if (ms.size() > 2) return false;
    d->batch = 1; d->batch_inner = 1;
    d->a_batch = d->b_batch = d->c_batch = 0; d->a_batch_inner = d->b_batch_inner = d->c_batch_inner = 0;
    if (ms.size() == 1) { d->batch = ms[0]; d->a_batch = ma[0]; d->b_batch = mb[0]; d->c_batch = mc[0]; }
    if (ms.size() == 2) {
      d->batch = ms[0]; d->a_batch = ma[0]; d->b_batch = mb[0]; d->c_batch = mc[0];
      d->batch_inner = ms[1]; d->a_batch_inner = ma[1]; d->b_batch_inner = mb[1]; d->c_batch_inner = mc[1];
    }
    return true;
  };
  if (!fill(A, B)) {
    TensorRec Ac, Bc;
    AG_RETURN_IF_ERROR(make_contiguous(A, &Ac));
    AG_RETURN_IF_ERROR(make_contiguous(B, &Bc));
    keep_alive->push_back(Ac); keep_alive->push_back(Bc);
    A = Ac; B = Bc;
    if (!fill(A, B)) return Status::compute("matmul batch layout cannot be expressed in two stride levels");
  }
  d->a = A.data(); d->b = B.data(); d->c = c.data();
  d->dtype = A.dtype; d->b_dtype = B.dtype;
  return Status::OK();
}

// float32 matmul on the tensor cores: each operand is split into three bf16 terms (kernels/index_quant.cu
// split_bf16x3) and one bf16 GEMM over the six-fold K extent accumulates the six largest cross terms in
// float32, smallest first; C, bias and residual stay float32. Error is ~2^-22 relative to the exact
// product (inside the reference's 1e-4 tolerance by three orders of magnitude) at about a sixth of the
// bf16 tensor rate, against the CUDA-core kernel's ~30 TFLOP/s. Taken for products large enough to pay for
// the two split passes and whose layouts the TMA path accepts; *done stays false otherwise.
namespace {
bool g_f32_split = true;
bool g_pitch_rows = [] { const char* v = std::getenv("APPLEGPU_PITCH_ROWS"); return !(v && v[0] == '0'); }();   // APPLEGPU_PITCH_ROWS=0: always dense outputs
}
void set_f32_split(bool on) { g_f32_split = on; }
static Status matmul_f32_split(cudaStream_t s, const k::GemmDesc& g, bool* done) {
  *done = false;
  if (!g_f32_split) return Status::OK();
  const double flops = 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch * (double)g.batch_inner;
  if (flops < 2.0e9 || g.batch_inner != 1 || g.k % 8 != 0 || g.m < 64 || g.n < 64) return Status::OK();
  if (g.a_col != 1 || g.a_row % 4 != 0 || g.a_batch % 4 != 0) return Status::OK();
  const bool b_nmajor = g.b_col == 1;            // [K, N] rows
  const bool b_kmajor = g.b_row == 1;            // [N, K] rows (a transposed view)
  if (!b_nmajor && !b_kmajor) return Status::OK();
  if (b_nmajor && (g.n % 8 != 0 || g.b_row % 4 != 0)) return Status::OK();
  if (b_kmajor && !b_nmajor && g.b_col % 4 != 0) return Status::OK();
  if (g.b_batch % 4 != 0) return Status::OK();
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(g.a) || !al16(g.b)) return Status::OK();
  const int64_t a_copies = (g.batch > 1 && g.a_batch != 0) ? g.batch : 1;
  const int64_t b_copies = (g.batch > 1 && g.b_batch != 0) ? g.batch : 1;
  if (a_copies > 65535 || b_copies > 65535) return Status::OK();
  TensorRec a2, b2;
  AG_RETURN_IF_ERROR(alloc_out({a_copies, g.m, 6 * g.k}, DType::BF16, &a2, nullptr));
  AG_RETURN_IF_ERROR(alloc_out({b_copies, 6 * g.k, g.n}, DType::BF16, &b2, nullptr));
  k::GemmDesc h = g;
  h.dtype = DType::BF16; h.b_dtype = DType::BF16; h.c_f32 = true;
  h.k = 6 * g.k;
  h.a = a2.data(); h.a_row = 6 * g.k; h.a_col = 1; h.a_batch = a_copies > 1 ? g.m * 6 * g.k : 0;
  h.b = b2.data();
  if (b_nmajor) { h.b_row = g.n; h.b_col = 1; } else { h.b_row = 1; h.b_col = 6 * g.k; }
  h.b_batch = b_copies > 1 ? 6 * g.k * g.n : 0;
  if (std::string(k::matmul_path(h)) != "tcgen05") return Status::OK();   // e.g. the CUDA-core kernel is forced
  AG_LAUNCH(k::split_bf16x3(s, static_cast<const float*>(g.a), a2.data(), g.m, g.k, g.a_row, a_copies, g.a_batch, /*stack_rows=*/false, /*b_side=*/false));
  if (b_nmajor) AG_LAUNCH(k::split_bf16x3(s, static_cast<const float*>(g.b), b2.data(), g.k, g.n, g.b_row, b_copies, g.b_batch, /*stack_rows=*/true, /*b_side=*/true));
  else AG_LAUNCH(k::split_bf16x3(s, static_cast<const float*>(g.b), b2.data(), g.n, g.k, g.b_col, b_copies, g.b_batch, /*stack_rows=*/false, /*b_side=*/true));
  AG_LAUNCH(k::matmul(s, h));
  *done = true;
  return Status::OK();
}

static k::UnOp unop_of(Op op) {
  switch (op) {
    case Op::Neg: return k::UnOp::Neg; case Op::Relu: return k::UnOp::Relu; case Op::Exp: return k::UnOp::Exp;
    case Op::Log: return k::UnOp::Log; case Op::Sqrt: return k::UnOp::Sqrt; case Op::Tanh: return k::UnOp::Tanh;
    case Op::Sin: return k::UnOp::Sin; case Op::Cos: return k::UnOp::Cos; case Op::Gelu: return k::UnOp::Gelu;
    case Op::GeluExact: return k::UnOp::GeluExact; case Op::Sigmoid: return k::UnOp::Sigmoid; case Op::Abs: return k::UnOp::Abs;
    case Op::Sign: return k::UnOp::Sign; default: return k::UnOp::Copy;
  }
}

bool g_fused_attention = true;  // false: always compose attention from GEMM + softmax + GEMM

// `dst` is the already allocated destination, shaped [.., Tq, dv] with any leading strides (the
// merge-heads form passes a [B, h, T, dv] view of a [B, T, h*dv] buffer).
static Status attention_exec(const TensorRec& q, const TensorRec& kk, const TensorRec& v, bool causal, const TensorRec& dst) {
  const Dims& out_shape = dst.shape;
  // softmax[_causal]((Q K^T) * 1/sqrt(d_k)) V with the score matrix materialised in the storage
  // dtype, as ops.rs:1559-1569 / :1605-1615 compose it; the scale rides in the first GEMM's epilogue.
  DeviceCtx& ctx = DeviceCtx::get();
  int qn = (int)q.shape.size(), kn = (int)kk.shape.size();
  int64_t tq = q.shape[qn - 2], dk = q.shape[qn - 1], tk = kk.shape[kn - 2];
  Dims sshape(out_shape.begin(), out_shape.end() - 1);
  sshape.push_back(tk);
  // Single-kernel form when the shapes allow it: leading dims (batch, heads) equal on Q, K, V.
  if (!ctx.dry && qn <= 4 && qn >= 2 && kn == qn && (int)v.shape.size() == qn && q.strides.back() == 1 && kk.strides.back() == 1 &&
      v.strides.back() == 1 && std::equal(q.shape.begin(), q.shape.end() - 2, kk.shape.begin()) &&
      std::equal(q.shape.begin(), q.shape.end() - 2, v.shape.begin()) && g_fused_attention) {
    k::AttnDesc ad;
    ad.dtype = q.dtype; ad.q = q.data(); ad.k = kk.data(); ad.v = v.data();
    ad.batch = qn == 4 ? q.shape[0] : 1; ad.heads = qn >= 3 ? q.shape[qn - 3] : 1;
    ad.tq = tq; ad.tk = tk; ad.d = dk; ad.dv = v.shape.back();
    auto lead = [&](const TensorRec& t, int64_t* sb, int64_t* sh, int64_t* st) {
      int n = (int)t.shape.size();
      *st = t.strides[n - 2];
      *sh = n >= 3 ? t.strides[n - 3] : 0;
      *sb = n == 4 ? t.strides[0] : 0;
    };
    lead(q, &ad.q_b, &ad.q_h, &ad.q_t); lead(kk, &ad.k_b, &ad.k_h, &ad.k_t); lead(v, &ad.v_b, &ad.v_h, &ad.v_t);
    ad.scale = 1.0f / std::sqrt((float)dk); ad.causal = causal;
    ad.o = dst.data();
    lead(dst, &ad.o_b, &ad.o_h, &ad.o_t);
    const bool same_dtype = q.dtype == kk.dtype && q.dtype == v.dtype && q.dtype == dst.dtype;
    if (same_dtype && k::attention_fused_eligible(ad)) {
      AG_LAUNCH(k::attention(ctx.stream, ad));
      return Status::OK();
    }
    if (same_dtype && dst.strides.back() == 1 && k::attention_f32_eligible(ad)) {
      AG_LAUNCH(k::attention_f32(ctx.stream, ad));
      return Status::OK();
    }
  }
  TensorRec scores;
  AG_RETURN_IF_ERROR(alloc_out(sshape, q.dtype, &scores, nullptr));
  if (ctx.dry) return Status::OK();
  (void)tq;
  TensorRec kt = kk;  // K^T as a view
  std::swap(kt.shape[kn - 1], kt.shape[kn - 2]);
  std::swap(kt.strides[kn - 1], kt.strides[kn - 2]);
  std::vector<TensorRec> keep;
  k::GemmDesc g1;
  AG_RETURN_IF_ERROR(build_gemm(q, kt, scores, &g1, &keep));
  g1.ep.alpha = 1.0f / std::sqrt((float)dk);
  AG_LAUNCH(k::matmul(ctx.stream, g1));
  AG_LAUNCH(k::softmax(ctx.stream, scores.view(), causal, scores.view()));
  k::GemmDesc g2;
  AG_RETURN_IF_ERROR(build_gemm(scores, v, dst, &g2, &keep));
  AG_LAUNCH(k::matmul(ctx.stream, g2));
  return Status::OK();
}

// Algorithmic work of a node: flops for contractions, bytes (inputs + output) otherwise.
static double node_work(const OpNode& node, const std::vector<const TensorRec*>& in) {
  const OpKind& kd = node.op;
  double out_elems = (double)numel_of(node.out_shape);
  if (kd.op == Op::Matmul || kd.op == Op::FusedLinear || kd.op == Op::MatmulInt8) {
    double k = in[0]->shape.empty() ? 1.0 : (double)in[0]->shape.back();
    if (kd.op == Op::FusedLinear && kd.i2 == 1 && !in[1]->shape.empty()) out_elems *= (double)in[1]->shape.back();  // rows x vocab, not rows
    return 2.0 * out_elems * k;
  }
  if (kd.op == Op::FusedAttention) {
    const Dims& q = in[0]->shape; const Dims& kk = in[1]->shape;
    double bh = 1; for (size_t i = 0; i + 2 < q.size(); i++) bh *= (double)q[i];
    double tq = (double)q[q.size() - 2], d = (double)q.back(), tk = (double)kk[kk.size() - 2], dv = (double)node.out_shape.back();
    return 2.0 * bh * tq * tk * (d + dv);
  }
  double bytes = out_elems * (double)dtype_size(node.out_dtype);
  if (kd.op == Op::Embedding || kd.op == Op::FusedEmbedAdd) return 2.0 * bytes * (kd.op == Op::FusedEmbedAdd ? 1.5 : 1.0);
  for (auto* t : in) bytes += (double)t->nbytes();
  return bytes;
}

static Status execute_node_impl(const OpNode& node, const std::vector<const TensorRec*>& in, TensorRec* out, std::shared_ptr<Buffer> out_buf);

// A fused linear that may be held back for chaining: 16-bit, neither the int8-weight nor the row-argmax form, and every
// operand contiguous (so that preparing it launches no copy that would have to see a held product's result).
static bool linear_deferrable(const OpNode& node, const std::vector<const TensorRec*>& in) {
  if (!chain::active() || node.op.op != Op::FusedLinear || node.op.i1 == 1 || node.op.i2 == 1 || DeviceCtx::get().dry) return false;
  if (in.size() < 2 || !(in[0]->dtype == DType::BF16 || in[0]->dtype == DType::F16) || in[1]->dtype != in[0]->dtype) return false;
  if (in[0]->shape.size() != 2) return false;
  for (size_t i = 0; i < in.size(); i++) if (i != 1 && !in[i]->contiguous()) return false;   // the weight may be a strided view
  return true;
}

Status execute_node(const OpNode& node, const std::vector<const TensorRec*>& in, TensorRec* out, std::shared_ptr<Buffer> out_buf) {
  {
    // host-visible mode: the host may have read or written any operand since its last use on the device
    const DeviceCtx& ctx = DeviceCtx::get();
    if (ctx.host_visible) {
      for (const TensorRec* t : in) if (t && t->buf && !t->buf->borrowed) ctx.prefetch(t->buf->ptr, t->buf->capacity);
      if (out_buf && !out_buf->borrowed) ctx.prefetch(out_buf->ptr, out_buf->capacity);
    }
  }
  // layout-only ops that return views launch nothing: no span (an event pair around nothing would only add host work)
  const bool view_only = !out_buf && (node.op.op == Op::Transpose || node.op.op == Op::Slice || node.op.op == Op::Reshape);
  // a held-back linear is launched before any other node runs (view-only nodes launch nothing and touch no data)
  const bool may_defer = linear_deferrable(node, in);
  if (!view_only && !may_defer) AG_RETURN_IF_ERROR(chain::flush());
  if (may_defer) {
    // its span, if any, is opened where it is launched
    chain::t_span = node.op.kernel_name() + dtype_suffix(node.out_dtype);
    chain::t_work = profile::enabled() ? node_work(node, in) : 0.0;
    return execute_node_impl(node, in, out, out_buf);
  }
  if (!profile::enabled() || view_only) return execute_node_impl(node, in, out, out_buf);
  std::string name = node.op.kernel_name();
  if (node.op.op == Op::FusedElementwise) name = "fused_elementwise";
  if (!profile::wanted(name)) return execute_node_impl(node, in, out, out_buf);
  profile::Scope scope(name + dtype_suffix(node.out_dtype), node_work(node, in));
  return execute_node_impl(node, in, out, out_buf);
}

static Status execute_node_impl(const OpNode& node, const std::vector<const TensorRec*>& in, TensorRec* out, std::shared_ptr<Buffer> out_buf) {
  DeviceCtx& ctx = DeviceCtx::get();
  AG_RETURN_IF_ERROR(ctx.make_current());
  const OpKind& kd = node.op;
  cudaStream_t s = ctx.stream;
  const bool dry = ctx.dry;

  // layout-only ops first: they may return views
  switch (kd.op) {
    case Op::Transpose: {
      TensorRec v = *in[0];
      std::swap(v.shape[kd.i0], v.shape[kd.i1]);
      std::swap(v.strides[kd.i0], v.strides[kd.i1]);
      if (!out_buf) { *out = v; out->has_meta = true; return Status::OK(); }
      AG_RETURN_IF_ERROR(alloc_out(node.out_shape, node.out_dtype, out, out_buf));
      if (!dry) AG_LAUNCH(k::copy_strided(s, v.view(), out->view()));
      return Status::OK();
    }
    case Op::Slice: {
      TensorRec v = *in[0];
      v.byte_offset += (size_t)(kd.i1 * v.strides[kd.i0]) * dtype_size(v.dtype);
      v.shape[kd.i0] = kd.i2 - kd.i1;
      if (!out_buf) { *out = v; out->has_meta = true; return Status::OK(); }
      AG_RETURN_IF_ERROR(alloc_out(node.out_shape, node.out_dtype, out, out_buf));
      if (!dry) AG_LAUNCH(k::copy_strided(s, v.view(), out->view()));
      return Status::OK();
    }
    case Op::Reshape: {
      Dims ns;
      if (!out_buf && view_strides(in[0]->shape, in[0]->strides, node.out_shape, &ns)) {
        *out = *in[0]; out->shape = node.out_shape; out->strides = ns; out->has_meta = true;
        return Status::OK();
      }
      // gather into a contiguous buffer of the old shape, then relabel
      AG_RETURN_IF_ERROR(alloc_out(in[0]->shape, node.out_dtype, out, out_buf));
      if (!dry) AG_LAUNCH(k::copy_strided(s, in[0]->view(), out->view()));
      out->shape = node.out_shape; out->strides = contiguous_strides(node.out_shape);
      return Status::OK();
    }
    default: break;
  }

  if (kd.op == Op::FusedAttention) {
    AG_RETURN_IF_ERROR(alloc_out(node.out_shape, node.out_dtype, out, out_buf));
    TensorRec dst = *out;
    if (kd.i0 == 1) {
      // merge-heads form: the node's result is [B, T, h*dv] (or [B*T, h*dv]); attention writes it
      // through a [B, h, T, dv] view, so no transpose copy follows.
      const Dims& l = kd.shape;  // logical [B, h, T, dv]
      dst.shape = l;
      dst.strides = {l[2] * l[1] * l[3], l[3], l[1] * l[3], 1};
    }
    return attention_exec(*in[0], *in[1], *in[2], kd.causal, dst);
  }

  // A large 16-bit product whose rows are not a multiple of 16 bytes (the 50257-wide LM head) gets a
  // row pitch rounded up to 16 bytes: the GEMM's epilogue then stores 64-byte row segments instead of
  // 2-byte elements. The result is an ordinary strided view; consumers that need dense rows copy it,
  // argmax and reshape read it as it lies.
  bool pitched = false;
  if ((kd.op == Op::Matmul || (kd.op == Op::FusedLinear && kd.i2 != 1 && kd.i1 != 1 && !kd.has_residual)) && !out_buf && !dry && g_pitch_rows &&
      node.out_shape.size() == 2 && dtype_size(node.out_dtype) == 2 && node.out_shape[1] % 8 != 0 && node.out_shape[1] >= 1024 &&
      node.out_shape[0] >= 128) {
    const int64_t pitch = (node.out_shape[1] + 15) / 16 * 16;   // 32-byte rows: the GEMM stores one row per lane with 256-bit accesses
    out->shape = node.out_shape; out->strides = {pitch, 1}; out->dtype = node.out_dtype; out->byte_offset = 0; out->has_meta = true;
    AG_RETURN_IF_ERROR(Shared::get().pool.acquire((size_t)(node.out_shape[0] * pitch) * 2, &out->buf));
    pitched = true;
  }
  if (!pitched) AG_RETURN_IF_ERROR(alloc_out(node.out_shape, node.out_dtype, out, out_buf));
  if (dry) return Status::OK();
  TView ov = out->view();

  switch (kd.op) {
    case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: {
      k::BinOp bop = kd.op == Op::Add ? k::BinOp::Add : kd.op == Op::Sub ? k::BinOp::Sub : kd.op == Op::Mul ? k::BinOp::Mul : k::BinOp::Div;
      AG_LAUNCH(k::binary(s, bop, in[0]->view(), in[1]->view(), ov));
      return Status::OK();
    }
    case Op::Neg: case Op::Relu: case Op::Exp: case Op::Log: case Op::Sqrt: case Op::Tanh: case Op::Sin: case Op::Cos:
    case Op::Gelu: case Op::GeluExact: case Op::Sigmoid: case Op::Abs: case Op::Sign:
      AG_LAUNCH(k::unary(s, unop_of(kd.op), in[0]->view(), ov));
      return Status::OK();
    case Op::ScalarMul:
      AG_LAUNCH(k::scalar_mul(s, in[0]->view(), kd.f0, ov));
      return Status::OK();
    case Op::FusedElementwise: {
      std::vector<TView> views;
      for (auto* t : in) views.push_back(t->view());
      AG_LAUNCH(k::fused_elementwise(s, kd.prog, views.data(), ov));
      return Status::OK();
    }
    case Op::Matmul: case Op::FusedLinear: case Op::MatmulInt8: {
      std::vector<TensorRec> keep;
      k::GemmDesc g;
      size_t idx = 2;
      const bool int8_w = kd.op == Op::MatmulInt8 || (kd.op == Op::FusedLinear && kd.i1 == 1);
      if (int8_w) {
        // x [.., M, K] @ (w_q [N, K] * scales[N])^T: B is K-major int8, the per-channel scales go to the
        // epilogue. With f16/bf16 activations and more than one row block the tensor-core kernel reads the
        // int8 weights as they lie and widens them in its prologue (one launch, no widened copy in global
        // memory). Shapes that kernel does not take (a single row block: decode steps; K not a multiple of
        // 16) get the weights widened (exactly) into a pooled [N, K] buffer of the activation type first.
        TensorRec x, w;
        AG_RETURN_IF_ERROR(make_contiguous(*in[0], &x));
        AG_RETURN_IF_ERROR(make_contiguous(*in[1], &w));
        keep.push_back(x); keep.push_back(w);
        g.dtype = x.dtype; g.b_dtype = DType::I8;
        g.a = x.data(); g.b = w.data(); g.c = out->data();
        g.k = x.shape.back(); g.m = numel_of(x.shape) / (g.k ? g.k : 1); g.n = w.shape[0];
        g.batch = 1; g.batch_inner = 1;
        g.a_row = g.k; g.a_col = 1; g.a_batch = 0;
        g.b_row = 1; g.b_col = g.k; g.b_batch = 0;
        g.c_row = g.n; g.c_batch = 0;
        g.ep.b_scales = (const float*)in[2]->data();
        if ((x.dtype == DType::BF16 || x.dtype == DType::F16) && g.k % 8 == 0 && g.m > 0 && g.n > 0 && !dry && !k::matmul_w8_fused_eligible(g)) {
          TensorRec wide;
          AG_RETURN_IF_ERROR(alloc_out(w.shape, x.dtype, &wide, nullptr));
          AG_LAUNCH(k::cast(s, w.view(), wide.view()));
          keep.push_back(wide);
          g.b = wide.data(); g.b_dtype = x.dtype;
        }
        idx = 3;
      } else if (kd.op == Op::FusedLinear && kd.i2 == 1) {
        // Row argmax of a product that is never stored: out is int32 [rows...]; the GEMM merges per-row
        // (value, column) keys into a zeroed u64 scratch, a small kernel turns them into indices.
        TensorRec cmeta;
        cmeta.dtype = in[0]->dtype;
        cmeta.shape = {in[0]->shape[in[0]->shape.size() - 2], in[1]->shape.back()};
        cmeta.strides = contiguous_strides(cmeta.shape);
        AG_RETURN_IF_ERROR(build_gemm(*in[0], *in[1], cmeta, &g, &keep));
        if (dry) return Status::OK();
        if (std::string(k::matmul_path(g)) == "tcgen05" && g.batch == 1 && g.batch_inner == 1) {
          TensorRec keys;
          AG_RETURN_IF_ERROR(alloc_out({g.m}, DType::I64, &keys, nullptr));
          cudaError_t ce = cudaMemsetAsync(keys.data(), 0, (size_t)g.m * 8, s);
          if (ce != cudaSuccess) return Status::compute(std::string("argmax keys: ") + cudaGetErrorString(ce));
          g.c = nullptr;
          g.ep.argmax_keys = static_cast<unsigned long long*>(keys.data());
          AG_LAUNCH(k::matmul(s, g));
          AG_LAUNCH(k::argmax_finalize(s, g.ep.argmax_keys, static_cast<int32_t*>(out->data()), g.m));
          return Status::OK();
        }
        // operands the tensor-core kernel cannot take: materialise the product, then the plain argmax
        TensorRec prod;
        AG_RETURN_IF_ERROR(alloc_out(cmeta.shape, cmeta.dtype, &prod, nullptr));
        g.c = prod.data();
        AG_LAUNCH(k::matmul(s, g));
        TView pv = prod.view();
        AG_LAUNCH(k::argmax(s, pv, ov));
        return Status::OK();
      } else {
        AG_RETURN_IF_ERROR(build_gemm(*in[0], *in[1], *out, &g, &keep));
      }
      if (kd.op == Op::FusedLinear) {
        g.ep.alpha = kd.f0;
        g.ep.act = kd.act;
        TensorRec tmp;
        if (kd.has_bias) { AG_RETURN_IF_ERROR(make_contiguous(*in[idx++], &tmp)); keep.push_back(tmp); g.ep.bias = keep.back().data(); }
        if (kd.has_residual) {
          AG_RETURN_IF_ERROR(make_contiguous(*in[idx++], &tmp)); keep.push_back(tmp);
          if (keep.back().shape != out->shape) return Status::compute("fused residual shape mismatch");
          g.ep.residual = keep.back().data();
        }
        if (kd.has_ln) {
          if (!in[idx]->contiguous() || !in[idx + 1]->contiguous()) return Status::compute("linear_fused: column sums and row statistics must be contiguous");
          g.ep.ln_colsum = static_cast<const float*>(in[idx]->data()); g.ep.ln_stats = static_cast<const long long*>(in[idx + 1]->data());
          g.ep.ln_eps = kd.f1;
          idx += 2;
        }
        if (kd.has_stats_out) { if (!in[idx]->contiguous()) return Status::compute("linear_fused: row statistics must be contiguous"); g.ep.stats_out = static_cast<long long*>(in[idx++]->data()); }
        if (kd.has_stats_zero) { if (!in[idx]->contiguous()) return Status::compute("linear_fused: row statistics must be contiguous"); g.ep.stats_zero = static_cast<long long*>(in[idx++]->data()); }
      }
      if (!int8_w && g.dtype == DType::F32 && g.b_dtype == DType::F32 && !dry) {
        bool done = false;
        AG_RETURN_IF_ERROR(matmul_f32_split(s, g, &done));
        if (done) return Status::OK();
      }
      if (linear_deferrable(node, in)) {
        // held back for chaining with the linears that follow; everything it touches stays alive until it is launched
        for (const TensorRec* t : in) keep.push_back(*t);
        keep.push_back(*out);
        return chain::submit(g, std::move(keep));
      }
      AG_LAUNCH(k::matmul(s, g));
      return Status::OK();
    }
    case Op::Softmax: case Op::SoftmaxCausal: {
      TensorRec c; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c));
      AG_LAUNCH(k::softmax(s, c.view(), kd.op == Op::SoftmaxCausal, ov));
      return Status::OK();
    }
    case Op::LayerNorm: {
      TensorRec c, g, b;
      AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c)); AG_RETURN_IF_ERROR(make_contiguous(*in[1], &g)); AG_RETURN_IF_ERROR(make_contiguous(*in[2], &b));
      AG_LAUNCH(k::layer_norm(s, c.view(), g.view(), b.view(), kd.f0, ov));
      return Status::OK();
    }
    case Op::Embedding: {
      TensorRec w, ix; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &w)); AG_RETURN_IF_ERROR(make_contiguous(*in[1], &ix));
      AG_LAUNCH(k::embedding(s, w.view(), ix.view(), ov));
      return Status::OK();
    }
    case Op::FusedEmbedAdd: {
      TensorRec w0, i0, w1, i1;
      AG_RETURN_IF_ERROR(make_contiguous(*in[0], &w0)); AG_RETURN_IF_ERROR(make_contiguous(*in[1], &i0));
      AG_RETURN_IF_ERROR(make_contiguous(*in[2], &w1)); AG_RETURN_IF_ERROR(make_contiguous(*in[3], &i1));
      AG_LAUNCH(k::embedding_add(s, w0.view(), i0.view(), w1.view(), i1.view(), ov));
      return Status::OK();
    }
    case Op::AddBias: {
      TensorRec c, b; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c)); AG_RETURN_IF_ERROR(make_contiguous(*in[1], &b));
      AG_LAUNCH(k::add_bias(s, c.view(), b.view(), kd.act, ov));
      return Status::OK();
    }
    case Op::Argmax: {
      // rows may carry a pitch (a padded GEMM output, also seen through a reshape): the kernel takes a row stride
      const TensorRec& t = *in[0];
      bool rows_ok = !t.shape.empty() && t.strides.back() == 1 && t.shape.size() >= 2;
      if (rows_ok) {
        const int64_t pitch = t.strides[t.shape.size() - 2];
        int64_t expect = pitch;
        for (int d = (int)t.shape.size() - 2; d >= 0 && rows_ok; d--) {
          if (t.shape[d] != 1 && t.strides[d] != expect) rows_ok = false;
          expect *= t.shape[d];
        }
        rows_ok = rows_ok && pitch >= t.shape.back();
      }
      if (rows_ok && !t.contiguous()) {
        TView v = t.view();
        AG_LAUNCH(k::argmax(s, v, ov));
        return Status::OK();
      }
      TensorRec c; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c));
      AG_LAUNCH(k::argmax(s, c.view(), ov));
      return Status::OK();
    }
    case Op::Sum: case Op::Mean: {
      TensorRec c; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c));
      AG_LAUNCH(k::sum_last(s, c.view(), ov, kd.op == Op::Mean));
      return Status::OK();
    }
    case Op::Concat: {
      // two strided copies into disjoint slices of the output, one launch
      int64_t dim = kd.i0;
      TensorRec lo = *out, hi = *out;
      lo.shape[dim] = in[0]->shape[dim];
      hi.shape[dim] = in[1]->shape[dim];
      hi.byte_offset += (size_t)(in[0]->shape[dim] * out->strides[dim]) * dtype_size(out->dtype);
      AG_LAUNCH(k::copy_strided_pair(s, in[0]->view(), lo.view(), in[1]->view(), hi.view()));
      return Status::OK();
    }
    case Op::Gather: case Op::IndexSelect: {
      TensorRec c, ix; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c)); AG_RETURN_IF_ERROR(make_contiguous(*in[1], &ix));
      if (kd.op == Op::Gather) AG_LAUNCH(k::gather2d(s, c.view(), (int)kd.i0, ix.view(), ov));
      else AG_LAUNCH(k::index_select2d(s, c.view(), (int)kd.i0, ix.view(), ov));
      return Status::OK();
    }
    case Op::ThresholdBackward: {
      TensorRec g, x; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &g)); AG_RETURN_IF_ERROR(make_contiguous(*in[1], &x));
      AG_LAUNCH(k::threshold_backward(s, g.view(), x.view(), kd.f0, ov));
      return Status::OK();
    }
    case Op::Cast: {
      TensorRec c; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c));
      AG_LAUNCH(k::cast(s, c.view(), ov));
      return Status::OK();
    }
    case Op::Quantize: {
      TensorRec c; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c));
      AG_LAUNCH(k::quantize(s, c.view(), kd.f0, (int)kd.i0, ov));
      return Status::OK();
    }
    case Op::Dequantize: {
      TensorRec c; AG_RETURN_IF_ERROR(make_contiguous(*in[0], &c));
      AG_LAUNCH(k::dequantize(s, c.view(), kd.f0, (int)kd.i0, ov));
      return Status::OK();
    }
    default:
      return Status::compute(std::string(op_debug_name(kd.op)) + " is unsupported on this backend");
  }
}

}  // namespace ag
