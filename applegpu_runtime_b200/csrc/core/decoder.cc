// GPT-2 greedy decoder with a preallocated KV cache and a captured step.
//
// The reference's generate loop (python/applegpu_runtime/models/generate.py:83-127) calls gpt2_forward once per token
// (models/gpt2.py:47-180): every step re-records ~300 ops, grows the KV cache by concatenation (gpt2.py:122-127) and
// reads the whole logits matrix back to pick a token on the host. Here a decode step is a fixed list of kernel
// launches on fixed buffers: the cache is [B, heads, T_max, 64] per layer and is appended in place, the current
// length, the step counter and the picked tokens live in device memory, and the LM head takes the row maximum in its
// epilogue. Because nothing about the launch list depends on the length, the step is captured once as a CUDA graph
// and replayed; the host issues one graph launch per token and reads the tokens back once at the end.
// Arithmetic per layer is the op sequence of gpt2.py:94-169 (layer_norm, c_attn + bias, attention over the cache,
// c_proj + bias + residual, layer_norm, c_fc + bias + tanh-GELU, c_proj + bias + residual), then ln_f and the tied
// LM head; greedy choice = first index of the row maximum, as generate.py:46-48.
#include "runtime.h"
#include <atomic>
#include <cmath>
#include <cstdlib>

namespace ag {

struct Gpt2DecoderCfg { int n_layer, n_head, n_embd, vocab, n_positions, batch, max_len; };

class Gpt2Decoder {
 public:
  Gpt2DecoderCfg cfg{};
  DType dtype = DType::F32;
  // weights: wte, wpe, ln_f.weight, ln_f.bias, then per layer ln_1.{weight,bias}, c_attn.{weight,bias}, attn c_proj.{weight,bias},
  // ln_2.{weight,bias}, c_fc.{weight,bias}, mlp c_proj.{weight,bias}
  std::vector<TensorRec> w;
  std::shared_ptr<Buffer> kv, act, small, layer_table;
  int engine = 0;                     // 0: one kernel per op (default, faster); 1: the layers as one persistent cooperative kernel
  cudaGraphExec_t exec = nullptr;
  int launches_per_step = 0;
  int prompt_len = 0, steps_done = 0;
  bool primed = false;

  ~Gpt2Decoder() { if (exec) cudaGraphExecDestroy(exec); }

  size_t esz() const { return dtype_size(dtype); }
  int d() const { return cfg.n_embd; }
  size_t cache_layer_bytes() const { return (size_t)cfg.batch * cfg.n_head * cfg.max_len * 64 * esz(); }
  uint8_t* kcache(int l) const { return static_cast<uint8_t*>(kv->ptr) + (size_t)(2 * l) * cache_layer_bytes(); }
  uint8_t* vcache(int l) const { return static_cast<uint8_t*>(kv->ptr) + (size_t)(2 * l + 1) * cache_layer_bytes(); }
  // activations of one step: x, x2, xn [B, d]; att [B, d]; qkv [B, 3d]; ff [B, 4d]; logits [B, vocab] (float32 models)
  uint8_t* act_at(size_t elems_before) const { return static_cast<uint8_t*>(act->ptr) + ((elems_before * esz() + 255) / 256) * 256; }
  uint8_t* x() const { return act_at(0); }
  uint8_t* x2() const { return act_at((size_t)cfg.batch * d() * 1 + 128); }
  uint8_t* xn() const { return act_at((size_t)cfg.batch * d() * 2 + 256); }
  uint8_t* att() const { return act_at((size_t)cfg.batch * d() * 3 + 384); }
  uint8_t* qkv() const { return act_at((size_t)cfg.batch * d() * 4 + 512); }
  uint8_t* ff() const { return act_at((size_t)cfg.batch * d() * 7 + 640); }
  uint8_t* logits() const { return act_at((size_t)cfg.batch * d() * 11 + 768); }
  size_t act_bytes() const { return ((size_t)cfg.batch * d() * 11 + 1024) * esz() + (size_t)cfg.batch * cfg.vocab * 4 + 4096; }
  // small: counters {step, len} | grid barrier word (offset 128) | tok [B] | pos_ids [B] | keys u64 [B] | history [max_len, B]
  int* counters() const { return static_cast<int*>(small->ptr); }
  unsigned int* barrier_word() const { return reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(small->ptr) + 128); }
  int32_t* tok() const { return reinterpret_cast<int32_t*>(static_cast<uint8_t*>(small->ptr) + 256); }
  int32_t* pos_ids() const { return reinterpret_cast<int32_t*>(static_cast<uint8_t*>(small->ptr) + 256 + 4 * 1024); }
  unsigned long long* keys() const { return reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(small->ptr) + 256 + 8 * 1024); }
  int32_t* history() const { return reinterpret_cast<int32_t*>(static_cast<uint8_t*>(small->ptr) + 256 + 16 * 1024); }
  size_t small_bytes() const { return 256 + 16 * 1024 + (size_t)cfg.max_len * cfg.batch * 4; }

  // c = act(layer_norm?(a) @ w + bias) + residual with w [kdim, ndim] (Conv1D layout)
  // The split-K linears of a step leave QKV and FC1 unfinished (float partials in their own workspace regions): attention
  // and FC2 add the partials up themselves, which takes the fence + counter + reload by a last CTA off the tail of two of
  // a layer's five launches. APPLEGPU_DECODE_DEFER=0 finishes every linear in its own launch.
  static bool defer_enabled() {
    static const bool on = [] { const char* v = std::getenv("APPLEGPU_DECODE_DEFER"); return !(v && v[0] == '0'); }();
    return on;
  }
  k::GemmDesc linear_desc(const void* a, int kdim, const TensorRec& wgt, const TensorRec& bias, void* c, int ndim, k::Act act, const void* residual) const {
    k::GemmDesc g;
    g.dtype = dtype; g.b_dtype = dtype; g.a = a; g.b = wgt.data(); g.c = c;
    g.m = cfg.batch; g.n = ndim; g.k = kdim; g.batch = 1; g.batch_inner = 1;
    g.a_row = kdim; g.a_col = 1; g.a_batch = 0;
    g.b_row = ndim; g.b_col = 1; g.b_batch = 0;
    g.c_row = ndim; g.c_batch = 0;
    g.ep.bias = bias.data(); g.ep.act = act; g.ep.residual = residual;
    return g;
  }
  // A layer with QKV and FC1 left unfinished; false when a shape does not take the split-K kernel (the caller then runs
  // the layer launch by launch).
  bool layer_deferrable(const TensorRec* lw) const {
    const int D = d();
    if (!defer_enabled() || D / 128 > 8 || cfg.batch > 16) return false;
    k::GemmDesc q = linear_desc(x(), D, lw[2], lw[3], qkv(), 3 * D, k::Act::None, nullptr);
    q.ln_gamma = lw[0].data(); q.ln_beta = lw[1].data();
    k::GemmDesc f = linear_desc(x(), D, lw[8], lw[9], ff(), 4 * D, k::Act::None, nullptr);
    f.ln_gamma = lw[6].data(); f.ln_beta = lw[7].data();
    k::GemmDesc f2 = linear_desc(nullptr, 4 * D, lw[10], lw[11], x(), D, k::Act::None, x2());
    k::GemmDesc pr = linear_desc(att(), D, lw[4], lw[5], x2(), D, k::Act::None, x());
    return k::decode_linear_eligible(q) && k::decode_linear_eligible(f) && k::decode_linear_eligible(f2) && k::decode_linear_eligible(pr);
  }
  Status enqueue_layer_deferred(cudaStream_t s, int l, uint8_t* cur, uint8_t* other, float scale) {
    const TensorRec* lw = &w[4 + 12 * l];
    const int D = d(), slabs = (D + 127) / 128;
    k::DecodeLinearOpts o;
    // ln_1(x) @ W_qkv: partials only (region 1)
    k::GemmDesc g = linear_desc(cur, D, lw[2], lw[3], qkv(), 3 * D, k::Act::None, nullptr);
    g.ln_gamma = lw[0].data(); g.ln_beta = lw[1].data(); g.ln_eps = 1e-5f;
    o = k::DecodeLinearOpts(); o.region = 1; o.partial_only = true;
    AG_RETURN_IF_ERROR(k::decode_linear(s, g, o));
    // attention adds them (+ bias) into q | k | v itself
    AG_RETURN_IF_ERROR(k::attention_decode(s, dtype, nullptr, kcache(l), vcache(l), att(), counters() + 1, cfg.batch, cfg.n_head, cfg.max_len, scale,
                                           k::decode_partial_region(1), slabs, lw[3].data()));
    // x2 = x + att @ W_proj + b (finished in its own launch: the residual stream is read by every CTA of the next one)
    g = linear_desc(att(), D, lw[4], lw[5], other, D, k::Act::None, cur);
    AG_RETURN_IF_ERROR(k::decode_linear(s, g));
    // ln_2(x2) @ W_fc: partials only (region 2)
    g = linear_desc(other, D, lw[8], lw[9], ff(), 4 * D, k::Act::None, nullptr);
    g.ln_gamma = lw[6].data(); g.ln_beta = lw[7].data(); g.ln_eps = 1e-5f;
    o = k::DecodeLinearOpts(); o.region = 2; o.partial_only = true;
    AG_RETURN_IF_ERROR(k::decode_linear(s, g, o));
    // x = x2 + gelu(those partials + b_fc) @ W_fc2 + b
    g = linear_desc(nullptr, 4 * D, lw[10], lw[11], cur, D, k::Act::None, other);
    o = k::DecodeLinearOpts(); o.xp = k::decode_partial_region(2); o.xp_slabs = slabs; o.xp_bias = lw[9].data(); o.xp_act = k::Act::GeluTanh;
    AG_RETURN_IF_ERROR(k::decode_linear(s, g, o));
    launches_per_step += 5;
    return Status::OK();
  }

  Status linear(cudaStream_t s, const void* a, int kdim, const TensorRec& wgt, const TensorRec& bias, void* c, int ndim, k::Act act, const void* residual,
                const TensorRec* ln_g = nullptr, const TensorRec* ln_b = nullptr) {
    k::GemmDesc g;
    g.dtype = dtype; g.b_dtype = dtype; g.a = a; g.b = wgt.data(); g.c = c;
    g.m = cfg.batch; g.n = ndim; g.k = kdim; g.batch = 1; g.batch_inner = 1;
    g.a_row = kdim; g.a_col = 1; g.a_batch = 0;
    g.b_row = ndim; g.b_col = 1; g.b_batch = 0;
    g.c_row = ndim; g.c_batch = 0;
    g.ep.bias = bias.data(); g.ep.act = act; g.ep.residual = residual;
    static const bool fuse_ln = [] { const char* v = std::getenv("APPLEGPU_DECODE_FUSE_LN"); return !(v && v[0] == '0'); }();
    if (ln_g && fuse_ln) { g.ln_gamma = ln_g->data(); g.ln_beta = ln_b->data(); g.ln_eps = 1e-5f; }
    if (k::decode_linear_eligible(g) && (fuse_ln || !ln_g)) {
      launches_per_step++;
      return k::decode_linear(s, g);
    }
    g.ln_gamma = g.ln_beta = nullptr;
    // shapes the cluster kernel does not take: a separate layer_norm, then the general matmul dispatch
    if (ln_g) {
      AG_RETURN_IF_ERROR(k::layer_norm(s, v2(const_cast<void*>(a), cfg.batch, kdim), ln_g->view(), ln_b->view(), 1e-5f, v2(xn(), cfg.batch, kdim)));
      g.a = xn();
      launches_per_step++;
    }
    launches_per_step++;
    return k::matmul(s, g);
  }
  TView v2(void* p, int64_t rows, int64_t cols) const { return TView::make(p, dtype, {rows, cols}); }

  // One decode step: consumes tok / pos_ids, appends to the caches at *len, leaves the next token in tok.
  // The device table of per-layer weight and cache pointers the persistent kernel walks (built once).
  Status ensure_layer_table(cudaStream_t s) {
    if (layer_table) return Status::OK();
    const size_t bytes = k::decode_layers_table_bytes(cfg.n_layer);
    std::vector<uint8_t> host(bytes);
    for (int l = 0; l < cfg.n_layer; l++) {
      const void* w12[12];
      for (int i = 0; i < 12; i++) w12[i] = w[4 + 12 * (size_t)l + i].data();
      k::decode_layers_fill_entry(host.data(), l, w12, kcache(l), vcache(l));
    }
    AG_RETURN_IF_ERROR(Shared::get().pool.acquire(bytes, &layer_table));
    cudaError_t e = cudaMemcpyAsync(layer_table->ptr, host.data(), bytes, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);   // `host` goes out of scope
    if (e != cudaSuccess) { layer_table.reset(); return Status::compute(std::string("decoder: layer table: ") + cudaGetErrorString(e)); }
    return Status::OK();
  }

  Status enqueue_step(cudaStream_t s) {
    launches_per_step = 0;
    const int B = cfg.batch, D = d();
    uint8_t* cur = x();
    uint8_t* other = x2();
    if (engine == 1) {
      // embeddings and all layers: one cooperative launch (plus the memset that clears its barrier word)
      AG_RETURN_IF_ERROR(k::decode_layers(s, dtype, layer_table->ptr, cfg.n_layer, cfg.n_head, D, cfg.max_len, B, w[0].data(), w[1].data(), tok(), pos_ids(),
                                          counters() + 1, x(), x2(), att(), barrier_word(), k::matmul_status_word()));
      launches_per_step += 2;
      return enqueue_head(s, cur);
    }
    TView tokv = TView::make(tok(), DType::I32, {B}), posv = TView::make(pos_ids(), DType::I32, {B});
    AG_RETURN_IF_ERROR(k::embedding_add(s, w[0].view(), tokv, w[1].view(), posv, v2(x(), B, D)));
    launches_per_step++;
    const float scale = 1.0f / std::sqrt(64.0f);
    for (int l = 0; l < cfg.n_layer; l++) {
      const TensorRec* lw = &w[4 + 12 * l];
      if (layer_deferrable(lw)) { AG_RETURN_IF_ERROR(enqueue_layer_deferred(s, l, cur, other, scale)); continue; }
      // ln_1 and ln_2 run in the prologue of the projection that consumes them (the kernel stages its 8..16 rows whole)
      AG_RETURN_IF_ERROR(linear(s, cur, D, lw[2], lw[3], qkv(), 3 * D, k::Act::None, nullptr, &lw[0], &lw[1]));
      AG_RETURN_IF_ERROR(k::attention_decode(s, dtype, qkv(), kcache(l), vcache(l), att(), counters() + 1, B, cfg.n_head, cfg.max_len, scale));
      AG_RETURN_IF_ERROR(linear(s, att(), D, lw[4], lw[5], other, D, k::Act::None, cur));           // x + c_proj(attn)
      AG_RETURN_IF_ERROR(linear(s, other, D, lw[8], lw[9], ff(), 4 * D, k::Act::GeluTanh, nullptr, &lw[6], &lw[7]));
      AG_RETURN_IF_ERROR(linear(s, ff(), 4 * D, lw[10], lw[11], cur, D, k::Act::None, other));      // x + c_proj(gelu(c_fc))
      launches_per_step += 1;
    }
    return enqueue_head(s, cur);
  }

  // ln_f, the tied LM head with the greedy pick, and the step's bookkeeping.
  Status enqueue_head(cudaStream_t s, uint8_t* cur) {
    const int B = cfg.batch, D = d();
    AG_RETURN_IF_ERROR(k::layer_norm(s, v2(cur, B, D), w[2].view(), w[3].view(), 1e-5f, v2(xn(), B, D)));
    launches_per_step++;
    // tied LM head: wte [V, d] read as the K-major operand; greedy pick = first index of the row maximum
    k::GemmDesc g;
    g.dtype = dtype; g.b_dtype = dtype; g.a = xn(); g.b = w[0].data();
    g.m = B; g.n = cfg.vocab; g.k = D; g.batch = 1; g.batch_inner = 1;
    g.a_row = D; g.a_col = 1; g.a_batch = 0; g.b_row = 1; g.b_col = D; g.b_batch = 0; g.c_row = cfg.vocab; g.c_batch = 0;
    unsigned long long* finish_keys = nullptr;
    if (dtype != DType::F32 && std::string(k::matmul_path(g)) == "tcgen05") {
      // the keys are zero here: prefill clears them and every step's last kernel clears them again after reading them
      g.c = nullptr; g.ep.argmax_keys = keys();
      AG_RETURN_IF_ERROR(k::matmul(s, g));
      finish_keys = keys();        // no finalize launch: the step's last kernel turns the keys into tokens
      launches_per_step += 1;
    } else {
      g.c = logits();
      AG_RETURN_IF_ERROR(k::matmul(s, g));
      TView lg = TView::make(logits(), dtype, {(int64_t)B, (int64_t)cfg.vocab});
      AG_RETURN_IF_ERROR(k::argmax(s, lg, TView::make(tok(), DType::I32, {B})));
      launches_per_step += 2;
    }
    AG_RETURN_IF_ERROR(k::decode_finish(s, tok(), history(), pos_ids(), counters(), counters() + 1, B, cfg.max_len, finish_keys));
    launches_per_step++;
    return Status::OK();
  }
};

static std::mutex g_dec_mu;
static std::unordered_map<uint64_t, std::unique_ptr<Gpt2Decoder>> g_decoders;
static uint64_t g_dec_next = 1;

Status decoder_create(const std::vector<TensorRec>& weights, const Gpt2DecoderCfg& cfg, uint64_t* handle) {
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.dry) return Status::compute("no CUDA device (dry-run mode)");
  if (cfg.n_layer <= 0 || cfg.n_head <= 0 || cfg.batch <= 0 || cfg.max_len <= 1) return Status::invalid("decoder: bad configuration");
  if (cfg.n_embd != cfg.n_head * 64) return Status::unsupported("decoder: head dimension must be 64");
  if (cfg.batch > 16) return Status::unsupported("decoder: at most 16 sequences per step");
  if (cfg.batch > 1024 || cfg.max_len > cfg.n_positions || cfg.max_len > 8192) return Status::invalid("decoder: max_len exceeds the position table");
  if ((int)weights.size() != 4 + 12 * cfg.n_layer) return Status::invalid("decoder: expected 4 + 12 * n_layer weight tensors");
  auto dec = std::make_unique<Gpt2Decoder>();
  dec->cfg = cfg;
  dec->dtype = weights[0].dtype;
  if (!(dec->dtype == DType::F32 || dec->dtype == DType::F16 || dec->dtype == DType::BF16)) return Status::unsupported("decoder: float weights only");
  for (const TensorRec& t : weights) {
    if (!t.buf || !t.contiguous() || t.dtype != dec->dtype) return Status::invalid("decoder: weights must be materialised, contiguous and of one dtype");
  }
  const int D = cfg.n_embd;
  auto expect = [&](size_t i, Dims shape) { return weights[i].shape == shape; };
  if (!expect(0, {cfg.vocab, D}) || !expect(1, {cfg.n_positions, D}) || !expect(2, {D}) || !expect(3, {D})) return Status::invalid("decoder: embedding / ln_f shapes");
  for (int l = 0; l < cfg.n_layer; l++) {
    size_t o = 4 + 12 * (size_t)l;
    if (!expect(o, {D}) || !expect(o + 1, {D}) || !expect(o + 2, {D, 3 * D}) || !expect(o + 3, {3 * D}) || !expect(o + 4, {D, D}) || !expect(o + 5, {D}) ||
        !expect(o + 6, {D}) || !expect(o + 7, {D}) || !expect(o + 8, {D, 4 * D}) || !expect(o + 9, {4 * D}) || !expect(o + 10, {4 * D, D}) || !expect(o + 11, {D}))
      return Status::invalid("decoder: layer " + std::to_string(l) + " weight shapes");
  }
  dec->w = weights;
  BufferPool& pool = Shared::get().pool;
  AG_RETURN_IF_ERROR(pool.acquire(2 * (size_t)cfg.n_layer * dec->cache_layer_bytes(), &dec->kv));
  AG_RETURN_IF_ERROR(pool.acquire(dec->act_bytes(), &dec->act));
  AG_RETURN_IF_ERROR(pool.acquire(dec->small_bytes(), &dec->small));
  std::lock_guard<std::mutex> g(g_dec_mu);
  *handle = g_dec_next++;
  g_decoders[*handle] = std::move(dec);
  return Status::OK();
}

static Gpt2Decoder* find_decoder(uint64_t h) {
  auto it = g_decoders.find(h);
  return it == g_decoders.end() ? nullptr : it->second.get();
}

// kv: k0, v0, k1, v1, ... each [B, heads, prompt_len, 64] (any strides); first_tokens: int32 [B]
Status decoder_prefill(uint64_t handle, const std::vector<TensorRec>& kvs, const TensorRec& first_tokens, int prompt_len) {
  std::lock_guard<std::mutex> g(g_dec_mu);
  Gpt2Decoder* dec = find_decoder(handle);
  if (!dec) return Status::invalid("decoder: unknown handle");
  DeviceCtx& ctx = DeviceCtx::get();
  const Gpt2DecoderCfg& c = dec->cfg;
  if ((int)kvs.size() != 2 * c.n_layer) return Status::invalid("decoder: expected 2 * n_layer cache tensors");
  if (prompt_len < 1 || prompt_len >= c.max_len) return Status::invalid("decoder: prompt does not fit the cache");
  if (first_tokens.dtype != DType::I32 || numel_of(first_tokens.shape) != c.batch || !first_tokens.contiguous()) return Status::invalid("decoder: first tokens must be int32 [batch]");
  const Dims want = {c.batch, c.n_head, prompt_len, 64};
  for (int i = 0; i < 2 * c.n_layer; i++) {
    if (kvs[i].shape != want || kvs[i].dtype != dec->dtype) return Status::invalid("decoder: cache tensor " + std::to_string(i) + " has the wrong shape or dtype");
    TView dst;
    dst.ptr = (i & 1) ? dec->vcache(i / 2) : dec->kcache(i / 2);
    dst.dtype = dec->dtype; dst.shape = want;
    dst.strides = {(int64_t)c.n_head * c.max_len * 64, (int64_t)c.max_len * 64, 64, 1};
    AG_RETURN_IF_ERROR(k::copy_strided(ctx.stream, kvs[i].view(), dst));
  }
  cudaError_t e = cudaMemcpyAsync(dec->tok(), first_tokens.data(), (size_t)c.batch * 4, cudaMemcpyDeviceToDevice, ctx.stream);
  if (e != cudaSuccess) return Status::compute(std::string("decoder: ") + cudaGetErrorString(e));
  AG_RETURN_IF_ERROR(k::decode_reset(ctx.stream, dec->counters(), dec->pos_ids(), c.batch, prompt_len));
  {
    // the row-argmax keys of the LM head start at zero; from then on each step's last kernel clears them after reading them
    cudaError_t ce = cudaMemsetAsync(dec->keys(), 0, (size_t)c.batch * 8, ctx.stream);
    if (ce != cudaSuccess) return Status::compute(std::string("decoder: ") + cudaGetErrorString(ce));
  }
  dec->prompt_len = prompt_len; dec->steps_done = 0; dec->primed = true;
  return Status::OK();
}

// Runs n_steps decode steps and copies the n_steps x batch picked tokens to host_tokens (waits for the stream).
Status decoder_steps(uint64_t handle, int n_steps, int32_t* host_tokens, bool use_graph) {
  std::lock_guard<std::mutex> g(g_dec_mu);
  Gpt2Decoder* dec = find_decoder(handle);
  if (!dec) return Status::invalid("decoder: unknown handle");
  if (!dec->primed) return Status::invalid("decoder: prefill first");
  if (n_steps <= 0) return Status::OK();
  const Gpt2DecoderCfg& c = dec->cfg;
  if (dec->prompt_len + dec->steps_done + n_steps > c.max_len) return Status::invalid("decoder: the cache is full");
  DeviceCtx& ctx = DeviceCtx::get();
  AG_RETURN_IF_ERROR(ctx.make_current());
  extern std::atomic<uint64_t> g_launch_count;
  if (dec->engine == 1) AG_RETURN_IF_ERROR(dec->ensure_layer_table(ctx.stream));
  int first = 0;
  if (use_graph && !dec->exec) {
    // The very first step runs launch by launch (one-time kernel attributes are set outside any capture); then one
    // step is captured, programmatic dependent launches included (they become programmatic edges of the graph: the
    // linear kernels fetch their weights ahead of the dependency wait). APPLEGPU_DECODE_PDL=0 captures plain edges.
    // A failed capture leaves exec null and the remaining steps are issued launch by launch as well.
    AG_RETURN_IF_ERROR(dec->enqueue_step(ctx.stream));
    g_launch_count.fetch_add((uint64_t)dec->launches_per_step, std::memory_order_relaxed);
    first = 1;
    if (n_steps > 1) {
      static const bool pdl_in_graph = [] { const char* v = std::getenv("APPLEGPU_DECODE_PDL"); return !(v && v[0] == '0'); }();
      if (!pdl_in_graph) k::set_pdl_override(0);
      cudaGraph_t graph = nullptr;
      Status st = Status::OK();
      if (cudaStreamBeginCapture(ctx.stream, cudaStreamCaptureModeRelaxed) == cudaSuccess) {
        st = dec->enqueue_step(ctx.stream);
        cudaError_t ce = cudaStreamEndCapture(ctx.stream, &graph);
        if (st.ok() && ce == cudaSuccess && graph) {
          if (cudaGraphInstantiate(&dec->exec, graph, 0) != cudaSuccess) { dec->exec = nullptr; cudaGetLastError(); }
        } else cudaGetLastError();
        if (graph) cudaGraphDestroy(graph);
      } else cudaGetLastError();
      k::set_pdl_override(-1);
      if (!st.ok()) return st;
    }
  }
  for (int i = first; i < n_steps; i++) {
    if (use_graph && dec->exec) {
      cudaError_t e = cudaGraphLaunch(dec->exec, ctx.stream);
      if (e != cudaSuccess) return Status::compute(std::string("decoder: graph launch: ") + cudaGetErrorString(e));
      g_launch_count.fetch_add((uint64_t)dec->launches_per_step, std::memory_order_relaxed);
    } else {
      AG_RETURN_IF_ERROR(dec->enqueue_step(ctx.stream));
      g_launch_count.fetch_add((uint64_t)dec->launches_per_step, std::memory_order_relaxed);
    }
  }
  TensorRec hist;
  hist.buf = dec->small; hist.dtype = DType::I32; hist.shape = {(int64_t)n_steps, (int64_t)c.batch}; hist.strides = {(int64_t)c.batch, 1};
  hist.byte_offset = (size_t)(reinterpret_cast<uint8_t*>(dec->history()) - static_cast<uint8_t*>(dec->small->ptr)) + (size_t)dec->steps_done * c.batch * 4;
  hist.has_meta = true;
  dec->steps_done += n_steps;
  return download(hist, host_tokens, (size_t)n_steps * c.batch * 4, true);   // waits, and reports a timed-out tensor-core wait
}

// engine 0: one kernel per op; 1: the layers as one persistent cooperative kernel. A captured step of the other engine is dropped.
Status decoder_set_engine(uint64_t handle, int engine) {
  std::lock_guard<std::mutex> g(g_dec_mu);
  Gpt2Decoder* dec = find_decoder(handle);
  if (!dec) return Status::invalid("decoder: unknown handle");
  if (engine != 0 && engine != 1) return Status::invalid("decoder: engine must be 0 or 1");
  if (engine != dec->engine) {
    DeviceCtx& ctx = DeviceCtx::get();
    if (ctx.ready && !ctx.dry) cudaStreamSynchronize(ctx.stream);
    if (dec->exec) { cudaGraphExecDestroy(dec->exec); dec->exec = nullptr; }
    dec->engine = engine;
  }
  return Status::OK();
}

int decoder_launches_per_step(uint64_t handle) {
  std::lock_guard<std::mutex> g(g_dec_mu);
  Gpt2Decoder* dec = find_decoder(handle);
  return dec ? dec->launches_per_step : -1;
}
int decoder_uses_graph(uint64_t handle) {
  std::lock_guard<std::mutex> g(g_dec_mu);
  Gpt2Decoder* dec = find_decoder(handle);
  return dec ? (dec->exec ? 1 : 0) : -1;
}

void decoder_destroy(uint64_t handle) {
  std::lock_guard<std::mutex> g(g_dec_mu);
  auto it = g_decoders.find(handle);
  if (it == g_decoders.end()) return;
  DeviceCtx& ctx = DeviceCtx::get();
  if (ctx.ready && !ctx.dry) cudaStreamSynchronize(ctx.stream);   // a replayed graph may still be running on these buffers
  g_decoders.erase(it);
}

}  // namespace ag
