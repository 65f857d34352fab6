// Fusion pass.
//
// Part 1 restates the reference rule (fusion.rs:60-142, :243-285): walk the execution order,
// start a chain at an element-wise node, extend it while the next node is element-wise, consumes
// the current one, and the current one has exactly one consumer; chains of length >= 2 become one
// FusedElementwise node that keeps the last node's id, with the leaf inputs in first-use order.
// Where upstream emits MSL text per chain (fusion.rs:167-238), this build emits a small
// accumulator program that one pre-compiled kernel interprets, so no run-time compilation.
//
// Part 2 adds graph-level rewrites upstream lists as future work: a linear layer's epilogue
// (matmul -> scalar_mul / add_bias -> gelu|relu -> + residual) collapses into the GEMM kernel,
// matmul(Q, K^T) -> scalar_mul -> softmax[_causal] -> matmul(., V) becomes one attention node,
// and embedding + embedding becomes one gather-add. Each rewrite fires only when every
// intermediate has exactly one consumer, the same safety rule as Part 1.
#include "runtime.h"
#include <algorithm>
#include <cmath>

namespace ag { namespace fusion {

static bool g_elementwise = true;
static bool g_patterns = true;
void set_enabled(bool elementwise, bool patterns) { g_elementwise = elementwise; g_patterns = patterns; }
void get_enabled(bool* elementwise, bool* patterns) { *elementwise = g_elementwise; *patterns = g_patterns; }

static int8_t prog_opcode(const OpKind& k, bool* is_binary) {
  *is_binary = false;
  switch (k.op) {
    case Op::Add: *is_binary = true; return (int8_t)k::BinOp::Add;
    case Op::Sub: *is_binary = true; return (int8_t)k::BinOp::Sub;
    case Op::Mul: *is_binary = true; return (int8_t)k::BinOp::Mul;
    case Op::Div: *is_binary = true; return (int8_t)k::BinOp::Div;
    case Op::Neg: return (int8_t)k::UnOp::Neg; case Op::Relu: return (int8_t)k::UnOp::Relu;
    case Op::Exp: return (int8_t)k::UnOp::Exp; case Op::Log: return (int8_t)k::UnOp::Log;
    case Op::Sqrt: return (int8_t)k::UnOp::Sqrt; case Op::Tanh: return (int8_t)k::UnOp::Tanh;
    case Op::Sin: return (int8_t)k::UnOp::Sin; case Op::Cos: return (int8_t)k::UnOp::Cos;
    case Op::Gelu: return (int8_t)k::UnOp::Gelu; case Op::Sigmoid: return (int8_t)k::UnOp::Sigmoid;
    case Op::Abs: return (int8_t)k::UnOp::Abs; case Op::Sign: return (int8_t)k::UnOp::Sign;
    default: return -1;
  }
}

static std::string unary_expr(Op op, const std::string& e) {
  switch (op) {
    case Op::Neg: return "(-" + e + ")"; case Op::Relu: return "max(" + e + ", 0.0f)";
    case Op::Exp: return "exp(" + e + ")"; case Op::Log: return "log(" + e + ")"; case Op::Sqrt: return "sqrt(" + e + ")";
    case Op::Tanh: return "tanh(" + e + ")"; case Op::Sin: return "sin(" + e + ")"; case Op::Cos: return "cos(" + e + ")";
    case Op::Gelu: return "gelu(" + e + ")"; case Op::Sigmoid: return "(1.0f / (1.0f + exp(-" + e + ")))";
    case Op::Abs: return "abs(" + e + ")"; case Op::Sign: return "sign(" + e + ")";
    default: return e;
  }
}
static std::string binary_expr(Op op, const std::string& l, const std::string& r) {
  const char* sym = op == Op::Add ? " + " : op == Op::Sub ? " - " : op == Op::Mul ? " * " : " / ";
  return "(" + l + sym + r + ")";
}

struct Chain { std::vector<uint64_t> ids; std::vector<uint64_t> leaves; };

static std::vector<Chain> find_chains(const Graph& g, const std::vector<uint64_t>& order) {
  std::vector<Chain> chains;
  std::unordered_set<uint64_t> consumed;
  // position of each id in the order, so "first successor in execution order" is cheap
  // only element-wise nodes can start or extend a chain: consumers are tracked for those alone
  std::unordered_set<uint64_t> elem;
  for (uint64_t id : order) {
    const OpNode* n = g.get_node(id);
    if (n && n->op.is_elementwise()) elem.insert(id);
  }
  if (elem.size() < 2) return chains;
  std::unordered_map<uint64_t, std::vector<uint64_t>> consumers;
  for (uint64_t id : order) {
    const OpNode* n = g.get_node(id);
    if (!n) continue;
    for (uint64_t in : n->inputs) {
      if (!elem.count(in)) continue;
      auto& v = consumers[in];
      if (v.empty() || v.back() != id) v.push_back(id);
    }
  }
  for (uint64_t id : order) {
    if (consumed.count(id) || !elem.count(id)) continue;
    const OpNode* n = g.get_node(id);
    if (!n || !n->op.is_elementwise()) continue;
    Chain c;
    c.ids.push_back(id);
    uint64_t cur = id;
    while (true) {
      if (g.ref_count(cur) != 1) break;
      auto it = consumers.find(cur);
      if (it == consumers.end() || it->second.empty()) break;
      uint64_t next = it->second.front();
      const OpNode* nn = g.get_node(next);
      if (!nn || !nn->op.is_elementwise() || consumed.count(next)) break;
      if (std::find(c.ids.begin(), c.ids.end(), next) != c.ids.end()) break;
      if ((int)c.ids.size() >= k::kFusedMaxInstrs) break;
      c.ids.push_back(next);
      cur = next;
    }
    if (c.ids.size() < 2) continue;
    for (uint64_t cid : c.ids) {
      const OpNode* cn = g.get_node(cid);
      for (uint64_t in : cn->inputs)
        if (std::find(c.ids.begin(), c.ids.end(), in) == c.ids.end() && std::find(c.leaves.begin(), c.leaves.end(), in) == c.leaves.end())
          c.leaves.push_back(in);
    }
    // The interpreter kernel binds at most kFusedMaxInputs leaves: trim the chain until it fits.
    while (c.leaves.size() > (size_t)k::kFusedMaxInputs && c.ids.size() > 2) {
      c.ids.pop_back();
      c.leaves.clear();
      for (uint64_t cid : c.ids) {
        const OpNode* cn = g.get_node(cid);
        for (uint64_t in : cn->inputs)
          if (std::find(c.ids.begin(), c.ids.end(), in) == c.ids.end() && std::find(c.leaves.begin(), c.leaves.end(), in) == c.leaves.end())
            c.leaves.push_back(in);
      }
    }
    if (c.leaves.size() > (size_t)k::kFusedMaxInputs) continue;
    for (uint64_t cid : c.ids) consumed.insert(cid);
    chains.push_back(std::move(c));
  }
  return chains;
}

static OpNode build_fused(const Graph& g, const Chain& c) {
  OpNode fused;
  const OpNode* last = g.get_node(c.ids.back());
  fused.id = last->id;
  fused.inputs = c.leaves;
  fused.out_shape = last->out_shape;
  fused.out_dtype = last->out_dtype;
  fused.op.op = Op::FusedElementwise;
  fused.op.function_name = "fused_" + std::to_string(next_fused_id());
  k::FusedProgram& p = fused.op.prog;
  p.n_inputs = (int)c.leaves.size();
  p.n_instrs = 0;
  std::unordered_map<uint64_t, std::string> expr;
  for (size_t i = 0; i < c.leaves.size(); i++) expr[c.leaves[i]] = "in" + std::to_string(i);
  uint64_t prev = 0;
  for (size_t pos = 0; pos < c.ids.size(); pos++) {
    const OpNode* n = g.get_node(c.ids[pos]);
    bool is_bin = false;
    int8_t code = prog_opcode(n->op, &is_bin);
    auto operand = [&](uint64_t in) -> int8_t {
      if (pos > 0 && in == prev) return -1;  // the running accumulator
      auto it = std::find(c.leaves.begin(), c.leaves.end(), in);
      return (int8_t)(it - c.leaves.begin());
    };
    k::FusedInstr ins;
    ins.op = code; ins.is_binary = is_bin ? 1 : 0;
    ins.a = operand(n->inputs[0]);
    ins.b = is_bin ? operand(n->inputs[1]) : 0;
    p.instrs[p.n_instrs++] = ins;
    expr[n->id] = is_bin ? binary_expr(n->op.op, expr[n->inputs[0]], expr[n->inputs[1]]) : unary_expr(n->op.op, expr[n->inputs[0]]);
    prev = n->id;
  }
  fused.op.expr = expr[last->id];
  return fused;
}

// ── graph-level rewrites ────────────────────────────────────────────────────
struct Rewriter {
  // Consumers of an id inside this evaluation: how many distinct nodes, and which one when it is the only one.
  struct Cons { uint64_t first = 0, last = 0; uint32_t n = 0; };
  Graph& g;
  const std::unordered_set<uint64_t>& keep;
  std::unordered_map<uint64_t, Cons> consumers;
  std::unordered_set<uint64_t> removed;
  const std::unordered_set<uint64_t>* released = nullptr;   // ids whose caller-side handle is gone (null: unknown)

  Rewriter(Graph& gr, const std::vector<uint64_t>& order, const std::unordered_set<uint64_t>& kp) : g(gr), keep(kp) {
    consumers.reserve(order.size() * 2);
    for (uint64_t id : order) {
      const OpNode* n = g.get_node(id);
      if (!n) continue;
      for (uint64_t in : n->inputs) {
        Cons& c = consumers[in];
        if (c.n == 0) { c.first = c.last = id; c.n = 1; }
        else if (c.last != id) { c.last = id; c.n++; }   // nodes arrive in order: one node's inputs are visited together
      }
    }
  }
  // The single consumer of `id` inside this evaluation, or null if it has several, none,
  // is referenced elsewhere in the graph, or must be kept materialised.
  const OpNode* sole_consumer(uint64_t id) {
    if (keep.count(id)) return nullptr;
    if (g.ref_count(id) != 1) return nullptr;
    auto it = consumers.find(id);
    if (it == consumers.end() || it->second.n != 1) return nullptr;
    if (removed.count(it->second.first)) return nullptr;
    return g.get_node(it->second.first);
  }
  void replace(const std::vector<uint64_t>& old_ids, OpNode fused) {
    // consumer bookkeeping for the fused node's inputs: the old nodes that read an input become one reader
    for (size_t i = 0; i < fused.inputs.size(); i++) {
      const uint64_t in = fused.inputs[i];
      if (std::find(fused.inputs.begin(), fused.inputs.begin() + i, in) != fused.inputs.begin() + i) continue;
      uint32_t readers = 0;
      for (uint64_t oid : old_ids) {
        const OpNode* on = g.get_node(oid);
        if (on && std::find(on->inputs.begin(), on->inputs.end(), in) != on->inputs.end()) readers++;
      }
      Cons& c = consumers[in];
      if (readers == 0) { if (c.n == 0) c.first = fused.id; c.last = fused.id; c.n++; continue; }
      c.n -= (readers - 1);
      if (c.n <= 1) { c.n = 1; c.first = fused.id; }
      c.last = fused.id;
    }
    for (uint64_t id : old_ids) { g.remove_node(id); if (id != fused.id) removed.insert(id); }
    g.add_node(std::move(fused));
  }
};

// reshape([M, N] -> [.., N]) of a linear layer's output followed by an activation or a residual add: apply
// the op to the 2-D tensor and reshape afterwards, so that the linear rewrite below sees
// matmul -> add_bias -> gelu -> add as one chain even when the program reshapes to [batch, tokens, features]
// between the ops (what torch's nn.Linear on a 3-D input records). The activation takes the reshape's id and
// the reshape takes the activation's, so ids that later nodes refer to keep their shapes; for an add the
// other operand gets a 2-D reshape (a view at run time) and the pair moves to the add's place in the order.
static void sink_row_reshapes(Graph& g, std::vector<uint64_t>& order, const std::unordered_set<uint64_t>& keep,
                              const std::unordered_set<uint64_t>* released, std::vector<uint64_t>* minted) {
  if (!released || !minted) return;   // the reshape's id changes meaning: only when its caller-side handle is known to be gone
  // candidates first (a reshape of a 2-D linear-layer node to 3 or more dims): most graphs have none
  auto candidate = [&](const OpNode* r) -> const OpNode* {
    if (!r || r->op.op != Op::Reshape || r->inputs.size() != 1 || r->out_shape.size() < 3) return nullptr;
    const OpNode* x = g.get_node(r->inputs[0]);
    if (!x || x->out_shape.size() != 2 || r->out_shape.back() != x->out_shape[1]) return nullptr;
    const Op xo = x->op.op;
    if (!(xo == Op::Matmul || xo == Op::MatmulInt8 || xo == Op::AddBias || xo == Op::ScalarMul || xo == Op::Gelu || xo == Op::GeluExact || xo == Op::Relu)) return nullptr;
    return x;
  };
  bool any = false;
  for (uint64_t id : order) if (candidate(g.get_node(id))) { any = true; break; }
  if (!any) return;
  std::unordered_map<uint64_t, std::vector<uint64_t>> consumers;
  consumers.reserve(order.size() * 2);
  for (uint64_t id : order) {
    const OpNode* n = g.get_node(id);
    if (!n) continue;
    for (uint64_t in : n->inputs) {
      auto& v = consumers[in];
      if (std::find(v.begin(), v.end(), id) == v.end()) v.push_back(id);
    }
  }
  std::unordered_map<uint64_t, std::vector<uint64_t>> before;   // ids to emit right before a node
  std::unordered_set<uint64_t> moved;
  for (size_t oi = 0; oi < order.size(); oi++) {
    const uint64_t rid = order[oi];
    const OpNode* r = g.get_node(rid);
    if (!r || r->op.op != Op::Reshape || r->inputs.size() != 1) continue;
    if (keep.count(rid) || g.ref_count(rid) != 1 || !released->count(rid)) continue;
    auto ci = consumers.find(rid);
    if (ci == consumers.end() || ci->second.size() != 1) continue;
    const OpNode* x = candidate(r);
    if (!x) continue;
    const OpNode* c = g.get_node(ci->second[0]);
    if (!c || c->out_shape != r->out_shape || c->out_dtype != r->out_dtype || keep.count(x->id)) continue;
    const uint64_t cid = c->id, xid = x->id;
    const Dims flat = x->out_shape;
    const Op co = c->op.op;
    if (co == Op::Gelu || co == Op::GeluExact || co == Op::Relu) {
      OpNode act = *c, rs = *r;
      g.remove_node(cid); g.remove_node(rid);
      act.id = rid; act.inputs = {xid}; act.out_shape = flat;
      rs.id = cid; rs.inputs = {rid};
      g.add_node(std::move(act)); g.add_node(std::move(rs));
    } else if (co == Op::Add && c->inputs.size() == 2 && c->inputs[0] != c->inputs[1]) {
      const bool first = c->inputs[0] == rid;
      const uint64_t other = first ? c->inputs[1] : c->inputs[0];
      const OpNode* on = g.get_node(other);
      if (!on || on->out_shape != r->out_shape || on->out_dtype != r->out_dtype) continue;   // pending and not broadcast
      OpNode add = *c, rs = *r, o2;
      o2.id = next_fused_id(); o2.op.op = Op::Reshape; o2.op.shape = flat; o2.inputs = {other}; o2.out_shape = flat; o2.out_dtype = on->out_dtype;
      g.remove_node(cid); g.remove_node(rid);
      add.id = rid; add.out_shape = flat;
      if (first) add.inputs = {xid, o2.id}; else add.inputs = {o2.id, xid};
      rs.id = cid; rs.inputs = {rid};
      const uint64_t o2id = o2.id;
      g.add_node(std::move(o2)); g.add_node(std::move(add)); g.add_node(std::move(rs));
      moved.insert(rid);
      minted->push_back(o2id);
      before[cid] = {o2id, rid};
      auto& oc = consumers[other];
      std::replace(oc.begin(), oc.end(), cid, o2id);
      consumers[o2id] = {rid};
    }
  }
  if (moved.empty()) return;
  std::vector<uint64_t> next;
  next.reserve(order.size() + before.size());
  for (uint64_t id : order) {
    if (moved.count(id)) continue;
    auto b = before.find(id);
    if (b != before.end()) for (uint64_t pre : b->second) next.push_back(pre);
    next.push_back(id);
  }
  order.swap(next);
}

static void rewrite_linear(Rewriter& rw, uint64_t id) {
  const OpNode* mm = rw.g.get_node(id);
  if (!mm || !(mm->op.op == Op::Matmul || mm->op.op == Op::MatmulInt8)) return;
  if (mm->out_dtype == DType::F64) return;
  std::vector<uint64_t> chain{id};
  OpNode fused;
  fused.op.op = Op::FusedLinear;
  fused.op.i1 = mm->op.op == Op::MatmulInt8 ? 1 : 0;   // inputs are then (x, int8 weights [N,K], scales [N])
  fused.op.f0 = 1.0f;
  fused.inputs = mm->inputs;
  fused.out_shape = mm->out_shape;
  fused.out_dtype = mm->out_dtype;
  uint64_t cur = id;
  uint64_t bias_in = 0, res_in = 0;
  int stage = 0;  // 0: after matmul, 1: after scale, 2: after bias, 3: after activation, 4: after residual
  while (stage < 4) {
    const OpNode* c = rw.sole_consumer(cur);
    if (!c) break;
    if (c->out_shape != fused.out_shape || c->out_dtype != fused.out_dtype) break;
    if (c->op.op == Op::ScalarMul && stage < 1) { fused.op.f0 = c->op.f0; stage = 1; }
    else if (c->op.op == Op::AddBias && stage < 2 && c->inputs[0] == cur && c->out_shape.size() == 2) { bias_in = c->inputs[1]; fused.op.has_bias = true; stage = 2; }
    else if ((c->op.op == Op::Gelu || c->op.op == Op::GeluExact || c->op.op == Op::Relu) && stage < 3) {
      fused.op.act = c->op.op == Op::Gelu ? k::Act::GeluTanh : c->op.op == Op::GeluExact ? k::Act::GeluErf : k::Act::Relu;
      stage = 3;
    } else if (c->op.op == Op::Add && stage < 4) {
      uint64_t other = c->inputs[0] == cur ? c->inputs[1] : c->inputs[0];
      if (other == cur) break;
      // the residual must already exist when the GEMM runs and must not broadcast
      const OpNode* on = rw.g.get_node(other);
      Dims os;
      if (on) os = on->out_shape; else os = fused.out_shape;  // materialised tensors are checked at run time
      if (on && os != fused.out_shape) break;
      res_in = other; fused.op.has_residual = true; stage = 4;
    } else break;
    chain.push_back(c->id);
    cur = c->id;
  }
  if (chain.size() < 2) return;
  if (fused.op.has_bias) fused.inputs.push_back(bias_in);
  if (fused.op.has_residual) fused.inputs.push_back(res_in);
  fused.id = cur;
  rw.replace(chain, std::move(fused));
}

static void rewrite_attention(Rewriter& rw, uint64_t id) {
  // id: the first matmul (Q x K^T)
  const OpNode* mm1 = rw.g.get_node(id);
  if (!mm1 || mm1->op.op != Op::Matmul) return;
  const OpNode* kt = rw.g.get_node(mm1->inputs[1]);
  if (!kt || kt->op.op != Op::Transpose) return;
  int64_t nd = (int64_t)kt->out_shape.size();
  if (!((kt->op.i0 == nd - 2 && kt->op.i1 == nd - 1) || (kt->op.i1 == nd - 2 && kt->op.i0 == nd - 1))) return;
  if (rw.keep.count(kt->id) || rw.g.ref_count(kt->id) != 1) return;
  const OpNode* sc = rw.sole_consumer(id);
  if (!sc || sc->op.op != Op::ScalarMul) return;
  const OpNode* sm = rw.sole_consumer(sc->id);
  if (!sm || !(sm->op.op == Op::Softmax || sm->op.op == Op::SoftmaxCausal)) return;
  const OpNode* mm2 = rw.sole_consumer(sm->id);
  if (!mm2 || mm2->op.op != Op::Matmul || mm2->inputs[0] != sm->id || mm2->inputs[1] == sm->id) return;
  int64_t dk = mm1->out_shape.empty() ? 0 : 0;
  (void)dk;
  OpNode fused;
  fused.id = mm2->id;
  fused.op.op = Op::FusedAttention;
  fused.op.causal = sm->op.op == Op::SoftmaxCausal;
  fused.op.f0 = sc->op.f0;
  fused.inputs = {mm1->inputs[0], kt->inputs[0], mm2->inputs[1]};
  fused.out_shape = mm2->out_shape;
  fused.out_dtype = mm2->out_dtype;
  // The attention executor derives the scale from d_k; only fuse when the recorded scale is that value.
  // (d_k is the last dim of K, i.e. the second-to-last dim of K^T.)
  int64_t d_k = kt->out_shape[nd - 2];
  float expect = 1.0f / std::sqrt((float)d_k);
  if (std::fabs(sc->op.f0 - expect) > 1e-6f * expect) return;
  // batch dims must match exactly (no broadcasting inside the fused form)
  rw.replace({kt->id, mm1->id, sc->id, sm->id, mm2->id}, std::move(fused));
}

// attention([B,h,T,d]) -> transpose_dims(1,2) -> reshape([B*T, h*d] or [B, T, h*d]): the head merge every
// transformer block does. The attention node takes over the reshape's id and shape and writes its
// output in [B, T, h, d] order directly (upstream: two materialising copies, lazy.rs:1891-1917, :2246-2262).
static void rewrite_attention_merge(Rewriter& rw, uint64_t id) {
  const OpNode* at = rw.g.get_node(id);
  if (!at || at->op.op != Op::FusedAttention || at->op.i0 != 0 || at->out_shape.size() != 4) return;
  const OpNode* tr = rw.sole_consumer(id);
  if (!tr || tr->op.op != Op::Transpose) return;
  if (!((tr->op.i0 == 1 && tr->op.i1 == 2) || (tr->op.i0 == 2 && tr->op.i1 == 1))) return;
  const OpNode* rs = rw.sole_consumer(tr->id);
  if (!rs || rs->op.op != Op::Reshape) return;
  const Dims& l = at->out_shape;  // [B, h, T, dv]
  const Dims& r = rs->out_shape;
  bool ok = (r.size() == 2 && r[0] == l[0] * l[2] && r[1] == l[1] * l[3]) ||
            (r.size() == 3 && r[0] == l[0] && r[1] == l[2] && r[2] == l[1] * l[3]);
  if (!ok) return;
  OpNode fused = *at;
  fused.id = rs->id;
  fused.op.i0 = 1;
  fused.op.shape = l;
  fused.out_shape = r;
  rw.replace({at->id, tr->id, rs->id}, std::move(fused));
}

// add_bias -> gelu | gelu_exact | relu outside a linear layer: one pass over the tensor instead of two.
static void rewrite_bias_act(Rewriter& rw, uint64_t id) {
  const OpNode* ab = rw.g.get_node(id);
  if (!ab || ab->op.op != Op::AddBias || ab->op.act != k::Act::None) return;
  const OpNode* c = rw.sole_consumer(id);
  if (!c || !(c->op.op == Op::Gelu || c->op.op == Op::GeluExact || c->op.op == Op::Relu)) return;
  if (c->out_shape != ab->out_shape || c->out_dtype != ab->out_dtype) return;
  OpNode fused = *ab;
  fused.id = c->id;
  fused.op.act = c->op.op == Op::Gelu ? k::Act::GeluTanh : c->op.op == Op::GeluExact ? k::Act::GeluErf : k::Act::Relu;
  rw.replace({ab->id, c->id}, std::move(fused));
}

// matmul -> [reshape that keeps the last dim]* -> argmax, each with one consumer: the product is never
// needed as a tensor, so the GEMM's epilogue takes the row maximum itself (a greedy-decoding LM head
// then neither writes nor re-reads the [rows, vocab] logits). Half-precision 2-D products only: that is
// what the tensor-core kernel computes; the executor falls back to matmul + argmax if operands turn
// out not to be eligible for it.
static void rewrite_matmul_argmax(Rewriter& rw, uint64_t id) {
  const OpNode* mm = rw.g.get_node(id);
  if (!mm || mm->op.op != Op::Matmul) return;
  if (!(mm->out_dtype == DType::BF16 || mm->out_dtype == DType::F16) || mm->out_shape.size() != 2) return;
  // Unlike the other rewrites this one removes a tensor a caller is likely to come back to (the logits),
  // so it only fires once the caller has dropped its handles to the product and its reshapes.
  auto dropped = [&](uint64_t nid) { return rw.released && rw.released->count(nid) != 0; };
  if (!dropped(id)) return;
  std::vector<uint64_t> chain{id};
  const OpNode* c = rw.sole_consumer(id);
  while (c && c->op.op == Op::Reshape && !c->out_shape.empty() && c->out_shape.back() == mm->out_shape.back()) {
    if (!dropped(c->id)) return;
    chain.push_back(c->id);
    c = rw.sole_consumer(c->id);
  }
  if (!c || c->op.op != Op::Argmax) return;
  chain.push_back(c->id);
  OpNode fused;
  fused.id = c->id;
  fused.op.op = Op::FusedLinear;
  fused.op.f0 = 1.0f;
  fused.op.i2 = 1;                       // row argmax instead of a stored product
  fused.inputs = mm->inputs;
  fused.out_shape = c->out_shape;
  fused.out_dtype = c->out_dtype;
  rw.replace(chain, std::move(fused));
}

static void rewrite_embed_add(Rewriter& rw, uint64_t id) {
  const OpNode* add = rw.g.get_node(id);
  if (!add || add->op.op != Op::Add || add->inputs.size() != 2 || add->inputs[0] == add->inputs[1]) return;
  const OpNode* e0 = rw.g.get_node(add->inputs[0]);
  const OpNode* e1 = rw.g.get_node(add->inputs[1]);
  if (!e0 || !e1 || e0->op.op != Op::Embedding || e1->op.op != Op::Embedding) return;
  if (e0->out_shape != e1->out_shape || e0->out_dtype != e1->out_dtype) return;
  if (rw.keep.count(e0->id) || rw.keep.count(e1->id) || rw.g.ref_count(e0->id) != 1 || rw.g.ref_count(e1->id) != 1) return;
  size_t esz = dtype_size(e0->out_dtype);
  if ((e0->out_shape.back() * (int64_t)esz) % 16 != 0) return;
  OpNode fused;
  fused.id = add->id;
  fused.op.op = Op::FusedEmbedAdd;
  fused.inputs = {e0->inputs[0], e0->inputs[1], e1->inputs[0], e1->inputs[1]};
  fused.out_shape = add->out_shape;
  fused.out_dtype = add->out_dtype;
  rw.replace({e0->id, e1->id, add->id}, std::move(fused));
}

std::vector<uint64_t> optimize(Graph& g, const std::vector<uint64_t>& order, const std::unordered_set<uint64_t>& keep,
                               const std::unordered_set<uint64_t>* released, std::vector<uint64_t>* minted) {
  std::vector<uint64_t> cur = order;
  if (g_patterns) {
    sink_row_reshapes(g, cur, keep, released, minted);
    Rewriter rw(g, cur, keep);
    rw.released = released;
    for (uint64_t id : order) { if (!rw.removed.count(id)) rewrite_attention(rw, id); }
    for (uint64_t id : order) { if (!rw.removed.count(id)) rewrite_attention_merge(rw, id); }
    for (uint64_t id : order) { if (!rw.removed.count(id)) rewrite_linear(rw, id); }
    for (uint64_t id : order) { if (!rw.removed.count(id)) rewrite_embed_add(rw, id); }
    for (uint64_t id : order) { if (!rw.removed.count(id)) rewrite_bias_act(rw, id); }
    for (uint64_t id : order) { if (!rw.removed.count(id)) rewrite_matmul_argmax(rw, id); }
    std::vector<uint64_t> next;
    for (uint64_t id : cur) if (!rw.removed.count(id) && g.has_node(id)) next.push_back(id);
    cur.swap(next);
    // A fused node keeps the id of the last node it absorbed, and its extra inputs (bias, residual)
    // were recorded before that node, so the original order is still a valid topological order.
  }
  if (g_elementwise) {
    std::vector<Chain> chains = find_chains(g, cur);
    if (!chains.empty()) {
      std::unordered_set<uint64_t> gone;
      for (const Chain& c : chains) {
        // never swallow an intermediate the caller asked to keep
        bool blocked = false;
        for (size_t i = 0; i + 1 < c.ids.size(); i++) if (keep.count(c.ids[i])) blocked = true;
        if (blocked) continue;
        OpNode fused = build_fused(g, c);
        for (uint64_t id : c.ids) { g.remove_node(id); if (id != fused.id) gone.insert(id); }
        g.add_node(std::move(fused));
      }
      std::vector<uint64_t> next;
      for (uint64_t id : cur) if (!gone.count(id)) next.push_back(id);
      cur.swap(next);
    }
  }
  return cur;
}

}}  // namespace ag::fusion
