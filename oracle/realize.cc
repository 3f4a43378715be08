// TEST INFRASTRUCTURE, NOT PRODUCT CODE. Nothing under kurumi_b200/ may call into this file.
//
// CPU restatement of kurumi's view-fused f32 evaluator, the single-threaded CPU path the
// reference itself runs for an all-f32 graph. It is the timed CPU baseline.
//   gate + entry:   kurumi_core/src/realize/eval.rs:22-103  (all nodes F32 and lowered, else interpret)
//   scheduler:      kurumi_core/src/realize/sched.rs:32-159 (movement rewrites a view, elementwise
//                   ops grow one lazy expression, reduce / contraction / multi-consumer nodes
//                   materialise once)
//   tape executor:  kurumi_core/src/realize/tape/{compile,run}.rs (postfix tape over leaves with
//                   affine offsets, one loop per instruction over the innermost row)
//   views:          kurumi_core/src/lower/index/movement.rs:10-118
// Views are held here as shape + per-axis stride + base + pad guards; a reshape of a
// non-contiguous view lowers when the strides allow it and otherwise materialises, which is the
// same observable rule as the reference's symbolic simplifier for the views its ops produce.
// Like a compiled Plan (realize/plan.rs:21-53) constants are read in place, not copied per call.
#include <algorithm>
#include <cmath>
#include <limits>
#include <memory>
#include <unordered_map>
#include <unordered_set>

#include "interp.h"

namespace ko {
using namespace ku;

namespace {

using Buf = std::shared_ptr<const std::vector<float>>;

struct Guard { size_t axis; int64_t lo, hi; };
struct View {
  Shape shape;
  std::vector<int64_t> stride;
  int64_t base = 0;
  bool contiguous = true;
  std::vector<Guard> guards;
  static View source(const Shape& s) {
    View v; v.shape = s;
    auto st = row_major_strides(s);
    v.stride.assign(st.begin(), st.end());
    return v;
  }
};

struct Expr;
using ExprP = std::shared_ptr<const Expr>;
struct Expr {
  enum K { Load, Unary, Add, Mul, Max } k;
  OpKind un = OpKind::Neg;
  Buf buf; View view;
  ExprP a, b;
};

struct Realized {
  bool fused = false;
  Buf buf; View view;      // leaf
  Shape shape; ExprP expr; // fused
  const Shape& shp() const { return fused ? shape : view.shape; }
};

long* g_kernels = nullptr;
void bump() { if (g_kernels) ++*g_kernels; }

// read a leaf through its view into a fresh row-major buffer (lower/index/eval.rs `read`)
std::vector<float> read_view(const std::vector<float>& buf, const View& v) {
  const size_t n = numel(v.shape);
  std::vector<float> out(n);
  std::vector<size_t> c(v.shape.size(), 0);
  for (size_t i = 0; i < n; ++i) {
    int64_t off = v.base;
    for (size_t d = 0; d < c.size(); ++d) off += static_cast<int64_t>(c[d]) * v.stride[d];
    bool ok = true;
    for (auto& g : v.guards) { int64_t x = static_cast<int64_t>(c[g.axis]); if (x < g.lo || x >= g.hi) { ok = false; break; } }
    out[i] = ok ? buf[static_cast<size_t>(off)] : 0.0f;
    for (size_t d = c.size(); d-- > 0;) { if (++c[d] < v.shape[d]) break; c[d] = 0; }
  }
  return out;
}

// ---- tape (realize/tape.rs:29-66, tape/compile.rs, tape/run.rs) ---------------------------------
struct Leaf { Buf buf; std::vector<int64_t> coeffs; int64_t base; std::vector<Guard> guards; };
struct Instr { enum K { Load, Unary, Binary } k; uint32_t leaf = 0; OpKind op = OpKind::Neg; };

void compile(const Expr& e, std::vector<Leaf>& leaves, std::vector<Instr>& tape) {
  switch (e.k) {
    case Expr::Load: tape.push_back({Instr::Load, static_cast<uint32_t>(leaves.size()), OpKind::Neg}); leaves.push_back({e.buf, e.view.stride, e.view.base, e.view.guards}); return;
    case Expr::Unary: compile(*e.a, leaves, tape); tape.push_back({Instr::Unary, 0, e.un}); return;
    default:
      compile(*e.a, leaves, tape);
      compile(*e.b, leaves, tape);
      tape.push_back({Instr::Binary, 0, e.k == Expr::Add ? OpKind::Add : e.k == Expr::Mul ? OpKind::Mul : OpKind::Max});
  }
}

void apply_unary(OpKind op, const float* s, float* d, size_t n) {
  switch (op) {
    case OpKind::Neg: for (size_t i = 0; i < n; ++i) d[i] = -s[i]; break;
    case OpKind::Recip: for (size_t i = 0; i < n; ++i) d[i] = 1.0f / s[i]; break;
    case OpKind::Sqrt: for (size_t i = 0; i < n; ++i) d[i] = std::sqrt(s[i]); break;
    case OpKind::Exp2: for (size_t i = 0; i < n; ++i) d[i] = std::exp2(s[i]); break;
    case OpKind::Log2: for (size_t i = 0; i < n; ++i) d[i] = std::log2(s[i]); break;
    case OpKind::Sin: for (size_t i = 0; i < n; ++i) d[i] = std::sin(s[i]); break;
    default: break;
  }
}
void apply_binary(OpKind op, const float* a, const float* b, float* d, size_t n) {
  switch (op) {
    case OpKind::Add: for (size_t i = 0; i < n; ++i) d[i] = a[i] + b[i]; break;
    case OpKind::Mul: for (size_t i = 0; i < n; ++i) d[i] = a[i] * b[i]; break;
    default: for (size_t i = 0; i < n; ++i) d[i] = std::fmax(a[i], b[i]); break;
  }
}

void load_row(float* row, const Leaf& l, int64_t base, size_t inner, size_t rank, const std::vector<size_t>& coord) {
  const int64_t ic = rank == 0 ? 0 : l.coeffs[rank - 1];
  const std::vector<float>& buf = *l.buf;
  if (l.guards.empty()) {
    if (ic == 1) std::copy(buf.begin() + base, buf.begin() + base + static_cast<int64_t>(inner), row);
    else if (ic == 0) std::fill(row, row + inner, buf[static_cast<size_t>(base)]);
    else for (size_t i = 0; i < inner; ++i) row[i] = buf[static_cast<size_t>(base + ic * static_cast<int64_t>(i))];
    return;
  }
  for (size_t i = 0; i < inner; ++i) {
    bool ok = true;
    for (auto& g : l.guards) {
      int64_t c = g.axis == rank - 1 ? static_cast<int64_t>(i) : static_cast<int64_t>(coord[g.axis]);
      if (c < g.lo || c >= g.hi) { ok = false; break; }
    }
    row[i] = ok ? buf[static_cast<size_t>(base + ic * static_cast<int64_t>(i))] : 0.0f;
  }
}

std::vector<float> eval_fused(const Expr& expr, const Shape& shape) {
  bump();
  std::vector<Leaf> leaves;
  std::vector<Instr> tape;
  compile(expr, leaves, tape);
  const size_t rank = shape.size(), total = numel(shape);
  std::vector<float> out(total);
  if (total == 0) return out;
  const size_t inner = rank == 0 ? 1 : shape[rank - 1], outer = total / inner;
  size_t depth = 0, sp0 = 0;
  for (auto& in : tape) { if (in.k == Instr::Load) depth = std::max(depth, ++sp0); else if (in.k == Instr::Binary) --sp0; }
  static thread_local std::vector<float> scratch;
  if (scratch.size() < depth * inner) scratch.resize(depth * inner);
  std::vector<const float*> src(std::max<size_t>(depth, 1), nullptr);
  std::vector<size_t> coord(rank ? rank - 1 : 0, 0);
  std::vector<int64_t> base;
  for (auto& l : leaves) base.push_back(l.base);
  const size_t last = tape.size() - 1;
  for (size_t row = 0; row < outer; ++row) {
    float* out_row = out.data() + row * inner;
    size_t sp = 0;
    for (size_t ii = 0; ii < tape.size(); ++ii) {
      const Instr& in = tape[ii];
      if (in.k == Instr::Load) {
        const Leaf& l = leaves[in.leaf];
        const int64_t ic = rank == 0 ? 0 : l.coeffs[rank - 1];
        if (l.guards.empty() && ic == 1) src[sp] = l.buf->data() + base[in.leaf];  // contiguous row: read in place
        else { float* r = scratch.data() + sp * inner; load_row(r, l, base[in.leaf], inner, rank, coord); src[sp] = r; }
        ++sp;
        if (ii == last) std::copy(src[sp - 1], src[sp - 1] + inner, out_row);
      } else if (in.k == Instr::Unary) {
        if (ii == last) apply_unary(in.op, src[sp - 1], out_row, inner);
        else { float* d = scratch.data() + (sp - 1) * inner; apply_unary(in.op, src[sp - 1], d, inner); src[sp - 1] = d; }
      } else {
        const float *a = src[sp - 2], *b = src[sp - 1];
        if (ii == last) apply_binary(in.op, a, b, out_row, inner);
        else { float* d = scratch.data() + (sp - 2) * inner; apply_binary(in.op, a, b, d, inner); src[sp - 2] = d; }
        --sp;
      }
    }
    for (size_t i = coord.size(); i-- > 0;) {  // advance the outer odometer, leaf bases incrementally
      if (coord[i] + 1 < shape[i]) { ++coord[i]; for (size_t li = 0; li < leaves.size(); ++li) base[li] += leaves[li].coeffs[i]; break; }
      const int64_t back = static_cast<int64_t>(shape[i]) - 1;
      for (size_t li = 0; li < leaves.size(); ++li) base[li] -= leaves[li].coeffs[i] * back;
      coord[i] = 0;
    }
  }
  return out;
}

// ---- realized helpers (realize/expr.rs:64-138) --------------------------------------------------
Realized leaf(Buf b, View v) { Realized r; r.buf = std::move(b); r.view = std::move(v); return r; }
ExprP as_expr(const Realized& r) {
  if (r.fused) return r.expr;
  auto e = std::make_shared<Expr>(); e->k = Expr::Load; e->buf = r.buf; e->view = r.view; return e;
}
Realized into_leaf(const Realized& r) {
  if (!r.fused) return r;
  return leaf(std::make_shared<const std::vector<float>>(eval_fused(*r.expr, r.shape)), View::source(r.shape));
}
std::vector<float> force_vec(const Realized& r) { return r.fused ? eval_fused(*r.expr, r.shape) : read_view(*r.buf, r.view); }
Buf force_contig(const Realized& r) {
  if (!r.fused && r.view.contiguous && r.view.guards.empty()) return r.buf;
  return std::make_shared<const std::vector<float>>(force_vec(r));
}

// ---- movement algebra ---------------------------------------------------------------------------
bool try_reshape(const View& v, const Shape& ns, View* out) {
  if (v.contiguous) { *out = View::source(ns); out->base = v.base; return true; }
  // stride-compatible regrouping of axes (sizes multiply out in matching contiguous chunks)
  std::vector<int64_t> nst(ns.size(), 0);
  size_t oi = 0, ni = 0;
  const size_t on = v.shape.size(), nn = ns.size();
  while (oi < on && ni < nn) {
    size_t op_ = v.shape[oi], np = ns[ni];
    size_t oj = oi + 1, nj = ni + 1;
    while (op_ != np) {
      if (op_ < np) { if (oj >= on) return false; op_ *= v.shape[oj++]; }
      else { if (nj >= nn) return false; np *= ns[nj++]; }
    }
    for (size_t k = oi; k + 1 < oj; ++k)
      if (v.shape[k + 1] != 1 && v.stride[k] != v.stride[k + 1] * static_cast<int64_t>(v.shape[k + 1])) return false;
    int64_t s = v.stride[oj - 1];
    for (size_t k = nj; k-- > ni;) { nst[k] = s; s *= static_cast<int64_t>(ns[k]); }
    oi = oj; ni = nj;
  }
  while (oi < on) if (v.shape[oi++] != 1) return false;
  while (ni < nn) { if (ns[ni] != 1) return false; nst[ni++] = 0; }
  out->shape = ns; out->stride = nst; out->base = v.base; out->contiguous = false; out->guards.clear();
  return true;
}

Realized movement(const Realized& src, const Op& op) {
  Realized l = into_leaf(src);
  if (!l.view.guards.empty()) {  // a padded source materialises before further movement
    bump();
    Shape s = l.view.shape;
    l = leaf(std::make_shared<const std::vector<float>>(read_view(*l.buf, l.view)), View::source(s));
  }
  const View& v = l.view;
  View o;
  switch (op.kind) {
    case OpKind::Permute:
      o.base = v.base; o.contiguous = v.contiguous;
      for (size_t i = 0; i < op.perm.size(); ++i) { o.shape.push_back(v.shape[op.perm[i]]); o.stride.push_back(v.stride[op.perm[i]]); if (op.perm[i] != i) o.contiguous = false; }
      break;
    case OpKind::Expand:
      o = v; o.shape = op.shape; o.contiguous = v.contiguous && op.shape == v.shape;
      for (size_t d = 0; d < v.shape.size(); ++d) if (v.shape[d] == 1 && op.shape[d] != 1) o.stride[d] = 0;
      break;
    case OpKind::Slice:
      o.base = v.base; o.contiguous = false;
      for (size_t d = 0; d < v.shape.size(); ++d) {
        auto& r = op.ranges[d];
        o.shape.push_back((r[1] - r[0] + r[2] - 1) / r[2]);
        o.stride.push_back(v.stride[d] * static_cast<int64_t>(r[2]));
        o.base += v.stride[d] * static_cast<int64_t>(r[0]);
      }
      break;
    case OpKind::Flip:
      o = v; o.contiguous = false;
      for (size_t ax : op.perm) { o.base += v.stride[ax] * (static_cast<int64_t>(v.shape[ax]) - 1); o.stride[ax] = -v.stride[ax]; }
      break;
    case OpKind::Pad:
      o.base = v.base; o.contiguous = false; o.stride = v.stride;
      for (size_t d = 0; d < v.shape.size(); ++d) {
        size_t lo = op.ranges[d][0], hi = op.ranges[d][1];
        o.shape.push_back(lo + v.shape[d] + hi);
        o.base -= v.stride[d] * static_cast<int64_t>(lo);
        if (lo || hi) o.guards.push_back({d, static_cast<int64_t>(lo), static_cast<int64_t>(lo + v.shape[d])});
      }
      break;
    case OpKind::Reshape:
      if (!try_reshape(v, op.shape, &o)) {  // non-contiguous reshape: materialise, then it lowers freely
        bump();
        Shape s = v.shape;
        l = leaf(std::make_shared<const std::vector<float>>(read_view(*l.buf, l.view)), View::source(s));
        o = View::source(op.shape);
      }
      break;
    default: throw Error("realize: not a movement op");
  }
  return leaf(l.buf, o);
}

bool op_fused(OpKind k) {
  switch (k) {
    case OpKind::Const: case OpKind::Cast: case OpKind::Add: case OpKind::Mul: case OpKind::Max: case OpKind::Neg:
    case OpKind::Recip: case OpKind::Sqrt: case OpKind::Exp2: case OpKind::Log2: case OpKind::Sin: case OpKind::Sum:
    case OpKind::ReduceMax: case OpKind::Reshape: case OpKind::Permute: case OpKind::Expand: case OpKind::Slice:
    case OpKind::Flip: case OpKind::Pad: case OpKind::DotGeneral:
      return true;
    default: return false;
  }
}

bool fused_supported(const Graph& g, NodeId id, bool allow_input) {
  for (NodeId n : reachable(g, {id})) {
    const Node& node = g.node(n);
    bool ok = op_fused(node.op.kind) || (allow_input && node.op.kind == OpKind::Input);
    if (node.dtype != DType::F32 || !ok) return false;
  }
  return true;
}

Buf buf_of(const Tensor& t) {
  return std::make_shared<const std::vector<float>>(t.data<float>(), t.data<float>() + t.len());
}

}  // namespace

bool plan_supported(const Graph& g, NodeId root) { return fused_supported(g, root, true); }

Tensor force(const Graph& g, NodeId root, const Feeds& feeds, long* kernels) {
  if (!fused_supported(g, root, !feeds.empty())) {
    if (kernels) *kernels = -1;
    return interpret_many(g, {root}, feeds, false)[0];
  }
  long count = 0;
  g_kernels = &count;
  std::unordered_map<NodeId, size_t> consumers;
  std::vector<NodeId> order = reachable(g, {root});
  for (NodeId id : order) for (NodeId s : g.node(id).src) ++consumers[s];
  // Constant / feed buffers: held once per call-site (static cache keyed by the tensor object) so
  // replay does not re-copy weights, as a compiled Plan does.
  static thread_local std::unordered_map<const Tensor*, std::pair<TensorPtr, Buf>> cache;
  auto cached = [&](const TensorPtr& t) -> Buf {
    auto it = cache.find(t.get());
    if (it != cache.end() && it->second.first == t) return it->second.second;
    if (cache.size() > 64) cache.clear();
    Buf b = buf_of(*t);
    cache[t.get()] = {t, b};
    return b;
  };
  std::unordered_map<NodeId, Realized> memo;
  for (NodeId id : order) {
    const Node& n = g.node(id);
    auto in = [&](size_t i) -> const Realized& { return memo.at(n.src[i]); };
    Realized r;
    switch (n.op.kind) {
      case OpKind::Const: r = leaf(cached(n.op.data), View::source(n.op.shape)); break;
      case OpKind::Input: {
        auto it = feeds.find(id);
        if (it == feeds.end()) throw Error("panic: realize: missing feed for an Input node");
        r = leaf(cached(it->second), View::source(it->second->shape));
        break;
      }
      case OpKind::Cast: r = in(0); break;  // all-f32 graph: identity
      case OpKind::Permute: case OpKind::Expand: case OpKind::Slice: case OpKind::Flip: case OpKind::Pad: case OpKind::Reshape:
        r = movement(in(0), n.op);
        break;
      case OpKind::Neg: case OpKind::Recip: case OpKind::Sqrt: case OpKind::Exp2: case OpKind::Log2: case OpKind::Sin: {
        auto e = std::make_shared<Expr>(); e->k = Expr::Unary; e->un = n.op.kind; e->a = as_expr(in(0));
        r.fused = true; r.shape = in(0).shp(); r.expr = e;
        break;
      }
      case OpKind::Add: case OpKind::Mul: case OpKind::Max: {
        auto e = std::make_shared<Expr>();
        e->k = n.op.kind == OpKind::Add ? Expr::Add : n.op.kind == OpKind::Mul ? Expr::Mul : Expr::Max;
        e->a = as_expr(in(0)); e->b = as_expr(in(1));
        r.fused = true; r.shape = in(0).shp(); r.expr = e;
        break;
      }
      case OpKind::Sum: case OpKind::ReduceMax: {  // boundary: materialise the producer, then the interpreter's fold
        Buf b = force_contig(in(0));
        auto vec = std::make_shared<std::vector<float>>(numel(n.shape));
        reduce_f32(n.op.kind, b->data(), in(0).shp(), n.op.axis, vec->data());
        bump();
        r = leaf(vec, View::source(n.shape));
        break;
      }
      case OpKind::DotGeneral: {
        std::vector<Val> vals;
        for (size_t i = 0; i < n.src.size(); ++i) {
          Buf b = force_contig(in(i));
          Val v; v.shape = in(i).shp(); v.dtype = DType::F32; v.bytes.resize(b->size() * 4);
          std::memcpy(v.bytes.data(), b->data(), b->size() * 4);
          vals.push_back(std::move(v));
        }
        std::vector<const Val*> ptrs;
        for (auto& v : vals) ptrs.push_back(&v);
        Val o = eval_op(n, ptrs, false);
        bump();
        auto vec = std::make_shared<std::vector<float>>(o.bytes.size() / 4);
        std::memcpy(vec->data(), o.bytes.data(), o.bytes.size());
        r = leaf(vec, View::source(o.shape));
        break;
      }
      default: throw Error("realize: op not lowered by the fused executor");
    }
    if (r.fused && consumers[id] > 1) r = into_leaf(r);  // multi-consumer fused node: materialise once
    memo.emplace(id, std::move(r));
  }
  const Realized& rr = memo.at(root);
  Tensor out;
  out.dtype = DType::F32;
  out.shape = rr.shp();
  std::vector<float> v = force_vec(rr);
  out.bytes.resize(v.size() * 4);
  if (!v.empty()) std::memcpy(out.bytes.data(), v.data(), v.size() * 4);
  g_kernels = nullptr;
  if (kernels) *kernels = count;
  return out;
}

}  // namespace ko
