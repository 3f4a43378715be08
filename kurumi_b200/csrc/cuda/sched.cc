#include <cstring>
#include "sched.h"

#include <cstdio>

#include <algorithm>
#include <cmath>

#include "kernels.h"

namespace ku::cu {

namespace {
uint64_t elem_bits(DType dt, double v) {
  uint8_t tmp[16] = {0};
  f64_to_elem(dt, v, tmp);
  uint64_t b = 0;
  std::memcpy(&b, tmp, std::min<size_t>(8, dtype_width(dt)));
  return b;
}
View broadcast_view(const Shape& s) {
  View v;
  v.shape = s;
  v.stride.assign(s.size(), 0);
  return v;
}
bool has_guards(const Fused& f) {
  for (auto& l : f.leaves) if (!l.view.guards.empty()) return true;
  return false;
}
int find_acc(const Fused& f) {
  for (size_t i = 0; i < f.leaves.size(); ++i) if (f.leaves[i].kind == LeafKind::Acc) return static_cast<int>(i);
  return -1;
}
}  // namespace

Scheduler::Scheduler(const KernelLoader* load, const Graph& g, int sm_count, const std::vector<bool>* plan) : load_(load), g_(g), sm_(sm_count), plan_(plan) {}

int Scheduler::new_slot(Slot::Kind k, DType dt, const Shape& shape, NodeId node) {
  Slot s;
  s.kind = k; s.dtype = dt; s.shape = shape; s.node = node;
  s.bytes = numel(shape) * dtype_width(dt);
  prog_.slots.push_back(s);
  return static_cast<int>(prog_.slots.size()) - 1;
}

Fused Scheduler::buffer_value(int slot, DType dt, const Shape& shape) const {
  Leaf l;
  l.kind = LeafKind::Buffer; l.dtype = dt; l.slot = slot; l.view = View::source(shape);
  return fused_leaf(shape, l);
}

Fused Scheduler::imm_value(const Shape& shape, DType dt, uint64_t bits) const {
  Leaf l;
  l.kind = LeafKind::Imm; l.dtype = dt; l.imm = bits; l.view = broadcast_view(shape);
  return fused_leaf(shape, l);
}

size_t Scheduler::op_nodes(const Fused& f) const {
  size_t n = 0;
  for (auto& x : f.nodes) if (x.op != OpKind::Input) ++n;
  return n;
}

double Scheduler::leaf_bytes(const Fused& f) const {
  double total = 0;
  std::vector<int> seen;
  for (auto& l : f.leaves) {
    if (l.kind != LeafKind::Buffer || std::find(seen.begin(), seen.end(), l.slot) != seen.end()) continue;
    seen.push_back(l.slot);
    double touched = 1;
    for (size_t d = 0; d < l.view.shape.size(); ++d) if (l.view.stride[d] != 0) touched *= static_cast<double>(l.view.shape[d]);
    total += std::min(touched * static_cast<double>(dtype_width(l.dtype)), static_cast<double>(prog_.slots[static_cast<size_t>(l.slot)].bytes));
  }
  return total;
}

void Scheduler::push_launch(const Emitted& e, const Fused& f, int out_slot, double flops) {
  Launch L;
  L.name = e.family;
  L.kernel = (*load_)(e.source, e.entry, e.fmad);
  L.grid[0] = e.grid; L.block[0] = e.block; L.smem = e.smem; L.cluster[0] = e.cluster;
  for (int li : e.leaf_args) {
    Arg a;
    a.kind = Arg::SlotPtr;
    a.slot = f.leaves[static_cast<size_t>(li)].slot;
    L.args.push_back(a);
  }
  Arg o;
  o.kind = Arg::SlotPtr; o.slot = out_slot;
  L.args.push_back(o);
  L.algo_bytes = leaf_bytes(f) + static_cast<double>(prog_.slots[static_cast<size_t>(out_slot)].bytes);
  L.flops = flops;
  prog_.launches.push_back(std::move(L));
}

void Scheduler::note_acc_use(const Fused& f, bool fusable_here) {
  for (auto& l : f.leaves)
    if (l.kind == LeafKind::Acc) {
      PendingGemm& pg = gemms_[static_cast<size_t>(l.gemm)];
      ++pg.uses;
      if (!fusable_here) pg.fusable = false;
    }
}

std::vector<bool> Scheduler::fuse_plan() const {
  std::vector<bool> p;
  for (auto& g : gemms_) p.push_back(g.uses == 1 && g.fusable);
  return p;
}

// ---- contraction emission -------------------------------------------------------------------------
void Scheduler::emit_gemm(int id, const Fused* epi, int out_slot) {
  PendingGemm& pg = gemms_[static_cast<size_t>(id)];
  if (dry() || numel(pg.out_shape) == 0) return;
  const GemmDesc& d = pg.desc;
  Launch L;
  std::vector<int> epi_leaf_args;
  if (d.k == 0) {  // empty contraction: the accumulator is 0 everywhere
    Fused z = epi ? *epi : imm_value({static_cast<size_t>(d.batch), static_cast<size_t>(d.m), static_cast<size_t>(d.n)}, d.dtype, 0);
    if (epi) for (auto& l : z.leaves) if (l.kind == LeafKind::Acc) { l.kind = LeafKind::Imm; l.imm = 0; l.view = broadcast_view(z.shape); }
    push_launch(emit_pointwise(z, sm_), z, out_slot);
    return;
  }
  if (!build_gemm_tc(*load_, d, epi, sm_, &L, &epi_leaf_args)) {
    Emitted e = emit_gemm_simt(d, epi, sm_);
    L.name = e.family;
    L.kernel = (*load_)(e.source, e.entry, false);
    L.grid[0] = static_cast<unsigned>((d.n + 63) / 64); L.grid[1] = static_cast<unsigned>((d.m + 63) / 64); L.grid[2] = static_cast<unsigned>(d.batch);
    L.block[0] = 256;
    epi_leaf_args = e.leaf_args;
    Arg a; a.kind = Arg::SlotPtr; a.slot = pg.a_slot; L.args.push_back(a);
    Arg b; b.kind = Arg::SlotPtr; b.slot = pg.b_slot; L.args.push_back(b);
    Arg c; c.kind = Arg::SlotPtr; c.slot = out_slot; L.args.push_back(c);
  } else {
    for (auto& a : L.args) {  // the builder leaves operand slots symbolic: -1 = A, -2 = B, -3 = C
      int* s = a.kind == Arg::Tmap ? &a.tm.slot : &a.slot;
      if (*s == -1) *s = pg.a_slot; else if (*s == -2) *s = pg.b_slot; else if (*s == -3) *s = out_slot;
    }
  }
  for (int li : epi_leaf_args) {
    Arg a; a.kind = Arg::SlotPtr; a.slot = epi->leaves[static_cast<size_t>(li)].slot;
    L.args.push_back(a);
  }
  const double w = static_cast<double>(dtype_width(d.in_dtype));
  L.algo_bytes = static_cast<double>(d.batch) * (static_cast<double>(d.m * d.k) + static_cast<double>(d.k * d.n)) * w + (epi ? leaf_bytes(*epi) : 0.0) +
                 static_cast<double>(prog_.slots[static_cast<size_t>(out_slot)].bytes);
  L.flops = 2.0 * static_cast<double>(d.batch) * static_cast<double>(d.m) * static_cast<double>(d.n) * static_cast<double>(d.k);
  prog_.launches.push_back(std::move(L));
}

int Scheduler::force_gemm(int id) {
  PendingGemm& pg = gemms_[static_cast<size_t>(id)];
  if (pg.result_slot >= 0) return pg.result_slot;
  const int slot = new_slot(Slot::Temp, pg.desc.dtype, pg.out_shape);
  pg.result_slot = slot;
  emit_gemm(id, nullptr, slot);
  return slot;
}

Fused Scheduler::resolve_acc(const Fused& f) {
  if (find_acc(f) < 0) return f;
  if (dry()) note_acc_use(f, false);
  Fused r = f;
  for (auto& l : r.leaves)
    if (l.kind == LeafKind::Acc) {
      const int slot = force_gemm(l.gemm);
      l.kind = LeafKind::Buffer; l.slot = slot; l.gemm = -1;
    }
  return r;
}

Fused Scheduler::materialize(const Fused& f0, int out_slot) {
  const Fused* f = &f0;
  Fused tmp;
  const int acc = find_acc(f0);
  if (acc >= 0) {
    const Leaf& al = f0.leaves[static_cast<size_t>(acc)];
    PendingGemm& pg = gemms_[static_cast<size_t>(al.gemm)];
    size_t n_acc = 0;
    for (auto& l : f0.leaves) if (l.kind == LeafKind::Acc) ++n_acc;
    const bool identity = n_acc == 1 && f0.shape == pg.out_shape && al.view == View::source(pg.out_shape) && pg.result_slot < 0;
    if (dry()) {
      note_acc_use(f0, identity);
      const int slot = out_slot >= 0 ? out_slot : new_slot(Slot::Temp, f0.dtype(), f0.shape);
      return buffer_value(slot, f0.dtype(), f0.shape);
    }
    bool fused_done = false;
    if (identity && plan_ && (*plan_)[static_cast<size_t>(al.gemm)]) {
      // view every leaf as [batch, m, n]
      Fused epi = f0;
      const Shape s3 = {static_cast<size_t>(pg.desc.batch), static_cast<size_t>(pg.desc.m), static_cast<size_t>(pg.desc.n)};
      bool ok = !has_guards(epi);
      for (auto& l : epi.leaves) { View r; if (ok && l.view.reshape(s3, &r)) l.view = r; else ok = false; }
      if (ok) {
        epi.shape = s3;
        const int slot = out_slot >= 0 ? out_slot : new_slot(Slot::Temp, f0.dtype(), f0.shape);
        emit_gemm(al.gemm, &epi, slot);
        fused_done = true;
        return buffer_value(slot, f0.dtype(), f0.shape);
      }
    }
    if (!fused_done) { tmp = resolve_acc(f0); f = &tmp; }
  }
  if (out_slot < 0 && f->is_plain_buffer() && f->root_leaf().view.is_contiguous()) return *f;
  const int slot = out_slot >= 0 ? out_slot : new_slot(Slot::Temp, f->dtype(), f->shape);
  if (!dry() && numel(f->shape) > 0) push_launch(emit_pointwise(*f, sm_), *f, slot);
  return buffer_value(slot, f->dtype(), f->shape);
}

// ---- movement ---------------------------------------------------------------------------------------
Fused Scheduler::movement(const Node& n, Fused f) {
  const Op& op = n.op;
  // a padded value materialises before further movement; and zero-fill applies to the padded VALUE
  // (pad(f(x)) != f(pad(x)) in general), so an expression is written out before it is padded
  if (has_guards(f) || (op.kind == OpKind::Pad && op_nodes(f) > 0)) f = materialize(f);
  if (op.kind == OpKind::Reshape) {
    bool ok = true;
    for (auto& l : f.leaves) { View r; if (!l.view.reshape(op.shape, &r)) { ok = false; break; } }
    if (!ok) f = materialize(f);
  }
  for (auto& l : f.leaves) {
    switch (op.kind) {
      case OpKind::Permute: l.view = l.view.permute(op.perm); break;
      case OpKind::Expand: l.view = l.view.expand(op.shape); break;
      case OpKind::Slice: l.view = l.view.slice(op.ranges); break;
      case OpKind::Flip: l.view = l.view.flip(op.perm); break;
      case OpKind::Pad: l.view = l.view.pad(op.ranges); break;
      case OpKind::Reshape: { View r; if (!l.view.reshape(op.shape, &r)) throw Error::backend("internal: reshape of a contiguous view failed"); l.view = r; break; }
      default: throw Error::backend("internal: not a movement op");
    }
  }
  f.shape = n.shape;
  return f;
}

Fused Scheduler::combine(OpKind op, DType dt, const std::vector<const Fused*>& in) {
  Fused r;
  r.shape = in[0]->shape;
  FNode n;
  n.op = op; n.dtype = dt;
  for (size_t i = 0; i < in.size(); ++i) n.in[i] = import_expr(r, *in[i], in[i]->root);
  r.root = add_node(r, n);
  return r;
}

Fused Scheduler::elementwise(const Node& n, const std::vector<Fused>& in0) {
  std::vector<Fused> in = in0;
  auto ptr_leaves = [](const Fused& f) { size_t c = 0; for (auto& l : f.leaves) if (l.kind == LeafKind::Buffer) ++c; return c; };
  size_t total_nodes = 0, total_leaves = 0;
  for (auto& f : in) { total_nodes += f.nodes.size(); total_leaves += ptr_leaves(f); }
  if (total_nodes > 160 || total_leaves > 20)  // keep kernels and their argument lists bounded
    for (auto& f : in) if (op_nodes(f) > 0) f = materialize(f);
  std::vector<const Fused*> p;
  for (auto& f : in) p.push_back(&f);
  return combine(n.op.kind, n.dtype, p);
}

// ---- reductions / softmax ---------------------------------------------------------------------------
Fused Scheduler::reduce(OpKind k, const Fused& f0, size_t axis) {
  Fused f = resolve_acc(f0);
  Shape os = f.shape;
  os.erase(os.begin() + static_cast<long>(axis));
  const int slot = new_slot(Slot::Temp, f.dtype(), os);
  if (!dry() && numel(os) > 0) push_launch(emit_reduce(f, k, axis, sm_), f, slot);
  return buffer_value(slot, f.dtype(), os);
}

Fused Scheduler::softmax(OpKind k, const Fused& f0, size_t axis, float eps) {
  Fused f = resolve_acc(f0);
  const int slot = new_slot(Slot::Temp, f.dtype(), f.shape);
  if (!dry() && numel(f.shape) > 0) {
    Launch L;
    std::vector<int> leaf_args;
    size_t scratch = 0;
    if (k == OpKind::Softmax && build_softmax_groups(*load_, f, axis, sm_, &L, &leaf_args, &scratch)) {
      const int sslot = new_slot(Slot::Temp, DType::U8, {scratch});
      prog_.slots[static_cast<size_t>(sslot)].zero_init = true;
      for (int li : leaf_args) { Arg a; a.kind = Arg::SlotPtr; a.slot = f.leaves[static_cast<size_t>(li)].slot; L.args.push_back(a); }
      Arg o; o.kind = Arg::SlotPtr; o.slot = slot; L.args.push_back(o);
      Arg sc; sc.kind = Arg::SlotPtr; sc.slot = sslot; L.args.push_back(sc);
      Arg ep; ep.kind = Arg::Epoch; L.args.push_back(ep);
      Arg st; st.kind = Arg::Status; L.args.push_back(st);
      L.algo_bytes = leaf_bytes(f) + static_cast<double>(prog_.slots[static_cast<size_t>(slot)].bytes);
      prog_.launches.push_back(std::move(L));
    } else if (k == OpKind::Softmax && (L = Launch(), leaf_args.clear(), build_softmax_panels(*load_, f, axis, sm_, &L, &leaf_args, &scratch))) {
      const int sslot = new_slot(Slot::Temp, DType::U8, {scratch});
      for (int li : leaf_args) { Arg a; a.kind = Arg::SlotPtr; a.slot = f.leaves[static_cast<size_t>(li)].slot; L.args.push_back(a); }
      Arg o; o.kind = Arg::SlotPtr; o.slot = slot; L.args.push_back(o);
      Arg sc; sc.kind = Arg::SlotPtr; sc.slot = sslot; L.args.push_back(sc);
      Arg st; st.kind = Arg::Status; L.args.push_back(st);
      L.zero_slot = sslot;
      L.zero_bytes = 16384;
      L.algo_bytes = leaf_bytes(f) + static_cast<double>(prog_.slots[static_cast<size_t>(slot)].bytes);
      prog_.launches.push_back(std::move(L));
    } else if (k == OpKind::Softmax && (L = Launch(), leaf_args.clear(), build_softmax_two_pass(f, axis, &L, &scratch))) {
      const int sslot = new_slot(Slot::Temp, DType::U8, {scratch});
      for (auto& a : L.args) { if (a.slot == -3) a.slot = slot; else if (a.slot == -1) a.slot = sslot; }
      L.algo_bytes = leaf_bytes(f) + static_cast<double>(prog_.slots[static_cast<size_t>(slot)].bytes);
      prog_.launches.push_back(std::move(L));
    } else if (k == OpKind::Softmax && build_softmax_transposed(*load_, f, axis, sm_, &L, &leaf_args)) {
      for (int li : leaf_args) { Arg a; a.kind = Arg::SlotPtr; a.slot = f.leaves[static_cast<size_t>(li)].slot; L.args.push_back(a); }
      Arg o; o.kind = Arg::SlotPtr; o.slot = slot; L.args.push_back(o);
      if (L.status_arg) { Arg st; st.kind = Arg::Status; L.args.push_back(st); }
      L.algo_bytes = leaf_bytes(f) + static_cast<double>(prog_.slots[static_cast<size_t>(slot)].bytes);
      prog_.launches.push_back(std::move(L));
    } else {
      push_launch(emit_softmax(f, k, axis, eps, sm_), f, slot);
    }
  }
  return buffer_value(slot, f.dtype(), f.shape);
}

// ---- contraction ------------------------------------------------------------------------------------
namespace {
// root = Cast(to a wider float) of an fp8 value: the products of two such operands are exactly the
// products of the fp8 values, so the kernel may read the fp8 bytes directly
bool is_f8_cast(const Fused& f) {
  const FNode& r = f.nodes[static_cast<size_t>(f.root)];
  if (r.op != OpKind::Cast || !is_float(r.dtype) || dtype_width(r.dtype) < 2) return false;
  return f.nodes[static_cast<size_t>(r.in[0])].dtype == DType::F8E4M3;
}
// the fp8 value under such a cast, as its own expression
Fused f8_source(const Fused& f) {
  Fused r;
  r.shape = f.shape;
  r.root = import_expr(r, f, f.nodes[static_cast<size_t>(f.root)].in[0]);
  return r;
}
}  // namespace

Fused Scheduler::dot_general(DType dt, const Shape& out_shape, const Fused& a0, const Fused& b0, const std::vector<size_t>& lc,
                             const std::vector<size_t>& rc, const std::vector<size_t>& lb, const std::vector<size_t>& rb) {
  if (!is_numeric(dt)) throw Error::backend(std::string("dot_general on ") + dtype_name(dt) + " is not supported by the CUDA backend");
  const bool f8 = is_f8_cast(a0) && is_f8_cast(b0);
  auto lf = free_axes(a0.shape.size(), lb, lc), rf = free_axes(b0.shape.size(), rb, rc);
  int64_t B = 1, M = 1, N = 1, K = 1;
  for (size_t i : lb) B *= static_cast<int64_t>(a0.shape[i]);
  for (size_t i : lf) M *= static_cast<int64_t>(a0.shape[i]);
  for (size_t i : rf) N *= static_cast<int64_t>(b0.shape[i]);
  for (size_t i : lc) K *= static_cast<int64_t>(a0.shape[i]);
  struct Operand { int slot; View v; };
  auto canon = [&](const Fused& x0, const std::vector<size_t>& perm, const Shape& s3) -> Operand {
    int slot;
    View view;
    const DType in_dt = f8 ? DType::F8E4M3 : dt;
    {
      Fused x = resolve_acc(f8 ? f8_source(x0) : x0);
      if (!x.is_plain_buffer() || has_guards(x)) x = materialize(x);
      slot = x.root_leaf().slot; view = x.root_leaf().view;
    }
    View p = view.permute(perm), r;
    if (!p.reshape(s3, &r)) {
      Leaf l; l.kind = LeafKind::Buffer; l.dtype = in_dt; l.slot = slot; l.view = p;
      Fused t = materialize(fused_leaf(p.shape, l));
      slot = t.root_leaf().slot;
      View::source(p.shape).reshape(s3, &r);
    }
    return {slot, r};
  };
  std::vector<size_t> pa = lb, pb = rb;
  pa.insert(pa.end(), lf.begin(), lf.end()); pa.insert(pa.end(), lc.begin(), lc.end());
  pb.insert(pb.end(), rc.begin(), rc.end()); pb.insert(pb.end(), rf.begin(), rf.end());
  Operand A = canon(a0, pa, {static_cast<size_t>(B), static_cast<size_t>(M), static_cast<size_t>(K)});
  Operand Bv = canon(b0, pb, {static_cast<size_t>(B), static_cast<size_t>(K), static_cast<size_t>(N)});
  PendingGemm pg;
  pg.desc.dtype = dt; pg.desc.in_dtype = f8 ? DType::F8E4M3 : dt;
  pg.desc.batch = B; pg.desc.m = M; pg.desc.n = N; pg.desc.k = K;
  pg.desc.a_bs = A.v.stride[0]; pg.desc.a_ms = A.v.stride[1]; pg.desc.a_ks = A.v.stride[2]; pg.desc.a_base = A.v.base;
  pg.desc.b_bs = Bv.v.stride[0]; pg.desc.b_ks = Bv.v.stride[1]; pg.desc.b_ns = Bv.v.stride[2]; pg.desc.b_base = Bv.v.base;
  pg.a_slot = A.slot; pg.b_slot = Bv.slot; pg.out_shape = out_shape;
  gemms_.push_back(pg);
  Leaf l;
  l.kind = LeafKind::Acc; l.dtype = dt; l.gemm = static_cast<int>(gemms_.size()) - 1; l.view = View::source(out_shape);
  return fused_leaf(out_shape, l);
}

Fused Scheduler::dot(const Node& n, const Fused& a, const Fused& b) {
  return dot_general(n.dtype, n.shape, a, b, n.op.lc, n.op.rc, n.op.lb, n.op.rb);
}

// ---- attention --------------------------------------------------------------------------------------
// Op::Sdpa (kurumi_core/src/graph/op.rs:55-58); the math is the interpreter's decomposition,
// kurumi_core/src/interp/nn.rs:125-172. The tiled tensor-core kernel takes the shapes it
// supports; everything else runs the same decomposition on device through the generic kernels.
Fused Scheduler::attention(DType dt, const Shape& shape, bool causal, float scale, const Fused& q, const Fused& k, const Fused& v) {
  const size_t r = shape.size();
  const size_t S = shape[r - 2], dh = shape[r - 1];
  if (dry()) return buffer_value(new_slot(Slot::Temp, dt, shape), dt, shape);
  Launch L;
  if (!build_attention(*load_, dt, shape, causal, scale, sm_, &L)) throw Error::backend("internal: attention kernel rejected a supported shape");
  const int slot = new_slot(Slot::Temp, dt, shape);
  const int slots[4] = {q.root_leaf().slot, k.root_leaf().slot, v.root_leaf().slot, slot};
  for (auto& a : L.args) { int* s = a.kind == Arg::Tmap ? &a.tm.slot : &a.slot; if ((a.kind == Arg::Tmap || a.kind == Arg::SlotPtr) && *s < 0) *s = slots[-*s - 1]; }
  size_t bh = 1;
  for (size_t i = 0; i + 2 < r; ++i) bh *= shape[i];
  L.algo_bytes = 4.0 * static_cast<double>(numel(shape) * dtype_width(dt));
  L.flops = 4.0 * static_cast<double>(dh) * static_cast<double>(bh) * (causal ? static_cast<double>(S) * (S + 1) / 2.0 : static_cast<double>(S) * S);
  prog_.launches.push_back(std::move(L));
  return buffer_value(slot, dt, shape);
}

bool Scheduler::match_sdpa(NodeId id, SdpaMatch* m) const {
  auto uses = [&](NodeId x) { auto it = consumers_.find(x); return it == consumers_.end() ? size_t(0) : it->second; };
  const Node& n = g_.node(id);
  const size_t r = n.shape.size();
  if (n.op.kind != OpKind::DotGeneral || r < 2) return false;
  std::vector<size_t> batch;
  for (size_t i = 0; i + 2 < r; ++i) batch.push_back(i);
  if (n.op.lc != std::vector<size_t>{r - 1} || n.op.rc != std::vector<size_t>{r - 2} || n.op.lb != batch || n.op.rb != batch) return false;
  std::vector<NodeId> inner;
  const NodeId attn_id = n.src[0], v = n.src[1];
  const Node& attn = g_.node(attn_id);
  if (attn.op.kind != OpKind::Softmax || attn.op.axis != r - 1 || uses(attn_id) != 1) return false;
  inner.push_back(attn_id);
  NodeId sc_id = attn.src[0];
  bool causal = false;
  // a scalar constant expanded to a shape: Expand(Const of one element)
  auto scalar_of = [&](NodeId x, double* val) {
    const Node& e = g_.node(x);
    if (e.op.kind != OpKind::Expand || uses(x) != 1) return false;
    const Node& c = g_.node(e.src[0]);
    if (c.op.kind != OpKind::Const || numel(c.shape) != 1 || uses(e.src[0]) != 1) return false;
    *val = elem_to_f64(c.dtype, c.op.data->bytes.data());
    inner.push_back(x); inner.push_back(e.src[0]);
    return true;
  };
  // the causal bias: [Cast] <- Expand <- Reshape <- Const f32 [S, S] holding 0 on and below the diagonal, -inf above
  auto causal_bias_of = [&](NodeId x, size_t S) {
    std::vector<NodeId> chain;
    NodeId cur = x;
    if (g_.node(cur).op.kind == OpKind::Cast) { chain.push_back(cur); cur = g_.node(cur).src[0]; }
    if (g_.node(cur).op.kind != OpKind::Expand) return false;
    chain.push_back(cur); cur = g_.node(cur).src[0];
    if (g_.node(cur).op.kind != OpKind::Reshape) return false;
    chain.push_back(cur); cur = g_.node(cur).src[0];
    const Node& c = g_.node(cur);
    chain.push_back(cur);
    if (c.op.kind != OpKind::Const || c.dtype != DType::F32 || c.shape != Shape{S, S}) return false;
    for (NodeId y : chain) if (uses(y) != 1) return false;
    const float* d = c.op.data->data<float>();
    for (size_t i = 0; i < S; ++i)
      for (size_t j = 0; j < S; ++j) {
        const float want = j > i ? -std::numeric_limits<float>::infinity() : 0.0f;
        if (!(d[i * S + j] == want)) return false;
      }
    inner.insert(inner.end(), chain.begin(), chain.end());
    return true;
  };
  const size_t S = n.shape[r - 2];
  if (g_.node(sc_id).op.kind == OpKind::Add) {
    if (uses(sc_id) != 1) return false;
    const Node& add = g_.node(sc_id);
    NodeId scores = add.src[0], bias = add.src[1];
    if (g_.node(scores).op.kind != OpKind::Mul) std::swap(scores, bias);
    if (!causal_bias_of(bias, S)) return false;
    inner.push_back(sc_id);
    sc_id = scores;
    causal = true;
  }
  const Node& mul = g_.node(sc_id);
  if (mul.op.kind != OpKind::Mul || uses(sc_id) != 1) return false;
  inner.push_back(sc_id);
  NodeId raw_id = mul.src[0], inv = mul.src[1];
  if (g_.node(raw_id).op.kind != OpKind::DotGeneral) std::swap(raw_id, inv);
  double scale = 0;
  if (!scalar_of(inv, &scale) || !(scale > 0)) return false;
  const Node& raw = g_.node(raw_id);
  if (raw.op.kind != OpKind::DotGeneral || uses(raw_id) != 1) return false;
  if (raw.op.lc != std::vector<size_t>{r - 1} || raw.op.rc != std::vector<size_t>{r - 1} || raw.op.lb != batch || raw.op.rb != batch) return false;
  inner.push_back(raw_id);
  const NodeId q = raw.src[0], k = raw.src[1];
  if (g_.shape(q) != n.shape || g_.shape(k) != n.shape || g_.shape(v) != n.shape) return false;   // self-attention shapes only
  if (g_.dtype(q) != n.dtype || !attention_supported(n.dtype, n.shape)) return false;
  m->q = q; m->k = k; m->v = v; m->causal = causal; m->scale = static_cast<float>(scale); m->interior = std::move(inner);
  return true;
}

Fused Scheduler::sdpa(const Node& n, const Fused& q0, const Fused& k0, const Fused& v0) {
  const DType dt = n.dtype;
  const size_t r = n.shape.size();
  const size_t S = n.shape[r - 2], dh = n.shape[r - 1];
  const float scale = 1.0f / std::sqrt(static_cast<float>(dh));
  Fused q = materialize(resolve_acc(q0)), k = materialize(resolve_acc(k0)), v = materialize(resolve_acc(v0));
  if (attention_supported(dt, n.shape)) return attention(dt, n.shape, n.op.causal, scale, q, k, v);
  std::vector<size_t> batch;
  for (size_t i = 0; i + 2 < r; ++i) batch.push_back(i);
  Shape ss(n.shape.begin(), n.shape.end() - 2);
  ss.push_back(S); ss.push_back(S);
  Fused raw = dot_general(dt, ss, q, k, {r - 1}, {r - 1}, batch, batch);
  Fused x = raw;
  if (dt == DType::F64) {
    Fused sc = imm_value(ss, DType::F64, elem_bits(DType::F64, static_cast<double>(scale)));
    x = combine(OpKind::Mul, DType::F64, {&x, &sc});
  } else {
    if (dt != DType::F32) x = combine(OpKind::Cast, DType::F32, {&x});
    Fused sc = imm_value(ss, DType::F32, elem_bits(DType::F32, static_cast<double>(scale)));
    x = combine(OpKind::Mul, DType::F32, {&x, &sc});
    if (dt != DType::F32) x = combine(OpKind::Cast, dt, {&x});
  }
  if (n.op.causal) {
    auto iota = [&](size_t axis) {
      Leaf l;
      l.kind = LeafKind::Iota; l.dtype = DType::I32; l.view = View::source(ss);
      l.iota_len = static_cast<int64_t>(ss[axis]);
      l.iota_stride = 1;
      for (size_t i = axis + 1; i < ss.size(); ++i) l.iota_stride *= static_cast<int64_t>(ss[i]);
      return fused_leaf(ss, l);
    };
    Fused qi = iota(r - 2), kj = iota(r - 1);
    Fused mask = combine(OpKind::CmpLt, DType::BOOL, {&qi, &kj});  // key j > query i
    Fused ninf = imm_value(ss, dt, elem_bits(dt, -std::numeric_limits<double>::infinity()));
    x = combine(OpKind::Where, dt, {&mask, &ninf, &x});
  }
  Fused attn = softmax(OpKind::Softmax, x, r - 1, 0.f);
  return dot_general(dt, n.shape, attn, v, {r - 1}, {r - 2}, batch, batch);
}

// ---- weight-only quantised matmul ---------------------------------------------------------------------
// Lowered onto the primitives above (kurumi_core/src/interp/contract.rs:69-99 is the semantics): the packed
// weight becomes a fused pointwise expression W[n][c] = field(n, c) * scale(n, c / group) (+ min) over views of
// the operands - a byte is shared by 8 / bits columns (expand + reshape), its field index is an iota - and
// the contraction act x W^T runs on the regular paths: true f32 for an f32 activation; for a 16-bit
// activation the dequantised weight is rounded to that dtype and the tensor cores accumulate in f32.
Fused Scheduler::view_step(OpKind k, Fused f, const Shape& shape) {
  Node tmp;
  tmp.op.kind = k;
  tmp.op.shape = shape;
  tmp.shape = shape;
  return movement(tmp, std::move(f));
}

Fused Scheduler::quant_matmul(const Node& n, const std::vector<Fused>& in) {
  const Op& op = n.op;
  const size_t M = n.shape[0], N = n.shape[1], K = in[0].shape[1];
  const size_t per = 8 / op.bits, ng = K / op.group_size;
  const Shape nk{N, K};
  // a few activation rows: one kernel that streams the packed weight once
  if (quant_gemv_supported(n.dtype, static_cast<int64_t>(M), static_cast<int64_t>(N), static_cast<int64_t>(K), op.bits, static_cast<int64_t>(op.group_size))) {
    const int slot = new_slot(Slot::Temp, n.dtype, n.shape);
    auto plain = [](const Fused& f) {
      if (!f.is_plain_buffer()) return false;
      const View& v = f.root_leaf().view;
      if (!v.guards.empty() || v.base != 0) return false;
      const std::vector<size_t> rm = row_major_strides(v.shape);
      for (size_t d = 0; d < rm.size(); ++d) if (v.shape[d] > 1 && v.stride[d] != static_cast<int64_t>(rm[d])) return false;
      return true;
    };
    auto dense = [&](const Fused& f0) { Fused f = resolve_acc(f0); return plain(f) ? f : materialize(f); };   // a contiguous buffer of its own
    Fused qw = dense(in[1]), sc = dense(in[2]), act = dense(in[0]);
    Fused mn = op.symmetric ? sc : dense(in[3]);
    if (plain(qw) && plain(sc) && plain(mn) && plain(act)) {
      if (!dry()) {
        Launch L;
        if (!build_quant_gemv(*load_, n.dtype, static_cast<int64_t>(M), static_cast<int64_t>(N), static_cast<int64_t>(K), op.bits, static_cast<int64_t>(op.group_size), op.symmetric, sm_, &L))
          throw Error::backend("internal: quantised gemv kernel rejected a supported shape");
        const int slots[5] = {qw.root_leaf().slot, sc.root_leaf().slot, mn.root_leaf().slot, act.root_leaf().slot, slot};
        for (auto& a : L.args) if (a.kind == Arg::SlotPtr && a.slot < 0) a.slot = slots[-a.slot - 1];
        prog_.launches.push_back(std::move(L));
      }
      return buffer_value(slot, n.dtype, n.shape);
    }
  }
  // byte of column c: packed[n][c / per]
  Fused q = view_step(OpKind::Reshape, resolve_acc(in[1]), {N, K / per, 1});
  q = view_step(OpKind::Expand, q, {N, K / per, per});
  q = view_step(OpKind::Reshape, q, nk);
  Fused qi = combine(OpKind::Cast, DType::I32, {&q});
  // field index c % per (K is a multiple of per, so the flat index serves) times the field width
  Leaf il;
  il.kind = LeafKind::Iota; il.dtype = DType::I32; il.view = View::source(nk);
  il.iota_len = static_cast<int64_t>(per);
  il.iota_stride = 1;
  Fused field = fused_leaf(nk, il);
  Fused width = imm_value(nk, DType::I32, elem_bits(DType::I32, static_cast<double>(op.bits)));
  Fused shift = combine(OpKind::Mul, DType::I32, {&field, &width});
  Fused raw = combine(OpKind::Shr, DType::I32, {&qi, &shift});
  Fused mask = imm_value(nk, DType::I32, elem_bits(DType::I32, static_cast<double>((1u << op.bits) - 1)));
  raw = combine(OpKind::And, DType::I32, {&raw, &mask});
  if (op.symmetric) {   // sign-extend the field: (raw << (32 - bits)) >> (32 - bits), arithmetic
    Fused sh = imm_value(nk, DType::I32, elem_bits(DType::I32, static_cast<double>(32 - op.bits)));
    raw = combine(OpKind::Shl, DType::I32, {&raw, &sh});
    raw = combine(OpKind::Shr, DType::I32, {&raw, &sh});
  }
  Fused w = combine(OpKind::Cast, DType::F32, {&raw});
  auto per_group = [&](const Fused& g16) {   // [N, ng] f16 -> f32 value of every column's group
    Fused g = view_step(OpKind::Reshape, resolve_acc(g16), {N, ng, 1});
    g = view_step(OpKind::Expand, g, {N, ng, op.group_size});
    g = view_step(OpKind::Reshape, g, nk);
    return combine(OpKind::Cast, DType::F32, {&g});
  };
  Fused sc = per_group(in[2]);
  w = combine(OpKind::Mul, DType::F32, {&w, &sc});
  if (!op.symmetric) {
    Fused mn = per_group(in[3]);
    w = combine(OpKind::Add, DType::F32, {&w, &mn});
  }
  const DType dt = n.dtype;
  Fused act = resolve_acc(in[0]);
  if (dt == DType::F32 || dt == DType::F64) {
    if (dt == DType::F64) w = combine(OpKind::Cast, DType::F64, {&w});
    return dot_general(dt, {M, N}, act, w, {1}, {1}, {}, {});
  }
  if (dt == DType::BF16 || dt == DType::F16) {
    Fused wl = combine(OpKind::Cast, dt, {&w});
    return dot_general(dt, {M, N}, act, wl, {1}, {1}, {}, {});
  }
  // fp8 activations: contract in f32 and round once, as the interpreter does
  Fused a32 = combine(OpKind::Cast, DType::F32, {&act});
  Fused r = dot_general(DType::F32, {M, N}, a32, w, {1}, {1}, {}, {});
  return combine(OpKind::Cast, dt, {&r});
}

// ---- indexing and sorting -----------------------------------------------------------------------------
// Gather / GatherAlong / Scatter / ScatterAlong / Argsort (kurumi_core/src/interp/indexing/**, interp/sort.rs) run over
// contiguous operands; a scatter first writes the operand into the result buffer (fused with whatever produced it), then
// folds the updates in.
Fused Scheduler::dense(const Fused& f0) {
  Fused f = resolve_acc(f0);
  if (f.is_plain_buffer() && f.root_leaf().view.is_contiguous()) return f;
  return materialize(f);
}

Fused Scheduler::indexing(const Node& n, const std::vector<Fused>& in) {
  const Op& op = n.op;
  const Shape& os = g_.shape(n.src[0]);
  const DType dt = g_.dtype(n.src[0]);
  const size_t axis = op.axis;
  int64_t pre = 1, post = 1;
  for (size_t d = 0; d < axis; ++d) pre *= static_cast<int64_t>(os[d]);
  for (size_t d = axis + 1; d < os.size(); ++d) post *= static_cast<int64_t>(os[d]);
  const int64_t da = static_cast<int64_t>(os[axis]);
  auto launch = [&](const Emitted& e, std::initializer_list<int> slots) {
    Launch L;
    L.name = e.family;
    L.kernel = (*load_)(e.source, e.entry, false);
    L.grid[0] = e.grid; L.block[0] = e.block; L.smem = e.smem;
    for (int sl : slots) { Arg a; a.kind = Arg::SlotPtr; a.slot = sl; L.args.push_back(a); }
    for (int sl : slots) L.algo_bytes += static_cast<double>(prog_.slots[static_cast<size_t>(sl)].bytes);
    prog_.launches.push_back(std::move(L));
  };
  if (op.kind == OpKind::Argsort) {
    Fused x = dense(in[0]);
    const int slot = new_slot(Slot::Temp, DType::I64, n.shape);
    if (!dry() && numel(n.shape) > 0) {
      int64_t lpad = 1;
      while (lpad < da) lpad <<= 1;
      const int64_t key = (dt == DType::F64 || dtype_width(dt) == 8) ? 8 : 4;
      if (lpad * (key + 4) > 200 * 1024) {
        // longer than one CTA's shared memory: the same network over a padded copy in global scratch, chunk sorts and the
        // narrow steps in shared memory, the wide steps one launch each
        if (da >= (int64_t(1) << 30)) throw Error::backend("argsort along an axis of " + std::to_string(da) + " elements: positions are kept in 32 bits");
        int64_t lp = 0;
        size_t kb = 0;
        const Emitted e = emit_argsort_long(dt, op.descending, pre, da, post, &lp, &kb);
        const int64_t lines = pre * post, ch = 4096;
        const size_t ids_off = (static_cast<size_t>(lines * lp) * kb + 255) / 256 * 256;
        const int scratch = new_slot(Slot::Temp, DType::U8, {ids_off + static_cast<size_t>(lines * lp) * 4});
        auto step = [&](const char* entry, unsigned grid, unsigned block, std::initializer_list<Arg> args, double bytes) {
          Launch L;
          L.name = e.family;
          L.kernel = (*load_)(e.source, entry, false);
          L.grid[0] = grid; L.block[0] = block;
          for (const Arg& a : args) L.args.push_back(a);
          L.algo_bytes = bytes;
          prog_.launches.push_back(std::move(L));
        };
        auto ptr_arg = [](int sl, size_t off) { Arg a; a.kind = Arg::SlotPtr; a.slot = sl; a.byte_offset = static_cast<int64_t>(off); return a; };
        auto int_arg = [](int64_t v) { Arg a; a.kind = Arg::Bytes; a.bytes.resize(8); std::memcpy(a.bytes.data(), &v, 8); return a; };
        const unsigned chunk_ctas = static_cast<unsigned>(lines * (lp / ch));
        const unsigned wide = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((lines * (lp / 2) + 255) / 256, static_cast<int64_t>(sm_) * 16)));
        step("ku_asl_chunks", chunk_ctas, 1024, {ptr_arg(x.root_leaf().slot, 0), ptr_arg(scratch, 0), ptr_arg(scratch, ids_off)},
             static_cast<double>(prog_.slots[static_cast<size_t>(x.root_leaf().slot)].bytes));
        for (int64_t k = 2 * ch; k <= lp; k <<= 1) {
          for (int64_t j = k / 2; j >= ch; j >>= 1) step("ku_asl_global", wide, 256, {ptr_arg(scratch, 0), ptr_arg(scratch, ids_off), int_arg(k), int_arg(j)}, 0.0);
          step("ku_asl_local", chunk_ctas, 1024, {ptr_arg(scratch, 0), ptr_arg(scratch, ids_off), int_arg(k)}, 0.0);
        }
        step("ku_asl_out", static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((lines * da + 255) / 256, static_cast<int64_t>(sm_) * 16))), 256,
             {ptr_arg(scratch, ids_off), ptr_arg(slot, 0)}, static_cast<double>(prog_.slots[static_cast<size_t>(slot)].bytes));
      } else {
        launch(emit_argsort(dt, op.descending, pre, da, post, sm_), {x.root_leaf().slot, slot});
      }
    }
    return buffer_value(slot, DType::I64, n.shape);
  }
  const DType idt = g_.dtype(n.src[1]);
  const Shape& is = g_.shape(n.src[1]);
  if (op.kind == OpKind::Gather || op.kind == OpKind::GatherAlong) {
    Fused x = dense(in[0]), ix = dense(in[1]);
    const int slot = new_slot(Slot::Temp, dt, n.shape);
    if (!dry() && numel(n.shape) > 0) {
      if (da == 0) throw Error::backend("gather from an empty axis");
      if (op.kind == OpKind::Gather) launch(emit_gather(dt, idt, pre, da, post, static_cast<int64_t>(numel(is)), sm_), {x.root_leaf().slot, ix.root_leaf().slot, slot});
      else launch(emit_gather_along(dt, idt, pre, da, static_cast<int64_t>(is[axis]), post, sm_), {x.root_leaf().slot, ix.root_leaf().slot, slot});
    }
    return buffer_value(slot, dt, n.shape);
  }
  // scatters: the operand goes into the result buffer first
  Fused ix = dense(in[1]), up = dense(in[2]);
  const int slot = new_slot(Slot::Temp, dt, n.shape);
  materialize(resolve_acc(in[0]), slot);
  const bool along = op.kind == OpKind::ScatterAlong;
  const int64_t k = along ? static_cast<int64_t>(is[axis]) : static_cast<int64_t>(numel(is));
  if (!dry() && numel(n.shape) > 0 && numel(is) > 0)
    launch(emit_scatter(dt, idt, along, op.combine, pre, da, post, k, sm_), {ix.root_leaf().slot, up.root_leaf().slot, slot});
  return buffer_value(slot, dt, n.shape);
}

// ---- the walk ---------------------------------------------------------------------------------------
Fused Scheduler::value_of(NodeId id) { return memo_.at(id); }

Fused Scheduler::eval_node(NodeId id) {
  const Node& n = g_.node(id);
  if (is_complex(n.dtype)) throw Error::backend("complex dtypes are not supported by the CUDA backend");
  const Op& op = n.op;
  std::vector<Fused> in;
  for (NodeId s : n.src) in.push_back(memo_.at(s));
  switch (op.kind) {
    case OpKind::Const: {
      if (numel(n.shape) == 1) {
        uint64_t bits = 0;
        std::memcpy(&bits, op.data->bytes.data(), std::min<size_t>(8, dtype_width(n.dtype)));
        return imm_value(n.shape, n.dtype, bits);
      }
      return buffer_value(new_slot(Slot::Const, n.dtype, n.shape, id), n.dtype, n.shape);
    }
    case OpKind::Input: return buffer_value(new_slot(Slot::Feed, n.dtype, n.shape, id), n.dtype, n.shape);
    case OpKind::Iota: {
      Leaf l;
      l.kind = LeafKind::Iota; l.dtype = n.dtype; l.view = View::source(n.shape);
      l.iota_len = static_cast<int64_t>(n.shape[op.axis]);
      l.iota_stride = 1;
      for (size_t i = op.axis + 1; i < n.shape.size(); ++i) l.iota_stride *= static_cast<int64_t>(n.shape[i]);
      return fused_leaf(n.shape, l);
    }
    case OpKind::RandUniform: {
      Leaf l;
      l.kind = LeafKind::Rand; l.dtype = DType::F32; l.view = View::source(n.shape);
      const Node& sn = g_.node(n.src[0]);
      if (!is_int(sn.dtype)) throw Error::backend("rand_uniform seed must be an integer tensor");
      if (sn.op.kind == OpKind::Const && numel(sn.shape) >= 1) {
        l.imm = static_cast<uint64_t>(sat_cast<int64_t>(0));
        double v = elem_to_f64(sn.dtype, sn.op.data->bytes.data());
        (void)v;
        // read the first element exactly as an i64 (sign-extending signed types), then as u64
        int64_t s = 0;
        switch (sn.dtype) {
          case DType::U8: s = *sn.op.data->data<uint8_t>(); break;
          case DType::U16: s = *sn.op.data->data<uint16_t>(); break;
          case DType::U32: s = *sn.op.data->data<uint32_t>(); break;
          case DType::U64: s = static_cast<int64_t>(*sn.op.data->data<uint64_t>()); break;
          case DType::I8: s = *sn.op.data->data<int8_t>(); break;
          case DType::I16: s = *sn.op.data->data<int16_t>(); break;
          case DType::I32: s = *sn.op.data->data<int32_t>(); break;
          default: s = *sn.op.data->data<int64_t>(); break;
        }
        l.imm = static_cast<uint64_t>(s);
      } else {
        Fused seed = materialize(in[0]);
        l.slot = seed.root_leaf().slot;
        l.seed_dtype = sn.dtype;
      }
      return fused_leaf(n.shape, l);
    }
    case OpKind::Detach: return in[0];
    case OpKind::Cast:
      if (g_.dtype(n.src[0]) == n.dtype) return in[0];
      return elementwise(n, in);
    case OpKind::Bitcast: case OpKind::Add: case OpKind::Mul: case OpKind::Max: case OpKind::Neg: case OpKind::IDiv:
    case OpKind::And: case OpKind::Or: case OpKind::Xor: case OpKind::Shl: case OpKind::Shr: case OpKind::CmpLt: case OpKind::CmpEq:
    case OpKind::Where: case OpKind::Recip: case OpKind::Sqrt: case OpKind::Exp2: case OpKind::Log2: case OpKind::Sin: case OpKind::Floor:
      return elementwise(n, in);
    case OpKind::Sum: case OpKind::Prod: case OpKind::ReduceMax: return reduce(op.kind, in[0], op.axis);
    case OpKind::Softmax: case OpKind::RmsNorm: return softmax(op.kind, in[0], op.axis, op.eps);
    case OpKind::Sdpa: return sdpa(n, in[0], in[1], in[2]);
    case OpKind::Reshape: case OpKind::Permute: case OpKind::Expand: case OpKind::Slice: case OpKind::Flip: case OpKind::Pad:
      return movement(n, in[0]);
    case OpKind::DotGeneral: return dot(n, in[0], in[1]);
    case OpKind::QuantMatmul: return quant_matmul(n, in);
    case OpKind::Gather: case OpKind::GatherAlong: case OpKind::Scatter: case OpKind::ScatterAlong: case OpKind::Argsort: return indexing(n, in);
    case OpKind::ArgReduce: {
      Fused f = resolve_acc(in[0]);
      const int slot = new_slot(Slot::Temp, DType::I64, n.shape);
      if (!dry() && numel(n.shape) > 0) {
        if (g_.shape(n.src[0])[op.axis] == 0) throw Error::backend("argreduce over an empty axis");
        push_launch(emit_arg_reduce(f, op.axis, op.arg_min, sm_), f, slot);
      }
      return buffer_value(slot, DType::I64, n.shape);
    }
  }
  throw Error::backend(std::string("op ") + op_name(op.kind) + " has no CUDA kernel");
}

Program Scheduler::compile(const std::vector<NodeId>& roots) {
  const std::vector<NodeId> order = reachable(g_, roots);
  for (NodeId id : order) for (NodeId s : g_.node(id).src) ++consumers_[s];
  for (NodeId id : order) {
    SdpaMatch m;
    if (match_sdpa(id, &m)) {
      for (NodeId x : m.interior) skipped_[x] = true;
      sdpa_matches_.emplace(id, std::move(m));
    }
  }
  for (NodeId id : order) {
    if (skipped_.count(id)) continue;
    auto sm = sdpa_matches_.find(id);
    if (sm != sdpa_matches_.end()) {
      const SdpaMatch& m = sm->second;
      Fused q = materialize(resolve_acc(memo_.at(m.q))), k = materialize(resolve_acc(memo_.at(m.k))), v = materialize(resolve_acc(memo_.at(m.v)));
      memo_.emplace(id, attention(g_.dtype(id), g_.shape(id), m.causal, m.scale, q, k, v));
      continue;
    }
    Fused f = eval_node(id);
    // a shared, expensive expression is written once instead of being recomputed per consumer
    if (consumers_[id] > 1 && op_nodes(f) > 24 && find_acc(f) < 0) f = materialize(f);
    memo_.emplace(id, std::move(f));
  }
  for (NodeId root : roots) {
    const Fused& f = memo_.at(root);
    const Node& n = g_.node(root);
    // a value that already sits alone in a scratch buffer becomes the output in place
    if (find_acc(f) < 0 && f.is_plain_buffer() && f.root_leaf().view.is_contiguous() &&
        prog_.slots[static_cast<size_t>(f.root_leaf().slot)].kind == Slot::Temp) {
      Slot& s = prog_.slots[static_cast<size_t>(f.root_leaf().slot)];
      s.kind = Slot::Out; s.node = root; s.shape = n.shape;
      prog_.out_slots.push_back(f.root_leaf().slot);
      continue;
    }
    const int slot = new_slot(Slot::Out, n.dtype, n.shape, root);
    materialize(f, slot);
    prog_.out_slots.push_back(slot);
  }
  prog_.graph_nodes = g_.size();
  return std::move(prog_);
}

Program compile_program(Runtime& rt, const Graph& g, const std::vector<NodeId>& roots) {
  Scheduler dry(nullptr, g, rt.sm_count(), nullptr);
  dry.compile(roots);
  const std::vector<bool> plan = dry.fuse_plan();
  const KernelLoader load = [&rt](const std::string& src, const std::string& entry, bool fmad) { return rt.kernel(src, entry, fmad); };
  Scheduler real(&load, g, rt.sm_count(), &plan);
  return real.compile(roots);
}

std::vector<std::string> compile_check(const Graph& g, const std::vector<NodeId>& roots, int sm_count) {
  Scheduler dry(nullptr, g, sm_count, nullptr);
  dry.compile(roots);
  const std::vector<bool> plan = dry.fuse_plan();
  const KernelLoader load = [](const std::string& src, const std::string& entry, bool fmad) {
    std::string log;
    if (std::getenv("KURUMI_CUDA_DUMP")) fprintf(stderr, "---- kurumi_cuda kernel %s ----\n%s\n", entry.c_str(), src.c_str());
    std::string cubin = Runtime::compile_to_cubin(src, fmad, &log);
    if (cubin.find(entry) == std::string::npos) throw Error::backend("compiled cubin lacks entry point " + entry);
    return Kernel{};
  };
  Scheduler real(&load, g, sm_count, &plan);
  Program p = real.compile(roots);
  std::vector<std::string> names;
  for (auto& l : p.launches) names.push_back(l.name);
  return names;
}

}  // namespace ku::cu
