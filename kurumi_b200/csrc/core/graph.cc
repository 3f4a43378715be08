#include "graph.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <sstream>
#include <unordered_set>

namespace ku {

std::string shape_str(const Shape& s) {
  std::ostringstream o;
  o << "[";
  for (size_t i = 0; i < s.size(); ++i) o << (i ? ", " : "") << s[i];
  o << "]";
  return o.str();
}

std::vector<size_t> row_major_strides(const Shape& s) {
  std::vector<size_t> st(s.size(), 1);
  for (size_t i = s.size(); i-- > 1;) st[i - 1] = st[i] * s[i];
  return st;
}

const char* op_name(OpKind k) {
  static const char* n[] = {"Const", "Input", "Iota", "RandUniform", "Cast", "Bitcast", "Detach", "Add", "Mul", "Max",
                            "Neg", "IDiv", "And", "Or", "Xor", "Shl", "Shr", "CmpLt", "CmpEq", "Where", "Recip", "Sqrt",
                            "Exp2", "Log2", "Sin", "Floor", "Sum", "Prod", "ReduceMax", "Softmax", "RmsNorm", "Sdpa",
                            "Reshape", "Permute", "Expand", "Slice", "Flip", "Pad", "DotGeneral", "QuantMatmul", "ArgReduce",
                            "Gather", "GatherAlong", "Scatter", "ScatterAlong", "Argsort"};
  return n[static_cast<size_t>(k)];
}

static std::atomic<uint64_t> g_graph_counter{1};

void* (*HostMem::alloc)(size_t) = [](size_t bytes) -> void* { return std::malloc(bytes ? bytes : 1); };
void (*HostMem::release)(void*, size_t) = [](void* p, size_t) { std::free(p); };
void (*HostMem::copy)(void*, const void*, size_t) = [](void* dst, const void* src, size_t bytes) { if (bytes) std::memcpy(dst, src, bytes); };
Graph::Graph() : id_(g_graph_counter.fetch_add(1)) {}

const Node& Graph::node(NodeId i) const {
  if (i >= nodes_.size()) throw Error("panic: index out of bounds: the len is " + std::to_string(nodes_.size()) + " but the index is " + std::to_string(i));
  return nodes_[i];
}

std::vector<size_t> free_axes(size_t rank, const std::vector<size_t>& batch, const std::vector<size_t>& contract) {
  std::vector<size_t> out;
  for (size_t i = 0; i < rank; ++i)
    if (std::find(batch.begin(), batch.end(), i) == batch.end() && std::find(contract.begin(), contract.end(), i) == contract.end())
      out.push_back(i);
  return out;
}

// ---- inference (kurumi_core/src/graph/infer.rs) -----------------------------------------------
DType Graph::infer_dtype(const Op& op, const std::vector<NodeId>& src) const {
  switch (op.kind) {
    case OpKind::Const: return op.data->dtype;
    case OpKind::Input: case OpKind::Iota: case OpKind::Cast: case OpKind::Bitcast: return op.to;
    case OpKind::CmpLt: case OpKind::CmpEq: return DType::BOOL;
    case OpKind::ArgReduce: case OpKind::Argsort: return DType::I64;   // indices
    case OpKind::RandUniform: return DType::F32;
    case OpKind::Where: return node(src[1]).dtype;
    default: return node(src[0]).dtype;
  }
}

Shape Graph::derive_shape(const Op& op, const std::vector<NodeId>& src) const {
  auto ishape = [&](size_t i) -> const Shape& { return node(src[i]).shape; };
  switch (op.kind) {
    case OpKind::Const: case OpKind::Input: case OpKind::Iota: case OpKind::RandUniform:
    case OpKind::Reshape: case OpKind::Expand:
      return op.shape;
    case OpKind::Sum: case OpKind::Prod: case OpKind::ReduceMax: case OpKind::ArgReduce: {
      Shape s = ishape(0);
      s.erase(s.begin() + static_cast<long>(op.axis));
      return s;
    }
    case OpKind::Permute: {
      Shape o;
      for (size_t p : op.perm) o.push_back(ishape(0)[p]);
      return o;
    }
    case OpKind::Slice: {
      Shape o;
      for (auto& r : op.ranges) o.push_back((r[1] - r[0] + r[2] - 1) / r[2]);
      return o;
    }
    case OpKind::Pad: {
      Shape o;
      for (size_t d = 0; d < op.ranges.size(); ++d) o.push_back(op.ranges[d][0] + ishape(0)[d] + op.ranges[d][1]);
      return o;
    }
    case OpKind::DotGeneral: {
      const Shape &a = ishape(0), &b = ishape(1);
      Shape o;
      for (size_t i : op.lb) o.push_back(a[i]);
      for (size_t i : free_axes(a.size(), op.lb, op.lc)) o.push_back(a[i]);
      for (size_t i : free_axes(b.size(), op.rb, op.rc)) o.push_back(b[i]);
      return o;
    }
    case OpKind::QuantMatmul: return Shape{ishape(0)[0], ishape(1)[0]};   // act [M, K] x dequant(qweight) [N, K]^T
    case OpKind::Gather: {   // kurumi_core/src/graph/infer.rs:96-99
      const Shape &a = ishape(0), &ix = ishape(1);
      Shape o(a.begin(), a.begin() + static_cast<long>(op.axis));
      o.insert(o.end(), ix.begin(), ix.end());
      o.insert(o.end(), a.begin() + static_cast<long>(op.axis) + 1, a.end());
      return o;
    }
    case OpKind::GatherAlong: return ishape(1);   // the index shape
    default: return ishape(0);  // elementwise, Softmax, RmsNorm, Sdpa, Flip
  }
}

NodeId Graph::push(Op op, std::vector<NodeId> src) {
  for (NodeId s : src) (void)node(s);
  DType dt = infer_dtype(op, src);
  Shape sh = derive_shape(op, src);
  NodeId id = static_cast<NodeId>(nodes_.size());
  nodes_.push_back(Node{std::move(op), dt, std::move(src), std::move(sh)});
  return id;
}

// ---- guards (kurumi_core/src/graph/check.rs) --------------------------------------------------
void Graph::same_shape(const char* op, NodeId a, NodeId b) const {
  if (shape(a) != shape(b)) throw Error::shape(op, shape_str(shape(a)) + " vs " + shape_str(shape(b)));
}
void Graph::same_dtype(const char* op, NodeId a, NodeId b) const {
  if (dtype(a) != dtype(b)) throw Error::shape(op, std::string("dtype ") + dtype_name(dtype(a)) + " vs " + dtype_name(dtype(b)));
}
void Graph::require(const char* op, NodeId a, bool ok, const char* want) const {
  if (!ok) throw Error::shape(op, std::string(want) + " dtype required, got " + dtype_name(dtype(a)));
}
void Graph::reduce_axis_ok(const char* op, NodeId a, size_t axis) const {
  size_t rank = shape(a).size();
  if (axis >= rank) throw Error::shape(op, "axis " + std::to_string(axis) + " out of range for rank " + std::to_string(rank));
}
NodeId Graph::bin(const char* name, OpKind k, NodeId a, NodeId b) {
  same_shape(name, a, b);
  same_dtype(name, a, b);
  Op op; op.kind = k;
  return push(std::move(op), {a, b});
}

// ---- leaves -------------------------------------------------------------------------------------
NodeId Graph::constant(Tensor t) {
  if (t.bytes.size() != numel(t.shape) * dtype_width(t.dtype))
    throw Error::shape("constant", "data length " + std::to_string(t.len()) + " != shape " + shape_str(t.shape));
  Op op; op.kind = OpKind::Const; op.shape = t.shape;
  op.data = std::make_shared<const Tensor>(std::move(t));
  return push(std::move(op), {});
}
NodeId Graph::constant_f32(std::vector<float> v, Shape shape) { return constant(Tensor::from_f32(v.data(), v.size(), std::move(shape))); }
NodeId Graph::input(Shape shape, DType dt) { Op op; op.kind = OpKind::Input; op.shape = std::move(shape); op.to = dt; return push(std::move(op), {}); }
NodeId Graph::iota(Shape shape, size_t axis, DType dt) {
  if (axis >= shape.size()) throw Error::shape("iota", "axis " + std::to_string(axis) + " out of range for rank " + std::to_string(shape.size()));
  Op op; op.kind = OpKind::Iota; op.shape = std::move(shape); op.axis = axis; op.to = dt;
  return push(std::move(op), {});
}
NodeId Graph::rand_uniform(Shape shape, uint64_t seed) {
  Tensor t = Tensor::make(DType::I64, {1});
  int64_t s = static_cast<int64_t>(seed);
  std::memcpy(t.bytes.data(), &s, 8);
  NodeId sn = constant(std::move(t));
  Op op; op.kind = OpKind::RandUniform; op.shape = std::move(shape);
  return push(std::move(op), {sn});
}
NodeId Graph::rand_uniform_keyed(Shape shape, NodeId seed) {
  if (!is_int(dtype(seed))) throw Error::shape("rand_uniform", std::string("seed must be integer, got ") + dtype_name(dtype(seed)));
  Op op; op.kind = OpKind::RandUniform; op.shape = std::move(shape);
  return push(std::move(op), {seed});
}
NodeId Graph::cast(NodeId a, DType to) { Op op; op.kind = OpKind::Cast; op.to = to; return push(std::move(op), {a}); }
NodeId Graph::detach(NodeId a) { Op op; op.kind = OpKind::Detach; return push(std::move(op), {a}); }
NodeId Graph::bitcast(NodeId a, DType to) {
  DType from = dtype(a);
  if (dtype_width(from) != dtype_width(to))
    throw Error::shape("bitcast", std::string("width ") + dtype_name(from) + "(" + std::to_string(dtype_width(from)) + ") != " + dtype_name(to) + "(" + std::to_string(dtype_width(to)) + ")");
  Op op; op.kind = OpKind::Bitcast; op.to = to;
  return push(std::move(op), {a});
}

// ---- primitives ---------------------------------------------------------------------------------
NodeId Graph::add(NodeId a, NodeId b) { same_shape("add", a, b); same_dtype("add", a, b); require("add", a, is_arith(dtype(a)), "numeric or complex"); Op op; op.kind = OpKind::Add; return push(std::move(op), {a, b}); }
NodeId Graph::mul(NodeId a, NodeId b) { same_shape("mul", a, b); same_dtype("mul", a, b); require("mul", a, is_arith(dtype(a)), "numeric or complex"); Op op; op.kind = OpKind::Mul; return push(std::move(op), {a, b}); }
NodeId Graph::max(NodeId a, NodeId b) { same_shape("max", a, b); same_dtype("max", a, b); require("max", a, is_numeric(dtype(a)), "numeric"); Op op; op.kind = OpKind::Max; return push(std::move(op), {a, b}); }
NodeId Graph::neg(NodeId a) {
  if (!(is_signed(dtype(a)) || is_complex(dtype(a)))) throw Error(std::string("panic: neg requires signed/complex, got ") + dtype_name(dtype(a)));
  Op op; op.kind = OpKind::Neg; return push(std::move(op), {a});
}
NodeId Graph::unary_float(const char* name, OpKind k, NodeId a, bool allow_complex) {
  if (!(is_float(dtype(a)) || (allow_complex && is_complex(dtype(a)))))
    throw Error(std::string("panic: ") + name + " requires a float dtype, got " + dtype_name(dtype(a)));
  Op op; op.kind = k; return push(std::move(op), {a});
}
NodeId Graph::recip(NodeId a) { return unary_float("recip", OpKind::Recip, a, true); }
NodeId Graph::sqrt(NodeId a) { return unary_float("sqrt", OpKind::Sqrt, a, true); }
NodeId Graph::exp2(NodeId a) { return unary_float("exp2", OpKind::Exp2, a, true); }
NodeId Graph::log2(NodeId a) { return unary_float("log2", OpKind::Log2, a, true); }
NodeId Graph::sin(NodeId a) { return unary_float("sin", OpKind::Sin, a, false); }
NodeId Graph::floor(NodeId a) { return unary_float("floor", OpKind::Floor, a, false); }
NodeId Graph::idiv(NodeId a, NodeId b) { if (!is_int(dtype(a))) throw Error::shape("idiv", std::string("requires integer dtype, got ") + dtype_name(dtype(a))); return bin("idiv", OpKind::IDiv, a, b); }
NodeId Graph::shl(NodeId a, NodeId b) { if (!is_int(dtype(a))) throw Error::shape("shl", std::string("requires integer dtype, got ") + dtype_name(dtype(a))); return bin("shl", OpKind::Shl, a, b); }
NodeId Graph::shr(NodeId a, NodeId b) { if (!is_int(dtype(a))) throw Error::shape("shr", std::string("requires integer dtype, got ") + dtype_name(dtype(a))); return bin("shr", OpKind::Shr, a, b); }
NodeId Graph::bit_and(NodeId a, NodeId b) { require("and", a, !is_float(dtype(a)) && !is_complex(dtype(a)), "bool/integer"); return bin("and", OpKind::And, a, b); }
NodeId Graph::bit_or(NodeId a, NodeId b) { require("or", a, !is_float(dtype(a)) && !is_complex(dtype(a)), "bool/integer"); return bin("or", OpKind::Or, a, b); }
NodeId Graph::bit_xor(NodeId a, NodeId b) { require("xor", a, !is_float(dtype(a)) && !is_complex(dtype(a)), "bool/integer"); return bin("xor", OpKind::Xor, a, b); }
NodeId Graph::cmp_lt(NodeId a, NodeId b) { require("cmp_lt", a, !is_complex(dtype(a)), "orderable (non-complex)"); return bin("cmp_lt", OpKind::CmpLt, a, b); }
NodeId Graph::cmp_eq(NodeId a, NodeId b) { require("cmp_eq", a, !is_complex(dtype(a)), "orderable (non-complex)"); return bin("cmp_eq", OpKind::CmpEq, a, b); }
NodeId Graph::select(NodeId cond, NodeId a, NodeId b) {
  same_shape("select", cond, a); same_shape("select", a, b); same_dtype("select", a, b);
  if (dtype(cond) != DType::BOOL) throw Error::shape("select", std::string("cond must be BOOL, got ") + dtype_name(dtype(cond)));
  Op op; op.kind = OpKind::Where; return push(std::move(op), {cond, a, b});
}
NodeId Graph::sum(NodeId a, size_t axis) { reduce_axis_ok("sum", a, axis); require("sum", a, is_arith(dtype(a)), "numeric or complex"); Op op; op.kind = OpKind::Sum; op.axis = axis; return push(std::move(op), {a}); }
NodeId Graph::prod(NodeId a, size_t axis) { reduce_axis_ok("prod", a, axis); require("prod", a, is_arith(dtype(a)), "numeric or complex"); Op op; op.kind = OpKind::Prod; op.axis = axis; return push(std::move(op), {a}); }
NodeId Graph::reduce_max(NodeId a, size_t axis) { reduce_axis_ok("reduce_max", a, axis); require("reduce_max", a, is_numeric(dtype(a)), "numeric"); Op op; op.kind = OpKind::ReduceMax; op.axis = axis; return push(std::move(op), {a}); }
// kurumi_core/src/graph/ops/core/reduce.rs:24-33
// ---- indexing (kurumi_core/src/graph/ops/core/indexing.rs:21-136) --------------------------------
NodeId Graph::gather(NodeId operand, NodeId indices, size_t axis) {
  reduce_axis_ok("gather", operand, axis);
  if (!is_int(dtype(indices))) throw Error::shape("gather", std::string("indices must be integer, got ") + dtype_name(dtype(indices)));
  Op op; op.kind = OpKind::Gather; op.axis = axis;
  return push(std::move(op), {operand, indices});
}
NodeId Graph::gather_along(NodeId operand, NodeId indices, size_t axis) {
  reduce_axis_ok("gather_along", operand, axis);
  if (!is_int(dtype(indices))) throw Error::shape("gather_along", std::string("indices must be integer, got ") + dtype_name(dtype(indices)));
  const Shape &os = shape(operand), &is = shape(indices);
  bool ok = is.size() == os.size();
  for (size_t d = 0; ok && d < os.size(); ++d) if (d != axis && is[d] != os[d]) ok = false;
  if (!ok) throw Error::shape("gather_along", "indices " + shape_str(is) + " must match operand " + shape_str(os) + " except axis " + std::to_string(axis));
  Op op; op.kind = OpKind::GatherAlong; op.axis = axis;
  return push(std::move(op), {operand, indices});
}
NodeId Graph::scatter(NodeId operand, NodeId indices, NodeId updates, size_t axis, uint8_t combine) {
  reduce_axis_ok("scatter", operand, axis);
  if (combine > 3) throw Error::shape("scatter", "unknown combiner " + std::to_string(combine));
  if (!is_int(dtype(indices))) throw Error::shape("scatter", std::string("indices must be integer, got ") + dtype_name(dtype(indices)));
  same_dtype("scatter", operand, updates);
  const Shape &os = shape(operand), &is = shape(indices);
  Shape want(os.begin(), os.begin() + static_cast<long>(axis));
  want.insert(want.end(), is.begin(), is.end());
  want.insert(want.end(), os.begin() + static_cast<long>(axis) + 1, os.end());
  if (shape(updates) != want) throw Error::shape("scatter", "updates shape " + shape_str(shape(updates)) + " != " + shape_str(want));
  if (combine != 0 && !is_numeric(dtype(operand))) throw Error::shape("scatter", "Add/Max combiner needs a numeric operand");
  Op op; op.kind = OpKind::Scatter; op.axis = axis; op.combine = combine;
  return push(std::move(op), {operand, indices, updates});
}
NodeId Graph::scatter_along(NodeId operand, NodeId indices, NodeId updates, size_t axis, uint8_t combine) {
  reduce_axis_ok("scatter_along", operand, axis);
  if (combine > 3) throw Error::shape("scatter_along", "unknown combiner " + std::to_string(combine));
  if (!is_int(dtype(indices))) throw Error::shape("scatter_along", std::string("indices must be integer, got ") + dtype_name(dtype(indices)));
  if (combine != 0 && !is_numeric(dtype(operand))) throw Error::shape("scatter_along", "Add/Max combiner needs a numeric operand");
  same_dtype("scatter_along", operand, updates);
  if (shape(indices) != shape(updates)) throw Error::shape("scatter_along", "indices and updates must share a shape");
  const Shape &os = shape(operand), &is = shape(indices);
  bool ok = is.size() == os.size();
  for (size_t d = 0; ok && d < os.size(); ++d) if (d != axis && is[d] != os[d]) ok = false;
  if (!ok) throw Error::shape("scatter_along", "indices " + shape_str(is) + " must match operand " + shape_str(os) + " except axis " + std::to_string(axis));
  Op op; op.kind = OpKind::ScatterAlong; op.axis = axis; op.combine = combine;
  return push(std::move(op), {operand, indices, updates});
}
NodeId Graph::argsort(NodeId a, size_t axis, bool descending) {
  reduce_axis_ok("argsort", a, axis);
  require("argsort", a, is_numeric(dtype(a)), "numeric");
  Op op; op.kind = OpKind::Argsort; op.axis = axis; op.descending = descending;
  return push(std::move(op), {a});
}
NodeId Graph::sort(NodeId a, size_t axis, bool descending) { return gather_along(a, argsort(a, axis, descending), axis); }

NodeId Graph::argmax(NodeId a, size_t axis) { reduce_axis_ok("argmax", a, axis); require("argmax", a, is_numeric(dtype(a)), "numeric"); Op op; op.kind = OpKind::ArgReduce; op.axis = axis; op.arg_min = false; return push(std::move(op), {a}); }
NodeId Graph::argmin(NodeId a, size_t axis) { reduce_axis_ok("argmin", a, axis); require("argmin", a, is_numeric(dtype(a)), "numeric"); Op op; op.kind = OpKind::ArgReduce; op.axis = axis; op.arg_min = true; return push(std::move(op), {a}); }
NodeId Graph::softmax(NodeId a, size_t axis) { reduce_axis_ok("softmax", a, axis); require("softmax", a, is_float(dtype(a)), "float"); Op op; op.kind = OpKind::Softmax; op.axis = axis; return push(std::move(op), {a}); }
NodeId Graph::rmsnorm(NodeId a, size_t axis, float eps) { reduce_axis_ok("rmsnorm", a, axis); require("rmsnorm", a, is_float(dtype(a)), "float"); Op op; op.kind = OpKind::RmsNorm; op.axis = axis; op.eps = eps; return push(std::move(op), {a}); }

NodeId Graph::reshape(NodeId a, Shape sh) {
  size_t from = numel(shape(a)), to = numel(sh);
  if (from != to) throw Error::shape("reshape", "numel " + std::to_string(from) + " -> " + std::to_string(to));
  Op op; op.kind = OpKind::Reshape; op.shape = std::move(sh);
  return push(std::move(op), {a});
}
NodeId Graph::permute(NodeId a, std::vector<size_t> perm) {
  size_t rank = shape(a).size();
  std::vector<size_t> sorted = perm;
  std::sort(sorted.begin(), sorted.end());
  bool ok = sorted.size() == rank;
  for (size_t i = 0; ok && i < rank; ++i) ok = sorted[i] == i;
  if (!ok) throw Error::shape("permute", shape_str(perm) + " is not a permutation of 0.." + std::to_string(rank));
  Op op; op.kind = OpKind::Permute; op.perm = std::move(perm);
  return push(std::move(op), {a});
}
NodeId Graph::expand(NodeId a, Shape sh) {
  const Shape& from = shape(a);
  bool ok = from.size() == sh.size();
  for (size_t i = 0; ok && i < sh.size(); ++i) ok = from[i] == sh[i] || from[i] == 1;
  if (!ok) throw Error::shape("expand", shape_str(from) + " -> " + shape_str(sh));
  Op op; op.kind = OpKind::Expand; op.shape = std::move(sh);
  return push(std::move(op), {a});
}
NodeId Graph::slice_step(NodeId a, std::vector<std::array<size_t, 3>> ranges) {
  const Shape& s = shape(a);
  if (ranges.size() != s.size()) throw Error::shape("slice", "rank " + std::to_string(s.size()) + " vs " + std::to_string(ranges.size()) + " ranges");
  for (size_t d = 0; d < s.size(); ++d) {
    if (ranges[d][2] == 0) throw Error::shape("slice", "step must be >= 1");
    if (ranges[d][0] > ranges[d][1] || ranges[d][1] > s[d])
      throw Error::shape("slice", "[" + std::to_string(ranges[d][0]) + ", " + std::to_string(ranges[d][1]) + ") out of [0, " + std::to_string(s[d]) + "]");
  }
  Op op; op.kind = OpKind::Slice; op.ranges = std::move(ranges);
  return push(std::move(op), {a});
}
NodeId Graph::slice(NodeId a, std::vector<std::array<size_t, 2>> ranges) {
  std::vector<std::array<size_t, 3>> r;
  for (auto& x : ranges) r.push_back({x[0], x[1], 1});
  return slice_step(a, std::move(r));
}
NodeId Graph::flip(NodeId a, std::vector<size_t> axes) {
  size_t rank = shape(a).size();
  for (size_t k = 0; k < axes.size(); ++k) {
    if (axes[k] >= rank) throw Error::shape("flip", "axis " + std::to_string(axes[k]) + " out of range for rank " + std::to_string(rank));
    if (std::find(axes.begin(), axes.begin() + static_cast<long>(k), axes[k]) != axes.begin() + static_cast<long>(k))
      throw Error::shape("flip", "axis " + std::to_string(axes[k]) + " repeated");
  }
  Op op; op.kind = OpKind::Flip; op.perm = std::move(axes);
  return push(std::move(op), {a});
}
NodeId Graph::pad(NodeId a, std::vector<std::array<size_t, 2>> pads) {
  size_t rank = shape(a).size();
  if (pads.size() != rank) throw Error::shape("pad", "rank " + std::to_string(rank) + " vs " + std::to_string(pads.size()) + " pads");
  Op op; op.kind = OpKind::Pad;
  for (auto& p : pads) op.ranges.push_back({p[0], p[1], 0});
  return push(std::move(op), {a});
}

static void check_axes(const std::vector<size_t>& axes, size_t rank) {
  for (size_t k = 0; k < axes.size(); ++k) {
    if (axes[k] >= rank) throw Error::shape("dot_general", "axis " + std::to_string(axes[k]) + " out of range for rank " + std::to_string(rank));
    for (size_t j = 0; j < k; ++j)
      if (axes[j] == axes[k]) throw Error::shape("dot_general", "axis " + std::to_string(axes[k]) + " used twice");
  }
}
NodeId Graph::dot_general(NodeId a, NodeId b, std::vector<size_t> lc, std::vector<size_t> rc, std::vector<size_t> lb, std::vector<size_t> rb) {
  const Shape sa = shape(a), sb = shape(b);
  same_dtype("dot_general", a, b);
  require("dot_general", a, is_arith(dtype(a)), "numeric or complex");
  if (lc.size() != rc.size()) throw Error::shape("dot_general", "contract count mismatch");
  if (lb.size() != rb.size()) throw Error::shape("dot_general", "batch count mismatch");
  std::vector<size_t> aa = lb, ba = rb;
  aa.insert(aa.end(), lc.begin(), lc.end());
  ba.insert(ba.end(), rc.begin(), rc.end());
  check_axes(aa, sa.size());
  check_axes(ba, sb.size());
  for (size_t i = 0; i < lb.size(); ++i)
    if (sa[lb[i]] != sb[rb[i]]) throw Error::shape("dot_general", "batch dim " + std::to_string(sa[lb[i]]) + " vs " + std::to_string(sb[rb[i]]));
  for (size_t i = 0; i < lc.size(); ++i)
    if (sa[lc[i]] != sb[rc[i]]) throw Error::shape("dot_general", "contract dim " + std::to_string(sa[lc[i]]) + " vs " + std::to_string(sb[rc[i]]));
  Op op; op.kind = OpKind::DotGeneral; op.lc = std::move(lc); op.rc = std::move(rc); op.lb = std::move(lb); op.rb = std::move(rb);
  return push(std::move(op), {a, b});
}

// ---- decompositions -----------------------------------------------------------------------------
// kurumi_core/src/graph/ops/core/elementwise.rs:83-94: a 1-element Const in `like`'s dtype
// (converted through the f64 cast path), reshaped to rank-many 1s and expanded.
NodeId Graph::scalar(NodeId like, float v) {
  Shape sh = shape(like);
  Tensor t = Tensor::from_f32(&v, 1, Shape(sh.size(), 1));
  if (dtype(like) != DType::F32) t = cast_tensor(t, dtype(like));
  NodeId c = constant(std::move(t));
  return expand(c, sh);
}
NodeId Graph::sub(NodeId a, NodeId b) { return add(a, neg(b)); }
NodeId Graph::div(NodeId a, NodeId b) { return mul(a, recip(b)); }
NodeId Graph::abs(NodeId a) { return max(a, neg(a)); }
NodeId Graph::square(NodeId a) { return mul(a, a); }
NodeId Graph::min(NodeId a, NodeId b) { return select(cmp_lt(a, b), a, b); }
NodeId Graph::clamp_min(NodeId a, float lo) { return max(a, scalar(a, lo)); }
NodeId Graph::exp(NodeId x) { NodeId s = scalar(x, 1.44269504088896340736f); return exp2(mul(x, s)); }
NodeId Graph::ln(NodeId x) { NodeId l = log2(x); return mul(l, scalar(l, 0.693147180559945309417f)); }
NodeId Graph::cos(NodeId x) { NodeId hp = scalar(x, 1.57079632679489661923f); return sin(add(x, hp)); }
NodeId Graph::sigmoid(NodeId x) {
  NodeId e = exp(neg(x));
  NodeId one = scalar(x, 1.0f);
  return recip(add(one, e));
}
NodeId Graph::tanh(NodeId x) {
  NodeId two = scalar(x, 2.0f);
  NodeId s = sigmoid(mul(x, two));
  NodeId two2 = scalar(x, 2.0f);
  NodeId s2 = mul(s, two2);
  NodeId one = scalar(x, 1.0f);
  return sub(s2, one);
}
NodeId Graph::relu(NodeId x) { return max(x, scalar(x, 0.0f)); }
NodeId Graph::silu(NodeId x) { return mul(x, sigmoid(x)); }
NodeId Graph::gelu(NodeId x) {
  NodeId x2 = mul(x, x);
  NodeId x3 = mul(x2, x);
  NodeId c = scalar(x, 0.044715f);
  NodeId inner = add(x, mul(c, x3));
  NodeId k = scalar(x, std::sqrt(2.0f / 3.14159265358979323846f));
  NodeId t = tanh(mul(k, inner));
  NodeId one = scalar(x, 1.0f);
  NodeId onep = add(one, t);
  NodeId half = scalar(x, 0.5f);
  NodeId hx = mul(half, x);
  return mul(hx, onep);
}
NodeId Graph::logical_not(NodeId b) {
  Shape sh = shape(b);
  Tensor t = Tensor::make(DType::BOOL, Shape(sh.size(), 1));
  t.bytes[0] = 1;
  NodeId c = expand(constant(std::move(t)), sh);
  return bit_xor(b, c);
}
NodeId Graph::gt(NodeId a, NodeId b) { return cmp_lt(b, a); }
NodeId Graph::ge(NodeId a, NodeId b) { return logical_not(cmp_lt(a, b)); }
NodeId Graph::le(NodeId a, NodeId b) { return logical_not(cmp_lt(b, a)); }
NodeId Graph::ne(NodeId a, NodeId b) { return logical_not(cmp_eq(a, b)); }
NodeId Graph::mean(NodeId x, size_t axis) {
  reduce_axis_ok("mean", x, axis);
  float n = static_cast<float>(shape(x)[axis]);
  NodeId s = sum(x, axis);
  return mul(s, scalar(s, 1.0f / n));
}
NodeId Graph::reduce_min(NodeId x, size_t axis) { return neg(reduce_max(neg(x), axis)); }
NodeId Graph::transpose(NodeId x, size_t i, size_t j) {
  size_t r = shape(x).size();
  if (i >= r || j >= r) throw Error::shape("transpose", "axes out of range");
  std::vector<size_t> perm(r);
  for (size_t k = 0; k < r; ++k) perm[k] = k;
  std::swap(perm[i], perm[j]);
  return permute(x, perm);
}
NodeId Graph::broadcast_to(NodeId x, Shape sh) {
  const Shape xs = shape(x);
  if (xs.size() < sh.size()) {
    Shape s(sh.size() - xs.size(), 1);
    s.insert(s.end(), xs.begin(), xs.end());
    x = reshape(x, s);
  }
  return expand(x, std::move(sh));
}
// kurumi_core/src/graph/ops/core/random.rs:28-49
NodeId Graph::randn(Shape sh, uint64_t seed) {
  NodeId u1 = clamp_min(rand_uniform(sh, seed), 1e-7f);
  NodeId u2 = rand_uniform(sh, seed ^ 0xD1B54A32D192ED03ull);
  NodeId lu = ln(u1);
  NodeId r2 = mul(lu, scalar(lu, -2.0f));
  NodeId r = sqrt(r2);
  NodeId ang = mul(u2, scalar(u2, 6.28318530717958647692f));
  return mul(r, cos(ang));
}
NodeId Graph::rand_range(Shape sh, uint64_t seed, float lo, float hi) {
  NodeId u = rand_uniform(std::move(sh), seed);
  NodeId su = mul(u, scalar(u, hi - lo));
  return add(su, scalar(su, lo));
}

// kurumi_core/src/graph/ops/nn/attention.rs:78-153
NodeId Graph::sdpa(NodeId q, NodeId k, NodeId v, bool causal) {
  require("sdpa", q, is_float(dtype(q)), "float");
  const Shape qs = shape(q), ks = shape(k), vs = shape(v);
  size_t r = qs.size();
  if (r < 2) throw Error::shape("sdpa", "need rank>=2, got " + shape_str(qs));
  size_t batch = 1;
  for (size_t i = 0; i + 2 < r; ++i) batch *= qs[i];
  size_t s = qs[r - 2];
  size_t scores_bytes = batch * s * s * 4;
  if (qs == ks && qs == vs && scores_bytes > (size_t(1) << 30)) return sdpa_fused(q, k, v, causal);
  return sdpa_decomposed(q, k, v, causal);
}
NodeId Graph::sdpa_fused(NodeId q, NodeId k, NodeId v, bool causal) {
  const Shape qs = shape(q), ks = shape(k), vs = shape(v);
  if (qs != ks || qs != vs) throw Error::shape("sdpa_fused", "q/k/v must share shape: " + shape_str(qs) + " " + shape_str(ks) + " " + shape_str(vs));
  size_t r = qs.size();
  if (r < 2 || qs[r - 1] == 0) throw Error::shape("sdpa_fused", "need rank>=2 with dh>0, got " + shape_str(qs));
  same_dtype("sdpa_fused", q, k);
  same_dtype("sdpa_fused", q, v);
  Op op; op.kind = OpKind::Sdpa; op.causal = causal;
  return push(std::move(op), {q, k, v});
}
// kurumi_core/src/graph/ops/core/contract.rs:52-116
NodeId Graph::quant_matmul(NodeId act, NodeId qweight, NodeId scales, const NodeId* mins, uint8_t bits, size_t group_size) {
  const Shape sa = shape(act), sq = shape(qweight);
  if (sa.size() != 2 || sq.size() != 2)
    throw Error::shape("quant_matmul", "act rank " + std::to_string(sa.size()) + ", qweight rank " + std::to_string(sq.size()) + ": both must be rank-2");
  if (dtype(qweight) != DType::U8) throw Error::shape("quant_matmul", std::string("qweight must be U8, got ") + dtype_name(dtype(qweight)));
  if (dtype(scales) != DType::F16) throw Error::shape("quant_matmul", std::string("scales must be F16, got ") + dtype_name(dtype(scales)));
  if (mins && dtype(*mins) != DType::F16) throw Error::shape("quant_matmul", std::string("mins must be F16, got ") + dtype_name(dtype(*mins)));
  if (!is_float(dtype(act))) throw Error::shape("quant_matmul", std::string("act must be float, got ") + dtype_name(dtype(act)));
  const size_t k = sa[1], n = sq[0];
  if (!(bits == 2 || bits == 4 || bits == 8)) throw Error::shape("quant_matmul", "bits " + std::to_string(bits) + " must be 2, 4, or 8");
  if (group_size == 0 || k % group_size != 0)
    throw Error::shape("quant_matmul", "K " + std::to_string(k) + " must be a nonzero multiple of group_size " + std::to_string(group_size));
  if (sq[1] * 8 != k * bits)
    throw Error::shape("quant_matmul", "qweight cols " + std::to_string(sq[1]) + " must equal K*bits/8 = " + std::to_string(k) + "*" + std::to_string(bits) + "/8");
  const size_t want = n * (k / group_size);
  if (numel(shape(scales)) != want) throw Error::shape("quant_matmul", "scales must have N*K/group_size = " + std::to_string(want) + " entries");
  if (mins && numel(shape(*mins)) != want) throw Error::shape("quant_matmul", "mins must have N*K/group_size = " + std::to_string(want) + " entries");
  Op op; op.kind = OpKind::QuantMatmul; op.bits = bits; op.group_size = group_size; op.symmetric = mins == nullptr;
  std::vector<NodeId> src{act, qweight, scales};
  if (mins) src.push_back(*mins);
  return push(std::move(op), std::move(src));
}

// kurumi_core/src/quant.rs:38-88
void quantize(const float* w, size_t rows, size_t cols, uint8_t bits, size_t group_size, bool symmetric, uint8_t* packed, uint16_t* scales, uint16_t* mins) {
  if (!(bits == 2 || bits == 4 || bits == 8)) throw Error::shape("quantize", "bits must be 2, 4, or 8");
  if (group_size == 0 || cols % group_size != 0) throw Error::shape("quantize", "cols must be a multiple of group_size");
  if (!w || !packed || !scales || (!symmetric && !mins)) throw Error::shape("quantize", "null buffer");
  const size_t ng = cols / group_size, rb = cols * bits / 8, per = 8 / bits;
  std::memset(packed, 0, rows * rb);
  auto put = [&](size_t r, size_t c, uint8_t v) {
    const size_t i = r * rb + c / per, shift = (c % per) * bits;
    const uint8_t mask = static_cast<uint8_t>((1u << bits) - 1);
    packed[i] = static_cast<uint8_t>((packed[i] & ~(mask << shift)) | ((v & mask) << shift));
  };
  auto f16_of = [](float f) { uint16_t h; f64_to_elem(DType::F16, static_cast<double>(f), &h); return h; };
  auto f32_of = [](uint16_t h) { return static_cast<float>(elem_to_f64(DType::F16, &h)); };
  for (size_t r = 0; r < rows; ++r)
    for (size_t g = 0; g < ng; ++g) {
      const float* grp = w + r * cols + g * group_size;
      const size_t si = r * ng + g;
      if (symmetric) {
        float amax = 0.0f;
        for (size_t i = 0; i < group_size; ++i) amax = std::fmax(amax, std::fabs(grp[i]));
        const int qlo = -(1 << (bits - 1)), qhi = (1 << (bits - 1)) - 1;
        scales[si] = f16_of(amax > 0.0f ? amax / static_cast<float>(qhi) : 1.0f);
        const float sv = f32_of(scales[si]);
        for (size_t i = 0; i < group_size; ++i) {
          float q = std::round(grp[i] / sv);
          q = std::fmin(std::fmax(q, static_cast<float>(qlo)), static_cast<float>(qhi));
          put(r, g * group_size + i, static_cast<uint8_t>(static_cast<int>(q) & ((1 << bits) - 1)));
        }
      } else {
        float mn = std::numeric_limits<float>::infinity(), mx = -std::numeric_limits<float>::infinity();
        for (size_t i = 0; i < group_size; ++i) { mn = std::fmin(mn, grp[i]); mx = std::fmax(mx, grp[i]); }
        const float qmax = static_cast<float>((1u << bits) - 1);
        scales[si] = f16_of(mx > mn ? (mx - mn) / qmax : 1.0f);
        mins[si] = f16_of(mn);
        const float sv = f32_of(scales[si]), mv = f32_of(mins[si]);
        for (size_t i = 0; i < group_size; ++i) {
          float q = std::round((grp[i] - mv) / sv);
          q = std::fmin(std::fmax(q, 0.0f), qmax);
          put(r, g * group_size + i, static_cast<uint8_t>(static_cast<unsigned>(q)));
        }
      }
    }
}

std::vector<float> dequantize(const uint8_t* packed, const uint16_t* scales, const uint16_t* mins, size_t rows, size_t cols, uint8_t bits, size_t group_size) {
  const size_t ng = cols / group_size, rb = cols * bits / 8, per = 8 / bits;
  std::vector<float> out(rows * cols);
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      const size_t gi = r * ng + c / group_size;
      const uint8_t raw = static_cast<uint8_t>((packed[r * rb + c / per] >> ((c % per) * bits)) & ((1u << bits) - 1));
      const float scale = static_cast<float>(elem_to_f64(DType::F16, scales + gi));
      if (mins) {
        out[r * cols + c] = static_cast<float>(raw) * scale + static_cast<float>(elem_to_f64(DType::F16, mins + gi));
      } else {
        const int sh = 32 - bits;   // sign-extend the field
        const int v = static_cast<int>(static_cast<uint32_t>(raw) << sh) >> sh;
        out[r * cols + c] = static_cast<float>(v) * scale;
      }
    }
  return out;
}

NodeId Graph::causal_bias(size_t s, const Shape& out_shape) {
  std::vector<float> data(s * s, 0.0f);
  for (size_t i = 0; i < s; ++i)
    for (size_t j = i + 1; j < s; ++j) data[i * s + j] = -std::numeric_limits<float>::infinity();
  NodeId bias = constant_f32(std::move(data), {s, s});
  size_t rank = out_shape.size();
  Shape full(rank, 1);
  full[rank - 2] = s; full[rank - 1] = s;
  return expand(reshape(bias, full), out_shape);
}
NodeId Graph::sdpa_decomposed(NodeId q, NodeId k, NodeId v, bool causal) {
  const Shape qs = shape(q);
  size_t r = qs.size();
  if (r < 2) throw Error::shape("sdpa", "need rank>=2, got " + shape_str(qs));
  size_t s = qs[r - 2], dh = qs[r - 1];
  std::vector<size_t> batch;
  for (size_t i = 0; i + 2 < r; ++i) batch.push_back(i);
  NodeId raw = dot_general(q, k, {r - 1}, {r - 1}, batch, batch);
  NodeId inv = scalar(raw, 1.0f / std::sqrt(static_cast<float>(dh)));
  NodeId scores = mul(raw, inv);
  if (causal) {
    DType dt = dtype(scores);
    NodeId bias = causal_bias(s, shape(scores));
    if (dt != DType::F32) bias = cast(bias, dt);
    scores = add(scores, bias);
  }
  NodeId attn = softmax(scores, r - 1);
  return dot_general(attn, v, {r - 1}, {r - 2}, batch, batch);
}

// ---- inspect / passes ---------------------------------------------------------------------------
std::vector<NodeId> reachable(const Graph& g, const std::vector<NodeId>& roots) {
  std::vector<NodeId> order;
  std::unordered_set<NodeId> seen;
  std::vector<std::pair<NodeId, bool>> stack;
  for (size_t i = roots.size(); i-- > 0;) stack.push_back({roots[i], false});
  while (!stack.empty()) {
    auto [id, expanded] = stack.back();
    stack.pop_back();
    if (expanded) { order.push_back(id); continue; }
    if (!seen.insert(id).second) continue;
    stack.push_back({id, true});
    for (NodeId s : g.node(id).src)
      if (!seen.count(s)) stack.push_back({s, false});
  }
  return order;
}

std::string dump(const Graph& g, NodeId root) {
  std::ostringstream o;
  for (NodeId id : reachable(g, {root})) {
    const Node& n = g.node(id);
    o << "%" << id << " = " << op_name(n.op.kind);
    if (n.op.kind == OpKind::Const || n.op.kind == OpKind::Input) o << shape_str(n.op.shape);
    o << "(";
    for (size_t i = 0; i < n.src.size(); ++i) o << (i ? ", " : "") << "%" << n.src[i];
    o << ") : " << shape_str(n.shape) << " " << dtype_name(n.dtype) << "\n";
  }
  return o.str();
}

NodeId amp(Graph& g, NodeId root) { return amp_to(g, root, DType::F16); }

NodeId amp_to(Graph& g, NodeId root, DType target) {
  if (!(target == DType::F16 || target == DType::BF16 || target == DType::F8E4M3))
    throw Error::shape("amp", std::string("unsupported target dtype ") + dtype_name(target));
  std::unordered_map<NodeId, NodeId> remap;
  for (NodeId id : reachable(g, {root})) {
    std::vector<NodeId> src_old = g.node(id).src;
    if (src_old.empty()) { remap[id] = id; continue; }
    std::vector<NodeId> src;
    for (NodeId s : src_old) src.push_back(remap.at(s));
    Op op = g.node(id).op;
    DType dt = g.dtype(id);
    NodeId nw;
    if (op.kind == OpKind::DotGeneral && target != DType::F8E4M3 && dt == DType::F32) {
      NodeId a = g.cast(src[0], target), b = g.cast(src[1], target);
      nw = g.cast(g.push(op, {a, b}), DType::F32);
    } else if (op.kind == OpKind::DotGeneral && target == DType::F8E4M3 && (dt == DType::F32 || dt == DType::BF16 || dt == DType::F16)) {
      auto quant = [&](NodeId x) {
        const Node& n = g.node(x);
        if (n.op.kind == OpKind::Cast && g.dtype(n.src[0]) == DType::F8E4M3) return x;  // already fp8 values
        return g.cast(g.cast(x, DType::F8E4M3), dt);
      };
      NodeId a = quant(src[0]), b = quant(src[1]);
      nw = (a == src_old[0] && b == src_old[1]) ? id : g.push(op, {a, b});
    } else if (src == src_old) {
      nw = id;
    } else {
      nw = g.push(op, src);
    }
    remap[id] = nw;
  }
  return remap.at(root);
}

Tensor cast_tensor(const Tensor& src, DType to) {
  Tensor out = Tensor::make(to, src.shape);
  size_t n = src.len(), ws = dtype_width(src.dtype), wd = dtype_width(to);
  if (src.dtype == to) { out.bytes = src.bytes; return out; }
  for (size_t i = 0; i < n; ++i) f64_to_elem(to, elem_to_f64(src.dtype, src.bytes.data() + i * ws), out.bytes.data() + i * wd);
  return out;
}

}  // namespace ku
