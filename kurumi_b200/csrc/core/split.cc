#include "split.h"

#include <algorithm>
#include <unordered_map>

namespace ku {

namespace {
constexpr int kWhole = -1, kUnset = -2;

struct Walk {
  const Graph& g;
  size_t parts;
  std::unordered_map<NodeId, int> axis;   // per node: the axis that carries the root's row index, or kWhole
  std::string why;

  bool fail(NodeId id, const std::string& what) {
    why = std::string(op_name(g.node(id).op.kind)) + " (node " + std::to_string(id) + "): " + what;
    return false;
  }
  // `id` needs source `s` cut along `a` (or whole)
  bool want(NodeId id, NodeId s, int a) {
    auto it = axis.find(s);
    if (it == axis.end() || it->second == kUnset) { axis[s] = a; return true; }
    if (it->second != a) return fail(id, "operand node " + std::to_string(s) + " is needed both along axis " + std::to_string(it->second) + " and " + (a == kWhole ? std::string("whole") : "along axis " + std::to_string(a)));
    return true;
  }
  bool all(NodeId id, int a) {
    for (NodeId s : g.node(id).src) if (!want(id, s, a)) return false;
    return true;
  }

  bool visit(NodeId id) {
    const Node& n = g.node(id);
    const Op& op = n.op;
    const int a = axis.at(id);
    if (a == kWhole) return all(id, kWhole);
    const size_t ax = static_cast<size_t>(a);
    if (ax >= n.shape.size() || n.shape[ax] % parts != 0) return fail(id, "extent " + (ax < n.shape.size() ? std::to_string(n.shape[ax]) : std::string("?")) + " does not divide into " + std::to_string(parts) + " parts");
    switch (op.kind) {
      case OpKind::Const: return fail(id, "a constant lies along the split axis");
      case OpKind::Input: return true;
      case OpKind::Iota: return op.axis == ax ? fail(id, "counts along the split axis") : true;
      case OpKind::RandUniform: return fail(id, "draws depend on the absolute element index");
      case OpKind::Cast: case OpKind::Bitcast: case OpKind::Detach:
      case OpKind::Add: case OpKind::Mul: case OpKind::Max: case OpKind::Neg: case OpKind::IDiv: case OpKind::And: case OpKind::Or: case OpKind::Xor:
      case OpKind::Shl: case OpKind::Shr: case OpKind::CmpLt: case OpKind::CmpEq: case OpKind::Where:
      case OpKind::Recip: case OpKind::Sqrt: case OpKind::Exp2: case OpKind::Log2: case OpKind::Sin: case OpKind::Floor:
        for (NodeId s : n.src) if (g.shape(s) != n.shape) return fail(id, "operand shape differs from the result's");
        return all(id, a);
      case OpKind::Sum: case OpKind::Prod: case OpKind::ReduceMax: case OpKind::ArgReduce:
        return want(id, n.src[0], static_cast<int>(ax < op.axis ? ax : ax + 1));
      case OpKind::Softmax: case OpKind::RmsNorm:
        if (op.axis == ax) return fail(id, "normalises along the split axis");
        return want(id, n.src[0], a);
      case OpKind::Sdpa:
        if (ax + 2 >= n.shape.size()) return fail(id, "attention separates over its batch axes only");
        return all(id, a);
      case OpKind::Reshape: {
        const Shape& in = g.shape(n.src[0]);
        size_t outer = 1;
        for (size_t d = 0; d < ax; ++d) outer *= n.shape[d];
        size_t acc = 1;
        for (size_t d = 0; d < in.size(); ++d) {
          if (acc == outer && in[d] % parts == 0 && in[d] > 1) {
            // the part's elements must be one contiguous run of the source axis: everything after it has the same extent
            size_t in_inner = 1, out_inner = 1;
            for (size_t e = d + 1; e < in.size(); ++e) in_inner *= in[e];
            for (size_t e = ax + 1; e < n.shape.size(); ++e) out_inner *= n.shape[e];
            if ((in[d] / parts) * in_inner == (n.shape[ax] / parts) * out_inner) return want(id, n.src[0], static_cast<int>(d));
          }
          acc *= in[d];
        }
        return fail(id, "the split axis does not map onto one axis of the operand");
      }
      case OpKind::Permute: return want(id, n.src[0], static_cast<int>(op.perm[ax]));
      case OpKind::Expand: {
        const Shape& in = g.shape(n.src[0]);
        if (in.size() != n.shape.size()) return fail(id, "rank changes");
        if (in[ax] == 1 && n.shape[ax] != 1) return want(id, n.src[0], kWhole);
        return want(id, n.src[0], a);
      }
      case OpKind::Slice:
        if (!(op.ranges[ax][0] == 0 && op.ranges[ax][1] == g.shape(n.src[0])[ax] && op.ranges[ax][2] == 1)) return fail(id, "cuts the split axis");
        return want(id, n.src[0], a);
      case OpKind::Flip:
        for (size_t f : op.perm) if (f == ax) return fail(id, "reverses the split axis");
        return want(id, n.src[0], a);
      case OpKind::Pad:
        if (op.ranges[ax][0] != 0 || op.ranges[ax][1] != 0) return fail(id, "pads the split axis");
        return want(id, n.src[0], a);
      case OpKind::DotGeneral: {
        const size_t nb = op.lb.size();
        const auto lf = free_axes(g.shape(n.src[0]).size(), op.lb, op.lc), rf = free_axes(g.shape(n.src[1]).size(), op.rb, op.rc);
        if (ax < nb) return want(id, n.src[0], static_cast<int>(op.lb[ax])) && want(id, n.src[1], static_cast<int>(op.rb[ax]));
        if (ax < nb + lf.size()) return want(id, n.src[0], static_cast<int>(lf[ax - nb])) && want(id, n.src[1], kWhole);
        return want(id, n.src[0], kWhole) && want(id, n.src[1], static_cast<int>(rf[ax - nb - lf.size()]));
      }
      case OpKind::Gather: {   // out = operand[..axis] ++ indices.shape ++ operand[axis+1..]
        const size_t ir = g.shape(n.src[1]).size();
        if (ax < op.axis) return want(id, n.src[0], a) && want(id, n.src[1], kWhole);
        if (ax < op.axis + ir) return want(id, n.src[0], kWhole) && want(id, n.src[1], static_cast<int>(ax - op.axis));
        return want(id, n.src[0], static_cast<int>(ax - ir + 1)) && want(id, n.src[1], kWhole);
      }
      case OpKind::GatherAlong:
        if (ax == op.axis) return want(id, n.src[0], kWhole) && want(id, n.src[1], a);
        return all(id, a);
      case OpKind::Scatter: {
        if (ax == op.axis) return fail(id, "scatters along the split axis");
        const size_t ir = g.shape(n.src[1]).size();
        return want(id, n.src[0], a) && want(id, n.src[1], kWhole) && want(id, n.src[2], static_cast<int>(ax < op.axis ? ax : ax + ir - 1));
      }
      case OpKind::ScatterAlong:
        if (ax == op.axis) return fail(id, "scatters along the split axis");
        return all(id, a);
      case OpKind::Argsort:
        if (ax == op.axis) return fail(id, "sorts along the split axis");
        return want(id, n.src[0], a);
      case OpKind::QuantMatmul:
        if (ax != 0) return fail(id, "separates over activation rows only");
        if (!want(id, n.src[0], 0)) return false;
        for (size_t i = 1; i < n.src.size(); ++i) if (!want(id, n.src[i], kWhole)) return false;
        return true;
    }
    return fail(id, "not handled");
  }
};
}  // namespace

bool row_split(const Graph& g, NodeId root, size_t parts, SplitPlan* out, std::string* why) {
  auto no = [&](const std::string& m) { if (why) *why = m; return false; };
  if (parts < 1) return no("parts must be at least 1");
  const Node& rn = g.node(root);
  if (rn.shape.empty() || rn.shape[0] == 0 || rn.shape[0] % parts != 0) return no("the root's first extent does not divide into " + std::to_string(parts) + " parts");
  const std::vector<NodeId> order = reachable(g, {root});
  Walk w{g, parts, {}, {}};
  w.axis[root] = 0;
  for (size_t i = order.size(); i-- > 0;)   // consumers before their operands
    if (!w.visit(order[i])) return no(w.why);

  // record the part graph: same ops, the extents along each node's split axis divided by `parts`
  SplitPlan plan;
  plan.parts = parts;
  std::unordered_map<NodeId, NodeId> map;
  for (NodeId id : order) {
    const Node& n = g.node(id);
    const int a = w.axis.at(id);
    Op op = n.op;
    Shape want_shape = n.shape;
    if (a >= 0) want_shape[static_cast<size_t>(a)] /= parts;
    switch (op.kind) {
      case OpKind::Input: case OpKind::Iota: case OpKind::Reshape: case OpKind::Expand: op.shape = want_shape; break;
      case OpKind::Slice: if (a >= 0) op.ranges[static_cast<size_t>(a)][1] = want_shape[static_cast<size_t>(a)]; break;
      default: break;
    }
    std::vector<NodeId> src;
    for (NodeId s : n.src) src.push_back(map.at(s));
    const NodeId nid = plan.graph.push(std::move(op), std::move(src));
    if (plan.graph.shape(nid) != want_shape || plan.graph.dtype(nid) != n.dtype)
      return no(std::string(op_name(n.op.kind)) + " (node " + std::to_string(id) + "): part shape " + shape_str(plan.graph.shape(nid)) + " is not the expected " + shape_str(want_shape));
    map[id] = nid;
    if (n.op.kind == OpKind::Input) plan.inputs.push_back({id, nid, a});
  }
  std::sort(plan.inputs.begin(), plan.inputs.end(), [](const SplitInput& x, const SplitInput& y) { return x.orig < y.orig; });
  plan.root = map.at(root);
  *out = std::move(plan);
  return true;
}

}  // namespace ku
