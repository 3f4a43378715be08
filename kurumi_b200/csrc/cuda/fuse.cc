#include "fuse.h"

namespace ku::cu {

int add_leaf(Fused& f, const Leaf& l) {
  for (size_t i = 0; i < f.leaves.size(); ++i)
    if (f.leaves[i].same(l)) return static_cast<int>(i);
  f.leaves.push_back(l);
  return static_cast<int>(f.leaves.size()) - 1;
}

int add_node(Fused& f, const FNode& n) {
  for (size_t i = 0; i < f.nodes.size(); ++i) {
    const FNode& m = f.nodes[i];
    if (m.op == n.op && m.dtype == n.dtype && m.leaf == n.leaf && m.in[0] == n.in[0] && m.in[1] == n.in[1] && m.in[2] == n.in[2])
      return static_cast<int>(i);
  }
  f.nodes.push_back(n);
  return static_cast<int>(f.nodes.size()) - 1;
}

int import_expr(Fused& dst, const Fused& src, int node) {
  std::vector<int> map(src.nodes.size(), -1);
  std::vector<bool> need(src.nodes.size(), false);
  need[static_cast<size_t>(node)] = true;
  for (size_t i = src.nodes.size(); i-- > 0;)
    if (need[i]) for (int k = 0; k < 3; ++k) if (src.nodes[i].in[k] >= 0) need[static_cast<size_t>(src.nodes[i].in[k])] = true;
  for (size_t i = 0; i < src.nodes.size(); ++i) {
    if (!need[i]) continue;
    FNode n = src.nodes[i];
    if (n.op == OpKind::Input) n.leaf = add_leaf(dst, src.leaves[static_cast<size_t>(n.leaf)]);
    for (int k = 0; k < 3; ++k) if (n.in[k] >= 0) n.in[k] = map[static_cast<size_t>(n.in[k])];
    map[i] = add_node(dst, n);
  }
  return map[static_cast<size_t>(node)];
}

Fused fused_leaf(const Shape& shape, const Leaf& l) {
  Fused f;
  f.shape = shape;
  FNode n;
  n.op = OpKind::Input;
  n.dtype = l.dtype;
  n.leaf = add_leaf(f, l);
  f.root = add_node(f, n);
  return f;
}

}  // namespace ku::cu
