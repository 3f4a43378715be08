#include "serialize.h"

#include <cstring>
#include <limits>
#include <unordered_map>

namespace ku {

namespace {
constexpr char kMagic[4] = {'K', 'G', 'P', 'H'};
constexpr uint8_t kVersion = 2;

// the reference's op tags (kurumi_core/src/graph/serialize/encode/op.rs:10-169) for the primitives of this library
struct TagRow { OpKind kind; uint8_t tag; };
constexpr TagRow kTags[] = {
    {OpKind::Const, 0},   {OpKind::Input, 1},   {OpKind::Iota, 2},      {OpKind::RandUniform, 3}, {OpKind::Cast, 4},     {OpKind::Bitcast, 5},
    {OpKind::Detach, 6},  {OpKind::Add, 7},     {OpKind::Mul, 8},       {OpKind::Max, 9},         {OpKind::Neg, 10},     {OpKind::IDiv, 11},
    {OpKind::And, 12},    {OpKind::Or, 13},     {OpKind::Xor, 14},      {OpKind::Shl, 15},        {OpKind::Shr, 16},     {OpKind::CmpLt, 17},
    {OpKind::CmpEq, 18},  {OpKind::Where, 19},  {OpKind::Recip, 20},    {OpKind::Sqrt, 21},       {OpKind::Exp2, 22},    {OpKind::Log2, 23},
    {OpKind::Sin, 24},    {OpKind::Floor, 25},  {OpKind::Sum, 26},      {OpKind::Prod, 27},       {OpKind::ReduceMax, 28}, {OpKind::Softmax, 30},
    {OpKind::RmsNorm, 31}, {OpKind::Sdpa, 32},  {OpKind::Reshape, 33},  {OpKind::Permute, 34},    {OpKind::Expand, 35},  {OpKind::Slice, 36},
    {OpKind::Flip, 37},   {OpKind::Pad, 38},    {OpKind::DotGeneral, 39}, {OpKind::QuantMatmul, 40}, {OpKind::ArgReduce, 29},
    {OpKind::Gather, 50}, {OpKind::Scatter, 51}, {OpKind::GatherAlong, 52}, {OpKind::ScatterAlong, 53}, {OpKind::Argsort, 54},
};
uint8_t tag_of(OpKind k) {
  for (const TagRow& r : kTags) if (r.kind == k) return r.tag;
  throw Error::shape("serialize_graph", std::string("no wire tag for ") + op_name(k));
}
bool kind_of(uint8_t tag, OpKind* k) {
  for (const TagRow& r : kTags) if (r.tag == tag) { *k = r.kind; return true; }
  return false;
}

// ---- writer ---------------------------------------------------------------------------------------
struct Writer {
  std::vector<uint8_t> o;
  void u8(uint8_t v) { o.push_back(v); }
  void u32(uint32_t v) { for (int i = 0; i < 4; ++i) o.push_back(static_cast<uint8_t>(v >> (8 * i))); }
  void u64(uint64_t v) { for (int i = 0; i < 8; ++i) o.push_back(static_cast<uint8_t>(v >> (8 * i))); }
  void f32(float v) { uint32_t b; std::memcpy(&b, &v, 4); u32(b); }
  void vec(const std::vector<size_t>& v) { u32(static_cast<uint32_t>(v.size())); for (size_t x : v) u64(x); }
  void str(const std::string& s) { u32(static_cast<uint32_t>(s.size())); o.insert(o.end(), s.begin(), s.end()); }
  void dtype(DType d) { u8(static_cast<uint8_t>(d)); }
};

void write_op(Writer& w, const Op& op) {
  w.u8(tag_of(op.kind));
  switch (op.kind) {
    case OpKind::Const:
      w.dtype(op.data->dtype);
      w.u64(op.data->bytes.size());
      w.o.insert(w.o.end(), op.data->bytes.begin(), op.data->bytes.end());
      w.vec(op.shape);
      break;
    case OpKind::Input: w.vec(op.shape); w.dtype(op.to); break;
    case OpKind::Iota: w.vec(op.shape); w.u64(op.axis); w.dtype(op.to); break;
    case OpKind::RandUniform: w.vec(op.shape); break;
    case OpKind::Cast: case OpKind::Bitcast: w.dtype(op.to); break;
    case OpKind::Sum: case OpKind::Prod: case OpKind::ReduceMax: case OpKind::Softmax: w.u64(op.axis); break;
    case OpKind::ArgReduce: w.u64(op.axis); w.u8(op.arg_min ? 1 : 0); break;
    case OpKind::Gather: case OpKind::GatherAlong: w.u64(op.axis); break;
    case OpKind::Scatter: case OpKind::ScatterAlong: w.u64(op.axis); w.u8(op.combine); break;
    case OpKind::Argsort: w.u64(op.axis); w.u8(op.descending ? 1 : 0); break;
    case OpKind::RmsNorm: w.u64(op.axis); w.f32(op.eps); break;
    case OpKind::Sdpa: w.u8(op.causal ? 1 : 0); break;
    case OpKind::Reshape: case OpKind::Expand: w.vec(op.shape); break;
    case OpKind::Permute: case OpKind::Flip: w.vec(op.perm); break;
    case OpKind::Slice:
      w.u32(static_cast<uint32_t>(op.ranges.size()));
      for (auto& r : op.ranges) { w.u64(r[0]); w.u64(r[1]); w.u64(r[2]); }
      break;
    case OpKind::Pad:
      w.u32(static_cast<uint32_t>(op.ranges.size()));
      for (auto& r : op.ranges) { w.u64(r[0]); w.u64(r[1]); }
      break;
    case OpKind::DotGeneral: w.vec(op.lc); w.vec(op.rc); w.vec(op.lb); w.vec(op.rb); break;
    case OpKind::QuantMatmul: w.u8(op.bits); w.u64(op.group_size); w.u8(op.symmetric ? 1 : 0); break;
    default: break;   // attribute-free primitives
  }
}

// nodes listed in `order` (already topological) are written with ids renumbered to their position
std::vector<uint8_t> write_blob(const Graph& g, const std::vector<NodeId>& order, const std::vector<Entry>& entries, bool drop_unreachable_inputs) {
  std::unordered_map<NodeId, uint32_t> remap;
  for (size_t i = 0; i < order.size(); ++i) remap[order[i]] = static_cast<uint32_t>(i);
  auto id_of = [&](NodeId n, const char* what) {
    auto it = remap.find(n);
    if (it == remap.end()) throw Error::shape("serialize_graph", std::string(what) + " node " + std::to_string(n) + " is not part of the written graph");
    return it->second;
  };
  Writer w;
  w.o.insert(w.o.end(), kMagic, kMagic + 4);
  w.u8(kVersion);
  w.u32(static_cast<uint32_t>(order.size()));
  for (NodeId n : order) {
    const Node& node = g.node(n);
    write_op(w, node.op);
    w.u32(static_cast<uint32_t>(node.src.size()));
    for (NodeId s : node.src) w.u32(id_of(s, "source"));
  }
  w.u32(static_cast<uint32_t>(entries.size()));
  for (const Entry& e : entries) {
    w.str(e.name);
    w.u32(static_cast<uint32_t>(e.outputs.size()));
    for (NodeId o : e.outputs) w.u32(id_of(o, "output"));
    std::vector<const InputBinding*> kept;
    for (const InputBinding& b : e.inputs) {
      if (remap.count(b.node)) kept.push_back(&b);
      else if (!drop_unreachable_inputs) (void)id_of(b.node, "input");
    }
    w.u32(static_cast<uint32_t>(kept.size()));
    for (const InputBinding* b : kept) {
      if (b->role > 1) throw Error::shape("serialize_graph", "bad input role " + std::to_string(b->role));
      w.u32(remap[b->node]);
      w.u8(b->role);
      w.str(b->name);
    }
  }
  return std::move(w.o);
}

// ---- reader ---------------------------------------------------------------------------------------
Error bad(const std::string& msg) { return Error::shape("deserialize_graph", msg); }

struct Reader {
  const uint8_t* p;
  size_t len, pos = 0;
  const uint8_t* take(size_t n) {
    if (n > len - pos) throw bad("unexpected end of graph blob");
    const uint8_t* s = p + pos;
    pos += n;
    return s;
  }
  uint8_t u8() { return take(1)[0]; }
  uint32_t u32() { const uint8_t* s = take(4); return static_cast<uint32_t>(s[0]) | (static_cast<uint32_t>(s[1]) << 8) | (static_cast<uint32_t>(s[2]) << 16) | (static_cast<uint32_t>(s[3]) << 24); }
  uint64_t u64() { uint64_t lo = u32(); uint64_t hi = u32(); return lo | (hi << 32); }
  size_t usize() {
    const uint64_t v = u64();
    if (v > std::numeric_limits<size_t>::max() / 2) throw bad("size field out of range");
    return static_cast<size_t>(v);
  }
  float f32() { uint32_t b = u32(); float v; std::memcpy(&v, &b, 4); return v; }
  // a count of items that each take at least `min_item_bytes`: bounded by what is left in the blob
  size_t count(size_t min_item_bytes) {
    const size_t n = u32();
    if (min_item_bytes && n > (len - pos) / min_item_bytes) throw bad("unexpected end of graph blob");
    return n;
  }
  std::vector<size_t> vec() { const size_t n = count(8); std::vector<size_t> v(n); for (auto& x : v) x = usize(); return v; }
  std::string str() {
    const size_t n = count(1);
    const uint8_t* s = take(n);
    std::string out(reinterpret_cast<const char*>(s), n);
    // names are UTF-8: reject byte sequences that are not
    for (size_t i = 0; i < n;) {
      const unsigned char c = static_cast<unsigned char>(out[i]);
      const size_t extra = c < 0x80 ? 0 : (c >> 5) == 0x6 ? 1 : (c >> 4) == 0xE ? 2 : (c >> 3) == 0x1E ? 3 : 4;
      if (extra == 4 || extra > n - 1 - i) throw bad("invalid utf8 in name");
      for (size_t k = 1; k <= extra; ++k)
        if ((static_cast<unsigned char>(out[i + k]) >> 6) != 0x2) throw bad("invalid utf8 in name");
      i += extra + 1;
    }
    return out;
  }
  DType dtype() {
    const uint8_t t = u8();
    if (t > 16) throw bad("unknown dtype tag " + std::to_string(t));
    return static_cast<DType>(t);
  }
};

// total element count of a shape, refusing overflow
size_t checked_numel(const Shape& s) {
  size_t n = 1;
  for (size_t d : s) {
    if (d != 0 && n > (std::numeric_limits<size_t>::max() / 16) / d) throw bad("shape " + shape_str(s) + " is too large");
    n *= d;
  }
  return n;
}

// reads one node and appends it through the checked builders, so that a hostile blob produces an error
NodeId read_node(Reader& r, Graph& g, size_t index) {
  const uint8_t tag = r.u8();
  OpKind kind;
  if (!kind_of(tag, &kind)) throw bad("op tag " + std::to_string(tag) + " is not a primitive this backend evaluates");
  // attributes
  Op op;
  op.kind = kind;
  Tensor payload;
  std::vector<std::array<size_t, 2>> pads;
  switch (kind) {
    case OpKind::Const: {
      payload.dtype = r.dtype();
      const size_t nbytes = r.usize();
      const uint8_t* bytes = r.take(nbytes);
      payload.shape = r.vec();
      const size_t want = checked_numel(payload.shape), width = dtype_width(payload.dtype);
      if (nbytes != want * width) throw bad("Const payload has " + std::to_string(nbytes / width) + " elements, shape " + shape_str(payload.shape) + " needs " + std::to_string(want));
      payload.bytes.assign(bytes, bytes + nbytes);
      break;
    }
    case OpKind::Input: op.shape = r.vec(); op.to = r.dtype(); checked_numel(op.shape); break;
    case OpKind::Iota: op.shape = r.vec(); op.axis = r.usize(); op.to = r.dtype(); checked_numel(op.shape); break;
    case OpKind::RandUniform: op.shape = r.vec(); checked_numel(op.shape); break;
    case OpKind::Cast: case OpKind::Bitcast: op.to = r.dtype(); break;
    case OpKind::Sum: case OpKind::Prod: case OpKind::ReduceMax: case OpKind::Softmax: op.axis = r.usize(); break;
    case OpKind::ArgReduce: {
      op.axis = r.usize();
      const uint8_t kind = r.u8();
      if (kind > 1) throw bad("unknown argkind " + std::to_string(kind));
      op.arg_min = kind == 1;
      break;
    }
    case OpKind::Gather: case OpKind::GatherAlong: op.axis = r.usize(); break;
    case OpKind::Scatter: case OpKind::ScatterAlong:
      op.axis = r.usize();
      op.combine = r.u8();
      if (op.combine > 3) throw bad("unknown scatter combiner " + std::to_string(op.combine));
      break;
    case OpKind::Argsort: op.axis = r.usize(); op.descending = r.u8() != 0; break;
    case OpKind::RmsNorm: op.axis = r.usize(); op.eps = r.f32(); break;
    case OpKind::Sdpa: op.causal = r.u8() != 0; break;
    case OpKind::Reshape: case OpKind::Expand: op.shape = r.vec(); checked_numel(op.shape); break;
    case OpKind::Permute: case OpKind::Flip: op.perm = r.vec(); break;
    case OpKind::Slice: {
      const size_t n = r.count(24);
      for (size_t i = 0; i < n; ++i) { const size_t a = r.usize(), b = r.usize(), c = r.usize(); op.ranges.push_back({a, b, c}); }
      break;
    }
    case OpKind::Pad: {
      const size_t n = r.count(16);
      for (size_t i = 0; i < n; ++i) { const size_t lo = r.usize(), hi = r.usize(); pads.push_back({lo, hi}); }
      break;
    }
    case OpKind::DotGeneral: op.lc = r.vec(); op.rc = r.vec(); op.lb = r.vec(); op.rb = r.vec(); break;
    case OpKind::QuantMatmul: op.bits = r.u8(); op.group_size = r.usize(); op.symmetric = r.u8() != 0; break;
    default: break;
  }
  // sources: each must already exist
  const size_t ns = r.count(4);
  std::vector<NodeId> src(ns);
  for (auto& s : src) {
    s = r.u32();
    if (s >= index) throw bad("node " + std::to_string(index) + " references source " + std::to_string(s) + " (not yet built)");
  }
  auto need = [&](size_t n) {
    if (src.size() != n) throw bad(std::string(op_name(kind)) + " node " + std::to_string(index) + " has " + std::to_string(src.size()) + " sources, needs " + std::to_string(n));
  };
  NodeId id = 0;
  switch (kind) {
    case OpKind::Const: need(0); id = g.constant(std::move(payload)); break;
    case OpKind::Input: need(0); id = g.input(op.shape, op.to); break;
    case OpKind::Iota: need(0); id = g.iota(op.shape, op.axis, op.to); break;
    case OpKind::RandUniform: need(1); id = g.rand_uniform_keyed(op.shape, src[0]); break;
    case OpKind::Cast: need(1); id = g.cast(src[0], op.to); break;
    case OpKind::Bitcast: need(1); id = g.bitcast(src[0], op.to); break;
    case OpKind::Detach: need(1); id = g.detach(src[0]); break;
    case OpKind::Add: need(2); id = g.add(src[0], src[1]); break;
    case OpKind::Mul: need(2); id = g.mul(src[0], src[1]); break;
    case OpKind::Max: need(2); id = g.max(src[0], src[1]); break;
    case OpKind::IDiv: need(2); id = g.idiv(src[0], src[1]); break;
    case OpKind::And: need(2); id = g.bit_and(src[0], src[1]); break;
    case OpKind::Or: need(2); id = g.bit_or(src[0], src[1]); break;
    case OpKind::Xor: need(2); id = g.bit_xor(src[0], src[1]); break;
    case OpKind::Shl: need(2); id = g.shl(src[0], src[1]); break;
    case OpKind::Shr: need(2); id = g.shr(src[0], src[1]); break;
    case OpKind::CmpLt: need(2); id = g.cmp_lt(src[0], src[1]); break;
    case OpKind::CmpEq: need(2); id = g.cmp_eq(src[0], src[1]); break;
    case OpKind::Where: need(3); id = g.select(src[0], src[1], src[2]); break;
    case OpKind::Neg: need(1); id = g.neg(src[0]); break;
    case OpKind::Recip: need(1); id = g.recip(src[0]); break;
    case OpKind::Sqrt: need(1); id = g.sqrt(src[0]); break;
    case OpKind::Exp2: need(1); id = g.exp2(src[0]); break;
    case OpKind::Log2: need(1); id = g.log2(src[0]); break;
    case OpKind::Sin: need(1); id = g.sin(src[0]); break;
    case OpKind::Floor: need(1); id = g.floor(src[0]); break;
    case OpKind::Sum: need(1); id = g.sum(src[0], op.axis); break;
    case OpKind::Prod: need(1); id = g.prod(src[0], op.axis); break;
    case OpKind::ReduceMax: need(1); id = g.reduce_max(src[0], op.axis); break;
    case OpKind::Softmax: need(1); id = g.softmax(src[0], op.axis); break;
    case OpKind::ArgReduce: need(1); id = op.arg_min ? g.argmin(src[0], op.axis) : g.argmax(src[0], op.axis); break;
    case OpKind::Gather: need(2); id = g.gather(src[0], src[1], op.axis); break;
    case OpKind::GatherAlong: need(2); id = g.gather_along(src[0], src[1], op.axis); break;
    case OpKind::Scatter: need(3); id = g.scatter(src[0], src[1], src[2], op.axis, op.combine); break;
    case OpKind::ScatterAlong: need(3); id = g.scatter_along(src[0], src[1], src[2], op.axis, op.combine); break;
    case OpKind::Argsort: need(1); id = g.argsort(src[0], op.axis, op.descending); break;
    case OpKind::RmsNorm: need(1); id = g.rmsnorm(src[0], op.axis, op.eps); break;
    case OpKind::Sdpa: need(3); id = g.sdpa_fused(src[0], src[1], src[2], op.causal); break;
    case OpKind::Reshape: need(1); id = g.reshape(src[0], op.shape); break;
    case OpKind::Permute: need(1); id = g.permute(src[0], op.perm); break;
    case OpKind::Expand: need(1); id = g.expand(src[0], op.shape); break;
    case OpKind::Slice: need(1); id = g.slice_step(src[0], op.ranges); break;
    case OpKind::Flip: need(1); id = g.flip(src[0], op.perm); break;
    case OpKind::Pad: need(1); id = g.pad(src[0], pads); break;
    case OpKind::DotGeneral: need(2); id = g.dot_general(src[0], src[1], op.lc, op.rc, op.lb, op.rb); break;
    case OpKind::QuantMatmul: need(op.symmetric ? 3 : 4); id = g.quant_matmul(src[0], src[1], src[2], op.symmetric ? nullptr : &src[3], op.bits, op.group_size); break;
  }
  if (id != index || g.size() != index + 1 || g.node(id).op.kind != kind)
    throw bad("node " + std::to_string(index) + " (" + op_name(kind) + ") did not rebuild as one primitive");
  return id;
}
}  // namespace

std::vector<uint8_t> serialize_graph(const Graph& g, const std::vector<NodeId>& outputs, const std::vector<InputBinding>& inputs) {
  std::vector<NodeId> order(g.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = static_cast<NodeId>(i);
  return write_blob(g, order, {Entry{"", outputs, inputs}}, false);
}

std::vector<uint8_t> serialize_reachable(const Graph& g, const std::vector<NodeId>& outputs, const std::vector<InputBinding>& inputs) {
  return write_blob(g, reachable(g, outputs), {Entry{"", outputs, inputs}}, true);
}

std::vector<uint8_t> serialize_multi(const Graph& g, const std::vector<Entry>& entries) {
  std::vector<NodeId> roots;
  for (const Entry& e : entries) roots.insert(roots.end(), e.outputs.begin(), e.outputs.end());
  return write_blob(g, reachable(g, roots), entries, true);
}

Runnable deserialize_graph(const uint8_t* bytes, size_t len) {
  if (!bytes && len) throw bad("null blob");
  Reader r{bytes, len};
  if (len < 4 || std::memcmp(r.take(4), kMagic, 4) != 0) throw bad("bad magic (not a KGPH graph blob)");
  const uint8_t ver = r.u8();
  if (ver != kVersion) throw bad("unsupported graph blob version " + std::to_string(ver));
  const size_t n = r.count(5);   // a node is at least a tag and a source count
  Runnable out;
  out.graph = std::make_unique<Graph>();
  for (size_t i = 0; i < n; ++i) read_node(r, *out.graph, i);
  const size_t ne = r.count(12);
  for (size_t e = 0; e < ne; ++e) {
    Entry entry;
    entry.name = r.str();
    const size_t no = r.count(4);
    for (size_t i = 0; i < no; ++i) {
      const NodeId o = r.u32();
      if (o >= n) throw bad("entry output " + std::to_string(o) + " is not a node of the blob");
      entry.outputs.push_back(o);
    }
    const size_t ni = r.count(9);
    for (size_t i = 0; i < ni; ++i) {
      InputBinding b;
      b.node = r.u32();
      if (b.node >= n) throw bad("entry input " + std::to_string(b.node) + " is not a node of the blob");
      b.role = r.u8();
      if (b.role > 1) throw bad("bad input role " + std::to_string(b.role));
      b.name = r.str();
      entry.inputs.push_back(std::move(b));
    }
    out.entries.push_back(std::move(entry));
  }
  if (out.entries.empty()) throw bad("graph blob has no entries");
  return out;
}

}  // namespace ku
