// extern "C" exports of include/kurumi.h. Behaviour follows kurumi/src/capi.rs (handles, last
// error, guard), kurumi/src/capi/eval.rs:9-146 (backend, eval, feeds), kurumi/src/capi/tensor.rs
// (tensor IO) and the builder wrappers under kurumi/src/capi/ops/**: null handles and bad node
// ids never crash, builders return KU_ERR, evals return NULL / -1, and the message is readable
// through ku_last_error() until the next failing call on the same thread.
#include "../../../include/kurumi.h"

#include <cstring>

#include "handles.h"
#include "../core/split.h"

using namespace ku;

namespace ku {
static thread_local std::string g_last_err;
static thread_local bool g_has_err = false;
void set_err(const std::string& msg) { g_last_err = msg; g_has_err = true; }
}  // namespace ku

namespace {
Shape to_shape(const size_t* p, size_t n) { return (p && n) ? Shape(p, p + n) : Shape{}; }
std::vector<size_t> to_vec(const size_t* p, size_t n) { return to_shape(p, n); }

bool dtype_from_u32(uint32_t u, DType* out) {
  if (u >= kNumDTypes) return false;
  *out = static_cast<DType>(u);
  return true;
}

template <typename F>
KuNode build(KuGraph* g, F&& f) {
  if (!g) { set_err("null graph handle"); return KU_ERR; }
  return guard<KuNode>(KU_ERR, [&]() -> KuNode { return f(g->g); });
}
}  // namespace

extern "C" {
KuNode ku_sdpa_fused(KuGraph* g, KuNode q, KuNode k, KuNode v, uint32_t causal);
KuNode ku_sdpa_decomposed(KuGraph* g, KuNode q, KuNode k, KuNode v, uint32_t causal);

const char* ku_last_error(void) { return g_has_err ? g_last_err.c_str() : nullptr; }

KuGraph* ku_graph_new(void) { return new KuGraph(); }
void ku_graph_free(KuGraph* g) { delete g; }

KuNode ku_input(KuGraph* g, const size_t* shape, size_t rank, uint32_t dtype) {
  return build(g, [&](Graph& gr) -> KuNode {
    DType dt;
    if (!dtype_from_u32(dtype, &dt)) throw Error("ku_input: bad dtype " + std::to_string(dtype));
    return gr.input(to_shape(shape, rank), dt);
  });
}
KuNode ku_constant_f32(KuGraph* g, const float* data, size_t len, const size_t* shape, size_t rank) {
  return build(g, [&](Graph& gr) -> KuNode {
    if (!data && len) throw Error("ku_constant_f32: null data");
    return gr.constant(Tensor::from_f32(data, len, to_shape(shape, rank)));
  });
}
KuNode ku_constant(KuGraph* g, uint32_t dtype, const uint8_t* data, size_t nbytes, const size_t* shape, size_t rank) {
  return build(g, [&](Graph& gr) -> KuNode {
    DType dt;
    if (!dtype_from_u32(dtype, &dt)) throw Error("ku_constant: bad dtype " + std::to_string(dtype));
    if (!data && nbytes) throw Error("ku_constant: null data");
    Tensor t;
    t.dtype = dt;
    t.shape = to_shape(shape, rank);
    t.bytes.assign(data, data + nbytes);
    if (dt == DType::BOOL) for (auto& b : t.bytes) b = b ? 1 : 0;
    return gr.constant(std::move(t));
  });
}
KuNode ku_scalar(KuGraph* g, KuNode like, float v) { return build(g, [&](Graph& gr) { return gr.scalar(like, v); }); }

#define KU_BIN(name, method) \
  KuNode name(KuGraph* g, KuNode a, KuNode b) { return build(g, [&](Graph& gr) { return gr.method(a, b); }); }
#define KU_UN(name, method) \
  KuNode name(KuGraph* g, KuNode x) { return build(g, [&](Graph& gr) { return gr.method(x); }); }
#define KU_AXIS(name, method) \
  KuNode name(KuGraph* g, KuNode x, size_t axis) { return build(g, [&](Graph& gr) { return gr.method(x, axis); }); }

KU_BIN(ku_add, add) KU_BIN(ku_sub, sub) KU_BIN(ku_mul, mul) KU_BIN(ku_div, div) KU_BIN(ku_max, max) KU_BIN(ku_min, min)
KU_BIN(ku_idiv, idiv) KU_BIN(ku_and, bit_and) KU_BIN(ku_or, bit_or) KU_BIN(ku_xor, bit_xor) KU_BIN(ku_shl, shl)
KU_BIN(ku_shr, shr) KU_BIN(ku_lt, cmp_lt) KU_BIN(ku_eq, cmp_eq) KU_BIN(ku_le, le) KU_BIN(ku_gt, gt) KU_BIN(ku_ge, ge)
KU_BIN(ku_ne, ne)

KU_UN(ku_neg, neg) KU_UN(ku_recip, recip) KU_UN(ku_sqrt, sqrt) KU_UN(ku_square, square) KU_UN(ku_abs, abs)
KU_UN(ku_floor, floor) KU_UN(ku_exp, exp) KU_UN(ku_exp2, exp2) KU_UN(ku_ln, ln) KU_UN(ku_log2, log2) KU_UN(ku_sin, sin)
KU_UN(ku_cos, cos) KU_UN(ku_relu, relu) KU_UN(ku_gelu, gelu) KU_UN(ku_silu, silu) KU_UN(ku_sigmoid, sigmoid)
KU_UN(ku_tanh, tanh) KU_UN(ku_logical_not, logical_not) KU_UN(ku_detach, detach)

KU_AXIS(ku_sum, sum) KU_AXIS(ku_prod, prod) KU_AXIS(ku_mean, mean) KU_AXIS(ku_reduce_max, reduce_max)
KU_AXIS(ku_reduce_min, reduce_min) KU_AXIS(ku_softmax, softmax) KU_AXIS(ku_argmax, argmax) KU_AXIS(ku_argmin, argmin)

KuNode ku_rmsnorm(KuGraph* g, KuNode x, size_t axis, float eps) { return build(g, [&](Graph& gr) { return gr.rmsnorm(x, axis, eps); }); }
KuNode ku_clamp_min(KuGraph* g, KuNode x, float v) { return build(g, [&](Graph& gr) { return gr.clamp_min(x, v); }); }

KuNode ku_matmul(KuGraph* g, KuNode a, KuNode b) { return build(g, [&](Graph& gr) { return gr.dot_general(a, b, {1}, {0}, {}, {}); }); }
KuNode ku_dot_general(KuGraph* g, KuNode a, KuNode b, const size_t* lc, size_t nlc, const size_t* rc, size_t nrc,
                      const size_t* lb, size_t nlb, const size_t* rb, size_t nrb) {
  return build(g, [&](Graph& gr) { return gr.dot_general(a, b, to_vec(lc, nlc), to_vec(rc, nrc), to_vec(lb, nlb), to_vec(rb, nrb)); });
}
KuNode ku_where(KuGraph* g, KuNode cond, KuNode a, KuNode b) { return build(g, [&](Graph& gr) { return gr.select(cond, a, b); }); }

KuNode ku_reshape(KuGraph* g, KuNode x, const size_t* shape, size_t rank) { return build(g, [&](Graph& gr) { return gr.reshape(x, to_shape(shape, rank)); }); }
KuNode ku_expand(KuGraph* g, KuNode x, const size_t* shape, size_t rank) { return build(g, [&](Graph& gr) { return gr.expand(x, to_shape(shape, rank)); }); }
KuNode ku_permute(KuGraph* g, KuNode x, const size_t* perm, size_t rank) { return build(g, [&](Graph& gr) { return gr.permute(x, to_vec(perm, rank)); }); }
KuNode ku_transpose(KuGraph* g, KuNode x, size_t i, size_t j) { return build(g, [&](Graph& gr) { return gr.transpose(x, i, j); }); }
KuNode ku_flip(KuGraph* g, KuNode x, const size_t* axes, size_t n) { return build(g, [&](Graph& gr) { return gr.flip(x, to_vec(axes, n)); }); }
KuNode ku_slice(KuGraph* g, KuNode x, const size_t* ranges, size_t rank) {
  return build(g, [&](Graph& gr) -> KuNode {
    if (!ranges && rank) throw Error("ku_slice: null ranges");
    std::vector<std::array<size_t, 2>> r;
    for (size_t d = 0; d < rank; ++d) r.push_back({ranges[2 * d], ranges[2 * d + 1]});
    return gr.slice(x, std::move(r));
  });
}
KuNode ku_slice_step(KuGraph* g, KuNode x, const size_t* ranges, size_t rank) {
  return build(g, [&](Graph& gr) -> KuNode {
    if (!ranges && rank) throw Error("ku_slice_step: null ranges");
    std::vector<std::array<size_t, 3>> r;
    for (size_t d = 0; d < rank; ++d) r.push_back({ranges[3 * d], ranges[3 * d + 1], ranges[3 * d + 2]});
    return gr.slice_step(x, std::move(r));
  });
}
KuNode ku_pad(KuGraph* g, KuNode x, const size_t* pads, size_t rank) {
  return build(g, [&](Graph& gr) -> KuNode {
    if (!pads && rank) throw Error("ku_pad: null pads");
    std::vector<std::array<size_t, 2>> r;
    for (size_t d = 0; d < rank; ++d) r.push_back({pads[2 * d], pads[2 * d + 1]});
    return gr.pad(x, std::move(r));
  });
}
KuNode ku_broadcast_to(KuGraph* g, KuNode x, const size_t* shape, size_t rank) { return build(g, [&](Graph& gr) { return gr.broadcast_to(x, to_shape(shape, rank)); }); }

KuNode ku_iota(KuGraph* g, const size_t* shape, size_t rank, size_t axis, uint32_t dtype) {
  return build(g, [&](Graph& gr) -> KuNode {
    DType dt;
    if (!dtype_from_u32(dtype, &dt)) throw Error("ku_iota: bad dtype " + std::to_string(dtype));
    return gr.iota(to_shape(shape, rank), axis, dt);
  });
}
KuNode ku_cast(KuGraph* g, KuNode x, uint32_t dtype) {
  return build(g, [&](Graph& gr) -> KuNode {
    DType dt;
    if (!dtype_from_u32(dtype, &dt)) throw Error("ku_cast: bad dtype " + std::to_string(dtype));
    return gr.cast(x, dt);
  });
}
KuNode ku_bitcast(KuGraph* g, KuNode x, uint32_t dtype) {
  return build(g, [&](Graph& gr) -> KuNode {
    DType dt;
    if (!dtype_from_u32(dtype, &dt)) throw Error("ku_bitcast: bad dtype " + std::to_string(dtype));
    return gr.bitcast(x, dt);
  });
}
// Graph::sdpa_fused / Graph::sdpa_decomposed of the Rust API (kurumi_core/src/graph/ops/nn/attention.rs:97-133);
// the reference's C header exposes only the auto-selecting ku_sdpa.
KuNode ku_sdpa_fused(KuGraph* g, KuNode q, KuNode k, KuNode v, uint32_t causal) { return build(g, [&](Graph& gr) { return gr.sdpa_fused(q, k, v, causal != 0); }); }
KuNode ku_sdpa_decomposed(KuGraph* g, KuNode q, KuNode k, KuNode v, uint32_t causal) { return build(g, [&](Graph& gr) { return gr.sdpa_decomposed(q, k, v, causal != 0); }); }
KuNode ku_sdpa(KuGraph* g, KuNode q, KuNode k, KuNode v, uint32_t causal) { return build(g, [&](Graph& gr) { return gr.sdpa(q, k, v, causal != 0); }); }

KuNode ku_rand_uniform(KuGraph* g, const size_t* shape, size_t rank, uint64_t seed) { return build(g, [&](Graph& gr) { return gr.rand_uniform(to_shape(shape, rank), seed); }); }
KuNode ku_randn(KuGraph* g, const size_t* shape, size_t rank, uint64_t seed) { return build(g, [&](Graph& gr) { return gr.randn(to_shape(shape, rank), seed); }); }
KuNode ku_rand_range(KuGraph* g, const size_t* shape, size_t rank, uint64_t seed, float lo, float hi) { return build(g, [&](Graph& gr) { return gr.rand_range(to_shape(shape, rank), seed, lo, hi); }); }
KuNode ku_rand_uniform_keyed(KuGraph* g, const size_t* shape, size_t rank, KuNode seed) { return build(g, [&](Graph& gr) { return gr.rand_uniform_keyed(to_shape(shape, rank), seed); }); }

// ---- backend + eval -------------------------------------------------------------------------
KuBackend* ku_backend_new(uint32_t kind) {
  return guard<KuBackend*>(nullptr, [&]() -> KuBackend* {
    std::unique_ptr<Backend> b = make_backend(kind);
    if (!b) return nullptr;
    auto* h = new KuBackend();
    h->b = std::move(b);
    return h;
  });
}
void ku_backend_free(KuBackend* b) { delete b; }

KuTensor* ku_eval(KuGraph* g, KuNode node, const KuBackend* backend) {
  if (!g || !backend) { set_err("ku_eval: null graph/backend handle"); return nullptr; }
  return guard<KuTensor*>(nullptr, [&]() -> KuTensor* {
    Tensor t = backend->b->eval(g->g, node);
    return new KuTensor{std::make_shared<const Tensor>(std::move(t))};
  });
}
KuTensor* ku_eval_with(KuGraph* g, KuNode node, const KuBackend* backend, const KuFeeds* feeds) {
  if (!g || !backend || !feeds) { set_err("ku_eval_with: null graph/backend/feeds handle"); return nullptr; }
  return guard<KuTensor*>(nullptr, [&]() -> KuTensor* {
    Tensor t = backend->b->eval_with(g->g, node, feeds->f);
    return new KuTensor{std::make_shared<const Tensor>(std::move(t))};
  });
}
int32_t ku_eval_many(KuGraph* g, const KuNode* ids, size_t n, const KuBackend* backend, const KuFeeds* feeds, KuTensor** out) {
  if (!g || !backend || !feeds || !out || (!ids && n > 0)) { set_err("ku_eval_many: null graph/backend/feeds/ids/out handle"); return -1; }
  return guard<int32_t>(-1, [&]() -> int32_t {
    std::vector<NodeId> v(ids, ids + n);
    std::vector<Tensor> ts = backend->b->eval_many_with(g->g, v, feeds->f);
    for (size_t i = 0; i < ts.size(); ++i) out[i] = new KuTensor{std::make_shared<const Tensor>(std::move(ts[i]))};
    return 0;
  });
}

// indexing, kurumi.h:245-253
KuNode ku_gather(KuGraph* g, KuNode x, KuNode idx, size_t axis) { return build(g, [&](Graph& gr) { return gr.gather(x, idx, axis); }); }
KuNode ku_gather_along(KuGraph* g, KuNode x, KuNode idx, size_t axis) { return build(g, [&](Graph& gr) { return gr.gather_along(x, idx, axis); }); }
KuNode ku_take_along_dim(KuGraph* g, KuNode x, KuNode idx, size_t axis) { return build(g, [&](Graph& gr) { return gr.gather_along(x, idx, axis); }); }
KuNode ku_sort(KuGraph* g, KuNode x, size_t axis, uint32_t descending) { return build(g, [&](Graph& gr) { return gr.sort(x, axis, descending != 0); }); }
KuNode ku_argsort(KuGraph* g, KuNode x, size_t axis, uint32_t descending) { return build(g, [&](Graph& gr) { return gr.argsort(x, axis, descending != 0); }); }
KuNode ku_scatter(KuGraph* g, KuNode operand, KuNode indices, KuNode updates, size_t axis, uint32_t combine) {
  return build(g, [&](Graph& gr) { if (combine > 3) throw Error("ku_scatter: bad combine " + std::to_string(combine)); return gr.scatter(operand, indices, updates, axis, static_cast<uint8_t>(combine)); });
}
KuNode ku_scatter_along(KuGraph* g, KuNode operand, KuNode indices, KuNode updates, size_t axis, uint32_t combine) {
  return build(g, [&](Graph& gr) { if (combine > 3) throw Error("ku_scatter_along: bad combine " + std::to_string(combine)); return gr.scatter_along(operand, indices, updates, axis, static_cast<uint8_t>(combine)); });
}

KuNode ku_quant_matmul(KuGraph* g, KuNode act, KuNode qweight, KuNode scales, KuNode mins, uint8_t bits, size_t group_size) {
  return build(g, [&](Graph& gr) { return gr.quant_matmul(act, qweight, scales, mins == KU_ERR ? nullptr : &mins, bits, group_size); });
}
void ku_quantize(const float* w, size_t rows, size_t cols, uint8_t bits, size_t group_size, uint32_t symmetric, uint8_t* out_packed, uint16_t* out_scales,
                 uint16_t* out_mins) {
  guard<int>(0, [&]() { ku::quantize(w, rows, cols, bits, group_size, symmetric != 0, out_packed, out_scales, out_mins); return 0; });
}
KuNode ku_amp(KuGraph* g, KuNode root) { return build(g, [&](Graph& gr) { return amp(gr, root); }); }
size_t ku_node_count(const KuGraph* g, KuNode root) {
  if (!g) return 0;
  return guard<size_t>(0, [&]() { return reachable(g->g, {root}).size(); });
}
size_t ku_dump(const KuGraph* g, KuNode root, uint8_t* out, size_t cap) {
  if (!g) return 0;
  return guard<size_t>(0, [&]() -> size_t {
    std::string s = dump(g->g, root);
    if (out && cap) std::memcpy(out, s.data(), std::min(cap, s.size()));
    return s.size();
  });
}
size_t ku_node_rank(const KuGraph* g, KuNode node) {
  if (!g) { set_err("null graph handle"); return SIZE_MAX; }
  return guard<size_t>(SIZE_MAX, [&]() { return g->g.shape(node).size(); });
}
void ku_node_shape(const KuGraph* g, KuNode node, size_t* out) {
  if (!g || !out) return;
  guard<int>(0, [&]() { const Shape& s = g->g.shape(node); for (size_t i = 0; i < s.size(); ++i) out[i] = s[i]; return 0; });
}
uint32_t ku_node_dtype(const KuGraph* g, KuNode node) {
  if (!g) { set_err("null graph handle"); return KU_ERR; }
  return guard<uint32_t>(KU_ERR, [&]() { return static_cast<uint32_t>(g->g.dtype(node)); });
}

// ---- runnable-graph blobs (kurumi/src/capi, kurumi.h:407-455) -----------------------------------
namespace {
std::vector<ku::InputBinding> bindings(const KuNode* nodes, const uint8_t* roles, const char* const* names, size_t n) {
  if (n && (!nodes || !roles || !names)) throw ku::Error::shape("ku_graph_serialize", "null input binding arrays");
  std::vector<ku::InputBinding> v(n);
  for (size_t i = 0; i < n; ++i) {
    if (!names[i]) throw ku::Error::shape("ku_graph_serialize", "null input name");
    v[i].node = nodes[i]; v[i].role = roles[i]; v[i].name = names[i];
  }
  return v;
}
size_t write_out(const std::vector<uint8_t>& blob, uint8_t* out, size_t cap) {   // size-then-write
  if (out && cap) std::memcpy(out, blob.data(), std::min(cap, blob.size()));
  return blob.size();
}
size_t write_name(const std::string& s, uint8_t* out, size_t cap) {
  if (out && cap) std::memcpy(out, s.data(), std::min(cap, s.size()));
  return s.size();
}
const ku::Entry* entry_of(const KuRunnable* h, size_t i) { return (h && i < h->r.entries.size()) ? &h->r.entries[i] : nullptr; }
}  // namespace

size_t ku_graph_serialize(const KuGraph* g, const KuNode* outputs, size_t n_out, const KuNode* in_nodes, const uint8_t* in_roles, const char* const* in_names,
                          size_t n_in, uint8_t* out, size_t cap) {
  if (!g || (n_out && !outputs)) { set_err("ku_graph_serialize: null graph/outputs"); return 0; }
  return guard<size_t>(0, [&]() {
    return write_out(ku::serialize_graph(g->g, std::vector<NodeId>(outputs, outputs + n_out), bindings(in_nodes, in_roles, in_names, n_in)), out, cap);
  });
}
size_t ku_graph_serialize_reachable(const KuGraph* g, const KuNode* outputs, size_t n_out, const KuNode* in_nodes, const uint8_t* in_roles,
                                    const char* const* in_names, size_t n_in, uint8_t* out, size_t cap) {
  if (!g || (n_out && !outputs)) { set_err("ku_graph_serialize_reachable: null graph/outputs"); return 0; }
  return guard<size_t>(0, [&]() {
    return write_out(ku::serialize_reachable(g->g, std::vector<NodeId>(outputs, outputs + n_out), bindings(in_nodes, in_roles, in_names, n_in)), out, cap);
  });
}
size_t ku_graph_serialize_multi(const KuGraph* g, size_t n_entries, const char* const* names, const uint32_t* out_counts, const KuNode* outputs,
                                const uint32_t* in_counts, const KuNode* in_nodes, const uint8_t* in_roles, const char* const* in_names, uint8_t* out, size_t cap) {
  if (!g || (n_entries && (!names || !out_counts || !in_counts))) { set_err("ku_graph_serialize_multi: null graph/entry arrays"); return 0; }
  return guard<size_t>(0, [&]() {
    std::vector<ku::Entry> entries(n_entries);
    size_t o = 0, i = 0;
    for (size_t e = 0; e < n_entries; ++e) {
      if (!names[e]) throw ku::Error::shape("ku_graph_serialize_multi", "null entry name");
      if (out_counts[e] && !outputs) throw ku::Error::shape("ku_graph_serialize_multi", "null outputs");
      entries[e].name = names[e];
      entries[e].outputs.assign(outputs + o, outputs + o + out_counts[e]);
      entries[e].inputs = bindings(in_counts[e] ? in_nodes + i : nullptr, in_counts[e] ? in_roles + i : nullptr, in_counts[e] ? in_names + i : nullptr, in_counts[e]);
      o += out_counts[e];
      i += in_counts[e];
    }
    return write_out(ku::serialize_multi(g->g, entries), out, cap);
  });
}
KuRunnable* ku_graph_deserialize(const uint8_t* bytes, size_t len) {
  if (!bytes && len) { set_err("ku_graph_deserialize: null bytes"); return nullptr; }
  return guard<KuRunnable*>(nullptr, [&]() { return new KuRunnable{ku::deserialize_graph(bytes, len)}; });
}
KuGraph* ku_runnable_take_graph(KuRunnable* h) {
  if (!h || !h->r.graph) { set_err("ku_runnable_take_graph: null handle or graph already taken"); return nullptr; }
  return guard<KuGraph*>(nullptr, [&]() {
    KuGraph* g = new KuGraph{std::move(*h->r.graph)};
    h->r.graph.reset();
    return g;
  });
}
size_t ku_runnable_output_count(const KuRunnable* h) { return ku_runnable_entry_output_count(h, 0); }
KuNode ku_runnable_output(const KuRunnable* h, size_t i) { return ku_runnable_entry_output(h, 0, i); }
size_t ku_runnable_input_count(const KuRunnable* h) { return ku_runnable_entry_input_count(h, 0); }
KuNode ku_runnable_input_node(const KuRunnable* h, size_t i) { return ku_runnable_entry_input_node(h, 0, i); }
uint32_t ku_runnable_input_role(const KuRunnable* h, size_t i) { return ku_runnable_entry_input_role(h, 0, i); }
size_t ku_runnable_input_name(const KuRunnable* h, size_t i, uint8_t* out, size_t cap) { return ku_runnable_entry_input_name(h, 0, i, out, cap); }
size_t ku_runnable_entry_count(const KuRunnable* h) { return h ? h->r.entries.size() : 0; }
size_t ku_runnable_entry_name(const KuRunnable* h, size_t i, uint8_t* out, size_t cap) {
  const ku::Entry* e = entry_of(h, i);
  return e ? write_name(e->name, out, cap) : 0;
}
size_t ku_runnable_entry_output_count(const KuRunnable* h, size_t i) { const ku::Entry* e = entry_of(h, i); return e ? e->outputs.size() : 0; }
KuNode ku_runnable_entry_output(const KuRunnable* h, size_t i, size_t j) {
  const ku::Entry* e = entry_of(h, i);
  if (!e || j >= e->outputs.size()) { set_err("ku_runnable_entry_output: index out of range"); return KU_ERR; }
  return e->outputs[j];
}
size_t ku_runnable_entry_input_count(const KuRunnable* h, size_t i) { const ku::Entry* e = entry_of(h, i); return e ? e->inputs.size() : 0; }
KuNode ku_runnable_entry_input_node(const KuRunnable* h, size_t i, size_t j) {
  const ku::Entry* e = entry_of(h, i);
  if (!e || j >= e->inputs.size()) { set_err("ku_runnable_entry_input_node: index out of range"); return KU_ERR; }
  return e->inputs[j].node;
}
uint32_t ku_runnable_entry_input_role(const KuRunnable* h, size_t i, size_t j) {
  const ku::Entry* e = entry_of(h, i);
  if (!e || j >= e->inputs.size()) { set_err("ku_runnable_entry_input_role: index out of range"); return KU_ERR; }
  return e->inputs[j].role;
}
size_t ku_runnable_entry_input_name(const KuRunnable* h, size_t i, size_t j, uint8_t* out, size_t cap) {
  const ku::Entry* e = entry_of(h, i);
  if (!e || j >= e->inputs.size()) return 0;
  return write_name(e->inputs[j].name, out, cap);
}
void ku_runnable_free(KuRunnable* h) { delete h; }

// ---- plan replay (kurumi/src/capi/eval.rs:152-182, kurumi_core/src/realize/plan.rs:13-58) ----------------------
KuPlan* ku_plan_compile(const KuGraph* g, KuNode node) {
  if (!g) { set_err("ku_plan_compile: null graph handle"); return nullptr; }
  return guard<KuPlan*>(nullptr, [&]() -> KuPlan* {
    (void)g->g.node(node);
    std::shared_ptr<ku::Backend> b = ku::plan_backend(g->g, node);
    if (!b) return nullptr;
    return new KuPlan{std::move(b), g->g.id(), node};
  });
}
KuTensor* ku_plan_run(const KuPlan* p, const KuGraph* g, const KuFeeds* feeds) {
  if (!p || !g || !feeds) { set_err("ku_plan_run: null plan/graph/feeds handle"); return nullptr; }
  return guard<KuTensor*>(nullptr, [&]() -> KuTensor* {
    if (g->g.id() != p->graph_id) throw Error("ku_plan_run: the plan was compiled from another graph");
    Tensor t = p->backend->eval_with(g->g, p->node, feeds->f);
    return new KuTensor{std::make_shared<const Tensor>(std::move(t))};
  });
}
void ku_plan_free(KuPlan* p) { delete p; }

// ---- row splitting (core/split.h) ---------------------------------------------------------------
KuGraph* ku_graph_row_split(const KuGraph* g, KuNode root, size_t parts, KuNode* part_root, KuNode* orig_inputs, KuNode* part_inputs, int32_t* axes, size_t cap, size_t* n_inputs) {
  if (!g) { set_err("ku_graph_row_split: null graph handle"); return nullptr; }
  return guard<KuGraph*>(nullptr, [&]() -> KuGraph* {
    ku::SplitPlan plan;
    std::string why;
    if (!ku::row_split(g->g, root, parts, &plan, &why)) { set_err("ku_graph_row_split: " + why); return nullptr; }
    if (part_root) *part_root = plan.root;
    if (n_inputs) *n_inputs = plan.inputs.size();
    for (size_t i = 0; i < plan.inputs.size() && i < cap; ++i) {
      if (orig_inputs) orig_inputs[i] = plan.inputs[i].orig;
      if (part_inputs) part_inputs[i] = plan.inputs[i].part;
      if (axes) axes[i] = plan.inputs[i].axis;
    }
    return new KuGraph{std::move(plan.graph)};
  });
}

// ---- feeds ------------------------------------------------------------------------------------
KuFeeds* ku_feeds_new(void) { return new KuFeeds(); }
void ku_feeds_free(KuFeeds* f) { delete f; }
void ku_feeds_set(KuFeeds* f, KuNode node, const KuTensor* tensor) {
  if (!f || !tensor) return;
  f->f[node] = tensor->t;  // tensors are immutable once built, so sharing the buffer is a copy
}

// ---- tensors ----------------------------------------------------------------------------------
KuTensor* ku_tensor_f32(const float* data, size_t len, const size_t* shape, size_t rank) {
  if (!data && len) { set_err("ku_tensor_f32: null data"); return nullptr; }
  return guard<KuTensor*>(nullptr, [&]() { return new KuTensor{std::make_shared<const Tensor>(Tensor::from_f32(data, len, to_shape(shape, rank)))}; });
}
KuTensor* ku_tensor_new(uint32_t dtype, const uint8_t* data, size_t nbytes, const size_t* shape, size_t rank) {
  DType dt;
  if (!dtype_from_u32(dtype, &dt)) { set_err("ku_tensor_new: bad dtype " + std::to_string(dtype)); return nullptr; }
  if (!data && nbytes) { set_err("ku_tensor_new: null data"); return nullptr; }
  return guard<KuTensor*>(nullptr, [&]() {
    Tensor t;
    t.dtype = dt;
    t.shape = to_shape(shape, rank);
    t.bytes.resize(nbytes);
    ku::HostMem::copy(t.bytes.data(), data, nbytes);
    if (dt == DType::BOOL) for (auto& b : t.bytes) b = b ? 1 : 0;
    return new KuTensor{std::make_shared<const Tensor>(std::move(t))};
  });
}
void ku_tensor_free(KuTensor* t) { delete t; }
size_t ku_tensor_rank(const KuTensor* t) { return t ? t->t->shape.size() : 0; }
void ku_tensor_shape(const KuTensor* t, size_t* out) {
  if (!t || !out) return;
  for (size_t i = 0; i < t->t->shape.size(); ++i) out[i] = t->t->shape[i];
}
size_t ku_tensor_len(const KuTensor* t) { return t ? t->t->len() : 0; }
uint32_t ku_tensor_dtype(const KuTensor* t) { return t ? static_cast<uint32_t>(t->t->dtype) : 0; }
ptrdiff_t ku_tensor_data_f32(const KuTensor* t, float* out, size_t cap) {
  if (!t || !out) return -1;
  if (t->t->dtype != DType::F32) { set_err(std::string("ku_tensor_data_f32: tensor is ") + dtype_name(t->t->dtype) + ", not F32"); return -1; }
  size_t n = std::min(t->t->len(), cap);
  std::memcpy(out, t->t->bytes.data(), n * 4);
  return static_cast<ptrdiff_t>(n);
}
size_t ku_tensor_nbytes(const KuTensor* t) { return t ? t->t->bytes.size() : 0; }
void ku_tensor_bytes(const KuTensor* t, uint8_t* out) {
  if (!t || !out) return;
  ku::HostMem::copy(out, t->t->bytes.data(), t->t->bytes.size());
}

}  // extern "C"
