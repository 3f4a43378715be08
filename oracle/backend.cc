// TEST INFRASTRUCTURE, NOT PRODUCT CODE. The backend factory of the oracle library: the same
// C ABI as the product (include/kurumi.h), evaluated on the CPU by the restated interpreter.
//   kind 0  (KU_CPU)  the reference interpreter, native dtypes (kurumi_core/src/backend.rs:34-46)
//   kind 64           the "f64 interpreter run": float results come back as F64 tensors
//   kind 65           the view-fused f32 evaluator with interpreter fallback (realize::force)
// plus a few exported helpers the tests use to pin the restatement against the reference's
// known answers (threefry KATs, dtype conversions).
#include <cstring>

#include "../kurumi_b200/csrc/capi/handles.h"
#include "interp.h"

namespace {
using namespace ku;
struct Interp : Backend {
  bool wide;
  explicit Interp(bool w) : wide(w) {}
  const char* name() const override { return wide ? "cpu-f64" : "cpu"; }
  Tensor eval_with(const Graph& g, NodeId id, const Feeds& feeds) override { return ko::interpret_many(g, {id}, feeds, wide)[0]; }
  std::vector<Tensor> eval_many_with(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds) override {
    return ko::interpret_many(g, ids, feeds, wide);
  }
};
struct Realize : Backend {
  const char* name() const override { return "cpu-realize"; }
  Tensor eval_with(const Graph& g, NodeId id, const Feeds& feeds) override { return ko::force(g, id, feeds, nullptr); }
};
}  // namespace

namespace ku {
std::unique_ptr<Backend> make_backend(uint32_t kind) {
  switch (kind) {
    case 0: return std::make_unique<Interp>(false);
    case 64: return std::make_unique<Interp>(true);
    case 65: return std::make_unique<Realize>();
    default: set_err("ku_backend_new: unknown kind " + std::to_string(kind)); return nullptr;
  }
}
// kurumi/src/capi/eval.rs:152-168: NULL off the f32 fused path
std::shared_ptr<Backend> plan_backend(const Graph& g, NodeId root) {
  if (!ko::plan_supported(g, root)) { set_err("ku_plan_compile: graph is not on the f32 fused plan path"); return nullptr; }
  return std::make_shared<Realize>();
}
}  // namespace ku

extern "C" {
uint64_t ko_threefry2x32(uint64_t key, uint64_t counter) { return ko::threefry2x32(key, counter); }
float ko_uniform_f32(uint64_t bits) { return ko::uniform_f32(bits); }
// realize::force_counted: evaluates and returns the pass count (-1 = interpreter fallback)
long ko_force_counted(KuGraph* g, uint32_t node, const KuFeeds* feeds, KuTensor** out) {
  return ku::guard<long>(-2, [&]() -> long {
    long k = 0;
    ku::Feeds none;
    ku::Tensor t = ko::force(g->g, node, feeds ? feeds->f : none, &k);
    if (out) *out = new KuTensor{std::make_shared<const ku::Tensor>(std::move(t))};
    return k;
  });
}
// cast `n` elements of dtype `from` to dtype `to` through f64 (dtype/convert.rs:14-47)
void ko_cast(uint32_t from, const uint8_t* src, size_t n, uint32_t to, uint8_t* dst) {
  size_t ws = ku::dtype_width(static_cast<ku::DType>(from)), wd = ku::dtype_width(static_cast<ku::DType>(to));
  for (size_t i = 0; i < n; ++i) ku::f64_to_elem(static_cast<ku::DType>(to), ku::elem_to_f64(static_cast<ku::DType>(from), src + i * ws), dst + i * wd);
}
// the amp variant with a target dtype (product entry point is ku_cuda_amp_to)
uint32_t ko_amp_to(KuGraph* g, uint32_t root, uint32_t dtype) {
  if (!g) return 0xFFFFFFFFu;
  return ku::guard<uint32_t>(0xFFFFFFFFu, [&]() { return ku::amp_to(g->g, root, static_cast<ku::DType>(dtype)); });
}
}
