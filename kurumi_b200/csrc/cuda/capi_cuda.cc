// extern "C" exports of include/kurumi_cuda.h.
#include "../../../include/kurumi_cuda.h"

#include <cstring>
#include <sstream>

#include "../capi/handles.h"
#include "backend.h"

using namespace ku;
using ku::cu::CudaBackend;
using ku::cu::DevTensor;

struct KuDevTensor { DevTensor* t; };
struct KuDevFeeds { ku::cu::DevFeeds f; };

namespace {
CudaBackend* cuda_of(const KuBackend* b) {
  if (!b) throw Error("null backend handle");
  auto* c = dynamic_cast<CudaBackend*>(b->b.get());
  if (!c) throw Error::backend("not a CUDA backend");
  return c;
}
}  // namespace

extern "C" {

KuBackend* ku_cuda_backend_new(int32_t device) {
  return guard<KuBackend*>(nullptr, [&]() {
    auto* h = new KuBackend();
    try { h->b = std::make_unique<CudaBackend>(device); } catch (...) { delete h; throw; }
    return h;
  });
}

KuDevTensor* ku_cuda_upload(const KuBackend* b, const KuTensor* t) {
  if (!t) { set_err("ku_cuda_upload: null tensor"); return nullptr; }
  return guard<KuDevTensor*>(nullptr, [&]() {
    DevTensor* d = cuda_of(b)->upload(t->t->dtype, t->t->shape, t->t->bytes.data(), t->t->bytes.size());
    cuda_of(b)->runtime().sync();  // the host tensor may be freed by the caller right away
    return new KuDevTensor{d};
  });
}
KuDevTensor* ku_cuda_upload_bytes(const KuBackend* b, uint32_t dtype, const void* data, size_t nbytes, const size_t* shape, size_t rank) {
  return guard<KuDevTensor*>(nullptr, [&]() {
    if (dtype >= kNumDTypes) throw Error("ku_cuda_upload_bytes: bad dtype " + std::to_string(dtype));
    if (!data && nbytes) throw Error("ku_cuda_upload_bytes: null data");
    Shape s = (shape && rank) ? Shape(shape, shape + rank) : Shape{};
    return new KuDevTensor{cuda_of(b)->upload(static_cast<DType>(dtype), s, data, nbytes)};
  });
}
KuTensor* ku_cuda_download(const KuBackend* b, const KuDevTensor* t) {
  if (!t) { set_err("ku_cuda_download: null tensor"); return nullptr; }
  return guard<KuTensor*>(nullptr, [&]() {
    Tensor h = Tensor::make_uninit(t->t->dtype, t->t->shape);
    cuda_of(b)->download(*t->t, h.bytes.data());
    return new KuTensor{std::make_shared<const Tensor>(std::move(h))};
  });
}
int32_t ku_cuda_download_bytes(const KuBackend* b, const KuDevTensor* t, void* out, size_t cap) {
  if (!t || !out) { set_err("ku_cuda_download_bytes: null tensor/out"); return -1; }
  return guard<int32_t>(-1, [&]() {
    if (cap < t->t->bytes) throw Error("ku_cuda_download_bytes: buffer too small");
    cuda_of(b)->download(*t->t, out);
    return 0;
  });
}
void ku_cuda_dev_free(const KuBackend* b, KuDevTensor* t) {
  if (!t) return;
  guard<int>(0, [&]() { cuda_of(b)->free_dev(t->t); return 0; });
  delete t;
}
void* ku_cuda_dev_ptr(const KuDevTensor* t) { return t ? t->t->ptr : nullptr; }
size_t ku_cuda_dev_nbytes(const KuDevTensor* t) { return t ? t->t->bytes : 0; }
size_t ku_cuda_dev_rank(const KuDevTensor* t) { return t ? t->t->shape.size() : 0; }
void ku_cuda_dev_shape(const KuDevTensor* t, size_t* out) {
  if (!t || !out) return;
  for (size_t i = 0; i < t->t->shape.size(); ++i) out[i] = t->t->shape[i];
}
uint32_t ku_cuda_dev_dtype(const KuDevTensor* t) { return t ? static_cast<uint32_t>(t->t->dtype) : 0; }

KuDevFeeds* ku_cuda_dev_feeds_new(void) { return new KuDevFeeds(); }
void ku_cuda_dev_feeds_free(KuDevFeeds* f) { delete f; }
void ku_cuda_dev_feeds_set(KuDevFeeds* f, KuNode node, const KuDevTensor* t) {
  if (!f || !t) return;
  f->f[node] = t->t;
}

int32_t ku_cuda_eval_device(KuGraph* g, const KuNode* ids, size_t n, const KuBackend* b, const KuFeeds* feeds, const KuDevFeeds* dev_feeds,
                            KuDevTensor** out) {
  if (!g || !b || !out || (!ids && n)) { set_err("ku_cuda_eval_device: null graph/backend/ids/out handle"); return -1; }
  return guard<int32_t>(-1, [&]() {
    std::vector<NodeId> v(ids, ids + n);
    Feeds none;
    ku::cu::DevFeeds dnone;
    auto outs = cuda_of(b)->eval_device(g->g, v, feeds ? feeds->f : none, dev_feeds ? dev_feeds->f : dnone);
    for (size_t i = 0; i < outs.size(); ++i) out[i] = new KuDevTensor{outs[i]};
    return 0;
  });
}

int32_t ku_cuda_sync(const KuBackend* b) { return guard<int32_t>(-1, [&]() { cuda_of(b)->runtime().check_status(); return 0; }); }
void* ku_cuda_stream(const KuBackend* b) { return guard<void*>(nullptr, [&]() { return static_cast<void*>(cuda_of(b)->runtime().stream()); }); }
int32_t ku_cuda_device(const KuBackend* b) { return guard<int32_t>(-1, [&]() { return cuda_of(b)->runtime().device(); }); }

size_t ku_cuda_stats(const KuBackend* b, uint64_t* out, size_t cap) {
  return guard<size_t>(0, [&]() -> size_t {
    const ku::cu::Stats& s = cuda_of(b)->runtime().stats;
    const uint64_t v[7] = {s.launches, s.nvrtc_compiles, s.nvrtc_hits, s.h2d_bytes, s.d2h_bytes, s.pool_allocs, s.pool_hits};
    size_t n = std::min<size_t>(cap, 7);
    for (size_t i = 0; out && i < n; ++i) out[i] = v[i];
    return n;
  });
}
void ku_cuda_profile_enable(const KuBackend* b, uint32_t on) { guard<int>(0, [&]() { cuda_of(b)->set_profiling(on != 0); return 0; }); }
size_t ku_cuda_profile_take(const KuBackend* b, uint8_t* out, size_t cap) {
  return guard<size_t>(0, [&]() -> size_t {
    std::ostringstream o;
    o.precision(9);
    for (auto& f : cuda_of(b)->take_profile()) o << f.name << " " << f.launches << " " << f.ms << " " << f.algo_bytes << " " << f.flops << "\n";
    std::string s = o.str();
    if (out && cap) std::memcpy(out, s.data(), std::min(cap, s.size()));
    return s.size();
  });
}

int32_t ku_cuda_comm_unique_id(uint8_t* out) {
  if (!out) { set_err("ku_cuda_comm_unique_id: null out"); return -1; }
  return guard<int32_t>(-1, [&]() { ku::cu::Comm::unique_id(out); return 0; });
}
int32_t ku_cuda_comm_init(const KuBackend* b, const uint8_t* id, int32_t rank, int32_t world) {
  if (!id) { set_err("ku_cuda_comm_init: null id"); return -1; }
  return guard<int32_t>(-1, [&]() { cuda_of(b)->comm_init(id, rank, world); return 0; });
}
void ku_cuda_comm_free(const KuBackend* b) { guard<int>(0, [&]() { cuda_of(b)->comm_free(); return 0; }); }
KuDevTensor* ku_cuda_all_gather_rows(const KuBackend* b, const KuDevTensor* shard) {
  if (!shard) { set_err("ku_cuda_all_gather_rows: null tensor"); return nullptr; }
  return guard<KuDevTensor*>(nullptr, [&]() { return new KuDevTensor{cuda_of(b)->all_gather_rows(*shard->t)}; });
}

void ku_cuda_release_graph(const KuBackend* b, const KuGraph* g) {
  if (!g) return;
  guard<int>(0, [&]() { cuda_of(b)->release_graph(g->g.id()); return 0; });
}

KuNode ku_cuda_amp_to(KuGraph* g, KuNode root, uint32_t dtype) {
  if (!g) { set_err("null graph handle"); return KU_ERR; }
  return guard<KuNode>(KU_ERR, [&]() -> KuNode {
    if (dtype >= kNumDTypes) throw Error("ku_cuda_amp_to: bad dtype " + std::to_string(dtype));
    return amp_to(g->g, root, static_cast<DType>(dtype));
  });
}

size_t ku_cuda_compile_check(KuGraph* g, const KuNode* ids, size_t n, uint8_t* out, size_t cap) {
  if (!g || (!ids && n)) { set_err("ku_cuda_compile_check: null graph/ids"); return static_cast<size_t>(-1); }
  return guard<size_t>(static_cast<size_t>(-1), [&]() -> size_t {
    std::vector<NodeId> v(ids, ids + n);
    std::string s;
    for (auto& name : ku::cu::compile_check(g->g, v, 148)) s += name + "\n";
    if (out && cap) std::memcpy(out, s.data(), std::min(cap, s.size()));
    return s.size();
  });
}

}  // extern "C"
