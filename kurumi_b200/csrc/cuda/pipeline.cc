// Host-buffer evaluation in row chunks. The drop-in call takes host tensors and returns a host tensor
// (kurumi_core/src/backend.rs:14-31, kurumi/src/capi/eval.rs:58-71); done in one piece that is upload, then
// kernels, then download, each waiting for the one before. When the root separates by rows (core/split.h) the
// backend instead evaluates the part graph chunk by chunk: the host-to-device copy of chunk c + 1, the kernels of
// chunk c and the device-to-host copy of chunk c - 1 overlap on three streams (PCIe is full duplex), the result lands
// directly in the page-locked storage of the returned tensor. One cudaMemcpyAsync / cudaMemcpy2DAsync per buffer and
// chunk (a slice along an inner axis is a pitched copy); ordering between the streams is by events.
#include <cstring>

#include "backend.h"
#include "hostmem.h"

namespace ku::cu {

namespace {
constexpr size_t kMinBytes = size_t(16) << 20;   // below this the three-stage pipeline costs more than it hides
}

void CudaBackend::destroy_pipeline(Pipeline& p) {
  for (auto& in : p.inputs) for (void*& d : in.dev) if (d) { rt_.free(d); d = nullptr; }
  for (cudaEvent_t e : p.ev_in) cudaEventDestroy(e);
  for (cudaEvent_t e : p.ev_k) cudaEventDestroy(e);
  if (p.ev_whole) cudaEventDestroy(p.ev_whole);
  if (p.h2d) cudaStreamDestroy(p.h2d);
  if (p.d2h) cudaStreamDestroy(p.d2h);
  p.ev_in.clear(); p.ev_k.clear(); p.ev_whole = nullptr; p.h2d = p.d2h = nullptr;
  p.usable = false;
}

CudaBackend::Pipeline* CudaBackend::pipeline_for(const Graph& g, NodeId root, const Feeds& feeds) {
  const auto key = std::make_pair(g.id(), root);
  auto it = pipelines_.find(key);
  if (it != pipelines_.end()) return it->second->usable ? it->second.get() : nullptr;
  auto p = std::make_unique<Pipeline>();
  Pipeline* res = nullptr;
  const Node& rn = g.node(root);
  size_t moved = numel(rn.shape) * dtype_width(rn.dtype);
  for (auto& kv : feeds) moved += kv.second->bytes.size();
  if (moved >= kMinBytes && !rn.shape.empty()) {
    for (size_t parts : {size_t(8), size_t(4), size_t(2)}) {
      std::string why;
      if (!row_split(g, root, parts, &p->plan, &why)) continue;
      bool sliced = false;
      for (auto& si : p->plan.inputs) sliced = sliced || si.axis >= 0;
      if (!sliced) break;   // nothing to stream: every part would need every input whole
      for (auto& si : p->plan.inputs) {
        ChunkInput in;
        in.si = si;
        const Node& n = g.node(si.orig);
        in.dtype = n.dtype;
        in.full_shape = n.shape;
        in.part_shape = p->plan.graph.shape(si.part);
        const size_t w = dtype_width(n.dtype);
        if (si.axis < 0) {
          in.outer = 1; in.width = in.pitch = numel(n.shape) * w;
        } else {
          const size_t a = static_cast<size_t>(si.axis);
          size_t inner = 1;
          for (size_t d = a + 1; d < n.shape.size(); ++d) inner *= n.shape[d];
          in.outer = 1;
          for (size_t d = 0; d < a; ++d) in.outer *= n.shape[d];
          in.width = n.shape[a] / parts * inner * w;
          in.pitch = n.shape[a] * inner * w;
        }
        p->inputs.push_back(in);
      }
      cuda_check(cudaStreamCreateWithFlags(&p->h2d, cudaStreamNonBlocking), "cudaStreamCreate");
      cuda_check(cudaStreamCreateWithFlags(&p->d2h, cudaStreamNonBlocking), "cudaStreamCreate");
      cuda_check(cudaEventCreateWithFlags(&p->ev_whole, cudaEventDisableTiming), "cudaEventCreate");
      for (size_t c = 0; c < parts; ++c) {
        cudaEvent_t a, b;
        cuda_check(cudaEventCreateWithFlags(&a, cudaEventDisableTiming), "cudaEventCreate");
        cuda_check(cudaEventCreateWithFlags(&b, cudaEventDisableTiming), "cudaEventCreate");
        p->ev_in.push_back(a); p->ev_k.push_back(b);
      }
      p->usable = true;
      res = p.get();
      break;
    }
  }
  pipelines_[key] = std::move(p);
  return res;
}

Tensor CudaBackend::run_pipeline(Pipeline& p, const Graph& g, NodeId root, const Feeds& feeds) {
  const size_t parts = p.plan.parts;
  const Node& rn = g.node(root);
  // every feed must be there and of the recorded shape before anything is queued
  std::vector<const Tensor*> host(p.inputs.size(), nullptr);
  for (size_t i = 0; i < p.inputs.size(); ++i) {
    auto h = feeds.find(p.inputs[i].si.orig);
    if (h == feeds.end()) throw Error("panic: interpret: missing feed for an Input node");
    const Tensor& t = *h->second;
    if (t.dtype != p.inputs[i].dtype || t.shape != p.inputs[i].full_shape)
      throw Error::backend("feed for node " + std::to_string(p.inputs[i].si.orig) + " has shape " + shape_str(t.shape) + " " + dtype_name(t.dtype) + ", the Input is " +
                           shape_str(p.inputs[i].full_shape) + " " + dtype_name(p.inputs[i].dtype));
    host[i] = &t;
  }
  for (auto& in : p.inputs) {
    const size_t bytes = std::max<size_t>(in.outer * in.width, 1);
    if (!in.dev[0]) in.dev[0] = rt_.alloc(bytes);
    if (in.si.axis >= 0 && !in.dev[1]) in.dev[1] = rt_.alloc(bytes);
  }
  Tensor result = Tensor::make_uninit(rn.dtype, rn.shape);
  const size_t chunk_bytes = result.bytes.size() / parts;
  const cudaStream_t compute = rt_.stream();
  std::vector<DevTensor*> outs;
  try {
    for (size_t i = 0; i < p.inputs.size(); ++i)
      if (p.inputs[i].si.axis < 0 && p.inputs[i].width) {
        cuda_check(cudaMemcpyAsync(p.inputs[i].dev[0], host[i]->bytes.data(), p.inputs[i].width, cudaMemcpyHostToDevice, p.h2d), "upload");
        rt_.stats.h2d_bytes += p.inputs[i].width;
      }
    cuda_check(cudaEventRecord(p.ev_whole, p.h2d), "cudaEventRecord");
    cuda_check(cudaStreamWaitEvent(compute, p.ev_whole, 0), "cudaStreamWaitEvent");
    std::vector<DevTensor> views(p.inputs.size());
    for (size_t c = 0; c < parts; ++c) {
      const size_t b = c & 1;
      if (c >= 2) cuda_check(cudaStreamWaitEvent(p.h2d, p.ev_k[c - 2], 0), "cudaStreamWaitEvent");   // the kernels of chunk c - 2 read this buffer
      DevFeeds dev_feeds;
      for (size_t i = 0; i < p.inputs.size(); ++i) {
        ChunkInput& in = p.inputs[i];
        DevTensor& v = views[i];
        v.dtype = in.dtype; v.shape = in.part_shape; v.owned = false; v.bytes = in.outer * in.width;
        if (in.si.axis < 0) {
          v.ptr = in.dev[0];
        } else {
          v.ptr = in.dev[b];
          const char* src = reinterpret_cast<const char*>(host[i]->bytes.data()) + c * in.width;
          if (in.outer == 1) cuda_check(cudaMemcpyAsync(v.ptr, src, in.width, cudaMemcpyHostToDevice, p.h2d), "upload");
          else if (in.width) cuda_check(cudaMemcpy2DAsync(v.ptr, in.width, src, in.pitch, in.width, in.outer, cudaMemcpyHostToDevice, p.h2d), "upload (pitched)");
          rt_.stats.h2d_bytes += v.bytes;
        }
        dev_feeds[in.si.part] = &v;
      }
      cuda_check(cudaEventRecord(p.ev_in[c], p.h2d), "cudaEventRecord");
      cuda_check(cudaStreamWaitEvent(compute, p.ev_in[c], 0), "cudaStreamWaitEvent");
      std::vector<DevTensor*> o = eval_device(p.plan.graph, {p.plan.root}, Feeds{}, dev_feeds);
      outs.push_back(o[0]);
      if (o[0]->bytes != chunk_bytes) throw Error::backend("internal: a chunk result has " + std::to_string(o[0]->bytes) + " bytes, expected " + std::to_string(chunk_bytes));
      cuda_check(cudaEventRecord(p.ev_k[c], compute), "cudaEventRecord");
      cuda_check(cudaStreamWaitEvent(p.d2h, p.ev_k[c], 0), "cudaStreamWaitEvent");
      if (chunk_bytes) cuda_check(cudaMemcpyAsync(result.bytes.data() + c * chunk_bytes, o[0]->ptr, chunk_bytes, cudaMemcpyDeviceToHost, p.d2h), "download");
      rt_.stats.d2h_bytes += chunk_bytes;
    }
    cuda_check(cudaStreamSynchronize(p.d2h), "cudaStreamSynchronize");
  } catch (...) {
    cudaStreamSynchronize(p.h2d); cudaStreamSynchronize(compute); cudaStreamSynchronize(p.d2h);
    for (DevTensor* d : outs) free_dev(d);
    throw;
  }
  // a chunk's memory goes back to the pool only now: the copies out ran on another stream
  for (DevTensor* d : outs) free_dev(d);
  if (uses_status_) rt_.check_status();
  return result;
}

void CudaBackend::comm_init(const uint8_t id[128], int rank, int world) {
  rt_.make_current();
  comm_.reset();
  comm_ = std::make_unique<Comm>(id, rank, world);
}

DevTensor* CudaBackend::all_gather_rows(const DevTensor& shard) {
  if (!comm_) throw Error::backend("all_gather_rows: no communicator (ku_cuda_comm_init first)");
  if (shard.shape.empty()) throw Error::backend("all_gather_rows: a scalar has no rows");
  rt_.make_current();
  auto* t = new DevTensor();
  t->dtype = shard.dtype;
  t->shape = shard.shape;
  t->shape[0] *= static_cast<size_t>(comm_->world());
  t->bytes = shard.bytes * static_cast<size_t>(comm_->world());
  t->ptr = rt_.alloc(std::max<size_t>(t->bytes, 1));
  try {
    if (shard.bytes) comm_->all_gather(shard.ptr, t->ptr, shard.bytes, rt_.stream());
  } catch (...) {
    rt_.free(t->ptr);
    delete t;
    throw;
  }
  return t;
}

void CudaBackend::release_graph(uint64_t graph_id) {
  rt_.make_current();
  rt_.sync();
  std::vector<uint64_t> part_graphs;
  for (auto it = pipelines_.begin(); it != pipelines_.end();) {
    if (it->first.first == graph_id) {
      part_graphs.push_back(it->second->plan.graph.id());
      destroy_pipeline(*it->second);
      it = pipelines_.erase(it);
    } else {
      ++it;
    }
  }
  for (uint64_t id : part_graphs) release_graph(id);
  for (auto it = programs_.begin(); it != programs_.end();) {
    if (it->first.first == graph_id) {
      for (void* p : it->second->temp_ptrs) if (p) rt_.free(p);
      it = programs_.erase(it);
    } else {
      ++it;
    }
  }
  for (auto it = consts_.begin(); it != consts_.end();) {
    if (it->first.first == graph_id) { rt_.free(it->second); it = consts_.erase(it); } else { ++it; }
  }
}

}  // namespace ku::cu
