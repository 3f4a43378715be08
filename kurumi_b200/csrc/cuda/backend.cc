#include "backend.h"

#include <cstring>
#include <mutex>

#include "../capi/handles.h"
#include "hostmem.h"

namespace ku::cu {

CudaBackend::CudaBackend(int device) : rt_(device) { install_pinned_host_memory(); }

CudaBackend::~CudaBackend() {
  rt_.make_current();
  cudaStreamSynchronize(rt_.stream());
  for (auto& kv : pipelines_) destroy_pipeline(*kv.second);
  for (auto& e : ev_pool_) { cudaEventDestroy(e.first); cudaEventDestroy(e.second); }
}

CudaBackend::Compiled& CudaBackend::program_for(const Graph& g, const std::vector<NodeId>& ids) {
  for (NodeId id : ids) (void)g.node(id);
  auto key = std::make_pair(g.id(), ids);
  auto it = programs_.find(key);
  if (it != programs_.end()) return *it->second;
  auto c = std::make_unique<Compiled>();
  c->prog = compile_program(rt_, g, ids);
  c->temp_ptrs.assign(c->prog.slots.size(), nullptr);
  Compiled& ref = *c;
  programs_[key] = std::move(c);
  return ref;
}

void* CudaBackend::const_ptr(const Graph& g, NodeId node) {
  auto key = std::make_pair(g.id(), node);
  auto it = consts_.find(key);
  if (it != consts_.end()) return it->second;
  const Tensor& t = *g.node(node).op.data;
  void* p = rt_.alloc(std::max<size_t>(t.bytes.size(), 1));
  if (!t.bytes.empty()) {
    cuda_check(cudaMemcpyAsync(p, t.bytes.data(), t.bytes.size(), cudaMemcpyHostToDevice, rt_.stream()), "constant upload");
    rt_.sync();  // the host buffer belongs to the graph; finish before anyone can free it
    rt_.stats.h2d_bytes += t.bytes.size();
  }
  consts_[key] = p;
  return p;
}

std::vector<DevTensor*> CudaBackend::eval_device(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds, const DevFeeds& dev_feeds) {
  rt_.make_current();
  Compiled& c = program_for(g, ids);
  Program& P = c.prog;
  std::vector<void*> ptr(P.slots.size(), nullptr);
  std::vector<void*> staged;  // host feeds uploaded for this run only
  for (size_t i = 0; i < P.slots.size(); ++i) {
    Slot& s = P.slots[i];
    switch (s.kind) {
      case Slot::Const: ptr[i] = const_ptr(g, s.node); break;
      case Slot::Feed: {
        auto d = dev_feeds.find(s.node);
        if (d != dev_feeds.end()) {
          if (d->second->dtype != s.dtype || d->second->shape != s.shape)
            throw Error::backend("feed for node " + std::to_string(s.node) + " has shape " + shape_str(d->second->shape) + " " + dtype_name(d->second->dtype) +
                                 ", the Input is " + shape_str(s.shape) + " " + dtype_name(s.dtype));
          ptr[i] = d->second->ptr;
          break;
        }
        auto h = feeds.find(s.node);
        if (h == feeds.end()) {
          for (void* p : staged) rt_.free(p);
          throw Error("panic: interpret: missing feed for an Input node");
        }
        const Tensor& t = *h->second;
        if (t.dtype != s.dtype || t.shape != s.shape) {
          for (void* p : staged) rt_.free(p);
          throw Error::backend("feed for node " + std::to_string(s.node) + " has shape " + shape_str(t.shape) + " " + dtype_name(t.dtype) + ", the Input is " +
                               shape_str(s.shape) + " " + dtype_name(s.dtype));
        }
        void* p = rt_.alloc(std::max<size_t>(s.bytes, 1));
        if (s.bytes) cuda_check(cudaMemcpyAsync(p, t.bytes.data(), s.bytes, cudaMemcpyHostToDevice, rt_.stream()), "feed upload");
        rt_.stats.h2d_bytes += s.bytes;
        staged.push_back(p);
        ptr[i] = p;
        break;
      }
      case Slot::Temp:
        if (!c.temp_ptrs[i]) {
          c.temp_ptrs[i] = rt_.alloc(std::max<size_t>(s.bytes, 1));
          if (s.zero_init && s.bytes) cuda_check(cudaMemsetAsync(c.temp_ptrs[i], 0, s.bytes, rt_.stream()), "cudaMemsetAsync(scratch)");
        }
        ptr[i] = c.temp_ptrs[i];
        break;
      case Slot::Out: ptr[i] = rt_.alloc(std::max<size_t>(s.bytes, 1)); break;
    }
  }
  // issue the cached launches
  for (Launch& L : P.launches) {
    if (L.persistent_clusters < 0) {  // persistent kernel: one wave of co-resident clusters
      const unsigned cl = L.cluster[0];
      const int fit = rt_.max_active_clusters(L.kernel, cl, L.block[0], L.smem);
      if (fit <= 0) throw Error::backend("kernel " + L.name + " cannot be launched with clusters of " + std::to_string(cl));
      L.persistent_clusters = std::min<int>(fit, static_cast<int>(L.grid[0] / cl));
      L.persistent_clusters = L.persistent_clusters / static_cast<int>(L.grid_multiple) * static_cast<int>(L.grid_multiple);
      if (L.persistent_clusters <= 0) throw Error::backend("kernel " + L.name + " needs " + std::to_string(L.grid_multiple) + " co-resident CTAs, the device fits " + std::to_string(fit));
      L.grid[0] = static_cast<unsigned>(L.persistent_clusters) * cl;
    }
    std::vector<void*> vals(L.args.size());
    std::vector<CUtensorMap> maps(L.args.size());
    std::vector<void*> argv(L.args.size());
    for (size_t a = 0; a < L.args.size(); ++a) {
      const Arg& A = L.args[a];
      if (A.kind == Arg::SlotPtr) {
        vals[a] = static_cast<char*>(ptr[static_cast<size_t>(A.slot)]) + A.byte_offset;
        argv[a] = &vals[a];
      } else if (A.kind == Arg::Status) {
        vals[a] = rt_.status_word();
        argv[a] = &vals[a];
        uses_status_ = true;
      } else if (A.kind == Arg::Epoch) {
        argv[a] = &L.epoch;
      } else if (A.kind == Arg::Bytes) {
        argv[a] = const_cast<uint8_t*>(A.bytes.data());
      } else {
        const TmapSpec& t = A.tm;
        maps[a] = rt_.tensor_map(static_cast<char*>(ptr[static_cast<size_t>(t.slot)]) + t.byte_offset, t.dt, t.rank, t.dims, t.strides, t.box, t.swz);
        argv[a] = &maps[a];
      }
    }
    size_t ev = 0;
    if (profiling_) {
      if (ev_used_ == ev_pool_.size()) {
        cudaEvent_t a, b;
        cuda_check(cudaEventCreate(&a), "cudaEventCreate");
        cuda_check(cudaEventCreate(&b), "cudaEventCreate");
        ev_pool_.push_back({a, b});
      }
      ev = ev_used_++;
      cuda_check(cudaEventRecord(ev_pool_[ev].first, rt_.stream()), "cudaEventRecord");
    }
    if (L.zero_slot >= 0) cuda_check(cudaMemsetAsync(ptr[static_cast<size_t>(L.zero_slot)], L.fill_byte, L.zero_bytes, rt_.stream()), "cudaMemsetAsync(control block)");
    if (L.host_launch) {
      L.host_launch(vals, rt_.stream());
      ++rt_.stats.launches;
    } else {
      // A cooperative grid is sized from an occupancy query; if the device can hold fewer CTAs at launch time (another
      // context shares it) the driver refuses the launch: drop whole CTA groups until it fits.
      ++L.epoch;
      for (;;) {
        try {
          rt_.launch(L.kernel, L.grid, L.block, L.cluster, L.smem, argv.data(), L.cooperative);
          break;
        } catch (const Error& e) {
          const bool too_large = std::string(e.what()).find("(720)") != std::string::npos;   // CUDA_ERROR_COOPERATIVE_LAUNCH_TOO_LARGE
          if (!L.cooperative || !too_large || L.grid[0] <= L.grid_multiple) throw;
          L.grid[0] -= L.grid_multiple;
        }
      }
    }
    if (profiling_) {
      cuda_check(cudaEventRecord(ev_pool_[ev].second, rt_.stream()), "cudaEventRecord");
      pending_.push_back({ev, &L});
    }
  }
  // staged feed buffers return to the pool; stream order keeps them valid until the kernels that read them finish,
  // because the pool hands memory only to later work on this same stream
  for (void* p : staged) rt_.free(p);
  std::vector<DevTensor*> outs;
  for (int os : P.out_slots) {
    const Slot& s = P.slots[static_cast<size_t>(os)];
    auto* t = new DevTensor();
    t->ptr = ptr[static_cast<size_t>(os)]; t->bytes = s.bytes; t->dtype = s.dtype; t->shape = s.shape;
    // the same slot requested twice: give the second handle its own copy
    for (DevTensor* prev : outs)
      if (prev->ptr == t->ptr) {
        t->ptr = rt_.alloc(std::max<size_t>(s.bytes, 1));
        if (s.bytes) cuda_check(cudaMemcpyAsync(t->ptr, prev->ptr, s.bytes, cudaMemcpyDeviceToDevice, rt_.stream()), "output copy");
        break;
      }
    outs.push_back(t);
  }
  return outs;
}

DevTensor* CudaBackend::upload(DType dt, const Shape& shape, const void* host, size_t bytes) {
  rt_.make_current();
  if (bytes != numel(shape) * dtype_width(dt)) throw Error::backend("upload: byte count does not match shape " + shape_str(shape));
  auto* t = new DevTensor();
  t->ptr = rt_.alloc(std::max<size_t>(bytes, 1)); t->bytes = bytes; t->dtype = dt; t->shape = shape;
  if (bytes) cuda_check(cudaMemcpyAsync(t->ptr, host, bytes, cudaMemcpyHostToDevice, rt_.stream()), "upload");
  rt_.stats.h2d_bytes += bytes;
  return t;
}

void CudaBackend::download(const DevTensor& t, void* host) {
  rt_.make_current();
  if (t.bytes) cuda_check(cudaMemcpyAsync(host, t.ptr, t.bytes, cudaMemcpyDeviceToHost, rt_.stream()), "download");
  if (uses_status_) rt_.check_status(); else rt_.sync();
  rt_.stats.d2h_bytes += t.bytes;
}

void CudaBackend::free_dev(DevTensor* t) {
  if (!t) return;
  if (t->owned) rt_.free(t->ptr);
  delete t;
}

std::vector<Tensor> CudaBackend::eval_many_with(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds) {
  if (ids.size() == 1 && !profiling_) {   // a large evaluation that separates by rows streams through the device in chunks
    rt_.make_current();
    (void)g.node(ids[0]);
    if (Pipeline* p = pipeline_for(g, ids[0], feeds)) {
      std::vector<Tensor> res;
      res.push_back(run_pipeline(*p, g, ids[0], feeds));
      return res;
    }
  }
  std::vector<DevTensor*> outs = eval_device(g, ids, feeds, DevFeeds{});
  std::vector<Tensor> res;
  try {
    for (DevTensor* d : outs) {
      Tensor t = Tensor::make_uninit(d->dtype, d->shape);
      download(*d, t.bytes.data());
      res.push_back(std::move(t));
    }
  } catch (...) {
    for (DevTensor* d : outs) free_dev(d);
    throw;
  }
  for (DevTensor* d : outs) free_dev(d);
  return res;
}

Tensor CudaBackend::eval_with(const Graph& g, NodeId id, const Feeds& feeds) { return std::move(eval_many_with(g, {id}, feeds)[0]); }

void CudaBackend::set_profiling(bool on) {
  drain_profile();
  profiling_ = on;
}

void CudaBackend::drain_profile() {
  if (pending_.empty()) return;
  rt_.sync();
  for (auto& p : pending_) {
    float ms = 0;
    cudaEventElapsedTime(&ms, ev_pool_[p.ev].first, ev_pool_[p.ev].second);
    FamilyTime& f = profile_[p.launch->name];
    f.name = p.launch->name;
    ++f.launches;
    f.ms += ms;
    f.algo_bytes += p.launch->algo_bytes;
    f.flops += p.launch->flops;
  }
  pending_.clear();
  ev_used_ = 0;
}

std::vector<FamilyTime> CudaBackend::take_profile() {
  drain_profile();
  std::vector<FamilyTime> v;
  for (auto& kv : profile_) v.push_back(kv.second);
  profile_.clear();
  return v;
}

}  // namespace ku::cu

namespace ku {
// The CUDA library creates only the CUDA backend: there is no CPU evaluator to fall back to.
std::unique_ptr<Backend> make_backend(uint32_t kind) {
  if (kind == 2) return std::make_unique<cu::CudaBackend>(0);
  if (kind == 0 || kind == 1) {
    set_err("ku_backend_new: libkurumi_cuda provides only KU_CUDA (2); kind " + std::to_string(kind) + " is not built into this library");
    return nullptr;
  }
  set_err("ku_backend_new: unknown kind " + std::to_string(kind));
  return nullptr;
}
// ku_plan_compile: one CUDA backend on device 0 serves every plan of the process; the program for `root` is compiled now
// (kernel generation and NVRTC), so that ku_plan_run only binds buffers and replays launches.
std::shared_ptr<Backend> plan_backend(const Graph& g, NodeId root) {
  static std::mutex mu;
  static std::weak_ptr<cu::CudaBackend> shared;
  std::lock_guard<std::mutex> lk(mu);
  std::shared_ptr<cu::CudaBackend> b = shared.lock();
  if (!b) { b = std::make_shared<cu::CudaBackend>(0); shared = b; }
  b->prepare(g, root);
  return b;
}
}  // namespace ku
