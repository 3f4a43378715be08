// The CUDA backend: kurumi's evaluation seam (kurumi_core/src/backend.rs:14-31) on a B200.
// A graph evaluation is compiled once into a Program (cached per graph id + roots, the role the
// reference's compile-once Plan plays, kurumi_core/src/realize/plan.rs:13-58) and replayed: the
// replay binds buffers and issues the cached launches on the backend's stream.
#pragma once
#include <map>
#include <memory>

#include "sched.h"

namespace ku::cu {

struct DevTensor {
  void* ptr = nullptr;
  size_t bytes = 0;
  DType dtype = DType::F32;
  Shape shape;
  bool owned = true;
};
using DevFeeds = std::unordered_map<NodeId, const DevTensor*>;

struct FamilyTime { std::string name; uint64_t launches = 0; double ms = 0, algo_bytes = 0, flops = 0; };

class CudaBackend : public Backend {
 public:
  explicit CudaBackend(int device);
  ~CudaBackend() override;
  const char* name() const override { return "cuda"; }
  Tensor eval_with(const Graph& g, NodeId id, const Feeds& feeds) override;
  std::vector<Tensor> eval_many_with(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds) override;

  // Device-resident evaluation: outputs stay in HBM; feeds may be host tensors, device tensors or both.
  std::vector<DevTensor*> eval_device(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds, const DevFeeds& dev_feeds);
  DevTensor* upload(DType dt, const Shape& shape, const void* host, size_t bytes);
  void download(const DevTensor& t, void* host);
  void free_dev(DevTensor* t);

  Runtime& runtime() { return rt_; }
  // Per-launch timing with CUDA events on the launching stream (off by default).
  void set_profiling(bool on);
  std::vector<FamilyTime> take_profile();

 private:
  struct Compiled {
    Program prog;
    std::vector<void*> temp_ptrs;  // persistent scratch, one per Temp slot (allocated on first run)
  };
  Compiled& program_for(const Graph& g, const std::vector<NodeId>& ids);
  void* const_ptr(const Graph& g, NodeId node);

  Runtime rt_;
  std::map<std::pair<uint64_t, std::vector<NodeId>>, std::unique_ptr<Compiled>> programs_;
  std::map<std::pair<uint64_t, NodeId>, void*> consts_;
  bool profiling_ = false;
  bool uses_status_ = false;  // some launched kernel reports through the device status word
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> ev_pool_;
  struct Pending { size_t ev; const Launch* launch; };
  std::vector<Pending> pending_;
  size_t ev_used_ = 0;
  std::map<std::string, FamilyTime> profile_;
  void drain_profile();
};

}  // namespace ku::cu
