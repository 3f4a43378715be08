// The CUDA backend: kurumi's evaluation seam (kurumi_core/src/backend.rs:14-31) on a B200.
// A graph evaluation is compiled once into a Program (cached per graph id + roots, the role the
// reference's compile-once Plan plays, kurumi_core/src/realize/plan.rs:13-58) and replayed: the
// replay binds buffers and issues the cached launches on the backend's stream.
#pragma once
#include <map>
#include <memory>

#include "../core/split.h"
#include "comm.h"
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

  // Multi-GPU assembly (comm.h): join the box's communicator, then gather row shards into [world * rows, ...] on every rank.
  void comm_init(const uint8_t id[128], int rank, int world);
  void comm_free() { comm_.reset(); }
  DevTensor* all_gather_rows(const DevTensor& shard);

  // Compile the program for one root ahead of its first evaluation (ku_plan_compile).
  void prepare(const Graph& g, NodeId root) { rt_.make_current(); (void)program_for(g, {root}); }

  // Forget everything cached for a graph (compiled programs with their scratch, uploaded constants, chunk pipelines).
  void release_graph(uint64_t graph_id);

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

  // A host-buffer evaluation cut into row chunks (core/split.h): the upload of chunk c + 1, the kernels of chunk c and
  // the download of chunk c - 1 run at the same time on three streams (pipeline.cc).
  struct ChunkInput {
    SplitInput si;
    DType dtype = DType::F32;
    Shape full_shape, part_shape;
    size_t outer = 1, width = 0, pitch = 0;   // the slice of part c: `outer` runs of `width` bytes, `pitch` bytes apart, from byte c * width
    void* dev[2] = {nullptr, nullptr};        // device copies: two in rotation for a sliced input, one for a whole one
  };
  struct Pipeline {
    bool usable = false;
    SplitPlan plan;
    std::vector<ChunkInput> inputs;
    cudaStream_t h2d = nullptr, d2h = nullptr;
    cudaEvent_t ev_whole = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_k;
  };
  Pipeline* pipeline_for(const Graph& g, NodeId root, const Feeds& feeds);
  Tensor run_pipeline(Pipeline& p, const Graph& g, NodeId root, const Feeds& feeds);
  void destroy_pipeline(Pipeline& p);

  Runtime rt_;
  std::unique_ptr<Comm> comm_;
  std::map<std::pair<uint64_t, NodeId>, std::unique_ptr<Pipeline>> pipelines_;
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
