// Device runtime of the CUDA backend: one context per backend handle with its own stream, a
// size-bucketed device memory pool, a per-graph constant cache (weights stay resident across
// evals, as the reference's Metal backend does: kurumi_metal/src/backend/eval_walk.rs:99-114) and
// an NVRTC kernel cache keyed by generated source (kurumi_metal/src/context/pipeline.rs:12-29
// plays that role for MSL). The CUDA runtime library is linked statically; driver entry points
// (module load, kernel launch, tensor maps) are fetched through cudaGetDriverEntryPoint, so the
// library loads on a machine without a GPU and only fails, loudly, when a backend is created.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/graph.h"

namespace ku::cu {

void cuda_check(cudaError_t e, const char* what);
void drv_check(CUresult r, const char* what);

struct Kernel {
  CUfunction fn = nullptr;
  int regs = 0;
  size_t static_smem = 0;
};

struct Stats {
  uint64_t launches = 0, nvrtc_compiles = 0, nvrtc_hits = 0, h2d_bytes = 0, d2h_bytes = 0, pool_allocs = 0, pool_hits = 0;
};

class Runtime {
 public:
  explicit Runtime(int device);
  ~Runtime();
  int device() const { return device_; }
  cudaStream_t stream() const { return stream_; }
  int sm_count() const { return sm_count_; }

  void* alloc(size_t bytes);
  void free(void* p);
  void sync();
  void make_current();

  // Compile (or fetch) `entry` from CUDA source for sm_100a.
  Kernel kernel(const std::string& source, const std::string& entry, bool fmad);
  // Compile to a cubin without touching a device (build check); throws with the NVRTC log.
  static std::string compile_to_cubin(const std::string& source, bool fmad, std::string* log_out);

  void launch(const Kernel& k, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3], unsigned smem,
              void** args, bool cooperative = false);

  // Largest number of clusters of this shape that can be resident at once (0 if it cannot launch).
  int max_active_clusters(const Kernel& k, unsigned cluster, unsigned block, unsigned smem);
  // A device word kernels set when a bounded wait gives up; check_status() throws and clears it.
  int* status_word() const { return status_; }
  void check_status();

  CUtensorMap tensor_map(const void* ptr, CUtensorMapDataType dt, unsigned rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz);

  Stats stats;

 private:
  int device_;
  int sm_count_ = 0;
  cudaStream_t stream_ = nullptr;
  int* status_ = nullptr;
  std::unordered_map<std::string, Kernel> kernels_;
  std::vector<CUmodule> modules_;
  std::multimap<size_t, void*> free_;
  std::unordered_map<void*, size_t> live_;
  // driver entry points
  CUresult (*cuModuleLoadData_)(CUmodule*, const void*) = nullptr;
  CUresult (*cuModuleUnload_)(CUmodule) = nullptr;
  CUresult (*cuModuleGetFunction_)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*cuLaunchKernelEx_)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
  CUresult (*cuFuncSetAttribute_)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*cuFuncGetAttribute_)(int*, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*cuTensorMapEncodeTiled_)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  CUresult (*cuGetErrorString_)(CUresult, const char**) = nullptr;
  CUresult (*cuOccupancyMaxActiveClusters_)(int*, CUfunction, const CUlaunchConfig*) = nullptr;
  friend void drv_check(CUresult, const char*);
};

}  // namespace ku::cu
