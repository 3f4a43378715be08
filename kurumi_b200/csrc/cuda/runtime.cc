#include "runtime.h"

#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace ku::cu {

void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Error::backend(std::string(what) + ": " + cudaGetErrorString(e));
}

static CUresult (*g_err_string)(CUresult, const char**) = nullptr;
void drv_check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* s = nullptr;
  if (g_err_string) g_err_string(r, &s);
  throw Error::backend(std::string(what) + ": " + (s ? s : "CUDA driver error") + " (" + std::to_string(static_cast<int>(r)) + ")");
}

template <typename F>
static void entry(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cuda_check(cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q), name);
  if (!p || q != cudaDriverEntryPointSuccess) throw Error::backend(std::string("driver entry point not found: ") + name);
  *out = reinterpret_cast<F>(p);
}

Runtime::Runtime(int device) : device_(device) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    throw Error::backend(std::string("ku_backend_new: no CUDA device (") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count 0") +
                         "); the CUDA backend has no CPU fallback");
  if (device < 0 || device >= n) throw Error::backend("ku_backend_new: device " + std::to_string(device) + " out of range");
  cuda_check(cudaSetDevice(device), "cudaSetDevice");
  cuda_check(cudaFree(nullptr), "context init");
  cudaDeviceProp prop;
  cuda_check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
  if (prop.major != 10) throw Error::backend(std::string("the CUDA backend is built for sm_100a only; device is sm_") + std::to_string(prop.major) + std::to_string(prop.minor));
  sm_count_ = prop.multiProcessorCount;
  cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  entry("cuModuleLoadData", &cuModuleLoadData_);
  entry("cuModuleUnload", &cuModuleUnload_);
  entry("cuModuleGetFunction", &cuModuleGetFunction_);
  entry("cuLaunchKernelEx", &cuLaunchKernelEx_);
  entry("cuFuncSetAttribute", &cuFuncSetAttribute_);
  entry("cuFuncGetAttribute", &cuFuncGetAttribute_);
  entry("cuTensorMapEncodeTiled", &cuTensorMapEncodeTiled_);
  entry("cuGetErrorString", &cuGetErrorString_);
  entry("cuOccupancyMaxActiveClusters", &cuOccupancyMaxActiveClusters_);
  g_err_string = cuGetErrorString_;
  cuda_check(cudaMalloc(&status_, 256), "cudaMalloc(status)");
  cuda_check(cudaMemsetAsync(status_, 0, 256, stream_), "cudaMemset(status)");
}

void Runtime::check_status() {
  int v = 0;
  cuda_check(cudaMemcpyAsync(&v, status_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "status read");
  sync();
  if (v != 0) {
    cudaMemsetAsync(status_, 0, sizeof(int), stream_);
    throw Error::backend("a kernel gave up a bounded wait (status " + std::to_string(v) + "); its results are invalid");
  }
}

int Runtime::max_active_clusters(const Kernel& k, unsigned cluster, unsigned block, unsigned smem) {
  if (smem > 48 * 1024) drv_check(cuFuncSetAttribute_(k.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, static_cast<int>(smem)), "cuFuncSetAttribute(smem)");
  if (cluster > 8) drv_check(cuFuncSetAttribute_(k.fn, CU_FUNC_ATTRIBUTE_NON_PORTABLE_CLUSTER_SIZE_ALLOWED, 1), "cuFuncSetAttribute(cluster)");
  CUlaunchConfig cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDimX = cluster * 64; cfg.gridDimY = 1; cfg.gridDimZ = 1;
  cfg.blockDimX = block; cfg.blockDimY = 1; cfg.blockDimZ = 1;
  cfg.sharedMemBytes = smem;
  cfg.hStream = stream_;
  CUlaunchAttribute attr[1];
  attr[0].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
  attr[0].value.clusterDim.x = cluster; attr[0].value.clusterDim.y = 1; attr[0].value.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  drv_check(cuOccupancyMaxActiveClusters_(&n, k.fn, &cfg), "cuOccupancyMaxActiveClusters");
  return n;
}

Runtime::~Runtime() {
  cudaSetDevice(device_);
  if (stream_) cudaStreamSynchronize(stream_);
  if (status_) cudaFree(status_);
  for (auto& kv : free_) cudaFree(kv.second);
  for (auto& kv : live_) cudaFree(kv.first);
  for (CUmodule m : modules_) cuModuleUnload_(m);
  if (stream_) cudaStreamDestroy(stream_);
}

void Runtime::make_current() { cuda_check(cudaSetDevice(device_), "cudaSetDevice"); }
void Runtime::sync() { cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize"); }

static size_t bucket(size_t bytes) {
  if (bytes < 512) return 512;
  if (bytes <= (size_t(1) << 20)) {  // next power of two
    size_t b = 512;
    while (b < bytes) b <<= 1;
    return b;
  }
  const size_t g = size_t(2) << 20;  // 2 MiB granules above 1 MiB
  return (bytes + g - 1) / g * g;
}

void* Runtime::alloc(size_t bytes) {
  const size_t b = bucket(bytes);
  auto it = free_.find(b);
  if (it != free_.end()) {
    void* p = it->second;
    free_.erase(it);
    live_[p] = b;
    ++stats.pool_hits;
    return p;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, b);
  if (e != cudaSuccess) {  // give cached blocks back to the driver and retry once
    cudaGetLastError();
    for (auto& kv : free_) cudaFree(kv.second);
    free_.clear();
    cuda_check(cudaMalloc(&p, b), "cudaMalloc");
  }
  live_[p] = b;
  ++stats.pool_allocs;
  return p;
}

void Runtime::free(void* p) {
  if (!p) return;
  auto it = live_.find(p);
  if (it == live_.end()) return;
  free_.emplace(it->second, p);
  live_.erase(it);
}

std::string Runtime::compile_to_cubin(const std::string& source, bool fmad, std::string* log_out) {
  nvrtcProgram prog;
  if (nvrtcCreateProgram(&prog, source.c_str(), "kurumi_kernel.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
    throw Error::backend("nvrtcCreateProgram failed");
  std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo", "--prec-div=true", "--prec-sqrt=true", "--ftz=false"};
  opts.push_back(fmad ? "--fmad=true" : "--fmad=false");
  const bool verbose = std::getenv("KURUMI_CUDA_VERBOSE") != nullptr;
  if (verbose) opts.push_back("--ptxas-options=-v");
  nvrtcResult r = nvrtcCompileProgram(prog, static_cast<int>(opts.size()), opts.data());
  size_t log_size = 0;
  nvrtcGetProgramLogSize(prog, &log_size);
  std::string log(log_size, '\0');
  if (log_size > 1) nvrtcGetProgramLog(prog, log.data());
  if (log_out) *log_out = log;
  if (verbose && log_size > 1) fprintf(stderr, "%s\n", log.c_str());
  if (r != NVRTC_SUCCESS) {
    nvrtcDestroyProgram(&prog);
    throw Error::backend("NVRTC compile failed: " + log);
  }
  size_t n = 0;
  nvrtcGetCUBINSize(prog, &n);
  std::string cubin(n, '\0');
  nvrtcGetCUBIN(prog, cubin.data());
  nvrtcDestroyProgram(&prog);
  return cubin;
}

Kernel Runtime::kernel(const std::string& source, const std::string& entry_name, bool fmad) {
  const std::string key = (fmad ? "F" : "N") + entry_name + "\n" + source;
  auto it = kernels_.find(key);
  if (it != kernels_.end()) { ++stats.nvrtc_hits; return it->second; }
  std::string log;
  if (std::getenv("KURUMI_CUDA_DUMP")) fprintf(stderr, "---- kurumi_cuda kernel %s ----\n%s\n", entry_name.c_str(), source.c_str());
  std::string cubin = compile_to_cubin(source, fmad, &log);
  ++stats.nvrtc_compiles;
  CUmodule mod;
  drv_check(cuModuleLoadData_(&mod, cubin.data()), "cuModuleLoadData");
  modules_.push_back(mod);
  Kernel k;
  drv_check(cuModuleGetFunction_(&k.fn, mod, entry_name.c_str()), "cuModuleGetFunction");
  cuFuncGetAttribute_(&k.regs, CU_FUNC_ATTRIBUTE_NUM_REGS, k.fn);
  int ss = 0;
  cuFuncGetAttribute_(&ss, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, k.fn);
  k.static_smem = static_cast<size_t>(ss);
  kernels_[key] = k;
  return k;
}

void Runtime::launch(const Kernel& k, const unsigned grid[3], const unsigned block[3], const unsigned cluster[3], unsigned smem, void** args, bool cooperative) {
  if (smem > 48 * 1024) drv_check(cuFuncSetAttribute_(k.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, static_cast<int>(smem)), "cuFuncSetAttribute(smem)");
  CUlaunchConfig cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDimX = grid[0]; cfg.gridDimY = grid[1]; cfg.gridDimZ = grid[2];
  cfg.blockDimX = block[0]; cfg.blockDimY = block[1]; cfg.blockDimZ = block[2];
  cfg.sharedMemBytes = smem;
  cfg.hStream = stream_;
  CUlaunchAttribute attr[2];
  unsigned na = 0;
  if (cluster && cluster[0] * cluster[1] * cluster[2] > 1) {
    attr[na].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr[na].value.clusterDim.x = cluster[0]; attr[na].value.clusterDim.y = cluster[1]; attr[na].value.clusterDim.z = cluster[2];
    ++na;
    if (cluster[0] * cluster[1] * cluster[2] > 8)
      drv_check(cuFuncSetAttribute_(k.fn, CU_FUNC_ATTRIBUTE_NON_PORTABLE_CLUSTER_SIZE_ALLOWED, 1), "cuFuncSetAttribute(cluster)");
  }
  if (cooperative) {   // CTAs that wait on one another must all be resident: the driver checks it
    attr[na].id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE;
    attr[na].value.cooperative = 1;
    ++na;
  }
  if (na) { cfg.attrs = attr; cfg.numAttrs = na; }
  drv_check(cuLaunchKernelEx_(&cfg, k.fn, args, nullptr), "cuLaunchKernelEx");
  ++stats.launches;
}

CUtensorMap Runtime::tensor_map(const void* ptr, CUtensorMapDataType dt, unsigned rank, const uint64_t* dims, const uint64_t* strides_bytes,
                                const uint32_t* box, CUtensorMapSwizzle swz) {
  CUtensorMap m;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (unsigned i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (unsigned i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];  // stride of dim i+1 (dim 0 is dense)
  drv_check(cuTensorMapEncodeTiled_(&m, dt, rank, const_cast<void*>(ptr), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
            "cuTensorMapEncodeTiled");
  return m;
}

}  // namespace ku::cu
