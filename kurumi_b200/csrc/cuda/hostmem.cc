#include "hostmem.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../core/graph.h"

namespace ku::cu {

namespace {
constexpr size_t kMinPinned = size_t(1) << 20, kGranule = size_t(2) << 20, kKeep = size_t(8) << 30;

struct Pool {
  std::mutex mu;
  std::multimap<size_t, void*> free_blocks;        // bucket size -> block
  std::unordered_map<const void*, size_t> live;    // block -> bucket size
  std::unordered_map<const void*, size_t> known;   // every block ever obtained (live or cached) -> bucket size
  size_t cached = 0;
};
Pool& pool() { static Pool* p = new Pool(); return *p; }   // never destroyed: tensors may outlive static teardown

void* pinned_alloc(size_t bytes) {
  if (bytes < kMinPinned) return std::malloc(bytes ? bytes : 1);
  const size_t b = (bytes + kGranule - 1) / kGranule * kGranule;
  Pool& P = pool();
  {
    std::lock_guard<std::mutex> lk(P.mu);
    auto it = P.free_blocks.find(b);
    if (it != P.free_blocks.end()) {
      void* p = it->second;
      P.free_blocks.erase(it);
      P.cached -= b;
      P.live[p] = b;
      return p;
    }
  }
  void* p = nullptr;
  if (cudaHostAlloc(&p, b, cudaHostAllocPortable) != cudaSuccess) {   // no page-locked memory to be had: plain memory still works
    cudaGetLastError();
    return std::malloc(bytes);
  }
  std::lock_guard<std::mutex> lk(P.mu);
  P.live[p] = b;
  P.known[p] = b;
  return p;
}

void pinned_release(void* p, size_t) {
  if (!p) return;
  Pool& P = pool();
  {
    std::lock_guard<std::mutex> lk(P.mu);
    auto it = P.live.find(p);
    if (it != P.live.end()) {
      const size_t b = it->second;
      P.live.erase(it);
      if (P.cached + b <= kKeep) {
        P.free_blocks.emplace(b, p);
        P.cached += b;
        return;
      }
      P.known.erase(p);
      cudaFreeHost(p);   // harmless if the runtime is already shutting down
      return;
    }
  }
  std::free(p);
}
}  // namespace

void install_pinned_host_memory() {
  static std::once_flag once;
  std::call_once(once, [] {
    HostMem::alloc = pinned_alloc;
    HostMem::release = pinned_release;
    HostMem::copy = host_copy;
  });
}

bool is_pinned_block(const void* p) {
  Pool& P = pool();
  std::lock_guard<std::mutex> lk(P.mu);
  return P.live.count(p) != 0;
}

void host_copy(void* dst, const void* src, size_t bytes) {
  constexpr size_t kParallelFrom = size_t(8) << 20;
  const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  const size_t nthreads = bytes < kParallelFrom ? 1 : std::min<size_t>({8, hw, bytes / (kParallelFrom / 2)});
  if (nthreads <= 1) { std::memcpy(dst, src, bytes); return; }
  const size_t piece = (bytes / nthreads + 4095) / 4096 * 4096;
  std::vector<std::thread> workers;
  for (size_t t = 1; t < nthreads; ++t) {
    const size_t lo = t * piece;
    if (lo >= bytes) break;
    const size_t n = std::min(piece, bytes - lo);
    workers.emplace_back([=] { std::memcpy(static_cast<char*>(dst) + lo, static_cast<const char*>(src) + lo, n); });
  }
  std::memcpy(dst, src, std::min(piece, bytes));
  for (auto& w : workers) w.join();
}

}  // namespace ku::cu
