// Page-locked host storage for the tensors this library hands out and takes in (ku_tensor_new, the results of
// ku_eval*): copies between such memory and the device run at the rate of the link and overlap with kernels, which
// pageable memory does not allow. Blocks of 1 MiB and more come from a pool of cudaHostAlloc'd buffers (freed
// tensors give their block back to the pool; the pool keeps at most 8 GiB); smaller ones stay on malloc. Installed
// into the core's HostMem hooks when the first CUDA backend is created. The reference's backends take and return
// plain host vectors (kurumi_core/src/dtype.rs:178-182); this is how the same interface is fed at PCIe speed.
#pragma once
#include <cstddef>

namespace ku::cu {

void install_pinned_host_memory();                       // idempotent, thread-safe
void host_copy(void* dst, const void* src, size_t bytes);   // memcpy, on several threads from 8 MiB on
bool is_pinned_block(const void* p);                     // whether p is the start of a live block of the pool

}  // namespace ku::cu
