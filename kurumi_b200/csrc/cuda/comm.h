// Assembly of a row-sharded result across the GPUs of one box over NCCL (NVLink / NVSwitch). The data path of a
// sharded evaluation has no exchange step (every rank evaluates its own rows, core/split.h); this is the optional
// all-gather that puts the pieces together, on the backend's own stream. One process per GPU, one communicator per
// backend; the caller carries the 128-byte id from rank 0 to the others (a file, a socket, torch.distributed).
// libnccl.so.2 is opened at run time (the copy already in the process, if any), so the library loads without it.
// The reference is single-device by construction (kurumi_core/src/backend.rs:14-31): no counterpart there.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace ku::cu {

class Comm {
 public:
  static void unique_id(uint8_t out[128]);
  Comm(const uint8_t id[128], int rank, int world);   // collective: every rank of the box calls it
  ~Comm();
  int rank() const { return rank_; }
  int world() const { return world_; }
  // recv (world * bytes) = the ranks' `send` buffers (bytes each) in rank order; queued on `stream`
  void all_gather(const void* send, void* recv, size_t bytes, cudaStream_t stream);

 private:
  void* comm_ = nullptr;
  int rank_ = 0, world_ = 1;
};

}  // namespace ku::cu
