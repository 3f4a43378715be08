#include "comm.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../core/graph.h"

namespace ku::cu {

namespace {
// the few NCCL declarations used here (nccl.h: ncclUniqueId is 128 opaque bytes passed by value, ncclUint8 = 1)
struct NcclId { char internal[128]; };
using GetUniqueId = int (*)(NcclId*);
using CommInitRank = int (*)(void**, int, NcclId, int);
using CommDestroy = int (*)(void*);
using AllGather = int (*)(const void*, void*, size_t, int, void*, cudaStream_t);
using GetErrorString = const char* (*)(int);

struct Nccl {
  GetUniqueId get_unique_id = nullptr;
  CommInitRank comm_init_rank = nullptr;
  CommDestroy comm_destroy = nullptr;
  AllGather all_gather = nullptr;
  GetErrorString error_string = nullptr;
};

const Nccl& nccl() {
  static Nccl api;
  static std::once_flag once;
  static std::string failure;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { failure = std::string("NCCL is not available: ") + dlerror(); return; }
    api.get_unique_id = reinterpret_cast<GetUniqueId>(dlsym(h, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<CommInitRank>(dlsym(h, "ncclCommInitRank"));
    api.comm_destroy = reinterpret_cast<CommDestroy>(dlsym(h, "ncclCommDestroy"));
    api.all_gather = reinterpret_cast<AllGather>(dlsym(h, "ncclAllGather"));
    api.error_string = reinterpret_cast<GetErrorString>(dlsym(h, "ncclGetErrorString"));
    if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_gather || !api.error_string) failure = "libnccl.so.2 lacks an expected entry point";
  });
  if (!failure.empty()) throw Error::backend(failure);
  return api;
}

void check(int r, const char* what) {
  if (r != 0) throw Error::backend(std::string(what) + ": " + nccl().error_string(r));
}
}  // namespace

void Comm::unique_id(uint8_t out[128]) {
  NcclId id;
  check(nccl().get_unique_id(&id), "ncclGetUniqueId");
  std::memcpy(out, id.internal, 128);
}

Comm::Comm(const uint8_t id[128], int rank, int world) : rank_(rank), world_(world) {
  if (world < 1 || rank < 0 || rank >= world) throw Error::backend("communicator: rank " + std::to_string(rank) + " outside a world of " + std::to_string(world));
  NcclId nid;
  std::memcpy(nid.internal, id, 128);
  check(nccl().comm_init_rank(&comm_, world, nid, rank), "ncclCommInitRank");
}

Comm::~Comm() {
  if (comm_) nccl().comm_destroy(comm_);
}

void Comm::all_gather(const void* send, void* recv, size_t bytes, cudaStream_t stream) {
  check(nccl().all_gather(send, recv, bytes, /* ncclUint8 */ 1, comm_, stream), "ncclAllGather");
}

}  // namespace ku::cu
