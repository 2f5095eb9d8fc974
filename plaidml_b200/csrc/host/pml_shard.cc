// The process-wide NCCL communicator of the sharded (one process per GPU) mode.
#include "pml_shard.h"

#include <dlfcn.h>

#include <cstring>
#include <stdexcept>

namespace pml {

ShardComm& ShardComm::instance() {
  static ShardComm comm;
  return comm;
}

void ShardComm::load() {
  if (lib_) return;
  // RTLD_NOLOAD first: a process that already holds NCCL (torch loads its own copy) must not get a second one.
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    throw std::runtime_error(std::string("The sharded mode needs NCCL (libnccl.so.2), which could not be loaded: ") +
                             dlerror());
  }
  auto sym = [&](const char* name) {
    void* p = dlsym(h, name);
    if (!p) throw std::runtime_error(std::string("libnccl.so.2 does not export ") + name);
    return p;
  };
  getUniqueId_ = reinterpret_cast<decltype(getUniqueId_)>(sym("ncclGetUniqueId"));
  commInitRank_ = reinterpret_cast<decltype(commInitRank_)>(sym("ncclCommInitRank"));
  allGather_ = reinterpret_cast<decltype(allGather_)>(sym("ncclAllGather"));
  commDestroy_ = reinterpret_cast<decltype(commDestroy_)>(sym("ncclCommDestroy"));
  errorString_ = reinterpret_cast<decltype(errorString_)>(sym("ncclGetErrorString"));
  lib_ = h;
}

void ShardComm::makeUniqueId(char* id128) {
  load();
  UniqueId id;
  std::memset(&id, 0, sizeof(id));
  const int rc = getUniqueId_(&id);
  if (rc != 0) throw std::runtime_error(std::string("ncclGetUniqueId: ") + errorString_(rc));
  std::memcpy(id128, id.internal, kShardIdBytes);
}

void ShardComm::init(int rank, int world, const char* id128) {
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("Shard rank outside the world size");
  if (comm_) throw std::runtime_error("The sharded mode is already initialised in this process");
  if (world == 1) {
    rank_ = 0;
    world_ = 1;
    return;
  }
  load();
  UniqueId id;
  std::memcpy(id.internal, id128, kShardIdBytes);
  void* comm = nullptr;
  const int rc = commInitRank_(&comm, world, id, rank);
  if (rc != 0 || comm == nullptr) throw std::runtime_error(std::string("ncclCommInitRank: ") + errorString_(rc));
  comm_ = comm;
  rank_ = rank;
  world_ = world;
}

void ShardComm::shutdown() {
  if (comm_) {
    commDestroy_(comm_);
    comm_ = nullptr;
  }
  rank_ = 0;
  world_ = 1;
}

void ShardComm::allGatherBytes(const void* send, void* recv, size_t bytes, cudaStream_t stream) {
  if (world_ == 1) {
    if (send != recv && bytes) {
      const cudaError_t e = cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) throw std::runtime_error(std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e));
    }
    return;
  }
  if (!comm_) throw std::runtime_error("The sharded mode is not initialised (pmlb_shard_init)");
  constexpr int kNcclUint8 = 1;   // ncclUint8 of nccl.h's ncclDataType_t
  const int rc = allGather_(send, recv, bytes, kNcclUint8, comm_, stream);
  if (rc != 0) throw std::runtime_error(std::string("ncclAllGather: ") + errorString_(rc));
}

}  // namespace pml
