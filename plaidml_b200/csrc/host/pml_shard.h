// One process per GPU: the process-wide communicator behind the library's two collectives.
//
// The contraction path shards along independent rows (rows of M, images of a batch) and has no
// exchange step of its own.  Two things around it do move data between ranks, and both are one
// NCCL all-gather over NVLink on buffers the executable already owns:
//   - a *replicated input* (the B matrix every rank multiplies its rows with): each rank uploads
//     1 / world of it from the host and the all-gather completes the copy on every GPU, so the
//     operand crosses the host link once per box instead of once per rank;
//   - a *gathered output*, when the caller wants every rank's rows on every rank.
// The reference splits one fixed problem over worker threads that share one memory
// (pmlc/dialect/pxa/transforms/cpu_thread.cc:49-92); the all-gather is what shared memory gives
// it for free.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy the process already holds when it
// runs under torch): libplaidml.so has no link-time dependency on it and single-GPU users never
// load it.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <string>

namespace pml {

constexpr size_t kShardIdBytes = 128;   // size of NCCL's unique id

class ShardComm {
 public:
  // The process's communicator; world() == 1 until init() succeeds.
  static ShardComm& instance();

  // Rank 0 makes the id, the caller carries it to the other ranks (a file, a store, MPI ...).
  void makeUniqueId(char* id128);
  // Collective over all ranks; the CUDA device that is current becomes this rank's device.
  void init(int rank, int world, const char* id128);
  void shutdown();

  int rank() const { return rank_; }
  int world() const { return world_; }
  bool active() const { return comm_ != nullptr; }

  // recv[r * bytes .. (r + 1) * bytes) = rank r's send[0 .. bytes), on `stream`.  send may be
  // recv + rank * bytes (in place).
  void allGatherBytes(const void* send, void* recv, size_t bytes, cudaStream_t stream);

 private:
  ShardComm() = default;
  void load();

  void* lib_ = nullptr;
  void* comm_ = nullptr;
  int rank_ = 0, world_ = 1;
  // entry points of NCCL's public C API (nccl.h): results are ints, 0 = success
  int (*getUniqueId_)(void*) = nullptr;
  struct UniqueId {
    char internal[kShardIdBytes];
  };
  int (*commInitRank_)(void**, int, UniqueId, int) = nullptr;   // the id travels by value
  int (*allGather_)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*commDestroy_)(void*) = nullptr;
  const char* (*errorString_)(int) = nullptr;
};

}  // namespace pml
