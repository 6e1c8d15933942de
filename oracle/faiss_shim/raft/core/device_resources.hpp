// Test infrastructure, not part of the product.  RAFT and RMM are not installed here; the reference's
// src/index/cagra_opt.cu and raft_help.cuh name a few of their classes in the functions that run a brute-force kNN
// (build_batch_knn_graphs, the time-partitioned insert).  These declarations let the translation unit compile so that
// its other functions -- the remote-edge kernels, enhance_global_connectivity, the three search launchers -- can be
// run as the reference for the oracle.  Nothing of RAFT or RMM is in here, and whatever would compute aborts: the
// oracle never calls the functions that use them.
#pragma once
#include <cuda_runtime.h>

#include <cfloat>   // the real headers bring FLT_MAX along; the reference's file relies on that
#include <cstddef>
#include <cstdio>
#include <cstdlib>

namespace grab_shim {
[[noreturn]] inline void unavailable(const char* what) {
  fprintf(stderr, "raft/rmm shim: %s is not available (RAFT and RMM are not installed)\n", what);
  abort();
}
}  // namespace grab_shim

namespace rmm {
struct cuda_stream_view {
  cudaStream_t s = nullptr;
  cuda_stream_view() = default;
  cuda_stream_view(cudaStream_t st) : s(st) {}
  cudaStream_t value() const { return s; }
};
namespace mr {
struct device_memory_resource {};
struct cuda_memory_resource : device_memory_resource {};
inline device_memory_resource* set_current_device_resource(device_memory_resource* r) { return r; }
}  // namespace mr
template <class T>
struct device_uvector {
  device_uvector(std::size_t, cuda_stream_view) { grab_shim::unavailable("rmm::device_uvector"); }
  T* data() { return nullptr; }
  std::size_t size() const { return 0; }
};
}  // namespace rmm

namespace raft {
struct device_resources {
  device_resources() = default;
  device_resources(cudaStream_t) {}
  device_resources(rmm::cuda_stream_view) {}
  void sync_stream() const { grab_shim::unavailable("raft::device_resources::sync_stream"); }
};
}  // namespace raft
