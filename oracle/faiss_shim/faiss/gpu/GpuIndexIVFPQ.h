// Test infrastructure: see StandardGpuResources.h in this directory.
#pragma once
#include <cstdint>

#include "StandardGpuResources.h"

namespace faiss {
namespace gpu {
struct GpuIndexIVFPQConfig {
  int device = 0;
  bool useFloat16LookupTables = false;
  bool usePrecomputedTables = false;
  bool interleavedLayout = false;
  bool use_cuvs = false;
  bool use_raft = false;
};
struct GpuIndexIVFPQ {
  int nprobe = 1;
  GpuIndexIVFPQ(StandardGpuResources*, int, int, int, int, MetricType, GpuIndexIVFPQConfig = GpuIndexIVFPQConfig()) {
    shim_unavailable("GpuIndexIVFPQ");
  }
  void train(int64_t, const float*) { shim_unavailable("GpuIndexIVFPQ::train"); }
  void add(int64_t, const float*) { shim_unavailable("GpuIndexIVFPQ::add"); }
  void search(int64_t, const float*, int64_t, float*, int64_t*) const { shim_unavailable("GpuIndexIVFPQ::search"); }
  void setNumProbes(int) { shim_unavailable("GpuIndexIVFPQ::setNumProbes"); }
};
}  // namespace gpu
}  // namespace faiss
