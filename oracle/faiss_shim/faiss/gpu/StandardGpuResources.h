// Test infrastructure, not part of the product.  FAISS is not installed here; the reference's src/index/cagra.cu
// names a few FAISS-GPU classes in ONE function (generate_knn_graph, its IVF-PQ candidate search).  These
// declarations let that translation unit compile so that its other functions -- prune, reverse graph, merge, build,
// the base search launcher -- can be run as the reference for the oracle.  Nothing of FAISS is in here, and every
// member aborts: the oracle never calls the function that uses them.
#pragma once
#include <cstddef>
#include <cstdio>
#include <cstdlib>

namespace faiss {
enum MetricType { METRIC_INNER_PRODUCT = 0, METRIC_L2 = 1 };
namespace gpu {
[[noreturn]] inline void shim_unavailable(const char* what) {
  fprintf(stderr, "faiss shim: %s is not available (FAISS is not installed)\n", what);
  abort();
}
struct StandardGpuResources {
  void setTempMemory(size_t) { shim_unavailable("StandardGpuResources::setTempMemory"); }
};
}  // namespace gpu
}  // namespace faiss
