// Harness around the REFERENCE's own graph-optimisation functions (test infrastructure; built into
// oracle/_ref/libgrab_ref.so from the reference sources where they lie, never shipped).
//
// src/index/cagra.cu holds optimize_prune (:286-401, kernel kern_prune :219-276), optimize_create_reverse_graph
// (:455-548), optimize_merge_graphs (:574-650), build (:665-711) and the base search launcher (:844-935).  The file
// also holds generate_knn_graph, which calls FAISS-GPU; oracle/faiss_shim/ declares the few FAISS names that
// function mentions (every member aborts) so that the translation unit compiles; nothing here calls it.  The
// functions are called exactly as they are; exceptions and CUDA errors become return codes.
#include <cuda_runtime.h>

#include <cstdint>
#include <exception>

#include "cagra.cuh"

namespace {
template <class F>
int guarded(F&& f) {
  try {
    f();
  } catch (const std::exception&) {
    return -1;
  }
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
}  // namespace

// cagra.cuh:74-78.  HOST graphs.
extern "C" int ref_optimize_prune(const uint32_t* h_knn, uint32_t* h_out, uint64_t n, uint32_t in_deg, uint32_t out_deg) {
  return guarded([&] { cagra::optimize_prune(h_knn, h_out, n, in_deg, out_deg); });
}

// cagra.cuh:91-95.
extern "C" int ref_optimize_reverse(const uint32_t* h_graph, uint32_t* h_rev, uint32_t* h_counts, uint64_t n,
                                    uint32_t deg) {
  return guarded([&] { cagra::optimize_create_reverse_graph(h_graph, h_rev, h_counts, n, deg); });
}

// cagra.cuh:105-109.  h_graph is updated in place.
extern "C" int ref_optimize_merge(uint32_t* h_graph, const uint32_t* h_rev, const uint32_t* h_counts, uint64_t n,
                                  uint32_t deg) {
  return guarded([&] { cagra::optimize_merge_graphs(h_graph, h_rev, h_counts, n, deg); });
}

// cagra.cuh:115-119.  The graph build() allocates is copied to d_out [n, deg] and freed.
extern "C" int ref_build(const float* d_dataset, uint64_t n, const uint32_t* d_raw_knn, uint32_t inter_deg, uint32_t deg,
                         uint32_t* d_out) {
  return guarded([&] {
    cagra::BuildParams p;
    p.intermediate_degree = inter_deg;
    p.graph_degree = deg;
    uint32_t* d_graph = nullptr;
    cagra::build(d_dataset, n, d_raw_knn, p, &d_graph);
    cudaMemcpy(d_out, d_graph, sizeof(uint32_t) * n * deg, cudaMemcpyDeviceToDevice);
    cudaFree(d_graph);
  });
}
