// Source-level stand-in for the reference's stateless header src/index/cagra.cuh: the same names, argument
// order and defaults in namespace cagra, each function a thin inline call into the C ABI of libgrab_anns
// (include/grab_anns.h).  Code written against the reference's header -- its own tests/test_knn_build.cu and
// tests/test_cagra_build.cu, for instance -- compiles against this one unchanged.
// Errors: the reference prints and exits the process on a CUDA error (src/index/cagra.cuh:9-17); here a
// non-zero status becomes a std::runtime_error carrying grab_last_error().
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "config.cuh"
#include "grab_anns.h"

#ifndef CUDA_CHECK
#define CUDA_CHECK(call)                                                                              \
  do {                                                                                                \
    cudaError_t err = call;                                                                           \
    if (err != cudaSuccess) {                                                                         \
      fprintf(stderr, "CUDA Error: %s at %s:%d\n", cudaGetErrorString(err), __FILE__, __LINE__);      \
      exit(1);                                                                                        \
    }                                                                                                 \
  } while (0)
#endif

namespace cagra {

constexpr int MAX_DEGREE = 512;  // src/index/cagra.cuh:21

// src/index/cagra.cuh:30-42: same fields and defaults; layout-compatible with the C structs they derive from.
struct BuildParams : grab_build_params {
  BuildParams() : grab_build_params{128, 64} {}
  BuildParams(uint32_t intermediate, uint32_t degree) : grab_build_params{intermediate, degree} {}
  BuildParams(const grab_build_params& p) : grab_build_params(p) {}
};
struct SearchParams : grab_search_params {
  SearchParams() : grab_search_params{64, 5, 0, 20, 12} {}
  SearchParams(uint32_t itopk, uint32_t width, uint32_t min_iter, uint32_t max_iter, uint32_t hash_bitlen)
      : grab_search_params{itopk, width, min_iter, max_iter, hash_bitlen} {}
  SearchParams(const grab_search_params& p) : grab_search_params(p) {}
  static constexpr uint32_t TEAM_SIZE = 8;  // lanes per vector here (the reference: 32)
};

namespace detail {
inline void check(int status, const char* what) {
  if (status != GRAB_OK) throw std::runtime_error(std::string(what) + ": " + grab_last_error());
}
}  // namespace detail

// src/index/cagra.cuh:59-63.  Device dataset, HOST output [num_dataset, k], self excluded, ascending distance.
inline void generate_knn_graph(const float* d_dataset, size_t num_dataset, uint32_t dim, uint32_t k,
                               uint32_t* h_knn_graph) {
  detail::check(grab_generate_knn_graph(d_dataset, num_dataset, dim, k, h_knn_graph), "generate_knn_graph");
}

// src/index/cagra.cuh:74-78.  Host graphs in and out.
inline void optimize_prune(const uint32_t* h_knn_graph, uint32_t* h_new_graph, size_t num_dataset,
                           uint32_t input_degree, uint32_t output_degree) {
  detail::check(grab_optimize_prune(h_knn_graph, h_new_graph, num_dataset, input_degree, output_degree),
                "optimize_prune");
}

// src/index/cagra.cuh:91-95.
inline void optimize_create_reverse_graph(const uint32_t* h_input_graph, uint32_t* h_rev_graph,
                                          uint32_t* h_rev_counts, size_t num_dataset, uint32_t degree) {
  detail::check(grab_optimize_create_reverse_graph(h_input_graph, h_rev_graph, h_rev_counts, num_dataset, degree),
                "optimize_create_reverse_graph");
}

// src/index/cagra.cuh:105-109.  h_graph is updated in place.
inline void optimize_merge_graphs(uint32_t* h_graph, const uint32_t* h_rev_graph, const uint32_t* h_rev_counts,
                                  size_t num_dataset, uint32_t degree) {
  detail::check(grab_optimize_merge_graphs(h_graph, h_rev_graph, h_rev_counts, num_dataset, degree),
                "optimize_merge_graphs");
}

// src/index/cagra.cuh:115-119.  *d_constructed_graph is cudaMalloc'd here and freed by the caller.
inline void build(const float* d_dataset, size_t num_dataset, const uint32_t* d_raw_knn_graph, BuildParams params,
                  uint32_t** d_constructed_graph) {
  detail::check(grab_build(d_dataset, num_dataset, d_raw_knn_graph, params, d_constructed_graph), "build");
}

// src/index/cagra.cuh:124-137.  Device pointers; ids int64, ascending distances.
inline void search(const float* d_dataset, size_t num_dataset, uint32_t dim, const uint32_t* d_graph,
                   uint32_t graph_degree, const float* d_queries, int64_t num_queries, int64_t k,
                   SearchParams params, int64_t* d_out_indices, float* d_out_dists,
                   const uint32_t* d_seeds = nullptr, const uint32_t num_seeds = 0) {
  detail::check(grab_search(d_dataset, dim, num_dataset, d_graph, graph_degree, d_queries, num_queries, k, params,
                            d_out_indices, d_out_dists, d_seeds, num_seeds, nullptr),
                "search");
}

// src/index/cagra.cuh:139-146.  The new vectors become rows [num_existing, num_existing + num_new) of the device
// graph; h_graph is accepted and left untouched, as the reference's body does (src/index/cagra.cu:938-1010 works
// on the device graph only).  The reference compiles the dimension in (config::DIM); here it is a trailing
// argument with that default.
inline void insert(const float* d_dataset, size_t num_existing, size_t num_new, const float* d_new_data,
                   uint32_t* d_graph, uint32_t* /*h_graph*/, uint32_t graph_degree, SearchParams search_params,
                   uint32_t dim = config::DIM) {
  detail::check(grab_insert(d_dataset, num_existing, num_new, d_new_data, d_graph, dim, graph_degree, search_params),
                "insert");
}

}  // namespace cagra
