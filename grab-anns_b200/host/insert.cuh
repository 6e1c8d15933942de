// Source-level stand-in for the host-callable part of the reference's src/index/insert.cuh: the neighbour search
// for new vectors and the two topology updates, same names and argument order in namespace cagra.  The
// reference's header also declares its kernels (fill / generate / apply); those are internal here.
#pragma once
#include "cagra.cuh"

namespace cagra {

// src/index/insert.cuh:38-48.  Searches the first num_existing nodes for the search_k nearest of every new
// vector; exact distances, ascending.
inline void find_near_nodes(const float* d_dataset, uint32_t dim, size_t num_existing, size_t num_new,
                            const float* d_new_data, const uint32_t* d_graph, uint32_t graph_degree,
                            uint32_t search_k, SearchParams params, int64_t* d_out_indices, float* d_out_dists) {
  detail::check(grab_find_near_nodes(d_dataset, num_existing, d_new_data, num_new, d_graph, dim, graph_degree,
                                     search_k, params, d_out_indices, d_out_dists),
                "find_near_nodes");
}

// src/index/insert.cuh:62-72 (insert.cu:372-440).  New rows from the search results, then one reverse edge per
// (old node, new node) request into a pseudo-random slot of the old node's weak half.
inline void update_topology_gpu_v1(uint32_t* d_graph, const int64_t* d_search_indices, size_t num_existing,
                                   size_t num_new, uint32_t graph_degree, uint32_t search_k) {
  detail::check(grab_update_topology_v1(d_graph, d_search_indices, num_existing, num_new, graph_degree, search_k,
                                        nullptr),
                "update_topology_gpu_v1");
  CUDA_CHECK(cudaDeviceSynchronize());
}

// src/index/insert.cuh:96-116 (insert.cu:1398-1573).  Local and global search results of the new vectors ->
// new rows (local columns from the bucket, remote columns from the rest) and mailbox-based reverse edges.  The
// distance arrays, the dataset and use_heuristic are part of the reference's signature; the slot rule it
// applies (the one reproduced here) reads none of them.
inline void update_topology_gpu_opt(uint32_t* d_graph, const float* /*d_dataset*/, size_t /*dim*/, size_t target_ts,
                                    const uint64_t* d_ts, int64_t* d_search_indices, float* /*d_search_dists*/,
                                    int64_t* d_search_global, float* /*d_search_global_dists*/, size_t num_existing,
                                    size_t num_new, uint32_t total_degree, uint32_t local_degree,
                                    uint32_t search_k_local, uint32_t search_k_global,
                                    bool /*use_heuristic*/ = false) {
  detail::check(grab_update_topology_opt(d_graph, d_ts, d_search_indices, d_search_global, num_existing, num_new,
                                         target_ts, total_degree, local_degree, search_k_local, search_k_global,
                                         nullptr),
                "update_topology_gpu_opt");
  CUDA_CHECK(cudaDeviceSynchronize());
}

}  // namespace cagra
