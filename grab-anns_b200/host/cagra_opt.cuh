// Source-level stand-in for the reference's src/index/cagra_opt.cuh (time-partitioned build, the three filtered
// searches and the time-partitioned insert): same names and argument order in namespace cagra, each an inline
// call into the C ABI of libgrab_anns.  A non-zero status becomes a std::runtime_error.
#pragma once
#include <vector>

#include "cagra.cuh"

namespace cagra {

// src/index/cagra_opt.cuh:21-31.  d_graph [total_num, total_degree] is written; d_ts holds the bucket id of
// every vector (device), bucket_sizes the vectors per bucket in id order.  h_ts is accepted for signature
// compatibility and not read (the device copy is the one used).
inline void build_time_partitioned_graph(const float* d_dataset, size_t total_num, uint32_t dim, uint32_t* d_graph,
                                         uint64_t* d_ts, uint64_t* /*h_ts*/, const std::vector<size_t>& bucket_sizes,
                                         uint32_t total_degree, uint32_t local_degree) {
  std::vector<uint64_t> sizes(bucket_sizes.begin(), bucket_sizes.end());
  detail::check(grab_build_time_partitioned_graph(d_dataset, total_num, dim, GRAB_METRIC_L2, d_graph, d_ts,
                                                  sizes.data(), static_cast<uint32_t>(sizes.size()), total_degree,
                                                  local_degree, GRAB_KNN_TC_SPLIT),
                "build_time_partitioned_graph");
}

// src/index/cagra_opt.cuh:33-46.
inline void search_opt(const float* d_dataset, uint32_t dim, size_t num_dataset, const uint32_t* d_graph,
                       uint32_t graph_degree, const float* d_queries, int64_t num_queries, int64_t k,
                       SearchParams params, int64_t* d_out_indices, float* d_out_dists, const uint32_t* d_seeds,
                       const uint32_t num_seeds_per_query, cudaStream_t stream = 0) {
  detail::check(grab_search(d_dataset, dim, num_dataset, d_graph, graph_degree, d_queries, num_queries, k, params,
                            d_out_indices, d_out_dists, d_seeds, num_seeds_per_query, stream),
                "search_opt");
}

// src/index/cagra_opt.cuh:48-62.  Only the first local_degree columns are followed, so a search seeded inside a
// bucket stays inside it.
inline void search_bucket_opt(const float* d_dataset, uint32_t dim, size_t num_dataset, const uint32_t* d_graph,
                              uint32_t total_degree, uint32_t local_degree, const float* d_queries,
                              int64_t num_queries, int64_t k, SearchParams params, int64_t* d_out_indices,
                              float* d_out_dists, const uint32_t* d_seeds, const uint32_t num_seeds_per_query,
                              cudaStream_t stream = 0) {
  detail::check(grab_search_bucket(d_dataset, dim, num_dataset, d_graph, total_degree, local_degree, d_queries,
                                   num_queries, k, params, d_out_indices, d_out_dists, d_seeds, num_seeds_per_query,
                                   stream),
                "search_bucket_opt");
}

// src/index/cagra_opt.cuh:64-80.  Results have start_bucket <= d_ts[id] < end_bucket.
inline void search_bucket_range(const float* d_dataset, uint32_t dim, size_t num_dataset, const uint32_t* d_graph,
                                uint64_t* d_ts, uint32_t total_degree, uint32_t local_degree, const float* d_queries,
                                int64_t num_queries, int64_t k, uint64_t start_bucket, uint64_t end_bucket,
                                SearchParams params, int64_t* d_out_indices, float* d_out_dists,
                                const uint32_t* d_seeds, const uint32_t num_seeds_per_query) {
  detail::check(grab_search_range(d_dataset, dim, num_dataset, d_graph, d_ts, total_degree, local_degree, d_queries,
                                  num_queries, k, start_bucket, end_bucket, params, d_out_indices, d_out_dists,
                                  d_seeds, num_seeds_per_query),
                "search_bucket_range");
}

// src/index/cagra_opt.cuh:82-95.  All new vectors belong to bucket target_ts.
inline void insert(const float* d_dataset, uint32_t* d_graph, const uint64_t* d_ts, const uint32_t* d_seeds,
                   size_t num_existing, size_t num_new, bool use_heuristic, int target_ts, const float* d_queries,
                   uint32_t dim, uint32_t total_degree, uint32_t local_degree, SearchParams params,
                   uint32_t num_seeds_per_query) {
  detail::check(grab_insert_opt(d_dataset, d_graph, d_ts, d_seeds, num_existing, num_new, use_heuristic ? 1 : 0,
                                static_cast<uint64_t>(target_ts), d_queries, dim, total_degree, local_degree, params,
                                num_seeds_per_query),
                "insert");
}

}  // namespace cagra
