// cagra::CagraIndex -- same public surface as the reference class (src/cagraIndex.hpp:12-119):
// host pointers in and out, int64 ids, ascending distances.  Everything underneath goes
// through the C ABI of libgrab_anns (include/grab_anns.h) to hand-written sm_100a kernels.
// Failures surface as std::runtime_error (the reference exits the process on CUDA errors,
// src/index/cagra.cuh:9-17, and throws for file / allocator errors).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cagra.cuh"
#include "device_buffer.hpp"
#include "grab_anns.h"

namespace cagra {

class CagraIndex {
 public:
  // dim must be a multiple of 4.  vmm_max_bytes bounds the virtual address range the growable
  // device buffers reserve (70 % vectors, 20 % graph, 10 % timestamps, src/cagraIndex.cu:14-20);
  // physical memory is mapped as the index grows.
  CagraIndex(uint32_t dim,
             uint32_t graph_degree = 64,
             size_t vmm_max_bytes = 20ULL * 1024 * 1024 * 1024);
  ~CagraIndex();

  // Appends vectors to the host mirror; nothing is searchable before build().  Timestamps are
  // optional, but query_range needs them for every vector.
  void add(size_t num_vectors,
           const float* add_vectors,
           const uint64_t* add_timestamps = nullptr);

  // kNN graph (tensor-core all-pairs + exact re-rank) -> prune -> reverse -> merge, all on the
  // device (the reference: FAISS IVF-PQ candidates and host hops, src/cagraIndex.cu:80-124).
  void build();

  // Batched insert into a built index: search for neighbours among the existing nodes, write the
  // new rows, repair reverse edges (src/cagraIndex.cu:126-212).  Batch size: setInsertBatch.
  void insert(size_t new_vectors,
              const float* insert_vectors,
              const uint64_t* insert_timestamps = nullptr);

  // Unfiltered search.  host_indices [num_queries, k] int64 (-1 = none), host_dists ascending.
  // seeds: optional [num_queries, num_seeds_per_query] entry points.
  void query(const float* host_queries,
             size_t num_queries,
             int k,
             int64_t* host_indices,
             float* host_dists,
             uint32_t* seeds = nullptr,
             size_t num_seeds_per_query = 0);

  // Search among vectors with start_ts <= timestamp < end_ts.  range_radius >= 0.99 means "nearly
  // everything": the unfiltered search runs instead, as in the reference (src/cagraIndex.cu:305-338).
  void query_range(const float* host_queries,
                   size_t num_queries,
                   int k,
                   float range_radius,
                   uint64_t start_ts,
                   uint64_t end_ts,
                   int64_t* host_indices,
                   float* host_dists,
                   uint32_t* seeds = nullptr,
                   size_t num_seeds_per_query = 0);

  void setBuildParams(uint32_t inter_degree, uint32_t graph_degree) {
    build_params_.intermediate_degree = inter_degree;
    build_params_.graph_degree = graph_degree;
  }
  // Unlike the reference, insert() does not overwrite these (it has its own parameter set).
  void setQueryParams(uint32_t itopk_size,
                      uint32_t search_width,
                      uint32_t min_iterations,
                      uint32_t max_iterations,
                      uint32_t hash_bitlen) {
    search_params_ = {itopk_size, search_width, min_iterations, max_iterations, hash_bitlen};
  }

  void* get_data() { return h_data_.data(); }
  const uint32_t* get_graph();  // copies the device graph into the host mirror and returns it
  size_t size() const { return h_data_.size() / dim_; }

  // dim, degree, size, vectors, graph -- the reference's raw layout (src/cagraIndex.cu:352-395).
  void save(const std::string& filepath);
  void load(const std::string& filepath);

  // additions (not in the reference): metric, kNN precision of build(), reproducible seeds
  void setMetric(int metric) { metric_ = metric; }
  void setKnnPrecision(int precision) { knn_precision_ = precision; }
  void setSeed(uint64_t seed) { seed_ = seed; }
  void setInsertBatch(size_t batch) { insert_batch_ = batch ? batch : 64; }
  // Small requests.  ctas_per_query: CTAs that co-operate on one query when the batch would leave most of the GPU
  // idle (GRAB_CTAS_AUTO = as many as fill it, the default; 1 = the reference's one CTA per query, bit-compatible
  // with the stateless search).  exact_below: a single-range query whose range holds at most this many vectors is
  // answered by an exact scan of the range instead of a graph walk (0 = never): with so few vectors in range the
  // filtered graph has no paths left between them, and the scan is both exact and cheaper.
  void setSmallBatchMode(uint32_t ctas_per_query, size_t exact_below) {
    ctas_per_query_ = ctas_per_query;
    exact_below_ = exact_below;
  }

 private:
  void upload_timestamps();
  uint32_t dim_, graph_degree_;
  size_t current_size_ = 0;
  std::vector<float> h_data_;
  std::vector<uint32_t> h_graph_;
  std::map<uint64_t, std::vector<uint32_t>> ts_to_ids_;
  std::vector<uint64_t> h_timestamps_;
  bool ts_sorted_ = true;
  std::unique_ptr<grab::DeviceBuffer> d_ts_, d_data_, d_graph_;
  BuildParams build_params_;
  SearchParams search_params_, insert_params_;
  int metric_ = GRAB_METRIC_L2, knn_precision_ = GRAB_KNN_TC_SPLIT;
  uint64_t seed_ = 0x9E3779B97F4A7C15ull;
  std::unique_ptr<grab::QueryArena, grab::QueryArenaDeleter> arena_;
  size_t insert_batch_ = 64;  // the reference's batch (src/cagraIndex.cu:165)
  uint32_t ctas_per_query_ = GRAB_CTAS_AUTO;
  size_t exact_below_ = 1024;
};

}  // namespace cagra
