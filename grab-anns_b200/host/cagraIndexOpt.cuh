// cagra::CagraIndexOpt -- the time-partitioned index, same public surface as the reference
// class (src/cagraIndexOpt.cuh:13-155): add / build / insert / query / query_local
// (search_bucket) / query_range (search_range) / save / load.
//
// The reference equates "timestamp" with "bucket id" (one bucket per distinct timestamp,
// src/cagraIndexOpt.cu:168-184).  Here the filter predicate runs on the raw timestamps and the
// graph layout uses bucket = timestamp / bucket_width; with the default width 1 both coincide
// with the reference.  query_range_batch takes one range per query (the reference takes one per
// call).
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

class CagraIndexOpt {
 public:
  CagraIndexOpt(uint32_t dim, uint32_t graph_degree = 32, uint32_t local_degree = 16,
                size_t vmm_max_bytes = 20ULL * 1024 * 1024 * 1024);
  ~CagraIndexOpt();

  void add(size_t num_vectors, const float* add_vectors, const uint64_t* add_timestamps);
  void build();
  void insert(size_t new_vectors, const float* insert_vectors, const uint64_t* insert_timestamps);
  void query(const float* host_queries, size_t num_queries, int k, uint64_t min_ts, uint64_t max_ts,
             int64_t* host_indices, float* host_dists, const uint32_t* seeds = nullptr,
             size_t num_seeds_per_query = 0);
  void query_local(const float* host_queries, size_t num_queries, int k, uint64_t target_timestamp,
                   int64_t* host_indices, float* host_dists, uint32_t local_degree);
  void query_range(const float* host_queries, size_t num_queries, int k, uint64_t start_bucket, uint64_t end_bucket,
                   int64_t* host_indices, float* host_dists, uint32_t local_degree);
  // one [start, end) per query; timestamps, not bucket ids
  void query_range_batch(const float* host_queries, size_t num_queries, int k, const uint64_t* start_ts,
                         const uint64_t* end_ts, int64_t* host_indices, float* host_dists);

  void setBuildParams(uint32_t inter_degree, uint32_t graph_degree) {
    build_params_.intermediate_degree = inter_degree;
    build_params_.graph_degree = graph_degree;
  }
  void setQueryParams(uint32_t itopk_size, uint32_t search_width, uint32_t min_iterations, uint32_t max_iterations,
                      uint32_t hash_bitlen) {
    search_params_ = {itopk_size, search_width, min_iterations, max_iterations, hash_bitlen};
  }
  const float* get_data() const { return h_data_.data(); }
  uint32_t* get_graph();
  std::vector<uint32_t> get_ids_by_timestamp(uint64_t ts) const;
  size_t size() const { return current_size_; }
  std::vector<uint32_t> sample_seeds_by_time(uint64_t min_ts, uint64_t max_ts, size_t num) const;
  void save(const std::string& filepath);
  void load(const std::string& filepath);

  // additions (not in the reference)
  void setBucketWidth(uint64_t width) { bucket_width_ = width ? width : 1; }
  void setMetric(int metric) { metric_ = metric; }
  void setKnnPrecision(int precision) { knn_precision_ = precision; }
  void setSeed(uint64_t seed) { seed_ = seed; }
  void setInsertBatch(size_t batch) { insert_batch_ = batch ? batch : 4096; }
  // Small requests.  ctas_per_query: CTAs that co-operate on one query when the batch would leave most of the GPU
  // idle (GRAB_CTAS_AUTO = as many as fill it, the default; 1 = the reference's one CTA per query, bit-compatible
  // with the stateless search).  exact_below: a single-range query whose range holds at most this many vectors is
  // answered by an exact scan of the range instead of a graph walk (0 = never): with so few vectors in range the
  // filtered graph has no paths left between them, and the scan is both exact and cheaper.
  void setSmallBatchMode(uint32_t ctas_per_query, size_t exact_below) {
    ctas_per_query_ = ctas_per_query;
    exact_below_ = exact_below;
  }
  // Insert behaviour beyond the reference's.  routed: seeds of the insert searches come from the entry-point
  // router (needs setRouter != 0 and sorted timestamps; otherwise the reference's seed rule applies).
  // repair_mode: how a new node is linked back into the rows of the old nodes it points to --
  //   0  the reference's rule: a pseudo-random slot, 10 % strong / 90 % weak half (src/index/insert.cu:693-712);
  //   1  (default) every request still gets a slot, but the one of the FARTHEST old neighbour in the weak half;
  //   2  a request replaces the farthest neighbour of the region only when it is closer.
  void setInsertMode(bool routed, int repair_mode) {
    insert_routed_ = routed;
    insert_repair_mode_ = repair_mode;
  }
  void setInsertSearchParams(uint32_t itopk, uint32_t width, uint32_t max_iterations, uint32_t hash_bitlen) {
    insert_params_routed_ = {itopk, width, 0, max_iterations, hash_bitlen};
  }
  // Entry-point router: searches that get no seeds from the caller start from members of the
  // query's nearest k-means centroids that pass the filter, instead of uniformly drawn ids.
  // centroids = 0 switches it off (the reference's behaviour), kRouterAuto picks about sqrt(n).
  // The centroids are trained on the first query after build/load; inserts only re-assign.
  static constexpr uint32_t kRouterAuto = 0xFFFFFFFFu;
  void setRouter(uint32_t centroids, uint32_t probes = 2, uint32_t seeds_per_query = 64) {
    router_centroids_ = centroids;
    router_probes_ = probes ? probes : 2;
    router_seeds_ = seeds_per_query ? seeds_per_query : 64;
    router_.reset();
  }

 private:
  uint64_t bucket_of(uint64_t ts) const { return ts / bucket_width_; }
  void range_search(const float* host_queries, size_t nq, int k, const uint64_t* lo, const uint64_t* hi,
                    uint64_t lo1, uint64_t hi1, int64_t* ids, float* dists, bool exact = false);
  uint32_t dim_, graph_degree_;
  size_t current_size_ = 0;
  std::vector<float> h_data_;
  std::vector<uint32_t> h_graph_;
  std::unique_ptr<grab::DeviceBuffer> d_data_, d_graph_, d_ts_, d_bucket_;
  std::map<uint64_t, std::vector<uint32_t>> ts_to_ids_;  // bucket id -> ids
  std::vector<uint64_t> h_timestamps_;
  bool ts_sorted_ = true;
  grab_build_params build_params_;
  grab_search_params search_params_;
  size_t local_degree_;
  uint64_t bucket_width_ = 1;
  int metric_ = GRAB_METRIC_L2, knn_precision_ = GRAB_KNN_TC_SPLIT;
  uint64_t seed_ = 0x9E3779B97F4A7C15ull;
  std::unique_ptr<grab::QueryArena, grab::QueryArenaDeleter> arena_;
  // the reference inserts 32 at a time (src/cagraIndexOpt.cu:590); the sparse mailboxes and the
  // exact kNN inside the batch make four-digit batches as good and far faster
  size_t insert_batch_ = 4096;
  uint32_t ctas_per_query_ = GRAB_CTAS_AUTO;
  size_t exact_below_ = 1024;
  bool insert_routed_ = true;
  int insert_repair_mode_ = 1;
  grab_search_params insert_params_ = {128, 4, 0, 100, 13};         // src/cagraIndexOpt.cu:596-602
  grab_search_params insert_params_routed_ = {128, 4, 0, 16, 12};   // from routed seeds
  struct RouterState;
  struct RouterDeleter { void operator()(RouterState*) const; };
  const grab_router* ensure_router();  // nullptr when switched off or the index is too small
  uint32_t router_centroids_ = kRouterAuto, router_probes_ = 2, router_seeds_ = 64;
  std::unique_ptr<RouterState, RouterDeleter> router_;
};

}  // namespace cagra
