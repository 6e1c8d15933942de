// timestamp::TimeStampIndex -- two-level index, same public surface as the reference class
// (src/timeStampIndex.cuh:39-95): one CagraIndex per timestamp bucket plus a "virtual" index
// over per-bucket centroids that routes a query to `probe_buckets` buckets.  The reference
// builds the centroids with FAISS k-means (src/timeStampIndex.cu:169-179); here Lloyd's
// iterations run on the GPU with the exact nearest-centroid scan as the assignment step.
// query_by_timestamp is declared but never defined in the reference
// (src/timeStampIndex.cuh:59); it is defined here as a search inside one bucket.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <shared_mutex>
#include <vector>

#include "cagraIndex.hpp"

namespace timestamp {

struct VirtualPointMeta {
  uint64_t target_timestamp;
  std::vector<uint32_t> entry_points;  // local ids inside the bucket
};
struct BucketContext {
  std::vector<uint64_t> local_to_global;
  size_t num_dirty = 0;
};
struct VectorLocation {
  uint64_t timestamp;
  size_t local_index;
};

class TimeStampIndex {
 public:
  TimeStampIndex(uint32_t dim, uint32_t degree = 32, size_t cluster_ratio = 1000);
  ~TimeStampIndex();
  uint64_t insert(const float* vectors, const uint64_t* timestamps, size_t num_vectors);
  void build_virtual_index();
  void query(const float* query, size_t topk, int64_t* out_indices, float* out_dists, int probe_buckets = 5);
  void query_by_timestamp(const float* query, size_t topk, uint64_t timestamp, int64_t* out_indices,
                          float* out_dists);
  size_t size() const;

 private:
  std::pair<cagra::CagraIndex*, BucketContext*> get_or_create_bucket(uint64_t ts);
  uint32_t dim_, graph_degree_;
  size_t cluster_ratio_;
  uint64_t global_count_ = 0;
  mutable std::shared_mutex mutex_;
  std::map<uint64_t, std::unique_ptr<cagra::CagraIndex>> buckets_;
  std::map<uint64_t, BucketContext> bucket_contexts_;
  std::unique_ptr<cagra::CagraIndex> virtual_index_;
  std::vector<VirtualPointMeta> virtual_meta_;
  std::vector<VectorLocation> id_to_location_;
};

}  // namespace timestamp
