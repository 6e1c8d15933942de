// timestamp::TimeStampIndex -- two-level index, same public surface as the reference class
// (src/timeStampIndex.cuh:39-95): one CagraIndex per timestamp bucket plus a "virtual" index
// over per-bucket centroids that routes a query to `probe_buckets` buckets.  The reference
// builds the centroids with FAISS k-means (src/timeStampIndex.cu:169-179); here Lloyd's
// iterations run on the device (grab_router_build: tiled nearest-centroid kernel, ordered means).
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
  // One CagraIndex of the given degree per distinct timestamp.  cluster_ratio is kept for source
  // compatibility; the number of centroids per bucket follows the reference's 16 * sqrt(n) rule
  // (src/timeStampIndex.cu:169-179).
  TimeStampIndex(uint32_t dim,
                 uint32_t degree = 32,
                 size_t cluster_ratio = 1000);
  ~TimeStampIndex();

  // Appends vectors to the buckets of their timestamps (CagraIndex::insert per bucket; a bucket is
  // created on first use).  Returns the global id of the first vector; ids are consecutive.  Takes
  // the writer lock.
  uint64_t insert(const float* vectors,
                  const uint64_t* timestamps,
                  size_t num_vectors);

  // k-means centroids of every bucket (on the device), up to five entry points per centroid, and a
  // CagraIndex over all centroids -- the router (src/timeStampIndex.cu:141-238).  Writer lock.
  void build_virtual_index();

  // One query: nearest centroids vote for buckets, the probe_buckets best are searched from their entry
  // points, the per-bucket results are merged by distance (src/timeStampIndex.cu:240-419).  Reader lock;
  // may be called from several threads.
  void query(const float* query,
             size_t topk,
             int64_t* out_indices,
             float* out_dists,
             int probe_buckets = 5);

  // Search inside the bucket of one timestamp (declared but never defined in the reference).
  void query_by_timestamp(const float* query,
                          size_t topk,
                          uint64_t timestamp,
                          int64_t* out_indices,
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
