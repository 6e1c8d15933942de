// C handles over the index classes (include/grab_index.h).
#include <cstring>
#include <exception>
#include <mutex>
#include <string>
#include <unordered_map>

#include "cagraIndex.hpp"
#include "cagraIndexOpt.cuh"
#include "../csrc/common.cuh"
#include "grab_index.h"
#include "timeStampIndex.cuh"

namespace {
template <class F>
int guarded(F&& f) {
  try {
    f();
    return GRAB_OK;
  } catch (const grab::StatusError& e) {  // CUDA failures, out of memory, file errors, device-side timeouts
    grab::set_last_error("%s", e.what());
    return e.status;
  } catch (const std::exception& e) {
    grab::set_last_error("%s", e.what());
    return GRAB_ERR_INVALID_ARGUMENT;
  } catch (...) {
    grab::set_last_error("unknown exception");
    return GRAB_ERR_INVALID_ARGUMENT;
  }
}
// Every handle belongs to the GPU that was current (or named, *_create_on) when it was made: calls through the
// handle run on that device whatever the calling thread's current device is, and leave the caller's device as it was.
std::mutex g_device_mutex;
std::unordered_map<void*, int> g_device_of;

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int device) {
    if (device < 0) return;
    if (cudaGetDevice(&prev) != cudaSuccess) throw grab::StatusError(GRAB_ERR_CUDA, "cudaGetDevice failed");
    if (prev != device) {
      if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();  // a refused device id must not linger as the thread's "last error" for other CUDA users
        throw grab::StatusError(GRAB_ERR_CUDA, "cudaSetDevice(" + std::to_string(device) + ") failed");
      }
      switched = true;
    }
  }
  ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
};

int device_of(void* h) {
  std::lock_guard<std::mutex> lock(g_device_mutex);
  auto it = g_device_of.find(h);
  return it == g_device_of.end() ? -1 : it->second;
}

// device < 0: the calling thread's current device
template <class F>
void* create_on(int device, F&& make) {
  void* out = nullptr;
  guarded([&] {
    DeviceGuard g(device);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw grab::StatusError(GRAB_ERR_CUDA, "cudaGetDevice failed");
    out = make();
    std::lock_guard<std::mutex> lock(g_device_mutex);
    g_device_of[out] = dev;
  });
  return out;
}

template <class F>
int guarded_on(void* h, F&& f) {
  return guarded([&] {
    DeviceGuard g(device_of(h));
    f();
  });
}

template <class T>
void destroy(void* h) {
  if (!h) return;
  guarded_on(h, [&] { delete static_cast<T*>(h); });
  std::lock_guard<std::mutex> lock(g_device_mutex);
  g_device_of.erase(h);
}

cagra::CagraIndexOpt* O(void* h) { return static_cast<cagra::CagraIndexOpt*>(h); }
cagra::CagraIndex* I(void* h) { return static_cast<cagra::CagraIndex*>(h); }
timestamp::TimeStampIndex* T(void* h) { return static_cast<timestamp::TimeStampIndex*>(h); }
}  // namespace

extern "C" {

void* grab_index_opt_create(uint32_t dim, uint32_t graph_degree, uint32_t local_degree, size_t vmm_max_bytes) {
  return grab_index_opt_create_on(-1, dim, graph_degree, local_degree, vmm_max_bytes);
}
void* grab_index_opt_create_on(int device, uint32_t dim, uint32_t graph_degree, uint32_t local_degree,
                               size_t vmm_max_bytes) {
  return create_on(device, [&]() -> void* { return new cagra::CagraIndexOpt(dim, graph_degree, local_degree, vmm_max_bytes); });
}
void grab_index_opt_destroy(void* h) { destroy<cagra::CagraIndexOpt>(h); }
int grab_index_opt_configure(void* h, uint64_t bucket_width, int metric, int knn_precision, uint64_t seed,
                             size_t insert_batch) {
  return guarded_on(h, [&] {
    O(h)->setBucketWidth(bucket_width); O(h)->setMetric(metric); O(h)->setKnnPrecision(knn_precision);
    O(h)->setSeed(seed); O(h)->setInsertBatch(insert_batch);
  });
}
int grab_index_opt_set_query_params(void* h, uint32_t itopk, uint32_t width, uint32_t min_iter, uint32_t max_iter,
                                    uint32_t hash_bitlen) {
  return guarded_on(h, [&] { O(h)->setQueryParams(itopk, width, min_iter, max_iter, hash_bitlen); });
}
int grab_index_opt_set_router(void* h, uint32_t centroids, uint32_t probes, uint32_t seeds_per_query) {
  return guarded_on(h, [&] { O(h)->setRouter(centroids, probes, seeds_per_query); });
}
int grab_index_opt_set_insert_mode(void* h, int routed, int repair_mode) {
  return guarded_on(h, [&] { O(h)->setInsertMode(routed != 0, repair_mode); });
}
int grab_index_opt_set_insert_search_params(void* h, uint32_t itopk, uint32_t width, uint32_t max_iter,
                                            uint32_t hash_bitlen) {
  return guarded_on(h, [&] { O(h)->setInsertSearchParams(itopk, width, max_iter, hash_bitlen); });
}
int grab_index_opt_set_small_batch_mode(void* h, uint32_t ctas_per_query, size_t exact_below) {
  return guarded_on(h, [&] { O(h)->setSmallBatchMode(ctas_per_query, exact_below); });
}
int grab_index_opt_add(void* h, size_t n, const float* v, const uint64_t* ts) { return guarded_on(h, [&] { O(h)->add(n, v, ts); }); }
int grab_index_opt_build(void* h) { return guarded_on(h, [&] { O(h)->build(); }); }
int grab_index_opt_insert(void* h, size_t n, const float* v, const uint64_t* ts) { return guarded_on(h, [&] { O(h)->insert(n, v, ts); }); }
int grab_index_opt_query(void* h, const float* q, size_t nq, int k, int64_t* ids, float* dists) {
  return guarded_on(h, [&] { O(h)->query(q, nq, k, 0, 0, ids, dists); });
}
int grab_index_opt_query_local(void* h, const float* q, size_t nq, int k, uint64_t target, int64_t* ids, float* dists) {
  return guarded_on(h, [&] { O(h)->query_local(q, nq, k, target, ids, dists, 0); });
}
int grab_index_opt_query_range(void* h, const float* q, size_t nq, int k, uint64_t s, uint64_t e, int64_t* ids, float* dists) {
  return guarded_on(h, [&] { O(h)->query_range(q, nq, k, s, e, ids, dists, 0); });
}
int grab_index_opt_query_range_batch(void* h, const float* q, size_t nq, int k, const uint64_t* s, const uint64_t* e,
                                     int64_t* ids, float* dists) {
  return guarded_on(h, [&] { O(h)->query_range_batch(q, nq, k, s, e, ids, dists); });
}
int grab_index_opt_get_graph(void* h, uint32_t* out, size_t cap) {
  return guarded_on(h, [&] {
    const uint32_t* g = O(h)->get_graph();
    (void)g;
    // the graph width is not stored in the handle API: copy what fits
    memcpy(out, g, cap * sizeof(uint32_t));
  });
}
size_t grab_index_opt_size(void* h) { return O(h)->size(); }
int grab_index_opt_save(void* h, const char* p) { return guarded_on(h, [&] { O(h)->save(p); }); }
int grab_index_opt_load(void* h, const char* p) { return guarded_on(h, [&] { O(h)->load(p); }); }

void* grab_index_create(uint32_t dim, uint32_t graph_degree, size_t vmm_max_bytes) {
  return grab_index_create_on(-1, dim, graph_degree, vmm_max_bytes);
}
void* grab_index_create_on(int device, uint32_t dim, uint32_t graph_degree, size_t vmm_max_bytes) {
  return create_on(device, [&]() -> void* { return new cagra::CagraIndex(dim, graph_degree, vmm_max_bytes); });
}
void grab_index_destroy(void* h) { destroy<cagra::CagraIndex>(h); }
int grab_index_configure(void* h, int metric, int knn_precision, uint64_t seed, size_t insert_batch) {
  return guarded_on(h, [&] { I(h)->setMetric(metric); I(h)->setKnnPrecision(knn_precision); I(h)->setSeed(seed); I(h)->setInsertBatch(insert_batch); });
}
int grab_index_set_small_batch_mode(void* h, uint32_t ctas_per_query, size_t exact_below) {
  return guarded_on(h, [&] { I(h)->setSmallBatchMode(ctas_per_query, exact_below); });
}
int grab_index_set_query_params(void* h, uint32_t itopk, uint32_t width, uint32_t min_iter, uint32_t max_iter,
                                uint32_t hash_bitlen) {
  return guarded_on(h, [&] { I(h)->setQueryParams(itopk, width, min_iter, max_iter, hash_bitlen); });
}
int grab_index_add(void* h, size_t n, const float* v, const uint64_t* ts) { return guarded_on(h, [&] { I(h)->add(n, v, ts); }); }
int grab_index_build(void* h) { return guarded_on(h, [&] { I(h)->build(); }); }
int grab_index_insert(void* h, size_t n, const float* v, const uint64_t* ts) { return guarded_on(h, [&] { I(h)->insert(n, v, ts); }); }
int grab_index_query(void* h, const float* q, size_t nq, int k, int64_t* ids, float* dists) {
  return guarded_on(h, [&] { I(h)->query(q, nq, k, ids, dists); });
}
int grab_index_query_range(void* h, const float* q, size_t nq, int k, float radius, uint64_t s, uint64_t e, int64_t* ids,
                           float* dists) {
  return guarded_on(h, [&] { I(h)->query_range(q, nq, k, radius, s, e, ids, dists); });
}
int grab_index_get_graph(void* h, uint32_t* out, size_t cap) {
  return guarded_on(h, [&] { memcpy(out, I(h)->get_graph(), cap * sizeof(uint32_t)); });
}
size_t grab_index_size(void* h) { return I(h)->size(); }
int grab_index_save(void* h, const char* p) { return guarded_on(h, [&] { I(h)->save(p); }); }
int grab_index_load(void* h, const char* p) { return guarded_on(h, [&] { I(h)->load(p); }); }

void* grab_tsindex_create(uint32_t dim, uint32_t degree, size_t cluster_ratio) {
  return grab_tsindex_create_on(-1, dim, degree, cluster_ratio);
}
void* grab_tsindex_create_on(int device, uint32_t dim, uint32_t degree, size_t cluster_ratio) {
  return create_on(device, [&]() -> void* { return new timestamp::TimeStampIndex(dim, degree, cluster_ratio); });
}
void grab_tsindex_destroy(void* h) { destroy<timestamp::TimeStampIndex>(h); }
int grab_tsindex_insert(void* h, const float* v, const uint64_t* ts, size_t n, uint64_t* first_id) {
  return guarded_on(h, [&] { const uint64_t id = T(h)->insert(v, ts, n); if (first_id) *first_id = id; });
}
int grab_tsindex_build_virtual_index(void* h) { return guarded_on(h, [&] { T(h)->build_virtual_index(); }); }
int grab_tsindex_query(void* h, const float* q, size_t topk, int64_t* ids, float* dists, int probe) {
  return guarded_on(h, [&] { T(h)->query(q, topk, ids, dists, probe); });
}
int grab_tsindex_query_by_timestamp(void* h, const float* q, size_t topk, uint64_t ts, int64_t* ids, float* dists) {
  return guarded_on(h, [&] { T(h)->query_by_timestamp(q, topk, ts, ids, dists); });
}
size_t grab_tsindex_size(void* h) { return T(h)->size(); }

}  // extern "C"
