/*
 * grab_index.h -- C handles over the three index classes, for hosts that cannot include C++
 * (the tests and the benchmark drive them through ctypes).  The reference exposes the classes
 * only (src/cagraIndex.hpp:12, src/cagraIndexOpt.cuh:13, src/timeStampIndex.cuh:39); each
 * function below forwards to the method of the same name.  All pointers are HOST pointers, as
 * in the classes.  Exceptions become a status; the message is in grab_last_error().
 */
#ifndef GRAB_INDEX_H_
#define GRAB_INDEX_H_
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* cagra::CagraIndexOpt */
void* grab_index_opt_create(uint32_t dim, uint32_t graph_degree, uint32_t local_degree, size_t vmm_max_bytes);
/* The same on a named GPU.  A handle belongs to the device it was made on (the calling thread's current one for the
 * plain *_create): every call through it runs there whatever the caller's current device is, and leaves the
 * caller's device as it was -- one host thread can drive indexes on several GPUs.  The reference compiles one
 * device id in (src/index/common.cuh:5-7). */
void* grab_index_opt_create_on(int device, uint32_t dim, uint32_t graph_degree, uint32_t local_degree,
                               size_t vmm_max_bytes);
void grab_index_opt_destroy(void* h);
int grab_index_opt_configure(void* h, uint64_t bucket_width, int metric, int knn_precision, uint64_t seed,
                             size_t insert_batch);
int grab_index_opt_set_query_params(void* h, uint32_t itopk, uint32_t width, uint32_t min_iter, uint32_t max_iter,
                                    uint32_t hash_bitlen);
/* Entry-point router of the searches that get no seeds from the caller: centroids = 0 off,
 * 0xFFFFFFFF (default) about sqrt(n); probes / seeds_per_query = 0 keep 2 / 64. */
int grab_index_opt_set_router(void* h, uint32_t centroids, uint32_t probes, uint32_t seeds_per_query);
/* Insert behaviour beyond the reference's.  routed (default 1) = the insert searches start from the router's
 * seeds (needs a router and sorted timestamps).  repair_mode = how a new node is linked back into the rows of the
 * old nodes it points to: 0 the reference's pseudo-random slot (src/index/insert.cu:693-712); 1 (default) every
 * request still gets a slot, the one of the farthest old neighbour in the weak half; 2 only requests closer than
 * the region's farthest neighbour replace it.  0 / 0 restores the reference's rules. */
int grab_index_opt_set_insert_mode(void* h, int routed, int repair_mode);
/* Search parameters of routed inserts (default itopk 128, width 4, 16 iterations, hash 2^12). */
int grab_index_opt_set_insert_search_params(void* h, uint32_t itopk, uint32_t width, uint32_t max_iter,
                                            uint32_t hash_bitlen);
/* Small requests: ctas_per_query as in grab_search_args (GRAB_CTAS_AUTO is the default of the classes); a
 * single-range query whose range holds at most exact_below vectors (default 1024, 0 = never) is answered by an
 * exact scan of the range.  No counterpart in the reference. */
int grab_index_opt_set_small_batch_mode(void* h, uint32_t ctas_per_query, size_t exact_below);
int grab_index_opt_add(void* h, size_t n, const float* vectors, const uint64_t* timestamps);
int grab_index_opt_build(void* h);
int grab_index_opt_insert(void* h, size_t n, const float* vectors, const uint64_t* timestamps);
int grab_index_opt_query(void* h, const float* queries, size_t nq, int k, int64_t* ids, float* dists);
int grab_index_opt_query_local(void* h, const float* queries, size_t nq, int k, uint64_t target_timestamp,
                               int64_t* ids, float* dists);
int grab_index_opt_query_range(void* h, const float* queries, size_t nq, int k, uint64_t start, uint64_t end,
                               int64_t* ids, float* dists);
int grab_index_opt_query_range_batch(void* h, const float* queries, size_t nq, int k, const uint64_t* start,
                                     const uint64_t* end, int64_t* ids, float* dists);
int grab_index_opt_get_graph(void* h, uint32_t* out, size_t capacity_words);
size_t grab_index_opt_size(void* h);
int grab_index_opt_save(void* h, const char* path);
int grab_index_opt_load(void* h, const char* path);

/* cagra::CagraIndex */
void* grab_index_create(uint32_t dim, uint32_t graph_degree, size_t vmm_max_bytes);
void* grab_index_create_on(int device, uint32_t dim, uint32_t graph_degree, size_t vmm_max_bytes);
void grab_index_destroy(void* h);
int grab_index_configure(void* h, int metric, int knn_precision, uint64_t seed, size_t insert_batch);
int grab_index_set_small_batch_mode(void* h, uint32_t ctas_per_query, size_t exact_below);
int grab_index_set_query_params(void* h, uint32_t itopk, uint32_t width, uint32_t min_iter, uint32_t max_iter,
                                uint32_t hash_bitlen);
int grab_index_add(void* h, size_t n, const float* vectors, const uint64_t* timestamps_or_null);
int grab_index_build(void* h);
int grab_index_insert(void* h, size_t n, const float* vectors, const uint64_t* timestamps_or_null);
int grab_index_query(void* h, const float* queries, size_t nq, int k, int64_t* ids, float* dists);
int grab_index_query_range(void* h, const float* queries, size_t nq, int k, float range_radius, uint64_t start,
                           uint64_t end, int64_t* ids, float* dists);
int grab_index_get_graph(void* h, uint32_t* out, size_t capacity_words);
size_t grab_index_size(void* h);
int grab_index_save(void* h, const char* path);
int grab_index_load(void* h, const char* path);

/* timestamp::TimeStampIndex */
void* grab_tsindex_create(uint32_t dim, uint32_t degree, size_t cluster_ratio);
void* grab_tsindex_create_on(int device, uint32_t dim, uint32_t degree, size_t cluster_ratio);
void grab_tsindex_destroy(void* h);
int grab_tsindex_insert(void* h, const float* vectors, const uint64_t* timestamps, size_t n, uint64_t* first_id);
int grab_tsindex_build_virtual_index(void* h);
int grab_tsindex_query(void* h, const float* query, size_t topk, int64_t* ids, float* dists, int probe_buckets);
int grab_tsindex_query_by_timestamp(void* h, const float* query, size_t topk, uint64_t timestamp, int64_t* ids,
                                    float* dists);
size_t grab_tsindex_size(void* h);

#ifdef __cplusplus
}
#endif
#endif /* GRAB_INDEX_H_ */
