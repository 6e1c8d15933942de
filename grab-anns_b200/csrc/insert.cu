// Batched insert: neighbour search for the new vectors, then the topology update.
//
// v1  : src/index/cagra.cu:938-1015 (cagra::insert) = find_near_nodes (insert.cu:140-219:
//       search over the old nodes with search_k = 2*degree, exact distances, sorted) +
//       update_topology_gpu_v1.
// opt : src/index/cagra_opt.cu:1674-1981 (time-partitioned cagra::insert) = global search
//       over the old nodes + bucket search from in-bucket seeds + exact kNN inside the batch
//       (the reference asks RAFT), the two "local" lists merged by distance
//       (merge_topk_kernel, cagra_opt.cu:1476-1652), then update_topology_gpu_opt.
// The searches return canonical exact fp32 distances already sorted, so the reference's
// separate refine / sort kernels (insert.cu:24-137) have no counterpart here.
#include "common.cuh"

namespace grab {

int graph_search_impl(const grab_search_args*);
int knn_blocks_impl(const float*, uint64_t, uint32_t, int, const uint64_t*, uint32_t, uint32_t, int, uint32_t*,
                    float*, cudaStream_t);
int update_topology_v1_impl(uint32_t*, const int64_t*, uint64_t, uint64_t, uint32_t, uint32_t, cudaStream_t);
int update_topology_opt_impl(uint32_t*, const uint64_t*, int64_t*, int64_t*, uint64_t, uint64_t, uint64_t,
                             uint32_t, uint32_t, uint32_t, uint32_t, cudaStream_t, const float* = nullptr, uint32_t = 0,
                             int = 0, bool = true, int = 1);

#define GRAB_TRY(expr)              \
  do {                              \
    int _rc = (expr);               \
    if (_rc != GRAB_OK) return _rc; \
  } while (0)

// view of a pooled scratch buffer
struct Buf {
  void* ptr;
  template <class T> T* as() { return static_cast<T*>(ptr); }
};

__global__ void fill_empty_kernel(int64_t* ids, float* dists, uint64_t total) {
  const uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  ids[i] = -1;
  dists[i] = kFltMax;
}

// Per new vector: merge the bucket-search list [ka] with the intra-batch kNN list [kb] (local
// ids + id_offset), keep the ka best by (dist, id).  cagra_opt.cu:1476-1652.
__global__ void merge_two_lists_kernel(int64_t* __restrict__ ids_a, float* __restrict__ dists_a, uint32_t ka,
                                       const uint32_t* __restrict__ ids_b, const float* __restrict__ dists_b,
                                       uint32_t kb, uint64_t id_offset, uint32_t padded) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
  const uint64_t row = blockIdx.x;
  for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) {
    uint64_t key = kMaxKey;
    if (i < ka) {
      const int64_t id = ids_a[row * ka + i];
      if (id >= 0) key = make_key(dists_a[row * ka + i], static_cast<uint32_t>(id));
    } else if (i < ka + kb) {
      const uint32_t id = ids_b[row * kb + (i - ka)];
      if (id != kInvalid) key = make_key(dists_b[row * kb + (i - ka)], static_cast<uint32_t>(id + id_offset));
    }
    keys[i] = key;
  }
  __syncthreads();
  block_bitonic_sort(keys, padded);
  for (uint32_t i = threadIdx.x; i < ka; i += blockDim.x) {
    const uint64_t key = keys[i];
    ids_a[row * ka + i] = key == kMaxKey ? -1 : static_cast<int64_t>(key_id(key));
    dists_a[row * ka + i] = key == kMaxKey ? kFltMax : key_dist(key);
  }
}

static grab_search_args insert_search_args(const float* d_dataset, uint32_t dim, uint64_t n, const uint32_t* d_graph,
                                           uint32_t deg, const float* d_queries, uint64_t nq, uint32_t k,
                                           grab_search_params params, int64_t* ids, float* dists, int metric) {
  grab_search_args a;
  memset(&a, 0, sizeof(a));
  a.d_dataset = d_dataset; a.n = n; a.dim = dim; a.metric = metric;
  a.d_graph = d_graph; a.graph_degree = deg;
  a.d_queries = d_queries; a.nq = nq; a.k = k; a.params = params;
  a.seed = 0x51ED270B3A4D9C35ull + n;
  a.d_out_ids = ids; a.d_out_dists = dists; a.id_scale = 1;
  return a;
}

int insert_v1_impl(const float* d_dataset, uint64_t num_existing, uint64_t num_new, const float* d_new_vectors,
                   uint32_t* d_graph, uint32_t dim, uint32_t degree, grab_search_params params, int metric) {
  GRAB_REQUIRE(d_dataset && d_new_vectors && d_graph, "insert: null pointer");
  if (num_new == 0) return GRAB_OK;
  GRAB_REQUIRE(num_existing >= 1, "insert: the index is empty (build it first)");
  const uint32_t search_k = 2 * degree;  // cagra.cu:958
  ScopedDeviceBuffer ids, dists;
  GRAB_CUDA_TRY(ids.alloc(sizeof(int64_t) * num_new * search_k));
  GRAB_CUDA_TRY(dists.alloc(sizeof(float) * num_new * search_k));
  grab_search_args a = insert_search_args(d_dataset, dim, num_existing, d_graph, degree, d_new_vectors, num_new,
                                          search_k, params, ids.as<int64_t>(), dists.as<float>(), metric);
  a.filter.kind = GRAB_FILTER_NONE;
  GRAB_TRY(graph_search_impl(&a));
  GRAB_TRY(update_topology_v1_impl(d_graph, ids.as<int64_t>(), num_existing, num_new, degree, search_k, nullptr));
  GRAB_CUDA_TRY(cudaDeviceSynchronize());
  return GRAB_OK;
}

// Uniform pseudo-random seeds inside an id range, one list per query (splitmix64 of (seed, query, slot)).
__global__ void uniform_seeds_kernel(uint32_t* __restrict__ seeds, uint64_t nq, uint32_t spq, uint32_t begin,
                                     uint32_t len, uint64_t seed) {
  const uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (i >= nq * spq) return;
  uint64_t x = seed ^ (i * 0x9e3779b97f4a7c15ull + 0x632be59bd9b4e019ull);
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  seeds[i] = len ? begin + static_cast<uint32_t>(x % len) : kInvalid;
}

// A second stream and two events per device, so that the global and the bucket search of a batch overlap.
struct SideStream {
  cudaStream_t st = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
static SideStream* side_stream() {
  static SideStream per_device[16];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  SideStream& s = per_device[dev];
  if (!s.st) {
    if (cudaStreamCreateWithFlags(&s.st, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  }
  return &s;
}

int route_seeds_impl(const grab_router*, const float*, uint64_t, uint64_t, const grab_filter*, uint32_t, uint32_t,
                     uint64_t, uint32_t*, void*, size_t, cudaStream_t);

int insert_opt_impl(const float* d_dataset, uint32_t* d_graph, const uint64_t* d_bucket, const uint32_t* d_seeds,
                    uint64_t num_existing, uint64_t num_new, uint64_t target_bucket, const float* d_queries,
                    uint32_t dim, uint32_t total_degree, uint32_t local_degree, grab_search_params params,
                    uint32_t num_seeds_per_query, int metric, const InsertOptions* opt) {
  GRAB_REQUIRE(d_dataset && d_graph && d_bucket && d_queries, "insert: null pointer");
  if (num_new == 0) return GRAB_OK;
  GRAB_REQUIRE(num_existing >= 1, "insert: the index is empty (build it first)");
  const uint32_t search_k = params.itopk_size;  // cagra_opt.cu:1691
  GRAB_REQUIRE(search_k >= 2 && search_k <= 512, "insert: itopk_size %u outside [2,512]", search_k);
  const InsertOptions defaults;
  const InsertOptions& o = opt ? *opt : defaults;
  cudaStream_t st = o.stream;
  SideStream* side = side_stream();
  GRAB_REQUIRE(side, "insert: could not create the side stream");
  StageTimer tm("insert_opt batch");
  // pooled scratch: thousands of batches must not pay cudaMalloc / cudaFree each
  Buf ig{pool_get(kPoolInsIdsG, sizeof(int64_t) * num_new * search_k, false)};
  Buf dg{pool_get(kPoolInsDistG, sizeof(float) * num_new * search_k, false)};
  Buf il{pool_get(kPoolInsIdsL, sizeof(int64_t) * num_new * search_k, false)};
  Buf dl{pool_get(kPoolInsDistL, sizeof(float) * num_new * search_k, false)};
  const size_t ws_bytes = grab_graph_search_workspace_bytes(num_new, params.hash_bitlen);
  void* ws = pool_get(kPoolSearchWs, ws_bytes, false);
  void* ws2 = pool_get(kPoolSearchWs2, ws_bytes, false);
  if (!ig.ptr || !dg.ptr || !il.ptr || !dl.ptr || !ws || !ws2) {
    set_last_error("insert: out of device memory for the batch scratch");
    return GRAB_ERR_CUDA;
  }
  uint32_t* seeds_g = nullptr;
  uint32_t* seeds_l = nullptr;
  void* rws = nullptr;
  void* rws2 = nullptr;
  size_t rws_bytes = 0;
  if (o.router) {
    rws_bytes = grab_route_seeds_workspace_bytes(num_new, o.probes);
    seeds_g = static_cast<uint32_t*>(pool_get(kPoolInsSeedsG, sizeof(uint32_t) * num_new * o.routed_seeds, false));
    seeds_l = static_cast<uint32_t*>(pool_get(kPoolInsSeedsL, sizeof(uint32_t) * num_new * o.routed_seeds, false));
    rws = pool_get(kPoolRouteWs, rws_bytes, false);
    rws2 = pool_get(kPoolRouteWs2, rws_bytes, false);
    if (!seeds_g || !seeds_l || !rws || !rws2) {
      set_last_error("insert: out of device memory for the routing scratch");
      return GRAB_ERR_CUDA;
    }
  }
  const uint64_t total = num_new * search_k;
  const uint64_t seed = 0x51ED270B3A4D9C35ull + num_existing;
  // the bucket search runs on the side stream, next to the global search
  GRAB_CUDA_TRY(cudaEventRecord(side->fork, st));
  GRAB_CUDA_TRY(cudaStreamWaitEvent(side->st, side->fork, 0));
  // global search over the old nodes, all columns (cagra_opt.cu:1725-1740); seeds: the router's, else self-drawn
  {
    grab_search_args a = insert_search_args(d_dataset, dim, num_existing, d_graph, total_degree, d_queries, num_new,
                                            search_k, params, ig.as<int64_t>(), dg.as<float>(), metric);
    a.filter.kind = GRAB_FILTER_NONE;
    a.d_ws = ws; a.ws_bytes = ws_bytes; a.stream = st;
    if (o.router) {
      GRAB_TRY(route_seeds_impl(o.router, d_queries, num_new, num_existing, nullptr, o.probes, o.routed_seeds, seed,
                                seeds_g, rws, rws_bytes, st));
      a.d_seeds = seeds_g;
      a.seeds_per_query = o.routed_seeds;
    }
    GRAB_TRY(graph_search_impl(&a));
  }
  // bucket search from in-bucket seeds, local columns only (cagra_opt.cu:1779-1795)
  const bool routed_bucket = o.router && o.bucket_has_old_members;
  if (routed_bucket || (d_seeds && num_seeds_per_query > 0)) {
    grab_search_args a = insert_search_args(d_dataset, dim, num_existing, d_graph, total_degree, d_queries, num_new,
                                            search_k, params, il.as<int64_t>(), dl.as<float>(), metric);
    a.filter.kind = GRAB_FILTER_PREFIX;
    a.filter.active_degree = local_degree;
    a.d_seeds = d_seeds;
    a.seeds_per_query = num_seeds_per_query;
    a.d_ws = ws2; a.ws_bytes = ws_bytes; a.stream = side->st;
    if (routed_bucket && o.bucket_end > o.router_covers) {
      // the bucket holds nodes the router has not been told about (inserted after its last assignment): uniform
      // seeds from the bucket's id range, one list per new vector
      const uint64_t cnt = num_new * o.routed_seeds;
      uniform_seeds_kernel<<<(unsigned)((cnt + 255) / 256), 256, 0, side->st>>>(
          seeds_l, num_new, o.routed_seeds, static_cast<uint32_t>(o.bucket_begin),
          static_cast<uint32_t>(o.bucket_end - o.bucket_begin), seed + 2);
      GRAB_CUDA_TRY(cudaGetLastError());
      a.d_seeds = seeds_l;
      a.seeds_per_query = o.routed_seeds;
    } else if (routed_bucket) {
      // members of the nearest centroids that lie in the target bucket (bucket ids are non-decreasing in the id,
      // so the bucket is one id window)
      grab_filter bf;
      memset(&bf, 0, sizeof(bf));
      bf.kind = GRAB_FILTER_TS_RANGE;
      bf.d_ts = d_bucket;
      bf.lo = target_bucket;
      bf.hi = target_bucket + 1;
      bf.ts_sorted = 1;
      GRAB_TRY(route_seeds_impl(o.router, d_queries, num_new, num_existing, &bf, o.probes, o.routed_seeds, seed + 1,
                                seeds_l, rws2, rws_bytes, side->st));
      a.d_seeds = seeds_l;
      a.seeds_per_query = o.routed_seeds;
    }
    GRAB_TRY(graph_search_impl(&a));
  } else {
    fill_empty_kernel<<<(unsigned)((total + 255) / 256), 256, 0, side->st>>>(il.as<int64_t>(), dl.as<float>(), total);
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  GRAB_CUDA_TRY(cudaEventRecord(side->join, side->st));
  GRAB_CUDA_TRY(cudaStreamWaitEvent(st, side->join, 0));
  tm.mark("global + bucket search");
  // exact kNN inside the batch, tmp = min(n, search_k/2) wide (cagra_opt.cu:1877-1928)
  const uint32_t tmp = static_cast<uint32_t>(num_new < search_k / 2 ? num_new : search_k / 2);
  if (num_new >= 2 && tmp >= 1) {
    Buf bi{pool_get(kPoolInsBatchIds, sizeof(uint32_t) * num_new * tmp, false)};
    Buf bd{pool_get(kPoolInsBatchDist, sizeof(float) * num_new * tmp, false)};
    if (!bi.ptr || !bd.ptr) {
      set_last_error("insert: out of device memory for the batch scratch");
      return GRAB_ERR_CUDA;
    }
    const uint64_t offs[2] = {0, num_new};
    GRAB_TRY(knn_blocks_impl(d_queries, num_new, dim, metric, offs, 1, tmp, 0, bi.as<uint32_t>(), bd.as<float>(), st));
    const uint32_t padded = next_pow2(search_k + tmp);
    merge_two_lists_kernel<<<(unsigned)num_new, 128, sizeof(uint64_t) * padded, st>>>(
        il.as<int64_t>(), dl.as<float>(), search_k, bi.as<uint32_t>(), bd.as<float>(), tmp, num_existing, padded);
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  tm.mark("batch kNN + merge");
  GRAB_TRY(update_topology_opt_impl(d_graph, d_bucket, il.as<int64_t>(), ig.as<int64_t>(), num_existing, num_new,
                                    target_bucket, total_degree, local_degree, search_k, search_k, st,
                                    o.repair_mode ? d_dataset : nullptr, dim, metric, o.sync, o.repair_mode));
  tm.mark("topology update");
  return GRAB_OK;
}

}  // namespace grab

using namespace grab;

extern "C" {

int grab_find_near_nodes(const float* d_dataset, uint64_t num_existing, const float* d_queries, uint64_t num_queries,
                         const uint32_t* d_graph, uint32_t dim, uint32_t graph_degree, uint32_t search_k,
                         grab_search_params params, int64_t* d_out_indices, float* d_out_dists) {
  GRAB_REQUIRE(d_dataset && d_queries && d_graph && d_out_indices && d_out_dists, "find_near_nodes: null pointer");
  grab_search_args a = insert_search_args(d_dataset, dim, num_existing, d_graph, graph_degree, d_queries, num_queries,
                                          search_k, params, d_out_indices, d_out_dists, GRAB_METRIC_L2);
  a.filter.kind = GRAB_FILTER_NONE;
  GRAB_TRY(graph_search_impl(&a));
  GRAB_CUDA_TRY(cudaDeviceSynchronize());
  return GRAB_OK;
}

int grab_insert(const float* d_dataset, uint64_t num_existing, uint64_t num_new, const float* d_new_vectors,
                uint32_t* d_graph, uint32_t dim, uint32_t graph_degree, grab_search_params params) {
  return insert_v1_impl(d_dataset, num_existing, num_new, d_new_vectors, d_graph, dim, graph_degree, params,
                        GRAB_METRIC_L2);
}

int grab_insert_opt(const float* d_dataset, uint32_t* d_graph, const uint64_t* d_ts, const uint32_t* d_seeds,
                    uint64_t num_existing, uint64_t num_new, int use_heuristic, uint64_t target_ts,
                    const float* d_queries, uint32_t dim, uint32_t total_degree, uint32_t local_degree,
                    grab_search_params params, uint32_t num_seeds_per_query) {
  (void)use_heuristic;  // the reference compiles a heuristic variant but never runs it (insert.cu:1425)
  return insert_opt_impl(d_dataset, d_graph, d_ts, d_seeds, num_existing, num_new, target_ts, d_queries, dim,
                         total_degree, local_degree, params, num_seeds_per_query, GRAB_METRIC_L2, nullptr);
}

}  // extern "C"
