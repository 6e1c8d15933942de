// extern "C" entry points of libgrab_anns.so and the build orchestration behind them.
#include <chrono>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace grab {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

static int g_trace = -1;
int trace_level() {
  if (g_trace < 0) {
    const char* e = getenv("GRAB_TRACE");
    g_trace = e ? atoi(e) : 0;
  }
  return g_trace;
}
static double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
StageTimer::StageTimer(const char* s) : scope(s) {
  if (trace_level() > 0) {
    cudaDeviceSynchronize();
    t0 = now_s();
  }
}
void StageTimer::mark(const char* stage) {
  if (trace_level() > 0) {
    cudaDeviceSynchronize();
    const double t = now_s();
    fprintf(stderr, "[grab trace] %-28s %-22s %9.3f ms\n", scope, stage, (t - t0) * 1e3);
    t0 = t;
  }
}

namespace {
struct PoolEntry { void* ptr = nullptr; size_t bytes = 0; };
PoolEntry g_pool[16][kPoolSlots];
std::mutex g_pool_mutex;
}  // namespace

void* pool_get(int slot, size_t bytes, bool zeroed) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  PoolEntry& e = g_pool[dev][slot];
  if (e.bytes < bytes) {
    if (e.ptr) cudaFree(e.ptr);
    e.ptr = nullptr;
    e.bytes = 0;
    const size_t want = bytes + bytes / 2 + 256;  // headroom: the index grows with every batch
    if (cudaMalloc(&e.ptr, want) != cudaSuccess) {
      cudaGetLastError();
      if (cudaMalloc(&e.ptr, bytes) != cudaSuccess) { e.ptr = nullptr; return nullptr; }
      e.bytes = bytes;
    } else {
      e.bytes = want;
    }
    if (zeroed) cudaMemset(e.ptr, 0, e.bytes);
  }
  return e.ptr;
}

void pool_drop(int slot) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  PoolEntry& e = g_pool[dev][slot];
  if (e.ptr) cudaFree(e.ptr);
  e.ptr = nullptr;
  e.bytes = 0;
}

// implemented in the kernel translation units
int exact_search_impl(const float*, uint64_t, uint32_t, int, const grab_filter*, const float*, uint64_t,
                      uint32_t, int64_t*, float*, void*, size_t, cudaStream_t);
int knn_blocks_impl(const float*, uint64_t, uint32_t, int, const uint64_t*, uint32_t, uint32_t, int,
                    uint32_t*, float*, cudaStream_t);
int knn_tc_impl(const float*, uint64_t, uint32_t, int, const uint64_t*, uint32_t, uint32_t, int, int, uint32_t*,
                float*, cudaStream_t);
int router_build_impl(const float*, uint32_t, uint64_t, int, uint32_t, uint32_t, uint64_t, float*, float*, uint32_t*,
                      uint32_t*, cudaStream_t);
int route_seeds_impl(const grab_router*, const float*, uint64_t, uint64_t, const grab_filter*, uint32_t, uint32_t,
                     uint64_t, uint32_t*, void*, size_t, cudaStream_t);
int nearest_centroids_impl(const grab_router*, const float*, uint64_t, uint32_t, uint32_t*, cudaStream_t);
int merge_topk_impl(const float*, const int64_t*, uint64_t, uint32_t, uint32_t, int64_t*, float*,
                    cudaStream_t);
int graph_search_impl(const grab_search_args*);
int route_status_impl(const void*, cudaStream_t);
int prune_device_impl(const uint32_t*, uint32_t*, uint64_t, uint32_t, uint32_t, uint8_t*, cudaStream_t);
int reverse_device_impl(const uint32_t*, uint32_t*, uint32_t*, uint64_t, uint32_t, cudaStream_t);
int merge_device_impl(uint32_t*, const uint32_t*, const uint32_t*, uint64_t, uint32_t, cudaStream_t);
int remote_edges_impl(uint32_t*, const uint64_t*, uint32_t*, uint64_t, uint32_t, uint32_t, uint32_t,
                      cudaStream_t);
int inject_reverse_impl(uint32_t*, uint64_t, uint32_t, uint32_t, uint32_t, cudaStream_t);
int update_topology_v1_impl(uint32_t*, const int64_t*, uint64_t, uint64_t, uint32_t, uint32_t, cudaStream_t);
int update_topology_opt_impl(uint32_t*, const uint64_t*, int64_t*, int64_t*, uint64_t, uint64_t, uint64_t,
                             uint32_t, uint32_t, uint32_t, uint32_t, cudaStream_t, const float* = nullptr, uint32_t = 0,
                             int = 0, bool = true, int = 1);

#define GRAB_TRY(expr)            \
  do {                            \
    int _rc = (expr);             \
    if (_rc != GRAB_OK) return _rc; \
  } while (0)

// kNN stage: exact SIMT scan, or tensor-core candidates + exact re-rank
static int knn_dispatch(const float* d_dataset, uint64_t n, uint32_t dim, int metric, const uint64_t* offs,
                        uint32_t nb, uint32_t k, int mode, int precision, uint32_t* out, float* out_d,
                        cudaStream_t st) {
  if (precision == GRAB_KNN_EXACT_SCAN)
    return knn_blocks_impl(d_dataset, n, dim, metric, offs, nb, k, mode, out, out_d, st);
  if (precision == GRAB_KNN_TC_BF16 || precision == GRAB_KNN_TC_SPLIT)
    return knn_tc_impl(d_dataset, n, dim, metric, offs, nb, k, mode, precision, out, out_d, st);
  set_last_error("knn: unknown precision %d", precision);
  return GRAB_ERR_INVALID_ARGUMENT;
}

// prune -> reverse -> merge over a device kNN graph (cagra.cu:665-711 without the host hops)
static int optimize_pipeline(const uint32_t* d_knn, uint32_t* d_graph, uint64_t n, uint32_t in_deg,
                             uint32_t deg, cudaStream_t st) {
  StageTimer tm("optimize");
  ScopedDeviceBuffer rev, cnt;
  GRAB_CUDA_TRY(rev.alloc(sizeof(uint32_t) * n * deg));
  GRAB_CUDA_TRY(cnt.alloc(sizeof(uint32_t) * n));
  GRAB_TRY(prune_device_impl(d_knn, d_graph, n, in_deg, deg, nullptr, st));
  tm.mark("prune");
  GRAB_TRY(reverse_device_impl(d_graph, rev.as<uint32_t>(), cnt.as<uint32_t>(), n, deg, st));
  tm.mark("reverse");
  GRAB_TRY(merge_device_impl(d_graph, rev.as<uint32_t>(), cnt.as<uint32_t>(), n, deg, st));
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  tm.mark("merge");
  return GRAB_OK;
}

}  // namespace grab

using namespace grab;

extern "C" {

int grab_abi_version(void) { return GRAB_ABI_VERSION; }
void grab_set_trace(int level) { g_trace = level; }

const char* grab_status_string(int status) {
  switch (status) {
    case GRAB_OK: return "ok";
    case GRAB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case GRAB_ERR_UNSUPPORTED: return "unsupported configuration";
    case GRAB_ERR_CUDA: return "CUDA error";
    case GRAB_ERR_WORKSPACE: return "workspace too small";
    case GRAB_ERR_IO: return "I/O error";
    case GRAB_ERR_TIMEOUT: return "device-side wait timed out";
    case GRAB_ERR_NCCL: return "NCCL error";
    default: return "unknown status";
  }
}

const char* grab_last_error(void) { return g_last_error; }

int grab_exact_search(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                      const grab_filter* filter, const float* d_queries, uint64_t nq, uint32_t k,
                      int64_t* d_out_ids, float* d_out_dists, void* d_ws, size_t ws_bytes, void* stream) {
  return exact_search_impl(d_dataset, n, dim, metric, filter, d_queries, nq, k, d_out_ids, d_out_dists,
                           d_ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int grab_graph_search(const grab_search_args* args) { return graph_search_impl(args); }

static grab_search_args base_args(const float* d_dataset, uint32_t dim, uint64_t n, const uint32_t* d_graph,
                                  uint32_t deg, const float* d_queries, int64_t nq, int64_t k,
                                  grab_search_params params, int64_t* ids, float* dists,
                                  const uint32_t* d_seeds, uint32_t spq, void* stream) {
  grab_search_args a;
  memset(&a, 0, sizeof(a));
  a.d_dataset = d_dataset; a.n = n; a.dim = dim; a.metric = GRAB_METRIC_L2;
  a.d_graph = d_graph; a.graph_degree = deg;
  a.d_queries = d_queries; a.nq = nq > 0 ? (uint64_t)nq : 0; a.k = k > 0 ? (uint32_t)k : 0;
  a.params = params; a.d_seeds = d_seeds; a.seeds_per_query = spq;
  a.seed = 0x9E3779B97F4A7C15ull;
  a.d_out_ids = ids; a.d_out_dists = dists; a.id_scale = 1; a.id_offset = 0; a.stream = stream;
  return a;
}

int grab_search(const float* d_dataset, uint32_t dim, uint64_t num_dataset, const uint32_t* d_graph,
                uint32_t graph_degree, const float* d_queries, int64_t num_queries, int64_t k,
                grab_search_params params, int64_t* d_out_indices, float* d_out_dists,
                const uint32_t* d_seeds, uint32_t num_seeds_per_query, void* stream) {
  grab_search_args a = base_args(d_dataset, dim, num_dataset, d_graph, graph_degree, d_queries, num_queries,
                                 k, params, d_out_indices, d_out_dists, d_seeds, num_seeds_per_query, stream);
  a.filter.kind = GRAB_FILTER_NONE;
  GRAB_TRY(graph_search_impl(&a));
  GRAB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return GRAB_OK;
}

int grab_search_bucket(const float* d_dataset, uint32_t dim, uint64_t num_dataset, const uint32_t* d_graph,
                       uint32_t total_degree, uint32_t local_degree, const float* d_queries,
                       int64_t num_queries, int64_t k, grab_search_params params, int64_t* d_out_indices,
                       float* d_out_dists, const uint32_t* d_seeds, uint32_t num_seeds_per_query,
                       void* stream) {
  grab_search_args a = base_args(d_dataset, dim, num_dataset, d_graph, total_degree, d_queries, num_queries,
                                 k, params, d_out_indices, d_out_dists, d_seeds, num_seeds_per_query, stream);
  a.filter.kind = GRAB_FILTER_PREFIX;
  a.filter.active_degree = local_degree;
  GRAB_TRY(graph_search_impl(&a));
  GRAB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return GRAB_OK;
}

int grab_search_range(const float* d_dataset, uint32_t dim, uint64_t num_dataset, const uint32_t* d_graph,
                      const uint64_t* d_ts, uint32_t total_degree, uint32_t local_degree,
                      const float* d_queries, int64_t num_queries, int64_t k, uint64_t start_bucket,
                      uint64_t end_bucket, grab_search_params params, int64_t* d_out_indices,
                      float* d_out_dists, const uint32_t* d_seeds, uint32_t num_seeds_per_query) {
  (void)local_degree;  // the reference walks all columns in range mode (search.cu:744-745)
  grab_search_args a = base_args(d_dataset, dim, num_dataset, d_graph, total_degree, d_queries, num_queries,
                                 k, params, d_out_indices, d_out_dists, d_seeds, num_seeds_per_query, nullptr);
  a.filter.kind = GRAB_FILTER_TS_RANGE;
  a.filter.d_ts = d_ts;
  a.filter.lo = start_bucket;
  a.filter.hi = end_bucket;
  GRAB_TRY(graph_search_impl(&a));
  GRAB_CUDA_TRY(cudaDeviceSynchronize());
  return GRAB_OK;
}

int grab_knn_graph_blocks(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                          const uint64_t* h_block_offsets, uint32_t num_blocks, uint32_t k, int mode,
                          int precision, uint32_t* d_out_knn, float* d_out_dists, void* stream) {
  return knn_dispatch(d_dataset, n, dim, metric, h_block_offsets, num_blocks, k, mode, precision, d_out_knn,
                      d_out_dists, static_cast<cudaStream_t>(stream));
}

int grab_generate_knn_graph(const float* d_dataset, uint64_t num_dataset, uint32_t dim, uint32_t k,
                            uint32_t* h_knn_graph) {
  GRAB_REQUIRE(h_knn_graph, "generate_knn_graph: null output");
  ScopedDeviceBuffer out;
  GRAB_CUDA_TRY(out.alloc(sizeof(uint32_t) * num_dataset * k));
  const uint64_t offs[2] = {0, num_dataset};
  // tensor-core candidates (split precision) + exact re-rank; wide rows fall back to the scan
  GRAB_TRY(knn_dispatch(d_dataset, num_dataset, dim, GRAB_METRIC_L2, offs, 1, k, 0,
                        k <= 204 ? GRAB_KNN_TC_SPLIT : GRAB_KNN_EXACT_SCAN, out.as<uint32_t>(), nullptr, nullptr));
  GRAB_CUDA_TRY(cudaMemcpy(h_knn_graph, out.ptr, sizeof(uint32_t) * num_dataset * k, cudaMemcpyDeviceToHost));
  return GRAB_OK;
}

int grab_optimize_prune_device(const uint32_t* d_knn, uint32_t* d_out, uint64_t n, uint32_t input_degree,
                               uint32_t output_degree, uint8_t* d_detour_or_null, void* stream) {
  return prune_device_impl(d_knn, d_out, n, input_degree, output_degree, d_detour_or_null,
                           static_cast<cudaStream_t>(stream));
}
int grab_optimize_reverse_graph_device(const uint32_t* d_graph, uint32_t* d_rev, uint32_t* d_rev_counts,
                                       uint64_t n, uint32_t degree, void* stream) {
  return reverse_device_impl(d_graph, d_rev, d_rev_counts, n, degree, static_cast<cudaStream_t>(stream));
}
int grab_optimize_merge_graphs_device(uint32_t* d_graph, const uint32_t* d_rev, const uint32_t* d_rev_counts,
                                      uint64_t n, uint32_t degree, void* stream) {
  return merge_device_impl(d_graph, d_rev, d_rev_counts, n, degree, static_cast<cudaStream_t>(stream));
}

int grab_optimize_prune(const uint32_t* h_knn_graph, uint32_t* h_new_graph, uint64_t n, uint32_t in_deg,
                        uint32_t out_deg) {
  GRAB_REQUIRE(h_knn_graph && h_new_graph, "optimize_prune: null pointer");
  ScopedDeviceBuffer in, out;
  GRAB_CUDA_TRY(in.alloc(sizeof(uint32_t) * n * in_deg));
  GRAB_CUDA_TRY(out.alloc(sizeof(uint32_t) * n * out_deg));
  GRAB_CUDA_TRY(cudaMemcpy(in.ptr, h_knn_graph, sizeof(uint32_t) * n * in_deg, cudaMemcpyHostToDevice));
  GRAB_TRY(prune_device_impl(in.as<uint32_t>(), out.as<uint32_t>(), n, in_deg, out_deg, nullptr, nullptr));
  GRAB_CUDA_TRY(cudaMemcpy(h_new_graph, out.ptr, sizeof(uint32_t) * n * out_deg, cudaMemcpyDeviceToHost));
  return GRAB_OK;
}

int grab_optimize_create_reverse_graph(const uint32_t* h_input_graph, uint32_t* h_rev_graph,
                                       uint32_t* h_rev_counts, uint64_t n, uint32_t degree) {
  GRAB_REQUIRE(h_input_graph && h_rev_graph && h_rev_counts, "create_reverse_graph: null pointer");
  ScopedDeviceBuffer g, rev, cnt;
  GRAB_CUDA_TRY(g.alloc(sizeof(uint32_t) * n * degree));
  GRAB_CUDA_TRY(rev.alloc(sizeof(uint32_t) * n * degree));
  GRAB_CUDA_TRY(cnt.alloc(sizeof(uint32_t) * n));
  GRAB_CUDA_TRY(cudaMemcpy(g.ptr, h_input_graph, sizeof(uint32_t) * n * degree, cudaMemcpyHostToDevice));
  GRAB_TRY(reverse_device_impl(g.as<uint32_t>(), rev.as<uint32_t>(), cnt.as<uint32_t>(), n, degree, nullptr));
  GRAB_CUDA_TRY(cudaMemcpy(h_rev_graph, rev.ptr, sizeof(uint32_t) * n * degree, cudaMemcpyDeviceToHost));
  GRAB_CUDA_TRY(cudaMemcpy(h_rev_counts, cnt.ptr, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost));
  return GRAB_OK;
}

int grab_optimize_merge_graphs(uint32_t* h_graph, const uint32_t* h_rev_graph, const uint32_t* h_rev_counts,
                               uint64_t n, uint32_t degree) {
  GRAB_REQUIRE(h_graph && h_rev_graph && h_rev_counts, "merge_graphs: null pointer");
  ScopedDeviceBuffer g, rev, cnt;
  GRAB_CUDA_TRY(g.alloc(sizeof(uint32_t) * n * degree));
  GRAB_CUDA_TRY(rev.alloc(sizeof(uint32_t) * n * degree));
  GRAB_CUDA_TRY(cnt.alloc(sizeof(uint32_t) * n));
  GRAB_CUDA_TRY(cudaMemcpy(g.ptr, h_graph, sizeof(uint32_t) * n * degree, cudaMemcpyHostToDevice));
  GRAB_CUDA_TRY(cudaMemcpy(rev.ptr, h_rev_graph, sizeof(uint32_t) * n * degree, cudaMemcpyHostToDevice));
  GRAB_CUDA_TRY(cudaMemcpy(cnt.ptr, h_rev_counts, sizeof(uint32_t) * n, cudaMemcpyHostToDevice));
  GRAB_TRY(merge_device_impl(g.as<uint32_t>(), rev.as<uint32_t>(), cnt.as<uint32_t>(), n, degree, nullptr));
  GRAB_CUDA_TRY(cudaMemcpy(h_graph, g.ptr, sizeof(uint32_t) * n * degree, cudaMemcpyDeviceToHost));
  return GRAB_OK;
}

int grab_build(const float* d_dataset, uint64_t num_dataset, const uint32_t* d_raw_knn_graph,
               grab_build_params params, uint32_t** d_constructed_graph) {
  (void)d_dataset;
  GRAB_REQUIRE(d_raw_knn_graph && d_constructed_graph, "build: null pointer");
  uint32_t* d_graph = nullptr;
  GRAB_CUDA_TRY(cudaMalloc(&d_graph, sizeof(uint32_t) * num_dataset * params.graph_degree));
  int rc = optimize_pipeline(d_raw_knn_graph, d_graph, num_dataset, params.intermediate_degree,
                             params.graph_degree, nullptr);
  if (rc != GRAB_OK) {
    cudaFree(d_graph);
    return rc;
  }
  *d_constructed_graph = d_graph;
  return GRAB_OK;
}

int grab_remote_edges_device(uint32_t* d_graph, const uint64_t* d_bucket, uint32_t* d_cand, uint64_t n,
                             uint32_t total_degree, uint32_t local_degree, uint32_t gk, void* stream) {
  return remote_edges_impl(d_graph, d_bucket, d_cand, n, total_degree, local_degree, gk,
                           static_cast<cudaStream_t>(stream));
}
int grab_inject_reverse_remote_device(uint32_t* d_graph, uint64_t n, uint32_t total_degree,
                                      uint32_t local_degree, uint32_t max_rev, void* stream) {
  return inject_reverse_impl(d_graph, n, total_degree, local_degree, max_rev, static_cast<cudaStream_t>(stream));
}

// int64 search results -> the uint32 candidate lists the remote-edge kernel consumes
static __global__ void ids_to_cand_kernel(const int64_t* __restrict__ ids, uint64_t count, uint32_t* __restrict__ cand) {
  const uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (i < count) cand[i] = ids[i] < 0 ? kInvalid : static_cast<uint32_t>(ids[i]);
}

// Cross-bucket candidates by search instead of all-pairs (what the reference obtains from a
// FAISS IVF-PQ index over the whole dataset, cagra_opt.cu:813-847): every vector is a query;
// seeds are members of its nearest router centroids, spread evenly over all ids and hence over
// all buckets; the search walks the local edges already in the graph (prefix filter), so each
// seeded bucket contributes its neighbourhood of the query; the gk best overall are the
// candidates (own-bucket hits and the vector itself are skipped by the remote-edge kernel).
// Linear in N where the all-pairs stage is quadratic.
static int global_candidates_by_search(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                                       const uint32_t* d_graph, uint32_t total_degree, uint32_t local_degree,
                                       uint32_t gk, uint32_t iterations, uint32_t width, uint32_t* d_cand) {
  StageTimer tm("global candidates (routed search)");
  uint32_t C = 256;
  while (C < 8192 && static_cast<uint64_t>(C) * C < n) C *= 2;
  ScopedDeviceBuffer cen, norms, offs, members;
  GRAB_CUDA_TRY(cen.alloc(sizeof(float) * C * dim));
  GRAB_CUDA_TRY(norms.alloc(sizeof(float) * C));
  GRAB_CUDA_TRY(offs.alloc(sizeof(uint32_t) * (C + 1)));
  GRAB_CUDA_TRY(members.alloc(sizeof(uint32_t) * n));
  GRAB_TRY(router_build_impl(d_dataset, dim, n, metric, C, 10, 0, cen.as<float>(), norms.as<float>(),
                             offs.as<uint32_t>(), members.as<uint32_t>(), nullptr));
  grab_router r{};
  r.num_centroids = C; r.dim = dim; r.metric = metric;
  r.d_centroids = cen.as<float>(); r.d_centroid_norms = norms.as<float>();
  r.d_member_offsets = offs.as<uint32_t>(); r.d_members = members.as<uint32_t>();
  tm.mark("router");
  const uint64_t chunk = 1ull << 18;
  const uint32_t S = 64, probes = 4;
  grab_search_params p{gk > 128 ? 256u : 128u, width ? width : 4, 0, iterations ? iterations : 10, 12};
  ScopedDeviceBuffer seeds, ids, dists, rws, sws;
  const size_t rws_bytes = grab_route_seeds_workspace_bytes(chunk, probes);
  const size_t sws_bytes = grab_graph_search_workspace_bytes(chunk, p.hash_bitlen);
  GRAB_CUDA_TRY(seeds.alloc(sizeof(uint32_t) * chunk * S));
  GRAB_CUDA_TRY(ids.alloc(sizeof(int64_t) * chunk * gk));
  GRAB_CUDA_TRY(dists.alloc(sizeof(float) * chunk * gk));
  GRAB_CUDA_TRY(rws.alloc(rws_bytes));
  GRAB_CUDA_TRY(sws.alloc(sws_bytes));
  for (uint64_t q0 = 0; q0 < n; q0 += chunk) {
    const uint64_t nq = n - q0 < chunk ? n - q0 : chunk;
    const float* q = d_dataset + q0 * dim;
    GRAB_TRY(route_seeds_impl(&r, q, nq, n, nullptr, probes, S, 0x5eed5eedull + q0, seeds.as<uint32_t>(), rws.ptr,
                              rws_bytes, nullptr));
    grab_search_args a;
    memset(&a, 0, sizeof(a));
    a.d_dataset = d_dataset; a.n = n; a.dim = dim; a.metric = metric;
    a.d_graph = d_graph; a.graph_degree = total_degree;
    a.d_queries = q; a.nq = nq; a.k = gk; a.params = p;
    a.filter.kind = GRAB_FILTER_PREFIX; a.filter.active_degree = local_degree;
    a.d_seeds = seeds.as<uint32_t>(); a.seeds_per_query = S; a.seed = 0x5eed5eedull + q0;
    a.d_out_ids = ids.as<int64_t>(); a.d_out_dists = dists.as<float>();
    a.id_scale = 1; a.d_ws = sws.ptr; a.ws_bytes = sws_bytes;
    GRAB_TRY(graph_search_impl(&a));
    ids_to_cand_kernel<<<static_cast<unsigned>((nq * gk + 255) / 256), 256>>>(ids.as<int64_t>(), nq * gk, d_cand + q0 * gk);
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  GRAB_CUDA_TRY(cudaDeviceSynchronize());
  tm.mark("search");
  return GRAB_OK;
}

int grab_build_time_partitioned_graph_ex(const float* d_dataset, uint64_t total_num, uint32_t dim, int metric,
                                         uint32_t* d_graph, const uint64_t* d_bucket,
                                         const uint64_t* h_bucket_sizes, uint32_t num_buckets,
                                         uint32_t total_degree, uint32_t local_degree,
                                         const grab_tp_build_options* options) {
  GRAB_REQUIRE(d_dataset && d_graph && d_bucket && h_bucket_sizes, "build_time_partitioned_graph: null pointer");
  GRAB_REQUIRE(num_buckets >= 1, "build_time_partitioned_graph: no buckets");
  GRAB_REQUIRE(total_degree >= 4 && total_degree <= 256 && local_degree >= 1 && local_degree <= total_degree,
               "build_time_partitioned_graph: bad degrees %u/%u", local_degree, total_degree);
  const int knn_precision = options ? options->knn_precision : GRAB_KNN_TC_SPLIT;
  int global_mode = options ? options->global_candidates : GRAB_GLOBAL_AUTO;
  GRAB_REQUIRE(global_mode >= GRAB_GLOBAL_AUTO && global_mode <= GRAB_GLOBAL_ROUTED_SEARCH,
               "build_time_partitioned_graph: unknown global_candidates mode %d", global_mode);
  std::vector<uint64_t> offs(num_buckets + 1, 0);
  for (uint32_t b = 0; b < num_buckets; ++b) offs[b + 1] = offs[b] + h_bucket_sizes[b];
  GRAB_REQUIRE(offs[num_buckets] == total_num, "build_time_partitioned_graph: bucket sizes sum to %llu, not %llu",
               (unsigned long long)offs[num_buckets], (unsigned long long)total_num);
  // Local phase (cagra_opt.cu:946-1090): per-bucket kNN of width 2*total_degree, then
  // prune / reverse / merge to total_degree.  Edges never leave a bucket, so one pass over
  // all N is the same as the reference's per-bucket passes.
  const uint32_t inter = 2 * total_degree;
  StageTimer tm("time_partitioned_build");
  {
    ScopedDeviceBuffer knn;
    GRAB_CUDA_TRY(knn.alloc(sizeof(uint32_t) * total_num * inter));
    GRAB_TRY(knn_dispatch(d_dataset, total_num, dim, metric, offs.data(), num_buckets, inter, 0,
                          inter <= 204 ? knn_precision : GRAB_KNN_EXACT_SCAN, knn.as<uint32_t>(), nullptr, nullptr));
    tm.mark("local kNN");
    GRAB_TRY(optimize_pipeline(knn.as<uint32_t>(), d_graph, total_num, inter, total_degree, nullptr));
    tm.mark("prune+reverse+merge");
  }
  if (local_degree == total_degree || num_buckets == 1) return GRAB_OK;
  // Global phase (cagra_opt.cu:796-907): candidates from other buckets, ascending exact
  // distance, width global_k = clamp(roundup32(4*remote), 64, 256) (cagra_opt.cu:808-810).
  const uint32_t remote = total_degree - local_degree;
  uint32_t gk = remote * 4;
  gk = (gk + 32) - (gk % 32);
  if (gk < 64) gk = 64;
  if (gk > 256) gk = 256;
  // all-pairs is exact but quadratic (0.4 s at 1M x 128, 75 s at 12.5M x 96); the reference itself takes these
  // candidates from an approximate index (IVF-PQ, cagra_opt.cu:813-847).  From 2^19 vectors on the routed search
  // takes over: at 1M x 128 with 6 parents x 12 iterations it needs 0.21 s instead of 0.40 s and the finished
  // graph answers 10 % range queries at recall 0.970 instead of 0.973; from 2^21 vectors on, where the candidates
  // dominate the build, 4 x 10 (within 1 pp of the all-pairs graph).
  uint32_t gc_iterations = options ? options->search_iterations : 0, gc_width = options ? options->search_width : 0;
  if (global_mode == GRAB_GLOBAL_AUTO) {
    global_mode = total_num >= (1ull << 19) ? GRAB_GLOBAL_ROUTED_SEARCH : GRAB_GLOBAL_ALL_PAIRS;
    if (total_num < (1ull << 21)) {
      if (!gc_iterations) gc_iterations = 12;
      if (!gc_width) gc_width = 6;
    }
  }
  if (total_num < 4096) global_mode = GRAB_GLOBAL_ALL_PAIRS;
  {
    ScopedDeviceBuffer cand;
    GRAB_CUDA_TRY(cand.alloc(sizeof(uint32_t) * total_num * gk));
    if (global_mode == GRAB_GLOBAL_ROUTED_SEARCH) {
      GRAB_TRY(global_candidates_by_search(d_dataset, total_num, dim, metric, d_graph, total_degree, local_degree, gk,
                                           gc_iterations, gc_width, cand.as<uint32_t>()));
    } else {
      GRAB_TRY(knn_dispatch(d_dataset, total_num, dim, metric, offs.data(), num_buckets, gk, 1,
                            gk <= 204 ? knn_precision : GRAB_KNN_EXACT_SCAN, cand.as<uint32_t>(), nullptr, nullptr));
    }
    tm.mark("global candidates");
    GRAB_TRY(remote_edges_impl(d_graph, d_bucket, cand.as<uint32_t>(), total_num, total_degree, local_degree,
                               gk, nullptr));
    GRAB_TRY(inject_reverse_impl(d_graph, total_num, total_degree, local_degree, 32, nullptr));
    tm.mark("remote edges + inject");
  }
  GRAB_CUDA_TRY(cudaDeviceSynchronize());
  return GRAB_OK;
}

int grab_build_time_partitioned_graph(const float* d_dataset, uint64_t total_num, uint32_t dim, int metric,
                                      uint32_t* d_graph, const uint64_t* d_bucket,
                                      const uint64_t* h_bucket_sizes, uint32_t num_buckets,
                                      uint32_t total_degree, uint32_t local_degree, int knn_precision) {
  grab_tp_build_options o;
  o.knn_precision = knn_precision;
  o.global_candidates = GRAB_GLOBAL_AUTO;
  o.search_iterations = 0;
  o.search_width = 0;
  return grab_build_time_partitioned_graph_ex(d_dataset, total_num, dim, metric, d_graph, d_bucket, h_bucket_sizes,
                                              num_buckets, total_degree, local_degree, &o);
}

int grab_update_topology_v1(uint32_t* d_graph, const int64_t* d_search_indices, uint64_t num_existing,
                            uint64_t num_new, uint32_t graph_degree, uint32_t search_k, void* stream) {
  return update_topology_v1_impl(d_graph, d_search_indices, num_existing, num_new, graph_degree, search_k,
                                 static_cast<cudaStream_t>(stream));
}
int grab_update_topology_opt(uint32_t* d_graph, const uint64_t* d_bucket, int64_t* d_local_knn,
                             int64_t* d_global_knn, uint64_t num_existing, uint64_t num_new,
                             uint64_t target_bucket, uint32_t total_degree, uint32_t local_degree,
                             uint32_t k_local, uint32_t k_global, void* stream) {
  return update_topology_opt_impl(d_graph, d_bucket, d_local_knn, d_global_knn, num_existing, num_new,
                                  target_bucket, total_degree, local_degree, k_local, k_global,
                                  static_cast<cudaStream_t>(stream));
}

int grab_merge_topk(const float* d_dists, const int64_t* d_ids, uint64_t nq, uint32_t parts, uint32_t k,
                    int64_t* d_out_ids, float* d_out_dists, void* stream) {
  return merge_topk_impl(d_dists, d_ids, nq, parts, k, d_out_ids, d_out_dists, static_cast<cudaStream_t>(stream));
}

int grab_router_build(const float* d_dataset, uint32_t dim, uint64_t n, int metric, uint32_t num_centroids,
                      uint32_t iterations, uint64_t max_sample, float* d_centroids, float* d_centroid_norms,
                      uint32_t* d_member_offsets, uint32_t* d_members, void* stream) {
  return router_build_impl(d_dataset, dim, n, metric, num_centroids, iterations, max_sample, d_centroids,
                           d_centroid_norms, d_member_offsets, d_members, static_cast<cudaStream_t>(stream));
}

int grab_nearest_centroids(const grab_router* router, const float* d_rows, uint64_t m, uint32_t probes,
                           uint32_t* d_out, void* stream) {
  return nearest_centroids_impl(router, d_rows, m, probes, d_out, static_cast<cudaStream_t>(stream));
}

int grab_route_seeds(const grab_router* router, const float* d_queries, uint64_t nq, uint64_t n,
                     const grab_filter* filter, uint32_t probes, uint32_t seeds_per_query, uint64_t seed,
                     uint32_t* d_seeds, void* d_ws, size_t ws_bytes, void* stream) {
  return route_seeds_impl(router, d_queries, nq, n, filter, probes, seeds_per_query, seed, d_seeds, d_ws, ws_bytes,
                          static_cast<cudaStream_t>(stream));
}

int grab_route_status(const void* d_ws, void* stream) {
  return route_status_impl(d_ws, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
