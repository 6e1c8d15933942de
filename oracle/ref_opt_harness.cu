// Harness around the REFERENCE's own time-partitioned code (test infrastructure; built into
// oracle/_ref/libgrab_ref.so from the reference sources where they lie, never shipped).
//
// src/index/cagra_opt.cu holds the remote-edge selection kernel (update_remote_edges_kernel, :209-303), the reverse
// injection (kern_make_global_rev_graph :457-482, kern_inject_global_reverse_edges :487-600, driven by
// enhance_global_connectivity :739-793) and the three search launchers (search_opt :1108-1210, search_bucket_opt
// :1212-1328, search_bucket_range :1330-1442).  The file also runs FAISS IVF-PQ and RAFT brute force in other
// functions; oracle/faiss_shim/ declares the names those mention (everything that would compute aborts) so that
// the translation unit compiles; nothing here calls them.  Kernels are launched with the reference's own launch
// shape (256 threads, one per node: cagra_opt.cu:864-877, :753-781).
#include <cuda_runtime.h>

#include <cstdint>
#include <exception>

#include "cagra.cuh"
#include "cagra_opt.cuh"

namespace cagra {
// defined in cagra_opt.cu, not declared in cagra_opt.cuh
__global__ void update_remote_edges_kernel(uint32_t* d_graph, uint64_t* d_ts, uint32_t* d_global_knn,
                                           const float* d_global_dists, size_t num_dataset, uint32_t total_degree,
                                           uint32_t local_degree, uint32_t global_k);
__global__ void kern_make_global_rev_graph(const uint32_t* d_graph, uint32_t* d_rev_graph, uint32_t* d_rev_counts,
                                           size_t num_dataset, uint32_t total_degree, uint32_t local_degree,
                                           uint32_t max_rev_degree);
__global__ void kern_inject_global_reverse_edges(uint32_t* d_graph, const uint32_t* d_rev_graph,
                                                 const uint32_t* d_rev_counts, size_t num_dataset,
                                                 uint32_t total_degree, uint32_t local_degree,
                                                 uint32_t max_rev_degree);
void enhance_global_connectivity(size_t num_dataset, uint32_t* d_graph, uint32_t total_degree, uint32_t local_degree);
}  // namespace cagra

namespace {
int done() {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
template <class F>
int guarded(F&& f) {
  try {
    f();
  } catch (const std::exception&) {
    return -1;
  }
  return done();
}
unsigned blocks(uint64_t n) { return static_cast<unsigned>((n + 255) / 256); }
}  // namespace

// d_cand [n, gk] is consumed (taken candidates are overwritten), as in the reference.
extern "C" int ref_update_remote_edges(uint32_t* d_graph, uint64_t* d_ts, uint32_t* d_cand, uint64_t n,
                                       uint32_t total_deg, uint32_t local_deg, uint32_t gk) {
  cagra::update_remote_edges_kernel<<<blocks(n), 256>>>(d_graph, d_ts, d_cand, nullptr, n, total_deg, local_deg, gk);
  return done();
}

// d_rev [n, max_rev], d_cnt [n] (zeroed here).  The order inside a list is an atomics race.
extern "C" int ref_make_global_rev(const uint32_t* d_graph, uint32_t* d_rev, uint32_t* d_cnt, uint64_t n,
                                   uint32_t total_deg, uint32_t local_deg, uint32_t max_rev) {
  cudaMemset(d_cnt, 0, sizeof(uint32_t) * n);
  cagra::kern_make_global_rev_graph<<<blocks(n), 256>>>(d_graph, d_rev, d_cnt, n, total_deg, local_deg, max_rev);
  return done();
}

extern "C" int ref_inject_global_rev(uint32_t* d_graph, const uint32_t* d_rev, const uint32_t* d_cnt, uint64_t n,
                                     uint32_t total_deg, uint32_t local_deg, uint32_t max_rev) {
  cagra::kern_inject_global_reverse_edges<<<blocks(n), 256>>>(d_graph, d_rev, d_cnt, n, total_deg, local_deg, max_rev);
  return done();
}

extern "C" int ref_enhance_global_connectivity(uint64_t n, uint32_t* d_graph, uint32_t total_deg, uint32_t local_deg) {
  return guarded([&] { cagra::enhance_global_connectivity(n, d_graph, total_deg, local_deg); });
}

// The reference's own launchers (they draw their xor mask from std::random_device: only the part of a search that
// starts from provided seeds is reproducible).  mode 0 search_opt, 1 search_bucket_opt, 2 search_bucket_range.
extern "C" int ref_search_launcher(int mode, const float* d_dataset, uint32_t dim, uint64_t n, const uint32_t* d_graph,
                                   uint32_t total_deg, uint32_t local_deg, uint64_t* d_ts, uint64_t lo, uint64_t hi,
                                   const float* d_queries, int64_t nq, int64_t k, uint32_t itopk, uint32_t width,
                                   uint32_t max_iter, uint32_t hash_bitlen, const uint32_t* d_seeds, uint32_t spq,
                                   int64_t* d_out_ids, float* d_out_dists) {
  return guarded([&] {
    cagra::SearchParams p;
    p.itopk_size = itopk; p.search_width = width; p.min_iterations = 0; p.max_iterations = max_iter;
    p.hash_bitlen = hash_bitlen;
    if (mode == 0)
      cagra::search_opt(d_dataset, dim, n, d_graph, total_deg, d_queries, nq, k, p, d_out_ids, d_out_dists, d_seeds, spq);
    else if (mode == 1)
      cagra::search_bucket_opt(d_dataset, dim, n, d_graph, total_deg, local_deg, d_queries, nq, k, p, d_out_ids,
                               d_out_dists, d_seeds, spq);
    else
      cagra::search_bucket_range(d_dataset, dim, n, d_graph, d_ts, total_deg, local_deg, d_queries, nq, k, lo, hi, p,
                                 d_out_ids, d_out_dists, d_seeds, spq);
  });
}
