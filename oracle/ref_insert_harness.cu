// Harness around the REFERENCE's own insert kernels (test infrastructure; built into
// oracle/_ref/libgrab_ref.so from the reference sources where they lie, never shipped).
//
// src/index/insert.cu compiles stand-alone except for one symbol, cagra::search (the base
// launcher, src/index/cagra.cu:844-935).  When cagra.cu is part of the build (GRAB_REF_WITH_CAGRA_CU, see
// ref_build_harness.cu) that launcher is the reference's own; otherwise its parameter arithmetic is
// restated below so that the reference's find_near_nodes links.  The topology functions
// update_topology_gpu_v1 (insert.cu:372-440) and update_topology_gpu_opt (:1398-1573) are called
// as they are; the three kernels of the latter (:448, :579, :653) are also launched one by one,
// because the mailbox order of :579 is an atomics race and only the stages around it are
// deterministic.
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include <stdexcept>

#include "insert.cuh"
#include "search.cuh"
#include "smem_cal.cuh"

namespace cagra {

// defined in insert.cu, not declared in insert.cuh
__global__ void fill_new_nodes_kernel_opt(uint32_t* d_graph, const uint64_t* d_ts, int64_t* d_local_knn,
                                          int64_t* d_global_knn, size_t num_existing, size_t num_new,
                                          uint32_t total_degree, uint32_t local_degree, uint32_t search_k_local,
                                          uint32_t search_k_global);
__global__ void generate_update_requests_kernel_opt(const uint32_t* d_graph, uint32_t* d_local_req_counts,
                                                    uint32_t* d_local_req_lists, uint32_t* d_remote_req_counts,
                                                    uint32_t* d_remote_req_lists, size_t num_existing,
                                                    size_t num_new, size_t target_ts, const uint64_t* d_ts,
                                                    uint32_t total_degree, uint32_t local_degree,
                                                    uint32_t local_max_requests, uint32_t remote_max_requests);
__global__ void apply_topology_updates_kernel_opt(uint32_t* d_graph, const uint32_t* d_local_req_counts,
                                                  const uint32_t* d_local_req_lists, uint32_t max_requests_local,
                                                  const uint32_t* d_remote_req_counts,
                                                  const uint32_t* d_remote_req_lists, uint32_t max_requests_remote,
                                                  const uint64_t* d_ts, size_t num_existing, uint32_t total_degree,
                                                  uint32_t local_degree);

namespace {
__global__ void widen_ids_kernel(const uint32_t* src, int64_t* dst, size_t count) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < count) dst[i] = static_cast<int64_t>(src[i]);
}
}  // namespace

#ifndef GRAB_REF_WITH_CAGRA_CU  // with cagra.cu compiled in, the reference's own launcher is linked instead
// cagra.cu:844-935 restated: itopk = max(k, itopk, 64); queue = max(256, pow2(itopk + W*deg)); seed
// target itopk/4; the xor mask is fixed here (the reference draws std::random_device).  Only the
// shared-memory visited table (hash_bitlen <= 13) is supported: the reference's global-table branch
// allocates one table for all queries (:879-882), which is not worth restating.
void search(const float* d_dataset, size_t num_dataset, uint32_t dim, const uint32_t* d_graph, uint32_t graph_degree,
            const float* d_queries, int64_t num_queries, int64_t k, SearchParams params, int64_t* d_out_indices,
            float* d_out_dists, const uint32_t* d_seeds, const uint32_t num_seeds_per_query) {
  if (d_graph == nullptr) throw std::runtime_error("Graph is null!");
  if (params.hash_bitlen > 13) throw std::runtime_error("harness: hash_bitlen > 13 not restated");
  const uint32_t topk = static_cast<uint32_t>(k);
  uint32_t itopk = std::max(topk, params.itopk_size);
  if (itopk < 64) itopk = 64;
  const size_t smem = cagra::detail::calculate_and_check_smem(itopk, dim, params.search_width, graph_degree,
                                                              params.hash_bitlen);
  const uint32_t cap = std::max(cagra::config::BLOCK_SIZE,
                                cagra::detail::next_power_of_2(itopk + params.search_width * graph_degree));
  uint32_t* d_ids32 = nullptr;
  if (cudaMalloc(&d_ids32, sizeof(uint32_t) * num_queries * topk) != cudaSuccess)
    throw std::runtime_error("harness: cudaMalloc");
  cagra::device::search_kernel<<<dim3((unsigned)num_queries), dim3(cagra::config::BLOCK_SIZE), smem>>>(
      d_ids32, d_out_dists, d_queries, d_dataset, d_graph, d_seeds, num_seeds_per_query, nullptr,
      (uint32_t)num_queries, num_dataset, dim, graph_degree, topk, itopk, params.search_width, params.max_iterations,
      params.itopk_size / 4, 0x9E3779B97F4A7C15ull, params.hash_bitlen, nullptr, cap);
  const size_t total = static_cast<size_t>(num_queries) * topk;
  widen_ids_kernel<<<(unsigned)((total + 255) / 256), 256>>>(d_ids32, d_out_indices, total);
  cudaDeviceSynchronize();
  cudaFree(d_ids32);
}
#endif  // GRAB_REF_WITH_CAGRA_CU

}  // namespace cagra

namespace {
int done() {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
}  // namespace

extern "C" int ref_update_topology_v1(uint32_t* d_graph, const int64_t* d_found, uint64_t num_existing,
                                      uint64_t num_new, uint32_t degree, uint32_t search_k) {
  cagra::update_topology_gpu_v1(d_graph, d_found, num_existing, num_new, degree, search_k);
  return done();
}

extern "C" int ref_insert_opt_fill(uint32_t* d_graph, const uint64_t* d_ts, int64_t* d_local, int64_t* d_global,
                                   uint64_t num_existing, uint64_t num_new, uint32_t total_degree,
                                   uint32_t local_degree, uint32_t k_local, uint32_t k_global) {
  const int block = 256, grid = static_cast<int>((num_new + block - 1) / block);   // insert.cu:1424-1425
  cagra::fill_new_nodes_kernel_opt<<<grid, block>>>(d_graph, d_ts, d_local, d_global, num_existing, num_new,
                                                    total_degree, local_degree, k_local, k_global);
  return done();
}

// Mailboxes: counts u32[num_existing + num_new] zeroed by the caller; lists
// u32[(num_existing + num_new) * max] with max = local/2 and (total-local)/2 (insert.cu:1479-1480).
extern "C" int ref_insert_opt_generate(const uint32_t* d_graph, uint32_t* d_lcount, uint32_t* d_llist,
                                       uint32_t* d_rcount, uint32_t* d_rlist, uint64_t num_existing,
                                       uint64_t num_new, uint64_t target_ts, const uint64_t* d_ts,
                                       uint32_t total_degree, uint32_t local_degree) {
  const int block = 256, grid = static_cast<int>((num_new + block - 1) / block);
  cagra::generate_update_requests_kernel_opt<<<grid, block>>>(
      d_graph, d_lcount, d_llist, d_rcount, d_rlist, num_existing, num_new, target_ts, d_ts, total_degree,
      local_degree, local_degree / 2, (total_degree - local_degree) / 2);
  return done();
}

extern "C" int ref_insert_opt_apply(uint32_t* d_graph, const uint32_t* d_lcount, const uint32_t* d_llist,
                                    const uint32_t* d_rcount, const uint32_t* d_rlist, const uint64_t* d_ts,
                                    uint64_t num_existing, uint32_t total_degree, uint32_t local_degree) {
  const int block = 256, grid = static_cast<int>((num_existing + block - 1) / block);  // insert.cu:1529
  cagra::apply_topology_updates_kernel_opt<<<grid, block>>>(d_graph, d_lcount, d_llist, local_degree / 2, d_rcount,
                                                            d_rlist, (total_degree - local_degree) / 2, d_ts,
                                                            num_existing, total_degree, local_degree);
  return done();
}

// The whole function as the reference's insert calls it (cagra_opt.cu:1935-1958): mailbox order races.
extern "C" int ref_update_topology_opt(uint32_t* d_graph, const float* d_dataset, uint64_t dim, uint64_t target_ts,
                                       const uint64_t* d_ts, int64_t* d_local, float* d_local_d, int64_t* d_global,
                                       float* d_global_d, uint64_t num_existing, uint64_t num_new,
                                       uint32_t total_degree, uint32_t local_degree, uint32_t k_local,
                                       uint32_t k_global) {
  cagra::update_topology_gpu_opt(d_graph, d_dataset, dim, target_ts, d_ts, d_local, d_local_d, d_global, d_global_d,
                                 num_existing, num_new, total_degree, local_degree, k_local, k_global, false);
  return done();
}

// insert.cu:140-219 as it is: batches of 64 through cagra::search (above), exact re-score, warp sort.
extern "C" int ref_find_near_nodes(const float* d_dataset, uint32_t dim, uint64_t num_existing, uint64_t num_new,
                                   const float* d_new, const uint32_t* d_graph, uint32_t degree, uint32_t search_k,
                                   uint32_t itopk, uint32_t width, uint32_t max_iter, uint32_t hash_bitlen,
                                   int64_t* d_out_ids, float* d_out_dists) {
  cagra::SearchParams p;
  p.itopk_size = itopk;
  p.search_width = width;
  p.max_iterations = max_iter;
  p.hash_bitlen = hash_bitlen;
  try {
    cagra::find_near_nodes(d_dataset, dim, num_existing, num_new, d_new, d_graph, degree, search_k, p, d_out_ids,
                           d_out_dists);
  } catch (const std::exception&) {
    return -1;
  }
  return done();
}
