// Harness around the REFERENCE's own search kernels (test infrastructure; built into
// oracle/_ref/libgrab_ref.so from the reference sources where they lie, never shipped).
//
// The reference's launchers (src/index/cagra_opt.cu:1108-1442) need FAISS/RAFT to compile, its
// kernels (src/index/search.cu) do not.  The launcher arithmetic is restated here: itopk floor,
// queue capacity, seed target, shared-memory size (src/index/smem_cal.cuh:28-76), global hashmap
// for hash_bitlen > 13.  Results are uint32 ids (widened by the caller) and fp32 distances.
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>

#include "search.cuh"
#include "smem_cal.cuh"

namespace {
struct Launch {
  uint32_t itopk, cap, seeds_target;
  size_t smem;
  uint32_t* pre_hash = nullptr;
};

int prepare(Launch& L, int mode, uint32_t dim, uint32_t deg, uint32_t k, uint32_t itopk_param, uint32_t width,
            uint32_t hash_bitlen, uint32_t seeds_per_query, int64_t nq) {
  L.itopk = std::max(k, itopk_param);
  const uint32_t floor_ = mode == 1 ? 128u : 64u;          // cagra_opt.cu:1129, :1243, :1355
  if (L.itopk < floor_) L.itopk = floor_;
  L.smem = cagra::detail::calculate_and_check_smem(L.itopk, dim, width, deg, hash_bitlen);
  if (L.smem > 48 * 1024) return -2;                        // the reference never raises the limit
  const uint32_t raw = L.itopk + width * deg;
  L.cap = std::max(cagra::config::BLOCK_SIZE, cagra::detail::next_power_of_2(raw));
  if (L.cap != 256 && L.cap != 512 && L.cap != 1024) return -3;  // capacities the kernels can sort
  if (mode == 0) L.seeds_target = std::max(32u, seeds_per_query);   // cagra_opt.cu:1150
  else L.seeds_target = seeds_per_query;                           // :1276, :1386
  if (L.seeds_target > L.itopk) L.seeds_target = L.itopk;
  if (hash_bitlen > 13) {
    const size_t bytes = (size_t(1) << hash_bitlen) * sizeof(uint32_t) * nq;
    if (cudaMalloc(&L.pre_hash, bytes) != cudaSuccess) return -4;
    cudaMemset(L.pre_hash, 0xFF, bytes);
  }
  return 0;
}
}  // namespace

extern "C" int ref_search(int mode, const float* d_dataset, uint32_t dim, uint64_t n, const uint32_t* d_graph,
                          uint32_t deg, uint32_t active_deg, uint64_t* d_ts, uint64_t lo, uint64_t hi,
                          const float* d_queries, int64_t nq, uint32_t k, uint32_t itopk_param, uint32_t width,
                          uint32_t max_iter, uint32_t hash_bitlen, const uint32_t* d_seeds,
                          uint32_t seeds_per_query, uint64_t xor_mask, uint32_t* d_out_ids, float* d_out_dists,
                          float* elapsed_ms) {
  Launch L;
  int rc = prepare(L, mode, dim, deg, k, itopk_param, width, hash_bitlen, seeds_per_query, nq);
  if (rc != 0) return rc;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  dim3 grid((unsigned)nq), block(cagra::config::BLOCK_SIZE);
  cudaEventRecord(e0);
  if (mode == 0) {
    cagra::device::search_kernel<<<grid, block, L.smem>>>(
        d_out_ids, d_out_dists, d_queries, d_dataset, d_graph, d_seeds, seeds_per_query, nullptr, (uint32_t)nq, n,
        dim, deg, k, L.itopk, width, max_iter, L.seeds_target, xor_mask, hash_bitlen, L.pre_hash, L.cap);
  } else if (mode == 1) {
    cagra::device::search_kernel_bucket<<<grid, block, L.smem>>>(
        d_out_ids, d_out_dists, d_queries, d_dataset, d_graph, d_seeds, seeds_per_query, nullptr, (uint32_t)nq, n,
        dim, deg, active_deg, k, L.itopk, width, max_iter, L.seeds_target, xor_mask, hash_bitlen, L.pre_hash, L.cap);
  } else {
    cagra::device::search_kernel_range<<<grid, block, L.smem>>>(
        d_out_ids, d_out_dists, d_queries, d_dataset, d_graph, d_seeds, d_ts, seeds_per_query, nullptr,
        (uint32_t)nq, n, dim, deg, active_deg, lo, hi, k, L.itopk, width, max_iter, L.seeds_target, xor_mask,
        hash_bitlen, L.pre_hash, L.cap);
  }
  cudaEventRecord(e1);
  cudaError_t err = cudaDeviceSynchronize();
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  if (elapsed_ms) *elapsed_ms = ms;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (L.pre_hash) cudaFree(L.pre_hash);
  return err == cudaSuccess ? 0 : (int)err;
}
