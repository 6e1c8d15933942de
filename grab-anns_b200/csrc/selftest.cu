// Device-level unit-test entry points for the building blocks of the graph search.  The reference ships
// such tests as stand-alone executables (tests/test_bitonic.cu:73-156 warp sort against std::sort,
// tests/test_sort_impl.cu:111-121 queue capacities 64..512, tests/test_hashmap.cu:144-187 insert successes
// against the number of unique keys at three load factors); these entry points let the same known-answer
// inputs run through the code of search_blocks.cuh exactly as graph_search_kernel instantiates it.
// They are not part of the search path.
#include "common.cuh"
#include "search_blocks.cuh"

namespace grab {

// One warp per list: fold `ncand` unsorted candidate keys into the sorted list of m keys with the routine the
// search kernel would pick for this m (64: registers x2, 128: registers x4, else shared memory).
// variant 0 = as the shared-list kernel dispatches, 1 = force the shared-memory version, 2 = merge by rank
// (ncand <= 32, m 64 / 128), 3 = two register-sorted runs folded in (ncand <= 256, m 64 / 128).
__global__ void selftest_sort_merge_kernel(const uint64_t* __restrict__ top_in, const uint64_t* __restrict__ cand_in,
                                           uint32_t m, uint32_t ncand, uint32_t cand_stride, int variant,
                                           uint64_t* __restrict__ top_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* top = reinterpret_cast<uint64_t*>(smem_raw);
  uint64_t* cand = top + m;
  const uint32_t lane = threadIdx.x;
  const size_t list = blockIdx.x;
  for (uint32_t i = lane; i < m; i += 32) top[i] = top_in[list * m + i];
  for (uint32_t i = lane; i < ncand; i += 32) cand[i] = cand_in[list * cand_stride + i];
  __syncwarp();
  if (ncand > 0 && variant == 2) {
    // merge by rank (the warp-split kernel's path for a handful of kept keys): ncand <= 32, m = 64 or 128
    const uint64_t c = lane < ncand ? cand[lane] : kMaxKey;
    if (m == 64) { uint64_t t[2]; warp_merge_by_rank<2>(top, c, ncand, lane, t); }
    else { uint64_t t[4]; warp_merge_by_rank<4>(top, c, ncand, lane, t); }
  } else if (ncand > 0 && variant == 3) {
    // the warp-split kernel's path for many kept keys: the candidates are cut in two runs, each sorted in
    // registers as its warp would, then both are folded into the list
    const uint32_t n0 = ncand / 2, n1 = ncand - n0;
    uint64_t* run1 = cand + n0;
    auto sort_run = [&](uint64_t* keys, uint32_t n) {
      if (n <= 1) return;
      if (n <= 32) warp_sort_regs<1>(keys, n, lane);
      else if (n <= 64) warp_sort_regs<2>(keys, n, lane);
      else warp_sort_regs_128(keys, n, lane);
    };
    sort_run(cand, n0);
    __syncwarp();
    sort_run(run1, n1);
    __syncwarp();
    if (m == 64) {
      uint64_t t[2];
      warp_merge_runs_regs<2>(top, cand, n0 < m ? n0 : m, run1, n1 < m ? n1 : m, lane, t);
      __syncwarp();
      for (int r = 0; r < 2; ++r) top[lane + 32 * r] = t[r];
    } else {
      uint64_t t[4];
      warp_merge_runs_regs<4>(top, cand, n0 < m ? n0 : m, run1, n1 < m ? n1 : m, lane, t);
      __syncwarp();
      for (int r = 0; r < 4; ++r) top[lane + 32 * r] = t[r];
    }
  } else if (ncand > 0) {
    if (variant == 0 && m == 64 && ncand <= 64) {
      warp_sort_merge_regs<2>(top, cand, ncand, lane);
    } else if (variant == 0 && m == 128 && ncand <= 128) {
      warp_sort_merge_regs_128(top, cand, ncand, lane);
    } else {
      uint32_t padded = 32;
      while (padded < ncand) padded <<= 1;
      for (uint32_t i = ncand + lane; i < padded; i += 32) cand[i] = kMaxKey;
      __syncwarp();
      warp_bitonic_sort_smem(cand, padded, lane);
      warp_merge_into_topk(top, m, cand, ncand, lane);
    }
  }
  __syncwarp();
  for (uint32_t i = lane; i < m; i += 32) top_out[list * m + i] = top[i];
}

// One CTA of `threads` threads inserts nkeys keys into one table (shared memory up to 2^13 slots as in the
// kernel, else the caller's global table), thread t taking keys t, t + threads, ...: concurrent inserts as in
// the expansion phase.  success[i] = 1 when key i was newly inserted.
__global__ void selftest_hash_kernel(uint32_t* __restrict__ table_global, uint32_t bitlen,
                                     const uint32_t* __restrict__ keys, uint32_t nkeys,
                                     uint32_t* __restrict__ success) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t hsize = 1u << bitlen;
  const bool local = bitlen <= 13;
  uint32_t* table = local ? reinterpret_cast<uint32_t*>(smem_raw) : table_global;
  for (uint32_t i = threadIdx.x; i < hsize; i += blockDim.x) table[i] = kInvalid;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < nkeys; i += blockDim.x) success[i] = hash_insert(table, bitlen, keys[i]) ? 1u : 0u;
  __syncthreads();
  if (local)
    for (uint32_t i = threadIdx.x; i < hsize; i += blockDim.x) table_global[i] = table[i];
}

}  // namespace grab

extern "C" int grab_selftest_sort_merge(const uint64_t* d_top, const uint64_t* d_cand, uint64_t lists, uint32_t m,
                                        uint32_t ncand, uint32_t cand_stride, int variant, uint64_t* d_out,
                                        void* stream) {
  using namespace grab;
  GRAB_REQUIRE(d_top && d_cand && d_out, "selftest_sort_merge: null pointer");
  GRAB_REQUIRE(m >= 64 && m <= 1024 && (m & (m - 1)) == 0, "selftest_sort_merge: m %u must be a power of two in [64,1024]", m);
  GRAB_REQUIRE(ncand <= cand_stride && cand_stride <= 2048, "selftest_sort_merge: ncand %u > stride %u or stride > 2048",
               ncand, cand_stride);
  GRAB_REQUIRE(variant < 2 || ((m == 64 || m == 128) && ncand <= (variant == 2 ? 32u : 256u)),
               "selftest_sort_merge: variant %d needs m 64 or 128 and fewer candidates", variant);
  if (lists == 0) return GRAB_OK;
  uint32_t padded = 32;
  while (padded < ncand) padded <<= 1;
  const size_t smem = sizeof(uint64_t) * (m + padded);
  GRAB_CUDA_TRY(cudaFuncSetAttribute(selftest_sort_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  selftest_sort_merge_kernel<<<static_cast<unsigned>(lists), 32, smem, static_cast<cudaStream_t>(stream)>>>(
      d_top, d_cand, m, ncand, cand_stride, variant, d_out);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

extern "C" int grab_selftest_hash_insert(uint32_t* d_table, uint32_t hash_bitlen, const uint32_t* d_keys,
                                         uint32_t nkeys, uint32_t threads, uint32_t* d_success, void* stream) {
  using namespace grab;
  GRAB_REQUIRE(d_table && d_keys && d_success, "selftest_hash_insert: null pointer");
  GRAB_REQUIRE(hash_bitlen >= 4 && hash_bitlen <= 20, "selftest_hash_insert: hash_bitlen %u outside [4,20]", hash_bitlen);
  GRAB_REQUIRE(threads >= 32 && threads <= 1024 && threads % 32 == 0, "selftest_hash_insert: bad thread count %u", threads);
  const size_t smem = hash_bitlen <= 13 ? sizeof(uint32_t) * (size_t(1) << hash_bitlen) : 0;
  selftest_hash_kernel<<<1, threads, smem, static_cast<cudaStream_t>(stream)>>>(d_table, hash_bitlen, d_keys, nkeys,
                                                                                 d_success);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}
