// Exchange step of the id-sharded multi-GPU search (no counterpart in the single-GPU reference, whose device is
// fixed at compile time: src/index/common.cuh:5-7).
//
// Every rank searches its own stripe of the index for the same queries and leaves, per query, `kp` ascending
// keys [ordered fp32 distance : 32 | global id : 32] (written by the search kernel's epilogue).  One NCCL
// all-gather moves them, and merge_runs_kernel folds the `parts` sorted runs of a query into the global top-k:
// every key computes its final rank as (its position in its own run) + (the number of smaller keys in each other
// run, by binary search), and writes itself straight to that slot -- no sort network, no barrier.  Keys are unique
// (global ids are), so the ranks are a permutation and the result is the (dist, id) order, bit for bit the one an
// unsharded index would give.
//
// NCCL is loaded at run time (dlopen) so that the library itself has no link-time dependency on it; entry points
// that need it return GRAB_ERR_NCCL when it is missing or fails.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "common.cuh"

namespace grab {

constexpr int kMergeWarps = 4;

// keys: [parts][nq][kp], every run ascending, empty slots = all ones at the tail.
__global__ void __launch_bounds__(32 * kMergeWarps)
merge_runs_kernel(const uint64_t* __restrict__ keys, uint64_t nq, uint32_t parts, uint32_t kp, uint32_t k,
                  int64_t* __restrict__ out_ids, float* __restrict__ out_dists, uint64_t* __restrict__ out_keys) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint64_t qi = blockIdx.x * static_cast<uint64_t>(blockDim.x >> 5) + warp;
  if (qi >= nq) return;  // whole warps leave together
  const uint32_t m = parts * kp;
  uint64_t* s = reinterpret_cast<uint64_t*>(smem_raw) + static_cast<size_t>(warp) * m;
  for (uint32_t e = lane; e < m; e += 32) {
    const uint32_t r = e / kp, i = e - r * kp;
    s[e] = keys[(static_cast<uint64_t>(r) * nq + qi) * kp + i];
  }
  __syncwarp();
  uint32_t valid = 0;
  for (uint32_t e = lane; e < m; e += 32) {
    const uint64_t key = s[e];
    if (key == kMaxKey) continue;
    ++valid;
    const uint32_t r = e / kp;
    uint32_t rank = e - r * kp;
    for (uint32_t o = 0; o < parts; ++o) {
      if (o == r) continue;
      const uint64_t* run = s + o * kp;
      uint32_t lo = 0, hi = kp;  // number of keys of run o below `key`
      while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (run[mid] < key) lo = mid + 1; else hi = mid;
      }
      rank += lo;
    }
    if (rank < k) {
      if (out_ids) out_ids[qi * k + rank] = static_cast<int64_t>(key & 0xFFFFFFFFull);
      if (out_dists) out_dists[qi * k + rank] = key_dist(key);
      if (out_keys) out_keys[qi * k + rank] = key;
    }
  }
  valid = __reduce_add_sync(0xFFFFFFFFu, valid);
  for (uint32_t i = valid + lane; i < k; i += 32) {
    if (out_ids) out_ids[qi * k + i] = -1;
    if (out_dists) out_dists[qi * k + i] = kFltMax;
    if (out_keys) out_keys[qi * k + i] = kMaxKey;
  }
}

int merge_sorted_keys_impl(const uint64_t* d_keys, uint64_t nq, uint32_t parts, uint32_t kp, uint32_t k,
                           int64_t* d_out_ids, float* d_out_dists, uint64_t* d_out_keys, cudaStream_t st) {
  GRAB_REQUIRE(d_keys && ((d_out_ids && d_out_dists) || d_out_keys), "merge_sorted_keys: null pointer");
  GRAB_REQUIRE(parts >= 1 && parts <= 64 && kp >= 1 && kp <= 1024 && k >= 1 && k <= 1024,
               "merge_sorted_keys: parts %u / run length %u / k %u outside [1,64] / [1,1024] / [1,1024]", parts, kp, k);
  if (nq == 0) return GRAB_OK;
  const size_t per_warp = sizeof(uint64_t) * parts * kp;
  int warps = kMergeWarps;
  while (warps > 1 && per_warp * warps > 96 * 1024) warps >>= 1;
  const size_t smem = per_warp * warps;
  if (smem > 200 * 1024) {
    set_last_error("merge_sorted_keys: %u runs of %u keys need %zu bytes of shared memory", parts, kp, smem);
    return GRAB_ERR_UNSUPPORTED;
  }
  GRAB_CUDA_TRY(cudaFuncSetAttribute(merge_runs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  const uint64_t blocks = (nq + warps - 1) / warps;
  merge_runs_kernel<<<static_cast<unsigned>(blocks), 32 * warps, smem, st>>>(d_keys, nq, parts, kp, k, d_out_ids,
                                                                              d_out_dists, d_out_keys);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

// ---------------------------------------------------------------------------------------------------------
// NCCL, resolved at run time.
// ---------------------------------------------------------------------------------------------------------
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*get_unique_id)(ncclUniqueId*) = nullptr;
  ncclResult_t (*comm_init_rank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*all_gather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*comm_destroy)(ncclComm_t) = nullptr;
  const char* (*get_error_string)(ncclResult_t) = nullptr;
  bool ok = false;
};

static NcclApi& nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    // a host process that already uses NCCL (torch.distributed) has it loaded: share that copy
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW);
    if (!h) return;
    api.handle = h;
    api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
    api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
    api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
    api.get_error_string = reinterpret_cast<decltype(api.get_error_string)>(dlsym(h, "ncclGetErrorString"));
    api.ok = api.get_unique_id && api.comm_init_rank && api.all_gather && api.comm_destroy && api.get_error_string;
  });
  return api;
}

static int nccl_fail(const char* what, ncclResult_t r) {
  NcclApi& a = nccl_api();
  set_last_error("%s failed: %s", what, a.get_error_string ? a.get_error_string(r) : "unknown NCCL error");
  return GRAB_ERR_NCCL;
}

}  // namespace grab

struct grab_comm {
  ncclComm_t comm;
  int world, rank, device;
};

extern "C" {

int grab_merge_sorted_keys(const uint64_t* d_keys, uint64_t nq, uint32_t parts, uint32_t run_length, uint32_t k,
                           int64_t* d_out_ids, float* d_out_dists, void* stream) {
  return grab::merge_sorted_keys_impl(d_keys, nq, parts, run_length, k, d_out_ids, d_out_dists, nullptr,
                                      static_cast<cudaStream_t>(stream));
}

int grab_comm_unique_id(void* out, size_t bytes) {
  using namespace grab;
  GRAB_REQUIRE(out && bytes >= GRAB_COMM_UNIQUE_ID_BYTES, "comm_unique_id: the buffer must hold %d bytes",
               GRAB_COMM_UNIQUE_ID_BYTES);
  static_assert(sizeof(ncclUniqueId) == GRAB_COMM_UNIQUE_ID_BYTES, "unique id size");
  NcclApi& a = nccl_api();
  if (!a.ok) {
    set_last_error("NCCL (libnccl.so.2) could not be loaded");
    return GRAB_ERR_NCCL;
  }
  ncclUniqueId id;
  const ncclResult_t r = a.get_unique_id(&id);
  if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
  memcpy(out, &id, sizeof(id));
  return GRAB_OK;
}

int grab_comm_create(const void* unique_id, int world, int rank, grab_comm** out) {
  using namespace grab;
  GRAB_REQUIRE(unique_id && out, "comm_create: null pointer");
  GRAB_REQUIRE(world >= 1 && rank >= 0 && rank < world, "comm_create: rank %d outside [0,%d)", rank, world);
  NcclApi& a = nccl_api();
  if (!a.ok) {
    set_last_error("NCCL (libnccl.so.2) could not be loaded");
    return GRAB_ERR_NCCL;
  }
  int device = 0;
  GRAB_CUDA_TRY(cudaGetDevice(&device));
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  ncclComm_t comm = nullptr;
  const ncclResult_t r = a.comm_init_rank(&comm, world, id, rank);
  if (r != ncclSuccess) return nccl_fail("ncclCommInitRank", r);
  *out = new grab_comm{comm, world, rank, device};
  return GRAB_OK;
}

int grab_comm_destroy(grab_comm* comm) {
  using namespace grab;
  if (!comm) return GRAB_OK;
  NcclApi& a = nccl_api();
  ncclResult_t r = ncclSuccess;
  if (a.ok && comm->comm) r = a.comm_destroy(comm->comm);
  delete comm;
  return r == ncclSuccess ? GRAB_OK : nccl_fail("ncclCommDestroy", r);
}

int grab_comm_world(const grab_comm* comm) { return comm ? comm->world : 1; }
int grab_comm_rank(const grab_comm* comm) { return comm ? comm->rank : 0; }

int grab_sharded_gather_merge(grab_comm* comm, const uint64_t* d_keys, uint64_t nq, uint32_t run_length, uint32_t k,
                              uint64_t* d_gather, size_t gather_bytes, int64_t* d_out_ids, float* d_out_dists,
                              void* stream) {
  using namespace grab;
  GRAB_REQUIRE(d_keys && d_out_ids && d_out_dists, "sharded_gather_merge: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int world = comm ? comm->world : 1;
  if (world == 1) return merge_sorted_keys_impl(d_keys, nq, 1, run_length, k, d_out_ids, d_out_dists, nullptr, st);
  const size_t need = sizeof(uint64_t) * nq * run_length * world;
  if (!d_gather || gather_bytes < need) {
    set_last_error("sharded_gather_merge: gather buffer %zu < %zu bytes", gather_bytes, need);
    return GRAB_ERR_WORKSPACE;
  }
  NcclApi& a = nccl_api();
  if (!a.ok) {
    set_last_error("NCCL (libnccl.so.2) could not be loaded");
    return GRAB_ERR_NCCL;
  }
  if (nq > 0) {
    const ncclResult_t r = a.all_gather(d_keys, d_gather, nq * run_length, ncclUint64, comm->comm, st);
    if (r != ncclSuccess) return nccl_fail("ncclAllGather", r);
  }
  return merge_sorted_keys_impl(d_gather, nq, static_cast<uint32_t>(world), run_length, k, d_out_ids, d_out_dists, nullptr, st);
}

}  // extern "C"
