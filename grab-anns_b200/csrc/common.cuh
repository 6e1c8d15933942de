// Shared device/host helpers: status codes, the canonical fp32 distance, (dist,id) keys.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/grab_anns.h"

namespace grab {

constexpr uint32_t kInvalid = 0xFFFFFFFFu;  // empty graph slot / empty hash slot (reference: hashmap.cuh:15)
constexpr uint32_t kMsb = 0x80000000u;      // "already expanded" flag on queue ids (reference: search.cu:51)
constexpr uint64_t kMaxKey = 0xFFFFFFFFFFFFFFFFull;
constexpr float kFltMax = 3.40282e38f;      // the reference's FLT_MAX literal (compute_distance.cuh:161)

void set_last_error(const char* fmt, ...);

#define GRAB_CUDA_TRY(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      ::grab::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
                             __FILE__, __LINE__);                                        \
      return GRAB_ERR_CUDA;                                                              \
    }                                                                                    \
  } while (0)

#define GRAB_REQUIRE(cond, ...)              \
  do {                                       \
    if (!(cond)) {                           \
      ::grab::set_last_error(__VA_ARGS__);   \
      return GRAB_ERR_INVALID_ARGUMENT;      \
    }                                        \
  } while (0)

// Order-preserving float -> uint32 map, so that (dist, id) pairs sort as one uint64.
__host__ __device__ __forceinline__ uint32_t float_to_ordered(float f) {
#ifdef __CUDA_ARCH__
  uint32_t b = __float_as_uint(f);
#else
  uint32_t b;
  memcpy(&b, &f, 4);
#endif
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ __forceinline__ float ordered_to_float(uint32_t o) {
  uint32_t b = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
#ifdef __CUDA_ARCH__
  return __uint_as_float(b);
#else
  float f;
  memcpy(&f, &b, 4);
  return f;
#endif
}
__host__ __device__ __forceinline__ uint64_t make_key(float dist, uint32_t id) {
  return (static_cast<uint64_t>(float_to_ordered(dist)) << 32) | id;
}
__host__ __device__ __forceinline__ float key_dist(uint64_t key) {
  return ordered_to_float(static_cast<uint32_t>(key >> 32));
}
__host__ __device__ __forceinline__ uint32_t key_id(uint64_t key) {
  return static_cast<uint32_t>(key & 0xFFFFFFFFull);
}

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------
// Canonical fp32 distance.  A vector is cut into float4 chunks; chunk c belongs to lane
// (c mod 8) of a team of 8 consecutive lanes; a lane accumulates its chunks in ascending
// order (x, y, z, w in order, one fused multiply-add each); the 8 partial sums are combined
// by a butterfly at xor-offsets 4, 2, 1 (all 8 lanes end with the same bits).  The CPU
// oracle evaluates exactly this expression, which is what makes ids bit-exact.
// It replaces the reference's 32-lane scalar-load variant (compute_distance.cuh:14-139).
// ---------------------------------------------------------------------------------------
constexpr int kTeam = 8;

template <int METRIC>
__device__ __forceinline__ float accum4(float acc, const float4& q, const float4& x) {
  if (METRIC == GRAB_METRIC_L2) {
    float d;
    d = q.x - x.x; acc = __fmaf_rn(d, d, acc);
    d = q.y - x.y; acc = __fmaf_rn(d, d, acc);
    d = q.z - x.z; acc = __fmaf_rn(d, d, acc);
    d = q.w - x.w; acc = __fmaf_rn(d, d, acc);
  } else {
    acc = __fmaf_rn(q.x, x.x, acc);
    acc = __fmaf_rn(q.y, x.y, acc);
    acc = __fmaf_rn(q.z, x.z, acc);
    acc = __fmaf_rn(q.w, x.w, acc);
  }
  return acc;
}

// Butterfly over the 8 lanes of a team; every lane of the warp must call it.
template <int METRIC>
__device__ __forceinline__ float team_reduce(float acc) {
  acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 4));
  acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 2));
  acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 1));
  return METRIC == GRAB_METRIC_L2 ? acc : -acc;
}

__device__ __forceinline__ float4 ldg_f4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}

// Distance between a query held in shared memory and a dataset row, computed by one team.
// `lane8` = lane index inside the team.  All 32 lanes of the warp must take part (lanes of
// teams without work pass valid=false and read nothing).
template <int METRIC>
__device__ __forceinline__ float team_distance_smem(const float* __restrict__ q_smem,
                                                    const float* __restrict__ row, uint32_t nchunk,
                                                    int lane8, bool valid) {
  float acc = 0.0f;
  if (valid) {
    for (uint32_t c = lane8; c < nchunk; c += kTeam) {
      const float4 x = ldg_f4(row + 4 * c);
      const float4 q = *reinterpret_cast<const float4*>(q_smem + 4 * c);
      acc = accum4<METRIC>(acc, q, x);
    }
  }
  return team_reduce<METRIC>(acc);
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

// First index in [0, n) whose value is >= x (n if none) in a non-decreasing array, found by a
// whole warp: every round the 32 lanes probe 32 evenly spaced positions, so 2^20 entries take
// four dependent loads instead of twenty.  All lanes must call it and get the same result.
__device__ __forceinline__ uint32_t warp_lower_bound_u64(const uint64_t* __restrict__ a, uint32_t n, uint64_t x) {
  const uint32_t lane = lane_id();
  uint32_t b = 0, e = n;  // the answer lies in [b, e]
  while (e - b > 32) {
    const uint32_t span = e - b;
    const uint32_t pos = b + static_cast<uint32_t>((static_cast<uint64_t>(lane + 1) * span) / 33);  // b < pos < e
    const uint32_t below = __ballot_sync(0xFFFFFFFFu, __ldg(a + pos) < x);  // a prefix of the lanes
    const uint32_t k = __popc(below);
    const uint32_t nb = k > 0 ? b + static_cast<uint32_t>((static_cast<uint64_t>(k) * span) / 33) + 1 : b;
    const uint32_t ne = k < 32 ? b + static_cast<uint32_t>((static_cast<uint64_t>(k + 1) * span) / 33) : e;
    b = nb;
    e = ne;
  }
  const uint32_t below = __ballot_sync(0xFFFFFFFFu, b + lane < e && __ldg(a + b + lane) < x);
  return b + __popc(below);
}

// Block-wide bitonic sort of `n` (power of two) uint64 keys in shared memory, ascending.
// Every thread of the block must call it.
__device__ __forceinline__ void block_bitonic_sort(uint64_t* keys, uint32_t n) {
  for (uint32_t size = 2; size <= n; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      for (uint32_t t = threadIdx.x; t < (n >> 1); t += blockDim.x) {
        const uint32_t lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
        const uint32_t hi = lo | stride;
        const bool up = (lo & size) == 0;
        const uint64_t a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
}
// The same search over a[b0, e0) of a non-decreasing uint32 array.
__device__ __forceinline__ uint32_t warp_lower_bound_u32(const uint32_t* __restrict__ a, uint32_t b0, uint32_t e0,
                                                         uint32_t x) {
  const uint32_t lane = lane_id();
  uint32_t b = b0, e = e0;
  while (e - b > 32) {
    const uint32_t span = e - b;
    const uint32_t pos = b + static_cast<uint32_t>((static_cast<uint64_t>(lane + 1) * span) / 33);
    const uint32_t below = __ballot_sync(0xFFFFFFFFu, __ldg(a + pos) < x);
    const uint32_t k = __popc(below);
    const uint32_t nb = k > 0 ? b + static_cast<uint32_t>((static_cast<uint64_t>(k) * span) / 33) + 1 : b;
    const uint32_t ne = k < 32 ? b + static_cast<uint32_t>((static_cast<uint64_t>(k + 1) * span) / 33) : e;
    b = nb;
    e = ne;
  }
  const uint32_t below = __ballot_sync(0xFFFFFFFFu, b + lane < e && __ldg(a + b + lane) < x);
  return b + __popc(below);
}
#endif  // __CUDACC__

inline uint32_t next_pow2(uint32_t v) {
  if (v <= 1) return 1;
  v--;
  v |= v >> 1; v |= v >> 2; v |= v >> 4; v |= v >> 8; v |= v >> 16;
  return v + 1;
}

// Stage timing for the multi-stage host pipelines (build, insert).  Off by default; enabled by
// grab_set_trace(1) or the environment variable GRAB_TRACE=1.  Each mark synchronises the
// device and prints the time since the previous mark to stderr.  The reference has
// std::chrono stage timers of the same kind (cagra_opt.cu:1700,1848,1935,1962-1972).
int trace_level();
struct StageTimer {
  const char* scope;
  double t0 = 0.0;
  explicit StageTimer(const char* s);
  void mark(const char* stage);
};

// Grow-only device scratch that survives across calls (per device, per slot), for pipelines
// that run thousands of small batches (insert): no cudaMalloc / cudaFree per batch.  `zeroed`
// slots are cleared when (re)allocated and the kernels that use them leave them all-zero
// again.  Not for concurrent callers: one insert pipeline at a time per device.
enum PoolSlot {
  kPoolMailCountsL = 0, kPoolMailCountsR, kPoolMailCursor, kPoolMailOffsets, kPoolMailTouched, kPoolMailCsr,
  kPoolMailMeta, kPoolInsIdsG, kPoolInsDistG, kPoolInsIdsL, kPoolInsDistL, kPoolInsBatchIds, kPoolInsBatchDist,
  kPoolSearchWs, kPoolSearchWs2, kPoolRouteWs, kPoolRouteWs2, kPoolInsSeedsG, kPoolInsSeedsL, kPoolSlots
};
void* pool_get(int slot, size_t bytes, bool zeroed);
// Frees a slot so that its next pool_get allocates (and, for zeroed slots, clears) it afresh: for error paths
// that may leave a "zero between batches" slot dirty.
void pool_drop(int slot);

// What the time-partitioned insert may be told beyond the reference's arguments (NULL = the reference's behaviour:
// self-drawn seeds for the global search, the caller's seed list for the bucket search, the reference's slot rule
// for the reverse edges, device synchronisation before returning).
struct InsertOptions {
  const grab_router* router = nullptr;  // seeds of both searches from the entry-point router (old nodes only)
  uint32_t probes = 2, routed_seeds = 32;
  bool bucket_has_old_members = false;  // with a router: whether the bucket search can be seeded at all
  // id range of the target bucket's members among the old nodes (contiguous: bucket ids are non-decreasing in the
  // id) and the number of leading ids the router's member lists cover.  A bucket the router does not cover
  // completely (nodes inserted after its last assignment) gets uniform seeds from its id range instead.
  uint64_t bucket_begin = 0, bucket_end = 0, router_covers = 0;
  // reverse edges: 0 = the reference's pseudo-random slot; 1 = every request takes the slot of the farthest old
  // neighbour in the weak half; 2 = a request replaces the farthest neighbour only when it is closer
  int repair_mode = 0;
  bool sync = true;                     // false: only enqueue on `stream`
  cudaStream_t stream = nullptr;
};

// Scratch allocation used by the stateless entry points when the caller passes no
// workspace: plain cudaMalloc, released on scope exit.
struct ScopedDeviceBuffer {
  void* ptr = nullptr;
  cudaError_t alloc(size_t bytes) { return cudaMalloc(&ptr, bytes ? bytes : 1); }
  ~ScopedDeviceBuffer() { if (ptr) cudaFree(ptr); }
  template <class T> T* as() { return static_cast<T*>(ptr); }
};

}  // namespace grab
