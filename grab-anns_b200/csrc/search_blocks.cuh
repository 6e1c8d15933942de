// Building blocks of the filtered graph search, shared by graph_search.cu and the device-level
// unit-test entry points of selftest.cu: the visited set (reference: src/index/hashmap.cuh:30-117),
// the search-queue keys, and the one-warp sort / merge networks that replace the reference's
// per-iteration full queue sort (src/index/search.cu:110-144, bitonic.cuh:53, warp_merge_sort.cuh:29).
#pragma once
#include "common.cuh"

namespace grab {

__device__ __forceinline__ bool hash_insert(uint32_t* table, uint32_t bitlen, uint32_t key) {
  // Open addressing, linear probe, slot = (key ^ key>>bitlen) & mask: hashmap.cuh:43-91.
  const uint32_t mask = (1u << bitlen) - 1;
  uint32_t idx = (key ^ (key >> bitlen)) & mask;
  for (uint32_t i = 0; i <= mask; ++i) {
    const uint32_t old = atomicCAS(&table[idx], kInvalid, key);
    if (old == kInvalid) return true;
    if (old == key) return false;
    idx = (idx + 1) & mask;
  }
  return false;  // full table reads as "visited", as in the reference (hashmap.cuh:89-90)
}

// Search-queue keys: [ordered dist : 32 | id : 31 | expanded flag : 1].  Raising the flag of an
// entry cannot move it past another entry (ids are unique), so the list stays sorted.
__device__ __forceinline__ uint64_t make_skey(float d, uint32_t id) {
  return (static_cast<uint64_t>(float_to_ordered(d)) << 32) | (static_cast<uint64_t>(id) << 1);
}
__device__ __forceinline__ uint32_t skey_id(uint64_t key) { return static_cast<uint32_t>(key & 0xFFFFFFFFull) >> 1; }
__device__ __forceinline__ bool skey_expanded(uint64_t key) { return (key & 1ull) != 0; }

__device__ __forceinline__ uint64_t mix64(uint64_t x) {  // splitmix64 finaliser
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

// Ascending bitonic sort of n (power of two, >= 32) keys in shared memory by ONE warp.
__device__ __forceinline__ void warp_bitonic_sort_smem(uint64_t* keys, uint32_t n, uint32_t lane) {
  for (uint32_t size = 2; size <= n; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      for (uint32_t t = lane; t < (n >> 1); t += 32) {
        const uint32_t lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
        const uint32_t hi = lo | stride;
        const bool up = (lo & size) == 0;
        const uint64_t a = keys[lo], b = keys[hi];
        if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
      }
      __syncwarp();
    }
  }
}

// Fold `ncand` sorted candidate keys into the sorted list top[0..m) (m a power of two), keeping
// the m smallest: top[m-1-i] = min(top[m-1-i], cand[i]) leaves a bitonic sequence, which one
// pass of bitonic merge stages sorts again.  One warp.
__device__ __forceinline__ void warp_merge_into_topk(uint64_t* top, uint32_t m, const uint64_t* cand,
                                                     uint32_t ncand, uint32_t lane) {
  const uint32_t lim = ncand < m ? ncand : m;
  for (uint32_t i = lane; i < lim; i += 32) {
    const uint64_t a = top[m - 1 - i], b = cand[i];
    if (b < a) top[m - 1 - i] = b;
  }
  __syncwarp();
  for (uint32_t stride = m >> 1; stride > 0; stride >>= 1) {
    for (uint32_t t = lane; t < (m >> 1); t += 32) {
      const uint32_t lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
      const uint32_t hi = lo | stride;
      const uint64_t a = top[lo], b = top[hi];
      if (a > b) { top[lo] = b; top[hi] = a; }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------
// Register versions of the two functions above for lists of 32*R keys (R = 2, 4): element e
// lives in register e/32 of lane e%32.  Compare-exchanges at strides below 32 are xor-shuffles,
// strides of 32 and more pair registers of the same lane; no shared-memory round trip and no
// warp barrier per stage, which is what the shared-memory versions spend their time on.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t v, uint32_t mask) {
  return __shfl_xor_sync(0xFFFFFFFFu, v, mask);
}

// One bitonic stage at STRIDE inside sorted blocks of `size` (a block is ascending when its
// index has bit `size` clear).  STRIDE is a compile-time constant so that register indices are.
template <int R, uint32_t STRIDE>
__device__ __forceinline__ void reg_bitonic_stage(uint64_t (&v)[R], uint32_t size, uint32_t lane) {
  if (STRIDE >= 32) {
    constexpr uint32_t RS = STRIDE >> 5;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if ((r & RS) == 0) {
        const bool up = (((static_cast<uint32_t>(r) << 5) & size) == 0);
        const uint64_t a = v[r], b = v[(r | RS) < R ? (r | RS) : r];
        const bool swap = (a > b) == up;
        v[r] = swap ? b : a;
        v[(r | RS) < R ? (r | RS) : r] = swap ? a : b;
      }
    }
  } else {
    const bool lower = (lane & STRIDE) == 0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t e = lane + (static_cast<uint32_t>(r) << 5);
      const bool up = (e & size) == 0;
      const uint64_t other = shfl_xor_u64(v[r], STRIDE);
      const bool keep_min = lower == up;
      const uint64_t mn = v[r] < other ? v[r] : other, mx = v[r] < other ? other : v[r];
      v[r] = keep_min ? mn : mx;
    }
  }
}

// All stages of one level (block size 2^LOG): strides 2^(LOG-1) ... 1.
template <int R, int LOG, int S = LOG - 1>
struct RegBitonicLevel {
  static __device__ __forceinline__ void run(uint64_t (&v)[R], uint32_t size, uint32_t lane) {
    reg_bitonic_stage<R, (1u << S)>(v, size, lane);
    RegBitonicLevel<R, LOG, S - 1>::run(v, size, lane);
  }
};
template <int R, int LOG>
struct RegBitonicLevel<R, LOG, -1> {
  static __device__ __forceinline__ void run(uint64_t (&)[R], uint32_t, uint32_t) {}
};

// Levels 1 .. LOG of a bitonic sort; levels above `padded` are skipped, the level equal to
// `padded` sorts ascending (direction bit taken from the full list length M).
template <int R, int LOG>
struct RegBitonicSort {
  static __device__ __forceinline__ void run(uint64_t (&v)[R], uint32_t padded, uint32_t lane) {
    RegBitonicSort<R, LOG - 1>::run(v, padded, lane);
    constexpr uint32_t SIZE = 1u << LOG;
    if (SIZE <= padded) RegBitonicLevel<R, LOG>::run(v, SIZE == padded ? 32u * R : SIZE, lane);  // uniform
  }
};
template <int R>
struct RegBitonicSort<R, 0> {
  static __device__ __forceinline__ void run(uint64_t (&)[R], uint32_t, uint32_t) {}
};

template <int R> struct Log2Of32R;
template <> struct Log2Of32R<1> { static constexpr int value = 5; };
template <> struct Log2Of32R<2> { static constexpr int value = 6; };
template <> struct Log2Of32R<4> { static constexpr int value = 7; };
template <> struct Log2Of32R<8> { static constexpr int value = 8; };

// Sorts the nkeep (<= 32*R) candidate keys and folds them into the sorted list top[0..32*R).
template <int R>
__device__ __forceinline__ void warp_sort_merge_regs(uint64_t* top, const uint64_t* cand, uint32_t nkeep,
                                                     uint32_t lane) {
  constexpr uint32_t M = 32u * R;
  constexpr int LOGM = Log2Of32R<R>::value;
  uint64_t c[R], t[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t e = lane + 32u * r;
    c[r] = e < nkeep ? cand[e] : kMaxKey;
    t[r] = top[e];
  }
  // only as many sort levels as the candidates need (padded to a power of two >= 32)
  uint32_t padded = 32;
  while (padded < nkeep) padded <<= 1;
  RegBitonicSort<R, LOGM>::run(c, padded, lane);
  // sorted candidates occupy elements [0, padded); top[M-1-i] = min(top[M-1-i], cand[i])
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint64_t partner = __shfl_sync(0xFFFFFFFFu, c[R - 1 - r], 31u - lane);  // element M-1-e
    t[r] = partner < t[r] ? partner : t[r];
  }
  RegBitonicLevel<R, LOGM>::run(t, M, lane);
#pragma unroll
  for (int r = 0; r < R; ++r) top[lane + 32u * r] = t[r];
}

// the 128-entry variant is kept out of line so that its registers do not count against the
// common 64-entry path
static __device__ __noinline__ void warp_sort_merge_regs_128(uint64_t* top, const uint64_t* cand, uint32_t nkeep,
                                                      uint32_t lane) {
  warp_sort_merge_regs<4>(top, cand, nkeep, lane);
}

// ---------------------------------------------------------------------------------------
// Two-stage variant used when every warp of the CTA collects its own candidates: each warp
// sorts ITS kept keys in registers (warp_sort_regs), then one warp folds both sorted runs
// into the sorted list (warp_merge_runs_regs).  Of two ascending runs a and b only the M
// smallest of their union can enter a list of M entries; min(a[e], b[M-1-e]) for e < M is a
// bitonic sequence that holds exactly those, so one merge level sorts it, and a second one
// folds it into the list as above.
// ---------------------------------------------------------------------------------------
// Ascending in-place sort of keys[0, count), count <= 32*R, by one warp.
template <int R>
__device__ __forceinline__ void warp_sort_regs(uint64_t* keys, uint32_t count, uint32_t lane) {
  uint64_t c[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t e = lane + 32u * r;
    c[r] = e < count ? keys[e] : kMaxKey;
  }
  RegBitonicSort<R, Log2Of32R<R>::value>::run(c, 32u * R, lane);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t e = lane + 32u * r;
    if (e < count) keys[e] = c[r];
  }
}
static __device__ __noinline__ void warp_sort_regs_128(uint64_t* keys, uint32_t count, uint32_t lane) {
  warp_sort_regs<4>(keys, count, lane);
}
static __device__ __noinline__ void warp_sort_regs_256(uint64_t* keys, uint32_t count, uint32_t lane) {
  warp_sort_regs<8>(keys, count, lane);
}

// top[0, 32*R) sorted; run0[0, n0) and run1[0, n1) ascending.  Leaves the 32*R smallest of the union,
// sorted, in t (element e in register e/32 of lane e%32); the caller stores it.
template <int R>
__device__ __forceinline__ void warp_merge_runs_regs(const uint64_t* top, const uint64_t* run0, uint32_t n0,
                                                     const uint64_t* run1, uint32_t n1, uint32_t lane,
                                                     uint64_t (&t)[R]) {
  constexpr uint32_t M = 32u * R;
  constexpr int LOGM = Log2Of32R<R>::value;
  uint64_t c[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t e = lane + 32u * r;
    const uint64_t a = e < n0 ? run0[e] : kMaxKey;
    const uint64_t b = (M - 1 - e) < n1 ? run1[M - 1 - e] : kMaxKey;
    c[r] = a < b ? a : b;
    t[r] = top[e];
  }
  RegBitonicLevel<R, LOGM>::run(c, M, lane);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint64_t partner = __shfl_sync(0xFFFFFFFFu, c[R - 1 - r], 31u - lane);  // element M-1-e
    t[r] = partner < t[r] ? partner : t[r];
  }
  RegBitonicLevel<R, LOGM>::run(t, M, lane);
}

// ---------------------------------------------------------------------------------------
// Merge by rank, for the common late-iteration case of a handful of kept keys: no sort at all.
// The list top[0, 32*R) is sorted, the K <= 32 candidate keys are NOT (lane j holds candidate j).
// All keys are distinct (ids are unique), so every key's position in the merged order is
//   list entry e    : e + #{candidates below it}
//   candidate j     : #{list entries below it} + #{candidates below it}
// and each key is written straight to that slot (if it is still inside the list).  One pass over
// the candidates by shuffle serves both counts.  The list is left sorted in shared memory AND in
// t (element e in register e/32 of lane e%32).
// ---------------------------------------------------------------------------------------
template <int R>
__device__ __forceinline__ void warp_merge_by_rank(uint64_t* top, uint64_t cand, uint32_t K, uint32_t lane,
                                                   uint64_t (&t)[R]) {
  constexpr uint32_t M = 32u * R;
#pragma unroll
  for (int r = 0; r < R; ++r) t[r] = top[lane + 32u * r];
  // candidates below each list entry / below my candidate
  uint32_t below_t[R];
#pragma unroll
  for (int r = 0; r < R; ++r) below_t[r] = 0;
  uint32_t below_c = 0;
  for (uint32_t j = 0; j < K; ++j) {
    const uint64_t cj = __shfl_sync(0xFFFFFFFFu, cand, j);
    below_c += cj < cand;
#pragma unroll
    for (int r = 0; r < R; ++r) below_t[r] += cj < t[r];
  }
  // list entries below my candidate: lower bound in the sorted list
  uint32_t lo = 0, hi = M;
  if (lane < K) {
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if (top[mid] < cand) lo = mid + 1; else hi = mid;
    }
  }
  __syncwarp();  // every read of the old list is done
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t pos = lane + 32u * r + below_t[r];
    if (pos < M) top[pos] = t[r];
  }
  if (lane < K && lo + below_c < M) top[lo + below_c] = cand;
  __syncwarp();
#pragma unroll
  for (int r = 0; r < R; ++r) t[r] = top[lane + 32u * r];
}

}  // namespace grab
