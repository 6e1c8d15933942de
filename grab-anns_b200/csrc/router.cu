// Entry-point router: filter-aware search seeds close to the query.
//
// The reference samples search seeds on the host, uniformly among the ids that pass the filter
// (cagraIndexOpt.cu:441-511 for query_range, :313-336 for query_local, cagraIndex.cu:267-296),
// and its two-level index routes a query through k-means centroids, each with a few entry
// points (timeStampIndex.cu:141-238 build_virtual_index, :240-419 query).  This file is the
// device version of both ideas in one structure:
//
//   build : Lloyd's k-means over a strided sample of the dataset (every step deterministic),
//           then every vector is assigned to its nearest centroid and the ids are grouped by
//           centroid, ascending inside each group (a CSR list).
//   route : per query the `probes` nearest centroids (one tiled fp32 GEMM-with-selection
//           kernel), then for every (centroid, filter window) pair a few members of the
//           centroid's id list that fall inside the window -- found by binary search because
//           the list is sorted by id and a sorted-timestamp range or a label range is an id
//           range.  Filters without id windows draw members and test the predicate.
//
// The result is the [nq, seeds_per_query] uint32 seed array every search entry point takes
// (d_seeds); slots that found nothing hold 0xFFFFFFFF and the search kernel fills them with
// its own pseudo-random draws.
#include "common.cuh"

namespace grab {
namespace {

constexpr int kRtBM = 64;        // rows (queries or vectors) per CTA
constexpr int kRtBN = 64;        // centroids per tile
constexpr int kRtBK = 32;        // dimensions per shared-memory stage
constexpr int kRtThreads = 256;  // 16 x 16 threads, 4 x 4 outputs each
constexpr uint32_t kMaxProbes = 16;
constexpr uint32_t kMaxSharedPairs = 64;  // (probe, window) pairs whose sub-runs are shared through shared memory
constexpr uint32_t kMaxSlices = 8;  // centroid slices of the routing launch (more CTAs for few queries)

__device__ __forceinline__ uint64_t rt_mix64(uint64_t x) {  // splitmix64 finaliser
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

// ---------------------------------------------------------------------------------------
// Nearest centroids.  score(x, c) = |c|^2 - 2 x.c (L2, the |x|^2 term is the same for all
// centroids) or -x.c (inner product); x.c is ONE fused-multiply-add chain over the dimensions
// in ascending order, so a CPU loop reproduces the bits.  Each row keeps its `P` best
// (score, centroid) keys, ties to the lower centroid id.
// ---------------------------------------------------------------------------------------
template <int METRIC>
__global__ void __launch_bounds__(kRtThreads)
nearest_centroids_kernel(const float* __restrict__ X, uint64_t m, uint32_t dim,
                         const float* __restrict__ cen, const float* __restrict__ cnorm, uint32_t C,
                         uint32_t P, uint32_t* __restrict__ out_ids, uint64_t* __restrict__ out_keys) {
  // blockIdx.x = row tile, blockIdx.y = slice of the centroids (gridDim.y slices of whole tiles).
  // out_ids  [m, P]             : centroid ids, best first (gridDim.y must be 1)
  // out_keys [m, gridDim.y, P]  : the slice's best (score, centroid) keys, merged by the consumer
  __shared__ __align__(16) float As[kRtBK][kRtBM + 4];
  __shared__ __align__(16) float Bs[kRtBK][kRtBN + 4];
  __shared__ float S[kRtBM][kRtBN + 1];
  __shared__ uint64_t top[kMaxProbes][kRtBM];

  const uint32_t tid = threadIdx.x;
  const uint32_t tx = tid & 15u, ty = tid >> 4;
  const uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * kRtBM;
  // this thread's two float4 of a 64 x 32 stage: rows lrow and lrow + 32, dimensions lk..lk+3
  const uint32_t lrow = tid >> 3, lk = (tid & 7u) * 4;
  const uint32_t tiles = (C + kRtBN - 1) / kRtBN;
  const uint32_t tiles_per = (tiles + gridDim.y - 1) / gridDim.y;
  const uint32_t c_begin = blockIdx.y * tiles_per * kRtBN;
  const uint32_t c_end = (c_begin + tiles_per * kRtBN) < C ? (c_begin + tiles_per * kRtBN) : C;

  for (uint32_t j = tid; j < kMaxProbes * kRtBM; j += kRtThreads) (&top[0][0])[j] = kMaxKey;

  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool r0 = row0 + lrow < m, r1 = row0 + lrow + 32 < m;
  const float* xa = X + (row0 + lrow) * dim + lk;
  const float* xb = xa + 32ull * dim;

  for (uint32_t c0 = c_begin; c0 < c_end; c0 += kRtBN) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    const bool b0 = c0 + lrow < C, b1 = c0 + lrow + 32 < C;
    const float* ca = cen + static_cast<uint64_t>(c0 + lrow) * dim + lk;
    const float* cb = ca + 32ull * dim;

    // software pipeline: the loads of stage s+1 are in flight while stage s is multiplied
    float4 a0 = zero4, a1 = zero4, q0 = zero4, q1 = zero4;
    if (lk < dim) {
      if (r0) a0 = ldg_f4(xa);
      if (r1) a1 = ldg_f4(xb);
      if (b0) q0 = ldg_f4(ca);
      if (b1) q1 = ldg_f4(cb);
    }
    for (uint32_t k0 = 0; k0 < dim; k0 += kRtBK) {
      __syncthreads();  // the previous stage (and the previous tile's row scan) is done
      As[lk + 0][lrow] = a0.x; As[lk + 1][lrow] = a0.y; As[lk + 2][lrow] = a0.z; As[lk + 3][lrow] = a0.w;
      As[lk + 0][lrow + 32] = a1.x; As[lk + 1][lrow + 32] = a1.y; As[lk + 2][lrow + 32] = a1.z; As[lk + 3][lrow + 32] = a1.w;
      Bs[lk + 0][lrow] = q0.x; Bs[lk + 1][lrow] = q0.y; Bs[lk + 2][lrow] = q0.z; Bs[lk + 3][lrow] = q0.w;
      Bs[lk + 0][lrow + 32] = q1.x; Bs[lk + 1][lrow + 32] = q1.y; Bs[lk + 2][lrow + 32] = q1.z; Bs[lk + 3][lrow + 32] = q1.w;
      __syncthreads();
      const uint32_t kn = k0 + kRtBK + lk;
      a0 = a1 = q0 = q1 = zero4;
      if (kn < dim) {
        if (r0) a0 = ldg_f4(xa + k0 + kRtBK);
        if (r1) a1 = ldg_f4(xb + k0 + kRtBK);
        if (b0) q0 = ldg_f4(ca + k0 + kRtBK);
        if (b1) q1 = ldg_f4(cb + k0 + kRtBK);
      }
#pragma unroll
      for (int kk = 0; kk < kRtBK; ++kk) {
        const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
        const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
        const float ar[4] = {av.x, av.y, av.z, av.w};
        const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(ar[i], br[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t c = c0 + tx * 4 + j;
      const float cn = (METRIC == GRAB_METRIC_L2 && c < C) ? __ldg(cnorm + c) : 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        S[ty * 4 + i][tx * 4 + j] = METRIC == GRAB_METRIC_L2 ? __fmaf_rn(-2.0f, acc[i][j], cn) : -acc[i][j];
    }
    __syncthreads();
    if (tid < kRtBM && row0 + tid < m) {  // one thread per row folds the tile into the row's list
      uint64_t worst = top[P - 1][tid];
      const uint32_t ncol = C - c0 < kRtBN ? C - c0 : kRtBN;
      for (uint32_t col = 0; col < ncol; ++col) {
        const uint64_t key = make_key(S[tid][col], c0 + col);
        if (key < worst) {
          uint32_t j = P - 1;
          while (j > 0 && top[j - 1][tid] > key) {
            top[j][tid] = top[j - 1][tid];
            --j;
          }
          top[j][tid] = key;
          worst = top[P - 1][tid];
        }
      }
    }
  }
  __syncthreads();
  for (uint32_t j = tid; j < kRtBM * P; j += kRtThreads) {
    const uint32_t r = j / P, p = j % P;
    if (row0 + r < m) {
      const uint64_t key = top[p][r];
      if (out_keys) out_keys[((row0 + r) * gridDim.y + blockIdx.y) * P + p] = key;
      else out_ids[(row0 + r) * P + p] = key == kMaxKey ? kInvalid : key_id(key);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Grouping ids by centroid, ascending inside each group, without a sort and without atomics
// on positions: ids are cut into chunks of consecutive ids; counts[chunk][c] is turned into
// the chunk's first slot inside group c by a column scan; one warp then walks its chunk in id
// order and hands out slots (lanes with the same centroid are ranked by lane index).
// ---------------------------------------------------------------------------------------
constexpr uint32_t kChunk = 2048;

__global__ void chunk_count_kernel(const uint32_t* __restrict__ assign, uint64_t n, uint32_t C,
                                   uint32_t* __restrict__ counts) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t c = assign[i];
  if (c < C) atomicAdd(&counts[(i / kChunk) * C + c], 1u);
}

__global__ void column_scan_kernel(uint32_t* __restrict__ counts, uint32_t nchunks, uint32_t C,
                                   uint32_t* __restrict__ totals) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  uint32_t run = 0;
  for (uint32_t ch = 0; ch < nchunks; ++ch) {
    const uint32_t v = counts[static_cast<uint64_t>(ch) * C + c];
    counts[static_cast<uint64_t>(ch) * C + c] = run;
    run += v;
  }
  totals[c] = run;
}

// offsets[0..C] = exclusive scan of totals; one CTA of 1024 threads.
__global__ void offsets_kernel(const uint32_t* __restrict__ totals, uint32_t C, uint32_t* __restrict__ offsets) {
  __shared__ uint32_t part[1024];
  const uint32_t t = threadIdx.x;
  const uint32_t per = (C + 1023) / 1024;
  const uint32_t b = t * per, e = b + per < C ? b + per : C;
  uint32_t s = 0;
  for (uint32_t c = b; c < e; ++c) s += totals[c];
  part[t] = s;
  __syncthreads();
  if (t == 0) {
    uint32_t run = 0;
    for (uint32_t j = 0; j < 1024; ++j) {
      const uint32_t v = part[j];
      part[j] = run;
      run += v;
    }
    offsets[C] = run;
  }
  __syncthreads();
  uint32_t run = part[t];
  for (uint32_t c = b; c < e; ++c) {
    offsets[c] = run;
    run += totals[c];
  }
}

__global__ void chunk_fill_kernel(const uint32_t* __restrict__ assign, uint64_t n, uint32_t C,
                                  uint32_t* __restrict__ counts, const uint32_t* __restrict__ offsets,
                                  uint32_t* __restrict__ members) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t begin = static_cast<uint64_t>(warp) * kChunk;
  if (begin >= n) return;
  const uint64_t end = begin + kChunk < n ? begin + kChunk : n;
  uint32_t* row = counts + static_cast<uint64_t>(warp) * C;  // private to this warp
  for (uint64_t i0 = begin; i0 < end; i0 += 32) {
    const uint64_t i = i0 + lane;
    const uint32_t c = i < end ? assign[i] : kInvalid;
    const bool valid = c < C;
    const uint32_t mask = __match_any_sync(0xFFFFFFFFu, c);
    const uint32_t rank = __popc(mask & ((1u << lane) - 1u));
    const int leader = __ffs(mask) - 1;
    uint32_t base = 0;
    if (valid && static_cast<int>(lane) == leader) {
      base = row[c];
      row[c] = base + __popc(mask);
    }
    base = __shfl_sync(0xFFFFFFFFu, base, leader);
    if (valid) members[offsets[c] + base + rank] = static_cast<uint32_t>(i);
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------
// k-means pieces.  Sample row s is dataset row floor(s * n / m).
// ---------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ X, uint64_t n, uint32_t dim, uint64_t m,
                                   uint64_t out_rows, float* __restrict__ out) {
  // out row r = X row floor((r * m / out_rows) * n / m): out_rows == m gives the sample itself,
  // out_rows == C gives C sample rows spread evenly (the initial centroids)
  const uint32_t nchunk = dim / 4;
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= out_rows * nchunk) return;
  const uint64_t r = idx / nchunk, c = idx % nchunk;
  const uint64_t s = r * m / out_rows;
  const uint64_t src = s * n / m;  // s < m <= n < 2^31: no overflow
  reinterpret_cast<float4*>(out)[r * nchunk + c] = ldg_f4(X + src * dim + 4 * c);
}

// Squared norm of a row held by one warp: lane l takes dimensions l, l+32, ... ascending
// (fused multiply-add), then a butterfly over xor 16, 8, 4, 2, 1.
__device__ __forceinline__ float warp_sqnorm(const float* v, uint32_t dim, uint32_t lane) {
  float acc = 0.0f;
  for (uint32_t k = lane; k < dim; k += 32) acc = __fmaf_rn(v[k], v[k], acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, o));
  return acc;
}

// One CTA per centroid: mean of its sample members, summed in ascending sample order with
// plain fp32 adds; empty groups keep the old centroid.  For the inner-product metric the mean
// is scaled to unit length (spherical k-means).  Also writes |c|^2.
__global__ void __launch_bounds__(128)
centroid_update_kernel(const float* __restrict__ sample, uint32_t dim, const uint32_t* __restrict__ offsets,
                       const uint32_t* __restrict__ members, int metric, float* __restrict__ cen,
                       float* __restrict__ cnorm) {
  extern __shared__ float v[];  // dim floats
  __shared__ float s_norm;
  const uint32_t c = blockIdx.x;
  const uint32_t b = offsets[c], e = offsets[c + 1];
  float* out = cen + static_cast<uint64_t>(c) * dim;
  for (uint32_t k = threadIdx.x; k < dim; k += blockDim.x) {
    float val = out[k];
    if (e > b) {
      float s = 0.0f;
      for (uint32_t j = b; j < e; ++j) s = __fadd_rn(s, __ldg(sample + static_cast<uint64_t>(members[j]) * dim + k));
      val = __fdiv_rn(s, static_cast<float>(e - b));
    }
    v[k] = val;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const float n2 = warp_sqnorm(v, dim, threadIdx.x);
    if (threadIdx.x == 0) s_norm = n2;
  }
  __syncthreads();
  if (metric == GRAB_METRIC_IP && e > b && s_norm > 0.0f) {
    const float len = __fsqrt_rn(s_norm);
    for (uint32_t k = threadIdx.x; k < dim; k += blockDim.x) v[k] = __fdiv_rn(v[k], len);
    __syncthreads();
    if (threadIdx.x < 32) {
      const float n2 = warp_sqnorm(v, dim, threadIdx.x);
      if (threadIdx.x == 0) s_norm = n2;
    }
    __syncthreads();
  }
  for (uint32_t k = threadIdx.x; k < dim; k += blockDim.x) out[k] = v[k];
  if (threadIdx.x == 0) cnorm[c] = s_norm;
}

// ---------------------------------------------------------------------------------------
// Seeds.  One warp per query.  Slot s: probe j = s mod p, t = s div p, window w = t mod nwin,
// pick r = t div nwin.  The members of centroid probes[j] inside window w form a sub-run of
// length L of the centroid's sorted id list; pick r takes element (start + r * step) mod L
// with step = max(1, L / per), per = ceil(S / (p * nwin)), start pseudo-random: picks of one
// pair are distinct, pairs are disjoint, so a query never gets the same seed twice.
// ---------------------------------------------------------------------------------------
struct RouteArgs {
  const uint64_t* keys;  // [nq, slices, T] (score, centroid) keys of every centroid slice, ascending
  uint32_t slices, T;    // T = p (exact keys) or p + extra (tf32 keys, re-scored here)
  int rescore;           // keys came from the tensor-core kernel
  const int* status;     // non-zero: the tensor-core kernel gave up, write "no seed" everywhere
  const float* queries; const float* cen; const float* cnorm; uint32_t dim; int metric;
  uint32_t p, S, C;
  uint64_t nq, n, seed;
  const uint32_t* offsets;
  const uint32_t* members;
  int filter_kind, ts_sorted;
  const uint64_t* ts; const uint64_t* lo; const uint64_t* hi; uint64_t lo1, hi1;
  const uint8_t* labels; const uint32_t* masks; uint32_t mask1; const uint32_t* label_offsets;
  uint32_t* seeds;  // [nq, S]
  uint32_t* id_windows;  // [nq, 4] or NULL: the id window of every query's range is left here for the search
};

__device__ __forceinline__ uint32_t lower_bound_u32(const uint32_t* a, uint32_t b, uint32_t e, uint32_t x) {
  while (b < e) {  // first position in [b,e) with a[pos] >= x
    const uint32_t mid = (b + e) >> 1;
    if (a[mid] < x) b = mid + 1; else e = mid;
  }
  return b;
}

__global__ void __launch_bounds__(256) route_seeds_kernel(RouteArgs a) {
  __shared__ uint32_t s_probes[8][kMaxProbes];
  __shared__ uint32_t s_pair_b[8][kMaxSharedPairs], s_pair_e[8][kMaxSharedPairs];
  const uint64_t q = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  if (q >= a.nq) return;  // whole warps leave together
  const uint32_t n32 = static_cast<uint32_t>(a.n);
  uint32_t* probes = s_probes[threadIdx.x >> 5];
  if (a.status && *a.status != 0) {
    for (uint32_t s = lane; s < a.S; s += 32) a.seeds[q * a.S + s] = kInvalid;
    return;
  }
  {
    // merge of the slices' lists: rounds of "smallest remaining key" (keys are distinct)
    uint64_t mine[kMaxSlices * kMaxProbes / 32];
    const uint32_t total = a.slices * a.T;
#pragma unroll
    for (uint32_t i = 0; i < kMaxSlices * kMaxProbes / 32; ++i)
      mine[i] = lane + 32 * i < total ? a.keys[q * total + lane + 32 * i] : kMaxKey;
    uint64_t cand_key = kMaxKey;  // lane j ends up with the j-th smallest key
    for (uint32_t j = 0; j < a.T; ++j) {
      uint64_t best = mine[0];
#pragma unroll
      for (uint32_t i = 1; i < kMaxSlices * kMaxProbes / 32; ++i) best = mine[i] < best ? mine[i] : best;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        best = other < best ? other : best;
      }
#pragma unroll
      for (uint32_t i = 0; i < kMaxSlices * kMaxProbes / 32; ++i)
        if (mine[i] == best) mine[i] = kMaxKey;
      if (lane == j) cand_key = best;
    }
    if (a.rescore) {
      // exact score of candidate `lane`: the same fused-multiply-add chain as the exact scan
      if (cand_key != kMaxKey) {
        const uint32_t c = key_id(cand_key);
        const float* qv = a.queries + q * a.dim;
        const float* cv = a.cen + static_cast<uint64_t>(c) * a.dim;
        float acc = 0.0f;
        for (uint32_t k = 0; k < a.dim; k += 4) {
          const float4 x = ldg_f4(qv + k), y = ldg_f4(cv + k);
          acc = __fmaf_rn(x.x, y.x, acc);
          acc = __fmaf_rn(x.y, y.y, acc);
          acc = __fmaf_rn(x.z, y.z, acc);
          acc = __fmaf_rn(x.w, y.w, acc);
        }
        const float sc = a.metric == GRAB_METRIC_L2 ? __fmaf_rn(-2.0f, acc, __ldg(a.cnorm + c)) : -acc;
        cand_key = make_key(sc, c);
      }
    }
    for (uint32_t j = 0; j < a.p; ++j) {  // the p best of the (re-scored) candidates, best first
      uint64_t best = cand_key;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        best = other < best ? other : best;
      }
      if (cand_key == best) cand_key = kMaxKey;
      if (lane == 0) probes[j] = best == kMaxKey ? kInvalid : key_id(best);
    }
    __syncwarp();
  }
  // the query's id windows
  uint32_t nwin = 1, wlo = 0, whi = n32, mask = 0;
  bool check = false;  // no id window: test the predicate on every pick
  uint64_t tlo = 0, thi = 0;
  if (a.filter_kind == GRAB_FILTER_TS_RANGE || (a.filter_kind == GRAB_FILTER_PREFIX && a.ts)) {
    tlo = a.lo ? a.lo[q] : a.lo1;
    thi = a.hi ? a.hi[q] : a.hi1;
    if (a.ts_sorted) {
      wlo = warp_lower_bound_u64(a.ts, n32, tlo);
      whi = warp_lower_bound_u64(a.ts, n32, thi);
      if (a.id_windows && lane == 0 && a.filter_kind == GRAB_FILTER_TS_RANGE)
        *reinterpret_cast<uint4*>(a.id_windows + q * 4) = make_uint4(wlo, whi, 0u, 0u);
      if (whi <= wlo) nwin = 0;
    } else {
      check = true;
      if (thi <= tlo) nwin = 0;
    }
  } else if (a.filter_kind == GRAB_FILTER_LABELS) {
    mask = a.masks ? a.masks[q] : a.mask1;
    if (a.label_offsets) nwin = __popc(mask);
    else { check = true; if (mask == 0) nwin = 0; }
  }
  const uint32_t p = a.p;
  const uint32_t pairs = p * (nwin ? nwin : 1);
  const uint32_t per = (a.S + pairs - 1) / pairs;

  // id window of label `w` of the mask (labels grouped by id), else the query's one window
  auto window_of = [&](uint32_t w, uint32_t& lo_id, uint32_t& hi_id) {
    lo_id = wlo;
    hi_id = whi;
    if (a.filter_kind == GRAB_FILTER_LABELS && a.label_offsets) {
      uint32_t mm = mask;
      for (uint32_t skip = w; skip > 0; --skip) mm &= mm - 1;
      const uint32_t lab = __ffs(mm) - 1;
      lo_id = a.label_offsets[lab];
      hi_id = a.label_offsets[lab + 1];
    }
  };
  // Sub-run [b, e) of every (probe j, window w) pair, pair index j + p*w: computed once per pair --
  // by the whole warp (32-way search) when the pairs are few, else one pair per lane -- and shared
  // through shared memory; the slots below only pick positions inside their pair's sub-run.
  uint32_t* pb = s_pair_b[threadIdx.x >> 5];
  uint32_t* pe = s_pair_e[threadIdx.x >> 5];
  const bool shared_pairs = nwin != 0 && pairs <= kMaxSharedPairs;
  if (shared_pairs) {
    if (pairs <= 4) {
      for (uint32_t pi = 0; pi < pairs; ++pi) {  // uniform across the warp
        const uint32_t c = probes[pi % p];
        uint32_t b = 0, e = 0;
        if (c < a.C) {
          uint32_t lo_id, hi_id;
          window_of(pi / p, lo_id, hi_id);
          const uint32_t rb = a.offsets[c], re = a.offsets[c + 1];
          b = warp_lower_bound_u32(a.members, rb, re, lo_id);
          e = warp_lower_bound_u32(a.members, b, re, hi_id);
        }
        if (lane == 0) { pb[pi] = b; pe[pi] = e; }
      }
    } else {
      for (uint32_t pi = lane; pi < pairs; pi += 32) {
        const uint32_t c = probes[pi % p];
        uint32_t b = 0, e = 0;
        if (c < a.C) {
          uint32_t lo_id, hi_id;
          window_of(pi / p, lo_id, hi_id);
          const uint32_t rb = a.offsets[c], re = a.offsets[c + 1];
          b = lower_bound_u32(a.members, rb, re, lo_id);
          e = lower_bound_u32(a.members, b, re, hi_id);
        }
        pb[pi] = b;
        pe[pi] = e;
      }
    }
    __syncwarp();
  }

  for (uint32_t s = lane; s < a.S; s += 32) {
    uint32_t id = kInvalid;
    if (nwin) {
      const uint32_t j = s % p, t = s / p, w = t % nwin, r = t / nwin;
      const uint32_t c = probes[j];
      if (c < a.C) {
        uint32_t b, e;
        if (shared_pairs) {
          b = pb[j + p * w];
          e = pe[j + p * w];
        } else {
          uint32_t lo_id, hi_id;
          window_of(w, lo_id, hi_id);
          const uint32_t rb = a.offsets[c], re = a.offsets[c + 1];
          b = lower_bound_u32(a.members, rb, re, lo_id);
          e = lower_bound_u32(a.members, b, re, hi_id);
        }
        const uint32_t L = e - b;
        if (r < L) {
          const uint32_t step = L / per > 1 ? L / per : 1;
          const uint32_t start = static_cast<uint32_t>(
              rt_mix64(a.seed ^ (q * 0x9e3779b97f4a7c15ull + (static_cast<uint64_t>(c) << 8) + w)) % L);
          const uint32_t pos = static_cast<uint32_t>((start + static_cast<uint64_t>(r) * step) % L);
          if (!check) {
            id = a.members[b + pos];
          } else {
            // a pick that fails the predicate is replaced by the next members of the run (4 tries);
            // tries of different picks may meet, the search kernel drops duplicate seeds
            for (uint32_t tr = 0; tr < 4 && tr < L; ++tr) {
              const uint32_t cand = a.members[b + (pos + tr) % L];
              bool ok;
              if (a.filter_kind == GRAB_FILTER_LABELS) ok = ((mask >> (a.labels[cand] & 31u)) & 1u) != 0;
              else { const uint64_t tv = a.ts[cand]; ok = tv >= tlo && tv < thi; }
              if (ok) { id = cand; break; }
            }
          }
        }
      }
    }
    a.seeds[q * a.S + s] = id;
  }
}

template <int METRIC>
cudaError_t launch_nearest(const float* X, uint64_t m, uint32_t dim, const float* cen, const float* cnorm,
                           uint32_t C, uint32_t P, uint32_t* out_ids, uint64_t* out_keys, uint32_t slices,
                           cudaStream_t st) {
  if (m == 0) return cudaSuccess;
  const dim3 grid(static_cast<unsigned>((m + kRtBM - 1) / kRtBM), slices);
  nearest_centroids_kernel<METRIC><<<grid, kRtThreads, 0, st>>>(X, m, dim, cen, cnorm, C, P, out_ids, out_keys);
  return cudaGetLastError();
}

cudaError_t nearest(int metric, const float* X, uint64_t m, uint32_t dim, const float* cen, const float* cnorm,
                    uint32_t C, uint32_t P, uint32_t* out_ids, cudaStream_t st, uint64_t* out_keys = nullptr,
                    uint32_t slices = 1) {
  return metric == GRAB_METRIC_L2
             ? launch_nearest<GRAB_METRIC_L2>(X, m, dim, cen, cnorm, C, P, out_ids, out_keys, slices, st)
             : launch_nearest<GRAB_METRIC_IP>(X, m, dim, cen, cnorm, C, P, out_ids, out_keys, slices, st);
}

// Centroid slices for a routing launch of nq queries: enough CTAs to fill the GPU a few times.
uint32_t route_slices(uint64_t nq, uint32_t C) {
  const uint64_t row_tiles = (nq + kRtBM - 1) / kRtBM;
  const uint32_t col_tiles = (C + kRtBN - 1) / kRtBN;
  uint32_t s = 1;
  while (s < kMaxSlices && s * 2 <= col_tiles && row_tiles * s < 4 * 148) s *= 2;
  return s;
}

// assign[m] -> offsets[C+1], members[m]; counts is scratch of ceil(m/kChunk) * C words
int group_by_centroid(const uint32_t* assign, uint64_t m, uint32_t C, uint32_t* counts, uint32_t* totals,
                      uint32_t* offsets, uint32_t* members, cudaStream_t st) {
  const uint32_t nchunks = static_cast<uint32_t>((m + kChunk - 1) / kChunk);
  GRAB_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(uint32_t) * static_cast<size_t>(nchunks) * C, st));
  chunk_count_kernel<<<static_cast<unsigned>((m + 255) / 256), 256, 0, st>>>(assign, m, C, counts);
  column_scan_kernel<<<(C + 255) / 256, 256, 0, st>>>(counts, nchunks, C, totals);
  offsets_kernel<<<1, 1024, 0, st>>>(totals, C, offsets);
  chunk_fill_kernel<<<(nchunks * 32 + 255) / 256, 256, 0, st>>>(assign, m, C, counts, offsets, members);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

}  // namespace

int router_build_impl(const float* d_dataset, uint32_t dim, uint64_t n, int metric, uint32_t C, uint32_t iterations,
                      uint64_t max_sample, float* d_centroids, float* d_cnorm, uint32_t* d_offsets,
                      uint32_t* d_members, cudaStream_t st) {
  GRAB_REQUIRE(d_dataset && d_centroids && d_cnorm && d_offsets && d_members, "router_build: null pointer");
  GRAB_REQUIRE(dim >= 4 && dim % 4 == 0, "router_build: dim %u must be a multiple of 4", dim);
  GRAB_REQUIRE(n >= 1 && n < (1ull << 31), "router_build: n must be in [1, 2^31)");
  GRAB_REQUIRE(C >= 1 && C <= 65536 && C <= n, "router_build: num_centroids %u outside [1, min(n, 65536)]", C);
  GRAB_REQUIRE(metric == GRAB_METRIC_L2 || metric == GRAB_METRIC_IP, "router_build: bad metric");
  GRAB_REQUIRE(dim * sizeof(float) <= 48 * 1024, "router_build: dim %u too large", dim);
  StageTimer timer("router_build");
  uint64_t m = max_sample ? max_sample : 64ull * C;  // k-means sample size
  if (m > n) m = n;
  if (m < C) m = C;
  const uint64_t big = n > m ? n : m;
  const uint32_t nchunks = static_cast<uint32_t>((big + kChunk - 1) / kChunk);
  ScopedDeviceBuffer sample, assign, counts, totals, soffs, smembers;
  if (iterations > 0) GRAB_CUDA_TRY(sample.alloc(sizeof(float) * m * dim));
  GRAB_CUDA_TRY(assign.alloc(sizeof(uint32_t) * big));
  GRAB_CUDA_TRY(counts.alloc(sizeof(uint32_t) * static_cast<size_t>(nchunks) * C));
  GRAB_CUDA_TRY(totals.alloc(sizeof(uint32_t) * C));
  const uint32_t nchunk4 = dim / 4;
  if (iterations > 0) {
    GRAB_CUDA_TRY(soffs.alloc(sizeof(uint32_t) * (C + 1)));
    GRAB_CUDA_TRY(smembers.alloc(sizeof(uint32_t) * m));
    gather_rows_kernel<<<static_cast<unsigned>((m * nchunk4 + 255) / 256), 256, 0, st>>>(
        d_dataset, n, dim, m, m, sample.as<float>());
    gather_rows_kernel<<<static_cast<unsigned>((static_cast<uint64_t>(C) * nchunk4 + 255) / 256), 256, 0, st>>>(
        d_dataset, n, dim, m, C, d_centroids);
    GRAB_CUDA_TRY(cudaGetLastError());
    // norms of the initial centroids: an update with empty groups keeps the rows and writes |c|^2
    GRAB_CUDA_TRY(cudaMemsetAsync(soffs.ptr, 0, sizeof(uint32_t) * (C + 1), st));
    centroid_update_kernel<<<C, 128, dim * sizeof(float), st>>>(sample.as<float>(), dim, soffs.as<uint32_t>(),
                                                                 smembers.as<uint32_t>(), GRAB_METRIC_L2, d_centroids,
                                                                 d_cnorm);
    for (uint32_t it = 0; it < iterations; ++it) {
      GRAB_CUDA_TRY(nearest(metric, sample.as<float>(), m, dim, d_centroids, d_cnorm, C, 1, assign.as<uint32_t>(), st));
      int rc = group_by_centroid(assign.as<uint32_t>(), m, C, counts.as<uint32_t>(), totals.as<uint32_t>(),
                                 soffs.as<uint32_t>(), smembers.as<uint32_t>(), st);
      if (rc != GRAB_OK) return rc;
      centroid_update_kernel<<<C, 128, dim * sizeof(float), st>>>(sample.as<float>(), dim, soffs.as<uint32_t>(),
                                                                   smembers.as<uint32_t>(), metric, d_centroids, d_cnorm);
      GRAB_CUDA_TRY(cudaGetLastError());
    }
    timer.mark("k-means on the sample");
  }
  GRAB_CUDA_TRY(nearest(metric, d_dataset, n, dim, d_centroids, d_cnorm, C, 1, assign.as<uint32_t>(), st));
  timer.mark("assignment");
  int rc = group_by_centroid(assign.as<uint32_t>(), n, C, counts.as<uint32_t>(), totals.as<uint32_t>(), d_offsets,
                             d_members, st);
  if (rc != GRAB_OK) return rc;
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));  // the scratch buffers are released on return
  timer.mark("member lists");
  return GRAB_OK;
}

bool route_tc_usable(const float*, uint64_t, uint32_t, const float*, uint32_t, uint32_t);
uint32_t route_tc_slices(uint64_t, uint32_t);
int route_tc_launch(int, const float*, uint64_t, uint32_t, const float*, const float*, uint32_t, uint32_t, uint32_t,
                    uint64_t*, int*, cudaStream_t);

int route_seeds_impl(const grab_router* r, const float* d_queries, uint64_t nq, uint64_t n, const grab_filter* f,
                     uint32_t probes, uint32_t S, uint64_t seed, uint32_t* d_seeds, void* d_ws, size_t ws_bytes,
                     cudaStream_t st) {
  GRAB_REQUIRE(r && r->d_centroids && r->d_centroid_norms && r->d_member_offsets && r->d_members,
               "route_seeds: incomplete router");
  GRAB_REQUIRE(d_queries && d_seeds, "route_seeds: null pointer");
  GRAB_REQUIRE(r->dim >= 4 && r->dim % 4 == 0, "route_seeds: dim %u must be a multiple of 4", r->dim);
  GRAB_REQUIRE(r->num_centroids >= 1, "route_seeds: router without centroids");
  GRAB_REQUIRE(n >= 1 && n < (1ull << 31), "route_seeds: n must be in [1, 2^31)");
  GRAB_REQUIRE(probes >= 1 && probes <= kMaxProbes, "route_seeds: probes %u outside [1,%u]", probes, kMaxProbes);
  GRAB_REQUIRE(S >= 1 && S <= 1024, "route_seeds: seeds_per_query %u outside [1,1024]", S);
  GRAB_REQUIRE(r->metric == GRAB_METRIC_L2 || r->metric == GRAB_METRIC_IP, "route_seeds: bad metric");
  if (nq == 0) return GRAB_OK;
  if (probes > r->num_centroids) probes = r->num_centroids;
  RouteArgs a{};
  a.p = probes; a.S = S; a.C = r->num_centroids; a.nq = nq; a.n = n; a.seed = seed;
  a.offsets = r->d_member_offsets; a.members = r->d_members; a.seeds = d_seeds;
  a.filter_kind = GRAB_FILTER_NONE;
  if (f) {
    a.filter_kind = f->kind;
    switch (f->kind) {
      case GRAB_FILTER_NONE: break;
      case GRAB_FILTER_PREFIX:
      case GRAB_FILTER_TS_RANGE:
        if (f->kind == GRAB_FILTER_TS_RANGE) GRAB_REQUIRE(f->d_ts, "route_seeds: ts filter without d_ts");
        GRAB_REQUIRE((f->d_lo == nullptr) == (f->d_hi == nullptr),
                     "route_seeds: d_lo and d_hi must both be given or both NULL");
        a.ts = f->d_ts; a.lo = f->d_lo; a.hi = f->d_hi; a.lo1 = f->lo; a.hi1 = f->hi; a.ts_sorted = f->ts_sorted;
        a.id_windows = f->d_id_windows;
        break;
      case GRAB_FILTER_LABELS:
        GRAB_REQUIRE(f->d_labels, "route_seeds: label filter without d_labels");
        a.labels = f->d_labels; a.masks = f->d_masks; a.mask1 = f->mask; a.label_offsets = f->d_label_offsets;
        break;
      default:
        set_last_error("route_seeds: unknown filter kind %d", f->kind);
        return GRAB_ERR_INVALID_ARGUMENT;
    }
  }
  const size_t need = grab_route_seeds_workspace_bytes(nq, probes);
  ScopedDeviceBuffer own;
  void* ws = d_ws;
  if (!ws) {
    GRAB_CUDA_TRY(own.alloc(need));
    ws = own.ptr;
  } else if (ws_bytes < need) {
    set_last_error("route_seeds: workspace %zu < %zu bytes", ws_bytes, need);
    return GRAB_ERR_WORKSPACE;
  }
  int* d_status = static_cast<int*>(ws);   // word 0 of the workspace: GRAB_OK, or GRAB_ERR_TIMEOUT from a stalled pipeline
  GRAB_CUDA_TRY(cudaMemsetAsync(d_status, 0, sizeof(int), st));
  uint64_t* d_keys = reinterpret_cast<uint64_t*>(static_cast<char*>(ws) + 256);
  const uint32_t T_tc = probes + 4 <= 16 ? probes + 4 : 16;
  a.queries = d_queries; a.cen = r->d_centroids; a.cnorm = r->d_centroid_norms; a.dim = r->dim; a.metric = r->metric;
  if (!(r->flags & GRAB_ROUTER_EXACT_SCAN) && probes + 4 <= 16 &&
      route_tc_usable(d_queries, nq, r->dim, r->d_centroids, r->num_centroids, T_tc)) {
    // tensor cores: tf32 scores, probes + 4 candidates per query, re-scored exactly by the seed kernel
    a.slices = route_tc_slices(nq, r->num_centroids);
    a.T = T_tc;
    a.rescore = 1;
    a.status = d_status;
    int rc = route_tc_launch(r->metric, d_queries, nq, r->dim, r->d_centroids, r->d_centroid_norms,
                             r->num_centroids, a.T, a.slices, d_keys, d_status, st);
    if (rc != GRAB_OK) return rc;
  } else {
    a.slices = route_slices(nq, r->num_centroids);
    a.T = probes;
    GRAB_CUDA_TRY(nearest(r->metric, d_queries, nq, r->dim, r->d_centroids, r->d_centroid_norms, r->num_centroids,
                          probes, nullptr, st, d_keys, a.slices));
  }
  a.keys = d_keys;
  route_seeds_kernel<<<static_cast<unsigned>((nq * 32 + 255) / 256), 256, 0, st>>>(a);
  GRAB_CUDA_TRY(cudaGetLastError());
  if (own.ptr) {
    // the call owns its workspace and has to wait for it anyway: report a stalled tensor-core pipeline
    // (all seeds of the batch were then written as "none") instead of returning degraded seeds silently
    int status = 0;
    GRAB_CUDA_TRY(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, st));
    GRAB_CUDA_TRY(cudaStreamSynchronize(st));
    if (status != GRAB_OK) {
      set_last_error("route_seeds: the tensor-core centroid ranking gave up on a bounded wait");
      return status == GRAB_ERR_TIMEOUT ? GRAB_ERR_TIMEOUT : GRAB_ERR_CUDA;
    }
  }
  return GRAB_OK;
}

int route_status_impl(const void* d_ws, cudaStream_t st) {
  GRAB_REQUIRE(d_ws, "route_status: null workspace");
  int status = 0;
  GRAB_CUDA_TRY(cudaMemcpyAsync(&status, d_ws, sizeof(int), cudaMemcpyDeviceToHost, st));
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  if (status != GRAB_OK) set_last_error("route_seeds: the tensor-core centroid ranking gave up on a bounded wait");
  return status == GRAB_OK ? GRAB_OK : (status == GRAB_ERR_TIMEOUT ? GRAB_ERR_TIMEOUT : GRAB_ERR_CUDA);
}

int nearest_centroids_impl(const grab_router* r, const float* d_rows, uint64_t m, uint32_t probes, uint32_t* d_out,
                           cudaStream_t st) {
  GRAB_REQUIRE(r && r->d_centroids && r->d_centroid_norms && d_rows && d_out, "nearest_centroids: null pointer");
  GRAB_REQUIRE(probes >= 1 && probes <= kMaxProbes, "nearest_centroids: probes %u outside [1,%u]", probes, kMaxProbes);
  GRAB_REQUIRE(r->dim >= 4 && r->dim % 4 == 0, "nearest_centroids: dim %u must be a multiple of 4", r->dim);
  GRAB_CUDA_TRY(nearest(r->metric, d_rows, m, r->dim, r->d_centroids, r->d_centroid_norms, r->num_centroids, probes,
                        d_out, st));
  return GRAB_OK;
}

}  // namespace grab

extern "C" size_t grab_route_seeds_workspace_bytes(uint64_t nq, uint32_t probes) {
  // a status word, then (score, centroid) keys of up to 8 centroid slices per query, probes + 4 each
  return 256 + ((sizeof(uint64_t) * nq * 8 * (probes + 4) + 255) / 256) * 256;
}
