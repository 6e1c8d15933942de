// Graph optimisation on the device: rank-based prune, reverse graph, interleaved merge,
// cross-bucket (remote) edges and their reverse injection, insert topology updates.
//
// The reference runs these as host-orchestrated pipelines with a device<->host round trip
// per stage (src/index/cagra.cu:286-650, cagra_opt.cu:209-600, insert.cu:225-765).  Here
// every stage is one or a few launches over device-resident graphs; integer results are
// identical to the CPU oracle.  Where the reference's outcome depends on an atomics race
// (slot claim order), the order is fixed: lists are grouped per destination in a CSR
// scratch and the first `cap` entries by an explicit key are kept.
#include "common.cuh"

namespace grab {

// =======================================================================================
// Exclusive prefix sum of uint32 counts (three small kernels; n up to 2^31).
// =======================================================================================
constexpr int kScanBlock = 1024;

__global__ void scan_block_sums_kernel(const uint32_t* __restrict__ in, uint64_t n,
                                       uint32_t* __restrict__ block_sums) {
  __shared__ uint32_t warp_sums[32];
  const uint64_t i = blockIdx.x * static_cast<uint64_t>(kScanBlock) + threadIdx.x;
  uint32_t v = i < n ? in[i] : 0;
  v = __reduce_add_sync(0xFFFFFFFFu, v);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    uint32_t s = warp_sums[threadIdx.x];
    s = __reduce_add_sync(0xFFFFFFFFu, s);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = s;
  }
}

__global__ void scan_block_offsets_kernel(uint32_t* __restrict__ block_sums, uint32_t nblocks) {
  // single CTA, sequential over chunks of 1024 with a running carry
  __shared__ uint32_t buf[kScanBlock];
  __shared__ uint32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (uint32_t base = 0; base < nblocks; base += kScanBlock) {
    const uint32_t i = base + threadIdx.x;
    const uint32_t v = i < nblocks ? block_sums[i] : 0;
    buf[threadIdx.x] = v;
    __syncthreads();
    for (uint32_t off = 1; off < kScanBlock; off <<= 1) {
      uint32_t t = threadIdx.x >= off ? buf[threadIdx.x - off] : 0;
      __syncthreads();
      buf[threadIdx.x] += t;
      __syncthreads();
    }
    const uint32_t incl = buf[threadIdx.x];
    const uint32_t c = carry;
    if (i < nblocks) block_sums[i] = c + incl - v;
    __syncthreads();
    if (threadIdx.x == kScanBlock - 1) carry = c + incl;
    __syncthreads();
  }
}

__global__ void scan_apply_kernel(const uint32_t* __restrict__ in, uint64_t n,
                                  const uint32_t* __restrict__ block_offsets,
                                  uint32_t* __restrict__ out) {
  __shared__ uint32_t buf[kScanBlock];
  const uint64_t i = blockIdx.x * static_cast<uint64_t>(kScanBlock) + threadIdx.x;
  const uint32_t v = i < n ? in[i] : 0;
  buf[threadIdx.x] = v;
  __syncthreads();
  for (uint32_t off = 1; off < kScanBlock; off <<= 1) {
    uint32_t t = threadIdx.x >= off ? buf[threadIdx.x - off] : 0;
    __syncthreads();
    buf[threadIdx.x] += t;
    __syncthreads();
  }
  if (i < n) out[i] = block_offsets[blockIdx.x] + buf[threadIdx.x] - v;
}

static cudaError_t exclusive_scan_u32(const uint32_t* in, uint64_t n, uint32_t* out,
                                      uint32_t* block_tmp, cudaStream_t st) {
  const uint32_t nblocks = static_cast<uint32_t>((n + kScanBlock - 1) / kScanBlock);
  scan_block_sums_kernel<<<nblocks, kScanBlock, 0, st>>>(in, n, block_tmp);
  scan_block_offsets_kernel<<<1, kScanBlock, 0, st>>>(block_tmp, nblocks);
  scan_apply_kernel<<<nblocks, kScanBlock, 0, st>>>(in, n, block_tmp, out);
  return cudaGetLastError();
}

// =======================================================================================
// Grouped lists: for every destination the first `cap` incoming sources by an explicit key.
// An "edge source" enumerates (dest, key, value) triples; three uses:
//   kind 0  reverse graph of columns [c0,c1): key = (column, src)      cagra.cu:418-548
//   kind 1  reverse of remote columns:        key = (src, column)      cagra_opt.cu:457-481
//   kind 2  insert mailboxes, new rows only:  key = (src, column)      insert.cu:579-640
// =======================================================================================
struct EdgeSource {
  const uint32_t* graph;
  uint32_t deg;
  uint32_t c0, c1;     // column window
  uint64_t row0, row1; // source rows
  uint64_t n_dest;     // valid destinations are < n_dest
  int col_major_key;   // 1: key (column, src); 0: key (src, column)
  const uint64_t* bucket;   // optional: drop edges whose destination bucket == skip_bucket
  uint64_t skip_bucket;
  int use_skip;
};

__device__ __forceinline__ bool edge_at(const EdgeSource& e, uint64_t idx, uint32_t* dest,
                                        uint64_t* key, uint32_t* src) {
  const uint32_t ncol = e.c1 - e.c0;
  const uint64_t r = e.row0 + idx / ncol;
  const uint32_t c = e.c0 + static_cast<uint32_t>(idx % ncol);
  const uint32_t d = e.graph[r * e.deg + c];
  if (d >= e.n_dest) return false;
  if (e.use_skip && e.bucket[d] == e.skip_bucket) return false;
  *dest = d;
  *src = static_cast<uint32_t>(r);
  *key = e.col_major_key ? ((static_cast<uint64_t>(c) << 32) | r) : ((r << 32) | c);
  return true;
}

__global__ void group_count_kernel(EdgeSource e, uint64_t total, uint32_t* __restrict__ counts) {
  const uint64_t idx = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  uint32_t d, s; uint64_t key;
  if (edge_at(e, idx, &d, &key, &s)) atomicAdd(&counts[d], 1u);
}

__global__ void group_fill_kernel(EdgeSource e, uint64_t total, const uint32_t* __restrict__ offsets,
                                  uint32_t* __restrict__ cursor, uint64_t* __restrict__ csr) {
  const uint64_t idx = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  uint32_t d, s; uint64_t key;
  if (edge_at(e, idx, &d, &key, &s)) {
    const uint32_t pos = offsets[d] + atomicAdd(&cursor[d], 1u);
    csr[pos] = key;
  }
}

// One warp per destination: the `cap` smallest keys of its segment, ascending, mapped back
// to source ids.  Segments up to 256 keys are sorted in shared memory; longer ones (hubs)
// take `cap` rounds of "smallest key above the previous one".
constexpr int kSelWarps = 4;
constexpr int kSelSort = 256;

__global__ void __launch_bounds__(kSelWarps * 32)
group_select_kernel(const uint64_t* __restrict__ csr, const uint32_t* __restrict__ offsets,
                    const uint32_t* __restrict__ counts, uint64_t n_dest, uint32_t cap,
                    int col_major_key, uint32_t* __restrict__ out /* [n_dest, cap] */) {
  __shared__ uint64_t sbuf[kSelWarps][kSelSort];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t d = blockIdx.x * static_cast<uint64_t>(kSelWarps) + warp;
  if (d >= n_dest) return;
  const uint32_t len = counts[d];
  const uint64_t* seg = csr + offsets[d];
  uint32_t* dst = out + d * cap;
  auto src_of = [&](uint64_t key) -> uint32_t {
    return col_major_key ? static_cast<uint32_t>(key & 0xFFFFFFFFull) : static_cast<uint32_t>(key >> 32);
  };
  if (len <= kSelSort) {
    uint64_t* keys = sbuf[warp];
    uint32_t padded = 32;
    while (padded < len) padded <<= 1;
    for (uint32_t i = lane; i < padded; i += 32) keys[i] = i < len ? seg[i] : kMaxKey;
    __syncwarp();
    for (uint32_t size = 2; size <= padded; size <<= 1)
      for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
        for (uint32_t t = lane; t < (padded >> 1); t += 32) {
          const uint32_t lo = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
          const uint32_t hi = lo | stride;
          const bool up = (lo & size) == 0;
          const uint64_t a = keys[lo], b = keys[hi];
          if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
        }
        __syncwarp();
      }
    for (uint32_t i = lane; i < cap; i += 32) dst[i] = i < len ? src_of(keys[i]) : kInvalid;
  } else {
    uint64_t last = 0;
    bool first = true;
    for (uint32_t r = 0; r < cap; ++r) {
      uint64_t best = kMaxKey;
      for (uint32_t i = lane; i < len; i += 32) {
        const uint64_t key = seg[i];
        if ((first || key > last) && key < best) best = key;
      }
      for (int off = 16; off > 0; off >>= 1) {
        const uint64_t o = __shfl_xor_sync(0xFFFFFFFFu, best, off);
        best = o < best ? o : best;
      }
      if (lane == 0) dst[r] = best == kMaxKey ? kInvalid : src_of(best);
      if (best == kMaxKey) {
        for (uint32_t i = r + 1 + lane; i < cap; i += 32) dst[i] = kInvalid;
        break;
      }
      last = best;
      first = false;
    }
  }
}

// Scratch for grouped lists.
struct GroupScratch {
  ScopedDeviceBuffer counts, offsets, cursor, block_tmp, csr;
  cudaError_t alloc(uint64_t n_dest, uint64_t total_edges) {
    cudaError_t e;
    if ((e = counts.alloc(sizeof(uint32_t) * n_dest)) != cudaSuccess) return e;
    if ((e = offsets.alloc(sizeof(uint32_t) * n_dest)) != cudaSuccess) return e;
    if ((e = cursor.alloc(sizeof(uint32_t) * n_dest)) != cudaSuccess) return e;
    if ((e = block_tmp.alloc(sizeof(uint32_t) * ((n_dest + kScanBlock - 1) / kScanBlock + 1))) != cudaSuccess) return e;
    return csr.alloc(sizeof(uint64_t) * total_edges);
  }
};

// counts_out receives the true number of incoming edges per destination.
static int grouped_lists(const EdgeSource& e, uint32_t cap, uint32_t* d_out, uint32_t* d_counts_out,
                         cudaStream_t st) {
  const uint64_t total = (e.row1 - e.row0) * (e.c1 - e.c0);
  GRAB_REQUIRE(total < (1ull << 32), "grouped_lists: %llu edges exceed 2^32", (unsigned long long)total);
  GroupScratch s;
  GRAB_CUDA_TRY(s.alloc(e.n_dest, total ? total : 1));
  uint32_t* counts = d_counts_out ? d_counts_out : s.counts.as<uint32_t>();
  GRAB_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(uint32_t) * e.n_dest, st));
  GRAB_CUDA_TRY(cudaMemsetAsync(s.cursor.ptr, 0, sizeof(uint32_t) * e.n_dest, st));
  if (total) {
    group_count_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(e, total, counts);
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  GRAB_CUDA_TRY(exclusive_scan_u32(counts, e.n_dest, s.offsets.as<uint32_t>(), s.block_tmp.as<uint32_t>(), st));
  if (total) {
    group_fill_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        e, total, s.offsets.as<uint32_t>(), s.cursor.as<uint32_t>(), s.csr.as<uint64_t>());
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  group_select_kernel<<<(unsigned)((e.n_dest + kSelWarps - 1) / kSelWarps), kSelWarps * 32, 0, st>>>(
      s.csr.as<uint64_t>(), s.offsets.as<uint32_t>(), counts, e.n_dest, cap, e.col_major_key, d_out);
  GRAB_CUDA_TRY(cudaGetLastError());
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));  // scratch is released on return
  return GRAB_OK;
}

// =======================================================================================
// Prune: detour counts (cagra.cu:219-276) + stable selection of the out_deg smallest
// (count, rank) (cagra.cu:367-392), fused; one warp per node.  The reference's inner
// O(K) scan over A's row is replaced by a shared-memory table id -> smallest rank.
// =======================================================================================
constexpr int kPruneWarps = 4;

__global__ void __launch_bounds__(kPruneWarps * 32)
prune_kernel(const uint32_t* __restrict__ knn, uint32_t* __restrict__ out, uint64_t n,
             uint32_t in_deg, uint32_t out_deg, uint32_t tsize, uint8_t* __restrict__ detour_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t per_warp = 2 * in_deg + 2 * tsize;  // uint32 words
  uint32_t* base = reinterpret_cast<uint32_t*>(smem_raw) + warp * per_warp;
  uint32_t* rowA = base;            // [in_deg]
  uint32_t* cnt = rowA + in_deg;    // [in_deg]
  uint32_t* tkey = cnt + in_deg;    // [tsize]
  uint32_t* tval = tkey + tsize;    // [tsize]
  const uint64_t a = blockIdx.x * static_cast<uint64_t>(kPruneWarps) + warp;
  if (a >= n) return;
  const uint32_t tmask = tsize - 1;

  for (uint32_t i = lane; i < in_deg; i += 32) {
    rowA[i] = knn[a * in_deg + i];
    cnt[i] = 0;
  }
  for (uint32_t i = lane; i < tsize; i += 32) {
    tkey[i] = kInvalid;  // slot empty (the id 0xFFFFFFFF itself is tracked by first_pad below)
    tval[i] = kInvalid;
  }
  __syncwarp();
  // table: id -> smallest rank holding it; note duplicates
  uint32_t first_pad = kInvalid;
  bool dup = false;
  for (uint32_t r = lane; r < in_deg; r += 32) {
    const uint32_t id = rowA[r];
    if (id == kInvalid) {
      first_pad = min(first_pad, r);
      continue;
    }
    uint32_t h = (id * 2654435761u) & tmask;
    for (;;) {
      const uint32_t old = atomicCAS(&tkey[h], kInvalid, id);
      if (old == kInvalid || old == id) {
        if (old == id) dup = true;
        atomicMin(&tval[h], r);
        break;
      }
      h = (h + 1) & tmask;
    }
  }
  uint32_t pads = __popc(__ballot_sync(0xFFFFFFFFu, first_pad != kInvalid));
  first_pad = __reduce_min_sync(0xFFFFFFFFu, first_pad);
  // more than one pad entry counts as a duplicate id (pads match pads in the reference)
  uint32_t npad = 0;
  for (uint32_t r = lane; r < in_deg; r += 32) npad += rowA[r] == kInvalid;
  npad = __reduce_add_sync(0xFFFFFFFFu, npad);
  (void)pads;
  const bool any_dup = __any_sync(0xFFFFFFFFu, dup) || npad > 1;
  __syncwarp();

  auto rank_of = [&](uint32_t id) -> uint32_t {
    if (id == kInvalid) return first_pad;
    uint32_t h = (id * 2654435761u) & tmask;
    for (;;) {
      const uint32_t kx = tkey[h];
      if (kx == id) return tval[h];
      if (kx == kInvalid) return kInvalid;
      h = (h + 1) & tmask;
    }
  };

  for (uint32_t kAD = 0; kAD + 1 < in_deg; ++kAD) {
    const uint32_t D = rowA[kAD];
    if (D == kInvalid || D >= n) continue;
    const uint32_t* rowD = knn + static_cast<size_t>(D) * in_deg;
    for (uint32_t kDB = lane; kDB < in_deg; kDB += 32) {
      const uint32_t c = __ldg(rowD + kDB);
      uint32_t r = rank_of(c);
      if (r == kInvalid) continue;
      if (r <= kAD) {
        if (!any_dup) continue;
        // rare: the id occurs again further right; take the first rank > kAD holding it
        r = kInvalid;
        for (uint32_t x = kAD + 1; x < in_deg; ++x)
          if (rowA[x] == c) { r = x; break; }
        if (r == kInvalid) continue;
      }
      atomicAdd(&cnt[r], 1u);
    }
  }
  __syncwarp();
  for (uint32_t r = lane; r < in_deg; r += 32) {
    const uint32_t c = cnt[r] > 255 ? 255 : cnt[r];
    cnt[r] = c;
    if (detour_out) detour_out[a * in_deg + r] = static_cast<uint8_t>(c);
  }
  __syncwarp();
  // stable selection: position = number of (count, rank) pairs strictly smaller
  for (uint32_t r = lane; r < in_deg; r += 32) {
    const uint32_t c = cnt[r];
    uint32_t pos = 0;
    for (uint32_t x = 0; x < in_deg; ++x) {
      const uint32_t cx = cnt[x];
      pos += (cx < c) || (cx == c && x < r);
    }
    if (pos < out_deg) out[a * out_deg + pos] = rowA[r];
  }
}

int prune_device_impl(const uint32_t* d_knn, uint32_t* d_out, uint64_t n, uint32_t in_deg,
                      uint32_t out_deg, uint8_t* d_detour, cudaStream_t st) {
  GRAB_REQUIRE(d_knn && d_out, "optimize_prune: null pointer");
  // the reference throws above 512 (cagra.cu:295-297)
  GRAB_REQUIRE(in_deg >= 1 && in_deg <= 512, "optimize_prune: input degree %u outside [1,512]", in_deg);
  GRAB_REQUIRE(out_deg >= 1 && out_deg <= in_deg, "optimize_prune: output degree %u outside [1,%u]",
               out_deg, in_deg);
  if (n == 0) return GRAB_OK;
  const uint32_t tsize = next_pow2(2 * in_deg);
  const size_t smem = sizeof(uint32_t) * kPruneWarps * (2 * in_deg + 2 * tsize);
  GRAB_CUDA_TRY(cudaFuncSetAttribute(prune_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  prune_kernel<<<(unsigned)((n + kPruneWarps - 1) / kPruneWarps), kPruneWarps * 32, smem, st>>>(
      d_knn, d_out, n, in_deg, out_deg, tsize, d_detour);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

int reverse_device_impl(const uint32_t* d_graph, uint32_t* d_rev, uint32_t* d_rev_counts, uint64_t n,
                        uint32_t deg, cudaStream_t st) {
  GRAB_REQUIRE(d_graph && d_rev && d_rev_counts, "create_reverse_graph: null pointer");
  GRAB_REQUIRE(deg >= 1 && deg <= 512, "create_reverse_graph: degree %u outside [1,512]", deg);
  if (n == 0) return GRAB_OK;
  EdgeSource e{};
  e.graph = d_graph; e.deg = deg; e.c0 = 0; e.c1 = deg; e.row0 = 0; e.row1 = n; e.n_dest = n;
  e.col_major_key = 1;
  return grouped_lists(e, deg, d_rev, d_rev_counts, st);
}

// =======================================================================================
// Interleaved merge (cagra.cu:574-650), one warp per node: the serial take-one-from-each
// walk is kept, the duplicate test runs across the lanes.
// =======================================================================================
constexpr int kMergeWarps = 4;

__global__ void __launch_bounds__(kMergeWarps * 32)
merge_graphs_kernel(uint32_t* __restrict__ graph, const uint32_t* __restrict__ rev,
                    const uint32_t* __restrict__ rev_counts, uint64_t n, uint32_t deg) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* so = reinterpret_cast<uint32_t*>(smem_raw) + warp * 3 * deg;
  uint32_t* sr = so + deg;
  uint32_t* nn = sr + deg;
  const uint64_t j = blockIdx.x * static_cast<uint64_t>(kMergeWarps) + warp;
  if (j >= n) return;
  for (uint32_t i = lane; i < deg; i += 32) {
    so[i] = graph[j * deg + i];
    sr[i] = rev[j * deg + i];
  }
  __syncwarp();
  uint32_t rc = rev_counts[j];
  if (rc > deg) rc = deg;
  uint32_t sz = 0, co = 0, cr = 0;
  auto is_dup = [&](uint32_t c) -> bool {
    bool d = false;
    for (uint32_t i = lane; i < sz; i += 32) d |= (nn[i] == c);
    return __any_sync(0xFFFFFFFFu, d);
  };
  while (sz < deg) {
    bool added = false;
    while (co < deg) {
      const uint32_t c = so[co++];
      if (c == static_cast<uint32_t>(j)) continue;
      if (is_dup(c)) continue;
      if (lane == 0) nn[sz] = c;
      ++sz;
      __syncwarp();
      added = true;
      break;
    }
    if (sz >= deg) break;
    while (cr < rc) {
      const uint32_t c = sr[cr++];
      if (c >= n) continue;
      if (c == static_cast<uint32_t>(j)) continue;
      if (is_dup(c)) continue;
      if (lane == 0) nn[sz] = c;
      ++sz;
      __syncwarp();
      added = true;
      break;
    }
    if (!added) break;
  }
  for (uint32_t i = lane; i < sz; i += 32) graph[j * deg + i] = nn[i];
}

int merge_device_impl(uint32_t* d_graph, const uint32_t* d_rev, const uint32_t* d_rev_counts,
                      uint64_t n, uint32_t deg, cudaStream_t st) {
  GRAB_REQUIRE(d_graph && d_rev && d_rev_counts, "merge_graphs: null pointer");
  GRAB_REQUIRE(deg >= 1 && deg <= 512, "merge_graphs: degree %u outside [1,512]", deg);
  if (n == 0) return GRAB_OK;
  const size_t smem = sizeof(uint32_t) * kMergeWarps * 3 * deg;
  merge_graphs_kernel<<<(unsigned)((n + kMergeWarps - 1) / kMergeWarps), kMergeWarps * 32, smem, st>>>(
      d_graph, d_rev, d_rev_counts, n, deg);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

// =======================================================================================
// Remote edges (cagra_opt.cu:209-303): one thread per node walks its candidate list three
// times (nearby third, far part, back-fill).  `bucket` is the reference's d_ts.
// =======================================================================================
__global__ void remote_edges_kernel(uint32_t* __restrict__ graph, const uint64_t* __restrict__ bucket,
                                    uint32_t* __restrict__ cand, uint64_t n, uint32_t total_deg,
                                    uint32_t local_deg, uint32_t gk) {
  const uint64_t t = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (t >= n) return;
  uint32_t* row = graph + t * total_deg;
  uint32_t* mc = cand + t * gk;
  const uint64_t my = bucket[t];
  const uint64_t total_buckets = bucket[n - 1] + 1;
  const uint64_t span = total_buckets / 5 > 1 ? total_buckets / 5 : 1;
  const uint64_t mn = my >= span ? my - span : 0;
  const uint64_t mx = my + span >= total_buckets ? total_buckets - 1 : my + span;
  int nearby = 0;
  const int nearby_max = static_cast<int>(total_deg - local_deg) / 3;
  for (uint32_t k = 0; k < gk && nearby_max > 0; ++k) {
    const uint32_t c = mc[k];
    if (c == static_cast<uint32_t>(t) || c == kInvalid) continue;
    const uint64_t b = bucket[c];
    if (b == my || b < mn || b > mx) continue;
    row[local_deg + nearby++] = c;
    mc[k] = kInvalid;
    if (nearby >= nearby_max) break;
  }
  int remote = 0;
  const int remote_max = static_cast<int>(total_deg - local_deg) - nearby;
  for (uint32_t k = 0; k < gk && remote_max > 0; ++k) {
    const uint32_t c = mc[k];
    if (c == static_cast<uint32_t>(t) || c == kInvalid) continue;
    const uint64_t b = bucket[c];
    if (b == my || (b >= mn && b <= mx)) continue;
    row[local_deg + nearby + remote++] = c;
    mc[k] = kInvalid;
    if (remote >= remote_max) break;
  }
  for (uint32_t k = 0; k < gk && remote < remote_max; ++k) {
    const uint32_t c = mc[k];
    if (c == static_cast<uint32_t>(t) || c == kInvalid) continue;
    if (bucket[c] == my) continue;
    row[local_deg + nearby + remote++] = c;
  }
}

__device__ __forceinline__ uint32_t wang_hash(uint32_t s) {  // cagra_opt.cu:33-40
  s = (s ^ 61u) ^ (s >> 16);
  s *= 9u;
  s = s ^ (s >> 4);
  s *= 0x27d4eb2du;
  s = s ^ (s >> 15);
  return s;
}

// cagra_opt.cu:487-600: inject reverse remote edges into the weak half of the remote part.
__global__ void inject_reverse_kernel(uint32_t* __restrict__ graph, const uint32_t* __restrict__ rev,
                                      const uint32_t* __restrict__ rev_counts, uint64_t n,
                                      uint32_t total_deg, uint32_t local_deg, uint32_t max_rev) {
  const uint64_t t = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (t >= n) return;
  const uint32_t num_remote = total_deg - local_deg;
  const int num_strong = static_cast<int>(num_remote) / 2;
  const int num_weak = static_cast<int>(num_remote) - num_strong;
  uint32_t* row = graph + t * total_deg;
  uint32_t cnt = rev_counts[t];
  if (cnt == 0) return;
  if (cnt > max_rev) cnt = max_rev;
  uint32_t rng = wang_hash(static_cast<uint32_t>(t));
  for (uint32_t i = 0; i < cnt; ++i) {
    const uint32_t c = rev[t * max_rev + i];
    bool exists = false;
    for (uint32_t r = 0; r < total_deg; ++r) exists |= (row[r] == c);
    if (exists) continue;
    bool injected = false;
    for (int w = num_strong; w < static_cast<int>(num_remote); ++w)
      if (row[local_deg + w] == kInvalid) {
        row[local_deg + w] = c;
        injected = true;
        break;
      }
    if (!injected && num_weak > 0) {
      rng = wang_hash(rng);
      row[local_deg + num_strong + (rng % static_cast<uint32_t>(num_weak))] = c;
    }
  }
}

int remote_edges_impl(uint32_t* d_graph, const uint64_t* d_bucket, uint32_t* d_cand, uint64_t n,
                      uint32_t total_deg, uint32_t local_deg, uint32_t gk, cudaStream_t st) {
  GRAB_REQUIRE(d_graph && d_bucket && d_cand, "remote_edges: null pointer");
  GRAB_REQUIRE(local_deg < total_deg && total_deg - local_deg >= 3 && total_deg - local_deg <= 64,
               "remote_edges: remote width %d outside [3,64]", (int)total_deg - (int)local_deg);
  if (n == 0) return GRAB_OK;
  remote_edges_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(d_graph, d_bucket, d_cand, n,
                                                                 total_deg, local_deg, gk);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

int inject_reverse_impl(uint32_t* d_graph, uint64_t n, uint32_t total_deg, uint32_t local_deg,
                        uint32_t max_rev, cudaStream_t st) {
  GRAB_REQUIRE(d_graph, "inject_reverse_remote: null pointer");
  GRAB_REQUIRE(local_deg < total_deg && max_rev >= 1 && max_rev <= 256, "inject_reverse_remote: bad sizes");
  if (n == 0) return GRAB_OK;
  ScopedDeviceBuffer rev, cnt;
  GRAB_CUDA_TRY(rev.alloc(sizeof(uint32_t) * n * max_rev));
  GRAB_CUDA_TRY(cnt.alloc(sizeof(uint32_t) * n));
  EdgeSource e{};
  e.graph = d_graph; e.deg = total_deg; e.c0 = local_deg; e.c1 = total_deg; e.row0 = 0; e.row1 = n;
  e.n_dest = n; e.col_major_key = 0;
  int rc = grouped_lists(e, max_rev, rev.as<uint32_t>(), cnt.as<uint32_t>(), st);
  if (rc != GRAB_OK) return rc;
  inject_reverse_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
      d_graph, rev.as<uint32_t>(), cnt.as<uint32_t>(), n, total_deg, local_deg, max_rev);
  GRAB_CUDA_TRY(cudaGetLastError());
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  return GRAB_OK;
}

// =======================================================================================
// Insert, v1 (insert.cu:225-440).  Requests are grouped per target and applied in
// ascending request index, the order the reference's stable radix sort leaves them in.
// =======================================================================================
__global__ void v1_fill_kernel(uint32_t* __restrict__ graph, const int64_t* __restrict__ found,
                               uint64_t num_existing, uint64_t num_new, uint32_t deg, uint32_t search_k) {
  const uint64_t idx = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (idx >= num_new * deg) return;
  const uint64_t i = idx / deg;
  const uint32_t k = static_cast<uint32_t>(idx % deg);
  uint32_t v = kInvalid;
  if (k < search_k) {
    const int64_t id = found[i * search_k + k];
    if (id >= 0 && id < static_cast<int64_t>(num_existing)) v = static_cast<uint32_t>(id);
  }
  graph[(num_existing + i) * deg + k] = v;
}

__global__ void v1_count_kernel(const int64_t* __restrict__ found, uint64_t total, uint64_t num_existing,
                                uint32_t* __restrict__ counts) {
  const uint64_t t = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (t >= total) return;
  const int64_t id = found[t];
  if (id >= 0 && id < static_cast<int64_t>(num_existing)) atomicAdd(&counts[id], 1u);
}

__global__ void v1_fill_req_kernel(const int64_t* __restrict__ found, uint64_t total, uint64_t num_existing,
                                   const uint32_t* __restrict__ offsets, uint32_t* __restrict__ cursor,
                                   uint32_t* __restrict__ req) {
  const uint64_t t = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (t >= total) return;
  const int64_t id = found[t];
  if (id >= 0 && id < static_cast<int64_t>(num_existing))
    req[offsets[id] + atomicAdd(&cursor[id], 1u)] = static_cast<uint32_t>(t);
}

// One thread per old node with mail: requests in ascending tid; `first_pos` = position of
// the segment leader in the reference's globally sorted request array = exclusive prefix of
// counts over targets (invalid requests sort last), which is exactly offsets[target].
__global__ void v1_apply_kernel(uint32_t* __restrict__ graph, const uint32_t* __restrict__ counts,
                                const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ req,
                                uint64_t num_existing, uint32_t deg, uint32_t search_k) {
  const uint64_t target = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (target >= num_existing) return;
  const uint32_t len = counts[target];
  if (len == 0) return;
  const uint32_t* seg = req + offsets[target];
  uint32_t* nb = graph + target * deg;
  const uint32_t num_prot = deg / 2, num_unprot = deg - num_prot;
  uint64_t rng = static_cast<uint32_t>(target) * 0x9e3779b97f4a7c15ull + offsets[target];
  uint32_t last = 0;
  for (uint32_t r = 0; r < len; ++r) {
    uint32_t best = kInvalid;
    for (uint32_t i = 0; i < len; ++i) {
      const uint32_t tid = seg[i];
      if ((r == 0 || tid > last) && tid < best) best = tid;
    }
    last = best;
    const uint32_t src = static_cast<uint32_t>(num_existing + best / search_k);
    bool exists = false;
    for (uint32_t c = 0; c < deg; ++c) exists |= (nb[c] == src);
    if (exists) continue;
    rng = rng * 6364136223846793005ull + 1;
    const uint32_t r1 = static_cast<uint32_t>(rng >> 32);
    const bool prot = (r1 % 10 == 0);
    rng = rng * 6364136223846793005ull + 1;
    const uint32_t r2 = static_cast<uint32_t>(rng >> 32);
    nb[prot ? r2 % num_prot : num_prot + (r2 % num_unprot)] = src;
  }
}

int update_topology_v1_impl(uint32_t* d_graph, const int64_t* d_found, uint64_t num_existing,
                            uint64_t num_new, uint32_t deg, uint32_t search_k, cudaStream_t st) {
  GRAB_REQUIRE(d_graph && d_found, "update_topology_v1: null pointer");
  GRAB_REQUIRE(deg >= 2 && deg <= 512 && search_k >= 1, "update_topology_v1: bad degree / search_k");
  if (num_new == 0) return GRAB_OK;
  const uint64_t total = num_new * search_k;
  GRAB_REQUIRE(total < (1ull << 32), "update_topology_v1: too many requests");
  v1_fill_kernel<<<(unsigned)((num_new * deg + 255) / 256), 256, 0, st>>>(d_graph, d_found, num_existing,
                                                                        num_new, deg, search_k);
  GRAB_CUDA_TRY(cudaGetLastError());
  if (num_existing == 0) return GRAB_OK;
  GroupScratch s;
  GRAB_CUDA_TRY(s.alloc(num_existing, 1));
  ScopedDeviceBuffer req;
  GRAB_CUDA_TRY(req.alloc(sizeof(uint32_t) * total));
  GRAB_CUDA_TRY(cudaMemsetAsync(s.counts.ptr, 0, sizeof(uint32_t) * num_existing, st));
  GRAB_CUDA_TRY(cudaMemsetAsync(s.cursor.ptr, 0, sizeof(uint32_t) * num_existing, st));
  v1_count_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d_found, total, num_existing,
                                                                  s.counts.as<uint32_t>());
  GRAB_CUDA_TRY(exclusive_scan_u32(s.counts.as<uint32_t>(), num_existing, s.offsets.as<uint32_t>(),
                                   s.block_tmp.as<uint32_t>(), st));
  v1_fill_req_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      d_found, total, num_existing, s.offsets.as<uint32_t>(), s.cursor.as<uint32_t>(), req.as<uint32_t>());
  v1_apply_kernel<<<(unsigned)((num_existing + 255) / 256), 256, 0, st>>>(
      d_graph, s.counts.as<uint32_t>(), s.offsets.as<uint32_t>(), req.as<uint32_t>(), num_existing, deg,
      search_k);
  GRAB_CUDA_TRY(cudaGetLastError());
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  return GRAB_OK;
}

// =======================================================================================
// Insert, time-partitioned (insert.cu:448-765).
// =======================================================================================
__global__ void opt_fill_kernel(uint32_t* __restrict__ graph, const uint64_t* __restrict__ bucket,
                                int64_t* __restrict__ local_knn, int64_t* __restrict__ global_knn,
                                uint64_t num_existing, uint64_t num_new, uint32_t total_deg,
                                uint32_t local_deg, uint32_t k_local, uint32_t k_global) {
  const uint64_t t = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (t >= num_new) return;
  const uint64_t me = num_existing + t;
  const uint64_t my = bucket[me];
  uint32_t* row = graph + me * total_deg;
  int64_t* lc = local_knn + t * k_local;
  uint32_t fl = 0;
  for (uint32_t k = 0; k < k_local && fl < local_deg; ++k) {
    const int64_t c64 = lc[k];
    const uint32_t c = static_cast<uint32_t>(c64);
    if (c64 < 0 || c == me || c >= 0x7fffffffu) continue;
    if (bucket[c] != my) continue;
    row[fl++] = c;
    lc[k] = -1;
  }
  int fr = 0;
  const int max_remote = static_cast<int>(total_deg - local_deg);
  int64_t* gc = global_knn + t * k_global;
  for (uint32_t k = 0; k < k_global && fr < max_remote; ++k) {
    const int64_t c64 = gc[k];
    const uint32_t c = static_cast<uint32_t>(c64);
    if (c64 < 0 || c == me) continue;
    bool ex = false;
    for (uint32_t i = 0; i < local_deg; ++i) ex |= (row[i] == c);
    if (ex) continue;
    if (bucket[c] != my) {
      row[local_deg + fr++] = c;
      gc[k] = -1;
    }
  }
  for (uint32_t i = 0; i < k_global && fr < max_remote; ++i) {
    const int64_t c64 = gc[i];
    const uint32_t c = static_cast<uint32_t>(c64);
    if (c64 < 0 || c == me) continue;
    row[local_deg + fr++] = c;
    gc[i] = -1;
  }
}

// ---------------------------------------------------------------------------------------
// Sparse mailboxes for the batched insert: only the old nodes that actually receive mail are
// visited (the reference clears and walks O(N) mailboxes for every batch of 32,
// insert.cu:1462-1560).  Per pass (local columns, then remote columns):
//   count   every edge of the new rows bumps counts[dest]; the first toucher appends dest to a list
//   offsets every touched dest claims a segment of the request array
//   fill    every edge writes its key (src, column) into its dest's segment
//   apply   one warp per touched dest sorts its segment, takes the first `cap` sources in
//           ascending (src, column) order and rewrites slots exactly as insert.cu:653-765 does
// counts / cursor live in pooled scratch that is all-zero between batches.
// ---------------------------------------------------------------------------------------
struct MailMeta {
  uint32_t n_touched;
  uint32_t csr_cursor;
};

__global__ void mail_count_kernel(EdgeSource e, uint64_t total, uint32_t* __restrict__ counts,
                                  uint32_t* __restrict__ touched, MailMeta* __restrict__ meta) {
  const uint64_t idx = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  uint32_t d, s; uint64_t key;
  if (edge_at(e, idx, &d, &key, &s) && atomicAdd(&counts[d], 1u) == 0) touched[atomicAdd(&meta->n_touched, 1u)] = d;
}

__global__ void mail_offsets_kernel(const uint32_t* __restrict__ touched, MailMeta* __restrict__ meta,
                                    const uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= meta->n_touched) return;
  const uint32_t d = touched[i];
  offsets[d] = atomicAdd(&meta->csr_cursor, counts[d]);
}

template <int REMOTE>
__global__ void __launch_bounds__(kSelWarps * 32)
mail_apply_kernel(uint32_t* __restrict__ graph, const uint64_t* __restrict__ bucket,
                  const uint32_t* __restrict__ touched, const MailMeta* __restrict__ meta,
                  uint32_t* __restrict__ counts, const uint32_t* __restrict__ counts_local,
                  const uint32_t* __restrict__ offsets, uint32_t* __restrict__ cursor,
                  const uint64_t* __restrict__ csr, uint32_t cap, uint32_t lmax, uint32_t total_deg,
                  uint32_t local_deg) {
  __shared__ uint64_t sbuf[kSelWarps][kSelSort];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t i = blockIdx.x * kSelWarps + warp;
  if (i >= meta->n_touched) return;
  const uint32_t t = touched[i];
  const uint32_t len = counts[t];
  const uint64_t* seg = csr + offsets[t];
  uint32_t* row = graph + static_cast<size_t>(t) * total_deg;
  const uint32_t take = len < cap ? len : cap;

  uint32_t rng = wang_hash(t);
  if (REMOTE) {  // the local pass of this node advanced the generator twice per applied request
    uint32_t lc = counts_local[t];
    if (lc > lmax) lc = lmax;
    for (uint32_t r = 0; r < 2 * lc; ++r) rng = wang_hash(rng);
  }
  auto apply = [&](uint32_t c) {  // executed by lane 0 only
    if (!REMOTE) {
      const uint32_t half = local_deg / 2, weak = local_deg - half;
      rng = wang_hash(rng);
      const bool atk = (rng % 100) < 10;
      const uint32_t ts = atk ? 0 : half, tl = atk ? half : weak;
      if (tl > 0) {
        rng = wang_hash(rng);
        row[ts + (rng % tl)] = c;
      }
    } else {
      const uint32_t rd = total_deg - local_deg;
      const int64_t mt = static_cast<int64_t>(bucket[t]), ct = static_cast<int64_t>(bucket[c]);
      const bool near = (ct >= mt - 20) && (ct <= mt + 20);
      const uint32_t nlen = rd / 3;
      const uint32_t ts = near ? local_deg : local_deg + rd / 3;
      const uint32_t tl = near ? nlen : rd - nlen;
      if (tl > 0) {
        rng = wang_hash(rng);
        row[ts + (rng % tl)] = c;
      }
    }
  };

  if (len <= kSelSort) {
    uint64_t* keys = sbuf[warp];
    uint32_t padded = 32;
    while (padded < len) padded <<= 1;
    for (uint32_t j = lane; j < padded; j += 32) keys[j] = j < len ? seg[j] : kMaxKey;
    __syncwarp();
    for (uint32_t size = 2; size <= padded; size <<= 1)
      for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
        for (uint32_t x = lane; x < (padded >> 1); x += 32) {
          const uint32_t lo = ((x & ~(stride - 1)) << 1) | (x & (stride - 1));
          const uint32_t hi = lo | stride;
          const bool up = (lo & size) == 0;
          const uint64_t a = keys[lo], b = keys[hi];
          if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
        }
        __syncwarp();
      }
    if (lane == 0)
      for (uint32_t r = 0; r < take; ++r) apply(static_cast<uint32_t>(keys[r] >> 32));
  } else {
    uint64_t last = 0;
    for (uint32_t r = 0; r < take; ++r) {
      uint64_t best = kMaxKey;
      for (uint32_t j = lane; j < len; j += 32) {
        const uint64_t key = seg[j];
        if ((r == 0 || key > last) && key < best) best = key;
      }
      for (int off = 16; off > 0; off >>= 1) {
        const uint64_t o = __shfl_xor_sync(0xFFFFFFFFu, best, off);
        best = o < best ? o : best;
      }
      if (lane == 0) apply(static_cast<uint32_t>(best >> 32));
      last = best;
    }
  }
  // leave the pooled arrays all-zero for the next batch (the local counts are still needed by
  // the remote pass and are cleared by mail_clear_kernel afterwards)
  if (lane == 0) {
    cursor[t] = 0;
    if (REMOTE) counts[t] = 0;
  }
}

// Distance-aware reverse-edge repair (alternatives to the reference's rule above, which overwrites a pseudo-random
// slot -- 10 % strong half / 90 % weak half, insert.cu:693-712 -- whatever it holds).  One warp per touched node t
// and column region [c0, c1): distances from t to the region's current neighbours and to every new node that asked
// to be linked (up to 256 requests); the requests are then taken nearest first.
//   ALWAYS = 1 (the class default): like the reference, every request up to the mailbox capacity (half the region)
//     gets a slot, so that every new node receives the in-edges that make it reachable -- but the slot it takes is
//     the FARTHEST old neighbour in the weak half of the region, not a random one; slots given to new nodes in this
//     pass are not evicted again.
//   ALWAYS = 0: a request replaces the farthest neighbour of the whole region only when it is closer (rows stay
//     "the nearest seen so far"; on data whose neighbourhoods are crowded few new nodes earn an in-edge, which
//     costs recall over the new region -- kept for comparison).
// Empty slots count as infinitely far, a request already present is skipped.  Ties go to the lower id / lower
// slot, so the result does not depend on the order in which the requests were posted.
constexpr int kRepairMaxRegion = 256;
constexpr int kRepairMaxReq = 256;

template <int METRIC, int REMOTE, int ALWAYS>
__global__ void __launch_bounds__(kSelWarps * 32)
mail_apply_dist_kernel(uint32_t* __restrict__ graph, const float* __restrict__ data, uint32_t dim,
                       const uint32_t* __restrict__ touched, const MailMeta* __restrict__ meta,
                       uint32_t* __restrict__ counts, const uint32_t* __restrict__ offsets,
                       uint32_t* __restrict__ cursor, const uint64_t* __restrict__ csr, uint32_t c0, uint32_t c1,
                       uint32_t total_deg) {
  __shared__ float s_rowd[kSelWarps][kRepairMaxRegion];
  __shared__ float s_reqd[kSelWarps][kRepairMaxReq];
  __shared__ uint32_t s_req[kSelWarps][kRepairMaxReq];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t i = blockIdx.x * kSelWarps + warp;
  if (i >= meta->n_touched) return;
  const uint32_t t = touched[i];
  const uint32_t len = counts[t];
  const uint64_t* seg = csr + offsets[t];
  uint32_t* row = graph + static_cast<size_t>(t) * total_deg + c0;
  const uint32_t rlen = c1 - c0;
  const uint32_t nreq = len < kRepairMaxReq ? len : kRepairMaxReq;
  float* rowd = s_rowd[warp];
  float* reqd = s_reqd[warp];
  uint32_t* req = s_req[warp];
  for (uint32_t j = lane; j < nreq; j += 32) req[j] = static_cast<uint32_t>(seg[j] >> 32);
  __syncwarp();
  // distances: items [0, rlen) are the row's slots, [rlen, rlen + nreq) the requests; four teams of 8 lanes
  const int lane8 = lane & (kTeam - 1);
  const uint32_t team = lane / kTeam;
  const uint32_t nchunk = dim / 4;
  const float* vt = data + static_cast<size_t>(t) * dim;
  for (uint32_t it0 = 0; it0 < rlen + nreq; it0 += 4) {
    const uint32_t it = it0 + team;
    uint32_t id = kInvalid;
    if (it < rlen) id = row[it];
    else if (it < rlen + nreq) id = req[it - rlen];
    const bool valid = id != kInvalid;
    float acc = 0.0f;
    if (valid) {
      const float* vx = data + static_cast<size_t>(id) * dim;
      for (uint32_t c = lane8; c < nchunk; c += kTeam) acc = accum4<METRIC>(acc, ldg_f4(vt + 4 * c), ldg_f4(vx + 4 * c));
    }
    const float d = team_reduce<METRIC>(acc);
    if (lane8 == 0) {
      if (it < rlen) rowd[it] = valid ? d : kFltMax;
      else if (it < rlen + nreq) reqd[it - rlen] = d;
    }
  }
  __syncwarp();
  // a request that is already a neighbour in this region, or a second copy of a request, is dropped
  for (uint32_t j = lane; j < nreq; j += 32) {
    const uint32_t src = req[j];
    bool dup = false;
    for (uint32_t x = 0; x < rlen; ++x) dup |= (row[x] == src);
    for (uint32_t x = 0; x < j; ++x) dup |= (req[x] == src);
    if (dup) reqd[j] = kFltMax;
  }
  __syncwarp();
  // ALWAYS: victims come from the weak half only, at most as many as the reference's mailbox holds
  const uint32_t v0 = ALWAYS ? rlen / 2 : 0;
  const uint32_t max_rounds = ALWAYS ? (rlen / 2 < nreq ? rlen / 2 : nreq) : nreq;
  for (uint32_t round = 0; round < max_rounds; ++round) {
    // nearest remaining request, by (distance, id)
    uint64_t best = kMaxKey;
    uint32_t best_j = 0;
    for (uint32_t j = lane; j < nreq; j += 32) {
      const float d = reqd[j];
      if (d < kFltMax) {
        const uint64_t key = make_key(d, req[j]);
        if (key < best) { best = key; best_j = j; }
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      const uint64_t ok = __shfl_xor_sync(0xFFFFFFFFu, best, off);
      const uint32_t oj = __shfl_xor_sync(0xFFFFFFFFu, best_j, off);
      if (ok < best) { best = ok; best_j = oj; }
    }
    if (best == kMaxKey) break;
    // farthest current neighbour among the candidate victims, by (distance, slot) descending; slots handed to a
    // new node in this pass carry -FLT_MAX and are never picked while an old neighbour is left
    uint64_t worst = 0;
    for (uint32_t x = v0 + lane; x < rlen; x += 32) {
      const uint64_t key = (static_cast<uint64_t>(float_to_ordered(rowd[x])) << 32) | (rlen - 1 - x);
      if (key >= worst) worst = key;
    }
    for (int off = 16; off > 0; off >>= 1) {
      const uint64_t ow = __shfl_xor_sync(0xFFFFFFFFu, worst, off);
      if (ow > worst) worst = ow;
    }
    const uint32_t slot = rlen - 1 - static_cast<uint32_t>(worst & 0xFFFFFFFFull);
    const float dnew = key_dist(best);
    if (ALWAYS) {
      if (static_cast<uint32_t>(worst >> 32) == float_to_ordered(-kFltMax)) break;  // only new nodes left in the weak half
    } else {
      if (!(float_to_ordered(dnew) < static_cast<uint32_t>(worst >> 32))) break;  // every remaining request is farther still
    }
    if (lane == 0) {
      row[slot] = key_id(best);
      rowd[slot] = ALWAYS ? -kFltMax : dnew;
      reqd[best_j] = kFltMax;
    }
    __syncwarp();
  }
  if (lane == 0) {
    cursor[t] = 0;
    if (REMOTE) counts[t] = 0;
  }
}

__global__ void mail_clear_kernel(const uint32_t* __restrict__ touched, const MailMeta* __restrict__ meta,
                                  uint32_t* __restrict__ counts) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < meta->n_touched) counts[touched[i]] = 0;
}

// d_dataset == NULL: the reference's slot rule.  Otherwise the distance-aware repair (regions of up to 256 columns),
// repair_mode 1 = every request takes the farthest weak-half slot, 2 = only requests closer than the farthest.
// sync: wait for the stream before returning (the stateless entry points do, the batched class insert does not).
int update_topology_opt_impl(uint32_t* d_graph, const uint64_t* d_bucket, int64_t* d_local_knn,
                             int64_t* d_global_knn, uint64_t num_existing, uint64_t num_new,
                             uint64_t target_bucket, uint32_t total_deg, uint32_t local_deg,
                             uint32_t k_local, uint32_t k_global, cudaStream_t st, const float* d_dataset,
                             uint32_t dim, int metric, bool sync, int repair_mode) {
  GRAB_REQUIRE(d_graph && d_bucket && d_local_knn && d_global_knn, "update_topology_opt: null pointer");
  GRAB_REQUIRE(local_deg >= 2 && local_deg < total_deg && total_deg - local_deg >= 2 && total_deg <= 512,
               "update_topology_opt: bad degrees %u/%u", local_deg, total_deg);
  if (num_new == 0) return GRAB_OK;
  opt_fill_kernel<<<(unsigned)((num_new + 127) / 128), 128, 0, st>>>(
      d_graph, d_bucket, d_local_knn, d_global_knn, num_existing, num_new, total_deg, local_deg, k_local,
      k_global);
  GRAB_CUDA_TRY(cudaGetLastError());
  if (num_existing == 0) return GRAB_OK;
  const uint64_t ntot = num_existing + num_new;
  const uint32_t lmax = local_deg / 2, rmax = (total_deg - local_deg) / 2;
  const uint64_t max_edges = num_new * (local_deg > total_deg - local_deg ? local_deg : total_deg - local_deg);
  GRAB_REQUIRE(max_edges < (1ull << 31), "update_topology_opt: batch too large");
  uint32_t* counts_l = static_cast<uint32_t*>(pool_get(kPoolMailCountsL, sizeof(uint32_t) * num_existing, true));
  uint32_t* counts_r = static_cast<uint32_t*>(pool_get(kPoolMailCountsR, sizeof(uint32_t) * num_existing, true));
  uint32_t* cursor = static_cast<uint32_t*>(pool_get(kPoolMailCursor, sizeof(uint32_t) * num_existing, true));
  uint32_t* offsets = static_cast<uint32_t*>(pool_get(kPoolMailOffsets, sizeof(uint32_t) * num_existing, false));
  uint32_t* touched = static_cast<uint32_t*>(pool_get(kPoolMailTouched, sizeof(uint32_t) * 2 * max_edges, false));
  uint64_t* csr = static_cast<uint64_t*>(pool_get(kPoolMailCsr, sizeof(uint64_t) * max_edges, false));
  MailMeta* meta = static_cast<MailMeta*>(pool_get(kPoolMailMeta, sizeof(MailMeta) * 2, false));
  if (!counts_l || !counts_r || !cursor || !offsets || !touched || !csr || !meta) {
    set_last_error("update_topology_opt: out of device memory for the mailbox scratch");
    return GRAB_ERR_CUDA;
  }
  // the counts and the cursor must be all-zero again when this call ends; if it ends early they are dropped and
  // allocated (zeroed) afresh by the next batch
  struct ZeroGuard {
    bool done = false;
    ~ZeroGuard() {
      if (!done) { pool_drop(kPoolMailCountsL); pool_drop(kPoolMailCountsR); pool_drop(kPoolMailCursor); }
    }
  } zero_guard;
  GRAB_CUDA_TRY(cudaMemsetAsync(meta, 0, sizeof(MailMeta) * 2, st));
  uint32_t* touched_l = touched;
  uint32_t* touched_r = touched + max_edges;
  EdgeSource e{};
  e.graph = d_graph; e.deg = total_deg; e.row0 = num_existing; e.row1 = ntot;
  e.n_dest = num_existing;  // mail for nodes of the batch itself is never applied (insert.cu:653-668)
  e.col_major_key = 0;
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 0) { e.c0 = 0; e.c1 = local_deg; e.use_skip = 0; }
    else { e.c0 = local_deg; e.c1 = total_deg; e.bucket = d_bucket; e.skip_bucket = target_bucket; e.use_skip = 1; }
    const uint64_t total = num_new * (e.c1 - e.c0);
    uint32_t* counts = pass == 0 ? counts_l : counts_r;
    uint32_t* tl = pass == 0 ? touched_l : touched_r;
    const unsigned eg = (unsigned)((total + 255) / 256);
    mail_count_kernel<<<eg, 256, 0, st>>>(e, total, counts, tl, meta + pass);
    mail_offsets_kernel<<<eg, 256, 0, st>>>(tl, meta + pass, counts, offsets);
    group_fill_kernel<<<eg, 256, 0, st>>>(e, total, offsets, cursor, csr);
    const unsigned ag = (unsigned)((total + kSelWarps - 1) / kSelWarps);  // upper bound on touched nodes
    if (d_dataset && e.c1 - e.c0 <= kRepairMaxRegion) {
#define GRAB_REPAIR(M, R, A)                                                                                       \
  mail_apply_dist_kernel<M, R, A><<<ag, kSelWarps * 32, 0, st>>>(d_graph, d_dataset, dim, tl, meta + pass, counts, \
                                                                offsets, cursor, csr, e.c0, e.c1, total_deg)
#define GRAB_REPAIR_M(M)                                                    \
  do {                                                                      \
    if (repair_mode == 2) { if (pass == 0) GRAB_REPAIR(M, 0, 0); else GRAB_REPAIR(M, 1, 0); } \
    else { if (pass == 0) GRAB_REPAIR(M, 0, 1); else GRAB_REPAIR(M, 1, 1); }                  \
  } while (0)
      if (metric == GRAB_METRIC_L2) GRAB_REPAIR_M(GRAB_METRIC_L2);
      else GRAB_REPAIR_M(GRAB_METRIC_IP);
#undef GRAB_REPAIR_M
#undef GRAB_REPAIR
    } else if (pass == 0)
      mail_apply_kernel<0><<<ag, kSelWarps * 32, 0, st>>>(d_graph, d_bucket, tl, meta + pass, counts, counts_l, offsets,
                                                          cursor, csr, lmax, lmax, total_deg, local_deg);
    else
      mail_apply_kernel<1><<<ag, kSelWarps * 32, 0, st>>>(d_graph, d_bucket, tl, meta + pass, counts, counts_l, offsets,
                                                          cursor, csr, rmax, lmax, total_deg, local_deg);
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  mail_clear_kernel<<<(unsigned)((num_new * local_deg + 255) / 256), 256, 0, st>>>(touched_l, meta, counts_l);
  GRAB_CUDA_TRY(cudaGetLastError());
  if (sync) GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  zero_guard.done = true;
  return GRAB_OK;
}

}  // namespace grab
