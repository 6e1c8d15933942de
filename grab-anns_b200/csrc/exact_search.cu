// Exact filtered brute force and exact block kNN (one scan kernel serves both).
//
// Replaces the CPU ground-truth routine tests/test_cagra_auto.cu:57-89 of the reference
// (exact filtered top-k) and the exact self-join it asks RAFT for
// (src/index/raft_help.cuh:74-172).  HBM/L2-bound streaming work: every lane issues 16-byte
// loads, a team of 8 lanes owns one vector, 32 teams per CTA, 4 vectors in flight per team.
// Top-k: keys (dist,id) below the running k-th key are appended to a shared-memory buffer
// that is bitonic-sorted into the top-k when it fills.
#include "common.cuh"
#include "windows.cuh"

namespace grab {

struct ScanFilter {
  int kind;  // grab_filter_kind (NONE / TS_RANGE / LABELS)
  const uint64_t* ts;
  const uint64_t* lo;
  const uint64_t* hi;
  uint64_t lo1, hi1;
  const uint8_t* labels;
  const uint32_t* masks;
  uint32_t mask1;
};


constexpr int kScanThreads = 256;
constexpr int kScanTeams = kScanThreads / kTeam;  // 32
constexpr int kScanUnroll = 4;                    // vectors in flight per team
constexpr int kScanStep = kScanTeams * kScanUnroll;
constexpr uint32_t kScanMinBuf = 2 * kScanStep;

__host__ __device__ inline uint32_t scan_total_slots(uint32_t k) {
  uint32_t v = k + kScanMinBuf;
  uint32_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

// CPL = float4 chunks per lane when dim is a compile-time 32*CPL (0 = generic dim).
template <int METRIC, int CPL>
__global__ void __launch_bounds__(kScanThreads)
exact_scan_kernel(const float* __restrict__ data, uint32_t dim, ScanFilter f,
                  const ScanWindow* __restrict__ windows, uint64_t n,
                  const float* __restrict__ queries, uint64_t nq, uint32_t k, uint32_t splits,
                  uint64_t* __restrict__ part_keys, int64_t* __restrict__ out_ids64,
                  uint32_t* __restrict__ out_ids32, float* __restrict__ out_dists) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t total = scan_total_slots(k);
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
  float* q_smem = reinterpret_cast<float*>(keys + total);
  __shared__ uint32_t s_count;
  __shared__ uint64_t s_thresh;

  const uint64_t qi = blockIdx.x / splits;
  const uint32_t split = blockIdx.x % splits;
  if (qi >= nq) return;
  const uint32_t tid = threadIdx.x;
  const int lane8 = tid & (kTeam - 1);
  const uint32_t team = tid / kTeam;
  const uint32_t nchunk = dim / 4;

  const float* q = queries + qi * dim;
  for (uint32_t i = tid; i < dim; i += kScanThreads) q_smem[i] = q[i];
  for (uint32_t i = tid; i < total; i += kScanThreads) keys[i] = kMaxKey;
  if (tid == 0) {
    s_count = 0;
    s_thresh = kMaxKey;
  }
  __syncthreads();

  float4 qreg[CPL > 0 ? CPL : 1];
  if (CPL > 0) {
#pragma unroll
    for (int c = 0; c < CPL; ++c)
      qreg[c] = *reinterpret_cast<const float4*>(q_smem + 4 * (lane8 + kTeam * c));
  }

  ScanWindow w;
  if (windows) {
    w = windows[qi];
  } else {
    w.begin = 0; w.end = static_cast<uint32_t>(n); w.xbegin = 0; w.xend = 0;
  }
  uint64_t lo = 0, hi = 0;
  uint32_t mask = 0;
  if (f.kind == GRAB_FILTER_TS_RANGE) {
    lo = f.lo ? f.lo[qi] : f.lo1;
    hi = f.hi ? f.hi[qi] : f.hi1;
  } else if (f.kind == GRAB_FILTER_LABELS) {
    mask = f.masks ? f.masks[qi] : f.mask1;
  }
  // this CTA's share of the window, in whole steps
  const uint32_t len = w.end > w.begin ? w.end - w.begin : 0;
  uint32_t per = (len + splits - 1) / splits;
  per = (per + kScanStep - 1) / kScanStep * kScanStep;
  const uint64_t my_begin = static_cast<uint64_t>(w.begin) + static_cast<uint64_t>(per) * split;
  uint64_t my_end = my_begin + per;
  if (my_end > w.end) my_end = w.end;
  const uint32_t buf_cap = total - k;

  for (uint64_t base = my_begin; base < my_end; base += kScanStep) {
    uint32_t id[kScanUnroll];
    bool ok[kScanUnroll];
#pragma unroll
    for (int u = 0; u < kScanUnroll; ++u) {
      const uint64_t j = base + static_cast<uint64_t>(u) * kScanTeams + team;
      id[u] = static_cast<uint32_t>(j);
      bool pass = j < my_end && !(id[u] >= w.xbegin && id[u] < w.xend);
      if (pass && f.kind == GRAB_FILTER_TS_RANGE) {
        const uint64_t t = __ldg(f.ts + j);
        pass = t >= lo && t < hi;
      } else if (pass && f.kind == GRAB_FILTER_LABELS) {
        pass = (mask >> __ldg(f.labels + j)) & 1u;
      }
      ok[u] = pass;
    }
    float acc[kScanUnroll];
#pragma unroll
    for (int u = 0; u < kScanUnroll; ++u) acc[u] = 0.0f;
    if (CPL > 0) {
      float4 x[kScanUnroll][CPL > 0 ? CPL : 1];
#pragma unroll
      for (int u = 0; u < kScanUnroll; ++u)
#pragma unroll
        for (int c = 0; c < CPL; ++c)
          if (ok[u]) x[u][c] = ldg_f4(data + static_cast<size_t>(id[u]) * dim + 4 * (lane8 + kTeam * c));
#pragma unroll
      for (int u = 0; u < kScanUnroll; ++u)
#pragma unroll
        for (int c = 0; c < CPL; ++c)
          if (ok[u]) acc[u] = accum4<METRIC>(acc[u], qreg[c], x[u][c]);
    } else {
      for (uint32_t c = lane8; c < nchunk; c += kTeam) {
        const float4 qv = *reinterpret_cast<const float4*>(q_smem + 4 * c);
        float4 x[kScanUnroll];
#pragma unroll
        for (int u = 0; u < kScanUnroll; ++u)
          if (ok[u]) x[u] = ldg_f4(data + static_cast<size_t>(id[u]) * dim + 4 * c);
#pragma unroll
        for (int u = 0; u < kScanUnroll; ++u)
          if (ok[u]) acc[u] = accum4<METRIC>(acc[u], qv, x[u]);
      }
    }
    const uint64_t thresh = s_thresh;
#pragma unroll
    for (int u = 0; u < kScanUnroll; ++u) {
      const float d = team_reduce<METRIC>(acc[u]);
      if (lane8 == 0 && ok[u]) {
        const uint64_t key = make_key(d, id[u]);
        if (key < thresh) {
          const uint32_t pos = atomicAdd(&s_count, 1u);
          keys[k + pos] = key;  // pos < buf_cap: the buffer is flushed before it can overflow
        }
      }
    }
    __syncthreads();
    // Every thread must take the same branch (the sort below contains barriers).  The count is copied out and a
    // second barrier keeps the next step's appends from changing it while slower warps are still reading it.
    const uint32_t appended = s_count;
    __syncthreads();
    if (appended + kScanStep > buf_cap) {
      block_bitonic_sort(keys, total);
      for (uint32_t i = k + tid; i < total; i += kScanThreads) keys[i] = kMaxKey;
      if (tid == 0) {
        s_count = 0;
        s_thresh = keys[k - 1];
      }
      __syncthreads();
    }
  }
  __syncthreads();
  block_bitonic_sort(keys, total);

  if (part_keys) {
    uint64_t* dst = part_keys + (qi * splits + split) * k;
    for (uint32_t i = tid; i < k; i += kScanThreads) dst[i] = keys[i];
  } else {
    for (uint32_t i = tid; i < k; i += kScanThreads) {
      const uint64_t key = keys[i];
      const bool empty = key == kMaxKey;
      if (out_ids64) out_ids64[qi * k + i] = empty ? -1 : static_cast<int64_t>(key_id(key));
      if (out_ids32) out_ids32[qi * k + i] = empty ? kInvalid : key_id(key);
      if (out_dists) out_dists[qi * k + i] = empty ? kFltMax : key_dist(key);
    }
  }
}

// Merge `parts` ascending key lists per query; ids are widened and optionally rescaled.
__global__ void merge_keys_kernel(const uint64_t* __restrict__ part_keys, uint32_t parts, uint32_t k,
                                  uint32_t padded, int64_t* __restrict__ out_ids,
                                  float* __restrict__ out_dists) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
  const uint64_t qi = blockIdx.x;
  const uint32_t m = parts * k;
  for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x)
    keys[i] = i < m ? part_keys[qi * m + i] : kMaxKey;
  __syncthreads();
  block_bitonic_sort(keys, padded);
  for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
    const uint64_t key = keys[i];
    const bool empty = key == kMaxKey;
    out_ids[qi * k + i] = empty ? -1 : static_cast<int64_t>(key_id(key));
    out_dists[qi * k + i] = empty ? kFltMax : key_dist(key);
  }
}

// Merge `parts` ascending (dist, int64 id) lists per query straight from the pair arrays: the
// keys are built in shared memory, so the exchange step of the sharded search needs no scratch
// and no extra pass.  Ids must be < 2^32.
__global__ void merge_pairs_kernel(const float* __restrict__ dists, const int64_t* __restrict__ ids, uint32_t parts,
                                   uint32_t k, uint32_t padded, int64_t* __restrict__ out_ids,
                                   float* __restrict__ out_dists) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
  const uint64_t qi = blockIdx.x;
  const uint32_t m = parts * k;
  for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) {
    uint64_t key = kMaxKey;
    if (i < m) {
      const int64_t id = ids[qi * m + i];
      if (id >= 0) key = make_key(dists[qi * m + i], static_cast<uint32_t>(id));
    }
    keys[i] = key;
  }
  __syncthreads();
  block_bitonic_sort(keys, padded);
  for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
    const uint64_t key = keys[i];
    const bool empty = key == kMaxKey;
    out_ids[qi * k + i] = empty ? -1 : static_cast<int64_t>(key_id(key));
    out_dists[qi * k + i] = empty ? kFltMax : key_dist(key);
  }
}

// (dist, int64 id) lists -> keys (ids must be < 2^32), for the public merge entry point.
__global__ void pack_keys_kernel(const float* __restrict__ dists, const int64_t* __restrict__ ids,
                                 uint64_t total, uint64_t* __restrict__ keys) {
  const uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int64_t id = ids[i];
  keys[i] = id < 0 ? kMaxKey : make_key(dists[i], static_cast<uint32_t>(id));
}

// lower_bound over a non-decreasing timestamp array: range [lo,hi) -> id window.
__global__ void ts_window_kernel(const uint64_t* __restrict__ ts, uint64_t n,
                                 const uint64_t* __restrict__ lo, const uint64_t* __restrict__ hi,
                                 uint64_t lo1, uint64_t hi1, uint64_t nq,
                                 ScanWindow* __restrict__ windows) {
  const uint64_t qi = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (qi >= nq) return;
  const uint64_t bounds[2] = {lo ? lo[qi] : lo1, hi ? hi[qi] : hi1};
  uint32_t res[2];
  for (int b = 0; b < 2; ++b) {
    uint64_t l = 0, r = n;
    while (l < r) {
      const uint64_t m = (l + r) >> 1;
      if (ts[m] < bounds[b]) l = m + 1; else r = m;
    }
    res[b] = static_cast<uint32_t>(l);
  }
  ScanWindow w;
  w.begin = res[0];
  w.end = res[1] > res[0] ? res[1] : res[0];
  w.xbegin = 0;
  w.xend = 0;
  windows[qi] = w;
}

template <int METRIC>
static cudaError_t launch_scan(const float* data, uint32_t dim, const ScanFilter& f,
                               const ScanWindow* windows, uint64_t n, const float* queries,
                               uint64_t nq, uint32_t k, uint32_t splits, uint64_t* part_keys,
                               int64_t* out64, uint32_t* out32, float* out_d, cudaStream_t st) {
  const size_t smem = sizeof(uint64_t) * scan_total_slots(k) + sizeof(float) * dim;
  const uint64_t grid = nq * splits;
#define GRAB_SCAN_LAUNCH(CPL)                                                                    \
  do {                                                                                           \
    cudaError_t e = cudaFuncSetAttribute(exact_scan_kernel<METRIC, CPL>,                         \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);\
    if (e != cudaSuccess) return e;                                                              \
    exact_scan_kernel<METRIC, CPL><<<(unsigned)grid, kScanThreads, smem, st>>>(                  \
        data, dim, f, windows, n, queries, nq, k, splits, part_keys, out64, out32, out_d);       \
  } while (0)
  if (dim == 96) GRAB_SCAN_LAUNCH(3);
  else if (dim == 128) GRAB_SCAN_LAUNCH(4);
  else GRAB_SCAN_LAUNCH(0);
#undef GRAB_SCAN_LAUNCH
  return cudaGetLastError();
}

static uint32_t choose_splits(uint64_t n, uint64_t nq, uint32_t k) {
  const uint64_t target_ctas = 148ull * 8;
  uint64_t s = nq >= target_ctas ? 1 : (target_ctas + nq - 1) / nq;
  const uint64_t max_by_len = n / 4096 > 0 ? n / 4096 : 1;
  if (s > max_by_len) s = max_by_len;
  if (s > 64) s = 64;
  while (s > 1 && s * k > 8192) --s;  // the merge sorts parts*k keys in shared memory
  return static_cast<uint32_t>(s);
}

int exact_search_impl(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                      const grab_filter* filter, const float* d_queries, uint64_t nq, uint32_t k,
                      int64_t* d_out_ids, float* d_out_dists, void* d_ws, size_t ws_bytes,
                      cudaStream_t st) {
  GRAB_REQUIRE(d_dataset && d_queries && d_out_ids && d_out_dists, "exact_search: null pointer");
  GRAB_REQUIRE(dim >= 4 && dim % 4 == 0, "exact_search: dim %u must be a multiple of 4", dim);
  GRAB_REQUIRE(k >= 1 && k <= 1024, "exact_search: k %u outside [1,1024]", k);
  GRAB_REQUIRE(n < (1ull << 31), "exact_search: n must be < 2^31");
  GRAB_REQUIRE(metric == GRAB_METRIC_L2 || metric == GRAB_METRIC_IP, "exact_search: bad metric");
  if (nq == 0) return GRAB_OK;
  ScanFilter f{};
  f.kind = GRAB_FILTER_NONE;
  bool window_from_ts = false;
  if (filter) {
    if (filter->kind == GRAB_FILTER_TS_RANGE) {
      GRAB_REQUIRE(filter->d_ts, "exact_search: ts filter without d_ts");
      GRAB_REQUIRE((filter->d_lo == nullptr) == (filter->d_hi == nullptr),
                   "exact_search: d_lo and d_hi must both be given or both NULL");
      f.ts = filter->d_ts; f.lo = filter->d_lo; f.hi = filter->d_hi;
      f.lo1 = filter->lo; f.hi1 = filter->hi;
      if (filter->ts_sorted) window_from_ts = true; else f.kind = GRAB_FILTER_TS_RANGE;
    } else if (filter->kind == GRAB_FILTER_LABELS) {
      GRAB_REQUIRE(filter->d_labels, "exact_search: label filter without d_labels");
      f.kind = GRAB_FILTER_LABELS;
      f.labels = filter->d_labels; f.masks = filter->d_masks; f.mask1 = filter->mask;
    } else {
      GRAB_REQUIRE(filter->kind == GRAB_FILTER_NONE, "exact_search: unsupported filter kind %d",
                   filter->kind);
    }
  }
  const uint32_t splits = choose_splits(n, nq, k);
  const size_t need = grab_exact_search_workspace_bytes(n, nq, k);
  ScopedDeviceBuffer own;
  if (!d_ws) {
    GRAB_CUDA_TRY(own.alloc(need));
    d_ws = own.ptr;
  } else if (ws_bytes < need) {
    set_last_error("exact_search: workspace %zu < %zu bytes", ws_bytes, need);
    return GRAB_ERR_WORKSPACE;
  }
  ScanWindow* windows = static_cast<ScanWindow*>(d_ws);
  uint64_t* part = reinterpret_cast<uint64_t*>(static_cast<char*>(d_ws) +
                                               ((sizeof(ScanWindow) * nq + 255) / 256) * 256);
  const ScanWindow* win_arg = nullptr;
  if (window_from_ts) {
    ts_window_kernel<<<(unsigned)((nq + 255) / 256), 256, 0, st>>>(f.ts, n, f.lo, f.hi, f.lo1, f.hi1,
                                                                   nq, windows);
    GRAB_CUDA_TRY(cudaGetLastError());
    win_arg = windows;
  }
  uint64_t* part_arg = splits > 1 ? part : nullptr;
  cudaError_t e;
  if (metric == GRAB_METRIC_L2)
    e = launch_scan<GRAB_METRIC_L2>(d_dataset, dim, f, win_arg, n, d_queries, nq, k, splits,
                                    part_arg, d_out_ids, nullptr, d_out_dists, st);
  else
    e = launch_scan<GRAB_METRIC_IP>(d_dataset, dim, f, win_arg, n, d_queries, nq, k, splits,
                                    part_arg, d_out_ids, nullptr, d_out_dists, st);
  GRAB_CUDA_TRY(e);
  if (splits > 1) {
    const uint32_t padded = next_pow2(splits * k);
    merge_keys_kernel<<<(unsigned)nq, 256, sizeof(uint64_t) * padded, st>>>(part, splits, k, padded,
                                                                          d_out_ids, d_out_dists);
    GRAB_CUDA_TRY(cudaGetLastError());
  }
  if (own.ptr) GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  return GRAB_OK;
}

int knn_blocks_impl(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                    const uint64_t* h_block_offsets, uint32_t num_blocks, uint32_t k, int mode,
                    uint32_t* d_out_knn, float* d_out_dists, cudaStream_t st) {
  GRAB_REQUIRE(d_dataset && h_block_offsets && d_out_knn, "knn_graph_blocks: null pointer");
  GRAB_REQUIRE(dim >= 4 && dim % 4 == 0, "knn_graph_blocks: dim %u must be a multiple of 4", dim);
  GRAB_REQUIRE(k >= 1 && k <= 1024, "knn_graph_blocks: k %u outside [1,1024]", k);
  GRAB_REQUIRE(n < (1ull << 31) && num_blocks >= 1, "knn_graph_blocks: bad sizes");
  GRAB_REQUIRE(h_block_offsets[0] == 0 && h_block_offsets[num_blocks] == n,
               "knn_graph_blocks: block offsets must span [0,n]");
  GRAB_REQUIRE(mode == 0 || mode == 1, "knn_graph_blocks: mode must be 0 or 1");
  if (n == 0) return GRAB_OK;
  ScopedDeviceBuffer offs, wins;
  GRAB_CUDA_TRY(offs.alloc(sizeof(uint64_t) * (num_blocks + 1)));
  GRAB_CUDA_TRY(wins.alloc(sizeof(ScanWindow) * n));
  GRAB_CUDA_TRY(cudaMemcpyAsync(offs.ptr, h_block_offsets, sizeof(uint64_t) * (num_blocks + 1),
                                cudaMemcpyHostToDevice, st));
  knn_window_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(offs.as<uint64_t>(), num_blocks, n,
                                                                mode, wins.as<ScanWindow>());
  GRAB_CUDA_TRY(cudaGetLastError());
  ScanFilter f{};
  f.kind = GRAB_FILTER_NONE;
  cudaError_t e;
  if (metric == GRAB_METRIC_L2)
    e = launch_scan<GRAB_METRIC_L2>(d_dataset, dim, f, wins.as<ScanWindow>(), n, d_dataset, n, k, 1,
                                    nullptr, nullptr, d_out_knn, d_out_dists, st);
  else
    e = launch_scan<GRAB_METRIC_IP>(d_dataset, dim, f, wins.as<ScanWindow>(), n, d_dataset, n, k, 1,
                                    nullptr, nullptr, d_out_knn, d_out_dists, st);
  GRAB_CUDA_TRY(e);
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  return GRAB_OK;
}

int merge_topk_impl(const float* d_dists, const int64_t* d_ids, uint64_t nq, uint32_t parts,
                    uint32_t k, int64_t* d_out_ids, float* d_out_dists, cudaStream_t st) {
  GRAB_REQUIRE(d_dists && d_ids && d_out_ids && d_out_dists, "merge_topk: null pointer");
  GRAB_REQUIRE(parts >= 1 && k >= 1 && (uint64_t)parts * k <= 8192,
               "merge_topk: parts*k = %llu exceeds 8192", (unsigned long long)parts * k);
  if (nq == 0) return GRAB_OK;
  const uint32_t padded = next_pow2(parts * k);
  const size_t smem = sizeof(uint64_t) * padded;
  const uint32_t threads = padded >= 512 ? 256 : (padded >= 128 ? 64 : 32);
  GRAB_CUDA_TRY(cudaFuncSetAttribute(merge_pairs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  merge_pairs_kernel<<<(unsigned)nq, threads, smem, st>>>(d_dists, d_ids, parts, k, padded, d_out_ids, d_out_dists);
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;  // stream-ordered: nothing allocated, nothing synchronised
}

}  // namespace grab

extern "C" size_t grab_exact_search_workspace_bytes(uint64_t n, uint64_t nq, uint32_t k) {
  const uint32_t splits = grab::choose_splits(n, nq, k);
  return ((sizeof(grab::ScanWindow) * nq + 255) / 256) * 256 + sizeof(uint64_t) * nq * splits * k +
         256;
}
