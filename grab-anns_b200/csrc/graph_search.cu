// Filtered graph search (timestamp range / bucket prefix / label mask / none).
//
// One kernel replaces the reference's three (src/index/search.cu:149 search_kernel, :375
// search_kernel_bucket, :589 search_kernel_range) and its building blocks
// (compute_distance.cuh:204-614, hashmap.cuh, the sorts of search.cu:110-144).  Same loop
// -- keep the best `itopk`, pick up to `search_width` unexpanded parents, expand their
// rows, repeat -- re-laid for B200:
//   * the filter predicate runs BEFORE the visited-set insert and before any vector is
//     fetched, so rejected neighbours cost 4+f bytes and never pollute the table
//     (the reference inserts first: compute_distance.cuh:572-584);
//   * survivors are compacted, then teams of 8 lanes gather one vector each with 16-byte
//     loads, 2 vectors in flight per team (the reference: one warp, scalar loads, per
//     neighbour);
//   * small CTAs (2 warps) and many of them per SM: the phases of one query (expand, gather,
//     merge) overlap with the phases of the others, which is what hides the gather latency;
//   * queue entries are single uint64 (dist,id) keys; a candidate enters the merge only if it
//     beats the current worst of the itopk list; one warp sorts those few keys and folds them
//     into the sorted itopk with a bitonic merge (the reference re-sorts the whole queue with
//     one warp every iteration, search.cu:702-716);
//   * the visited table is cleared when half full and re-seeded from the current itopk
//     (the reference: every 30 iterations, search.cu:692-697).
// HBM/latency-bound by design: no tensor cores.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "search_blocks.cuh"

namespace grab {

#ifndef GRAB_SEARCH_THREADS
#define GRAB_SEARCH_THREADS 64
#endif
constexpr int kSearchThreads = GRAB_SEARCH_THREADS;
constexpr int kSearchTeams = kSearchThreads / kTeam;  // 8 teams of 8 lanes
// vectors in flight per team and resident CTAs per SM the register budget is capped for
#ifndef GRAB_SEARCH_UNROLL
#define GRAB_SEARCH_UNROLL 2
#endif
#ifndef GRAB_SEARCH_CTAS_PER_SM
#define GRAB_SEARCH_CTAS_PER_SM 14
#endif
#ifndef GRAB_SEARCH_QREG
#define GRAB_SEARCH_QREG 0  // 1: the query's float4 chunks live in registers (fixed dims); 0: re-read from shared
                            // memory, which frees the registers for 14 CTAs per SM (measured faster)
#endif
constexpr int kSearchUnroll = GRAB_SEARCH_UNROLL;
constexpr int kSearchCtasPerSm = GRAB_SEARCH_CTAS_PER_SM;

struct SearchKernelArgs {
  const float* data;
  uint64_t n;
  uint32_t dim;
  const uint32_t* graph;
  uint32_t deg;         // row stride
  uint32_t active_deg;  // columns walked
  const float* queries;
  uint64_t nq;
  uint32_t k, itopk, width, max_iter, hash_bitlen;
  uint32_t num_seeds;  // seeds evaluated per query
  const uint32_t* seeds;
  uint32_t seeds_per_query;
  uint64_t seed;
  int filter_kind;
  const uint64_t* ts;
  const uint64_t* lo;
  const uint64_t* hi;
  uint64_t lo1, hi1;
  const uint8_t* labels;
  const uint32_t* masks;
  uint32_t mask1;
  const uint32_t* label_offsets;  // [33] id range per label (vectors grouped by label), or NULL
  const uint32_t* windows;  // [nq,4] id window per query (sorted ts), or NULL
  uint32_t* global_hash;    // [nq, 2^bitlen] when the table does not fit shared memory
  int64_t* out_ids;
  float* out_dists;
  uint64_t* out_keys;  // [nq,k] (ordered dist << 32 | result id), or NULL
  uint64_t id_scale, id_offset;
  unsigned long long* stats;  // grab_search_stats as 6 x u64, or NULL
  uint32_t ckeys_cap;
  uint32_t cand_cap, sort_cap;  // survivor list capacity; sort_cap = itopk rounded up to a power of two
  uint32_t inv_active_deg;      // ceil(2^32 / active_deg) (0 when active_deg == 1): e / active_deg = umulhi(e, inv)
  uint32_t parts;               // CTAs that co-operate on one query (warp-split kernel only); 1 = the plain search
};

template <int METRIC, int CPL>
__global__ void __launch_bounds__(kSearchThreads, kSearchCtasPerSm)
graph_search_kernel(const SearchKernelArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* queue = reinterpret_cast<uint64_t*>(smem_raw);                 // [sort_cap] sorted itopk list
  uint64_t* ckeys = queue + a.sort_cap;                                    // [cand_cap pow2] kept candidates
  float* q_smem = reinterpret_cast<float*>(ckeys + a.ckeys_cap);           // [dim]
  uint32_t* cand = reinterpret_cast<uint32_t*>(q_smem + a.dim);            // [cand_cap] survivor ids
  uint32_t* parents = cand + a.cand_cap;                                   // [width]
  uint32_t* hash = parents + ((a.width + 3) & ~3u);                        // [2^bitlen] (if local)
  __shared__ uint32_t s_ncand, s_nparents, s_hash_count, s_nkeep;
  __shared__ unsigned long long s_stats[6];

  const uint64_t qi = blockIdx.x;
  if (qi >= a.nq) return;
  const uint32_t tid = threadIdx.x;
  const int lane8 = tid & (kTeam - 1);
  const uint32_t team = tid / kTeam;
  const uint32_t nchunk = a.dim / 4;
  const uint32_t hsize = 1u << a.hash_bitlen;
  if (a.global_hash) hash = a.global_hash + qi * hsize;

  for (uint32_t i = tid; i < a.dim; i += kSearchThreads) q_smem[i] = a.queries[qi * a.dim + i];
  for (uint32_t i = tid; i < a.sort_cap; i += kSearchThreads) queue[i] = kMaxKey;
  for (uint32_t i = tid; i < hsize; i += kSearchThreads) hash[i] = kInvalid;
  if (tid == 0) { s_ncand = 0; s_nparents = 0; s_hash_count = 0; s_nkeep = 0; }
  if (tid < 6) s_stats[tid] = 0;

  uint64_t lo = 0, hi = 0;
  uint32_t mask = 0;
  if (a.filter_kind == GRAB_FILTER_TS_RANGE) {
    lo = a.lo ? a.lo[qi] : a.lo1;
    hi = a.hi ? a.hi[qi] : a.hi1;
  } else if (a.filter_kind == GRAB_FILTER_LABELS) {
    mask = a.masks ? a.masks[qi] : a.mask1;
  }
  // Timestamps that are non-decreasing in the id turn a range into an id window: the
  // predicate then reads nothing (the reference gathers d_ts[nbr], compute_distance.cuh:580).
  uint32_t wbeg = 0, wend = 0;
  const bool by_window = a.windows != nullptr && a.filter_kind == GRAB_FILTER_TS_RANGE;
  if (a.windows) {
    wbeg = a.windows[qi * 4];
    wend = a.windows[qi * 4 + 1];
    if (wend < wbeg) wend = wbeg;
  }
  auto passes = [&](uint32_t id) -> bool {
    if (by_window) return id >= wbeg && id < wend;
    if (a.filter_kind == GRAB_FILTER_TS_RANGE) {
      const uint64_t t = __ldg(a.ts + id);
      return t >= lo && t < hi;
    }
    if (a.filter_kind == GRAB_FILTER_LABELS) return (mask >> __ldg(a.labels + id)) & 1u;
    return true;
  };
  __syncthreads();

#if GRAB_SEARCH_QREG
  float4 qreg[CPL > 0 ? CPL : 1];
  if (CPL > 0) {
#pragma unroll
    for (int c = 0; c < CPL; ++c)
      qreg[c] = *reinterpret_cast<const float4*>(q_smem + 4 * (lane8 + kTeam * c));
  }
#define GRAB_Q(c) qreg[c]
#else
#define GRAB_Q(c) (*reinterpret_cast<const float4*>(q_smem + 4 * (lane8 + kTeam * (c))))
#endif

  // ---- seeds (compute_distance.cuh:204-269): provided ids, else pseudo-random ids ----
  {
    const uint32_t wlen = wend - wbeg;
    const bool generated_only = (a.seeds == nullptr);
    const bool by_label_range = a.filter_kind == GRAB_FILTER_LABELS && a.label_offsets != nullptr && mask != 0;
    const uint32_t nlab = __popc(mask);
    // without an id window a generated seed may fail the filter: allow 4 attempts per seed
    const uint32_t attempts = (generated_only && !a.windows && !by_label_range && a.filter_kind != GRAB_FILTER_NONE &&
                               a.filter_kind != GRAB_FILTER_PREFIX) ? 4 * a.num_seeds : a.num_seeds;
    for (uint32_t i = tid; i < attempts; i += kSearchThreads) {
      uint32_t id = kInvalid;
      if (a.seeds && i < a.seeds_per_query) id = a.seeds[qi * a.seeds_per_query + i];
      if (id >= a.n) {
        if (a.windows) {
          id = wlen ? wbeg + static_cast<uint32_t>(mix64(a.seed ^ (qi * 0x9e3779b97f4a7c15ull + i)) % wlen)
                    : kInvalid;
        } else if (by_label_range) {
          // round-robin over the query's labels, a pseudo-random member of the label's id range
          uint32_t m = mask;
          for (uint32_t skip = i % nlab; skip > 0; --skip) m &= m - 1;
          const uint32_t lab = __ffs(m) - 1;
          const uint32_t lb = a.label_offsets[lab], le = a.label_offsets[lab + 1];
          id = le > lb ? lb + static_cast<uint32_t>(mix64(a.seed ^ (qi * 0x9e3779b97f4a7c15ull + i)) % (le - lb))
                       : kInvalid;
        } else {
          // reference rule: (xor_mask * (i+1)) % n, compute_distance.cuh:236-238
          id = static_cast<uint32_t>(((a.seed | 1ull) * static_cast<uint64_t>(i + 1)) % a.n);
        }
      }
      if (id < a.n && passes(id) && hash_insert(hash, a.hash_bitlen, id)) {
        const uint32_t pos = atomicAdd(&s_ncand, 1u);
        if (pos < a.num_seeds) cand[pos] = id;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    if (s_ncand > a.num_seeds) s_ncand = a.num_seeds;
    s_hash_count = s_ncand;
    s_stats[4] += s_ncand;
  }
  __syncthreads();

  uint32_t iter = 0;
  for (;;) {
    // ---- distances of the compacted candidates: 8 teams, vectors gathered with 16-byte loads;
    //      a key is kept only if it beats the current worst entry of the itopk list ----
    const uint32_t ncand = s_ncand;
    const uint64_t worst = queue[a.sort_cap - 1];
    for (uint32_t j0 = 0; j0 < ncand; j0 += kSearchTeams * kSearchUnroll) {
      uint32_t id[kSearchUnroll];
      bool ok[kSearchUnroll];
      float acc[kSearchUnroll];
#pragma unroll
      for (int u = 0; u < kSearchUnroll; ++u) {
        const uint32_t j = j0 + u * kSearchTeams + team;
        ok[u] = j < ncand;
        id[u] = ok[u] ? cand[j] : 0;
        acc[u] = 0.0f;
      }
      if (CPL > 0) {
        float4 x[kSearchUnroll][CPL > 0 ? CPL : 1];
#pragma unroll
        for (int u = 0; u < kSearchUnroll; ++u)
#pragma unroll
          for (int c = 0; c < CPL; ++c)
            if (ok[u]) x[u][c] = ldg_f4(a.data + static_cast<size_t>(id[u]) * a.dim + 4 * (lane8 + kTeam * c));
#pragma unroll
        for (int u = 0; u < kSearchUnroll; ++u)
#pragma unroll
          for (int c = 0; c < CPL; ++c)
            if (ok[u]) acc[u] = accum4<METRIC>(acc[u], GRAB_Q(c), x[u][c]);
      } else {
        // any dimension: four chunks per vector in flight, accumulated in ascending chunk order
        for (uint32_t c0 = lane8; c0 < nchunk; c0 += 4 * kTeam) {
          float4 x[kSearchUnroll][4];
#pragma unroll
          for (int u = 0; u < kSearchUnroll; ++u)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t c = c0 + i * kTeam;
              if (ok[u] && c < nchunk) x[u][i] = ldg_f4(a.data + static_cast<size_t>(id[u]) * a.dim + 4 * c);
            }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t c = c0 + i * kTeam;
            if (c < nchunk) {
              const float4 qv = *reinterpret_cast<const float4*>(q_smem + 4 * c);
#pragma unroll
              for (int u = 0; u < kSearchUnroll; ++u)
                if (ok[u]) acc[u] = accum4<METRIC>(acc[u], qv, x[u][i]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kSearchUnroll; ++u) {
        const float d = team_reduce<METRIC>(acc[u]);
        if (lane8 == 0 && ok[u]) {
          const uint64_t key = make_skey(d, id[u]);
          if (key < worst) ckeys[atomicAdd(&s_nkeep, 1u)] = key;
        }
      }
    }
    __syncthreads();

    // ---- warp 0: sort the kept candidates and fold them into the sorted itopk list ----
    if (tid < 32) {
      const uint32_t nkeep = s_nkeep;
      if (nkeep > 0) {
        if (a.sort_cap == 64 && nkeep <= 64) {
          warp_sort_merge_regs<2>(queue, ckeys, nkeep, tid);
        } else if (a.sort_cap == 128 && nkeep <= 128) {
          warp_sort_merge_regs_128(queue, ckeys, nkeep, tid);
        } else {
          uint32_t padded = 32;
          while (padded < nkeep) padded <<= 1;
          for (uint32_t i = nkeep + tid; i < padded; i += 32) ckeys[i] = kMaxKey;
          __syncwarp();
          warp_bitonic_sort_smem(ckeys, padded, tid);
          warp_merge_into_topk(queue, a.sort_cap, ckeys, nkeep, tid);
        }
        __syncwarp();
      }
      if (tid == 0) s_nkeep = 0;
    }
    __syncthreads();

    // ---- visited table half full: clear and re-seed from the current itopk ----
    if (s_hash_count > hsize / 2) {  // uniform
      __syncthreads();
      for (uint32_t i = tid; i < hsize; i += kSearchThreads) hash[i] = kInvalid;
      __syncthreads();
      uint32_t kept = 0;
      for (uint32_t i = tid; i < a.sort_cap; i += kSearchThreads) {
        const uint64_t key = queue[i];
        if (key != kMaxKey) { hash_insert(hash, a.hash_bitlen, skey_id(key)); ++kept; }
      }
      kept = __reduce_add_sync(0xFFFFFFFFu, kept);
      if (tid == 0) { s_hash_count = 0; s_stats[5] += 1; }
      __syncthreads();
      if ((tid & 31) == 0) atomicAdd(&s_hash_count, kept);
    }
    if (iter >= a.max_iter) break;

    // ---- pick up to `width` unexpanded parents, best first (search.cu:38-107) ----
    if (tid < 32) {
      uint32_t found = 0;
      for (uint32_t j0 = 0; j0 < a.sort_cap && found < a.width; j0 += 32) {
        const uint32_t j = j0 + tid;
        uint64_t key = j < a.sort_cap ? queue[j] : kMaxKey;
        const bool fresh = key != kMaxKey && !skey_expanded(key);
        const uint32_t vote = __ballot_sync(0xFFFFFFFFu, fresh);
        if (fresh) {
          const uint32_t rank = found + __popc(vote & ((1u << tid) - 1));
          if (rank < a.width) {
            parents[rank] = skey_id(key);
            queue[j] = key | 1ull;
          }
        }
        found += __popc(vote);
      }
      if (found > a.width) found = a.width;
      if (tid == 0) { s_nparents = found; s_ncand = 0; }
    }
    __syncthreads();
    const uint32_t nparents = s_nparents;
    if (nparents == 0) break;

    // ---- expand: neighbour id -> filter -> visited set -> compacted survivor list.  A thread owns
    //      graph columns; the ids of up to four parents' rows are loaded before any is processed, so
    //      the row reads of an iteration overlap instead of queueing behind the hash probes ----
    uint32_t my_edges = 0;
    for (uint32_t col = tid; col < a.active_deg; col += kSearchThreads) {
      for (uint32_t p0 = 0; p0 < nparents; p0 += 4) {
        uint32_t nbv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          nbv[u] = p0 + u < nparents ? __ldg(a.graph + static_cast<size_t>(parents[p0 + u]) * a.deg + col) : kInvalid;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t nb = nbv[u];
          if (nb < a.n) {
            ++my_edges;
            if (passes(nb) && hash_insert(hash, a.hash_bitlen, nb)) {
              const uint32_t pos = atomicAdd(&s_ncand, 1u);
              cand[pos] = nb;
            }
          }
        }
      }
    }
    if (a.stats) {
      my_edges = __reduce_add_sync(0xFFFFFFFFu, my_edges);
      if ((tid & 31) == 0) atomicAdd(&s_stats[2], static_cast<unsigned long long>(my_edges));
    }
    __syncthreads();
    if (tid == 0) {
      s_hash_count += s_ncand;
      s_stats[0] += 1;
      s_stats[1] += nparents;
      s_stats[3] += s_ncand;
    }
    ++iter;
    __syncthreads();
  }

  // ---- results: ascending (dist,id); id = local*scale + offset; empty slots are -1 ----
  __syncthreads();
  for (uint32_t i = tid; i < a.k; i += kSearchThreads) {
    const uint64_t key = queue[i];
    const bool empty = key == kMaxKey;
    const uint64_t gid = static_cast<uint64_t>(skey_id(key)) * a.id_scale + a.id_offset;
    if (a.out_ids) a.out_ids[qi * a.k + i] = empty ? -1 : static_cast<int64_t>(gid);
    if (a.out_dists) a.out_dists[qi * a.k + i] = empty ? kFltMax : key_dist(key);
    if (a.out_keys) a.out_keys[qi * a.k + i] = empty ? kMaxKey : ((key & 0xFFFFFFFF00000000ull) | gid);
  }
  if (a.stats && tid < 6) atomicAdd(&a.stats[tid], s_stats[tid]);
}

// ---------------------------------------------------------------------------------------------------------
// Warp-split variant of the same search loop (lists of 64 or 128 entries, at most 256 candidates per warp and
// iteration).  The two warps of a CTA no longer share a survivor list: each expands its own half of the
// parents' edges, compacts its survivors by ballot (no shared counters), gathers THEIR vectors, keeps the keys
// that beat the list's worst entry and sorts them in registers; then warp 0 folds both sorted runs into the
// list and picks the next parents while the list is still in its registers.  Two block barriers per iteration
// instead of five, no shared-memory atomics outside the visited set, and the merge work is split over both
// warps.  Results are the same set the shared-list kernel finds whenever no candidate is dropped for capacity.
// ---------------------------------------------------------------------------------------------------------
#ifndef GRAB_SEARCH2_CTAS_PER_SM
#define GRAB_SEARCH2_CTAS_PER_SM 14
#endif
#ifndef GRAB_SEARCH_UNROLL_96
#define GRAB_SEARCH_UNROLL_96 2
#endif
// 1: while picking parents, prefetch into L2 the graph rows of the runners-up (the likely parents of the next
// iteration). Measured on B200: slower (1M x 128, k 10: 0.365 ms against 0.352 ms per launch; 12.5M x 96, k 100:
// 0.873 against 0.800 ms) - the extra requests compete with the vector gathers that bound the kernel. Off.
#ifndef GRAB_SEARCH_PREFETCH
#define GRAB_SEARCH_PREFETCH 0
#endif
// 1: the lane that admits a survivor (seed or neighbour) prefetches its vector into L2 at once, so that by the time
// the gather loop reaches it only the first round of loads still waits for DRAM.
#ifndef GRAB_SEARCH_PREFETCH_VEC
#define GRAB_SEARCH_PREFETCH_VEC 0
#endif
// 1: the lane that keeps a key (a possible future parent) prefetches that node's graph row into L2.
#ifndef GRAB_SEARCH_PREFETCH_ROW
#define GRAB_SEARCH_PREFETCH_ROW 0
#endif
#ifndef GRAB_RANK_MERGE_HALF
#define GRAB_RANK_MERGE_HALF 16
#endif
constexpr uint32_t kRankMergeHalf = GRAB_RANK_MERGE_HALF;  // per-warp kept keys up to which the merge is by rank (<= 16)

// Profiling build only (-DGRAB_SEARCH_PHASE_CLOCKS=1): SM cycles every warp spends in each phase of the loop, summed
// over all launches; read with grab_debug_search_phase_cycles(). Slots (warp 0: 0-7, warp 1: 8-15): start + seeds,
// gather, sort, first barrier, merge + pick, second barrier, table reset + expand, results.
#ifndef GRAB_SEARCH_PHASE_CLOCKS
#define GRAB_SEARCH_PHASE_CLOCKS 0
#endif
#if GRAB_SEARCH_PHASE_CLOCKS
__device__ unsigned long long g_phase_cycles[16];
#define GRAB_PHASE(i)                                                    \
  do {                                                                   \
    const long long now_ = clock64();                                    \
    if (lane == 0) s_phase[(i) + 8 * warp] += static_cast<uint32_t>(now_ - t_phase); \
    t_phase = now_;                                                      \
  } while (0)
#else
#define GRAB_PHASE(i)
#endif

__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  const char* c = static_cast<const char*>(p);
  for (uint32_t b = 0; b < bytes; b += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + b));
}

template <int METRIC, int CPL, int R>
__global__ void __launch_bounds__(kSearchThreads, GRAB_SEARCH2_CTAS_PER_SM)
graph_search_split_kernel(const SearchKernelArgs a) {
  static_assert(kSearchThreads == 64, "two warps per query");
  // vectors in flight per team: a 96-d row is three float4 per lane, so three of them cost the registers two 128-d
  // rows do, and a warp's survivors take a third fewer round trips to memory
  constexpr int U = CPL == 3 ? GRAB_SEARCH_UNROLL_96 : kSearchUnroll;
  constexpr uint32_t M = 32u * R;  // list length
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* queue = reinterpret_cast<uint64_t*>(smem_raw);                 // [M] sorted itopk list
  uint64_t* wkeys = queue + M;                                             // [2][wcap] kept keys per warp
  float* q_smem = reinterpret_cast<float*>(wkeys + 2 * a.ckeys_cap);       // [dim]
  uint32_t* wcand = reinterpret_cast<uint32_t*>(q_smem + a.dim);           // [2][wcap] survivor ids per warp
  uint32_t* parents = wcand + 2 * a.ckeys_cap;                             // [width]
  uint32_t* hash = parents + ((a.width + 3) & ~3u);                        // [2^bitlen] (if local)
  __shared__ uint32_t s_nparents, s_kept[2], s_inserted[2];
  __shared__ uint32_t s_stat[6];  // iterations, parents, edges, distances, seeds, resets (this query)

  // several CTAs per query: CTA `part` of query qi walks from its own share of the seeds with its own list; all of
  // them share ONE visited table in global memory, so a node is evaluated by exactly one of them and the lists are
  // disjoint; a merge of the sorted lists follows the launch
  const uint32_t parts = a.parts;
  const uint64_t qi = parts > 1 ? blockIdx.x / parts : blockIdx.x;
  const uint32_t part = parts > 1 ? static_cast<uint32_t>(blockIdx.x - qi * parts) : 0u;
  if (qi >= a.nq) return;
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5, lane = tid & 31u;
#if GRAB_SEARCH_PHASE_CLOCKS
  __shared__ uint32_t s_phase[16];
  if (tid < 16) s_phase[tid] = 0;
  long long t_phase = clock64();
#endif
  const int lane8 = tid & (kTeam - 1);
  const uint32_t wteam = lane / kTeam;  // team inside the warp, 0..3
  const uint32_t wcap = a.ckeys_cap;
  const uint32_t hsize = 1u << a.hash_bitlen;
  if (a.global_hash) hash = a.global_hash + qi * hsize;
  uint64_t* my_keys = wkeys + warp * wcap;
  uint32_t* my_cand = wcand + warp * wcap;

  for (uint32_t i = tid; i < a.dim / 4; i += kSearchThreads)
    reinterpret_cast<float4*>(q_smem)[i] = __ldg(reinterpret_cast<const float4*>(a.queries + qi * a.dim) + i);
  for (uint32_t i = tid; i < M; i += kSearchThreads) queue[i] = kMaxKey;
  if (parts == 1)  // a shared table is cleared by the host before the launch
    for (uint32_t i = tid; i < hsize / 4; i += kSearchThreads)
      reinterpret_cast<uint4*>(hash)[i] = make_uint4(kInvalid, kInvalid, kInvalid, kInvalid);
  if (tid == 0) s_nparents = 0;
  if (tid < 6) s_stat[tid] = 0;

  uint64_t lo = 0, hi = 0;
  uint32_t mask = 0;
  if (a.filter_kind == GRAB_FILTER_TS_RANGE) {
    lo = a.lo ? a.lo[qi] : a.lo1;
    hi = a.hi ? a.hi[qi] : a.hi1;
  } else if (a.filter_kind == GRAB_FILTER_LABELS) {
    mask = a.masks ? a.masks[qi] : a.mask1;
  }
  uint32_t wbeg = 0, wend = 0;
  const bool by_window = a.windows != nullptr && a.filter_kind == GRAB_FILTER_TS_RANGE;
  if (a.windows) {
    wbeg = a.windows[qi * 4];
    wend = a.windows[qi * 4 + 1];
    if (wend < wbeg) wend = wbeg;
  }
  auto passes = [&](uint32_t id) -> bool {
    if (by_window) return id >= wbeg && id < wend;
    if (a.filter_kind == GRAB_FILTER_TS_RANGE) {
      const uint64_t t = __ldg(a.ts + id);
      return t >= lo && t < hi;
    }
    if (a.filter_kind == GRAB_FILTER_LABELS) return (mask >> __ldg(a.labels + id)) & 1u;
    return true;
  };
  const uint32_t lt_mask = (1u << lane) - 1u;
  __syncthreads();

  // ---- seeds (compute_distance.cuh:204-269): provided ids, else pseudo-random ids; every warp keeps its own ----
  uint32_t ncand = 0;                     // warp-uniform: survivors in my_cand
  uint32_t inserted_total = 0;            // warp-uniform: ids this warp put into the visited set since the last clear
  {
    const uint32_t wlen = wend - wbeg;
    const bool generated_only = (a.seeds == nullptr);
    const bool by_label_range = a.filter_kind == GRAB_FILTER_LABELS && a.label_offsets != nullptr && mask != 0;
    const uint32_t nlab = __popc(mask);
    const uint32_t attempts = (generated_only && !a.windows && !by_label_range && a.filter_kind != GRAB_FILTER_NONE &&
                               a.filter_kind != GRAB_FILTER_PREFIX) ? 4 * a.num_seeds : a.num_seeds;
    // every provided / window-drawn attempt may be taken; blind draws (4 attempts per seed) stop at the quota
    const uint32_t my_quota = attempts == a.num_seeds ? wcap : (a.num_seeds + 1 - warp) / 2;
    const uint32_t my_attempts = (attempts + parts - 1 - part) / parts;  // attempts part, part + parts, ...
    for (uint32_t i0 = 0; i0 < my_attempts; i0 += kSearchThreads) {
      const uint32_t i = i0 + tid < my_attempts ? (i0 + tid) * parts + part : attempts;
      uint32_t id = kInvalid;
      if (i < attempts) {
        if (a.seeds && i < a.seeds_per_query) id = a.seeds[qi * a.seeds_per_query + i];
        if (id >= a.n) {
          if (a.windows) {
            id = wlen ? wbeg + static_cast<uint32_t>(mix64(a.seed ^ (qi * 0x9e3779b97f4a7c15ull + i)) % wlen) : kInvalid;
          } else if (by_label_range) {
            uint32_t m = mask;
            for (uint32_t skip = i % nlab; skip > 0; --skip) m &= m - 1;
            const uint32_t lab = __ffs(m) - 1;
            const uint32_t lb = a.label_offsets[lab], le = a.label_offsets[lab + 1];
            id = le > lb ? lb + static_cast<uint32_t>(mix64(a.seed ^ (qi * 0x9e3779b97f4a7c15ull + i)) % (le - lb))
                         : kInvalid;
          } else {
            id = static_cast<uint32_t>(((a.seed | 1ull) * static_cast<uint64_t>(i + 1)) % a.n);
          }
        }
      }
      const bool take = id < a.n && passes(id) && hash_insert(hash, a.hash_bitlen, id);
      const uint32_t vote = __ballot_sync(0xFFFFFFFFu, take);
      const uint32_t pos = ncand + __popc(vote & lt_mask);
      if (take && pos < my_quota) {
        my_cand[pos] = id;
        if (GRAB_SEARCH_PREFETCH_VEC) prefetch_l2(a.data + static_cast<size_t>(id) * a.dim, a.dim * 4);
      }
      ncand += __popc(vote);
    }
    inserted_total = ncand;
    if (ncand > my_quota) ncand = my_quota;
    if (a.stats && lane == 0) atomicAdd(&s_stat[4], ncand);
  }
  __syncwarp();
  GRAB_PHASE(0);

  uint32_t iter = 0;
  for (;;) {
    // ---- this warp's survivors: 4 teams, vectors gathered with 16-byte loads; a key is kept only if it beats
    //      the current worst entry of the list ----
    const uint64_t worst = queue[M - 1];
    uint32_t nkeep = 0;  // warp-uniform
    for (uint32_t j0 = 0; j0 < ncand; j0 += 4 * U) {
      uint32_t id[U];
      bool ok[U];
      float acc[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t j = j0 + u * 4 + wteam;
        ok[u] = j < ncand;
        id[u] = ok[u] ? my_cand[j] : 0;
        acc[u] = 0.0f;
      }
      if (CPL > 0) {
        float4 x[U][CPL > 0 ? CPL : 1];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int c = 0; c < CPL; ++c)
            if (ok[u]) x[u][c] = ldg_f4(a.data + static_cast<size_t>(id[u]) * a.dim + 4 * (lane8 + kTeam * c));
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int c = 0; c < CPL; ++c)
            if (ok[u])
              acc[u] = accum4<METRIC>(acc[u], *reinterpret_cast<const float4*>(q_smem + 4 * (lane8 + kTeam * c)), x[u][c]);
      } else {
        const uint32_t nchunk = a.dim / 4;
        for (uint32_t c0 = lane8; c0 < nchunk; c0 += 4 * kTeam) {
          float4 x[U][4];
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t c = c0 + i * kTeam;
              if (ok[u] && c < nchunk) x[u][i] = ldg_f4(a.data + static_cast<size_t>(id[u]) * a.dim + 4 * c);
            }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t c = c0 + i * kTeam;
            if (c < nchunk) {
              const float4 qv = *reinterpret_cast<const float4*>(q_smem + 4 * c);
#pragma unroll
              for (int u = 0; u < U; ++u)
                if (ok[u]) acc[u] = accum4<METRIC>(acc[u], qv, x[u][i]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float d = team_reduce<METRIC>(acc[u]);
        const uint64_t key = make_skey(d, id[u]);
        const bool keep = lane8 == 0 && ok[u] && key < worst;
        const uint32_t vote = __ballot_sync(0xFFFFFFFFu, keep);
        if (keep) {
          my_keys[nkeep + __popc(vote & lt_mask)] = key;
          if (GRAB_SEARCH_PREFETCH_ROW) prefetch_l2(a.graph + static_cast<size_t>(id[u]) * a.deg, a.active_deg * 4);
        }
        nkeep += __popc(vote);
      }
    }
    __syncwarp();
    GRAB_PHASE(1);
    // ---- a handful of kept keys (the usual case after the first iterations) is merged by rank and needs no
    //      sort; more are sorted here, by this warp, in registers ----
    if (nkeep > kRankMergeHalf) {
      if (nkeep <= 32) warp_sort_regs<1>(my_keys, nkeep, lane);
      else if (nkeep <= 64) warp_sort_regs<2>(my_keys, nkeep, lane);
      else if (nkeep <= 128) warp_sort_regs_128(my_keys, nkeep, lane);
      else warp_sort_regs_256(my_keys, nkeep, lane);
    }
    if (lane == 0) {
      s_kept[warp] = nkeep < M ? nkeep : M;
      s_inserted[warp] = inserted_total;
    }
    GRAB_PHASE(2);
    __syncthreads();
    GRAB_PHASE(3);

    // ---- warp 0: fold both runs into the list, pick up to `width` unexpanded parents, best first
    //      (search.cu:38-107), while the list is in registers ----
    const bool last = iter >= a.max_iter;
    if (warp == 0) {
      const uint32_t n0 = s_kept[0], n1 = s_kept[1];
      uint64_t t[R];
      if (n0 + n1 > 0 && n0 <= kRankMergeHalf && n1 <= kRankMergeHalf) {
        // neither warp sorted: lane j holds candidate j of the concatenation
        uint64_t cand = kMaxKey;
        if (lane < n0) cand = wkeys[lane];
        else if (lane < n0 + n1) cand = wkeys[wcap + lane - n0];
        warp_merge_by_rank<R>(queue, cand, n0 + n1, lane, t);
      } else if (n0 + n1 > 0) {
        // one run is sorted already; a short one that was left unsorted is sorted now
        if (n0 > 1 && n0 <= kRankMergeHalf) warp_sort_regs<1>(wkeys, n0, lane);
        if (n1 > 1 && n1 <= kRankMergeHalf) warp_sort_regs<1>(wkeys + wcap, n1, lane);
        __syncwarp();
        warp_merge_runs_regs<R>(queue, wkeys, n0, wkeys + wcap, n1, lane, t);
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) t[r] = queue[lane + 32u * r];
      }
      uint32_t found = 0;
      if (!last) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const bool fresh = t[r] != kMaxKey && !skey_expanded(t[r]);
          const uint32_t vote = __ballot_sync(0xFFFFFFFFu, fresh);
          if (fresh && found < (GRAB_SEARCH_PREFETCH ? 2u : 1u) * a.width) {
            const uint32_t rank = found + __popc(vote & lt_mask);
            if (rank < a.width) {
              parents[rank] = skey_id(t[r]);
              t[r] |= 1ull;
            } else if (GRAB_SEARCH_PREFETCH && rank < 2 * a.width) {
              // the runners-up are the likely parents of the NEXT iteration: pull their graph rows into L2 now
              const char* row = reinterpret_cast<const char*>(a.graph + static_cast<size_t>(skey_id(t[r])) * a.deg);
              for (uint32_t b = 0; b < a.active_deg * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + b));
            }
          }
          found += __popc(vote);
        }
        if (found > a.width) found = a.width;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) queue[lane + 32u * r] = t[r];
      if (lane == 0) s_nparents = found;
    }
    GRAB_PHASE(4);
    __syncthreads();
    GRAB_PHASE(5);

    // ---- visited table half full: clear and re-seed from the current list ----
    if (parts == 1 && s_inserted[0] + s_inserted[1] > hsize / 2) {  // uniform (a shared table is sized never to fill)
      for (uint32_t i = tid; i < hsize; i += kSearchThreads) hash[i] = kInvalid;
      __syncthreads();
      uint32_t kept = 0;
      for (uint32_t i = tid; i < M; i += kSearchThreads) {
        const uint64_t key = queue[i];
        if (key != kMaxKey) { hash_insert(hash, a.hash_bitlen, skey_id(key)); ++kept; }
      }
      inserted_total = __reduce_add_sync(0xFFFFFFFFu, kept);
      if (tid == 0) s_stat[5] += 1;
      __syncthreads();
    }
    const uint32_t nparents = s_nparents;
    if (last || nparents == 0) break;

    // ---- expand: flattened (parent, column) edges, thread t takes edges t, t+64, ...: neighbour id -> filter
    //      -> visited set -> this warp's survivor list ----
    ncand = 0;
    const uint32_t total_edges = nparents * a.active_deg;
    uint32_t my_edges = 0;
    for (uint32_t e0 = 0; e0 < total_edges; e0 += 4 * kSearchThreads) {
      uint32_t nbv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        // inside every group of 64 consecutive edges warp 0 takes the even and warp 1 the odd ones, so that both
        // warps see the same mix of local and cross-bucket columns (their survivor counts stay balanced)
        const uint32_t e = e0 + u * kSearchThreads + 2 * lane + warp;
        nbv[u] = kInvalid;
        if (e < total_edges) {
          const uint32_t p = a.inv_active_deg ? __umulhi(e, a.inv_active_deg) : e;  // e / active_deg
          const uint32_t col = e - p * a.active_deg;
          nbv[u] = __ldg(a.graph + static_cast<size_t>(parents[p]) * a.deg + col);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t nb = nbv[u];
        const bool valid = nb < a.n;
        my_edges += valid;
        const bool take = valid && passes(nb) && hash_insert(hash, a.hash_bitlen, nb);
        const uint32_t vote = __ballot_sync(0xFFFFFFFFu, take);
        if (take) {
          my_cand[ncand + __popc(vote & lt_mask)] = nb;
          if (GRAB_SEARCH_PREFETCH_VEC) prefetch_l2(a.data + static_cast<size_t>(nb) * a.dim, a.dim * 4);
        }
        ncand += __popc(vote);
      }
    }
    inserted_total += ncand;
    if (a.stats) {
      my_edges = __reduce_add_sync(0xFFFFFFFFu, my_edges);
      if (lane == 0) { atomicAdd(&s_stat[2], my_edges); atomicAdd(&s_stat[3], ncand); }
      if (tid == 0) { s_stat[0] += 1; s_stat[1] += nparents; }
    }
    ++iter;
    __syncwarp();
    GRAB_PHASE(6);
  }

  // ---- results: ascending (dist,id); id = local*scale + offset; empty slots are -1 ----
  for (uint32_t i = tid; i < a.k; i += kSearchThreads) {
    const uint64_t key = queue[i];
    const bool empty = key == kMaxKey;
    const uint64_t gid = static_cast<uint64_t>(skey_id(key)) * a.id_scale + a.id_offset;
    if (a.out_ids) a.out_ids[qi * a.k + i] = empty ? -1 : static_cast<int64_t>(gid);
    if (a.out_dists) a.out_dists[qi * a.k + i] = empty ? kFltMax : key_dist(key);
    // several CTAs per query: run `part` of query qi, laid out [part][query][k] for the merge of sorted runs
    if (a.out_keys) a.out_keys[(part * a.nq + qi) * a.k + i] = empty ? kMaxKey : ((key & 0xFFFFFFFF00000000ull) | gid);
  }
  if (a.stats) {
    __syncthreads();
    if (tid < 6) atomicAdd(&a.stats[tid], static_cast<unsigned long long>(s_stat[tid]));
  }
#if GRAB_SEARCH_PHASE_CLOCKS
  GRAB_PHASE(7);
  __syncthreads();
  if (tid < 16) atomicAdd(&g_phase_cycles[tid], static_cast<unsigned long long>(s_phase[tid]));
#endif
}

#if GRAB_SEARCH_PHASE_CLOCKS
extern "C" int grab_debug_search_phase_cycles(unsigned long long* out16, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out16, g_phase_cycles, sizeof(unsigned long long) * 16);
  if (e == cudaSuccess && reset) {
    unsigned long long zero[16] = {};
    e = cudaMemcpyToSymbol(g_phase_cycles, zero, sizeof(zero));
  }
  return e == cudaSuccess ? 0 : -1;
}
#endif

template <int METRIC, int R>
static cudaError_t launch_search_split(const SearchKernelArgs& a, size_t smem, cudaStream_t st) {
#define GRAB_SPLIT_LAUNCH(CPL)                                                                        \
  do {                                                                                                \
    cudaError_t e = cudaFuncSetAttribute(graph_search_split_kernel<METRIC, CPL, R>,                   \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    if (e != cudaSuccess) return e;                                                                   \
    graph_search_split_kernel<METRIC, CPL, R><<<(unsigned)(a.nq * a.parts), kSearchThreads, smem, st>>>(a);       \
  } while (0)
  if (a.dim == 96) GRAB_SPLIT_LAUNCH(3);
  else if (a.dim == 128) GRAB_SPLIT_LAUNCH(4);
  else GRAB_SPLIT_LAUNCH(0);
#undef GRAB_SPLIT_LAUNCH
  return cudaGetLastError();
}

// 0 = the shared-list kernel, 1 = the warp-split kernel where it applies (default).  GRAB_SEARCH_KERNEL=shared in
// the environment selects the former for comparisons.
static int search_kernel_choice() {
  static const int choice = [] {
    const char* v = getenv("GRAB_SEARCH_KERNEL");
    return (v && strcmp(v, "shared") == 0) ? 0 : 1;
  }();
  return choice;
}

static bool hash_bitlen_literal() {
  static const bool on = [] {
    const char* v = getenv("GRAB_SEARCH_HASH_EXACT");
    return v && v[0] == '1';
  }();
  return on;
}

template <int METRIC>
static cudaError_t launch_search(const SearchKernelArgs& a, size_t smem, cudaStream_t st) {
#define GRAB_SEARCH_LAUNCH(CPL)                                                                   \
  do {                                                                                            \
    cudaError_t e = cudaFuncSetAttribute(graph_search_kernel<METRIC, CPL>,                        \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return e;                                                               \
    graph_search_kernel<METRIC, CPL><<<(unsigned)a.nq, kSearchThreads, smem, st>>>(a);            \
  } while (0)
  if (a.dim == 96) GRAB_SEARCH_LAUNCH(3);
  else if (a.dim == 128) GRAB_SEARCH_LAUNCH(4);
  else GRAB_SEARCH_LAUNCH(0);
#undef GRAB_SEARCH_LAUNCH
  return cudaGetLastError();
}

// One warp per query: id window [first id with ts >= lo, first id with ts >= hi).
__global__ void ts_window4_kernel(const uint64_t* __restrict__ ts, uint64_t n,
                                  const uint64_t* __restrict__ lo, const uint64_t* __restrict__ hi,
                                  uint64_t lo1, uint64_t hi1, uint64_t nq,
                                  uint32_t* __restrict__ windows) {
  const uint64_t qi = (blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (qi >= nq) return;  // whole warps leave together
  const uint32_t wb = warp_lower_bound_u64(ts, static_cast<uint32_t>(n), lo ? lo[qi] : lo1);
  const uint32_t we = warp_lower_bound_u64(ts, static_cast<uint32_t>(n), hi ? hi[qi] : hi1);
  if (lane_id() == 0) *reinterpret_cast<uint4*>(windows + qi * 4) = make_uint4(wb, we, 0u, 0u);
}

// ---------------------------------------------------------------------------------------------------------
// Several CTAs per query (for batches that would leave most of the GPU idle with one CTA each).  The caller's
// (itopk, search_width, max_iterations) describe the single-CTA search; its budget of search_width * max_iterations
// expansions is spread over `parts` CTAs that each keep a short list (64 or 128 entries), expand
// max(1, search_width / parts) parents per iteration and share one visited table in global memory, sized so that
// it never fills (no reset).  The merge of the parts' sorted lists is the result.  Not the reference's algorithm
// (it has one CTA per query only, cagra_opt.cu:1394): results are valid top-k lists of evaluated nodes, checked
// on recall, not bit for bit.
// ---------------------------------------------------------------------------------------------------------
int merge_sorted_keys_impl(const uint64_t* d_keys, uint64_t nq, uint32_t parts, uint32_t kp, uint32_t k,
                           int64_t* d_out_ids, float* d_out_dists, uint64_t* d_out_keys, cudaStream_t st);

struct MultiPlan {
  uint32_t parts = 1, width = 0, iters = 0, list = 0, nseeds = 0, hash_bitlen = 0;
  size_t hash_off = 0, keys_off = 0, bytes = 0;  // workspace layout (after the id windows)
};

static uint32_t base_itopk(const grab_search_args* g) {
  uint32_t itopk = g->k > g->params.itopk_size ? g->k : g->params.itopk_size;
  const uint32_t floor_ = g->filter.kind == GRAB_FILTER_PREFIX ? 128u : 64u;
  return itopk < floor_ ? floor_ : itopk;
}

static uint32_t base_nseeds(const grab_search_args* g, uint32_t itopk) {
  const uint32_t spq = g->d_seeds ? g->seeds_per_query : 0;
  uint32_t nseeds;
  if (g->filter.kind == GRAB_FILTER_NONE) nseeds = spq > 32 ? spq : 32;
  else if (g->d_seeds) nseeds = spq;
  else nseeds = itopk / 4 > 32 ? itopk / 4 : 32;
  return nseeds > itopk ? itopk : nseeds;
}

static size_t windows_bytes(uint64_t nq) { return ((sizeof(uint32_t) * 4 * nq + 255) / 256) * 256; }

static MultiPlan plan_multi(const grab_search_args* g) {
  MultiPlan p;
  uint32_t parts = g->ctas_per_query;
  const uint32_t W = g->params.search_width ? g->params.search_width : 1;
  const uint32_t budget = W * (g->params.max_iterations ? g->params.max_iterations : 1);  // expansions per query
  if (parts == GRAB_CTAS_AUTO) {
    // Only long walks are split (a shared table in global memory, its clearing and the merge of the runs cost more
    // than a short walk gains: 1 000 queries of 40 expansions take 0.097 ms with one CTA each, 0.118 ms with two), over
    // at most 16 CTAs with at least 16 expansions each (1 query, 300 expansions: 0.75 ms with one CTA, 0.26 / 0.15 /
    // 0.40 ms with 4 / 16 / 64), and only while the batch leaves room on the GPU (148 SMs x 14 resident CTAs).
    const uint64_t room = g->nq ? 2072 / g->nq : 1;
    parts = budget < 64 ? 1u : static_cast<uint32_t>(room < 16 ? room : 16);
    if (parts > budget / 16) parts = budget / 16;
  }
  if (parts > 64) parts = 64;  // the merge takes up to 64 runs
  if (parts < 2 || g->k > 128 || search_kernel_choice() != 1) return p;
  p.parts = parts;
  p.width = W / parts ? W / parts : 1;
  p.iters = (budget + parts * p.width - 1) / (parts * p.width);
  if (p.iters < 2) p.iters = 2;
  p.list = g->k <= 64 ? 64 : 128;
  const uint32_t deg = g->filter.kind == GRAB_FILTER_PREFIX ? g->filter.active_degree : g->graph_degree;
  uint32_t nseeds = base_nseeds(g, base_itopk(g));
  if (!g->d_seeds && nseeds < 8 * parts) nseeds = 8 * parts;  // generated seeds: at least 8 per CTA
  p.nseeds = nseeds;
  const uint64_t inserts = 4ull * nseeds + static_cast<uint64_t>(parts) * p.iters * p.width * deg;
  uint32_t bits = 11;
  while (bits < 22 && (1ull << bits) < 2 * inserts) ++bits;
  p.hash_bitlen = bits;
  p.hash_off = windows_bytes(g->nq);
  p.keys_off = p.hash_off + sizeof(uint32_t) * (size_t(1) << bits) * g->nq;
  p.bytes = p.keys_off + sizeof(uint64_t) * parts * g->nq * g->k + 256;
  return p;
}

// Launcher rules restated from the reference: itopk = max(k, itopk) with floor 64
// (cagra_opt.cu:1126-1129, :1352-1355) or 128 for the bucket search (:1242-1243); seeds
// evaluated = clamp(max(32, provided), itopk) unfiltered (:1150-1151) or min(provided, itopk)
// filtered (:1276-1277, :1386-1387); with no seeds given a filtered search draws
// max(32, itopk/4) of its own (the class layer's rule, cagraIndexOpt.cu:441).
int graph_search_impl(const grab_search_args* g) {
  GRAB_REQUIRE(g, "graph_search: null args");
  GRAB_REQUIRE(g->d_dataset && g->d_graph && g->d_queries && ((g->d_out_ids && g->d_out_dists) || g->d_out_keys),
               "graph_search: null pointer (the reference throws \"Graph is null!\", cagra_opt.cu:1123)");
  GRAB_REQUIRE(g->dim >= 4 && g->dim % 4 == 0, "graph_search: dim %u must be a multiple of 4", g->dim);
  GRAB_REQUIRE(g->n >= 1 && g->n < (1ull << 31), "graph_search: n must be in [1, 2^31)");
  GRAB_REQUIRE(g->k >= 1 && g->k <= 1024, "graph_search: k %u outside [1,1024]", g->k);
  GRAB_REQUIRE(g->graph_degree >= 1 && g->graph_degree <= 512, "graph_search: bad graph degree %u",
               g->graph_degree);
  GRAB_REQUIRE(g->metric == GRAB_METRIC_L2 || g->metric == GRAB_METRIC_IP, "graph_search: bad metric");
  GRAB_REQUIRE(g->params.search_width >= 1 && g->params.search_width <= 64,
               "graph_search: search_width %u outside [1,64]", g->params.search_width);
  GRAB_REQUIRE(g->params.hash_bitlen >= 8 && g->params.hash_bitlen <= 20,
               "graph_search: hash_bitlen %u outside [8,20]", g->params.hash_bitlen);
  if (g->nq == 0) return GRAB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(g->stream);
  const grab_filter& f = g->filter;

  SearchKernelArgs a{};
  a.data = g->d_dataset; a.n = g->n; a.dim = g->dim; a.graph = g->d_graph;
  a.deg = g->graph_degree; a.active_deg = g->graph_degree;
  a.queries = g->d_queries; a.nq = g->nq; a.k = g->k;
  a.width = g->params.search_width; a.max_iter = g->params.max_iterations;
  a.hash_bitlen = g->params.hash_bitlen;
  a.seeds = g->d_seeds; a.seeds_per_query = g->d_seeds ? g->seeds_per_query : 0;
  a.seed = g->seed; a.filter_kind = f.kind;
  a.out_ids = g->d_out_ids; a.out_dists = g->d_out_dists; a.out_keys = g->d_out_keys;
  a.id_scale = g->id_scale ? g->id_scale : 1; a.id_offset = g->id_offset;
  GRAB_REQUIRE(!a.out_keys || (g->n - 1) * a.id_scale + a.id_offset < (1ull << 32),
               "graph_search: d_out_keys holds 32-bit result ids, (n-1)*id_scale+id_offset does not fit");
  a.stats = reinterpret_cast<unsigned long long*>(g->d_stats);

  const MultiPlan mp = plan_multi(g);
  GRAB_REQUIRE(mp.parts > 1 || g->ctas_per_query < 2 || g->ctas_per_query == GRAB_CTAS_AUTO,
               "graph_search: ctas_per_query %u needs k <= 128 (k = %u) and the warp-split kernel", g->ctas_per_query, g->k);
  uint32_t itopk = g->k > g->params.itopk_size ? g->k : g->params.itopk_size;
  uint32_t floor_ = 64;
  bool need_window = false;
  switch (f.kind) {
    case GRAB_FILTER_NONE: break;
    case GRAB_FILTER_PREFIX:
      GRAB_REQUIRE(f.active_degree >= 1 && f.active_degree <= g->graph_degree,
                   "graph_search: active_degree %u outside [1,%u]", f.active_degree, g->graph_degree);
      a.active_deg = f.active_degree;
      floor_ = 128;
      break;
    case GRAB_FILTER_TS_RANGE:
      GRAB_REQUIRE(f.d_ts, "graph_search: ts filter without d_ts");
      GRAB_REQUIRE((f.d_lo == nullptr) == (f.d_hi == nullptr),
                   "graph_search: d_lo and d_hi must both be given or both NULL");
      a.ts = f.d_ts; a.lo = f.d_lo; a.hi = f.d_hi; a.lo1 = f.lo; a.hi1 = f.hi;
      need_window = f.ts_sorted != 0;
      break;
    case GRAB_FILTER_LABELS:
      GRAB_REQUIRE(f.d_labels, "graph_search: label filter without d_labels");
      a.labels = f.d_labels; a.masks = f.d_masks; a.mask1 = f.mask;
      a.label_offsets = f.d_label_offsets;  // also fills holes (ids >= n) in a provided seed list
      break;
    default:
      set_last_error("graph_search: unknown filter kind %d", f.kind);
      return GRAB_ERR_INVALID_ARGUMENT;
  }
  if (itopk < floor_) itopk = floor_;
  a.itopk = itopk;
  uint32_t nseeds;
  if (f.kind == GRAB_FILTER_NONE) nseeds = a.seeds_per_query > 32 ? a.seeds_per_query : 32;
  else if (g->d_seeds) nseeds = a.seeds_per_query;
  else nseeds = itopk / 4 > 32 ? itopk / 4 : 32;
  if (nseeds > itopk) nseeds = itopk;
  a.parts = mp.parts;
  if (mp.parts > 1) {
    a.width = mp.width; a.max_iter = mp.iters; a.hash_bitlen = mp.hash_bitlen;
    itopk = a.itopk = mp.list;
    nseeds = mp.nseeds;
  }
  a.num_seeds = nseeds;
  a.cand_cap = a.width * a.deg > itopk ? a.width * a.deg : itopk;
  a.cand_cap = (a.cand_cap + 3) & ~3u;
  a.sort_cap = next_pow2(itopk);  // the itopk list is kept at a power-of-two length (>= the requested itopk)
  if (a.sort_cap < 64) a.sort_cap = 64;
  a.ckeys_cap = next_pow2(a.cand_cap);
  if (a.ckeys_cap < 32) a.ckeys_cap = 32;

  // hash_bitlen is an upper bound for the per-CTA table: 2^11 entries (8 KB) keep 14 CTAs resident per SM, and the
  // reset-when-half-full rule makes a small table only cost some repeated evaluations -- measured at 1M x 128, 10 000
  // queries: itopk 256 / width 6 / 50 iterations 12.1 ms with 2^13, 8.3 ms with 2^12, 7.6 ms with 2^11 (23 % more
  // distance evaluations, same recall); itopk 128 / width 4: 3.4 / 2.5 / 2.2 ms.  The table keeps at least 8 slots
  // per list entry, so that a reset (which re-inserts the list) leaves room.  GRAB_SEARCH_HASH_EXACT=1 in the
  // environment takes hash_bitlen literally.
  if (mp.parts == 1 && a.hash_bitlen <= 13 && !hash_bitlen_literal()) {
    uint32_t bits = 11;
    while ((1u << bits) < 8 * a.sort_cap && bits < 13) ++bits;
    if (a.hash_bitlen > bits) a.hash_bitlen = bits;
  }
  const bool local_hash = a.hash_bitlen <= 13 && mp.parts == 1;
  const size_t hash_bytes = sizeof(uint32_t) * (size_t(1) << a.hash_bitlen);
  // warp-split kernel: lists of 64 / 128 entries, at most 256 candidates per warp and iteration
  const uint32_t blind = (!g->d_seeds && !need_window && !(f.kind == GRAB_FILTER_LABELS && f.d_label_offsets) &&
                          f.kind != GRAB_FILTER_NONE && f.kind != GRAB_FILTER_PREFIX) ? 1u : 0u;
  const uint32_t warp_edges = (a.width * a.active_deg + kSearchThreads - 1) / kSearchThreads * 32;
  const uint32_t part_seeds = (nseeds + mp.parts - 1) / mp.parts;  // attempts of one CTA
  const uint32_t warp_seeds = blind ? (nseeds + 1) / 2 : (part_seeds + kSearchThreads - 1) / kSearchThreads * 32;
  uint32_t wcap = next_pow2(warp_edges > warp_seeds ? warp_edges : warp_seeds);
  if (wcap < 32) wcap = 32;
  // (a 256-entry list on this kernel -- 8 list registers per lane, 8 CTAs per SM -- was measured level with the
  // shared-list kernel, 7.69 against 7.57 ms at itopk 256 / width 6 / 50 iterations, and is left to the latter)
  const bool split = search_kernel_choice() == 1 && (a.sort_cap == 64 || a.sort_cap == 128) && wcap <= 256;
  a.inv_active_deg = a.active_deg > 1 ? static_cast<uint32_t>(((1ull << 32) + a.active_deg - 1) / a.active_deg) : 0;
  size_t smem = sizeof(uint64_t) * (a.sort_cap + a.ckeys_cap) + sizeof(float) * a.dim + sizeof(uint32_t) * a.cand_cap +
                sizeof(uint32_t) * ((a.width + 3) & ~3u) + (local_hash ? hash_bytes : 0);
  if (split) {
    a.ckeys_cap = wcap;  // per-warp capacity of the kept-key and survivor lists
    smem = sizeof(uint64_t) * (a.sort_cap + 2 * wcap) + sizeof(float) * a.dim + sizeof(uint32_t) * 2 * wcap +
           sizeof(uint32_t) * ((a.width + 3) & ~3u) + (local_hash ? hash_bytes : 0);
  }
  if (smem > 200 * 1024) {
    set_last_error("graph_search: itopk %u, width %u, degree %u, dim %u need %zu bytes of shared memory",
                   itopk, a.width, a.deg, a.dim, smem);
    return GRAB_ERR_UNSUPPORTED;
  }
  GRAB_REQUIRE(mp.parts == 1 || split, "graph_search: ctas_per_query %u: width %u x degree %u does not fit the "
               "warp-split kernel", mp.parts, a.width, a.active_deg);
  const size_t need = mp.parts > 1 ? mp.bytes : grab_graph_search_workspace_bytes(g->nq, a.hash_bitlen);
  ScopedDeviceBuffer own;
  void* ws = g->d_ws;
  if (!ws) {
    GRAB_CUDA_TRY(own.alloc(need));
    ws = own.ptr;
  } else if (g->ws_bytes < need) {
    set_last_error("graph_search: workspace %zu < %zu bytes", g->ws_bytes, need);
    return GRAB_ERR_WORKSPACE;
  }
  uint32_t* windows = static_cast<uint32_t*>(ws);
  if (need_window && f.d_id_windows) {
    a.windows = f.d_id_windows;  // left there by grab_route_seeds for these queries and this filter
  } else if (need_window) {
    ts_window4_kernel<<<(unsigned)((g->nq * 32 + 255) / 256), 256, 0, st>>>(f.d_ts, g->n, f.d_lo, f.d_hi,
                                                                           f.lo, f.hi, g->nq, windows);
    GRAB_CUDA_TRY(cudaGetLastError());
    a.windows = windows;
  }
  if (!local_hash) a.global_hash = reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + windows_bytes(g->nq));
  uint64_t* part_keys = nullptr;
  if (mp.parts > 1) {
    // the shared visited tables start empty; every CTA leaves its sorted top-k as packed keys for the merge
    GRAB_CUDA_TRY(cudaMemsetAsync(a.global_hash, 0xFF, mp.keys_off - mp.hash_off, st));
    part_keys = reinterpret_cast<uint64_t*>(static_cast<char*>(ws) + mp.keys_off);
    a.out_keys = part_keys; a.out_ids = nullptr; a.out_dists = nullptr;
  }
  cudaError_t e;
  if (split && a.sort_cap == 64)
    e = g->metric == GRAB_METRIC_L2 ? launch_search_split<GRAB_METRIC_L2, 2>(a, smem, st)
                                    : launch_search_split<GRAB_METRIC_IP, 2>(a, smem, st);
  else if (split)
    e = g->metric == GRAB_METRIC_L2 ? launch_search_split<GRAB_METRIC_L2, 4>(a, smem, st)
                                    : launch_search_split<GRAB_METRIC_IP, 4>(a, smem, st);
  else
    e = g->metric == GRAB_METRIC_L2 ? launch_search<GRAB_METRIC_L2>(a, smem, st)
                                    : launch_search<GRAB_METRIC_IP>(a, smem, st);
  GRAB_CUDA_TRY(e);
  if (mp.parts > 1) {
    const int rc = merge_sorted_keys_impl(part_keys, g->nq, mp.parts, g->k, g->k, g->d_out_ids, g->d_out_dists,
                                          g->d_out_keys, st);
    if (rc != GRAB_OK) return rc;
  }
  if (own.ptr) GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  return GRAB_OK;
}

size_t graph_search_workspace_bytes_for(const grab_search_args* g) {
  const MultiPlan mp = plan_multi(g);
  return mp.parts > 1 ? mp.bytes : grab_graph_search_workspace_bytes(g->nq, g->params.hash_bitlen);
}

}  // namespace grab

extern "C" size_t grab_graph_search_workspace_bytes_for(const grab_search_args* args) {
  return args ? grab::graph_search_workspace_bytes_for(args) : 0;
}

extern "C" size_t grab_graph_search_workspace_bytes(uint64_t nq, uint32_t hash_bitlen) {
  size_t b = ((sizeof(uint32_t) * 4 * nq + 255) / 256) * 256 + 256;
  if (hash_bitlen > 13) b += sizeof(uint32_t) * (size_t(1) << hash_bitlen) * nq;
  return b;
}
