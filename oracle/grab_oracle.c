/*
 * grab_oracle.c -- CPU restatement of the GRAB-ANNS hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: it
 * is loaded by the test-suite, by the smoke check and by the CPU-baseline leg of
 * the benchmark, and by nothing else.  The shipped library never links, loads
 * or calls it and has no CPU fallback.
 *
 * Each function cites the reference file:line (paths inside hxlou/GRAB-ANNS)
 * whose algorithm it restates.  Integer / index work is restated exactly
 * (where the reference is racy -- atomics order -- the deterministic order
 * chosen here is stated).  Floating point uses ONE canonical fp32 summation
 * order ("team of 8 lanes, float4 chunks", see orc_dist below) so that the CUDA
 * kernels can reproduce distances bit for bit; compile with -ffp-contract=off.
 *
 * Pinning: the reference ships no stored golden outputs; what it does ship are
 * known-answer tests (bitonic sort == std::sort of pairs, hashmap success
 * counts, constant-vector kNN ideal neighbours, exact brute force).  The test
 * suite runs this file against those known answers, and against outputs of the
 * reference's own code compiled for the GPU (search, insert, prune / reverse /
 * merge, remote edges / reverse injection: tests/golden/reference_*.npz and the
 * live three-way tests).  Parts whose reference behaviour comes from libraries
 * that are not in the reference tree (FAISS IVF-PQ candidate sets, RAFT brute
 * force, FAISS HNSW) are "parity unpinned".
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_INVALID 0xFFFFFFFFu
#define ORC_MSB 0x80000000u
#define ORC_FLT_MAX 3.40282e38f

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* Canonical fp32 distance.                                                   */
/* Reference arithmetic: Sum (a-b)^2 with lane-strided partial sums and a     */
/* butterfly reduction (src/index/compute_distance.cuh:120-139) on the GPU,   */
/* sequential sum on the CPU (tests/test_cagra_auto.cu:48-50).  The canonical */
/* order used by this project: the vector is cut into float4 chunks; chunk c  */
/* belongs to lane (c mod 8); every lane accumulates its chunks in ascending  */
/* order, elements x,y,z,w in order, with a fused multiply-add; the 8 lane    */
/* sums are then combined by a butterfly at xor-offsets 4, 2, 1.              */
/* metric 0: squared L2.  metric 1: negative inner product.                   */
/* ------------------------------------------------------------------------- */
float orc_dist(const float* q, const float* x, uint32_t dim, int metric) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  uint32_t nchunk = dim / 4;
  for (uint32_t t = 0; t < 8; ++t) {
    float a = 0.0f;
    for (uint32_t c = t; c < nchunk; c += 8) {
      for (uint32_t e = 0; e < 4; ++e) {
        float qa = q[4 * c + e], xa = x[4 * c + e];
        if (metric == 0) {
          float d = qa - xa;
          a = fmaf(d, d, a);
        } else {
          a = fmaf(qa, xa, a);
        }
      }
    }
    acc[t] = a;
  }
  for (uint32_t off = 4; off > 0; off >>= 1) {
    float nxt[8];
    for (uint32_t t = 0; t < 8; ++t) nxt[t] = acc[t] + acc[t ^ off];
    memcpy(acc, nxt, sizeof(acc));
  }
  return metric == 0 ? acc[0] : -acc[0];
}

/* order-preserving map float -> uint32 (ascending), used for (dist,id) keys */
static inline uint32_t f2ord(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
static inline float ord2f(uint32_t o) {
  uint32_t b = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
  float f;
  memcpy(&f, &b, 4);
  return f;
}
uint64_t orc_make_key(float dist, uint32_t id) { return ((uint64_t)f2ord(dist) << 32) | id; }

static int cmp_u64(const void* a, const void* b) {
  uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
  return (x > y) - (x < y);
}

/* ------------------------------------------------------------------------- */
/* Exact filtered brute force.  tests/test_cagra_auto.cu:57-89                */
/* (compute_ground_truth_range): per query scan every j passing the filter,   */
/* keep the k smallest.  The reference's partial_sort leaves equal distances  */
/* unordered; here ties go to the lower id.                                   */
/* filter: ts != NULL -> lo[q] <= ts[j] < hi[q];                              */
/*         labels != NULL -> bit labels[j] of masks[q] set; both NULL: none.  */
/* Missing results are id -1, dist FLT_MAX.                                   */
/* ------------------------------------------------------------------------- */
void orc_exact_search(const float* data, uint64_t n, uint32_t dim, const uint64_t* ts,
                      const uint8_t* labels, const float* queries, uint64_t nq, uint32_t k,
                      const uint64_t* lo, const uint64_t* hi, const uint32_t* masks, int metric,
                      int canonical, int64_t* out_ids, float* out_dists) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t qi = 0; qi < (int64_t)nq; ++qi) {
    const float* q = queries + (size_t)qi * dim;
    uint64_t* heap = (uint64_t*)malloc(sizeof(uint64_t) * (k + 1)); /* max-heap of keys */
    uint32_t hs = 0;
    for (uint64_t j = 0; j < n; ++j) {
      if (ts && !(ts[j] >= lo[qi] && ts[j] < hi[qi])) continue;
      if (labels && !((masks[qi] >> labels[j]) & 1u)) continue;
      const float* x = data + (size_t)j * dim;
      float d;
      if (canonical) {
        d = orc_dist(q, x, dim, metric);
      } else { /* the reference's sequential order, tests/test_cagra_auto.cu:48-50 */
        float r = 0;
        if (metric == 0)
          for (uint32_t i = 0; i < dim; ++i) {
            float t = q[i] - x[i];
            r += t * t;
          }
        else {
          for (uint32_t i = 0; i < dim; ++i) r += q[i] * x[i];
          r = -r;
        }
        d = r;
      }
      uint64_t key = orc_make_key(d, (uint32_t)j);
      if (hs < k) {
        uint32_t c = hs++;
        heap[c] = key;
        while (c > 0 && heap[(c - 1) / 2] < heap[c]) {
          uint64_t t = heap[c];
          heap[c] = heap[(c - 1) / 2];
          heap[(c - 1) / 2] = t;
          c = (c - 1) / 2;
        }
      } else if (key < heap[0]) {
        heap[0] = key;
        uint32_t c = 0;
        for (;;) {
          uint32_t l = 2 * c + 1, r = l + 1, m = c;
          if (l < hs && heap[l] > heap[m]) m = l;
          if (r < hs && heap[r] > heap[m]) m = r;
          if (m == c) break;
          uint64_t t = heap[c];
          heap[c] = heap[m];
          heap[m] = t;
          c = m;
        }
      }
    }
    qsort(heap, hs, sizeof(uint64_t), cmp_u64);
    for (uint32_t i = 0; i < k; ++i) {
      if (i < hs) {
        out_ids[(size_t)qi * k + i] = (int64_t)(heap[i] & 0xFFFFFFFFu);
        out_dists[(size_t)qi * k + i] = ord2f((uint32_t)(heap[i] >> 32));
      } else {
        out_ids[(size_t)qi * k + i] = -1;
        out_dists[(size_t)qi * k + i] = ORC_FLT_MAX;
      }
    }
    free(heap);
  }
}

/* ------------------------------------------------------------------------- */
/* Warp bitonic sort of 32*N (key,val) pairs.  src/index/bitonic.cuh:53-111.  */
/* Element g lives in lane g/N register g%N ("blocked" layout,                */
/* src/index/search.cu:110-144).  The network is restated step for step:      */
/* every element looks at its partner g^stride and keeps the smaller or the   */
/* larger according to the direction of its size-block; equal keys are never  */
/* exchanged (bitonic.cuh:17,33).                                             */
/* ------------------------------------------------------------------------- */
void orc_warp_sort(float* keys, uint32_t* vals, uint32_t total, int asc) {
  float* nk = (float*)malloc(sizeof(float) * total);
  uint32_t* nv = (uint32_t*)malloc(sizeof(uint32_t) * total);
  for (uint32_t size = 2; size <= total; size <<= 1) {
    for (uint32_t stride = size / 2; stride > 0; stride >>= 1) {
      for (uint32_t g = 0; g < total; ++g) {
        uint32_t p = g ^ stride;
        int direction = ((g & size) == 0) != !asc;
        int want_min = (g < p) == direction;
        float k = keys[g], ok = keys[p];
        nk[g] = k;
        nv[g] = vals[g];
        if (k != ok && ((k < ok) != want_min)) {
          nk[g] = ok;
          nv[g] = vals[p];
        }
      }
      memcpy(keys, nk, sizeof(float) * total);
      memcpy(vals, nv, sizeof(uint32_t) * total);
    }
  }
  free(nk);
  free(nv);
}

/* ------------------------------------------------------------------------- */
/* Visited set.  src/index/hashmap.cuh:30-117: open addressing, linear probe, */
/* slot = (key ^ (key >> bitlen)) & mask, 0xFFFFFFFF = empty.  Returns 1 when */
/* the key was newly inserted, 0 when present or when the table is full.      */
/* ------------------------------------------------------------------------- */
int orc_hash_insert(uint32_t* table, uint32_t bitlen, uint32_t key) {
  uint32_t size = 1u << bitlen, mask = size - 1;
  uint32_t idx = (key ^ (key >> bitlen)) & mask;
  for (uint32_t i = 0; i < size; ++i) {
    if (table[idx] == ORC_INVALID) {
      table[idx] = key;
      return 1;
    }
    if (table[idx] == key) return 0;
    idx = (idx + 1) & mask;
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Exact k-nearest-neighbour graph inside one contiguous id block             */
/* (what raft_help.cuh:74-172 build_batch_knn_graphs asks RAFT for, and what  */
/* cagra.cu:69-210 generate_knn_graph approximates with IVF-PQ + exact        */
/* re-rank).  Self is dropped and short rows are padded with 0xFFFFFFFF as in */
/* cagra.cu:175-199.  Ids are LOCAL to the block; ties go to the lower id.    */
/* ------------------------------------------------------------------------- */
void orc_knn_block(const float* data, uint64_t n, uint32_t dim, uint32_t k, int metric,
                   uint32_t* out) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * n);
    uint64_t m = 0;
    for (uint64_t j = 0; j < n; ++j) {
      if (j == (uint64_t)i) continue;
      keys[m++] = orc_make_key(orc_dist(data + (size_t)i * dim, data + (size_t)j * dim, dim, metric),
                               (uint32_t)j);
    }
    qsort(keys, m, sizeof(uint64_t), cmp_u64);
    for (uint32_t c = 0; c < k; ++c)
      out[(size_t)i * k + c] = c < m ? (uint32_t)(keys[c] & 0xFFFFFFFFu) : ORC_INVALID;
    free(keys);
  }
}

/* ------------------------------------------------------------------------- */
/* Rank-based prune.  Detour counts: src/index/cagra.cu:219-276 (kern_prune); */
/* selection: cagra.cu:367-392 (stable sort by count, ties keep the original  */
/* rank, first out_deg kept).                                                 */
/* count[kAB] = number of (kAD < kAB, kDB) with graph[D][kDB] == graph[A][kAB]*/
/* where D = graph[A][kAD] is valid and kAB is the FIRST rank > kAD holding   */
/* that id (the reference's inner loop breaks at the first match, and pads    */
/* 0xFFFFFFFF match pads exactly as there).  Clamped to 255.                  */
/* ------------------------------------------------------------------------- */
void orc_prune(const uint32_t* knn, uint32_t* out, uint64_t n, uint32_t in_deg, uint32_t out_deg,
               uint8_t* detour_out /* optional [n,in_deg] */) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t a = 0; a < (int64_t)n; ++a) {
    const uint32_t* rowA = knn + (size_t)a * in_deg;
    uint32_t* cnt = (uint32_t*)calloc(in_deg, sizeof(uint32_t));
    for (uint32_t kAD = 0; kAD + 1 < in_deg; ++kAD) {
      uint32_t d = rowA[kAD];
      if (d == ORC_INVALID || d >= n) continue; /* ids outside [0,n) are skipped, not dereferenced */
      const uint32_t* rowD = knn + (size_t)d * in_deg;
      for (uint32_t kDB = 0; kDB < in_deg; ++kDB) {
        uint32_t cand = rowD[kDB];
        for (uint32_t kAB = kAD + 1; kAB < in_deg; ++kAB) {
          if (rowA[kAB] == cand) {
            cnt[kAB]++;
            break;
          }
        }
      }
    }
    uint8_t* c8 = (uint8_t*)malloc(in_deg);
    for (uint32_t k = 0; k < in_deg; ++k) c8[k] = cnt[k] > 255 ? 255 : (uint8_t)cnt[k];
    if (detour_out) memcpy(detour_out + (size_t)a * in_deg, c8, in_deg);
    /* stable selection: ascending (count, rank) */
    uint32_t filled = 0;
    for (uint32_t level = 0; level < 256 && filled < out_deg; ++level)
      for (uint32_t k = 0; k < in_deg && filled < out_deg; ++k)
        if (c8[k] == level) out[(size_t)a * out_deg + filled++] = rowA[k];
    free(c8);
    free(cnt);
  }
}

/* ------------------------------------------------------------------------- */
/* Reverse graph.  src/index/cagra.cu:418-444 + 455-548: the reference sweeps */
/* the forward graph one COLUMN at a time (k = 0..deg-1) and every edge       */
/* src->dest claims the next free slot of dest by atomicAdd; only the first   */
/* deg claimants are stored, the counter keeps the true in-degree.  Inside a  */
/* column the order is a race in the reference; here it is ascending src.     */
/* ------------------------------------------------------------------------- */
void orc_reverse_graph(const uint32_t* graph, uint32_t* rev, uint32_t* rev_counts, uint64_t n,
                       uint32_t deg) {
  memset(rev, 0xFF, sizeof(uint32_t) * n * deg);
  memset(rev_counts, 0, sizeof(uint32_t) * n);
  for (uint32_t k = 0; k < deg; ++k)
    for (uint64_t s = 0; s < n; ++s) {
      uint32_t d = graph[s * deg + k];
      if (d >= n) continue;
      uint32_t pos = rev_counts[d]++;
      if (pos < deg) rev[(size_t)d * deg + pos] = (uint32_t)s;
    }
}

/* ------------------------------------------------------------------------- */
/* Interleaved merge.  src/index/cagra.cu:574-650: alternately take the next  */
/* not-yet-present forward edge and the next not-yet-present reverse edge,    */
/* skipping self (and reverse ids >= n), until deg entries; ONLY the filled   */
/* prefix is written back (cagra.cu:641-648), the tail keeps the pruned row.  */
/* ------------------------------------------------------------------------- */
void orc_merge_graphs(uint32_t* graph, const uint32_t* rev, const uint32_t* rev_counts, uint64_t n,
                      uint32_t deg) {
#pragma omp parallel for
  for (int64_t j = 0; j < (int64_t)n; ++j) {
    const uint32_t* so = graph + (size_t)j * deg;
    const uint32_t* sr = rev + (size_t)j * deg;
    uint32_t rc = rev_counts[j] > deg ? deg : rev_counts[j];
    uint32_t* nn = (uint32_t*)malloc(sizeof(uint32_t) * deg);
    uint32_t sz = 0, co = 0, cr = 0;
    while (sz < deg) {
      int added = 0;
      while (co < deg) {
        uint32_t c = so[co++];
        if (c == (uint32_t)j) continue;
        int dup = 0;
        for (uint32_t i = 0; i < sz; ++i) dup |= (nn[i] == c);
        if (dup) continue;
        nn[sz++] = c;
        added = 1;
        break;
      }
      if (sz >= deg) break;
      while (cr < rc) {
        uint32_t c = sr[cr++];
        if (c >= n) continue;
        if (c == (uint32_t)j) continue;
        int dup = 0;
        for (uint32_t i = 0; i < sz; ++i) dup |= (nn[i] == c);
        if (dup) continue;
        nn[sz++] = c;
        added = 1;
        break;
      }
      if (!added) break;
    }
    memcpy(graph + (size_t)j * deg, nn, sizeof(uint32_t) * sz);
    free(nn);
  }
}

/* ------------------------------------------------------------------------- */
/* Remote (cross-bucket) edges.  src/index/cagra_opt.cu:209-303               */
/* (update_remote_edges_kernel).  cand [n, gk]: global candidates, ascending  */
/* exact distance (cagra_opt.cu:48-148).  bucket[] plays the role of d_ts     */
/* (the reference's timestamps ARE bucket ids).  nearby third first, then far */
/* candidates, then anything from another bucket.  cand is consumed (used     */
/* entries are overwritten with 0xFFFFFFFF) exactly as in the reference.      */
/* ------------------------------------------------------------------------- */
void orc_remote_edges(uint32_t* graph, const uint64_t* bucket, uint32_t* cand, uint64_t n,
                      uint32_t total_deg, uint32_t local_deg, uint32_t gk) {
  uint64_t total_buckets = bucket[n - 1] + 1;
  uint64_t span = total_buckets / 5 > 1 ? total_buckets / 5 : 1;
  for (uint64_t t = 0; t < n; ++t) {
    uint32_t* row = graph + t * total_deg;
    uint32_t* mc = cand + t * gk;
    uint64_t my = bucket[t];
    uint64_t mn = my >= span ? my - span : 0;
    uint64_t mx = my + span >= total_buckets ? total_buckets - 1 : my + span;
    int nearby = 0, nearby_max = (int)(total_deg - local_deg) / 3;
    for (uint32_t k = 0; k < gk && nearby_max > 0; ++k) {
      uint32_t c = mc[k];
      if (c == (uint32_t)t || c == ORC_INVALID) continue;
      if (bucket[c] == my || bucket[c] < mn || bucket[c] > mx) continue;
      row[local_deg + nearby++] = c;
      mc[k] = ORC_INVALID;
      if (nearby >= nearby_max) break;
    }
    int remote = 0, remote_max = (int)(total_deg - local_deg) - nearby;
    for (uint32_t k = 0; k < gk && remote_max > 0; ++k) {
      uint32_t c = mc[k];
      if (c == (uint32_t)t || c == ORC_INVALID) continue;
      if (bucket[c] == my || (bucket[c] >= mn && bucket[c] <= mx)) continue;
      row[local_deg + nearby + remote++] = c;
      mc[k] = ORC_INVALID;
      if (remote >= remote_max) break;
    }
    for (uint32_t k = 0; k < gk && remote < remote_max; ++k) {
      uint32_t c = mc[k];
      if (c == (uint32_t)t || c == ORC_INVALID) continue;
      if (bucket[c] == my) continue;
      row[local_deg + nearby + remote++] = c;
    }
  }
}
/* NOTE on the two `_max > 0` guards above: with nearby_max == 0 the reference
 * loop (cagra_opt.cu:246-259) would still write one entry before its
 * `>= nearby_max` test; that only happens for total-local < 3, which the
 * library rejects, so the guard is unreachable for accepted parameters. */

static inline uint32_t wang_hash(uint32_t s) { /* cagra_opt.cu:33-40 */
  s = (s ^ 61u) ^ (s >> 16);
  s *= 9u;
  s = s ^ (s >> 4);
  s *= 0x27d4eb2du;
  s = s ^ (s >> 15);
  return s;
}
uint32_t orc_wang_hash(uint32_t s) { return wang_hash(s); }

/* ------------------------------------------------------------------------- */
/* Reverse injection of remote edges.  cagra_opt.cu:457-481 (reverse lists of */
/* the remote columns only, cap max_rev = 32, cagra_opt.cu:744) and           */
/* cagra_opt.cu:487-600 (inject into the weak half: first empty weak slot,    */
/* else a wang_hash-random weak slot).  The reference's claim order is a race */
/* (one thread per src, atomics); here it is ascending src, then column.      */
/* ------------------------------------------------------------------------- */
void orc_inject_reverse_remote(uint32_t* graph, uint64_t n, uint32_t total_deg, uint32_t local_deg,
                               uint32_t max_rev) {
  uint32_t* rev = (uint32_t*)malloc(sizeof(uint32_t) * n * max_rev);
  uint32_t* rc = (uint32_t*)calloc(n, sizeof(uint32_t));
  for (uint64_t s = 0; s < n; ++s)
    for (uint32_t k = local_deg; k < total_deg; ++k) {
      uint32_t d = graph[s * total_deg + k];
      if (d != ORC_INVALID && d < n) {
        uint32_t pos = rc[d]++;
        if (pos < max_rev) rev[(size_t)d * max_rev + pos] = (uint32_t)s;
      }
    }
  uint32_t num_remote = total_deg - local_deg;
  int num_strong = (int)num_remote / 2, num_weak = (int)num_remote - num_strong;
  for (uint64_t t = 0; t < n; ++t) {
    uint32_t* row = graph + t * total_deg;
    uint32_t cur[64];
    for (uint32_t i = 0; i < num_remote; ++i) cur[i] = row[local_deg + i];
    uint32_t cnt = rc[t];
    if (cnt == 0) continue;
    if (cnt > max_rev) cnt = max_rev;
    uint32_t rng = wang_hash((uint32_t)t);
    for (uint32_t i = 0; i < cnt; ++i) {
      uint32_t c = rev[(size_t)t * max_rev + i];
      int exists = 0;
      for (uint32_t r = 0; r < num_remote; ++r) exists |= (cur[r] == c);
      if (exists) continue;
      for (uint32_t l = 0; l < local_deg; ++l) exists |= (row[l] == c);
      if (exists) continue;
      int injected = 0;
      for (int w = num_strong; w < (int)num_remote; ++w)
        if (cur[w] == ORC_INVALID) {
          cur[w] = c;
          injected = 1;
          break;
        }
      if (!injected && num_weak > 0) {
        rng = wang_hash(rng);
        cur[num_strong + (rng % (uint32_t)num_weak)] = c;
      }
    }
    for (uint32_t i = 0; i < num_remote; ++i) row[local_deg + i] = cur[i];
  }
  free(rev);
  free(rc);
}

/* ------------------------------------------------------------------------- */
/* Graph search, one query.  Restates src/index/search.cu:149-372 (plain),    */
/* :375-586 (bucket: only the first active_degree columns),                   */
/* :589-783 (range: predicate lo <= ts[nbr] < hi), with the building blocks   */
/* compute_distance.cuh:204-269 (seeds), :274-383 / :386-505 / :512-614       */
/* (expansion), search.cu:38-107 (parent pick-up), hashmap.cuh.               */
/* mode 0 plain, 1 bucket, 2 range.  The queue holds `cap` (id,dist) slots:   */
/* [0,itopk) best so far, [itopk, itopk+W*deg) this round's candidates.       */
/* Warps run tasks in parallel in the reference; here tasks run in ascending  */
/* task id, which only matters when the visited table overflows.              */
/* Faithful quirks: (i) in range mode the visited insert happens BEFORE the   */
/* predicate (compute_distance.cuh:572-584) and rejected / visited tasks      */
/* leave their slot untouched (stale entries are re-sorted); (ii) the table   */
/* is cleared every 30 iterations and re-seeded from the first itopk entries  */
/* (search.cu:692-697); (iii) seeds outside [0,n) are replaced by             */
/* (xor_mask*(i+1)) % n (compute_distance.cuh:236-238); (iv) empty result     */
/* slots come back as id 0x7FFFFFFF, dist FLT_MAX (search.cu:779).            */
/* Sorting is by distance; equal distances keep no defined order in the       */
/* reference -- here (dist, slot value) ascending.                            */
/* stats (optional, 5 x u64): iterations, parents, edges examined, distances  */
/* computed, seeds evaluated.                                                 */
/* ------------------------------------------------------------------------- */
typedef struct {
  uint64_t key;
} qent;
static void sort_queue(uint32_t* ids, float* dists, uint32_t cap) {
  uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * cap);
  for (uint32_t i = 0; i < cap; ++i) keys[i] = orc_make_key(dists[i], ids[i]);
  qsort(keys, cap, sizeof(uint64_t), cmp_u64);
  for (uint32_t i = 0; i < cap; ++i) {
    ids[i] = (uint32_t)(keys[i] & 0xFFFFFFFFu);
    dists[i] = ord2f((uint32_t)(keys[i] >> 32));
  }
  free(keys);
}

void orc_graph_search_one(const float* data, uint64_t n, uint32_t dim, const uint32_t* graph,
                          uint32_t deg, uint32_t active_deg, const uint64_t* ts, uint64_t lo,
                          uint64_t hi, int mode, const float* q, const uint32_t* seeds,
                          uint32_t num_provided, uint32_t num_seeds, uint64_t xor_mask, uint32_t k,
                          uint32_t itopk, uint32_t width, uint32_t max_iter, uint32_t hash_bitlen,
                          uint32_t cap, int metric, uint32_t* out_ids, float* out_dists,
                          uint64_t* stats) {
  uint32_t hsize = 1u << hash_bitlen;
  uint32_t* hash = (uint32_t*)malloc(sizeof(uint32_t) * hsize);
  uint32_t* ids = (uint32_t*)malloc(sizeof(uint32_t) * cap);
  float* dists = (float*)malloc(sizeof(float) * cap);
  uint32_t* parents = (uint32_t*)malloc(sizeof(uint32_t) * width);
  memset(hash, 0xFF, sizeof(uint32_t) * hsize);
  for (uint32_t i = 0; i < cap; ++i) {
    ids[i] = ORC_INVALID;
    dists[i] = ORC_FLT_MAX;
  }
  uint64_t st_iter = 0, st_par = 0, st_edge = 0, st_dist = 0, st_seed = 0;
  for (uint32_t i = 0; i < num_seeds; ++i) {
    uint32_t id = ORC_INVALID;
    if (seeds && i < num_provided) id = seeds[i];
    if (id >= n) id = (uint32_t)((xor_mask * (uint64_t)(i + 1)) % n);
    ids[i] = id;
    dists[i] = orc_dist(q, data + (size_t)id * dim, dim, metric);
    orc_hash_insert(hash, hash_bitlen, id);
    st_seed++;
  }
  uint32_t iter = 0;
  for (; iter < max_iter; ++iter) {
    if (iter > 0 && iter % 30 == 0) {
      memset(hash, 0xFF, sizeof(uint32_t) * hsize);
      for (uint32_t i = 0; i < itopk; ++i) {
        uint32_t id = ids[i] & 0x7FFFFFFFu;
        if (id != ORC_INVALID) orc_hash_insert(hash, hash_bitlen, id);
      }
    }
    sort_queue(ids, dists, cap);
    uint32_t np = 0;
    for (uint32_t i = 0; i < width; ++i) parents[i] = ORC_INVALID;
    for (uint32_t j = 0; j < itopk && np < width; ++j)
      if ((ids[j] & ORC_MSB) == 0 && ids[j] != ORC_INVALID) {
        parents[np++] = ids[j];
        ids[j] |= ORC_MSB;
      }
    if (np == 0) break;
    st_iter++;
    st_par += np;
    uint32_t tasks = width * deg;
    for (uint32_t t = 0; t < tasks; ++t) {
      uint32_t pi = t / deg, off = t % deg;
      uint32_t* cid = ids + itopk + t;
      float* cd = dists + itopk + t;
      if (mode == 1 && off >= active_deg) {
        *cid = ORC_INVALID;
        *cd = ORC_FLT_MAX;
        continue;
      }
      uint32_t p = parents[pi];
      uint32_t nb = ORC_INVALID;
      if (p != ORC_INVALID) nb = graph[(size_t)p * deg + off];
      if (p == ORC_INVALID || nb == ORC_INVALID) {
        if (mode != 2) {
          *cid = ORC_INVALID;
          *cd = ORC_FLT_MAX;
        }
        continue;
      }
      st_edge++;
      int fresh = orc_hash_insert(hash, hash_bitlen, nb);
      if (mode == 2) {
        if (ts[nb] < lo || ts[nb] >= hi) continue;
        if (!fresh) continue;
      } else if (!fresh) {
        *cid = ORC_INVALID;
        *cd = ORC_FLT_MAX;
        continue;
      }
      *cid = nb;
      *cd = orc_dist(q, data + (size_t)nb * dim, dim, metric);
      st_dist++;
    }
  }
  sort_queue(ids, dists, cap);
  for (uint32_t i = 0; i < k; ++i) {
    out_ids[i] = ids[i] & 0x7FFFFFFFu;
    out_dists[i] = dists[i];
  }
  if (stats) {
    stats[0] += st_iter;
    stats[1] += st_par;
    stats[2] += st_edge;
    stats[3] += st_dist;
    stats[4] += st_seed;
  }
  free(hash);
  free(ids);
  free(dists);
  free(parents);
}

/* Launcher arithmetic of cagra_opt.cu:1108-1210 (mode 0: itopk floor 64,     */
/* seeds = clamp(max(32, provided), itopk)), :1212-1328 (mode 1: itopk floor  */
/* 128, seeds = min(provided, itopk)), :1330-1442 (mode 2: floor 64, seeds =  */
/* min(provided, itopk)); cap = max(256, pow2(itopk + W*deg)).  One range     */
/* [lo[q], hi[q]) per query (the reference takes one range per call).         */
static uint32_t next_pow2(uint32_t v) {
  if (v == 0) return 1;
  v--;
  v |= v >> 1;
  v |= v >> 2;
  v |= v >> 4;
  v |= v >> 8;
  v |= v >> 16;
  return v + 1;
}
void orc_graph_search(const float* data, uint64_t n, uint32_t dim, const uint32_t* graph,
                      uint32_t deg, uint32_t active_deg, const uint64_t* ts, const uint64_t* lo,
                      const uint64_t* hi, int mode, const float* queries, uint64_t nq,
                      const uint32_t* seeds, uint32_t seeds_per_query, uint64_t xor_mask,
                      uint32_t k, uint32_t itopk_param, uint32_t width, uint32_t max_iter,
                      uint32_t hash_bitlen, int metric, int64_t* out_ids, float* out_dists,
                      uint64_t* stats) {
  uint32_t itopk = k > itopk_param ? k : itopk_param;
  uint32_t floor_ = mode == 1 ? 128 : 64;
  if (itopk < floor_) itopk = floor_;
  uint32_t cap = next_pow2(itopk + width * deg);
  if (cap < 256) cap = 256;
  uint32_t target;
  if (mode == 0) {
    target = seeds_per_query > 32 ? seeds_per_query : 32;
  } else {
    target = seeds_per_query;
  }
  if (target > itopk) target = itopk;
  uint64_t tot[5] = {0, 0, 0, 0, 0};
#pragma omp parallel
  {
    uint64_t loc[5] = {0, 0, 0, 0, 0};
    uint32_t* oi = (uint32_t*)malloc(sizeof(uint32_t) * k);
#pragma omp for schedule(dynamic, 4)
    for (int64_t qi = 0; qi < (int64_t)nq; ++qi) {
      orc_graph_search_one(data, n, dim, graph, deg, active_deg, ts, lo ? lo[qi] : 0,
                           hi ? hi[qi] : 0, mode, queries + (size_t)qi * dim,
                           seeds ? seeds + (size_t)qi * seeds_per_query : NULL, seeds_per_query,
                           target, xor_mask, k, itopk, width, max_iter, hash_bitlen, cap, metric,
                           oi, out_dists + (size_t)qi * k, loc);
      for (uint32_t i = 0; i < k; ++i) out_ids[(size_t)qi * k + i] = (int64_t)oi[i];
    }
    free(oi);
#pragma omp critical
    for (int i = 0; i < 5; ++i) tot[i] += loc[i];
  }
  if (stats)
    for (int i = 0; i < 5; ++i) stats[i] = tot[i];
}

/* ------------------------------------------------------------------------- */
/* Insert, v1 topology update.  src/index/insert.cu:225-254 (new rows = first */
/* deg search hits that are valid old ids), :263-290 + thrust sort :424       */
/* (requests grouped by target; within a target the reference's radix sort is */
/* stable, so sources stay in request order = ascending tid), :296-368 (the   */
/* segment leader replaces a random slot: LCG, 10% first half / 90% second    */
/* half, skipped when the source is already present).                         */
/* found [num_new, search_k] int64.                                           */
/* ------------------------------------------------------------------------- */
void orc_insert_v1(uint32_t* graph, const int64_t* found, uint64_t num_existing, uint64_t num_new,
                   uint32_t deg, uint32_t search_k) {
  for (uint64_t i = 0; i < num_new; ++i)
    for (uint32_t k = 0; k < deg; ++k) {
      uint32_t v = ORC_INVALID;
      if (k < search_k) {
        int64_t idx = found[i * search_k + k];
        if (idx >= 0 && idx < (int64_t)num_existing) v = (uint32_t)idx;
      }
      graph[(num_existing + i) * deg + k] = v;
    }
  uint64_t total = num_new * search_k;
  uint64_t* req = (uint64_t*)malloc(sizeof(uint64_t) * total); /* (target<<32 | tid) */
  for (uint64_t t = 0; t < total; ++t) {
    int64_t idx = found[t];
    uint32_t key = (idx >= 0 && idx < (int64_t)num_existing) ? (uint32_t)idx : ORC_INVALID;
    req[t] = ((uint64_t)key << 32) | (uint32_t)t;
  }
  qsort(req, total, sizeof(uint64_t), cmp_u64);
  const uint32_t num_prot = deg / 2, num_unprot = deg - num_prot;
  for (uint64_t pos = 0; pos < total;) {
    uint32_t target = (uint32_t)(req[pos] >> 32);
    uint64_t end = pos;
    while (end < total && (uint32_t)(req[end] >> 32) == target) ++end;
    if (target != ORC_INVALID) {
      uint32_t* nb = graph + (size_t)target * deg;
      uint64_t rng = (uint64_t)target * 0x9e3779b97f4a7c15ULL + (uint32_t)pos;
      for (uint64_t x = pos; x < end; ++x) {
        uint32_t tid = (uint32_t)(req[x] & 0xFFFFFFFFu);
        uint32_t src = (uint32_t)(num_existing + tid / search_k);
        int exists = 0;
        for (uint32_t c = 0; c < deg; ++c) exists |= (nb[c] == src);
        if (exists) continue;
        rng = rng * 6364136223846793005ULL + 1;
        uint32_t r1 = (uint32_t)(rng >> 32);
        int prot = (r1 % 10 == 0);
        rng = rng * 6364136223846793005ULL + 1;
        uint32_t r2 = (uint32_t)(rng >> 32);
        uint32_t slot = prot ? r2 % num_prot : num_prot + (r2 % num_unprot);
        nb[slot] = src;
      }
    }
    pos = end;
  }
  free(req);
}

/* ------------------------------------------------------------------------- */
/* Insert, time-partitioned ("opt") topology update.                          */
/* Fill: src/index/insert.cu:448-577 -- local slots from same-bucket local    */
/* candidates, remote slots from other-bucket global candidates not already   */
/* local, then back-fill with any unused global candidate.                    */
/* Mailboxes: insert.cu:579-640 -- every edge of a new row posts the new id   */
/* to its target (local cap local_deg/2, remote cap remote/2, remote posts to */
/* targets in the new nodes' own bucket are dropped).  The reference's post   */
/* order is a race; here ascending new id, then column.                       */
/* Apply: insert.cu:653-765 -- per old node drain local then remote mail with */
/* wang_hash slot choice (10% strong / 90% weak half for local; nearby third  */
/* vs far part for remote by |bucket delta| <= 20).                           */
/* ------------------------------------------------------------------------- */
/* Stage 1 (insert.cu:448-577): rows of the new nodes; used candidates are overwritten with -1. */
void orc_insert_opt_fill(uint32_t* graph, const uint64_t* bucket, int64_t* local_knn, int64_t* global_knn,
                         uint64_t num_existing, uint64_t num_new, uint32_t total_deg, uint32_t local_deg,
                         uint32_t k_local, uint32_t k_global) {
  int max_remote = (int)(total_deg - local_deg);
  for (uint64_t t = 0; t < num_new; ++t) {
    uint64_t me = num_existing + t;
    uint64_t my = bucket[me];
    uint32_t* row = graph + me * total_deg;
    int64_t* lc = local_knn + t * k_local;
    uint32_t fl = 0;
    for (uint32_t k = 0; k < k_local && fl < local_deg; ++k) {
      int64_t c64 = lc[k];
      uint32_t c = (uint32_t)c64;
      if (c64 < 0 || c == me || c >= 0x7fffffffu) continue;
      if (bucket[c] != my) continue;
      row[fl++] = c;
      lc[k] = -1;
    }
    int fr = 0;
    int64_t* gc = global_knn + t * k_global;
    for (uint32_t k = 0; k < k_global && fr < max_remote; ++k) {
      int64_t c64 = gc[k];
      uint32_t c = (uint32_t)c64;
      if (c64 < 0 || c == me) continue;
      int ex = 0;
      for (uint32_t i = 0; i < local_deg; ++i) ex |= (row[i] == c);
      if (ex) continue;
      if (bucket[c] != my) {
        row[local_deg + fr++] = c;
        gc[k] = -1;
      }
    }
    for (uint32_t i = 0; i < k_global && fr < max_remote; ++i) {
      int64_t c64 = gc[i];
      uint32_t c = (uint32_t)c64;
      if (c64 < 0 || c == me) continue;
      row[local_deg + fr++] = c;
      gc[i] = -1;
    }
  }
}

/* Stage 2 (insert.cu:579-640): mailboxes.  lcnt/rcnt [num_existing+num_new] hold the TRUE request
 * counts; llist/rlist [.., local_deg/2] / [.., (total-local)/2] the first `max` senders in ascending
 * (new id, column) order. */
void orc_insert_opt_mailboxes(const uint32_t* graph, const uint64_t* bucket, uint64_t num_existing,
                              uint64_t num_new, uint64_t target_bucket, uint32_t total_deg,
                              uint32_t local_deg, uint32_t* lcnt, uint32_t* llist, uint32_t* rcnt,
                              uint32_t* rlist) {
  uint32_t lmax = local_deg / 2, rmax = (total_deg - local_deg) / 2;
  memset(lcnt, 0, sizeof(uint32_t) * (num_existing + num_new));
  memset(rcnt, 0, sizeof(uint32_t) * (num_existing + num_new));
  for (uint64_t t = 0; t < num_new; ++t) {
    uint32_t src = (uint32_t)(num_existing + t);
    const uint32_t* nb = graph + (size_t)src * total_deg;
    for (uint32_t i = 0; i < total_deg; ++i) {
      uint32_t d = nb[i];
      if (d == ORC_INVALID) continue;
      if (i < local_deg) {
        uint32_t pos = lcnt[d]++;
        if (pos < lmax) llist[(size_t)d * lmax + pos] = src;
      } else {
        if (bucket[d] == target_bucket) continue;
        uint32_t pos = rcnt[d]++;
        if (pos < rmax) rlist[(size_t)d * rmax + pos] = src;
      }
    }
  }
}

/* Stage 3 (insert.cu:653-765): every old node drains its local, then its remote mail. */
void orc_insert_opt_apply(uint32_t* graph, const uint64_t* bucket, uint64_t num_existing,
                          uint32_t total_deg, uint32_t local_deg, const uint32_t* lcnt,
                          const uint32_t* llist, const uint32_t* rcnt, const uint32_t* rlist) {
  uint32_t lmax = local_deg / 2, rmax = (total_deg - local_deg) / 2;
  for (uint64_t t = 0; t < num_existing; ++t) {
    uint32_t* row = graph + t * total_deg;
    uint32_t rng = wang_hash((uint32_t)t);
    uint32_t lc = lcnt[t];
    if (lc > 0) {
      if (lc > lmax) lc = lmax;
      uint32_t half = local_deg / 2, strong = half, weak = local_deg - half;
      for (uint32_t i = 0; i < lc; ++i) {
        uint32_t c = llist[(size_t)t * lmax + i];
        rng = wang_hash(rng);
        int atk = (rng % 100) < 10;
        uint32_t ts_ = atk ? 0 : half, tl = atk ? strong : weak;
        if (tl > 0) {
          rng = wang_hash(rng);
          row[ts_ + (rng % tl)] = c;
        }
      }
    }
    uint32_t rc = rcnt[t];
    if (rc > 0) {
      if (rc > rmax) rc = rmax;
      uint32_t rd = total_deg - local_deg;
      for (uint32_t i = 0; i < rc; ++i) {
        uint32_t c = rlist[(size_t)t * rmax + i];
        int64_t mt = (int64_t)bucket[t], ct = (int64_t)bucket[c];
        int near = (ct >= mt - 20) && (ct <= mt + 20);
        uint32_t nlen = rd / 3;
        uint32_t ts_ = near ? local_deg : local_deg + rd / 3;
        uint32_t tl = near ? nlen : rd - nlen;
        if (tl > 0) {
          rng = wang_hash(rng);
          row[ts_ + (rng % tl)] = c;
        }
      }
    }
  }
}

void orc_insert_opt(uint32_t* graph, const uint64_t* bucket, int64_t* local_knn, int64_t* global_knn,
                    uint64_t num_existing, uint64_t num_new, uint64_t target_bucket,
                    uint32_t total_deg, uint32_t local_deg, uint32_t k_local, uint32_t k_global) {
  orc_insert_opt_fill(graph, bucket, local_knn, global_knn, num_existing, num_new, total_deg, local_deg,
                      k_local, k_global);
  uint32_t lmax = local_deg / 2, rmax = (total_deg - local_deg) / 2;
  uint64_t ntot = num_existing + num_new;
  uint32_t* lcnt = (uint32_t*)malloc(sizeof(uint32_t) * ntot);
  uint32_t* rcnt = (uint32_t*)malloc(sizeof(uint32_t) * ntot);
  uint32_t* llist = (uint32_t*)malloc(sizeof(uint32_t) * ntot * (lmax ? lmax : 1));
  uint32_t* rlist = (uint32_t*)malloc(sizeof(uint32_t) * ntot * (rmax ? rmax : 1));
  orc_insert_opt_mailboxes(graph, bucket, num_existing, num_new, target_bucket, total_deg, local_deg,
                           lcnt, llist, rcnt, rlist);
  orc_insert_opt_apply(graph, bucket, num_existing, total_deg, local_deg, lcnt, llist, rcnt, rlist);
  free(lcnt);
  free(rcnt);
  free(llist);
  free(rlist);
}

/* ------------------------------------------------------------------------- */
/* Merge of per-shard top-k lists (multi-GPU exchange step; no counterpart in */
/* the single-GPU reference).  in_keys [nq, parts, k] ascending (dist,id)     */
/* keys with global ids -> global top-k.                                      */
/* ------------------------------------------------------------------------- */
void orc_merge_topk(const float* dists, const int64_t* ids, uint64_t nq, uint32_t parts, uint32_t k,
                    int64_t* out_ids, float* out_dists) {
  for (uint64_t q = 0; q < nq; ++q) {
    uint32_t m = parts * k;
    uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * m * 2);
    /* 64-bit ids: sort by (dist, id) with a two-word key */
    uint32_t cnt = 0;
    for (uint32_t i = 0; i < m; ++i) {
      int64_t id = ids[q * m + i];
      if (id < 0) continue;
      keys[2 * cnt] = f2ord(dists[q * m + i]);
      keys[2 * cnt + 1] = (uint64_t)id;
      cnt++;
    }
    /* insertion sort on pairs (m is small) */
    for (uint32_t i = 1; i < cnt; ++i) {
      uint64_t a = keys[2 * i], b = keys[2 * i + 1];
      int64_t j = (int64_t)i - 1;
      while (j >= 0 && (keys[2 * j] > a || (keys[2 * j] == a && keys[2 * j + 1] > b))) {
        keys[2 * j + 2] = keys[2 * j];
        keys[2 * j + 3] = keys[2 * j + 1];
        --j;
      }
      keys[2 * j + 2] = a;
      keys[2 * j + 3] = b;
    }
    for (uint32_t i = 0; i < k; ++i) {
      if (i < cnt) {
        out_ids[q * k + i] = (int64_t)keys[2 * i + 1];
        out_dists[q * k + i] = ord2f((uint32_t)keys[2 * i]);
      } else {
        out_ids[q * k + i] = -1;
        out_dists[q * k + i] = ORC_FLT_MAX;
      }
    }
    free(keys);
  }
}

/* ------------------------------------------------------------------------- */
/* Entry-point router (device form of the reference's host seed sampling,     */
/* cagraIndexOpt.cu:441-511, and of the k-means routing of its two-level      */
/* index, timeStampIndex.cu:141-238 and :240-419).  Restated step by step in  */
/* the arithmetic order the product fixes, so every output is bit-exact.      */
/* ------------------------------------------------------------------------- */

/* The P nearest centroids of every row, best first.  x.c is one fused multiply-add chain
 * over ascending dimensions; score = fma(-2, x.c, |c|^2) (L2) or -(x.c) (inner product);
 * ties go to the lower centroid id; missing entries are 0xFFFFFFFF. */
void orc_nearest_centroids(const float* X, uint64_t m, uint32_t dim, const float* cen, const float* cnorm,
                           uint32_t C, int metric, uint32_t P, uint32_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)m; ++r) {
    uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * C);
    for (uint32_t c = 0; c < C; ++c) {
      float acc = 0.0f;
      for (uint32_t k = 0; k < dim; ++k) acc = fmaf(X[r * dim + k], cen[(uint64_t)c * dim + k], acc);
      float s = metric == 0 ? fmaf(-2.0f, acc, cnorm[c]) : -acc;
      keys[c] = orc_make_key(s, c);
    }
    qsort(keys, C, sizeof(uint64_t), cmp_u64);
    for (uint32_t p = 0; p < P; ++p) out[r * P + p] = p < C ? (uint32_t)(keys[p] & 0xFFFFFFFFu) : 0xFFFFFFFFu;
    free(keys);
  }
}

/* ids 0..m-1 grouped by assign[], ascending inside each group. */
void orc_group_by_centroid(const uint32_t* assign, uint64_t m, uint32_t C, uint32_t* offsets, uint32_t* members) {
  uint32_t* cur = (uint32_t*)calloc(C + 1, sizeof(uint32_t));
  for (uint64_t i = 0; i < m; ++i) if (assign[i] < C) cur[assign[i] + 1]++;
  for (uint32_t c = 0; c < C; ++c) cur[c + 1] += cur[c];
  memcpy(offsets, cur, sizeof(uint32_t) * (C + 1));
  for (uint64_t i = 0; i < m; ++i) if (assign[i] < C) members[cur[assign[i]]++] = (uint32_t)i;
  free(cur);
}

static float sqnorm_32lanes(const float* v, uint32_t dim) {
  float lane[32];
  for (uint32_t l = 0; l < 32; ++l) {
    float acc = 0.0f;
    for (uint32_t k = l; k < dim; k += 32) acc = fmaf(v[k], v[k], acc);
    lane[l] = acc;
  }
  for (uint32_t o = 16; o > 0; o >>= 1) {
    float nxt[32];
    for (uint32_t l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ o];
    memcpy(lane, nxt, sizeof(lane));
  }
  return lane[0];
}

/* One Lloyd update: centroid = mean of its sample members (sequential fp32 sum in list
 * order, one division), empty groups keep the old row; inner product: scaled to unit length;
 * cnorm = squared norm (32 strided partial sums, butterfly 16..1). */
void orc_centroid_update(const float* sample, uint32_t dim, const uint32_t* offsets, const uint32_t* members,
                         int metric, uint32_t C, float* cen, float* cnorm) {
  for (uint32_t c = 0; c < C; ++c) {
    float* v = cen + (uint64_t)c * dim;
    const uint32_t b = offsets[c], e = offsets[c + 1];
    if (e > b)
      for (uint32_t k = 0; k < dim; ++k) {
        float s = 0.0f;
        for (uint32_t j = b; j < e; ++j) s = s + sample[(uint64_t)members[j] * dim + k];
        v[k] = s / (float)(e - b);
      }
    float n2 = sqnorm_32lanes(v, dim);
    if (metric == 1 && e > b && n2 > 0.0f) {
      const float len = sqrtf(n2);
      for (uint32_t k = 0; k < dim; ++k) v[k] = v[k] / len;
      n2 = sqnorm_32lanes(v, dim);
    }
    cnorm[c] = n2;
  }
}

static uint64_t mix64(uint64_t x) {
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

static uint32_t lower_bound_u32(const uint32_t* a, uint32_t b, uint32_t e, uint32_t x) {
  while (b < e) { uint32_t mid = (b + e) >> 1; if (a[mid] < x) b = mid + 1; else e = mid; }
  return b;
}

/* Seeds of one batch.  filter_kind 0 none, 1 timestamp range, 2 labels (3 = prefix: a range
 * when ts is given).  lo/hi and masks are per query (NULL -> lo1/hi1/mask1). */
void orc_route_seeds(const uint32_t* probes, uint32_t p, uint64_t nq, uint64_t n, uint32_t C,
                     const uint32_t* offsets, const uint32_t* members, int filter_kind, int ts_sorted,
                     const uint64_t* ts, const uint64_t* lo, const uint64_t* hi, uint64_t lo1, uint64_t hi1,
                     const uint8_t* labels, const uint32_t* masks, uint32_t mask1, const uint32_t* label_offsets,
                     uint32_t S, uint64_t seed, uint32_t* seeds) {
  for (uint64_t q = 0; q < nq; ++q) {
    uint32_t nwin = 1, wlo = 0, whi = (uint32_t)n, mask = 0;
    int check = 0;
    uint64_t tlo = 0, thi = 0;
    if (filter_kind == 1 || (filter_kind == 3 && ts)) {
      tlo = lo ? lo[q] : lo1;
      thi = hi ? hi[q] : hi1;
      if (ts_sorted) {
        uint32_t b = 0, e = (uint32_t)n;
        while (b < e) { uint32_t mid = (b + e) >> 1; if (ts[mid] < tlo) b = mid + 1; else e = mid; }
        wlo = b; e = (uint32_t)n;
        while (b < e) { uint32_t mid = (b + e) >> 1; if (ts[mid] < thi) b = mid + 1; else e = mid; }
        whi = b;
        if (whi <= wlo) nwin = 0;
      } else {
        check = 1;
        if (thi <= tlo) nwin = 0;
      }
    } else if (filter_kind == 2) {
      mask = masks ? masks[q] : mask1;
      if (label_offsets) nwin = (uint32_t)__builtin_popcount(mask);
      else { check = 1; if (mask == 0) nwin = 0; }
    }
    const uint32_t pairs = p * (nwin ? nwin : 1);
    const uint32_t per = (S + pairs - 1) / pairs;
    for (uint32_t s = 0; s < S; ++s) {
      uint32_t id = 0xFFFFFFFFu;
      if (nwin) {
        const uint32_t j = s % p, t = s / p, w = t % nwin, r = t / nwin;
        const uint32_t c = probes[q * p + j];
        if (c < C) {
          uint32_t lo_id = wlo, hi_id = whi;
          if (filter_kind == 2 && label_offsets) {
            uint32_t mm = mask;
            for (uint32_t skip = w; skip > 0; --skip) mm &= mm - 1;
            const uint32_t lab = (uint32_t)__builtin_ctz(mm);
            lo_id = label_offsets[lab];
            hi_id = label_offsets[lab + 1];
          }
          const uint32_t rb = offsets[c], re = offsets[c + 1];
          const uint32_t b = lower_bound_u32(members, rb, re, lo_id);
          const uint32_t e = lower_bound_u32(members, b, re, hi_id);
          const uint32_t L = e - b;
          if (r < L) {
            const uint32_t step = L / per > 1 ? L / per : 1;
            const uint32_t start = (uint32_t)(mix64(seed ^ (q * 0x9e3779b97f4a7c15ull + ((uint64_t)c << 8) + w)) % L);
            const uint32_t pos = (uint32_t)((start + (uint64_t)r * step) % L);
            if (!check) {
              id = members[b + pos];
            } else {
              for (uint32_t tr = 0; tr < 4 && tr < L; ++tr) {
                const uint32_t cand = members[b + (pos + tr) % L];
                int ok;
                if (filter_kind == 2) ok = ((mask >> (labels[cand] & 31u)) & 1u) != 0;
                else ok = ts[cand] >= tlo && ts[cand] < thi;
                if (ok) { id = cand; break; }
              }
            }
          }
        }
      }
      seeds[q * S + s] = id;
    }
  }
}
