/*
 * hnsw_baseline.c -- CPU HNSW (Malkov & Yashunin, "Efficient and robust approximate nearest
 * neighbor search using Hierarchical Navigable Small World graphs") written from the published
 * algorithm, as the CPU baseline beside the GPU numbers.
 *
 * TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference's CPU baseline harness is FAISS's
 * IndexHNSWFlat (tests/test_faiss_hnsw_insert.cpp:113-174: M = 32, efConstruction = 128,
 * efSearch = 64, L2, add base, timed add, 10 x 32 queries).  FAISS is a third-party dependency
 * that is not part of the reference tree and is not installed here, so this file restates the
 * published algorithm with the harness's parameters.  PARITY UNPINNED: nothing in the reference
 * stores outputs of that harness, and FAISS's implementation details (neighbour selection
 * heuristic variants, level assignment RNG) are not reproduced bit for bit.
 *
 * Layout: level-0 adjacency of width 2*M per node, upper levels of width M; insertion with
 * per-node locks so that OpenMP threads can add concurrently (as FAISS and hnswlib do).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
  uint32_t dim, M, M0, ef_construction;
  uint64_t n, capacity;
  const float* data;  /* borrowed: [capacity, dim] */
  int* level;         /* [capacity] */
  uint32_t* link0;    /* [capacity, M0 + 1]: count, then ids */
  uint32_t** linkup;  /* [capacity] -> [level, M + 1] */
  int max_level;
  uint32_t entry;
  double mult;
  uint64_t rng;
#ifdef _OPENMP
  omp_lock_t* locks;
  omp_lock_t global;
#endif
} hnsw_t;

static inline float l2(const float* a, const float* b, uint32_t dim) {
  float s = 0.f;
  for (uint32_t i = 0; i < dim; ++i) {
    const float d = a[i] - b[i];
    s += d * d;
  }
  return s;
}

static inline uint32_t* links(const hnsw_t* h, uint32_t id, int lev) {
  return lev == 0 ? h->link0 + (size_t)id * (h->M0 + 1) : h->linkup[id] + (size_t)(lev - 1) * (h->M + 1);
}

typedef struct { float d; uint32_t id; } cand_t;

/* binary heaps on cand_t: max-heap for results, min-heap for the frontier */
static void heap_push(cand_t* h, uint32_t* n, cand_t c, int maxheap) {
  uint32_t i = (*n)++;
  h[i] = c;
  while (i) {
    const uint32_t p = (i - 1) / 2;
    const int up = maxheap ? h[p].d < h[i].d : h[p].d > h[i].d;
    if (!up) break;
    const cand_t t = h[p]; h[p] = h[i]; h[i] = t;
    i = p;
  }
}
static cand_t heap_pop(cand_t* h, uint32_t* n, int maxheap) {
  const cand_t top = h[0];
  h[0] = h[--(*n)];
  uint32_t i = 0;
  for (;;) {
    uint32_t l = 2 * i + 1, r = l + 1, m = i;
    if (l < *n && (maxheap ? h[l].d > h[m].d : h[l].d < h[m].d)) m = l;
    if (r < *n && (maxheap ? h[r].d > h[m].d : h[r].d < h[m].d)) m = r;
    if (m == i) break;
    const cand_t t = h[m]; h[m] = h[i]; h[i] = t;
    i = m;
  }
  return top;
}

typedef struct {
  cand_t *res, *front;
  uint32_t* visited;  /* epoch marks */
  uint32_t epoch;
  uint64_t cap;
} scratch_t;

static scratch_t* scratch_new(uint64_t capacity, uint32_t ef_max) {
  scratch_t* s = (scratch_t*)calloc(1, sizeof(scratch_t));
  s->res = (cand_t*)malloc(sizeof(cand_t) * (ef_max + 2));
  s->front = (cand_t*)malloc(sizeof(cand_t) * (capacity + 2));
  s->visited = (uint32_t*)calloc(capacity, sizeof(uint32_t));
  s->cap = capacity;
  return s;
}
static void scratch_free(scratch_t* s) {
  free(s->res); free(s->front); free(s->visited); free(s);
}

/* Algorithm 2 (SEARCH-LAYER): ef nearest elements to q on one layer; result max-heap in s->res */
static uint32_t search_layer(const hnsw_t* h, scratch_t* s, const float* q, uint32_t ep, float ep_d, uint32_t ef,
                             int lev, int lock) {
  uint32_t nres = 0, nfront = 0;
  if (++s->epoch == 0) { memset(s->visited, 0, sizeof(uint32_t) * s->cap); s->epoch = 1; }
  s->visited[ep] = s->epoch;
  heap_push(s->res, &nres, (cand_t){ep_d, ep}, 1);
  heap_push(s->front, &nfront, (cand_t){ep_d, ep}, 0);
  uint32_t nb[260];
  while (nfront) {
    const cand_t c = heap_pop(s->front, &nfront, 0);
    if (nres >= ef && c.d > s->res[0].d) break;
#ifdef _OPENMP
    if (lock) omp_set_lock(&((hnsw_t*)h)->locks[c.id]);
#endif
    const uint32_t* l = links(h, c.id, lev);
    const uint32_t cnt = l[0];
    memcpy(nb, l + 1, sizeof(uint32_t) * cnt);
#ifdef _OPENMP
    if (lock) omp_unset_lock(&((hnsw_t*)h)->locks[c.id]);
#endif
    for (uint32_t i = 0; i < cnt; ++i) {
      const uint32_t e = nb[i];
      if (s->visited[e] == s->epoch) continue;
      s->visited[e] = s->epoch;
      const float d = l2(q, h->data + (size_t)e * h->dim, h->dim);
      if (nres < ef || d < s->res[0].d) {
        heap_push(s->front, &nfront, (cand_t){d, e}, 0);
        heap_push(s->res, &nres, (cand_t){d, e}, 1);
        if (nres > ef) heap_pop(s->res, &nres, 1);
      }
    }
  }
  return nres;
}

static int cmp_cand(const void* a, const void* b) {
  const cand_t *x = (const cand_t*)a, *y = (const cand_t*)b;
  return (x->d > y->d) - (x->d < y->d);
}

/* Algorithm 4 (SELECT-NEIGHBORS-HEURISTIC), no extension, keep-pruned off */
static uint32_t select_heuristic(const hnsw_t* h, cand_t* c, uint32_t n, uint32_t m, uint32_t* out) {
  qsort(c, n, sizeof(cand_t), cmp_cand);
  uint32_t k = 0;
  for (uint32_t i = 0; i < n && k < m; ++i) {
    int good = 1;
    for (uint32_t j = 0; j < k; ++j)
      if (l2(h->data + (size_t)c[i].id * h->dim, h->data + (size_t)out[j] * h->dim, h->dim) < c[i].d) { good = 0; break; }
    if (good) out[k++] = c[i].id;
  }
  return k;
}

hnsw_t* orc_hnsw_new(const float* data, uint64_t capacity, uint32_t dim, uint32_t M, uint32_t ef_construction,
                     uint64_t seed) {
  hnsw_t* h = (hnsw_t*)calloc(1, sizeof(hnsw_t));
  h->dim = dim; h->M = M; h->M0 = 2 * M; h->ef_construction = ef_construction;
  h->capacity = capacity; h->data = data;
  h->level = (int*)calloc(capacity, sizeof(int));
  h->link0 = (uint32_t*)calloc(capacity * (h->M0 + 1), sizeof(uint32_t));
  h->linkup = (uint32_t**)calloc(capacity, sizeof(uint32_t*));
  h->max_level = -1;
  h->mult = 1.0 / log((double)M);
  h->rng = seed * 6364136223846793005ULL + 1442695040888963407ULL;
#ifdef _OPENMP
  h->locks = (omp_lock_t*)malloc(sizeof(omp_lock_t) * capacity);
  for (uint64_t i = 0; i < capacity; ++i) omp_init_lock(&h->locks[i]);
  omp_init_lock(&h->global);
#endif
  return h;
}

void orc_hnsw_free(hnsw_t* h) {
  for (uint64_t i = 0; i < h->capacity; ++i) free(h->linkup[i]);
#ifdef _OPENMP
  for (uint64_t i = 0; i < h->capacity; ++i) omp_destroy_lock(&h->locks[i]);
  free(h->locks);
#endif
  free(h->level); free(h->link0); free(h->linkup); free(h);
}

static void add_one(hnsw_t* h, scratch_t* s, uint32_t id, int lev) {
  const float* q = h->data + (size_t)id * h->dim;
  h->level[id] = lev;
  if (lev > 0) h->linkup[id] = (uint32_t*)calloc((size_t)lev * (h->M + 1), sizeof(uint32_t));
#ifdef _OPENMP
  omp_set_lock(&h->global);
#endif
  const int top = h->max_level;
  uint32_t ep = h->entry;
  if (top < 0) {  /* first element */
    h->entry = id; h->max_level = lev;
#ifdef _OPENMP
    omp_unset_lock(&h->global);
#endif
    return;
  }
  const int hold_global = lev > top;  /* a new top level keeps the global lock until linked */
#ifdef _OPENMP
  if (!hold_global) omp_unset_lock(&h->global);
#endif
  float ep_d = l2(q, h->data + (size_t)ep * h->dim, h->dim);
  for (int l = top; l > lev; --l) {  /* Algorithm 1 lines 5-7: greedy descent, ef = 1 */
    int changed = 1;
    while (changed) {
      changed = 0;
#ifdef _OPENMP
      omp_set_lock(&h->locks[ep]);
#endif
      const uint32_t* ln = links(h, ep, l);
      uint32_t nb[260];
      const uint32_t cnt = ln[0];
      memcpy(nb, ln + 1, sizeof(uint32_t) * cnt);
#ifdef _OPENMP
      omp_unset_lock(&h->locks[ep]);
#endif
      for (uint32_t i = 0; i < cnt; ++i) {
        const float d = l2(q, h->data + (size_t)nb[i] * h->dim, h->dim);
        if (d < ep_d) { ep_d = d; ep = nb[i]; changed = 1; }
      }
    }
  }
  cand_t* cand = (cand_t*)malloc(sizeof(cand_t) * (h->ef_construction + 2 * h->M0 + 4));
  uint32_t sel[260];
  for (int l = lev < top ? lev : top; l >= 0; --l) {
    const uint32_t nres = search_layer(h, s, q, ep, ep_d, h->ef_construction, l, 1);
    memcpy(cand, s->res, sizeof(cand_t) * nres);
    const uint32_t m = h->M;  /* connections made per layer; lists may grow to Mmax before shrinking */
    const uint32_t k = select_heuristic(h, cand, nres, m, sel);
#ifdef _OPENMP
    omp_set_lock(&h->locks[id]);
#endif
    uint32_t* mine = links(h, id, l);
    mine[0] = k;
    memcpy(mine + 1, sel, sizeof(uint32_t) * k);
#ifdef _OPENMP
    omp_unset_lock(&h->locks[id]);
#endif
    const uint32_t mmax = l == 0 ? h->M0 : h->M;
    for (uint32_t i = 0; i < k; ++i) {  /* bidirectional links, shrink when over Mmax */
      const uint32_t e = sel[i];
#ifdef _OPENMP
      omp_set_lock(&h->locks[e]);
#endif
      uint32_t* le = links(h, e, l);
      if (le[0] < mmax) {
        le[1 + le[0]++] = id;
      } else {
        cand_t tmp[260];
        const float* ev = h->data + (size_t)e * h->dim;
        uint32_t nt = 0;
        tmp[nt++] = (cand_t){l2(ev, q, h->dim), id};
        for (uint32_t j = 0; j < le[0]; ++j) tmp[nt++] = (cand_t){l2(ev, h->data + (size_t)le[1 + j] * h->dim, h->dim), le[1 + j]};
        uint32_t keep[260];
        const uint32_t kk = select_heuristic(h, tmp, nt, mmax, keep);
        le[0] = kk;
        memcpy(le + 1, keep, sizeof(uint32_t) * kk);
      }
#ifdef _OPENMP
      omp_unset_lock(&h->locks[e]);
#endif
    }
    /* the closest found element is the entry point of the next layer */
    qsort(cand, nres, sizeof(cand_t), cmp_cand);
    ep = cand[0].id; ep_d = cand[0].d;
  }
  free(cand);
  if (hold_global) {
    h->entry = id; h->max_level = lev;
#ifdef _OPENMP
    omp_unset_lock(&h->global);
#endif
  }
}

/* Adds vectors [h->n, h->n + count) of the data array (already in place). */
void orc_hnsw_add(hnsw_t* h, uint64_t count) {
  const uint64_t start = h->n;
  int* levels = (int*)malloc(sizeof(int) * count);
  for (uint64_t i = 0; i < count; ++i) {  /* level = floor(-ln(U) * mL), drawn serially: reproducible */
    h->rng = h->rng * 6364136223846793005ULL + 1442695040888963407ULL;
    const double u = ((h->rng >> 11) + 1.0) / 9007199254740993.0;
    int l = (int)(-log(u) * h->mult);
    levels[i] = l > 30 ? 30 : l;
  }
  uint64_t first = 0;
  if (h->max_level < 0 && count > 0) {  /* the very first element is added alone */
    scratch_t* s = scratch_new(h->capacity, h->ef_construction);
    add_one(h, s, (uint32_t)start, levels[0]);
    scratch_free(s);
    first = 1;
  }
#pragma omp parallel
  {
    scratch_t* s = scratch_new(h->capacity, h->ef_construction);
#pragma omp for schedule(dynamic, 64)
    for (int64_t i = (int64_t)first; i < (int64_t)count; ++i) add_one(h, s, (uint32_t)(start + i), levels[i]);
    scratch_free(s);
  }
  free(levels);
  h->n = start + count;
}

/* Algorithm 5 (K-NN-SEARCH) for nq queries, OpenMP over queries.  ef >= k.  out: ascending. */
void orc_hnsw_search(const hnsw_t* h, const float* queries, uint64_t nq, uint32_t k, uint32_t ef, int64_t* out_ids,
                     float* out_dists) {
  if (ef < k) ef = k;
#pragma omp parallel
  {
    scratch_t* s = scratch_new(h->capacity, ef);
#pragma omp for schedule(dynamic, 8)
    for (int64_t qi = 0; qi < (int64_t)nq; ++qi) {
      const float* q = queries + (size_t)qi * h->dim;
      uint32_t ep = h->entry;
      float ep_d = l2(q, h->data + (size_t)ep * h->dim, h->dim);
      for (int l = h->max_level; l > 0; --l) {
        int changed = 1;
        while (changed) {
          changed = 0;
          const uint32_t* ln = links(h, ep, l);
          for (uint32_t i = 0; i < ln[0]; ++i) {
            const float d = l2(q, h->data + (size_t)ln[1 + i] * h->dim, h->dim);
            if (d < ep_d) { ep_d = d; ep = ln[1 + i]; changed = 1; }
          }
        }
      }
      const uint32_t nres = search_layer(h, s, q, ep, ep_d, ef, 0, 0);
      qsort(s->res, nres, sizeof(cand_t), cmp_cand);
      for (uint32_t i = 0; i < k; ++i) {
        out_ids[(size_t)qi * k + i] = i < nres ? (int64_t)s->res[i].id : -1;
        out_dists[(size_t)qi * k + i] = i < nres ? s->res[i].d : 3.40282e38f;
      }
    }
    scratch_free(s);
  }
}

int orc_hnsw_present(void) { return 1; }
