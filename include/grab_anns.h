/*
 * grab_anns.h -- C ABI of the B200-native GRAB-ANNS hot path (libgrab_anns.so).
 *
 * Every entry point returns an int status (GRAB_OK == 0), never exits the process and
 * never throws.  `grab_last_error()` gives the message of the calling thread's last
 * failure.  Unless a parameter says "host", pointers named d_* are DEVICE pointers owned
 * by the caller; `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * Entry points that take a stream only enqueue work on it; the reference-shaped ones
 * without a stream synchronise before returning, as the functions they replace do.
 *
 * Each declaration cites the reference interface it replaces (paths inside
 * hxlou/GRAB-ANNS).  Ids are uint32 inside graphs (0xFFFFFFFF = empty slot, bit 31 is
 * used as a flag during search, so one index holds < 2^31 vectors) and int64 in results.
 * Distances are fp32: squared L2, or the NEGATIVE inner product, so that results are
 * always ascending.  `dim` must be a multiple of 4.
 */
#ifndef GRAB_ANNS_H_
#define GRAB_ANNS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GRAB_ABI_VERSION 3

enum grab_status {
  GRAB_OK = 0,
  GRAB_ERR_INVALID_ARGUMENT = 1,
  GRAB_ERR_UNSUPPORTED = 2,
  GRAB_ERR_CUDA = 3,
  GRAB_ERR_WORKSPACE = 4,
  GRAB_ERR_IO = 5,
  GRAB_ERR_TIMEOUT = 6, /* a bounded device-side wait gave up */
  GRAB_ERR_NCCL = 7
};

enum grab_metric { GRAB_METRIC_L2 = 0, GRAB_METRIC_IP = 1 };

enum grab_filter_kind {
  GRAB_FILTER_NONE = 0,
  GRAB_FILTER_TS_RANGE = 1, /* lo <= ts[id] < hi          (search_kernel_range)  */
  GRAB_FILTER_LABELS = 2,   /* bit labels[id] of mask set (no reference counterpart) */
  GRAB_FILTER_PREFIX = 3    /* walk only the first `active_degree` columns (search_kernel_bucket) */
};

/* src/index/cagra.cuh:30-42 (BuildParams, SearchParams), same fields and defaults. */
typedef struct grab_build_params {
  uint32_t intermediate_degree; /* 128 */
  uint32_t graph_degree;        /* 64  */
} grab_build_params;

typedef struct grab_search_params {
  uint32_t itopk_size;     /* 64 */
  uint32_t search_width;   /* 5  */
  uint32_t min_iterations; /* 0 (carried, unused, as in the reference) */
  uint32_t max_iterations; /* 20 */
  uint32_t hash_bitlen;    /* 12: log2 of the visited table of a query.  An upper bound up to 13: the per-CTA table
                            * in shared memory holds max(2^11, 8 * itopk) slots at most (it is cleared and re-seeded
                            * from the list when half full, so a smaller table costs repeated evaluations, not
                            * results, and keeps more queries resident per SM); above 13 the table lives in global
                            * memory at the size asked for */
} grab_search_params;

/* Filter of one search call.  One [lo,hi) / mask per call (the reference's form) when
 * d_lo / d_masks are NULL, else one per query. */
typedef struct grab_filter {
  int32_t kind;            /* grab_filter_kind */
  int32_t ts_sorted;       /* ts is non-decreasing in id: a range is a contiguous id slice */
  const uint64_t* d_ts;    /* [n]  kind TS_RANGE */
  const uint64_t* d_lo;    /* [nq] or NULL */
  const uint64_t* d_hi;    /* [nq] or NULL */
  uint64_t lo, hi;         /* used when d_lo == NULL */
  const uint8_t* d_labels; /* [n]  kind LABELS, values < 32 */
  const uint32_t* d_masks; /* [nq] or NULL */
  uint32_t mask;           /* used when d_masks == NULL */
  uint32_t active_degree;  /* kind PREFIX */
  /* kind LABELS, optional: when the vectors are grouped by label (ids of label l are
   * [d_label_offsets[l], d_label_offsets[l+1])), 33 offsets on the device let the search draw its
   * own seeds inside the query's labels */
  const uint32_t* d_label_offsets;
  /* kind TS_RANGE with ts_sorted, optional: [nq,4] uint32 scratch shared by the two calls of a routed search.
   * grab_route_seeds WRITES every query's id window (first id with ts >= lo, first id with ts >= hi, 0, 0)
   * here; grab_graph_search, given the same pointer with the same queries and ranges, READS it instead of
   * searching the timestamp column again.  NULL: each call computes what it needs. */
  uint32_t* d_id_windows;
} grab_filter;

/* Per-launch counters of the graph search (all queries summed), the inputs of the
 * algorithmic-bytes figure: bytes = 4*dim*(nq + seeds + distances) + 4*deg*parents
 * + f*edges + 12*k*nq. */
typedef struct grab_search_stats {
  uint64_t iterations;
  uint64_t parents;   /* graph rows read */
  uint64_t edges;     /* valid neighbour ids examined (before filter / visited test) */
  uint64_t distances; /* neighbour vectors read and distance-evaluated */
  uint64_t seeds;     /* seed vectors evaluated */
  uint64_t hash_resets;
} grab_search_stats;

int grab_abi_version(void);
const char* grab_status_string(int status);
const char* grab_last_error(void);
/* Stage timers of the build / insert pipelines to stderr (also GRAB_TRACE=1 in the environment);
 * the reference prints std::chrono stage times the same way (cagra_opt.cu:1962-1972). */
void grab_set_trace(int level);

/* ------------------------------------------------------------------------------------ */
/* Exact filtered brute force on the GPU: tests/test_cagra_auto.cu:57-89                 */
/* (compute_ground_truth_range) with ties broken by the lower id.  Canonical fp32 order. */
/* Missing results: id -1, dist 3.40282e38.  d_ws may be NULL (scratch is then allocated */
/* and freed inside the call).                                                           */
/* ------------------------------------------------------------------------------------ */
size_t grab_exact_search_workspace_bytes(uint64_t n, uint64_t nq, uint32_t k);
int grab_exact_search(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                      const grab_filter* filter, const float* d_queries, uint64_t nq, uint32_t k,
                      int64_t* d_out_ids, float* d_out_dists, void* d_ws, size_t ws_bytes,
                      void* stream);

/* Same scan for callers that must not allocate (a serving loop that cannot afford the device
 * synchronisation of cudaMalloc/cudaFree, a host whose memory pool already owns the GPU): the
 * scratch is a fixed GRAB_NOALLOC_SCRATCH_BYTES array inside the library, held by every GPU that
 * loads it.  Requests needing more (grab_exact_search_workspace_bytes) fail with
 * GRAB_ERR_WORKSPACE.  All calls on a device share the array: calls that overlap on the GPU
 * race.  The first call on a device resolves the array's address; with lazy module loading that
 * is also when the array is placed in device memory, so make that call before the host's pool
 * claims the GPU and before any stream capture.  This entry point has no counterpart in the
 * reference. */
#define GRAB_NOALLOC_SCRATCH_BYTES (8u << 20)
int grab_exact_search_noalloc(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                              const grab_filter* filter, const float* d_queries, uint64_t nq,
                              uint32_t k, int64_t* d_out_ids, float* d_out_dists, void* stream);

/* ------------------------------------------------------------------------------------ */
/* Filtered graph search.  One entry point for the reference's three launchers           */
/* (src/index/cagra_opt.cuh:33-80: search_opt, search_bucket_opt, search_bucket_range;   */
/* src/index/cagra.cuh:121-134: search) and their kernels (src/index/search.cu:149,      */
/* :375, :589).  itopk floor, seed-count and queue rules follow cagra_opt.cu:1108-1442.  */
/* d_seeds [nq, seeds_per_query] uint32 or NULL (pseudo-random seeds inside the filter   */
/* when the filter allows it).  id_scale/id_offset: result id = local*id_scale+id_offset */
/* (striped shards; 1/0 for a single index).  d_stats may be NULL.  d_out_keys (optional, */
/* [nq,k] uint64): the results once more as ascending keys [ordered fp32 distance : 32 |  */
/* result id : 32] (all ones = empty) -- the form the sharded exchange step gathers; needs */
/* result ids < 2^32.  With d_out_keys given, d_out_ids / d_out_dists may be NULL.         */
/* ctas_per_query: 0 or 1 = one CTA per query, the reference's algorithm (grid = queries, */
/* cagra_opt.cu:1394).  n >= 2 = n CTAs co-operate on every query (for batches too small   */
/* to fill the GPU): the budget of search_width * max_iterations expansions is spread over  */
/* n CTAs with short lists of their own, disjoint shares of the seeds and ONE visited table */
/* per query in global memory; their sorted lists are merged.  Same result FORMAT, not the  */
/* same walk: judged on recall.  GRAB_CTAS_AUTO = as many as fill the GPU, for walks of 64   */
/* expansions and more (1 for shorter walks and for batches of about a thousand queries).  */
/* Needs k <= 128; workspace size from grab_graph_search_workspace_bytes_for().             */
/* ------------------------------------------------------------------------------------ */
#define GRAB_CTAS_AUTO 0xFFFFFFFFu
typedef struct grab_search_args {
  const float* d_dataset;
  uint64_t n;
  uint32_t dim;
  int32_t metric;
  const uint32_t* d_graph;
  uint32_t graph_degree; /* row stride */
  const float* d_queries;
  uint64_t nq;
  uint32_t k;
  grab_search_params params;
  grab_filter filter;
  const uint32_t* d_seeds;
  uint32_t seeds_per_query;
  uint64_t seed; /* replaces the reference's std::random_device xor mask */
  int64_t* d_out_ids;
  float* d_out_dists;
  uint64_t id_scale, id_offset;
  grab_search_stats* d_stats;
  void* d_ws;
  size_t ws_bytes;
  void* stream;
  uint64_t* d_out_keys;
  uint32_t ctas_per_query;
} grab_search_args;

size_t grab_graph_search_workspace_bytes(uint64_t nq, uint32_t hash_bitlen);
/* the same for a filled-in argument struct (d_ws / ws_bytes ignored): covers ctas_per_query > 1 */
size_t grab_graph_search_workspace_bytes_for(const grab_search_args* args);
int grab_graph_search(const grab_search_args* args);

/* Reference-shaped wrappers (same argument order as the functions they replace, int
 * status instead of void).  They synchronise before returning. */
int grab_search(const float* d_dataset, uint32_t dim, uint64_t num_dataset, const uint32_t* d_graph,
                uint32_t graph_degree, const float* d_queries, int64_t num_queries, int64_t k,
                grab_search_params params, int64_t* d_out_indices, float* d_out_dists,
                const uint32_t* d_seeds, uint32_t num_seeds_per_query,
                void* stream); /* cagra_opt.cuh:33-46 search_opt */
int grab_search_bucket(const float* d_dataset, uint32_t dim, uint64_t num_dataset,
                       const uint32_t* d_graph, uint32_t total_degree, uint32_t local_degree,
                       const float* d_queries, int64_t num_queries, int64_t k,
                       grab_search_params params, int64_t* d_out_indices, float* d_out_dists,
                       const uint32_t* d_seeds, uint32_t num_seeds_per_query,
                       void* stream); /* cagra_opt.cuh:48-62 search_bucket_opt */
int grab_search_range(const float* d_dataset, uint32_t dim, uint64_t num_dataset,
                      const uint32_t* d_graph, const uint64_t* d_ts, uint32_t total_degree,
                      uint32_t local_degree, const float* d_queries, int64_t num_queries, int64_t k,
                      uint64_t start_bucket, uint64_t end_bucket, grab_search_params params,
                      int64_t* d_out_indices, float* d_out_dists, const uint32_t* d_seeds,
                      uint32_t num_seeds_per_query); /* cagra_opt.cuh:64-80 search_bucket_range */

/* ------------------------------------------------------------------------------------ */
/* kNN graph.                                                                            */
/* grab_knn_graph_blocks: exact kNN inside each contiguous id block (self dropped, short */
/* rows padded with 0xFFFFFFFF, GLOBAL ids) -- src/index/raft_help.cuh:74-172            */
/* build_batch_knn_graphs plus the offsetting of cagra_opt.cu:1038-1044.                 */
/* h_block_offsets: host array [num_blocks+1].  mode 0: own block; mode 1: every vector  */
/* EXCEPT those of the own block (candidates for cross-bucket edges, the role of the     */
/* IVF-PQ self-search of cagra_opt.cu:813-856).  Output ascending exact distance.        */
/* precision: GRAB_KNN_EXACT_SCAN = every pair in canonical fp32 (SIMT scan);            */
/* GRAB_KNN_TC_BF16 / GRAB_KNN_TC_SPLIT = all-pairs tile on the tcgen05 tensor cores     */
/* (bf16, or hi+lo split bf16 ~ fp32 products), fused per-row top-(k+k/4) and an exact   */
/* fp32 re-rank of those candidates (k <= 204).                                          */
/* grab_generate_knn_graph: src/index/cagra.cuh:59-63 (device dataset, HOST output).     */
/* ------------------------------------------------------------------------------------ */
enum grab_knn_precision { GRAB_KNN_EXACT_SCAN = 0, GRAB_KNN_TC_BF16 = 1, GRAB_KNN_TC_SPLIT = 2 };
int grab_knn_graph_blocks(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                          const uint64_t* h_block_offsets, uint32_t num_blocks, uint32_t k,
                          int mode, int precision, uint32_t* d_out_knn, float* d_out_dists,
                          void* stream);
int grab_generate_knn_graph(const float* d_dataset, uint64_t num_dataset, uint32_t dim, uint32_t k,
                            uint32_t* h_knn_graph);

/* ------------------------------------------------------------------------------------ */
/* Graph optimisation.  *_device variants take device graphs and a stream; the           */
/* reference-shaped ones take HOST graphs as src/index/cagra.cuh:72-107 do.              */
/* prune: cagra.cu:219-276 + 367-392.  reverse: cagra.cu:418-444, 455-548 (slot order =  */
/* column, then ascending source id).  merge: cagra.cu:574-650.                          */
/* ------------------------------------------------------------------------------------ */
int grab_optimize_prune_device(const uint32_t* d_knn, uint32_t* d_out, uint64_t n,
                               uint32_t input_degree, uint32_t output_degree,
                               uint8_t* d_detour_or_null, void* stream);
int grab_optimize_reverse_graph_device(const uint32_t* d_graph, uint32_t* d_rev,
                                       uint32_t* d_rev_counts, uint64_t n, uint32_t degree,
                                       void* stream);
int grab_optimize_merge_graphs_device(uint32_t* d_graph, const uint32_t* d_rev,
                                      const uint32_t* d_rev_counts, uint64_t n, uint32_t degree,
                                      void* stream);
int grab_optimize_prune(const uint32_t* h_knn_graph, uint32_t* h_new_graph, uint64_t num_dataset,
                        uint32_t input_degree, uint32_t output_degree);
int grab_optimize_create_reverse_graph(const uint32_t* h_input_graph, uint32_t* h_rev_graph,
                                       uint32_t* h_rev_counts, uint64_t num_dataset,
                                       uint32_t degree);
int grab_optimize_merge_graphs(uint32_t* h_graph, const uint32_t* h_rev_graph,
                               const uint32_t* h_rev_counts, uint64_t num_dataset, uint32_t degree);
/* cagra.cuh:109-119 build: raw kNN graph (device) -> prune/reverse/merge -> a cudaMalloc'd
 * graph the caller frees with cudaFree. */
int grab_build(const float* d_dataset, uint64_t num_dataset, const uint32_t* d_raw_knn_graph,
               grab_build_params params, uint32_t** d_constructed_graph);

/* Cross-bucket edges: cagra_opt.cu:209-303 (selection) and :457-600, :739-790 (reverse
 * injection).  d_cand [n, gk] is consumed.  d_bucket [n]: bucket id per vector. */
int grab_remote_edges_device(uint32_t* d_graph, const uint64_t* d_bucket, uint32_t* d_cand,
                             uint64_t n, uint32_t total_degree, uint32_t local_degree, uint32_t gk,
                             void* stream);
int grab_inject_reverse_remote_device(uint32_t* d_graph, uint64_t n, uint32_t total_degree,
                                      uint32_t local_degree, uint32_t max_rev, void* stream);
/* cagra_opt.cuh:21-31 build_time_partitioned_graph: per-bucket local graphs of width
 * total_degree, then cross-bucket edges over columns >= local_degree.  h_bucket_sizes: host. */
int grab_build_time_partitioned_graph(const float* d_dataset, uint64_t total_num, uint32_t dim,
                                      int metric, uint32_t* d_graph, const uint64_t* d_bucket,
                                      const uint64_t* h_bucket_sizes, uint32_t num_buckets,
                                      uint32_t total_degree, uint32_t local_degree,
                                      int knn_precision);
/* The same build with its choices spelled out.  Cross-bucket candidates (the reference's
 * IVF-PQ search over the whole dataset, cagra_opt.cu:813-847) come either from the all-pairs
 * tensor-core kernel (exact top candidates, quadratic in N) or from a routed graph search over
 * the local edges (approximate, linear in N); AUTO takes all-pairs below 2^19 vectors, the routed search
 * with 6 parents x 12 iterations below 2^21 and with 4 x 10 from there on. */
enum grab_global_candidates { GRAB_GLOBAL_AUTO = 0, GRAB_GLOBAL_ALL_PAIRS = 1, GRAB_GLOBAL_ROUTED_SEARCH = 2 };
typedef struct grab_tp_build_options {
  int knn_precision;      /* grab_knn_precision */
  int global_candidates;  /* grab_global_candidates */
  uint32_t search_iterations; /* routed search: iterations per vector (0 = 10; AUTO: see above) */
  uint32_t search_width;      /* routed search: parents per iteration (0 = 4; AUTO: see above) */
} grab_tp_build_options;
int grab_build_time_partitioned_graph_ex(const float* d_dataset, uint64_t total_num, uint32_t dim,
                                         int metric, uint32_t* d_graph, const uint64_t* d_bucket,
                                         const uint64_t* h_bucket_sizes, uint32_t num_buckets,
                                         uint32_t total_degree, uint32_t local_degree,
                                         const grab_tp_build_options* options);

/* ------------------------------------------------------------------------------------ */
/* Insert: topology updates.  v1: src/index/insert.cuh:62-72 (insert.cu:225-440).        */
/* opt: src/index/insert.cuh:96-116 (insert.cu:448-765, 1398-1573); mailbox order is     */
/* ascending new id, then column.                                                        */
/* ------------------------------------------------------------------------------------ */
int grab_update_topology_v1(uint32_t* d_graph, const int64_t* d_search_indices,
                            uint64_t num_existing, uint64_t num_new, uint32_t graph_degree,
                            uint32_t search_k, void* stream);
int grab_update_topology_opt(uint32_t* d_graph, const uint64_t* d_bucket, int64_t* d_local_knn,
                             int64_t* d_global_knn, uint64_t num_existing, uint64_t num_new,
                             uint64_t target_bucket, uint32_t total_degree, uint32_t local_degree,
                             uint32_t k_local, uint32_t k_global, void* stream);

/* Neighbour search for new vectors over the first num_existing nodes: insert.cuh:38-60
 * find_near_nodes (exact distances, ascending). */
int grab_find_near_nodes(const float* d_dataset, uint64_t num_existing, const float* d_queries,
                         uint64_t num_queries, const uint32_t* d_graph, uint32_t dim,
                         uint32_t graph_degree, uint32_t search_k, grab_search_params params,
                         int64_t* d_out_indices, float* d_out_dists);
/* cagra.cuh:136-146 insert (v1): search_k = 2*degree search + v1 topology update.  The new
 * vectors are rows [num_existing, num_existing+num_new) of d_dataset / d_graph. */
int grab_insert(const float* d_dataset, uint64_t num_existing, uint64_t num_new,
                const float* d_new_vectors, uint32_t* d_graph, uint32_t dim, uint32_t graph_degree,
                grab_search_params params);
/* cagra_opt.cuh:82-93 insert (time-partitioned): global search + bucket search from d_seeds
 * [num_new, num_seeds_per_query] + exact kNN inside the batch, then the opt topology update.
 * All new vectors belong to bucket target_ts; d_ts holds the bucket id of every vector. */
int grab_insert_opt(const float* d_dataset, uint32_t* d_graph, const uint64_t* d_ts,
                    const uint32_t* d_seeds, uint64_t num_existing, uint64_t num_new,
                    int use_heuristic, uint64_t target_ts, const float* d_queries, uint32_t dim,
                    uint32_t total_degree, uint32_t local_degree, grab_search_params params,
                    uint32_t num_seeds_per_query);

/* ------------------------------------------------------------------------------------ */
/* Merge of `parts` ascending top-k lists per query into one (the exchange step of the   */
/* id-sharded multi-GPU search; also merges the splits of the exact scan).  No reference */
/* counterpart (the reference is single-GPU).  Lists [nq, parts, k]; ids < 0 are empty.  */
/* ------------------------------------------------------------------------------------ */
int grab_merge_topk(const float* d_dists, const int64_t* d_ids, uint64_t nq, uint32_t parts,
                    uint32_t k, int64_t* d_out_ids, float* d_out_dists, void* stream);

/* ------------------------------------------------------------------------------------ */
/* Id-sharded multi-GPU search: one process per GPU, ids striped gid % G == rank, the same */
/* queries on every rank, per-shard results exchanged with ONE all-gather and merged on the */
/* device.  No reference counterpart (its device is fixed at compile time,                 */
/* src/index/common.cuh:5-7).                                                             */
/* grab_merge_sorted_keys: d_keys [parts, nq, run_length] ascending keys as written to       */
/* grab_search_args.d_out_keys -> global top-k by (dist, id); a G-way merge by rank           */
/* computation (no sort).  Missing results: id -1, dist 3.40282e38.                          */
/* grab_comm_*: a communicator over NCCL (loaded at run time; GRAB_ERR_NCCL when it is        */
/* missing or a call fails).  Rank 0 makes the unique id, the host passes it to every rank    */
/* (any side channel), every rank calls grab_comm_create with its device current.             */
/* grab_sharded_gather_merge: all-gather of this rank's [nq, run_length] keys into d_gather   */
/* [world, nq, run_length] + the merge, both enqueued on `stream`; comm == NULL means one     */
/* shard.  Every rank must call it with the same nq / run_length / k.                         */
/* ------------------------------------------------------------------------------------ */
int grab_merge_sorted_keys(const uint64_t* d_keys, uint64_t nq, uint32_t parts, uint32_t run_length,
                           uint32_t k, int64_t* d_out_ids, float* d_out_dists, void* stream);
#define GRAB_COMM_UNIQUE_ID_BYTES 128
typedef struct grab_comm grab_comm;
int grab_comm_unique_id(void* out, size_t bytes);
int grab_comm_create(const void* unique_id, int world, int rank, grab_comm** out);
int grab_comm_destroy(grab_comm* comm);
int grab_comm_world(const grab_comm* comm);
int grab_comm_rank(const grab_comm* comm);
int grab_sharded_gather_merge(grab_comm* comm, const uint64_t* d_keys, uint64_t nq, uint32_t run_length,
                              uint32_t k, uint64_t* d_gather, size_t gather_bytes, int64_t* d_out_ids,
                              float* d_out_dists, void* stream);

/* ------------------------------------------------------------------------------------ */
/* Entry-point router: search seeds that pass the filter AND lie close to the query.     */
/* Device version of the reference's host seed sampling (cagraIndexOpt.cu:441-511 for    */
/* query_range, :313-336 for query_local; cagraIndex.cu:267-296) combined with the       */
/* k-means routing of its two-level index (timeStampIndex.cu:141-238 build_virtual_index,*/
/* :240-419 query).  The seed array it writes is the d_seeds / num_seeds_per_query input */
/* of grab_search, grab_search_bucket, grab_search_range and grab_graph_search.          */
/* ------------------------------------------------------------------------------------ */
typedef struct grab_router {
  uint32_t num_centroids;
  uint32_t dim;
  int metric;                       /* grab_metric the centroids were trained for */
  const float* d_centroids;         /* [num_centroids, dim] */
  const float* d_centroid_norms;    /* [num_centroids] squared norms */
  const uint32_t* d_member_offsets; /* [num_centroids + 1] */
  const uint32_t* d_members;        /* [n] ids grouped by nearest centroid, ascending inside a group */
  uint32_t flags;                   /* GRAB_ROUTER_* */
} grab_router;
/* grab_route_seeds ranks the centroids with the exact fp32 scan instead of the tensor cores
 * (tf32 products, probes + 4 candidates re-scored exactly).  Both give the same seeds unless
 * tf32 rounding moves a centroid more than four ranks. */
#define GRAB_ROUTER_EXACT_SCAN 1u

/* Trains `num_centroids` centroids (Lloyd, `iterations` rounds over a strided sample of
 * max_sample rows; 0 = 64 per centroid), assigns all n vectors and writes the four arrays a
 * grab_router points to (caller-allocated: [C,dim], [C], [C+1], [n]).  iterations == 0 keeps
 * the centroids and norms found in d_centroids / d_centroid_norms and only re-assigns (after
 * inserts).  Deterministic; synchronises the stream before returning. */
int grab_router_build(const float* d_dataset, uint32_t dim, uint64_t n, int metric, uint32_t num_centroids,
                      uint32_t iterations, uint64_t max_sample, float* d_centroids, float* d_centroid_norms,
                      uint32_t* d_member_offsets, uint32_t* d_members, void* stream);
/* The `probes` (1..16) nearest centroids of m rows, best first: d_out u32[m, probes]. */
int grab_nearest_centroids(const grab_router* router, const float* d_rows, uint64_t m, uint32_t probes,
                           uint32_t* d_out, void* stream);
size_t grab_route_seeds_workspace_bytes(uint64_t nq, uint32_t probes);
/* d_seeds u32[nq, seeds_per_query]: members of the `probes` nearest centroids that pass
 * `filter` (NULL = no filter; id windows for sorted timestamps and for labels with
 * d_label_offsets, predicate tests otherwise); 0xFFFFFFFF where nothing was found.  n = number
 * of indexed vectors.  d_ws may be NULL (then the call allocates and synchronises). */
int grab_route_seeds(const grab_router* router, const float* d_queries, uint64_t nq, uint64_t n,
                     const grab_filter* filter, uint32_t probes, uint32_t seeds_per_query, uint64_t seed,
                     uint32_t* d_seeds, void* d_ws, size_t ws_bytes, void* stream);
/* Outcome of the last grab_route_seeds that used the caller's workspace d_ws (the call itself only
 * enqueues work): waits for `stream`, reads the status word at offset 0 of the workspace and returns
 * GRAB_OK, or GRAB_ERR_TIMEOUT when the tensor-core centroid ranking gave up on a bounded wait (every
 * seed of that batch was then written as 0xFFFFFFFF and the search fell back to its own draws).  A call
 * without a workspace reports the same through its own return value. */
int grab_route_status(const void* d_ws, void* stream);

/* ------------------------------------------------------------------------------------ */
/* Device-level unit-test entry points for the search building blocks (not on the search */
/* path).  They run the code of csrc/search_blocks.cuh as graph_search_kernel instantiates */
/* it, so that the reference's own known-answer tests apply to it:                        */
/* tests/test_bitonic.cu:73-156 and tests/test_sort_impl.cu:111-121 (warp sort == sorted   */
/* input) and tests/test_hashmap.cu:144-187 (successful inserts == unique keys).          */
/* ------------------------------------------------------------------------------------ */
/* Per list (one warp each): the m sorted keys d_top[list] and ncand unsorted keys            */
/* d_cand[list, 0..ncand) -> the m smallest of their union, ascending, in d_out[list].        */
/* m: power of two in [64,1024].  variant 0 = the routine the shared-list kernel picks for     */
/* this m (registers for 64 and 128, shared memory above), 1 = the shared-memory routine,     */
/* 2 = merge by rank (ncand <= 32, m 64 / 128), 3 = the candidates as two register-sorted     */
/* runs folded into the list (ncand <= 256, m 64 / 128) -- the two paths of the warp-split    */
/* kernel.                                                                                    */
int grab_selftest_sort_merge(const uint64_t* d_top, const uint64_t* d_cand, uint64_t lists, uint32_t m,
                             uint32_t ncand, uint32_t cand_stride, int variant, uint64_t* d_out,
                             void* stream);
/* One CTA of `threads` threads inserts d_keys[0..nkeys) concurrently into an empty visited     */
/* table of 2^hash_bitlen slots (shared memory up to 2^13, as in the kernel); d_success[i] = 1  */
/* when key i was new; d_table [2^hash_bitlen] receives the final table.                        */
int grab_selftest_hash_insert(uint32_t* d_table, uint32_t hash_bitlen, const uint32_t* d_keys,
                              uint32_t nkeys, uint32_t threads, uint32_t* d_success, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GRAB_ANNS_H_ */
