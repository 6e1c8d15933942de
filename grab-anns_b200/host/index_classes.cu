// Host-side index classes (reference surface) on top of the C ABI.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <exception>
#include <fstream>
#include <mutex>
#include <random>
#include <stdexcept>

#include "cagraIndex.hpp"
#include "cagraIndexOpt.cuh"
#include "../csrc/common.cuh"
#include "timeStampIndex.cuh"

namespace grab {
int insert_v1_impl(const float*, uint64_t, uint64_t, const float*, uint32_t*, uint32_t, uint32_t, grab_search_params, int);
int insert_opt_impl(const float*, uint32_t*, const uint64_t*, const uint32_t*, uint64_t, uint64_t, uint64_t, const float*,
                    uint32_t, uint32_t, uint32_t, grab_search_params, uint32_t, int, const InsertOptions*);
}  // namespace grab

namespace {

void ok(int rc, const char* what) {
  if (rc != GRAB_OK) throw grab::StatusError(rc, std::string(what) + ": " + grab_last_error());
}
void cu(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw grab::StatusError(GRAB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

struct Scratch {
  void* p = nullptr;
  explicit Scratch(size_t bytes) { cu(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc"); }
  ~Scratch() { cudaFree(p); }
  template <class T> T* as() { return static_cast<T*>(p); }
};

// Uniform sample without replacement of `want` ids (all of them when fewer), the role of
// std::sample in the reference's seed selection (src/cagraIndexOpt.cu:313-336, 441-474).
std::vector<uint32_t> sample_ids(const std::vector<uint32_t>& ids, size_t want, uint64_t seed) {
  if (ids.size() <= want) return ids;
  std::vector<uint32_t> out;
  out.reserve(want);
  std::mt19937_64 rng(seed);
  std::sample(ids.begin(), ids.end(), std::back_inserter(out), want, rng);
  return out;
}

grab_search_args make_args(const float* d_data, uint64_t n, uint32_t dim, int metric, const uint32_t* d_graph,
                           uint32_t deg, const float* d_q, uint64_t nq, uint32_t k, grab_search_params p,
                           int64_t* ids, float* dists, uint64_t seed) {
  grab_search_args a;
  memset(&a, 0, sizeof(a));
  a.d_dataset = d_data; a.n = n; a.dim = dim; a.metric = metric; a.d_graph = d_graph; a.graph_degree = deg;
  a.d_queries = d_q; a.nq = nq; a.k = k; a.params = p; a.seed = seed;
  a.d_out_ids = ids; a.d_out_dists = dists; a.id_scale = 1;
  return a;
}

}  // namespace

// Per-index query scratch that survives across calls (grow-only): device copies of the queries, per-query
// ranges, seeds and results, the routing and search workspaces, page-locked staging for the caller's pageable
// arrays (filled and drained by a few host threads, so that the PCIe copies themselves are asynchronous and run
// at link speed), and two streams.  The reference allocates and
// frees all of this inside every query call (src/index/cagra_opt.cu:1136-1206: cudaMalloc / cudaFree plus two
// device-wide synchronisations per call); here a query performs no allocation once the largest batch has been
// seen.  Batches of 4096 queries and more are cut in two (8192 and more: four) parts on as many streams, so that
// the host-to-device copy of one part overlaps the search of the part before it and the result copy of that part
// the search of the next.  One caller at a time per index (the mutex serialises others), as in the reference.
namespace grab {
struct QueryArena {
  struct Buf {
    void* p = nullptr;
    size_t cap = 0;
    void need(size_t bytes) {
      if (bytes <= cap) return;
      if (p) cudaFree(p);
      p = nullptr;
      cap = 0;
      const size_t want = bytes + bytes / 4 + 256;
      cu(cudaMalloc(&p, want), "cudaMalloc (query scratch)");
      cap = want;
    }
    ~Buf() { if (p) cudaFree(p); }
    template <class T> T* as() { return static_cast<T*>(p); }
  };
  struct Pinned {  // page-locked host staging, grow-only
    void* p = nullptr;
    size_t cap = 0;
    void need(size_t bytes) {
      if (bytes <= cap) return;
      if (p) cudaFreeHost(p);
      p = nullptr;
      cap = 0;
      const size_t want = bytes + bytes / 4 + 256;
      cu(cudaHostAlloc(&p, want, cudaHostAllocDefault), "cudaHostAlloc (query staging)");
      cap = want;
    }
    ~Pinned() { if (p) cudaFreeHost(p); }
    template <class T> T* as() { return static_cast<T*>(p); }
  };
  struct Slot {
    cudaStream_t st = nullptr;
    Buf q, lo, hi, ids, dists, seeds, search_ws, route_ws, windows;
    Pinned h_in, h_out;  // [queries | lo | hi | seeds] and [ids | dists] of this half-batch
    ~Slot() { if (st) cudaStreamDestroy(st); }
  };
  static constexpr int kSlots = 4;
  Slot slot[kSlots];
  std::mutex mu;
};
void QueryArenaDeleter::operator()(QueryArena* a) const { delete a; }
}  // namespace grab

namespace {

grab::QueryArena& arena_of(std::unique_ptr<grab::QueryArena, grab::QueryArenaDeleter>& holder) {
  if (!holder) holder.reset(new grab::QueryArena());
  return *holder;
}

// memcpy by up to 8 host threads (a single thread moves ~10 GB/s, the PCIe link five times that)
void parallel_copy(void* dst, const void* src, size_t bytes) {
  constexpr size_t kPiece = 256 << 10;
  const long pieces = static_cast<long>((bytes + kPiece - 1) / kPiece);
  if (pieces <= 2) { memcpy(dst, src, bytes); return; }
#pragma omp parallel for num_threads(8) schedule(static)
  for (long i = 0; i < pieces; ++i) {
    const size_t off = static_cast<size_t>(i) * kPiece;
    memcpy(static_cast<char*>(dst) + off, static_cast<const char*>(src) + off, std::min(kPiece, bytes - off));
  }
}

// queries up, one filtered search (routed seeds, caller's seeds, or the kernel's own draws), results down.
// host_lo / host_hi: per-query ranges (NULL = the one range already in a.filter).
void run_search(grab::QueryArena& A, grab_search_args a, const float* host_q, size_t nq, uint32_t dim, int k,
                const uint32_t* host_seeds, size_t seeds_per_query, bool broadcast_seeds, const uint64_t* host_lo,
                const uint64_t* host_hi, int64_t* host_ids, float* host_dists, const grab_router* router = nullptr,
                uint32_t probes = 0, uint32_t routed_seeds = 0, bool exact_scan = false) {
  std::lock_guard<std::mutex> lock(A.mu);
  if (exact_scan) { router = nullptr; host_seeds = nullptr; seeds_per_query = 0; }
  const bool own_seeds = host_seeds && seeds_per_query;
  std::vector<uint32_t> expanded;
  if (own_seeds && broadcast_seeds) {
    expanded.resize(nq * seeds_per_query);
    for (size_t i = 0; i < nq; ++i) memcpy(expanded.data() + i * seeds_per_query, host_seeds, seeds_per_query * 4);
    host_seeds = expanded.data();
  }
  const size_t chunks = nq >= 8192 ? 4 : (nq >= 4096 ? 2 : 1);
  const size_t per = (nq + chunks - 1) / chunks;
  size_t count[grab::QueryArena::kSlots] = {0, 0, 0, 0};
  for (size_t c = 0; c < chunks; ++c) {
    grab::QueryArena::Slot& s = A.slot[c];
    const size_t q0 = c * per, m = std::min(per, nq - q0);
    count[c] = m;
    if (!s.st) cu(cudaStreamCreateWithFlags(&s.st, cudaStreamNonBlocking), "cudaStreamCreate");
    s.q.need(m * dim * sizeof(float));
    s.ids.need(m * k * sizeof(int64_t));
    s.dists.need(m * k * sizeof(float));
    // stage this half-batch in page-locked memory: [queries | lo | hi | seeds]
    const size_t qb = m * dim * sizeof(float), rb = host_lo ? m * sizeof(uint64_t) : 0;
    const size_t sb = own_seeds ? m * seeds_per_query * sizeof(uint32_t) : 0;
    s.h_in.need(qb + 2 * rb + sb);
    char* hin = s.h_in.as<char>();
    parallel_copy(hin, host_q + q0 * dim, qb);
    cu(cudaMemcpyAsync(s.q.p, hin, qb, cudaMemcpyHostToDevice, s.st), "H2D queries");
    grab_search_args ac = a;
    if (host_lo) {
      s.lo.need(rb);
      s.hi.need(rb);
      memcpy(hin + qb, host_lo + q0, rb);
      memcpy(hin + qb + rb, host_hi + q0, rb);
      cu(cudaMemcpyAsync(s.lo.p, hin + qb, rb, cudaMemcpyHostToDevice, s.st), "H2D range");
      cu(cudaMemcpyAsync(s.hi.p, hin + qb + rb, rb, cudaMemcpyHostToDevice, s.st), "H2D range");
      ac.filter.d_lo = s.lo.as<uint64_t>();
      ac.filter.d_hi = s.hi.as<uint64_t>();
    }
    ac.d_queries = s.q.as<float>();
    ac.nq = m;
    ac.d_out_ids = s.ids.as<int64_t>();
    ac.d_out_dists = s.dists.as<float>();
    ac.stream = s.st;
    if (router && !own_seeds) {
      // seeds from the entry-point router: members of the nearest centroids that pass the filter
      const size_t rws = grab_route_seeds_workspace_bytes(m, probes);
      s.route_ws.need(rws);
      s.seeds.need(m * routed_seeds * sizeof(uint32_t));
      if (ac.filter.kind == GRAB_FILTER_TS_RANGE && ac.filter.ts_sorted) {
        // the router leaves every query's id window here and the search reads it
        s.windows.need(m * 4 * sizeof(uint32_t));
        ac.filter.d_id_windows = s.windows.as<uint32_t>();
      }
      ok(grab_route_seeds(router, s.q.as<float>(), m, a.n, &ac.filter, probes, routed_seeds, a.seed,
                          s.seeds.as<uint32_t>(), s.route_ws.p, rws, s.st), "seed routing");
      ac.d_seeds = s.seeds.as<uint32_t>();
      ac.seeds_per_query = routed_seeds;
    } else if (own_seeds) {
      s.seeds.need(sb);
      parallel_copy(hin + qb + 2 * rb, host_seeds + q0 * seeds_per_query, sb);
      cu(cudaMemcpyAsync(s.seeds.p, hin + qb + 2 * rb, sb, cudaMemcpyHostToDevice, s.st), "H2D seeds");
      ac.d_seeds = s.seeds.as<uint32_t>();
      ac.seeds_per_query = static_cast<uint32_t>(seeds_per_query);
    }
    if (exact_scan) {
      // a range this narrow holds fewer vectors than a walk would visit: scan it (exact, and cheaper)
      const size_t sws = grab_exact_search_workspace_bytes(a.n, m, static_cast<uint32_t>(k));
      s.search_ws.need(sws);
      ok(grab_exact_search(ac.d_dataset, ac.n, ac.dim, ac.metric, &ac.filter, ac.d_queries, m, static_cast<uint32_t>(k),
                           ac.d_out_ids, ac.d_out_dists, s.search_ws.p, sws, s.st), "exact scan");
    } else {
      const size_t sws = grab_graph_search_workspace_bytes_for(&ac);
      s.search_ws.need(sws);
      ac.d_ws = s.search_ws.p;
      ac.ws_bytes = sws;
      ok(grab_graph_search(&ac), "graph search");
    }
    // results of this half leave as soon as its search is done, while the other half is staged and searched
    const size_t ib = m * k * sizeof(int64_t), db = m * k * sizeof(float);
    s.h_out.need(ib + db);
    cu(cudaMemcpyAsync(s.h_out.p, s.ids.p, ib, cudaMemcpyDeviceToHost, s.st), "D2H ids");
    cu(cudaMemcpyAsync(s.h_out.as<char>() + ib, s.dists.p, db, cudaMemcpyDeviceToHost, s.st), "D2H dists");
  }
  for (size_t c = 0; c < chunks; ++c) {
    grab::QueryArena::Slot& s = A.slot[c];
    const size_t q0 = c * per, m = count[c];
    cu(cudaStreamSynchronize(s.st), "query stream");
    if (router && !own_seeds) ok(grab_route_status(s.route_ws.p, s.st), "seed routing");
    const size_t ib = m * k * sizeof(int64_t), db = m * k * sizeof(float);
    parallel_copy(host_ids + q0 * k, s.h_out.p, ib);
    parallel_copy(host_dists + q0 * k, s.h_out.as<char>() + ib, db);
  }
}

void fill_no_data(int64_t* ids, float* dists, size_t count) {  // src/cagraIndexOpt.cu:341-347, 479-485
  for (size_t i = 0; i < count; ++i) { ids[i] = -1; dists[i] = -1.0f; }
}

}  // namespace

namespace cagra {

// =====================================================================================
// CagraIndex (reference: src/cagraIndex.cu)
// =====================================================================================
CagraIndex::CagraIndex(uint32_t dim, uint32_t graph_degree, size_t vmm_max_bytes)
    : dim_(dim), graph_degree_(graph_degree) {
  if (dim == 0 || dim % 4 != 0) throw std::runtime_error("CagraIndex: dim must be a positive multiple of 4");
  // capacity split 70 / 20 / 10 (src/cagraIndex.cu:14-20)
  d_data_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.70)));
  d_graph_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.20)));
  d_ts_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.10)));
  build_params_ = {std::max(128u, graph_degree * 2), graph_degree};  // src/cagraIndex.cu:22-24
  search_params_ = {256, 6, 1, 50, 13};                              // src/cagraIndex.cu:26-31
  insert_params_ = {128, 4, 0, 50, 13};
}
CagraIndex::~CagraIndex() = default;

void CagraIndex::upload_timestamps() {
  d_ts_->resize(h_timestamps_.size() * sizeof(uint64_t));
  cu(cudaMemcpy(d_ts_->data(), h_timestamps_.data(), h_timestamps_.size() * sizeof(uint64_t), cudaMemcpyHostToDevice),
     "H2D timestamps");
}

void CagraIndex::add(size_t num_vectors, const float* add_vectors, const uint64_t* add_timestamps) {
  if (num_vectors == 0) return;
  const size_t start = h_data_.size() / dim_;
  h_data_.insert(h_data_.end(), add_vectors, add_vectors + num_vectors * dim_);
  if (add_timestamps) {
    for (size_t i = 0; i < num_vectors; ++i) {
      const uint64_t ts = add_timestamps[i];
      if (!h_timestamps_.empty() && ts < h_timestamps_.back()) ts_sorted_ = false;
      h_timestamps_.push_back(ts);
      ts_to_ids_[ts].push_back(static_cast<uint32_t>(start + i));
    }
    upload_timestamps();
  }
}

void CagraIndex::build() {
  const size_t n = h_data_.size() / dim_;
  if (n == 0) return;
  current_size_ = n;
  d_data_->resize(n * dim_ * sizeof(float));
  cu(cudaMemcpy(d_data_->data(), h_data_.data(), n * dim_ * sizeof(float), cudaMemcpyHostToDevice), "H2D dataset");
  const uint32_t inter = build_params_.intermediate_degree;
  Scratch knn(n * inter * sizeof(uint32_t));
  const uint64_t offs[2] = {0, n};
  ok(grab_knn_graph_blocks(static_cast<float*>(d_data_->data()), n, dim_, metric_, offs, 1, inter, 0,
                           inter <= 204 ? knn_precision_ : GRAB_KNN_EXACT_SCAN, knn.as<uint32_t>(), nullptr, nullptr),
     "kNN graph");
  uint32_t* d_built = nullptr;
  grab_build_params bp = build_params_;
  bp.graph_degree = graph_degree_;
  ok(grab_build(static_cast<float*>(d_data_->data()), n, knn.as<uint32_t>(), bp, &d_built), "graph build");
  const size_t gbytes = n * graph_degree_ * sizeof(uint32_t);
  d_graph_->resize(gbytes);
  cu(cudaMemcpy(d_graph_->data(), d_built, gbytes, cudaMemcpyDeviceToDevice), "graph copy");
  cudaFree(d_built);
  h_graph_.resize(n * graph_degree_);
  cu(cudaMemcpy(h_graph_.data(), d_graph_->data(), gbytes, cudaMemcpyDeviceToHost), "D2H graph");
}

void CagraIndex::insert(size_t new_vectors, const float* insert_vectors, const uint64_t* insert_timestamps) {
  if (new_vectors == 0) return;
  if (current_size_ == 0) {  // src/cagraIndex.cu:134-139
    add(new_vectors, insert_vectors, insert_timestamps);
    build();
    return;
  }
  const size_t old_size = current_size_, new_size = old_size + new_vectors;
  add(new_vectors, insert_vectors, insert_timestamps);
  d_data_->resize(new_size * dim_ * sizeof(float));
  d_graph_->resize(new_size * graph_degree_ * sizeof(uint32_t));
  float* d_data = static_cast<float*>(d_data_->data());
  uint32_t* d_graph = static_cast<uint32_t*>(d_graph_->data());
  cu(cudaMemcpy(d_data + old_size * dim_, insert_vectors, new_vectors * dim_ * sizeof(float), cudaMemcpyHostToDevice),
     "H2D new vectors");
  for (size_t off = 0; off < new_vectors; off += insert_batch_) {
    const size_t cur = std::min(insert_batch_, new_vectors - off);
    ok(grab::insert_v1_impl(d_data, old_size + off, cur, d_data + (old_size + off) * dim_, d_graph, dim_, graph_degree_,
                            insert_params_, metric_),
       "insert");
  }
  current_size_ = new_size;
}

const uint32_t* CagraIndex::get_graph() {
  h_graph_.resize(current_size_ * graph_degree_);
  if (current_size_)
    cu(cudaMemcpy(h_graph_.data(), d_graph_->data(), h_graph_.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost), "D2H graph");
  return h_graph_.data();
}

void CagraIndex::query(const float* host_queries, size_t num_queries, int k, int64_t* host_indices, float* host_dists,
                       uint32_t* seeds, size_t num_seeds_per_query) {
  if (current_size_ == 0 || num_queries == 0) return;
  grab_search_args a = make_args(static_cast<float*>(d_data_->data()), current_size_, dim_, metric_,
                                 static_cast<uint32_t*>(d_graph_->data()), graph_degree_, nullptr, num_queries, k,
                                 search_params_, nullptr, nullptr, seed_);
  a.ctas_per_query = ctas_per_query_;
  a.filter.kind = GRAB_FILTER_NONE;
  run_search(arena_of(arena_), a, host_queries, num_queries, dim_, k, seeds, num_seeds_per_query, false, nullptr,
             nullptr, host_indices, host_dists);
}

void CagraIndex::query_range(const float* host_queries, size_t num_queries, int k, float range_radius, uint64_t start_ts,
                             uint64_t end_ts, int64_t* host_indices, float* host_dists, uint32_t* seeds,
                             size_t num_seeds_per_query) {
  if (current_size_ == 0 || num_queries == 0) return;
  if (range_radius >= 0.99f) {  // src/cagraIndex.cu:305-338: near-full ranges take the unfiltered search
    query(host_queries, num_queries, k, host_indices, host_dists, seeds, num_seeds_per_query);
    return;
  }
  if (h_timestamps_.size() < current_size_) throw std::runtime_error("query_range: the index holds no timestamps");
  grab_search_args a = make_args(static_cast<float*>(d_data_->data()), current_size_, dim_, metric_,
                                 static_cast<uint32_t*>(d_graph_->data()), graph_degree_, nullptr, num_queries, k,
                                 search_params_, nullptr, nullptr, seed_);
  a.ctas_per_query = ctas_per_query_;
  a.filter.kind = GRAB_FILTER_TS_RANGE;
  a.filter.d_ts = static_cast<uint64_t*>(d_ts_->data());
  a.filter.lo = start_ts;
  a.filter.hi = end_ts;
  a.filter.ts_sorted = ts_sorted_;
  // vectors inside the range (each map entry is one timestamp here)
  size_t in_range_count = 0;
  for (auto it = ts_to_ids_.lower_bound(start_ts); it != ts_to_ids_.end() && it->first < end_ts; ++it) {
    in_range_count += it->second.size();
    if (in_range_count > exact_below_) break;
  }
  if (in_range_count == 0) { fill_no_data(host_indices, host_dists, num_queries * k); return; }
  if (in_range_count <= exact_below_) {
    run_search(arena_of(arena_), a, host_queries, num_queries, dim_, k, nullptr, 0, false, nullptr, nullptr, host_indices,
               host_dists, nullptr, 0, 0, true);
    return;
  }
  std::vector<uint32_t> sampled;
  if (!ts_sorted_) {
    // one seed list for all queries, drawn from the ids inside the range (src/cagraIndex.cu:267-296)
    std::vector<uint32_t> in_range;
    for (auto it = ts_to_ids_.lower_bound(start_ts); it != ts_to_ids_.end() && it->first < end_ts; ++it)
      in_range.insert(in_range.end(), it->second.begin(), it->second.end());
    sampled = sample_ids(in_range, search_params_.itopk_size, seed_);
    if (sampled.empty()) { fill_no_data(host_indices, host_dists, num_queries * k); return; }
  }
  run_search(arena_of(arena_), a, host_queries, num_queries, dim_, k, sampled.empty() ? nullptr : sampled.data(),
             sampled.size(), true, nullptr, nullptr, host_indices, host_dists);
}

void CagraIndex::save(const std::string& filepath) {  // src/cagraIndex.cu:352-368: dim, degree, size, data, graph
  std::ofstream out(filepath, std::ios::binary);
  if (!out) throw grab::StatusError(GRAB_ERR_IO, "Cannot open file for save");
  get_graph();
  out.write(reinterpret_cast<const char*>(&dim_), sizeof(dim_));
  out.write(reinterpret_cast<const char*>(&graph_degree_), sizeof(graph_degree_));
  out.write(reinterpret_cast<const char*>(&current_size_), sizeof(current_size_));
  if (current_size_ > 0) {
    out.write(reinterpret_cast<const char*>(h_data_.data()), current_size_ * dim_ * sizeof(float));
    out.write(reinterpret_cast<const char*>(h_graph_.data()), current_size_ * graph_degree_ * sizeof(uint32_t));
  }
}

void CagraIndex::load(const std::string& filepath) {  // src/cagraIndex.cu:370-395
  std::ifstream in(filepath, std::ios::binary);
  if (!in) throw grab::StatusError(GRAB_ERR_IO, "Cannot open file for load");
  in.read(reinterpret_cast<char*>(&dim_), sizeof(dim_));
  in.read(reinterpret_cast<char*>(&graph_degree_), sizeof(graph_degree_));
  in.read(reinterpret_cast<char*>(&current_size_), sizeof(current_size_));
  if (!in) throw grab::StatusError(GRAB_ERR_IO, "load: truncated header");
  h_data_.resize(current_size_ * dim_);
  h_graph_.resize(current_size_ * graph_degree_);
  h_timestamps_.clear();
  ts_to_ids_.clear();
  if (current_size_ > 0) {
    in.read(reinterpret_cast<char*>(h_data_.data()), h_data_.size() * sizeof(float));
    in.read(reinterpret_cast<char*>(h_graph_.data()), h_graph_.size() * sizeof(uint32_t));
    if (!in) throw grab::StatusError(GRAB_ERR_IO, "load: truncated body");
    d_data_->resize(h_data_.size() * sizeof(float));
    d_graph_->resize(h_graph_.size() * sizeof(uint32_t));
    cu(cudaMemcpy(d_data_->data(), h_data_.data(), h_data_.size() * sizeof(float), cudaMemcpyHostToDevice), "H2D dataset");
    cu(cudaMemcpy(d_graph_->data(), h_graph_.data(), h_graph_.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "H2D graph");
  }
}

// =====================================================================================
// CagraIndexOpt (reference: src/cagraIndexOpt.cu)
// =====================================================================================
CagraIndexOpt::CagraIndexOpt(uint32_t dim, uint32_t graph_degree, uint32_t local_degree, size_t vmm_max_bytes)
    : dim_(dim), graph_degree_(graph_degree), local_degree_(local_degree) {
  if (dim == 0 || dim % 4 != 0) throw std::runtime_error("CagraIndexOpt: dim must be a positive multiple of 4");
  if (local_degree == 0 || local_degree > graph_degree) throw std::runtime_error("CagraIndexOpt: bad local_degree");
  d_data_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.70)));   // src/cagraIndexOpt.cu:23-29
  d_graph_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.20)));
  d_ts_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.05)));
  d_bucket_.reset(new grab::DeviceBuffer(static_cast<size_t>(vmm_max_bytes * 0.05)));
  build_params_ = {128, graph_degree};
  search_params_ = {256, 6, 1, 50, 13};  // src/cagraIndexOpt.cu:32-37
}
CagraIndexOpt::~CagraIndexOpt() = default;

void CagraIndexOpt::add(size_t num_vectors, const float* add_vectors, const uint64_t* add_timestamps) {
  if (num_vectors == 0) return;
  if (!add_timestamps) throw std::runtime_error("CagraIndexOpt::add: timestamps are mandatory");
  const size_t start = h_data_.size() / dim_, total = start + num_vectors;
  h_data_.resize(total * dim_);
  memcpy(h_data_.data() + start * dim_, add_vectors, num_vectors * dim_ * sizeof(float));
  h_timestamps_.resize(total);
  std::vector<uint64_t> buckets(num_vectors);
  for (size_t i = 0; i < num_vectors; ++i) {
    const uint64_t ts = add_timestamps[i];
    if (start + i > 0 && ts < h_timestamps_[start + i - 1]) ts_sorted_ = false;
    h_timestamps_[start + i] = ts;
    buckets[i] = bucket_of(ts);
    ts_to_ids_[buckets[i]].push_back(static_cast<uint32_t>(start + i));
  }
  d_ts_->resize(total * sizeof(uint64_t));
  d_bucket_->resize(total * sizeof(uint64_t));
  cu(cudaMemcpy(static_cast<uint64_t*>(d_ts_->data()) + start, add_timestamps, num_vectors * sizeof(uint64_t),
                cudaMemcpyHostToDevice), "H2D timestamps");
  cu(cudaMemcpy(static_cast<uint64_t*>(d_bucket_->data()) + start, buckets.data(), num_vectors * sizeof(uint64_t),
                cudaMemcpyHostToDevice), "H2D buckets");
}

std::vector<uint32_t> CagraIndexOpt::get_ids_by_timestamp(uint64_t ts) const {
  auto it = ts_to_ids_.find(bucket_of(ts));
  return it == ts_to_ids_.end() ? std::vector<uint32_t>{} : it->second;
}

std::vector<uint32_t> CagraIndexOpt::sample_seeds_by_time(uint64_t min_ts, uint64_t max_ts, size_t num) const {
  // src/cagraIndexOpt.cu:95-128: ids of buckets in [min, max], capped, then a uniform sample
  std::vector<uint32_t> cand;
  for (auto it = ts_to_ids_.lower_bound(bucket_of(min_ts)); it != ts_to_ids_.end() && it->first <= bucket_of(max_ts); ++it) {
    cand.insert(cand.end(), it->second.begin(), it->second.end());
    if (cand.size() > num * 100) break;
  }
  return sample_ids(cand, num, seed_);
}

struct CagraIndexOpt::RouterState {
  grab_router r{};
  std::unique_ptr<Scratch> cen, norms, offsets, members;
  size_t assigned = 0;  // vectors covered by the member lists
  size_t trained = 0;   // index size when the centroids were trained
};
void CagraIndexOpt::RouterDeleter::operator()(RouterState* s) const { delete s; }

const grab_router* CagraIndexOpt::ensure_router() {
  const size_t n = current_size_;
  if (router_centroids_ == 0 || n < 4096) return nullptr;
  if (router_ && router_->assigned == n) return &router_->r;
  uint32_t c = router_centroids_;
  if (c == kRouterAuto) {  // about sqrt(n), a power of two in [64, 4096]
    c = 64;
    while (c < 4096 && static_cast<size_t>(c) * c < n) c *= 2;
  }
  if (c > n / 8) c = static_cast<uint32_t>(n / 8);
  const bool retrain = !router_ || router_->r.num_centroids != c || n > 2 * router_->trained;
  if (retrain) {
    router_.reset(new RouterState());
    router_->cen.reset(new Scratch(static_cast<size_t>(c) * dim_ * sizeof(float)));
    router_->norms.reset(new Scratch(c * sizeof(float)));
    router_->offsets.reset(new Scratch((c + 1) * sizeof(uint32_t)));
    router_->trained = n;
  }
  router_->members.reset(new Scratch(n * sizeof(uint32_t)));
  ok(grab_router_build(static_cast<float*>(d_data_->data()), dim_, n, metric_, c, retrain ? 10 : 0, 0,
                       router_->cen->as<float>(), router_->norms->as<float>(), router_->offsets->as<uint32_t>(),
                       router_->members->as<uint32_t>(), nullptr),
     "router build");
  router_->r.num_centroids = c;
  router_->r.dim = dim_;
  router_->r.metric = metric_;
  router_->r.d_centroids = router_->cen->as<float>();
  router_->r.d_centroid_norms = router_->norms->as<float>();
  router_->r.d_member_offsets = router_->offsets->as<uint32_t>();
  router_->r.d_members = router_->members->as<uint32_t>();
  router_->r.flags = 0;
  router_->assigned = n;
  return &router_->r;
}

void CagraIndexOpt::build() {
  const size_t n = h_data_.size() / dim_;
  if (n == 0) return;
  router_.reset();  // centroids and member lists of the previous contents must not outlive them
  current_size_ = n;
  d_data_->resize(n * dim_ * sizeof(float));
  cu(cudaMemcpy(d_data_->data(), h_data_.data(), n * dim_ * sizeof(float), cudaMemcpyHostToDevice), "H2D dataset");
  d_graph_->resize(n * graph_degree_ * sizeof(uint32_t));
  // buckets = runs of equal consecutive bucket ids (src/cagraIndexOpt.cu:168-184)
  std::vector<uint64_t> sizes;
  uint64_t cur = bucket_of(h_timestamps_[0]);
  size_t count = 0;
  for (size_t i = 0; i < n; ++i) {
    const uint64_t b = bucket_of(h_timestamps_[i]);
    if (b == cur) { ++count; } else { sizes.push_back(count); cur = b; count = 1; }
  }
  sizes.push_back(count);
  ok(grab_build_time_partitioned_graph(static_cast<float*>(d_data_->data()), n, dim_, metric_,
                                       static_cast<uint32_t*>(d_graph_->data()), static_cast<uint64_t*>(d_bucket_->data()),
                                       sizes.data(), static_cast<uint32_t>(sizes.size()), graph_degree_,
                                       static_cast<uint32_t>(local_degree_), knn_precision_),
     "time-partitioned build");
  get_graph();
}

uint32_t* CagraIndexOpt::get_graph() {
  h_graph_.resize(current_size_ * graph_degree_);
  if (current_size_)
    cu(cudaMemcpy(h_graph_.data(), d_graph_->data(), h_graph_.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost), "D2H graph");
  return h_graph_.data();
}

void CagraIndexOpt::query(const float* host_queries, size_t num_queries, int k, uint64_t, uint64_t,
                          int64_t* host_indices, float* host_dists, const uint32_t* seeds, size_t num_seeds_per_query) {
  // the time bounds are ignored here, as in the reference (src/cagraIndexOpt.cu:226-227)
  if (current_size_ == 0 || num_queries == 0) return;
  grab_search_args a = make_args(static_cast<float*>(d_data_->data()), current_size_, dim_, metric_,
                                 static_cast<uint32_t*>(d_graph_->data()), graph_degree_, nullptr, num_queries, k,
                                 search_params_, nullptr, nullptr, seed_);
  a.ctas_per_query = ctas_per_query_;
  a.filter.kind = GRAB_FILTER_NONE;
  run_search(arena_of(arena_), a, host_queries, num_queries, dim_, k, seeds, num_seeds_per_query, false, nullptr,
             nullptr, host_indices, host_dists, ensure_router(), router_probes_, router_seeds_);
}

void CagraIndexOpt::query_local(const float* host_queries, size_t num_queries, int k, uint64_t target_timestamp,
                                int64_t* host_indices, float* host_dists, uint32_t) {
  // the local_degree argument is overwritten by the member, as in the reference (src/cagraIndexOpt.cu:310)
  if (current_size_ == 0 || num_queries == 0) return;
  auto it = ts_to_ids_.find(bucket_of(target_timestamp));
  std::vector<uint32_t> in_bucket;
  if (it != ts_to_ids_.end())
    for (uint32_t id : it->second)
      if (id < current_size_) in_bucket.push_back(id);
  if (in_bucket.empty()) { fill_no_data(host_indices, host_dists, num_queries * k); return; }
  const std::vector<uint32_t> seeds = sample_ids(in_bucket, std::max(32u, search_params_.itopk_size), seed_);
  grab_search_args a = make_args(static_cast<float*>(d_data_->data()), current_size_, dim_, metric_,
                                 static_cast<uint32_t*>(d_graph_->data()), graph_degree_, nullptr, num_queries, k,
                                 search_params_, nullptr, nullptr, seed_);
  a.ctas_per_query = ctas_per_query_;
  a.filter.kind = GRAB_FILTER_PREFIX;
  a.filter.active_degree = static_cast<uint32_t>(local_degree_);
  run_search(arena_of(arena_), a, host_queries, num_queries, dim_, k, seeds.data(), seeds.size(), true, nullptr,
             nullptr, host_indices, host_dists);
}

void CagraIndexOpt::range_search(const float* host_queries, size_t nq, int k, const uint64_t* lo, const uint64_t* hi,
                                 uint64_t lo1, uint64_t hi1, int64_t* ids, float* dists, bool exact) {
  grab_search_args a = make_args(static_cast<float*>(d_data_->data()), current_size_, dim_, metric_,
                                 static_cast<uint32_t*>(d_graph_->data()), graph_degree_, nullptr, nq, k, search_params_,
                                 nullptr, nullptr, seed_);
  a.ctas_per_query = ctas_per_query_;
  a.filter.kind = GRAB_FILTER_TS_RANGE;
  a.filter.d_ts = static_cast<uint64_t*>(d_ts_->data());
  a.filter.ts_sorted = ts_sorted_;
  if (!lo) {
    a.filter.lo = lo1;
    a.filter.hi = hi1;
    if (exact) {
      run_search(arena_of(arena_), a, host_queries, nq, dim_, k, nullptr, 0, false, nullptr, nullptr, ids, dists, nullptr,
                 0, 0, true);
      return;
    }
  }
  std::vector<uint32_t> seeds;
  size_t spq = 0;
  bool broadcast = true;
  const grab_router* router = ensure_router();
  if (!ts_sorted_ && !router) {
    // host seed sampling as the reference does it: up to 500 ids per bucket, then a uniform
    // sample of max(32, itopk/4) (src/cagraIndexOpt.cu:441-474); per query when ranges differ
    spq = std::max(32u, search_params_.itopk_size / 4);
    auto sample_range = [&](uint64_t s, uint64_t e, uint64_t salt) {
      std::vector<uint32_t> cand;
      for (auto it = ts_to_ids_.lower_bound(bucket_of(s)); it != ts_to_ids_.end() && it->first <= bucket_of(e ? e - 1 : 0); ++it) {
        size_t taken = 0;
        for (uint32_t id : it->second) {
          if (id >= current_size_ || h_timestamps_[id] < s || h_timestamps_[id] >= e) continue;
          cand.push_back(id);
          if (++taken >= 500) break;
        }
      }
      std::vector<uint32_t> out = sample_ids(cand, spq, seed_ + salt);
      out.resize(spq, 0xFFFFFFFFu);
      return out;
    };
    if (lo) {
      broadcast = false;
      seeds.reserve(nq * spq);
      for (size_t i = 0; i < nq; ++i) {
        auto s = sample_range(lo[i], hi[i], i);
        seeds.insert(seeds.end(), s.begin(), s.end());
      }
    } else {
      seeds = sample_range(lo1, hi1, 0);
    }
  }
  run_search(arena_of(arena_), a, host_queries, nq, dim_, k, seeds.empty() ? nullptr : seeds.data(), spq, broadcast,
             lo, hi, ids, dists, router, router_probes_, router_seeds_);
}

void CagraIndexOpt::query_range(const float* host_queries, size_t num_queries, int k, uint64_t start_bucket,
                                uint64_t end_bucket, int64_t* host_indices, float* host_dists, uint32_t) {
  if (current_size_ == 0 || num_queries == 0) return;
  // "no data in the range" early-out (src/cagraIndexOpt.cu:479-485); the same pass counts the vectors inside the
  // range up to the exact-scan threshold
  size_t inside = 0;
  for (auto it = ts_to_ids_.lower_bound(bucket_of(start_bucket)); it != ts_to_ids_.end() && inside <= exact_below_; ++it) {
    if (end_bucket == 0 || it->first > bucket_of(end_bucket - 1)) break;
    for (uint32_t id : it->second)
      if (id < current_size_ && h_timestamps_[id] >= start_bucket && h_timestamps_[id] < end_bucket && ++inside > exact_below_)
        break;
  }
  if (inside == 0) { fill_no_data(host_indices, host_dists, num_queries * k); return; }
  range_search(host_queries, num_queries, k, nullptr, nullptr, start_bucket, end_bucket, host_indices, host_dists,
               inside <= exact_below_);
}

void CagraIndexOpt::query_range_batch(const float* host_queries, size_t num_queries, int k, const uint64_t* start_ts,
                                      const uint64_t* end_ts, int64_t* host_indices, float* host_dists) {
  if (current_size_ == 0 || num_queries == 0) return;
  range_search(host_queries, num_queries, k, start_ts, end_ts, 0, 0, host_indices, host_dists);
}

void CagraIndexOpt::insert(size_t new_vectors, const float* insert_vectors, const uint64_t* insert_timestamps) {
  if (new_vectors == 0) return;
  if (!insert_timestamps) throw std::runtime_error("CagraIndexOpt::insert: timestamps are mandatory");
  if (current_size_ == 0) {
    add(new_vectors, insert_vectors, insert_timestamps);
    build();
    return;
  }
  const size_t first_new = current_size_, new_total = first_new + new_vectors;
  // The router (when it is on and the timestamps are sorted) covers the nodes present before this call; both
  // insert searches then start from routed seeds -- members of the new vector's nearest centroids, for the bucket
  // search those inside the target bucket -- instead of random ids / a host-sampled list shared by the whole batch,
  // and need a fraction of the iterations.
  const grab_router* router = (insert_routed_ && ts_sorted_) ? ensure_router() : nullptr;
  add(new_vectors, insert_vectors, insert_timestamps);
  if (!ts_sorted_) router = nullptr;
  try {
    d_data_->resize(new_total * dim_ * sizeof(float));
    d_graph_->resize(new_total * graph_degree_ * sizeof(uint32_t));
    float* d_data = static_cast<float*>(d_data_->data());
    uint32_t* d_graph = static_cast<uint32_t*>(d_graph_->data());
    cu(cudaMemcpy(d_data + first_new * dim_, insert_vectors, new_vectors * dim_ * sizeof(float), cudaMemcpyHostToDevice),
       "H2D new vectors");
    // search parameters of the insert path (src/cagraIndexOpt.cu:596-602: itopk 128, width 4, up to 100 iterations,
    // hash 2^13; kept apart from the user's query parameters, which the reference overwrites here).  Routed seeds
    // start next to the answer: a dozen iterations settle the 128 nearest.
    const grab_search_params ip = router ? insert_params_routed_ : insert_params_;
    const uint32_t spq = std::max(32u, ip.itopk_size);
    grab::InsertOptions io;
    io.router = router;
    io.probes = router_probes_;
    io.routed_seeds = 64;
    io.repair_mode = insert_repair_mode_;
    io.sync = false;  // batches are stream-ordered; one wait at the end of the call
    size_t old_size = first_new;
    size_t off = 0;
    while (off < new_vectors) {
      // the reference assumes one bucket per call (src/cagraIndexOpt.cu:560); runs of equal
      // bucket ids are inserted one after the other here
      const uint64_t target = bucket_of(insert_timestamps[off]);
      size_t run = 1;
      while (off + run < new_vectors && bucket_of(insert_timestamps[off + run]) == target) ++run;
      for (size_t b = 0; b < run; b += insert_batch_) {
        const size_t cur = std::min(insert_batch_, run - b);
        auto it = ts_to_ids_.find(target);
        const bool has_old = it != ts_to_ids_.end() && !it->second.empty() && it->second.front() < old_size;
        std::unique_ptr<Scratch> d_seeds;
        if (!router && has_old) {
          // host seed sampling as in the reference (src/cagraIndexOpt.cu:604-640): one list for the batch
          std::vector<uint32_t> in_bucket;
          for (uint32_t id : it->second) {
            if (id >= old_size) break;  // ids are appended in ascending order
            in_bucket.push_back(id);
          }
          std::vector<uint32_t> one = sample_ids(in_bucket, spq, seed_ + old_size);
          one.resize(spq, 0xFFFFFFFFu);
          std::vector<uint32_t> all(cur * spq);
          for (size_t i = 0; i < cur; ++i) memcpy(all.data() + i * spq, one.data(), spq * 4);
          d_seeds.reset(new Scratch(all.size() * 4));
          cu(cudaMemcpy(d_seeds->p, all.data(), all.size() * 4, cudaMemcpyHostToDevice), "H2D seeds");
        }
        io.bucket_has_old_members = has_old;
        if (has_old) {  // sorted timestamps: the bucket's old members are the id run [front, old_size) or [front, next bucket)
          io.bucket_begin = it->second.front();
          auto last_old = std::lower_bound(it->second.begin(), it->second.end(), static_cast<uint32_t>(old_size));
          io.bucket_end = static_cast<uint64_t>(*(last_old - 1)) + 1;
        }
        io.router_covers = first_new;  // ensure_router() ran at the start of this call
        ok(grab::insert_opt_impl(d_data, d_graph, static_cast<uint64_t*>(d_bucket_->data()),
                                 d_seeds ? d_seeds->as<uint32_t>() : nullptr, old_size, cur, target,
                                 d_data + old_size * dim_, dim_, graph_degree_, static_cast<uint32_t>(local_degree_), ip,
                                 d_seeds ? spq : 0, metric_, &io),
           "insert");
        if (d_seeds) cu(cudaDeviceSynchronize(), "insert batch");  // the seed list is freed on scope exit
        old_size += cur;
      }
      off += run;
    }
    cu(cudaDeviceSynchronize(), "insert");
  } catch (...) {
    // leave the index as it was before the call: the host mirrors must not run ahead of current_size_
    h_data_.resize(first_new * dim_);
    h_timestamps_.resize(first_new);
    for (auto it = ts_to_ids_.begin(); it != ts_to_ids_.end();) {
      while (!it->second.empty() && it->second.back() >= first_new) it->second.pop_back();
      it = it->second.empty() ? ts_to_ids_.erase(it) : std::next(it);
    }
    cudaDeviceSynchronize();
    throw;
  }
  current_size_ = new_total;
}

void CagraIndexOpt::save(const std::string& filepath) {  // "MCAG" v1, src/cagraIndexOpt.cu:725-794
  std::ofstream ofs(filepath, std::ios::binary);
  if (!ofs.is_open()) throw grab::StatusError(GRAB_ERR_IO, "Failed to open file for writing: " + filepath);
  get_graph();
  auto put = [&](const void* p, size_t b) { ofs.write(reinterpret_cast<const char*>(p), b); };
  const char magic[4] = {'M', 'C', 'A', 'G'};
  const uint32_t version = 1;
  put(magic, 4); put(&version, 4); put(&dim_, 4); put(&graph_degree_, 4);
  put(&local_degree_, sizeof(size_t)); put(&current_size_, sizeof(size_t));
  const size_t ts_size = h_timestamps_.size();
  put(&ts_size, sizeof(size_t)); put(h_timestamps_.data(), ts_size * sizeof(uint64_t));
  const size_t nb = ts_to_ids_.size();
  put(&nb, sizeof(size_t));
  for (const auto& e : ts_to_ids_) {
    const size_t cnt = e.second.size();
    put(&e.first, sizeof(uint64_t)); put(&cnt, sizeof(size_t)); put(e.second.data(), cnt * sizeof(uint32_t));
  }
  const size_t dsz = h_data_.size(), gsz = h_graph_.size();
  put(&dsz, sizeof(size_t)); put(h_data_.data(), dsz * sizeof(float));
  put(&gsz, sizeof(size_t)); put(h_graph_.data(), gsz * sizeof(uint32_t));
}

void CagraIndexOpt::load(const std::string& filepath) {  // src/cagraIndexOpt.cu:796-898
  std::ifstream ifs(filepath, std::ios::binary);
  if (!ifs.is_open()) throw grab::StatusError(GRAB_ERR_IO, "Failed to open file for reading: " + filepath);
  router_.reset();  // a file of the same size would otherwise keep the old index's centroids and member lists
  auto get = [&](void* p, size_t b) {
    ifs.read(reinterpret_cast<char*>(p), b);
    if (!ifs) throw grab::StatusError(GRAB_ERR_IO, "load: truncated file " + filepath);
  };
  char magic[4];
  uint32_t version = 0;
  get(magic, 4);
  if (memcmp(magic, "MCAG", 4) != 0) throw grab::StatusError(GRAB_ERR_IO, "load: bad magic in " + filepath);
  get(&version, 4);
  if (version != 1) throw grab::StatusError(GRAB_ERR_IO, "load: unsupported version");
  get(&dim_, 4); get(&graph_degree_, 4); get(&local_degree_, sizeof(size_t)); get(&current_size_, sizeof(size_t));
  size_t ts_size = 0, nb = 0, dsz = 0, gsz = 0;
  get(&ts_size, sizeof(size_t));
  h_timestamps_.resize(ts_size);
  get(h_timestamps_.data(), ts_size * sizeof(uint64_t));
  get(&nb, sizeof(size_t));
  ts_to_ids_.clear();
  for (size_t i = 0; i < nb; ++i) {
    uint64_t key; size_t cnt;
    get(&key, sizeof(uint64_t)); get(&cnt, sizeof(size_t));
    std::vector<uint32_t> ids(cnt);
    get(ids.data(), cnt * sizeof(uint32_t));
    ts_to_ids_[key] = std::move(ids);
  }
  get(&dsz, sizeof(size_t)); h_data_.resize(dsz); get(h_data_.data(), dsz * sizeof(float));
  get(&gsz, sizeof(size_t)); h_graph_.resize(gsz); get(h_graph_.data(), gsz * sizeof(uint32_t));
  ts_sorted_ = std::is_sorted(h_timestamps_.begin(), h_timestamps_.end());
  std::vector<uint64_t> buckets(ts_size);
  for (size_t i = 0; i < ts_size; ++i) buckets[i] = bucket_of(h_timestamps_[i]);
  d_data_->resize(dsz * sizeof(float));
  d_graph_->resize(gsz * sizeof(uint32_t));
  d_ts_->resize(ts_size * sizeof(uint64_t));
  d_bucket_->resize(ts_size * sizeof(uint64_t));
  if (dsz) cu(cudaMemcpy(d_data_->data(), h_data_.data(), dsz * sizeof(float), cudaMemcpyHostToDevice), "H2D dataset");
  if (gsz) cu(cudaMemcpy(d_graph_->data(), h_graph_.data(), gsz * sizeof(uint32_t), cudaMemcpyHostToDevice), "H2D graph");
  if (ts_size) {
    cu(cudaMemcpy(d_ts_->data(), h_timestamps_.data(), ts_size * sizeof(uint64_t), cudaMemcpyHostToDevice), "H2D ts");
    cu(cudaMemcpy(d_bucket_->data(), buckets.data(), ts_size * sizeof(uint64_t), cudaMemcpyHostToDevice), "H2D buckets");
  }
}

}  // namespace cagra

// =====================================================================================
// TimeStampIndex (reference: src/timeStampIndex.cu)
// =====================================================================================
namespace timestamp {

TimeStampIndex::TimeStampIndex(uint32_t dim, uint32_t degree, size_t cluster_ratio)
    : dim_(dim), graph_degree_(degree), cluster_ratio_(cluster_ratio) {}
TimeStampIndex::~TimeStampIndex() = default;

size_t TimeStampIndex::size() const {
  std::shared_lock<std::shared_mutex> lock(mutex_);
  return global_count_;
}

std::pair<cagra::CagraIndex*, BucketContext*> TimeStampIndex::get_or_create_bucket(uint64_t ts) {
  auto it = buckets_.find(ts);
  if (it == buckets_.end()) {
    // every bucket reserves its own address range: keep it modest (2 GiB)
    it = buckets_.emplace(ts, std::make_unique<cagra::CagraIndex>(dim_, graph_degree_, size_t(2) << 30)).first;
    bucket_contexts_[ts] = BucketContext{};
  }
  return {it->second.get(), &bucket_contexts_[ts]};
}

uint64_t TimeStampIndex::insert(const float* vectors, const uint64_t* timestamps, size_t num_vectors) {
  std::unique_lock<std::shared_mutex> lock(mutex_);  // src/timeStampIndex.cu:65-139
  const uint64_t start = global_count_;
  global_count_ += num_vectors;
  id_to_location_.resize(global_count_);
  std::map<uint64_t, std::pair<std::vector<float>, std::vector<uint64_t>>> groups;
  for (size_t i = 0; i < num_vectors; ++i) {
    auto& g = groups[timestamps[i]];
    g.first.insert(g.first.end(), vectors + i * dim_, vectors + (i + 1) * dim_);
    g.second.push_back(start + i);
  }
  for (auto& kv : groups) {
    auto bc = get_or_create_bucket(kv.first);
    const size_t local0 = bc.first->size();
    bc.first->insert(kv.second.second.size(), kv.second.first.data());
    for (size_t j = 0; j < kv.second.second.size(); ++j) {
      id_to_location_[kv.second.second[j]] = VectorLocation{kv.first, local0 + j};
      bc.second->local_to_global.push_back(kv.second.second[j]);
    }
    bc.second->num_dirty += kv.second.second.size();
  }
  return start;
}

// Lloyd's k-means over all n points on the device (the router's deterministic trainer: tiled
// nearest-centroid kernel, grouped member lists, ordered means); the reference calls
// faiss::Clustering here (src/timeStampIndex.cu:169-179).
static std::vector<float> kmeans(const float* h_data, size_t n, uint32_t dim, size_t kc, int iters) {
  Scratch dd(n * dim * sizeof(float)), dc(kc * dim * sizeof(float)), dn(kc * sizeof(float)),
      doff((kc + 1) * sizeof(uint32_t)), dmem(n * sizeof(uint32_t));
  cu(cudaMemcpy(dd.p, h_data, n * dim * sizeof(float), cudaMemcpyHostToDevice), "H2D kmeans data");
  ok(grab_router_build(dd.as<float>(), dim, n, GRAB_METRIC_L2, static_cast<uint32_t>(kc), static_cast<uint32_t>(iters), n,
                       dc.as<float>(), dn.as<float>(), doff.as<uint32_t>(), dmem.as<uint32_t>(), nullptr),
     "k-means");
  std::vector<float> cen(kc * dim);
  cu(cudaMemcpy(cen.data(), dc.p, cen.size() * sizeof(float), cudaMemcpyDeviceToHost), "D2H centroids");
  return cen;
}

void TimeStampIndex::build_virtual_index() {
  std::unique_lock<std::shared_mutex> lock(mutex_);  // src/timeStampIndex.cu:141-238
  if (buckets_.empty()) return;
  std::vector<float> all;
  std::vector<VirtualPointMeta> meta;
  for (auto& kv : buckets_) {
    cagra::CagraIndex* bucket = kv.second.get();
    const size_t n = bucket->size();
    if (n == 0) continue;
    size_t kc = 16 * std::max<size_t>(1, static_cast<size_t>(std::sqrt(static_cast<double>(n))));
    kc = std::min(kc, std::max<size_t>(1, n / 2));
    const std::vector<float> cen = kmeans(static_cast<const float*>(bucket->get_data()), n, dim_, kc, 30);
    const int entries = static_cast<int>(std::min<size_t>(5, n));
    std::vector<int64_t> ei(kc * entries);
    std::vector<float> ed(kc * entries);
    bucket->query(cen.data(), kc, entries, ei.data(), ed.data());
    for (size_t c = 0; c < kc; ++c) {
      all.insert(all.end(), cen.begin() + c * dim_, cen.begin() + (c + 1) * dim_);
      VirtualPointMeta m;
      m.target_timestamp = kv.first;
      for (int e = 0; e < entries; ++e)
        if (ei[c * entries + e] >= 0) m.entry_points.push_back(static_cast<uint32_t>(ei[c * entries + e]));
      meta.push_back(std::move(m));
    }
  }
  if (all.empty()) { virtual_index_.reset(); virtual_meta_.clear(); return; }
  virtual_index_ = std::make_unique<cagra::CagraIndex>(dim_, graph_degree_, size_t(2) << 30);
  virtual_index_->add(all.size() / dim_, all.data());
  virtual_index_->build();
  virtual_meta_ = std::move(meta);
}

void TimeStampIndex::query(const float* query, size_t topk, int64_t* out_indices, float* out_dists, int probe_buckets) {
  std::shared_lock<std::shared_mutex> lock(mutex_);  // src/timeStampIndex.cu:240-419
  if (!virtual_index_ || buckets_.empty()) {
    for (size_t i = 0; i < topk; ++i) { out_indices[i] = -1; out_dists[i] = -1.0f; }
    return;
  }
  const int vk = static_cast<int>(std::min<size_t>(static_cast<size_t>(probe_buckets) * 10, virtual_meta_.size()));
  std::vector<int64_t> vi(vk);
  std::vector<float> vd(vk);
  virtual_index_->query(query, 1, vk, vi.data(), vd.data());
  std::map<uint64_t, std::pair<int, std::vector<uint32_t>>> votes;
  for (int i = 0; i < vk; ++i) {
    if (vi[i] < 0 || static_cast<size_t>(vi[i]) >= virtual_meta_.size()) continue;
    const VirtualPointMeta& m = virtual_meta_[vi[i]];
    auto& v = votes[m.target_timestamp];
    ++v.first;
    v.second.insert(v.second.end(), m.entry_points.begin(), m.entry_points.end());
  }
  std::vector<std::pair<int, uint64_t>> ranked;
  for (auto& kv : votes) ranked.push_back({-kv.second.first, kv.first});
  std::stable_sort(ranked.begin(), ranked.end());
  std::vector<std::pair<float, int64_t>> all;
  const size_t probes = std::min<size_t>(probe_buckets, ranked.size());
  // the probed buckets are independent indexes with query scratch and streams of their own: search them side by
  // side, as the reference does (src/timeStampIndex.cu:318-372, an OpenMP loop over the buckets)
  std::vector<std::vector<std::pair<float, int64_t>>> found(probes);
  std::exception_ptr failure;
  int device = 0;
  cu(cudaGetDevice(&device), "cudaGetDevice");  // worker threads start on device 0: hand them the caller's device
#pragma omp parallel for schedule(dynamic) num_threads(8)
  for (long r = 0; r < static_cast<long>(probes); ++r) {
    try {
      cu(cudaSetDevice(device), "cudaSetDevice");
      const uint64_t ts = ranked[r].second;
      cagra::CagraIndex* bucket = buckets_.at(ts).get();
      const BucketContext& ctx = bucket_contexts_.at(ts);
      std::vector<uint32_t>& seeds = votes.at(ts).second;
      std::vector<int64_t> bi(topk);
      std::vector<float> bd(topk);
      bucket->query(query, 1, static_cast<int>(topk), bi.data(), bd.data(), seeds.data(), seeds.size());
      for (size_t k = 0; k < topk; ++k)
        if (bi[k] >= 0 && static_cast<size_t>(bi[k]) < ctx.local_to_global.size())
          found[r].push_back({bd[k], static_cast<int64_t>(ctx.local_to_global[bi[k]])});
    } catch (...) {
#pragma omp critical
      if (!failure) failure = std::current_exception();
    }
  }
  if (failure) std::rethrow_exception(failure);
  for (const auto& f : found) all.insert(all.end(), f.begin(), f.end());
  std::sort(all.begin(), all.end());
  for (size_t k = 0; k < topk; ++k) {
    out_indices[k] = k < all.size() ? all[k].second : -1;
    out_dists[k] = k < all.size() ? all[k].first : -1.0f;
  }
}

void TimeStampIndex::query_by_timestamp(const float* query, size_t topk, uint64_t timestamp, int64_t* out_indices,
                                        float* out_dists) {
  std::shared_lock<std::shared_mutex> lock(mutex_);
  auto it = buckets_.find(timestamp);
  if (it == buckets_.end() || it->second->size() == 0) {
    for (size_t i = 0; i < topk; ++i) { out_indices[i] = -1; out_dists[i] = -1.0f; }
    return;
  }
  const BucketContext& ctx = bucket_contexts_.at(timestamp);
  std::vector<int64_t> bi(topk);
  std::vector<float> bd(topk);
  it->second->query(query, 1, static_cast<int>(topk), bi.data(), bd.data());
  for (size_t k = 0; k < topk; ++k) {
    const bool valid = bi[k] >= 0 && static_cast<size_t>(bi[k]) < ctx.local_to_global.size();
    out_indices[k] = valid ? static_cast<int64_t>(ctx.local_to_global[bi[k]]) : -1;
    out_dists[k] = valid ? bd[k] : -1.0f;
  }
}

}  // namespace timestamp
