// grab_exact_search_noalloc: the exact filtered scan for callers that must not allocate.
//
// Who cannot allocate, and why: a serving loop in which cudaMalloc / cudaFree would stall
// every stream of the process (both synchronise the device); a host application whose memory
// pool has already claimed the whole GPU, so a further cudaMalloc fails; code that runs under
// a "no allocation after start-up" rule.  For them the scratch of the scan (per-query id
// windows and the per-split partial top-k lists) lives in a fixed array inside the library
// image instead of a caller workspace or a temporary allocation.
//
// Cost and limits: every GPU that loads the library carries the GRAB_NOALLOC_SCRATCH_BYTES
// array until the process exits.  A request whose scratch need
// (grab_exact_search_workspace_bytes) is larger is refused with GRAB_ERR_WORKSPACE.  All calls
// on a device share the one array: two calls that overlap on the GPU (different streams,
// different host threads) race on it -- serialise them.  Nothing in the array has to be
// cleared between calls: every word a call reads it has written earlier in the same call
// (windows by the window kernel, partial lists by the scan), so the previous call's leftovers
// are never observed.
//
// The first call on each device looks up the device address of the array (one
// cudaGetSymbolAddress).  With CUDA's default lazy module loading that lookup is also the moment
// the driver places this library's image -- and with it the array -- in the device's memory, so
// it is the one point at which device memory is taken: make that first call (any small request
// will do) before the host's memory pool claims the rest of the GPU, and before starting any
// stream capture.  Later calls take nothing.  No counterpart in the reference.
#include <mutex>

#include "common.cuh"

namespace grab {

int exact_search_impl(const float*, uint64_t, uint32_t, int, const grab_filter*, const float*, uint64_t, uint32_t,
                      int64_t*, float*, void*, size_t, cudaStream_t);

// In host code this name is only a handle for cudaGetSymbolAddress; the kernels get the
// device address that call returns.
static __device__ __align__(256) unsigned char g_noalloc_scratch[GRAB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_scratch_mutex;

static int scratch_for_current_device(void** out) {
  int dev = 0;
  GRAB_CUDA_TRY(cudaGetDevice(&dev));
  GRAB_REQUIRE(dev >= 0 && dev < kMaxDevices, "exact_search_noalloc: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    GRAB_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));  // with `dev` current: its copy of the array
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return GRAB_OK;
}

}  // namespace grab

extern "C" int grab_exact_search_noalloc(const float* d_dataset, uint64_t n, uint32_t dim, int metric,
                                         const grab_filter* filter, const float* d_queries, uint64_t nq,
                                         uint32_t k, int64_t* d_out_ids, float* d_out_dists, void* stream) {
  using namespace grab;
  const size_t need = grab_exact_search_workspace_bytes(n, nq, k);
  if (need > GRAB_NOALLOC_SCRATCH_BYTES) {
    set_last_error("exact_search_noalloc: this request needs %zu bytes of scratch, the built-in scratch holds %zu; "
                   "use fewer queries per call, or grab_exact_search with a caller workspace",
                   need, static_cast<size_t>(GRAB_NOALLOC_SCRATCH_BYTES));
    return GRAB_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != GRAB_OK) return rc;
  return exact_search_impl(d_dataset, n, dim, metric, filter, d_queries, nq, k, d_out_ids, d_out_dists, scratch,
                           GRAB_NOALLOC_SCRATCH_BYTES, static_cast<cudaStream_t>(stream));
}
