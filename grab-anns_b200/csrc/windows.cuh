// Per-row scan windows shared by the exact scan and the tensor-core kNN kernel.
#pragma once
#include <cstdint>

namespace grab {

// Row r scans ids [begin,end) except [xbegin,xend).
struct ScanWindow {
  uint32_t begin, end, xbegin, xend;
};

// kNN windows: row r (global id) scans its own block minus itself (mode 0) or everything
// except its own block (mode 1).  block_offsets: [num_blocks+1], ascending, on the device.
static __global__ void knn_window_kernel(const uint64_t* __restrict__ block_offsets, uint32_t num_blocks,
                                         uint64_t n, int mode, ScanWindow* __restrict__ windows) {
  const uint64_t r = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (r >= n) return;
  uint32_t l = 0, h = num_blocks;  // block b with offsets[b] <= r < offsets[b+1]
  while (h - l > 1) {
    const uint32_t m = (l + h) >> 1;
    if (block_offsets[m] <= r) l = m; else h = m;
  }
  ScanWindow w;
  if (mode == 0) {
    w.begin = static_cast<uint32_t>(block_offsets[l]);
    w.end = static_cast<uint32_t>(block_offsets[l + 1]);
    w.xbegin = static_cast<uint32_t>(r);
    w.xend = static_cast<uint32_t>(r + 1);
  } else {
    w.begin = 0;
    w.end = static_cast<uint32_t>(n);
    w.xbegin = static_cast<uint32_t>(block_offsets[l]);
    w.xend = static_cast<uint32_t>(block_offsets[l + 1]);
  }
  windows[r] = w;
}

}  // namespace grab
