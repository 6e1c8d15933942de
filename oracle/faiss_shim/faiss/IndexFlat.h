// Test infrastructure, not part of the product: FAISS is not installed here, and the reference's test programs
// use faiss::IndexFlatL2 only as their CPU ground truth (add, then search).  This header gives them that class
// with the same two calls, as a plain OpenMP brute force written for this repository; nothing of FAISS is in it.
// add() keeps a pointer to the caller's array instead of copying it (the programs search while the array is
// alive, and a copy of a 20 GB dataset would not fit beside it).
#pragma once
#include <algorithm>
#include <cstdint>
#include <utility>
#include <vector>

namespace faiss {

using idx_t = int64_t;

struct IndexFlatL2 {
  int d;
  idx_t ntotal = 0;
  std::vector<std::pair<const float*, idx_t>> blocks;  // (first row, rows)

  explicit IndexFlatL2(idx_t dim) : d(static_cast<int>(dim)) {}

  void add(idx_t n, const float* x) {
    blocks.emplace_back(x, n);
    ntotal += n;
  }

  // squared L2 distances, ascending; ids are positions in add() order; missing results are -1
  void search(idx_t nq, const float* q, idx_t k, float* distances, idx_t* labels) const {
#pragma omp parallel for schedule(dynamic, 1)
    for (idx_t i = 0; i < nq; ++i) {
      std::vector<std::pair<float, idx_t>> heap;  // max-heap of the k best
      heap.reserve(static_cast<size_t>(k) + 1);
      const float* qv = q + i * d;
      idx_t base = 0;
      for (const auto& b : blocks) {
        for (idx_t j = 0; j < b.second; ++j) {
          const float* v = b.first + j * static_cast<idx_t>(d);
          float s = 0.f;
          for (int c = 0; c < d; ++c) {
            const float t = qv[c] - v[c];
            s += t * t;
          }
          if (static_cast<idx_t>(heap.size()) < k) {
            heap.emplace_back(s, base + j);
            std::push_heap(heap.begin(), heap.end());
          } else if (s < heap.front().first) {
            std::pop_heap(heap.begin(), heap.end());
            heap.back() = {s, base + j};
            std::push_heap(heap.begin(), heap.end());
          }
        }
        base += b.second;
      }
      std::sort_heap(heap.begin(), heap.end());
      for (idx_t r = 0; r < k; ++r) {
        const bool have = r < static_cast<idx_t>(heap.size());
        distances[i * k + r] = have ? heap[r].first : 3.402823466e38f;
        labels[i * k + r] = have ? heap[r].second : -1;
      }
    }
  }
};

}  // namespace faiss
