// Test infrastructure: see device_resources.hpp in this directory.
#pragma once
#include "device_resources.hpp"

namespace raft {
template <class T, class I>
struct device_matrix_view {
  T* ptr;
  I rows, cols;
  T* data_handle() const { return ptr; }
  I extent(int d) const { return d == 0 ? rows : cols; }
};
template <class T, class I, class P, class R, class C>
device_matrix_view<T, I> make_device_matrix_view(P* ptr, R rows, C cols) {
  return device_matrix_view<T, I>{ptr, static_cast<I>(rows), static_cast<I>(cols)};
}
}  // namespace raft
