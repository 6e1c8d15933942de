// Test infrastructure: see ../core/device_resources.hpp.
#pragma once
#include "../core/device_mdspan.hpp"

namespace raft {
namespace neighbors {
namespace brute_force {
struct index_stub {};
template <class Res, class View>
index_stub build(const Res&, View) {
  grab_shim::unavailable("raft::neighbors::brute_force::build");
}
template <class... Args>
void search(Args&&...) {
  grab_shim::unavailable("raft::neighbors::brute_force::search");
}
}  // namespace brute_force
}  // namespace neighbors
}  // namespace raft
