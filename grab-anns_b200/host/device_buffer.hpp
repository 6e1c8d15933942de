// Growable device buffer with a stable base pointer.
//
// Same contract as the reference's DeviceBufferVMM (src/vmm_allocator.cuh:23-118): reserve a
// virtual range once, map more physical memory on resize, so device pointers handed to
// kernels stay valid while an index grows by inserts.  Differences: the device is a run-time
// argument (the reference compiles it in, vmm_allocator.cuh:31), the driver entry points are
// resolved at run time (no link-time dependency on libcuda), and when the driver offers no
// virtual memory management the buffer falls back to grow-and-copy.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <stdexcept>
#include <string>
#include <vector>

namespace grab {

class DeviceBuffer {
 public:
  explicit DeviceBuffer(size_t max_bytes, int device = -1);
  ~DeviceBuffer();
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;

  // Makes at least new_bytes usable; contents below the old size are kept.  Throws
  // std::runtime_error beyond max_bytes (the reference throws too, vmm_allocator.cuh:72-74).
  void resize(size_t new_bytes);
  void* data() const { return reinterpret_cast<void*>(base_); }
  size_t size() const { return size_; }
  size_t capacity() const { return max_bytes_; }
  bool uses_vmm() const { return vmm_; }
  void free();

 private:
  size_t max_bytes_ = 0, size_ = 0, mapped_ = 0, granularity_ = 0;
  int device_ = 0;
  bool vmm_ = false;
  CUdeviceptr base_ = 0;
  std::vector<std::pair<CUmemGenericAllocationHandle, size_t>> chunks_;
};

// Exception that carries the grab_status the C handles return for it (plain std::runtime_error maps to
// GRAB_ERR_INVALID_ARGUMENT there).
struct StatusError : std::runtime_error {
  int status;
  StatusError(int status_, const std::string& message) : std::runtime_error(message), status(status_) {}
};

// Query scratch an index keeps across calls (defined with the classes, index_classes.cu).
struct QueryArena;
struct QueryArenaDeleter { void operator()(QueryArena*) const; };

}  // namespace grab
