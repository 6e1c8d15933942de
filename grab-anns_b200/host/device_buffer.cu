#include "device_buffer.hpp"

namespace grab {
namespace {

struct Driver {
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addr_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  bool ok = false;
};

template <class F>
bool resolve(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      !p)
    return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

const Driver& driver() {
  static Driver d = [] {
    Driver x;
    x.ok = resolve("cuMemAddressReserve", x.reserve) && resolve("cuMemAddressFree", x.addr_free) &&
           resolve("cuMemCreate", x.create) && resolve("cuMemRelease", x.release) && resolve("cuMemMap", x.map) &&
           resolve("cuMemUnmap", x.unmap) && resolve("cuMemSetAccess", x.set_access) &&
           resolve("cuMemGetAllocationGranularity", x.granularity);
    return x;
  }();
  return d;
}

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

DeviceBuffer::DeviceBuffer(size_t max_bytes, int device) : max_bytes_(max_bytes) {
  if (device < 0) check(cudaGetDevice(&device_), "cudaGetDevice");
  else device_ = device;
  check(cudaFree(nullptr), "CUDA context");  // make sure a context exists before driver calls
  const Driver& d = driver();
  if (d.ok) {
    const CUmemAllocationProp p = prop_for(device_);
    if (d.granularity(&granularity_, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM) == CUDA_SUCCESS && granularity_ > 0) {
      const size_t reserve = (max_bytes_ + granularity_ - 1) / granularity_ * granularity_;
      if (d.reserve(&base_, reserve ? reserve : granularity_, 0, 0, 0) == CUDA_SUCCESS) {
        max_bytes_ = reserve ? reserve : granularity_;
        vmm_ = true;
      }
    }
  }
}

DeviceBuffer::~DeviceBuffer() { free(); }

void DeviceBuffer::resize(size_t new_bytes) {
  if (new_bytes <= size_) { size_ = new_bytes; return; }
  if (new_bytes > max_bytes_)
    throw std::runtime_error("DeviceBuffer: request of " + std::to_string(new_bytes) + " bytes exceeds the reserved " +
                             std::to_string(max_bytes_));
  if (vmm_) {
    const Driver& d = driver();
    if (new_bytes > mapped_) {
      // grow geometrically so a stream of small inserts maps O(log n) chunks
      size_t want = new_bytes - mapped_;
      if (want < mapped_ / 2) want = mapped_ / 2;
      size_t add = (want + granularity_ - 1) / granularity_ * granularity_;
      if (mapped_ + add > max_bytes_) add = max_bytes_ - mapped_;
      const CUmemAllocationProp p = prop_for(device_);
      CUmemGenericAllocationHandle h;
      if (d.create(&h, add, &p, 0) != CUDA_SUCCESS) throw std::runtime_error("DeviceBuffer: cuMemCreate failed (out of memory?)");
      if (d.map(base_ + mapped_, add, 0, h, 0) != CUDA_SUCCESS) {
        d.release(h);
        throw std::runtime_error("DeviceBuffer: cuMemMap failed");
      }
      CUmemAccessDesc acc{};
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      acc.location.id = device_;
      acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      if (d.set_access(base_ + mapped_, add, &acc, 1) != CUDA_SUCCESS) throw std::runtime_error("DeviceBuffer: cuMemSetAccess failed");
      chunks_.push_back({h, add});
      mapped_ += add;
    }
  } else {
    if (new_bytes > mapped_) {
      size_t cap = mapped_ ? mapped_ * 2 : new_bytes;
      if (cap < new_bytes) cap = new_bytes;
      if (cap > max_bytes_) cap = max_bytes_;
      void* p = nullptr;
      check(cudaMalloc(&p, cap), "cudaMalloc");
      if (base_) {
        check(cudaMemcpy(p, reinterpret_cast<void*>(base_), size_, cudaMemcpyDeviceToDevice), "cudaMemcpy");
        cudaFree(reinterpret_cast<void*>(base_));
      }
      base_ = reinterpret_cast<CUdeviceptr>(p);
      mapped_ = cap;
    }
  }
  size_ = new_bytes;
}

void DeviceBuffer::free() {
  if (vmm_) {
    const Driver& d = driver();
    cudaDeviceSynchronize();
    size_t off = 0;
    for (auto& c : chunks_) {
      d.unmap(base_ + off, c.second);
      d.release(c.first);
      off += c.second;
    }
    chunks_.clear();
    if (base_) d.addr_free(base_, max_bytes_);
    vmm_ = false;
  } else if (base_) {
    cudaFree(reinterpret_cast<void*>(base_));
  }
  base_ = 0;
  size_ = mapped_ = 0;
}

}  // namespace grab
