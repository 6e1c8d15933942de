// Stand-in for the reference's src/index/config.cuh: the compile-time constants its callers may name.  Nothing
// in this library depends on them (dimension, team size and block size are run-time or per-kernel choices here).
#pragma once
#include <cstddef>
#include <cstdint>

#ifndef CUDA_DEVICE_ID
#define CUDA_DEVICE_ID 0  // src/index/common.cuh:5-7
#endif

namespace cagra {
namespace config {

constexpr size_t MAX_SHARED_MEMORY = 48 * 1024;  // src/index/config.cuh:10
constexpr uint32_t DIM = 1024;                   // the dimension the reference's v1 insert is compiled for (:12)
constexpr uint32_t TEAM_SIZE = 32;               // (:13)
constexpr uint32_t BLOCK_SIZE = 256;             // (:14)
constexpr uint32_t DEFAULT_HASH_BITLEN = 12;     // (:16)

}  // namespace config
}  // namespace cagra
