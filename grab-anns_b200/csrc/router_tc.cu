// Nearest-centroid candidates of a query batch on the tensor cores (tcgen05, tf32 operands,
// fp32 accumulation in TMEM, TMA-staged tiles).
//
// The router needs, per query, the few centroids with the smallest |c|^2 - 2 q.c (or -q.c).
// That is a [nq x dim] x [dim x C] contraction followed by a per-row selection: here the
// contraction runs as tcgen05.mma.kind::tf32 straight from the fp32 queries and centroids
// (TMA copies the rows, the tensor core reads the upper 19 bits of every value), and the
// epilogue keeps each row's T smallest scores.  tf32 products carry ~1e-3 relative error, so
// T = probes + 4 candidates are kept and the consumer (the seed kernel) re-scores them with the
// exact fp32 chain and keeps the best `probes`: the result equals the exact scan unless tf32
// moved a true top-`probes` centroid more than four ranks down.
//
// One CTA per (128-query tile, slice of the centroid tiles); 6 warps:
//   warp 0  TMA producer (2-stage ring of [128 x 32 fp32] query and centroid tiles, 128B swizzle)
//   warp 1  MMA issuer   (4 x tcgen05.mma M128 N128 K8 per stage; owns the TMEM allocation)
//   warps 2-5 epilogue   (tcgen05.ld of the double-buffered 128 x 128 accumulator; thread r owns
//                         query row r: threshold mask, rare sorted insertions into the row's list)
// Every mbarrier wait is bounded; on expiry the kernel raises the status word, all roles leave,
// TMEM is released, and the seed kernel that follows writes "no seed" for every slot.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace grab {
namespace rtc {

using namespace tc;

constexpr int BM = 128, BN = 128, BK = 32;       // BK fp32 = one 128-byte swizzle row
constexpr int STAGES = 2;
constexpr int STAGE_BYTES = (BM + BN) * BK * 4;  // 32 KB
constexpr int THREADS = 192;
constexpr uint32_t kMaxT = 16;                   // candidates kept per row and slice
// Instruction descriptor: D fp32, A/B tf32, both K-major, N=128, M=128.
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);

struct Ctl {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) float cn[4][BN];       // centroid norms of the current tile, one copy per epilogue warp
  uint64_t list[kMaxT][BM];          // list[j][r]: j-th smallest key of row r so far
};

template <int METRIC>
__global__ void __launch_bounds__(THREADS, 2)
route_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_c,
                const float* __restrict__ cnorm, uint64_t nq, uint32_t C, uint32_t kblocks, uint32_t T,
                uint64_t* __restrict__ out_keys, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctl* ctl = reinterpret_cast<Ctl*>(ring + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &ctl->abort_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row0 = blockIdx.x * BM;
  const uint32_t col_tiles = (C + BN - 1) / BN;
  const uint32_t tiles_per = (col_tiles + gridDim.y - 1) / gridDim.y;
  const uint32_t jb = blockIdx.y * tiles_per;
  const uint32_t je = jb + tiles_per < col_tiles ? jb + tiles_per : col_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 4);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ============================ TMA producer ============================
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t issued_phase[STAGES];
      bool issued[STAGES];
      for (int s = 0; s < STAGES; ++s) { issued[s] = false; issued_phase[s] = 0; }
      bool ok = true;
      for (uint32_t j = jb; j < je && ok; ++j) {
        for (uint32_t kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, phase = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&ctl->empty[s]), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t bar = smem_u32(&ctl->full[s]);
          mbar_expect_tx(bar, STAGE_BYTES);
          const uint32_t dst = smem_u32(ring + s * STAGE_BYTES);
          tma_load_2d(dst, &map_q, bar, static_cast<int32_t>(kb * BK), static_cast<int32_t>(row0));
          tma_load_2d(dst + BM * BK * 4, &map_c, bar, static_cast<int32_t>(kb * BK), static_cast<int32_t>(j * BN));
          issued[s] = true;
          issued_phase[s] = phase;
        }
      }
      if (!ok) {
        // leaving early: give copies already in flight a bounded time to land
        for (int s = 0; s < STAGES; ++s)
          if (issued[s])
            for (uint32_t i = 0; i < (1u << 16); ++i)
              if (mbar_try_wait(smem_u32(&ctl->full[s]), issued_phase[s])) break;
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ============================
    if (lane == 0) {
      uint32_t it = 0, tile = 0;
      bool ok = true;
      for (uint32_t j = jb; j < je && ok; ++j) {
        const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
        if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, phase = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&ctl->full[s]), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(a_addr);
          const uint64_t db = smem_desc_sw128(a_addr + BM * BK * 4);
#pragma unroll
          for (uint32_t kk = 0; kk < BK / 8; ++kk) {
            // 8 fp32 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            tc_mma_tf32(d_tmem, da + 2 * kk, db + 2 * kk, kIdescTf32, (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&ctl->empty[s]));  // stage reusable once these MMAs have read it
        }
        if (!ok) break;
        tc_commit(smem_u32(&ctl->tmem_full[acc]));  // accumulator complete
        ++tile;
      }
    }
  } else {
    // ============================ epilogue (warps 2..5) ============================
    const uint32_t quarter = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t r_local = quarter * 32 + lane;
    const bool row_valid = static_cast<uint64_t>(row0) + r_local < nq;
    float* cn = ctl->cn[warp - 2];
    uint32_t cnt = 0, tile = 0;
    float thr = __int_as_float(0x7f800000);  // +inf until the list is full
    bool ok = true;
    for (uint32_t j = jb; j < je && ok; ++j) {
      const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
      const uint32_t c0 = j * BN;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < BN / 32; ++i) {
        const uint32_t c = c0 + i * 32 + lane;
        cn[i * 32 + lane] = (METRIC == GRAB_METRIC_L2 && c < C) ? __ldg(cnorm + c) : 0.0f;
      }
      __syncwarp();
      if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < BN / 32; ++chunk) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld32_issue(taddr + chunk * 32, v);
        tmem_ld_wait(v);
        const uint32_t cbase = c0 + chunk * 32;
        const float4* cn4 = reinterpret_cast<const float4*>(cn + chunk * 32);
        uint32_t m = 0;
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 y = cn4[i4];
          float d0, d1, d2, d3;
          if (METRIC == GRAB_METRIC_L2) {
            d0 = __fmaf_rn(-2.0f, __uint_as_float(v[4 * i4 + 0]), y.x);
            d1 = __fmaf_rn(-2.0f, __uint_as_float(v[4 * i4 + 1]), y.y);
            d2 = __fmaf_rn(-2.0f, __uint_as_float(v[4 * i4 + 2]), y.z);
            d3 = __fmaf_rn(-2.0f, __uint_as_float(v[4 * i4 + 3]), y.w);
          } else {
            d0 = -__uint_as_float(v[4 * i4 + 0]);
            d1 = -__uint_as_float(v[4 * i4 + 1]);
            d2 = -__uint_as_float(v[4 * i4 + 2]);
            d3 = -__uint_as_float(v[4 * i4 + 3]);
          }
          v[4 * i4 + 0] = __float_as_uint(d0);
          v[4 * i4 + 1] = __float_as_uint(d1);
          v[4 * i4 + 2] = __float_as_uint(d2);
          v[4 * i4 + 3] = __float_as_uint(d3);
          m |= (d0 < thr ? 1u : 0u) << (4 * i4 + 0);
          m |= (d1 < thr ? 1u : 0u) << (4 * i4 + 1);
          m |= (d2 < thr ? 1u : 0u) << (4 * i4 + 2);
          m |= (d3 < thr ? 1u : 0u) << (4 * i4 + 3);
        }
        m &= row_valid ? range_bits(cbase, 0, C) : 0u;
        while (m) {  // rare once the list is full and the threshold has tightened
          const uint32_t i = __ffs(m) - 1;
          m &= m - 1;
          const float d = __uint_as_float(pick32(v, i));
          if (!(d < thr)) continue;  // the threshold may have dropped since the mask was built
          const uint64_t key = make_key(d, cbase + i);
          uint32_t pos = cnt < T ? cnt : T - 1;
          if (cnt < T) ++cnt;
          while (pos > 0 && ctl->list[pos - 1][r_local] > key) {
            ctl->list[pos][r_local] = ctl->list[pos - 1][r_local];
            --pos;
          }
          ctl->list[pos][r_local] = key;
          if (cnt == T) thr = key_dist(ctl->list[T - 1][r_local]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
      ++tile;
    }
    if (ok && row_valid) {
      uint64_t* dst = out_keys + ((static_cast<uint64_t>(row0) + r_local) * gridDim.y + blockIdx.y) * T;
      for (uint32_t i = 0; i < T; ++i) dst[i] = i < cnt ? ctl->list[i][r_local] : kMaxKey;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
  if (threadIdx.x == 0 && ctl->abort_flag) *status = GRAB_ERR_TIMEOUT;
}

static int make_map_f32(CUtensorMap* map, const void* base, uint64_t rows, uint32_t dim) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_last_error("route_seeds: cuTensorMapEncodeTiled is not available from the driver");
    return GRAB_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {dim, rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(dim) * 4};
  const cuuint32_t box[2] = {BK, BM};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("route_seeds: cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    return GRAB_ERR_CUDA;
  }
  return GRAB_OK;
}

}  // namespace rtc

// The tensor-core path needs whole TMA boxes to exist and 16-byte aligned rows.
bool route_tc_usable(const float* d_queries, uint64_t nq, uint32_t dim, const float* d_centroids, uint32_t C,
                     uint32_t T) {
  return nq >= rtc::BM && C >= rtc::BN && dim >= rtc::BK && dim % 4 == 0 && T <= rtc::kMaxT &&
         (reinterpret_cast<uintptr_t>(d_queries) & 15u) == 0 && (reinterpret_cast<uintptr_t>(d_centroids) & 15u) == 0;
}

// Slices of the centroid tiles: as many as still fit one wave of 2 CTAs per SM.
uint32_t route_tc_slices(uint64_t nq, uint32_t C) {
  const uint64_t row_tiles = (nq + rtc::BM - 1) / rtc::BM;
  const uint32_t col_tiles = (C + rtc::BN - 1) / rtc::BN;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  uint32_t s = 1;
  while (s < 8 && s + 1 <= col_tiles && row_tiles * (s + 1) <= 2ull * static_cast<uint64_t>(sms)) ++s;
  return s;
}

// out_keys [nq, slices, T]: per slice of the centroid tiles the T smallest (tf32 score, centroid)
// keys of every query, ascending.  *d_status must be zero on entry; set on a stalled pipeline.
int route_tc_launch(int metric, const float* d_queries, uint64_t nq, uint32_t dim, const float* d_centroids,
                    const float* d_cnorm, uint32_t C, uint32_t T, uint32_t slices, uint64_t* out_keys, int* d_status,
                    cudaStream_t st) {
  using namespace rtc;
  CUtensorMap map_q, map_c;
  int rc = make_map_f32(&map_q, d_queries, nq, dim);
  if (rc != GRAB_OK) return rc;
  rc = make_map_f32(&map_c, d_centroids, C, dim);
  if (rc != GRAB_OK) return rc;
  const uint32_t kblocks = (dim + BK - 1) / BK;
  const size_t smem = STAGES * STAGE_BYTES + sizeof(Ctl) + 1024;
  const dim3 grid(static_cast<unsigned>((nq + BM - 1) / BM), slices);
  if (metric == GRAB_METRIC_L2) {
    GRAB_CUDA_TRY(cudaFuncSetAttribute(route_tc_kernel<GRAB_METRIC_L2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    route_tc_kernel<GRAB_METRIC_L2><<<grid, THREADS, smem, st>>>(map_q, map_c, d_cnorm, nq, C, kblocks, T, out_keys,
                                                                d_status);
  } else {
    GRAB_CUDA_TRY(cudaFuncSetAttribute(route_tc_kernel<GRAB_METRIC_IP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    route_tc_kernel<GRAB_METRIC_IP><<<grid, THREADS, smem, st>>>(map_q, map_c, d_cnorm, nq, C, kblocks, T, out_keys,
                                                                d_status);
  }
  GRAB_CUDA_TRY(cudaGetLastError());
  return GRAB_OK;
}

}  // namespace grab
