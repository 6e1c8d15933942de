// All-pairs kNN candidates on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// with a fused per-row running top-KC in the epilogue and an exact fp32 re-rank.
//
// This is the dense contraction of the build: it replaces the reference's per-bucket RAFT
// brute force (src/index/raft_help.cuh:74-172) and its FAISS IVF-PQ candidate searches
// (src/index/cagra.cu:76-131, cagra_opt.cu:813-847), followed -- as there
// (cagra.cu:138, cagra_opt.cu:48-148) -- by exact distances over the candidates.
//
//   d(x,y) = |y|^2 - 2 x.y  (+|x|^2, constant per row, dropped for ranking)
//
// x.y runs as bf16 x bf16 -> fp32 MMAs, M=128 rows x N=128 columns per tile, K = 64 per
// pipeline stage.  "Split" precision stores every value as hi+lo bf16 and concatenates
// [hi,lo,hi].[hi,hi,lo] along K, which recovers ~fp32 products at 3x the MMA work.
//
// Persistent CTAs, two per SM, 6 warps each:
//   warp 0   TMA producer   (cp.async.bulk.tensor 2D, 128B swizzle, 3-stage ring, mbarriers)
//   warp 1   MMA issuer     (one lane issues tcgen05.mma; tcgen05.commit frees ring stages and
//                            publishes the accumulator; owns the TMEM allocation)
//   warps 2-5 epilogue      (tcgen05.ld of a double-buffered 128x128 fp32 accumulator, the next
//                            32 columns in flight while the current 32 are tested; thread r owns
//                            row r: branch-free threshold mask, rare appends to the row's
//                            candidate buffer; a full buffer is cut back to its KC smallest by a
//                            warp-cooperative radix select -- no sort)
// Every mbarrier wait is bounded; on expiry the kernel raises a flag, all roles leave their
// loops, TMEM is released and the host sees GRAB_ERR_TIMEOUT.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "windows.cuh"

namespace grab {

namespace tc {

constexpr int BM = 128, BN = 128, BK = 64;  // BK bf16 = one 128-byte swizzle row
#ifndef GRAB_KNN_STAGES
#define GRAB_KNN_STAGES 3
#endif
constexpr int STAGES = GRAB_KNN_STAGES;
constexpr int CTAS_PER_SM = 2;
constexpr int STAGE_BYTES = (BM + BN) * BK * 2;  // 32 KB
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;  // one K block of either operand: 16 KB
// "A resident": when the whole K extent of a row tile fits kAresBlocks K blocks, the row tile's A operand is loaded
// ONCE per row tile and stays in shared memory for the sweep over the column tiles; only B streams through the ring
// (kAresStages stages of 16 KB).  Per 128 x 128 tile the SM then reads 48 KB instead of 96 KB through its L2 port,
// which is what bounds the MMA side of this kernel (measured: 0.28 s of the 0.37 s at 1M x 128 with no epilogue
// work at all, i.e. 72 bytes per clock and SM).
constexpr int kAresBlocks = 3;
constexpr int kAresStages = (STAGES * STAGE_BYTES - kAresBlocks * A_BYTES) / B_BYTES;  // same footprint: 3
// Epilogue warpgroups per CTA.  With two, warps 2-5 take the tiles of accumulator 0 and warps 6-9 those of
// accumulator 1 (consecutive column tiles), each group with candidate buffers and thresholds of its own, so that
// twice as many warps hide the epilogue's latencies; a row then leaves two candidate lists for the re-rank.
// Measured at 1M x 128 (96 registers, one TMEM buffer per thread): own-block sweep 53 -> 36 ms, but the cross-bucket
// sweep 333 -> 358 ms and the re-rank of two lists 29 -> 56 ms: whole build 0.60 -> 0.64 s.  Off.
#ifndef GRAB_KNN_EPI_WGS
#define GRAB_KNN_EPI_WGS 1
#endif
constexpr int EPI_WGS = GRAB_KNN_EPI_WGS;
static_assert(EPI_WGS == 1 || EPI_WGS == 2, "one epilogue warpgroup per accumulator at most");
constexpr int THREADS = 64 + 128 * EPI_WGS;
// Instruction descriptor: D fp32, A/B bf16, both K-major, N=128, M=128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);

// Profiling build only (-DGRAB_KNN_PHASE_CLOCKS=1): SM cycles the epilogue warps spend waiting for an accumulator,
// waiting for TMEM loads, in chunks without / with a value below a threshold, and in buffer cuts; summed over all
// launches, read with grab_debug_knn_phase_cycles().  Slots: 0 accumulator wait, 1 TMEM load wait, 2 chunks without a
// hit, 3 chunks with a hit, 4 cuts, 5 rest; 8-13 the event counts of slots 0-5.
#ifndef GRAB_KNN_PHASE_CLOCKS
#define GRAB_KNN_PHASE_CLOCKS 0
#endif
#if GRAB_KNN_PHASE_CLOCKS
__device__ unsigned long long g_knn_phase[16];
#define KNN_PHASE(i)                                                           \
  do {                                                                         \
    const long long now_ = clock64();                                          \
    if (lane == 0) { ph[i] += static_cast<unsigned long long>(now_ - t_ph); ++ph[8 + (i)]; } \
    t_ph = now_;                                                               \
  } while (0)
#else
#define KNN_PHASE(i)
#endif

// ------------------------------------------------------------------ epilogue helpers
__device__ __forceinline__ float fmin3(float a, float b, float c) {  // one instruction on sm_100
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Cut the candidate buffers of the rows that are (nearly) full back to their KC smallest keys
// and tighten the rows' thresholds.  Warp-cooperative, one row at a time: the row's keys sit in
// registers (element g = j*32 + lane), a 4-pass radix select on the ordered distance finds the
// KC-th smallest value, a ballot compaction writes the survivors back.  No ordering is produced:
// the exact re-rank sorts later.  Kept out of line: it runs rarely and would otherwise bloat
// the hot loop's instruction footprint.
// Capacity of a row's candidate buffer: a cut happens when fewer than 32 free slots are left and brings the row back to
// KC entries, so CAP - 32 - KC appends lie between two cuts of a row (96 / 160 / 96 / 224 for KC 32 / 64 / 128 / 256).
__host__ __device__ constexpr uint32_t cap_of(uint32_t kc) { return kc < 128 ? 4 * kc + (kc == 32 ? 32 : 0) : 2 * kc; }

template <int KC>
__device__ __noinline__ uint2 compress_rows(uint64_t* warp_buf, uint32_t* hist, uint32_t lane, uint32_t cnt,
                                            float thr, bool force) {
  constexpr uint32_t CAP = cap_of(KC);
  constexpr int NREG = CAP / 32;
  const uint32_t lt_mask = (1u << lane) - 1u;
  __syncwarp();
  uint32_t need = __ballot_sync(0xFFFFFFFFu, force ? (cnt > KC) : (cnt > CAP - 32));
  while (need) {
    const int src = __ffs(need) - 1;
    need &= need - 1;
    const uint32_t c_src = __shfl_sync(0xFFFFFFFFu, cnt, src);
    uint64_t* rb = warp_buf + static_cast<uint64_t>(src) * CAP;
    uint64_t k[NREG];
#pragma unroll
    for (int j = 0; j < NREG; ++j) {
      const uint32_t g = j * 32 + lane;
      k[j] = g < c_src ? rb[g] : kMaxKey;
    }
    uint32_t prefix = 0, hi_mask = 0, want = KC;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
      const uint32_t shift = 24 - 8 * pass;
      for (uint32_t b = lane; b < 256; b += 32) hist[b] = 0;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < NREG; ++j) {
        const uint32_t o = static_cast<uint32_t>(k[j] >> 32);
        if (j * 32 + lane < c_src && ((o ^ prefix) & hi_mask) == 0) atomicAdd(&hist[(o >> shift) & 255u], 1u);
      }
      __syncwarp();
      uint32_t local[8], sum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) { local[i] = hist[lane * 8 + i]; sum += local[i]; }
      uint32_t incl = sum;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if (static_cast<int>(lane) >= off) incl += t;
      }
      const uint32_t excl = incl - sum;
      const bool mine = excl < want && want <= incl;
      uint32_t digit = 0, before = 0;
      if (mine) {
        uint32_t run = excl;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (run + local[i] >= want) { digit = lane * 8 + i; before = run; break; }
          run += local[i];
        }
      }
      const uint32_t owner = __ffs(__ballot_sync(0xFFFFFFFFu, mine)) - 1;  // exactly one lane: want <= c_src
      digit = __shfl_sync(0xFFFFFFFFu, digit, owner & 31);
      before = __shfl_sync(0xFFFFFFFFu, before, owner & 31);
      want -= before;
      prefix |= digit << shift;
      hi_mask |= 0xFFu << shift;
      __syncwarp();
    }
    // `prefix` = ordered distance of the KC-th smallest key, `want` of the keys equal to it stay
    uint32_t base = 0, eq_seen = 0;
#pragma unroll
    for (int j = 0; j < NREG; ++j) {
      const uint32_t o = static_cast<uint32_t>(k[j] >> 32);
      const bool valid = j * 32 + lane < c_src;
      const bool eq = valid && o == prefix;
      const uint32_t eqm = __ballot_sync(0xFFFFFFFFu, eq);
      const bool take = (valid && o < prefix) || (eq && eq_seen + __popc(eqm & lt_mask) < want);
      eq_seen += __popc(eqm);
      const uint32_t tm = __ballot_sync(0xFFFFFFFFu, take);
      if (take) rb[base + __popc(tm & lt_mask)] = k[j];
      base += __popc(tm);
    }
    if (static_cast<int>(lane) == src) {
      cnt = KC;
      thr = ordered_to_float(prefix);
    }
  }
  __syncwarp();
  return make_uint2(cnt, __float_as_uint(thr));
}

struct TileRange {
  uint32_t row0, rows;       // rows of this tile that exist
  uint32_t jb, je;           // column tiles [jb, je)
  uint32_t skip_lo, skip_hi; // column tiles fully inside every row's exclusion are skipped
  uint32_t safe_lo, safe_hi; // columns inside every row's window ...
  uint32_t ex_lo, ex_hi;     // ... and outside [ex_lo, ex_hi) need no per-element mask
};

__device__ __forceinline__ TileRange tile_range(const ScanWindow* windows, uint64_t n, uint32_t rt) {
  TileRange t;
  t.row0 = rt * BM;
  const uint64_t last = (t.row0 + BM <= n ? t.row0 + BM : n) - 1;
  t.rows = static_cast<uint32_t>(last - t.row0 + 1);
  const ScanWindow a = windows[t.row0], b = windows[last];
  // windows are monotone in the row id (blocks are contiguous id ranges)
  t.jb = a.begin / BN;
  t.je = (b.end + BN - 1) / BN;
  t.skip_lo = a.xbegin > b.xbegin ? a.xbegin : b.xbegin;
  t.skip_hi = a.xend < b.xend ? a.xend : b.xend;
  t.safe_lo = b.begin;
  t.safe_hi = a.end;
  t.ex_lo = a.xbegin;
  t.ex_hi = b.xend;
  return t;
}
__device__ __forceinline__ bool tile_skipped(const TileRange& t, uint32_t j) {
  const uint32_t c0 = j * BN;
  return c0 >= t.skip_lo && c0 + BN <= t.skip_hi;
}

struct SharedCtl {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], a_full, a_empty;
  uint32_t tmem_base;
  int abort_flag;
  uint32_t hist[4 * EPI_WGS][256];    // radix-select histogram per epilogue warp
};

template <int KC, bool ARES>
__global__ void __launch_bounds__(THREADS, CTAS_PER_SM)
knn_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const ScanWindow* __restrict__ windows, uint64_t n, uint32_t kblocks, uint32_t last_kk,
              uint32_t num_row_tiles, uint64_t* __restrict__ scratch, uint64_t* __restrict__ out_keys,
              const float* __restrict__ thr0, int* __restrict__ status) {
  constexpr uint32_t CAP = cap_of(KC);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // stage s: A tile at s*STAGE_BYTES, B tile 16 KB after it; control block after the ring
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(ring + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &ctl->abort_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[a]), 4);
    }
    mbar_init(smem_u32(&ctl->a_full), 1);
    mbar_init(smem_u32(&ctl->a_empty), 1);
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
      uint32_t it = 0, nrt = 0;
      uint32_t issued_phase[STAGES];
      bool issued[STAGES];
      for (int s = 0; s < STAGES; ++s) { issued[s] = false; issued_phase[s] = 0; }
      bool a_issued = false;
      uint32_t a_phase = 0;
      constexpr uint32_t NST = ARES ? kAresStages : STAGES;
      unsigned char* b_ring = ring + kAresBlocks * A_BYTES;  // ARES: the B ring behind the resident A blocks
      bool ok = true;
      for (uint32_t rt = blockIdx.x; rt < num_row_tiles && ok; rt += gridDim.x) {
        const TileRange t = tile_range(windows, n, rt);
        if (ARES) {
          // the MMAs of the previous row tile must be done with A before it is overwritten
          if (!mbar_wait(smem_u32(&ctl->a_empty), (nrt & 1) ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t bar = smem_u32(&ctl->a_full);
          mbar_expect_tx(bar, kblocks * A_BYTES);
          for (uint32_t kb = 0; kb < kblocks; ++kb)
            tma_load_2d(smem_u32(ring + kb * A_BYTES), &map_a, bar, static_cast<int32_t>(kb * BK),
                        static_cast<int32_t>(t.row0));
          a_issued = true;
          a_phase = nrt & 1;
          ++nrt;
        }
        for (uint32_t j = t.jb; j < t.je && ok; ++j) {
          if (tile_skipped(t, j)) continue;
          for (uint32_t kb = 0; kb < kblocks; ++kb, ++it) {
            const uint32_t s = it % NST, phase = (it / NST) & 1;
            if (!mbar_wait(smem_u32(&ctl->empty[s]), phase ^ 1, abort_flag)) { ok = false; break; }
            const uint32_t bar = smem_u32(&ctl->full[s]);
            if (ARES) {
              mbar_expect_tx(bar, B_BYTES);
              tma_load_2d(smem_u32(b_ring + s * B_BYTES), &map_b, bar, static_cast<int32_t>(kb * BK),
                          static_cast<int32_t>(j * BN));
            } else {
              mbar_expect_tx(bar, STAGE_BYTES);
              const uint32_t dst = smem_u32(ring + s * STAGE_BYTES);
              tma_load_2d(dst, &map_a, bar, static_cast<int32_t>(kb * BK), static_cast<int32_t>(t.row0));
              tma_load_2d(dst + A_BYTES, &map_b, bar, static_cast<int32_t>(kb * BK), static_cast<int32_t>(j * BN));
            }
            issued[s] = true;
            issued_phase[s] = phase;
          }
        }
      }
      if (!ok) {
        // leaving early: give copies already in flight a bounded time to land
        for (int s = 0; s < STAGES; ++s)
          if (issued[s])
            for (uint32_t i = 0; i < (1u << 16); ++i)
              if (mbar_try_wait(smem_u32(&ctl->full[s]), issued_phase[s])) break;
        if (a_issued)
          for (uint32_t i = 0; i < (1u << 16); ++i)
            if (mbar_try_wait(smem_u32(&ctl->a_full), a_phase)) break;
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ============================
    if (lane == 0) {
      uint32_t it = 0, tile = 0, nrt = 0;
      constexpr uint32_t NST = ARES ? kAresStages : STAGES;
      unsigned char* b_ring = ring + kAresBlocks * A_BYTES;
      bool ok = true;
      for (uint32_t rt = blockIdx.x; rt < num_row_tiles && ok; rt += gridDim.x) {
        const TileRange t = tile_range(windows, n, rt);
        if (ARES) {
          if (!mbar_wait(smem_u32(&ctl->a_full), nrt & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        for (uint32_t j = t.jb; j < t.je && ok; ++j) {
          if (tile_skipped(t, j)) continue;
          const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
          if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (uint32_t kb = 0; kb < kblocks; ++kb, ++it) {
            const uint32_t s = it % NST, phase = (it / NST) & 1;
            if (!mbar_wait(smem_u32(&ctl->full[s]), phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(ARES ? ring + kb * A_BYTES : ring + s * STAGE_BYTES);
            const uint32_t b_addr = ARES ? smem_u32(b_ring + s * B_BYTES) : a_addr + A_BYTES;
            const uint64_t da = smem_desc_sw128(a_addr);
            const uint64_t db = smem_desc_sw128(b_addr);
            // the last K block holds operand columns only in its first last_kk slices of 16 (the rest is zero padding)
            const uint32_t nkk = kb + 1 == kblocks ? last_kk : BK / 16;
#pragma unroll
            for (uint32_t kk = 0; kk < BK / 16; ++kk) {
              // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
              if (kk < nkk) tc_mma_bf16(d_tmem, da + 2 * kk, db + 2 * kk, kIdesc, (kb | kk) != 0 ? 1u : 0u);
            }
            tc_commit(smem_u32(&ctl->empty[s]));  // stage reusable once these MMAs have read it
          }
          if (!ok) break;
          tc_commit(smem_u32(&ctl->tmem_full[acc]));  // accumulator complete
          ++tile;
        }
        if (ARES && ok) {
          tc_commit(smem_u32(&ctl->a_empty));  // arrives once every MMA of this row tile has read A
          ++nrt;
        }
      }
    }
  } else {
    // ============================ epilogue (warps 2..5, and 6..9 with two groups) ============================
    const uint32_t quarter = warp & 3;          // TMEM lane quarter this warp may read
    const uint32_t wg = (warp - 2) >> 2;        // epilogue warpgroup = the accumulator it serves when there are two
    const uint32_t r_local = quarter * 32 + lane;
    uint64_t* warp_buf = scratch + ((static_cast<uint64_t>(blockIdx.x) * EPI_WGS + wg) * BM + quarter * 32) * CAP;
    uint64_t* my_buf = warp_buf + static_cast<uint64_t>(lane) * CAP;
    uint32_t tile = 0;
    bool ok = true;

    uint32_t* hist = ctl->hist[warp - 2];
#if GRAB_KNN_PHASE_CLOCKS
    unsigned long long ph[16] = {};
    long long t_ph = clock64();
#endif

    for (uint32_t rt = blockIdx.x; rt < num_row_tiles && ok; rt += gridDim.x) {
      const TileRange t = tile_range(windows, n, rt);
      const bool row_valid = r_local < t.rows;
      ScanWindow w{0, 0, 0, 0};
      if (row_valid) w = windows[t.row0 + r_local];
      uint32_t cnt = 0;
      // the row's threshold starts at +inf, or at the bound a pass over a sample of the columns found for it
      float thr = thr0 != nullptr && row_valid ? thr0[t.row0 + r_local] : __int_as_float(0x7f800000);
      for (uint32_t j = t.jb; j < t.je && ok; ++j) {
        if (tile_skipped(t, j)) continue;
        const uint32_t acc = tile & 1, acc_phase = (tile >> 1) & 1;
        if (EPI_WGS == 2 && acc != wg) { ++tile; continue; }  // the other group's tile
        const uint32_t c0 = j * BN;
        KNN_PHASE(5);
        if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        KNN_PHASE(0);
        const bool need_mask = !(c0 >= t.safe_lo && c0 + BN <= t.safe_hi && (c0 + BN <= t.ex_lo || c0 >= t.ex_hi));
        const uint32_t taddr = tmem_base + ((quarter * 32) << 16) + acc * BN;

        // One 32-column chunk.  The accumulator already IS the ranking distance |y|^2 - 2 x.y (the column norm rides
        // along the contraction as three extra K columns against ones), so the common case costs one min per value:
        // a min tree over the chunk, one compare with the row's threshold, one warp vote.  Only chunks in which some
        // row has a value below its threshold build the per-element mask and append.
        auto process = [&](uint32_t (&v)[32], uint32_t chunk) {
#if defined(GRAB_KNN_PROBE_NO_EPILOGUE)  // timing probe only: results are wrong
          if (v[0] == 0x7fc12345u) my_buf[cnt++] = chunk;
          return;
#endif
          float m8[8];  // three-input minima: 16 instead of 24 operations for the groups of four, 4 instead of 7 above
#pragma unroll
          for (int i = 0; i < 8; ++i)
            m8[i] = fminf(fmin3(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2])),
                          __uint_as_float(v[4 * i + 3]));
          const float mn = fmin3(fmin3(m8[0], m8[1], m8[2]), fmin3(m8[3], m8[4], m8[5]), fminf(m8[6], m8[7]));
          const bool hit = row_valid && mn < thr;
          if (!__any_sync(0xFFFFFFFFu, hit)) { KNN_PHASE(2); return; }
          if (hit) {
            const uint32_t cbase = c0 + chunk * 32;
            // the min tree's first level already says which groups of four hold a value below the threshold
            // (usually one): only those are looked at element by element.  Measured and slower (full sweeps of the
            // 1M x 128 build, own block / other blocks): a warp-uniform loop over the union of the rows' group masks
            // with a switch per group 135 / 495 ms, appends straight from the registers of each flagged group without
            // the mask word 64 / 358 ms, against 55 / 339 ms for this form.
            uint32_t m = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (m8[i] < thr) {
                m |= (__uint_as_float(v[4 * i]) < thr ? 1u : 0u) << (4 * i);
                m |= (__uint_as_float(v[4 * i + 1]) < thr ? 1u : 0u) << (4 * i + 1);
                m |= (__uint_as_float(v[4 * i + 2]) < thr ? 1u : 0u) << (4 * i + 2);
                m |= (__uint_as_float(v[4 * i + 3]) < thr ? 1u : 0u) << (4 * i + 3);
              }
            }
            if (need_mask) m &= range_bits(cbase, w.begin, w.end) & ~range_bits(cbase, w.xbegin, w.xend);
            while (m) {
              const uint32_t i = __ffs(m) - 1;
              m &= m - 1;
              my_buf[cnt++] = make_key(__uint_as_float(pick32(v, i)), cbase + i);
            }
          }
          KNN_PHASE(3);
          if (__any_sync(0xFFFFFFFFu, cnt > CAP - 32)) {
            const uint2 r = compress_rows<KC>(warp_buf, hist, lane, cnt, thr, false);
            cnt = r.x;
            thr = __uint_as_float(r.y);
            KNN_PHASE(4);
          }
        };

#if defined(GRAB_KNN_PROBE_NO_TMEM_LOAD)  // timing probe only: the accumulator is never read
        if (false)
#endif
        if (EPI_WGS == 1) {
          // one group: the next 32 columns are in flight while the current 32 are tested
          uint32_t va[32], vb[32];
          tmem_ld32_issue(taddr, va);
          tmem_ld_wait(va);
          KNN_PHASE(1);
#pragma unroll 1
          for (uint32_t pair = 0; pair < BN / 64; ++pair) {
            tmem_ld32_issue(taddr + pair * 64 + 32, vb);
            process(va, 2 * pair);
            tmem_ld_wait(vb);
            KNN_PHASE(1);
            if (pair + 1 < BN / 64) tmem_ld32_issue(taddr + pair * 64 + 64, va);
            process(vb, 2 * pair + 1);
            if (pair + 1 < BN / 64) { tmem_ld_wait(va); KNN_PHASE(1); }
          }
        } else {
          // two groups: one buffer per thread (the register budget of 640 threads per SM); the other group's warps
          // cover the load latency
          uint32_t va[32];
#pragma unroll 1
          for (uint32_t chunk = 0; chunk < BN / 32; ++chunk) {
            tmem_ld32_issue(taddr + chunk * 32, va);
            tmem_ld_wait(va);
            KNN_PHASE(1);
            process(va, chunk);
          }
        }

        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
        ++tile;
      }
      if (!ok) break;
      // final cut of this row tile: at most KC candidates per row (unordered; the re-rank sorts)
      {
        const uint2 r = compress_rows<KC>(warp_buf, hist, lane, cnt, thr, true);
        cnt = r.x;
        thr = __uint_as_float(r.y);
      }
      for (uint32_t r = 0; r < 32; ++r) {
        const uint32_t c_r = __shfl_sync(0xFFFFFFFFu, cnt, r);
        const uint32_t row = t.row0 + quarter * 32 + r;
        if (row >= n) continue;  // uniform across the warp
        const uint64_t* rb = warp_buf + static_cast<uint64_t>(r) * CAP;
        for (uint32_t i = lane; i < KC; i += 32)
          out_keys[(static_cast<uint64_t>(row) * EPI_WGS + wg) * KC + i] = i < c_r ? rb[i] : kMaxKey;
      }
      __syncwarp();
    }
#if GRAB_KNN_PHASE_CLOCKS
    KNN_PHASE(5);
    if (lane == 0 && thr0 != nullptr)  // the seeded full sweeps only
      for (int i = 0; i < 16; ++i) atomicAdd(&g_knn_phase[i], ph[i]);
#endif
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
  if (threadIdx.x == 0 && ctl->abort_flag) *status = GRAB_ERR_TIMEOUT;
}

#if GRAB_KNN_PHASE_CLOCKS
}  // namespace tc
}  // namespace grab
extern "C" int grab_debug_knn_phase_cycles(unsigned long long* out16, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out16, grab::tc::g_knn_phase, sizeof(unsigned long long) * 16);
  if (e == cudaSuccess && reset) {
    unsigned long long zero[16] = {};
    e = cudaMemcpyToSymbol(grab::tc::g_knn_phase, zero, sizeof(zero));
  }
  return e == cudaSuccess ? 0 : -1;
}
namespace grab {
namespace tc {
#endif

// ------------------------------------------------------------------ operand preparation
// Deterministic column means: fixed row chunks, fixed summation order.
constexpr int kMeanChunk = 4096;
__global__ void mean_partial_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, float* __restrict__ partial) {
  const uint64_t r0 = static_cast<uint64_t>(blockIdx.x) * kMeanChunk;
  const uint64_t r1 = r0 + kMeanChunk < n ? r0 + kMeanChunk : n;
  for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
    float s = 0.0f;
    for (uint64_t r = r0; r < r1; ++r) s += x[r * dim + d];
    partial[static_cast<uint64_t>(blockIdx.x) * dim + d] = s;
  }
}
__global__ void mean_final_kernel(const float* __restrict__ partial, uint32_t nchunks, uint32_t dim, uint64_t n,
                                  float* __restrict__ mean) {
  const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= dim) return;
  float s = 0.0f;
  for (uint32_t c = 0; c < nchunks; ++c) s += partial[static_cast<uint64_t>(c) * dim + d];
  mean[d] = s / static_cast<float>(n);
}

// fp32 rows -> bf16 operands of  acc(x, y) = |y|^2 - 2 x.y  (the ranking distance itself; inner product: -2 x.y).
// With v = x - mean:  split == 0: A = [bf16(v), 1, 1, 1], B = [-2 bf16(v), n0, n1, n2], K = dim + 3;
// split == 1: hi = bf16(v), lo = bf16(v - hi): A = [hi, lo, hi, 1, 1, 1], B = -2 [hi, hi, lo] then n0, n1, n2,
// K = 3 dim + 3.  n0 + n1 + n2 = |v|^2 to 24 bits (three bf16 terms), carried through the contraction against the
// ones, so that the epilogue has no arithmetic left to do; -2 x is exact in bf16.  Columns up to kp are zero.
// One warp per row.
__global__ void prep_operands_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, const float* __restrict__ mean,
                                     int split, int metric, uint32_t kp, __nv_bfloat16* __restrict__ a,
                                     __nv_bfloat16* __restrict__ b) {
  const uint64_t r = (blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (r >= n) return;
  float s = 0.0f;
  for (uint32_t d = lane; d < dim; d += 32) {
    const float v = x[r * dim + d] - (mean ? mean[d] : 0.0f);
    s = __fmaf_rn(v, v, s);
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const __nv_bfloat16 hi2 = __float2bfloat16_rn(-2.0f * __bfloat162float(hi));
    if (!split) {
      a[r * kp + d] = hi;
      b[r * kp + d] = hi2;
    } else {
      const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
      const __nv_bfloat16 lo2 = __float2bfloat16_rn(-2.0f * __bfloat162float(lo));
      a[r * kp + d] = hi; a[r * kp + dim + d] = lo; a[r * kp + 2 * dim + d] = hi;
      b[r * kp + d] = hi2; b[r * kp + dim + d] = hi2; b[r * kp + 2 * dim + d] = lo2;
    }
  }
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
  const uint32_t used = split ? 3 * dim : dim;
  for (uint32_t d = used + lane; d < kp; d += 32) {
    a[r * kp + d] = __float2bfloat16_rn(d < used + 3 ? 1.0f : 0.0f);
    b[r * kp + d] = __float2bfloat16_rn(0.0f);
  }
  __syncwarp();
  if (lane == 0) {
    const float nrm = metric == GRAB_METRIC_L2 ? s : 0.0f;
    const __nv_bfloat16 n0 = __float2bfloat16_rn(nrm);
    const float r1 = nrm - __bfloat162float(n0);
    const __nv_bfloat16 n1 = __float2bfloat16_rn(r1);
    const __nv_bfloat16 n2 = __float2bfloat16_rn(r1 - __bfloat162float(n1));
    b[r * kp + used] = n0;
    b[r * kp + used + 1] = n1;
    b[r * kp + used + 2] = n2;
  }
}

// ------------------------------------------------------------------ exact re-rank
// One CTA per row: canonical fp32 distances of the KC candidates, sorted by (dist, id).
constexpr int kRerankThreads = 128;
template <int METRIC>
__global__ void __launch_bounds__(kRerankThreads)
rerank_kernel(const float* __restrict__ data, uint32_t dim, const uint64_t* __restrict__ cand_keys, uint32_t kc,
              uint32_t k, uint32_t* __restrict__ out_ids, float* __restrict__ out_dists) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
  float* q_smem = reinterpret_cast<float*>(keys + kc);
  const uint64_t row = blockIdx.x;
  const uint32_t tid = threadIdx.x;
  const int lane8 = tid & (kTeam - 1);
  const uint32_t team = tid / kTeam;
  constexpr uint32_t teams = kRerankThreads / kTeam;
  const uint32_t nchunk = dim / 4;
  for (uint32_t i = tid; i < dim; i += kRerankThreads) q_smem[i] = data[row * dim + i];
  __syncthreads();
  for (uint32_t j0 = 0; j0 < kc; j0 += teams) {
    const uint32_t j = j0 + team;
    const uint64_t ck = j < kc ? cand_keys[row * kc + j] : kMaxKey;
    const bool valid = ck != kMaxKey;
    const uint32_t id = key_id(ck);
    const float d = team_distance_smem<METRIC>(q_smem, data + static_cast<size_t>(id) * dim, nchunk, lane8, valid);
    if (lane8 == 0 && j < kc) keys[j] = valid ? make_key(d, id) : kMaxKey;
  }
  __syncthreads();
  block_bitonic_sort(keys, kc);
  for (uint32_t i = tid; i < k; i += kRerankThreads) {
    const uint64_t key = i < kc ? keys[i] : kMaxKey;
    out_ids[row * k + i] = key == kMaxKey ? kInvalid : key_id(key);
    if (out_dists) out_dists[row * k + i] = key == kMaxKey ? kFltMax : key_dist(key);
  }
}

// ------------------------------------------------------------------ threshold seeding
// A first pass over every `stride`-th column gives each row a bound on its final threshold: the kSeedKC-th
// smallest ranking distance among the sampled columns of the row's window.  About kSeedKC * stride columns of the
// full sweep lie below it, far more than the `want` the row keeps (it falls short only if kSeedKC of the row's
// true top-`want` columns are sampled: Binomial(want, 1/stride) >= kSeedKC, below 1e-9 for the sizes used), so the
// full sweep starts with a threshold that rejects all but a few hundred columns instead of tightening it from
// +inf over the first hundred thousand.  Windows in sample space: column c = stride * c'.
constexpr uint32_t kSeedKC = 32;

__global__ void sample_window_kernel(const ScanWindow* __restrict__ w, uint64_t n, uint32_t stride,
                                     ScanWindow* __restrict__ ws) {
  const uint64_t r = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  if (r >= n) return;
  const ScanWindow a = w[r];
  ScanWindow b;
  b.begin = (a.begin + stride - 1) / stride;
  b.end = (a.end + stride - 1) / stride;
  b.xbegin = (a.xbegin + stride - 1) / stride;
  b.xend = (a.xend + stride - 1) / stride;
  ws[r] = b;
}

// thr0[r] = the kSeedKC-th smallest of the row's sample keys (one list of kSeedKC per epilogue warpgroup); +inf when
// the sample held fewer (the row's window is small).  One warp per row; keys are distinct, so a key's rank is the
// number of keys below it.
__global__ void seed_threshold_kernel(const uint64_t* __restrict__ keys, uint64_t n, float* __restrict__ thr0) {
  const uint64_t r = (blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (r >= n) return;
  static_assert(kSeedKC == 32, "one key per lane and list");
  uint64_t mine[EPI_WGS];
  uint32_t below[EPI_WGS];
#pragma unroll
  for (int g = 0; g < EPI_WGS; ++g) { mine[g] = keys[(r * EPI_WGS + g) * kSeedKC + lane]; below[g] = 0; }
#pragma unroll
  for (int h = 0; h < EPI_WGS; ++h)
    for (uint32_t j = 0; j < 32; ++j) {
      const uint64_t o = __shfl_sync(0xFFFFFFFFu, mine[h], j);
#pragma unroll
      for (int g = 0; g < EPI_WGS; ++g) below[g] += o < mine[g];
    }
  float t = __int_as_float(0x7f800000);
  bool found = false;
#pragma unroll
  for (int g = 0; g < EPI_WGS; ++g)
    if (below[g] == kSeedKC - 1 && mine[g] != kMaxKey) { t = key_dist(mine[g]); found = true; }
  const uint32_t who = __ballot_sync(0xFFFFFFFFu, found);
  if (who == 0) { if (lane == 0) thr0[r] = t; }
  else if (lane == static_cast<uint32_t>(__ffs(who) - 1)) thr0[r] = t;
}

// ------------------------------------------------------------------ host side
// row_stride: the map views every row_stride-th row of the operand (`rows` of them)
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t kp, uint32_t row_stride = 1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_last_error("knn_tc: cuTensorMapEncodeTiled is not available from the driver");
    return GRAB_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {kp, rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kp) * 2 * row_stride};
  const cuuint32_t box[2] = {BK, BM};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("knn_tc: cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    return GRAB_ERR_CUDA;
  }
  return GRAB_OK;
}

}  // namespace tc

// GRAB_KNN_SEED=0 in the environment switches the threshold seeding off (for comparisons).
static bool seed_thresholds_enabled() {
  static const bool on = [] {
    const char* v = getenv("GRAB_KNN_SEED");
    return !(v && v[0] == '0');
  }();
  return on;
}

static bool a_resident_enabled() {
  static const bool on = [] {
    const char* v = getenv("GRAB_KNN_ARES");
    return !(v && v[0] == '0');
  }();
  return on;
}

// precision 1: bf16 operands; 2: split bf16 (hi+lo), close to fp32 products.
int knn_tc_impl(const float* d_dataset, uint64_t n, uint32_t dim, int metric, const uint64_t* h_block_offsets,
                uint32_t num_blocks, uint32_t k, int mode, int precision, uint32_t* d_out_knn,
                float* d_out_dists, cudaStream_t st) {
  using namespace tc;
  GRAB_REQUIRE(d_dataset && h_block_offsets && d_out_knn, "knn_tc: null pointer");
  GRAB_REQUIRE(dim >= 4 && dim % 4 == 0, "knn_tc: dim %u must be a multiple of 4", dim);
  GRAB_REQUIRE(n >= 1 && n < (1ull << 31) && num_blocks >= 1, "knn_tc: bad sizes");
  GRAB_REQUIRE(h_block_offsets[0] == 0 && h_block_offsets[num_blocks] == n, "knn_tc: block offsets must span [0,n]");
  GRAB_REQUIRE(mode == 0 || mode == 1, "knn_tc: mode must be 0 or 1");
  GRAB_REQUIRE(precision == 1 || precision == 2, "knn_tc: precision must be 1 (bf16) or 2 (split bf16)");
  const uint32_t want = k + k / 4 + 1;  // over-fetch: the exact re-rank picks the final k
  GRAB_REQUIRE(k >= 1 && want <= 256, "knn_tc: k %u too large for the tensor-core path (max 204)", k);
  const uint32_t kc = want <= 64 ? 64 : (want <= 128 ? 128 : 256);
  const int split = precision == 2;
  const uint32_t kused = (split ? 3 * dim : dim) + 3;  // + the three column-norm terms
  const uint32_t kp = (kused + BK - 1) / BK * BK;
  const uint32_t kblocks = kp / BK;
  const uint32_t last_kk = (kused - (kblocks - 1) * BK + 15) / 16;  // 16-wide MMA slices of the last K block in use
  const uint32_t num_row_tiles = static_cast<uint32_t>((n + BM - 1) / BM);
  int dev = 0, sms = 0;
  GRAB_CUDA_TRY(cudaGetDevice(&dev));
  GRAB_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const uint32_t max_ctas = static_cast<uint32_t>(sms) * CTAS_PER_SM;
  const uint32_t grid = num_row_tiles < max_ctas ? num_row_tiles : max_ctas;

  StageTimer tm(mode == 0 ? "knn_tc (own block)" : "knn_tc (other blocks)");
  ScopedDeviceBuffer offs, wins, a_op, b_op, mean, partial, scratch, keys, status;
  GRAB_CUDA_TRY(offs.alloc(sizeof(uint64_t) * (num_blocks + 1)));
  GRAB_CUDA_TRY(wins.alloc(sizeof(ScanWindow) * n));
  GRAB_CUDA_TRY(a_op.alloc(sizeof(__nv_bfloat16) * n * kp));
  GRAB_CUDA_TRY(b_op.alloc(sizeof(__nv_bfloat16) * n * kp));
  GRAB_CUDA_TRY(scratch.alloc(sizeof(uint64_t) * static_cast<uint64_t>(grid) * EPI_WGS * BM * cap_of(kc)));
  GRAB_CUDA_TRY(keys.alloc(sizeof(uint64_t) * n * kc * EPI_WGS));
  GRAB_CUDA_TRY(status.alloc(sizeof(int)));
  GRAB_CUDA_TRY(cudaMemsetAsync(status.ptr, 0, sizeof(int), st));
  GRAB_CUDA_TRY(cudaMemcpyAsync(offs.ptr, h_block_offsets, sizeof(uint64_t) * (num_blocks + 1), cudaMemcpyHostToDevice, st));
  knn_window_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(offs.as<uint64_t>(), num_blocks, n, mode, wins.as<ScanWindow>());
  GRAB_CUDA_TRY(cudaGetLastError());

  const float* d_mean = nullptr;
  if (metric == GRAB_METRIC_L2) {  // distances are translation invariant: centring shrinks |x|^2
    const uint32_t nchunks = static_cast<uint32_t>((n + kMeanChunk - 1) / kMeanChunk);
    GRAB_CUDA_TRY(mean.alloc(sizeof(float) * dim));
    GRAB_CUDA_TRY(partial.alloc(sizeof(float) * static_cast<uint64_t>(nchunks) * dim));
    mean_partial_kernel<<<nchunks, 128, 0, st>>>(d_dataset, n, dim, partial.as<float>());
    mean_final_kernel<<<(dim + 127) / 128, 128, 0, st>>>(partial.as<float>(), nchunks, dim, n, mean.as<float>());
    GRAB_CUDA_TRY(cudaGetLastError());
    d_mean = mean.as<float>();
  }
  __nv_bfloat16* pa = a_op.as<__nv_bfloat16>();
  __nv_bfloat16* pb = b_op.as<__nv_bfloat16>();
  prep_operands_kernel<<<(unsigned)((n * 32 + 255) / 256), 256, 0, st>>>(d_dataset, n, dim, d_mean, split, metric, kp, pa,
                                                                      pb);
  GRAB_CUDA_TRY(cudaGetLastError());

  tm.mark("alloc + operands");
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, pa, n, kp);
  if (rc != GRAB_OK) return rc;
  rc = make_map(&map_b, pb, n, kp);
  if (rc != GRAB_OK) return rc;

  const size_t smem = STAGES * STAGE_BYTES + sizeof(SharedCtl) + 1024;
  // the A operand of a row tile stays in shared memory when its K extent fits (GRAB_KNN_ARES=0 switches it off)
  const bool ares = kblocks <= static_cast<uint32_t>(kAresBlocks) && a_resident_enabled();
  // threshold seeding from every stride-th column (see above); skipped when the sweeps are short anyway
  const uint32_t stride = want <= 170 ? 16 : 32;
  uint64_t widest = 0;  // columns the widest row window sweeps
  for (uint32_t b = 0; b < num_blocks; ++b) {
    const uint64_t own = h_block_offsets[b + 1] - h_block_offsets[b];
    const uint64_t sweep = mode == 0 ? own : n - own;
    widest = sweep > widest ? sweep : widest;
  }
  const float* d_thr0 = nullptr;
  ScopedDeviceBuffer wins_s, keys_s, thr0;
  if (seed_thresholds_enabled() && widest >= static_cast<uint64_t>(stride) * kSeedKC * 8) {
    const uint64_t n_s = (n + stride - 1) / stride;
    GRAB_CUDA_TRY(wins_s.alloc(sizeof(ScanWindow) * n));
    GRAB_CUDA_TRY(keys_s.alloc(sizeof(uint64_t) * n * kSeedKC * EPI_WGS));
    GRAB_CUDA_TRY(thr0.alloc(sizeof(float) * n));
    sample_window_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(wins.as<ScanWindow>(), n, stride,
                                                                      wins_s.as<ScanWindow>());
    GRAB_CUDA_TRY(cudaGetLastError());
    CUtensorMap map_bs;
    rc = make_map(&map_bs, pb, n_s, kp, stride);
    if (rc != GRAB_OK) return rc;
    if (ares) {
      GRAB_CUDA_TRY(cudaFuncSetAttribute(knn_tc_kernel<kSeedKC, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      knn_tc_kernel<kSeedKC, true><<<grid, THREADS, smem, st>>>(map_a, map_bs, wins_s.as<ScanWindow>(), n, kblocks, last_kk,
                                                               num_row_tiles, scratch.as<uint64_t>(), keys_s.as<uint64_t>(),
                                                               nullptr, status.as<int>());
    } else {
      GRAB_CUDA_TRY(cudaFuncSetAttribute(knn_tc_kernel<kSeedKC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      knn_tc_kernel<kSeedKC, false><<<grid, THREADS, smem, st>>>(map_a, map_bs, wins_s.as<ScanWindow>(), n, kblocks, last_kk,
                                                                num_row_tiles, scratch.as<uint64_t>(), keys_s.as<uint64_t>(),
                                                                nullptr, status.as<int>());
    }
    GRAB_CUDA_TRY(cudaGetLastError());
    seed_threshold_kernel<<<(unsigned)((n * 32 + 255) / 256), 256, 0, st>>>(keys_s.as<uint64_t>(), n, thr0.as<float>());
    GRAB_CUDA_TRY(cudaGetLastError());
    d_thr0 = thr0.as<float>();
    tm.mark("threshold seeding (sampled columns)");
  }
#define GRAB_KNN_TC_LAUNCH(KC, AR)                                                                                        \
  do {                                                                                                                    \
    GRAB_CUDA_TRY(cudaFuncSetAttribute(knn_tc_kernel<KC, AR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
    knn_tc_kernel<KC, AR><<<grid, THREADS, smem, st>>>(map_a, map_b, wins.as<ScanWindow>(), n, kblocks, last_kk,          \
                                                      num_row_tiles, scratch.as<uint64_t>(), keys.as<uint64_t>(), d_thr0, \
                                                      status.as<int>());                                                  \
  } while (0)
  if (ares) {
    if (kc == 64) GRAB_KNN_TC_LAUNCH(64, true);
    else if (kc == 128) GRAB_KNN_TC_LAUNCH(128, true);
    else GRAB_KNN_TC_LAUNCH(256, true);
  } else {
    if (kc == 64) GRAB_KNN_TC_LAUNCH(64, false);
    else if (kc == 128) GRAB_KNN_TC_LAUNCH(128, false);
    else GRAB_KNN_TC_LAUNCH(256, false);
  }
#undef GRAB_KNN_TC_LAUNCH
  GRAB_CUDA_TRY(cudaGetLastError());
  tm.mark("tcgen05 all-pairs + top-k");
  const uint32_t kc_all = kc * EPI_WGS;  // candidates per row handed to the re-rank
  const size_t rsmem = sizeof(uint64_t) * kc_all + sizeof(float) * dim;
  if (metric == GRAB_METRIC_L2)
    rerank_kernel<GRAB_METRIC_L2><<<(unsigned)n, kRerankThreads, rsmem, st>>>(d_dataset, dim, keys.as<uint64_t>(), kc_all,
                                                                           k, d_out_knn, d_out_dists);
  else
    rerank_kernel<GRAB_METRIC_IP><<<(unsigned)n, kRerankThreads, rsmem, st>>>(d_dataset, dim, keys.as<uint64_t>(), kc_all,
                                                                           k, d_out_knn, d_out_dists);
  GRAB_CUDA_TRY(cudaGetLastError());
  tm.mark("exact re-rank");
  int h_status = 0;
  GRAB_CUDA_TRY(cudaMemcpyAsync(&h_status, status.ptr, sizeof(int), cudaMemcpyDeviceToHost, st));
  GRAB_CUDA_TRY(cudaStreamSynchronize(st));
  if (h_status != 0) {
    set_last_error("knn_tc: a bounded device-side wait expired (pipeline stalled)");
    return GRAB_ERR_TIMEOUT;
  }
  return GRAB_OK;
}

}  // namespace grab
