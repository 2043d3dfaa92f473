// int8 x int8 -> int32 GEMM on the Blackwell tensor cores (tcgen05.mma kind::i8, TMEM accumulator),
// operands streamed by TMA into 128-byte-swizzled shared memory.
//
//   C[m, n] = sum_k A[m, k] * W[n, k]      A (M, K) and W (N, K) both K-contiguous int8.
//
// One CTA produces one 128 x 128 output tile.  Warp 0 issues the TMA loads (one elected lane),
// warp 1 owns the TMEM allocation and issues the MMAs (one elected lane), warps 2..5 run the
// epilogue: tcgen05.ld of the int32 accumulator, scaling, conversion and stores.  Shared memory
// holds kStages x (A tile 16 KB + W tile 16 KB); two CTAs fit on an SM so that one CTA's epilogue
// overlaps the other's main loop.  Out-of-range rows / columns / K tails are zero-filled by TMA
// and masked in the epilogue, so M, N and K need no padding (K and the row pitches only have to be
// multiples of 16 bytes, the TMA rule).  Every wait is bounded; on expiry the kernel records
// QB_ERR_TIMEOUT in the device status word, frees its TMEM and returns.
#include <algorithm>
#include <cstdlib>
#include "tc_common.cuh"
#include "linear_epilogue.cuh"

namespace qb {

namespace {

constexpr int BM = 128, BN = 128, BK = 128;  // BK bytes of K per stage = one swizzle atom row
constexpr int kStages = 3;
constexpr int kThreads = 192;
constexpr int kTileBytes = BM * BK;  // 16 KB (A) and BN * BK = 16 KB (W)
constexpr int kSmemBytes = kStages * 2 * kTileBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kTmemCols = 128;

using namespace tc;

// 32 consecutive accumulator columns of one output row -> scaled, converted, stored (16-byte stores when the layout allows).
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], int m, int nb, int M, int N, const Epilogue& ep) {
  if (nb >= N) return;  // whole warp agrees
  if (ep.transpose) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (m < M && nb + j < N) ep.store((int)r[j], m, nb + j);
  } else if (m < M) {
    const bool full = nb + 32 <= N;
    if (ep.out_kind == kOutF16 && full && (ep.out_stride % 8 == 0) &&
        ((reinterpret_cast<uintptr_t>(ep.out) & 15) == 0) && (nb % 8 == 0)) {
      __half* dst = static_cast<__half*>(ep.out) + (int64_t)m * ep.out_stride + nb;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        __align__(16) __half2 h[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
          h[t] = __floats2half2_rn(ep.scaled((int)r[j + 2 * t], m, nb + j + 2 * t),
                                   ep.scaled((int)r[j + 2 * t + 1], m, nb + j + 2 * t + 1));
        *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(h);
      }
    } else if ((ep.out_kind == kOutS8Rne || ep.out_kind == kOutS8Away) && full && (ep.out_stride % 16 == 0) &&
               ((reinterpret_cast<uintptr_t>(ep.out) & 15) == 0) && (nb % 16 == 0)) {
      int8_t* dst = static_cast<int8_t*>(ep.out) + (int64_t)m * ep.out_stride + nb;
#pragma unroll
      for (int j = 0; j < 32; j += 16) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int b = j + 4 * t;
          w[t] = pack4_s8(ep.to_s8(ep.scaled((int)r[b], m, nb + b)), ep.to_s8(ep.scaled((int)r[b + 1], m, nb + b + 1)),
                          ep.to_s8(ep.scaled((int)r[b + 2], m, nb + b + 2)),
                          ep.to_s8(ep.scaled((int)r[b + 3], m, nb + b + 3)));
        }
        *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < N) ep.store((int)r[j], m, nb + j);
    }
  }
}

// kBN: tile width.  128 for general shapes; 64 for a single row of tiles (M <= 128, weight streaming), where narrower
// tiles put a CTA on every SM -- 83 CTAs of 128 columns cannot pull the weights of the 2.7B in_proj at HBM speed.
// a_rows: rows of A that exist (the TMA box of A; the MMA still multiplies 128 rows, the rest of the tile is whatever
// shared memory held, and those output rows are masked in the epilogue).
// kARows: rows of A a stage has room for (a multiple of 8; the MMA's 128-row read then runs on into the stages behind it, whose
// contents only reach masked output rows), kSt: stages.  Few rows of A leave room for a deeper ring: a decode batch of 16
// streams its weights through eight 12 KB stages instead of three 24 KB ones.
template <int kBN, int kARows = BM, int kSt = kStages>
__global__ void __launch_bounds__(kThreads)
gemm_s8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                       int M, int N, int K, int a_rows, Epilogue ep, int* status, int early) {
  if (early) grid_dependency_launch();
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  constexpr int kWBytes = kBN * BK;
  constexpr int kABytes = kARows * BK;
  static_assert(kARows % 8 == 0 && (BM - kARows) * BK <= kSt * kWBytes, "the 128-row read of the last stage must stay inside the ring");
  uint8_t* sW = smem + kSt * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSt * (kABytes + kWBytes));
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kSt;
  uint64_t* accum_bar = bars + 2 * kSt;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kSt + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * kBN;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSt; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(accum_bar, 1);
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // launched as a programmatic dependent: barriers, tensor memory and descriptors above were set up while the kernel
  // before this one may still have been running; A (and per-row scales) are read from here on, by TMA or past L1
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kSt;
        const uint32_t ph = (kb / kSt) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, status, QB_ERR_TIMEOUT)) break;
        mbar_arrive_expect_tx(&full_bar[s], (uint32_t)(a_rows * BK + kWBytes));
        tma_load_2d(sA + s * kABytes, &tmap_a, &full_bar[s], kb * BK, m0);
        tma_load_2d(sW + s * kWBytes, &tmap_w, &full_bar[s], kb * BK, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*c=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, 0, 0, BM, kBN);
      // descriptor words of stage 0; a stage / K step is one 32-bit add away (the issuer's instruction count per MMA
      // decides whether the tensor pipe stays fed)
      const SmemDesc da0 = make_smem_desc2(smem_u32(sA), 16, 1024, kSwizzle128B);
      const SmemDesc dw0 = make_smem_desc2(smem_u32(sW), 16, 1024, kSwizzle128B);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kSt;
        const uint32_t ph = (kb / kSt) & 1;
        ok = mbar_wait(&full_bar[s], ph, status, QB_ERR_TIMEOUT);
        if (!ok) break;
        tc_fence_after_sync();
        const SmemDesc da = desc_advance(da0, (uint32_t)s * kABytes);
        const SmemDesc dw = desc_advance(dw0, (uint32_t)s * kWBytes);
#pragma unroll
        for (int k = 0; k < BK / 32; ++k)
          umma_i8(tmem_base, desc_advance(da, k * 32), desc_advance(dw, k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
      }
      umma_commit(accum_bar);  // accumulator complete (arrives even after an aborted loop)
    }
  } else {
    // Epilogue warps 2..5: warp w may touch TMEM lanes [32 * (w % 4), 32 * (w % 4) + 32).
    const int q = warp & 3;
    const bool ok = mbar_wait(accum_bar, 0, status, QB_ERR_TIMEOUT);
    tc_fence_after_sync();
    if (ok) {
      const int m = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < kBN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, r);
        tmem_ld_wait();
        store_chunk(r, m, n0 + c, M, N, ep);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- persistent variant for large problems -------------------------------------------------------------------------------
// 128 x 256 tiles (one W tile byte feeds twice the MACs of the 128 x 128 kernel, which keeps the MMAs fed from shared
// memory at tensor speed), four 48 KB stages, one CTA per SM walking tiles round-robin, and two 256-column accumulators in
// TMEM so that the epilogue of a tile (warps 2..5) overlaps the main loop of the next one.  Tiles are ordered M-fastest:
// CTAs that run at the same time read the same W tile, which then comes from L2.
constexpr int PBN = 256;
constexpr int kPStages = 4;
constexpr int kPStageBytes = BM * BK + PBN * BK;   // 16 KB of A + 32 KB of W
constexpr int kPSmemBytes = kPStages * kPStageBytes + 1024 + 256;
// Eight epilogue warps (two per TMEM lane quarter, 128 columns each): with four, converting and storing a 128 x 256
// tile took about as long as the main loop of a K = 2560 tile and the MMA issuer waited for its accumulator.
constexpr int kPThreads = 64 + 256;

// bn: tile width actually used (a multiple of 16, <= 256; the TMA box of W has bn rows).  The host picks the width whose
// tile count fills whole rounds of the grid best: at 2048 rows the 2.7B out_proj (N = 2560) is 160 tiles of 256 columns on
// 148 SMs, two rounds with the second almost empty, or 224 tiles of 192 columns, two rounds of cheaper tiles.  Shared-memory
// slots and the TMEM accumulators keep their 256-column size.
__global__ void __launch_bounds__(kPThreads, 1)
gemm_s8_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                                  int M, int N, int K, int bn, Epilogue ep, int* status, int early) {
  if (early) grid_dependency_launch();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPStages * kPStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kPStages;
  uint64_t* acc_full = bars + 2 * kPStages;       // [2]
  uint64_t* acc_empty = bars + 2 * kPStages + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
  const int tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 1); }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // launched as a programmatic dependent: barriers, tensor memory and descriptors above were set up while the kernel
  // before this one may still have been running; A (and per-row scales) are read from here on, by TMA or past L1
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // k-iterations issued so far, over all tiles: the stage ring runs through tile boundaries
      for (int i = 0; i < my_tiles; ++i) {
        const int t = blockIdx.x + i * gridDim.x;
        const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * bn;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kPStages;
          ok = mbar_wait(&empty_bar[s], (uint32_t)(((it / kPStages) & 1) ^ 1), status, QB_ERR_TIMEOUT);
          if (!ok) break;
          uint8_t* stage = smem + s * kPStageBytes;
          mbar_arrive_expect_tx(&full_bar[s], (uint32_t)((BM + bn) * BK));
          tma_load_2d(stage, &tmap_a, &full_bar[s], kb * BK, m0);
          tma_load_2d(stage + BM * BK, &tmap_w, &full_bar[s], kb * BK, n0);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(/*c=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, 0, 0, BM, (uint32_t)bn);
      const SmemDesc da0 = make_smem_desc2(smem_u32(smem), 16, 1024, kSwizzle128B);
      int it = 0;
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int b = i & 1;
        ok = mbar_wait(&acc_empty[b], (uint32_t)(((i >> 1) & 1) ^ 1), status, QB_ERR_TIMEOUT);  // epilogue has drained it
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)(b * PBN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kPStages;
          ok = mbar_wait(&full_bar[s], (uint32_t)((it / kPStages) & 1), status, QB_ERR_TIMEOUT);
          if (!ok) break;
          tc_fence_after_sync();
          const SmemDesc da = desc_advance(da0, (uint32_t)s * kPStageBytes);
          const SmemDesc dw = desc_advance(da, BM * BK);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_i8(acc, desc_advance(da, k * 32), desc_advance(dw, k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        umma_commit(&acc_full[b]);
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;   // which half of the tile's 32-column chunks
    const bool lead = warp == 2 && lane == 0;
    const int nchunks = (bn + 31) / 32;
    const int c_begin = half == 0 ? 0 : ((nchunks + 1) / 2) * 32;
    const int c_end = half == 0 ? ((nchunks + 1) / 2) * 32 : nchunks * 32;
    for (int i = 0; i < my_tiles; ++i) {
      const int b = i & 1;
      const int t = blockIdx.x + i * gridDim.x;
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * bn;
      const int n_end = min(N, n0 + bn);      // columns past the tile belong to the next one (or to nobody)
      // one thread polls, the eight warps meet at a named barrier that also carries the outcome
      uint32_t ok = 1;
      if (lead) ok = mbar_wait(&acc_full[b], (uint32_t)((i >> 1) & 1), status, QB_ERR_TIMEOUT) ? 1u : 0u;
      uint32_t all_ok;
      asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                   : "=r"(all_ok) : "r"(ok) : "memory");
      if (!all_ok) break;
      tc_fence_after_sync();
      const int m = m0 + q * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * PBN);
      bool released = false;
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 64) {
        uint32_t r0[32], r1[32];
        const bool two = c + 32 < c_end;
        tmem_ld_32x32(acc + (uint32_t)c, r0);
        if (two) tmem_ld_32x32(acc + (uint32_t)c + 32, r1);
        tmem_ld_wait();
        if (c + 64 >= c_end) {  // the last columns are in registers: hand the accumulator back before storing them
          tc_fence_before_sync();
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (lead) mbar_arrive(&acc_empty[b]);
          released = true;
        }
        store_chunk(r0, m, n0 + c, M, n_end, ep);
        if (two) store_chunk(r1, m, n0 + c + 32, M, n_end, ep);
      }
      if (!released) {          // a half without chunks (tile narrower than 64 columns) still takes part in the hand-over
        tc_fence_before_sync();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (lead) mbar_arrive(&acc_empty[b]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- issue-rate measurement of tcgen05.mma kind::i8 -------------------------------------------------------------------
// One CTA per SM; operands (pseudo-random int8, the 128-byte-swizzled tile shapes of the GEMM above) sit in shared memory
// and are never reloaded; one thread issues `groups` x four M128 N256 K32 MMAs into two alternating accumulators and
// commits each group of four to a ring of mbarriers it waits on two groups behind, the way the GEMM's stage ring paces it.
// What comes out is the tensor pipe's dense int8 rate with shared-memory operands and no epilogue: the denominator of the
// GEMM rooflines.
constexpr int kPeakRing = 4;
__global__ void __launch_bounds__(128, 1) i8_mma_peak_kernel(int groups, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPStageBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kPeakRing);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kPStageBytes / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = (uint32_t)(i * 2654435761u) ^ (blockIdx.x * 40503u);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPeakRing; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes of the operands -> async proxy (MMA)
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = make_idesc(2, 1, 1, 0, 0, BM, PBN);
    const SmemDesc da = make_smem_desc2(smem_u32(smem), 16, 1024, kSwizzle128B);
    const SmemDesc dw = desc_advance(da, BM * BK);
    bool ok = true;
    for (int g = 0; g < groups && ok; ++g) {
      if (g >= kPeakRing) ok = mbar_wait_spin(&bars[g % kPeakRing], (uint32_t)(((g / kPeakRing) - 1) & 1), status, QB_ERR_TIMEOUT);
      if (!ok) break;
      const uint32_t acc = tmem_base + (uint32_t)((g & 1) * PBN);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_i8(acc, desc_advance(da, k * 32), desc_advance(dw, k * 32), idesc, g >= 2 ? 1u : (k ? 1u : 0u));
      umma_commit(&bars[g % kPeakRing]);
    }
    // drain: the last kPeakRing groups
    for (int g = max(0, groups - kPeakRing); g < groups && ok; ++g)
      ok = mbar_wait_spin(&bars[g % kPeakRing], (uint32_t)((g / kPeakRing) & 1), status, QB_ERR_TIMEOUT);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (fn != nullptr) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

}  // namespace

int encode_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encoder();
  QB_REQUIRE(enc != nullptr, QB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  QB_REQUIRE(r == CUDA_SUCCESS, QB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QB_OK;
}

int encode_tmap_4d(CUtensorMap* out, bool f16, bool swizzle128, const void* base, const uint64_t dims[4],
                   const uint64_t strides_bytes[3], const uint32_t box[4]) {
  EncodeTiledFn enc = get_encoder();
  QB_REQUIRE(enc != nullptr, QB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  const cuuint64_t gstride[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  const cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(out, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base),
                         gdim, gstride, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  QB_REQUIRE(r == CUDA_SUCCESS, QB_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with code %d", (int)r);
  return QB_OK;
}

int encode_tmap_f16_4d(CUtensorMap* out, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                       const uint32_t box[4]) {
  return encode_tmap_4d(out, true, true, base, dims, strides_bytes, box);
}

int launch_tensor_core_gemm(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int M, int N, int K,
                            const Epilogue& ep, cudaStream_t st) {
  // TMA rules: 16-byte aligned bases and pitches; the inner extent must cover whole 16-byte units.
  if (K % 16 != 0 || lda % 16 != 0 || ldw % 16 != 0 || !aligned(A, 16) || !aligned(W, 16)) return QB_ERR_UNSUPPORTED;
  if (M < 9) return QB_ERR_UNSUPPORTED;   // a few rows are weight-streaming work for the dp4a kernel
  CUtensorMap ta, tw;
  int rc = encode_tmap_2d_u8(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  if (rc != QB_OK) return rc;
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "device status word unavailable");
  static bool attr_set[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  const bool no_persistent = path_override(QB_PATH_GEMM_SMALL_TILES);
  const int64_t ptiles = ceil_div(M, BM) * ceil_div(N, PBN);
  if (!no_persistent && ptiles >= sm_count()) {   // enough 128 x 256 tiles to give every SM at least one
    // tile width: the one whose rounds of the grid cost least (rounds x width); ties go to the wider tile.  Only multiples
    // of 64 columns: 144 .. 240 in steps of 16 were measured too, and every width that is not a multiple of 64 ran 25-90 %
    // slower per column than its neighbours.  128- and 64-column tiles were measured at the 2.7B layer shapes as well (2048
    // and 8192 rows) and lost everywhere (10-20 % and 60-110 % slower): every column of W a tile does not cover is another
    // pass of the A tile through shared memory.
    int bn = PBN;
    int64_t best = INT64_MAX;
    for (int cand = PBN; cand >= 192; cand -= 64) {
      const int64_t t = ceil_div(M, BM) * ceil_div(N, cand);
      const int64_t cost = ceil_div(t, sm_count()) * cand;
      if (cost < best) { best = cost; bn = cand; }
    }
    rc = encode_tmap_2d_u8(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, BK);
    if (rc != QB_OK) return rc;
    static bool pattr_set[64] = {};
    if (dev >= 64 || !pattr_set[dev]) {
      QB_CUDA_OK(cudaFuncSetAttribute(gemm_s8_tcgen05_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmemBytes));
      if (dev < 64) pattr_set[dev] = true;
    }
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(M, BM) * ceil_div(N, bn), sm_count());
    launch_dependent(gemm_s8_tcgen05_persistent_kernel, dim3(grid), dim3(kPThreads), (size_t)kPSmemBytes, st, ta, tw, M, N, K, bn, ep, status,
                     early_overlap() ? 1 : 0);
    QB_LAUNCH_OK("gemm_s8_tcgen05_persistent_kernel");
    return QB_OK;
  }
  // a single row of tiles with too few 128-column tiles to occupy the GPU: 64-column tiles, and only the rows of A that exist
  const bool narrow = M <= BM && ceil_div(N, BN) < sm_count();
  const int bn = narrow ? 64 : BN;   // (32-column tiles were slower: every CTA re-reads the A tile)
  const int a_rows = narrow ? (int)std::min<int64_t>(BM, ceil_div(M, 8) * 8) : BM;
  if (narrow) {
    rc = encode_tmap_2d_u8(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, a_rows, BK);
    if (rc != QB_OK) return rc;
  }
  rc = encode_tmap_2d_u8(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, bn, BK);
  if (rc != QB_OK) return rc;
  constexpr int kSmem32 = 8 * (32 * BK + 64 * BK) + 1024 + 256;     // <64, 32 rows, 8 stages>
  constexpr int kSmem64 = 6 * (64 * BK + 64 * BK) + 1024 + 256;     // <64, 64 rows, 6 stages>
  if (dev >= 64 || !attr_set[dev]) {
    QB_CUDA_OK(cudaFuncSetAttribute(gemm_s8_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    QB_CUDA_OK(cudaFuncSetAttribute(gemm_s8_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    QB_CUDA_OK(cudaFuncSetAttribute(gemm_s8_tcgen05_kernel<64, 32, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem32));
    QB_CUDA_OK(cudaFuncSetAttribute(gemm_s8_tcgen05_kernel<64, 64, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem64));
    if (dev < 64) attr_set[dev] = true;
  }
  dim3 grid((unsigned)ceil_div(M, BM), (unsigned)ceil_div(N, bn));
  const int early = early_overlap() ? 1 : 0;
  if (bn == 64 && a_rows <= 32)
    launch_dependent(gemm_s8_tcgen05_kernel<64, 32, 8>, grid, dim3(kThreads), (size_t)kSmem32, st, ta, tw, M, N, K, a_rows, ep, status, early);
  else if (bn == 64 && a_rows <= 64)
    launch_dependent(gemm_s8_tcgen05_kernel<64, 64, 6>, grid, dim3(kThreads), (size_t)kSmem64, st, ta, tw, M, N, K, a_rows, ep, status, early);
  else if (bn == 64) launch_dependent(gemm_s8_tcgen05_kernel<64>, grid, dim3(kThreads), (size_t)kSmemBytes, st, ta, tw, M, N, K, a_rows, ep, status, early);
  else launch_dependent(gemm_s8_tcgen05_kernel<128>, grid, dim3(kThreads), (size_t)kSmemBytes, st, ta, tw, M, N, K, a_rows, ep, status, early);
  QB_LAUNCH_OK("gemm_s8_tcgen05_kernel");
  return QB_OK;
}

}  // namespace qb

// Measures the dense int8 tensor rate of the current device (see i8_mma_peak_kernel): runs `repeats` launches of `groups`
// MMA groups per SM on `stream`, times them with CUDA events and returns TOP/s in *tops.  Blocks the host.
extern "C" int qb_i8_mma_peak(int groups, int repeats, void* stream, double* tops, double* ms) {
  using namespace qb;
  QB_REQUIRE(groups > 0 && repeats > 0 && tops != nullptr, QB_ERR_INVALID_ARG, "i8_mma_peak: bad arguments");
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "device status word unavailable");
  static PerDeviceOnce attr;
  constexpr int smem = kPStageBytes + 1024 + 256;
  if (attr.first()) QB_CUDA_OK(cudaFuncSetAttribute(i8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaStream_t st = (cudaStream_t)stream;
  cudaEvent_t e0, e1;
  QB_CUDA_OK(cudaEventCreate(&e0));
  QB_CUDA_OK(cudaEventCreate(&e1));
  const int sms = sm_count();
  i8_mma_peak_kernel<<<sms, 128, smem, st>>>(groups, status);   // warm-up
  QB_CUDA_OK(cudaEventRecord(e0, st));
  for (int r = 0; r < repeats; ++r) i8_mma_peak_kernel<<<sms, 128, smem, st>>>(groups, status);
  QB_CUDA_OK(cudaEventRecord(e1, st));
  QB_CUDA_OK(cudaEventSynchronize(e1));
  QB_LAUNCH_OK("i8_mma_peak_kernel");
  float t = 0.f;
  QB_CUDA_OK(cudaEventElapsedTime(&t, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  const double ops = 2.0 * BM * PBN * 32 * 4.0 * groups * (double)sms * repeats;
  *tops = ops / (t * 1e-3) / 1e12;
  if (ms != nullptr) *ms = t;
  return QB_OK;
}
