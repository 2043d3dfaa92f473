// Fused Hadamard rotation + int8 quantisation on the Blackwell tensor cores, for fp16 rows of length S * 128.
//
//   out[r, :] = sat_int8(roundf((H x[r, :]) * scale)),   H = H_S (x) H_128,   element index = c * 128 + j
//
// H_128 is the Sylvester matrix; H_S is one of the reference's 12 / 20 / 28 / 40 matrices or a Sylvester matrix of order
// 2 .. 64.  Viewing a row as the S x 128 matrix X[c, j], Y = H_S X H_128^T, i.e. two small GEMMs per row:
//
//   GEMM1   T^T[j', (r, c)] = sum_j (H_128[j', j] / 128) X_r[c, j]      M = 128 (j'), N = R * S, K = 128
//   GEMM2   Y_r^T[j', c']   = sum_c T_r^T[j', c] H_S[c', c]             M = 128 (j'), N = Spad,  K = Spad, per row r
//
// The x tile arrives by TMA exactly as it lies in memory: its rows (r, c) are the K-major B operand of GEMM1.  H_128 is the
// A operand (entries +-2^-7, so the intermediate never exceeds max |x| and fits fp16).  The fp32 result of GEMM1 sits in
// TMEM with j' along the lanes; four warps read it, split every value into an fp16 pair hi + lo (22 significant bits),
// and write the pairs back into TMEM as the A operand of GEMM2 (tcgen05.mma reads A from tensor memory), so the
// intermediate never goes through shared memory.  GEMM2 runs once with hi and once more, accumulating, with lo; its
// B operand is H_S, zero-padded to Spad = ceil16(S).  The same four warps then scale, round half away from zero,
// saturate and store the bytes: lane j' holds out[r, c' * 128 + j'], so a warp writes one full 32-byte sector per store.
//
// One persistent CTA per SM, 576 threads: warp 0 = TMA producer (three stages), warp 1 = MMA issuer and TMEM owner,
// warps 2..9 and 10..17 = two converter / epilogue groups (two warps per TMEM lane quarter, half of the rows each),
// each group with its own half of TMEM (D, hi, lo), working on
// alternating units of R rows.  Every mbarrier wait is bounded.
#include <algorithm>
#include "tc_common.cuh"
#include "hadamard_tables.inc"

namespace qb {
namespace {
using namespace tc;

constexpr int kThreadsH = 64 + 512;   // TMA warp, MMA warp, two converter / epilogue groups of eight warps
constexpr int kStages = 3;
constexpr int kOffH128 = 0;                    // 2 atoms: 128 rows x 128 B each (K 0..63, 64..127)
constexpr int kOffHS = 32768;                  // 1 atom: up to 64 rows x 128 B
constexpr int kOffX = 32768 + 8192;            // kStages x (2 atoms of N rows x 128 B)
constexpr int kStatusHad = 401;

struct HadBars {
  uint64_t x_full[kStages], x_empty[kStages];
  uint64_t d1_ready[2], a_ready[2], d2_ready[2], buf_free[2];
  uint32_t tmem_slot;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// S = special order (rows of H_S), SPAD = ceil16(S), R = rows of x per unit (R * S a multiple of 16, R * SPAD <= 128).
template <int S, int SPAD, int R>
__global__ void __launch_bounds__(kThreadsH, 1)
hadamard_tc_kernel(const __grid_constant__ CUtensorMap tm_x, int8_t* __restrict__ out, int64_t out_rs, int64_t rows,
                   float scale128, const unsigned long long* __restrict__ neg_masks, int* status, int early) {
  if (early) grid_dependency_launch();
  constexpr int N1 = R * S;                      // GEMM1 N
  constexpr int W = R * SPAD;                    // TMEM columns of the D region of one buffer
  constexpr int kColHi = W, kColLo = W + W / 2;  // packed fp16 pairs: SPAD / 2 columns per row
  constexpr int kStageBytes = 2 * N1 * 128;
  static_assert(N1 % 16 == 0 && N1 <= 256 && 2 * W <= 256, "unit shape");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  HadBars& bars = *reinterpret_cast<HadBars*>(smem + kOffX + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t units = (rows + R - 1) / R;
  const int64_t my_units = blockIdx.x < units ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  // ---- constant operands: H_128 / 128 (A of GEMM1) and H_S (B of GEMM2), both K-major with the 128-byte swizzle ----
  for (int i = threadIdx.x; i < 128 * 16; i += kThreadsH) {  // one 16-byte piece (8 elements along K) per item
    const int m = i >> 4, piece = i & 15;                    // piece: 8 pieces per atom row, 2 atoms
    const int atom = piece >> 3, ch = piece & 7;
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k0 = atom * 64 + ch * 8 + 2 * e;
      const uint32_t lo = (__popc(m & k0) & 1) ? 0xA000u : 0x2000u;        // -+ 2^-7 in fp16
      const uint32_t hi = (__popc(m & (k0 + 1)) & 1) ? 0xA000u : 0x2000u;
      w[e] = lo | (hi << 16);
    }
    *reinterpret_cast<uint4*>(smem + kOffH128 + atom * 16384 + m * 128 + ((ch ^ (m & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  for (int i = threadIdx.x; i < SPAD * 8; i += kThreadsH) {
    const int n = i >> 3, ch = i & 7;
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t v[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int k = ch * 8 + 2 * e + t;
        uint32_t bits = 0;  // zero padding
        if (n < S && k < S) {
          bool neg;
          if (neg_masks != nullptr) neg = (neg_masks[n] >> k) & 1ULL;   // the reference's special matrices
          else neg = (__popc(n & k) & 1) != 0;                          // Sylvester
          bits = neg ? 0xBC00u : 0x3C00u;                               // -+ 1.0
        }
        v[t] = bits;
      }
      w[e] = v[0] | (v[1] << 16);
    }
    *reinterpret_cast<uint4*>(smem + kOffHS + n * 128 + ((ch ^ (n & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&bars.x_full[s], 1); mbar_init(&bars.x_empty[s], 1); }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&bars.d1_ready[g], 1); mbar_init(&bars.a_ready[g], 1); mbar_init(&bars.d2_ready[g], 1); mbar_init(&bars.buf_free[g], 1);
    }
    fence_barrier_init();
    prefetch_tensormap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(&bars.tmem_slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars.tmem_slot;
  grid_dependency_wait();   // launched as a programmatic dependent: the set-up above overlaps the predecessor's tail

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int64_t i = 0; i < my_units; ++i) {
        const int stg = (int)(i % kStages);
        const uint32_t par = (uint32_t)(((i / kStages) & 1) ^ 1);
        if (!mbar_wait(&bars.x_empty[stg], par, status, kStatusHad)) break;
        const int64_t u = blockIdx.x + i * gridDim.x;
        uint8_t* dst = smem + kOffX + stg * kStageBytes;
        mbar_arrive_expect_tx(&bars.x_full[stg], kStageBytes);
        // rows of the byte view of x: (row r, chunk c) -> 256 bytes; coordinate x in bytes, y in (r, c) rows
        tma_load_2d(dst, &tm_x, &bars.x_full[stg], 0, (int)(u * N1));
        tma_load_2d(dst + N1 * 128, &tm_x, &bars.x_full[stg], 128, (int)(u * N1));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t id1 = make_idesc(1, 0, 0, 0, 0, 128, N1);
      constexpr uint32_t id2 = make_idesc(1, 0, 0, 0, 0, 128, SPAD);
      // descriptor words built once; per instruction only a 32-bit add remains (the issuing thread's instruction
      // count per MMA, not the tensor pipe, limits these small MMAs)
      const SmemDesc dH = make_smem_desc2(smem_u32(smem + kOffH128), 16, 1024, kSwizzle128B);
      const SmemDesc dHS = make_smem_desc2(smem_u32(smem + kOffHS), 16, 1024, kSwizzle128B);
      const SmemDesc dX0 = make_smem_desc2(smem_u32(smem + kOffX), 16, 1024, kSwizzle128B);
      auto second = [&](int64_t i) -> bool {   // GEMM2 of local unit i: per row, hi then lo
        const int g = (int)(i & 1);
        if (!mbar_wait(&bars.a_ready[g], (uint32_t)((i >> 1) & 1), status, kStatusHad)) return false;
        tc_fence_after_sync();
        const uint32_t base = tmem + g * 256;
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int part = 0; part < 2; ++part) {
#pragma unroll
            for (int ks = 0; ks < SPAD / 16; ++ks) {
              const uint32_t a_t = base + (part ? kColLo : kColHi) + r * (SPAD / 2) + ks * 8;
              umma_f16_ta(base + r * SPAD, a_t, desc_advance(dHS, ks * 32), id2, (part | ks) != 0 ? 1u : 0u);
            }
          }
        }
        umma_commit(&bars.d2_ready[g]);
        return true;
      };
      bool ok = true;
      for (int64_t i = 0; i < my_units && ok; ++i) {
        const int g = (int)(i & 1), stg = (int)(i % kStages);
        ok = mbar_wait(&bars.x_full[stg], (uint32_t)((i / kStages) & 1), status, kStatusHad) &&
             mbar_wait(&bars.buf_free[g], (uint32_t)(((i >> 1) & 1) ^ 1), status, kStatusHad);
        if (!ok) break;
        tc_fence_after_sync();
        const SmemDesc dX = desc_advance(dX0, (uint32_t)stg * kStageBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16(tmem + g * 256, desc_advance(dH, (ks >> 2) * 16384 + (ks & 3) * 32),
                   desc_advance(dX, (ks >> 2) * (N1 * 128) + (ks & 3) * 32), id1, ks != 0 ? 1u : 0u);
        umma_commit(&bars.d1_ready[g]);
        umma_commit(&bars.x_empty[stg]);
        if (i > 0) ok = second(i - 1);
      }
      if (ok && my_units > 0) second(my_units - 1);
    }
  } else {
    // ---------------- converter / epilogue groups ----------------
    const int g = (warp - 2) >> 3;                 // 0 or 1
    const int sub = ((warp - 2) >> 2) & 1;         // which half of the unit's R rows (two warps share a TMEM lane quarter)
    const int q = warp & 3;                        // TMEM lane quarter this warp may touch
    constexpr int RH = R / 2;
    static_assert(R % 2 == 0, "the rows of a unit are split between two warps");
    const int jrow = q * 32 + lane;                // j' : lane of TMEM = position inside a 128-chunk of the output row
    const uint32_t tl = (uint32_t)(q * 32) << 16;
    const bool lead = (warp - 2) % 8 == 0 && lane == 0;
    auto gsync = [&]() {
      if (g == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
    };
    auto gwait = [&](uint64_t* bar, uint32_t parity) -> bool {
      uint32_t ok = 1;
      if (lead) ok = mbar_wait(bar, parity, status, kStatusHad) ? 1u : 0u;
      uint32_t r;
      if (g == 0)
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(r) : "r"(ok) : "memory");
      else
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 2, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(r) : "r"(ok) : "memory");
      return r != 0;
    };
    const uint32_t base = tmem + g * 256 + tl;
    for (int64_t i = g; i < my_units; i += 2) {
      const uint32_t ph = (uint32_t)((i >> 1) & 1);
      const int64_t u = blockIdx.x + i * gridDim.x;
      // ---- GEMM1 result -> fp16 pair (hi, lo) -> A operand of GEMM2, in tensor memory ----
      if (!gwait(&bars.d1_ready[g], ph)) break;
      tc_fence_after_sync();
      {
        // all loads of the unit first, one wait: the accumulators of R rows are R * SPAD registers
        uint32_t v[RH][SPAD / 16][16];
#pragma unroll
        for (int rr = 0; rr < RH; ++rr)
#pragma unroll
          for (int c16 = 0; c16 < SPAD / 16; ++c16) tmem_ld16(base + (sub * RH + rr) * S + c16 * 16, v[rr][c16]);
        tmem_ld_wait();
#pragma unroll
        for (int rr = 0; rr < RH; ++rr) {
          const int r = sub * RH + rr;
#pragma unroll
          for (int c16 = 0; c16 < SPAD / 16; ++c16) {
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int c = c16 * 16 + 2 * e;
              const float f0 = c < S ? __uint_as_float(v[rr][c16][2 * e]) : 0.0f;     // columns past S belong to the next row
              const float f1 = c + 1 < S ? __uint_as_float(v[rr][c16][2 * e + 1]) : 0.0f;
              const __half2 h = __floats2half2_rn(f0, f1);
              const float2 hf = __half22float2(h);
              const __half2 l = __floats2half2_rn(f0 - hf.x, f1 - hf.y);
              hi[e] = *reinterpret_cast<const uint32_t*>(&h);
              lo[e] = *reinterpret_cast<const uint32_t*>(&l);
            }
            tmem_st8(base + kColHi + r * (SPAD / 2) + c16 * 8, hi);
            tmem_st8(base + kColLo + r * (SPAD / 2) + c16 * 8, lo);
          }
        }
      }
      tmem_st_wait();
      tc_fence_before_sync();
      gsync();
      if (lead) mbar_arrive(&bars.a_ready[g]);
      // ---- GEMM2 result -> int8 ----
      if (!gwait(&bars.d2_ready[g], ph)) break;
      tc_fence_after_sync();
      {
        uint32_t v[RH][SPAD / 16][16];
#pragma unroll
        for (int rr = 0; rr < RH; ++rr)
#pragma unroll
          for (int c16 = 0; c16 < SPAD / 16; ++c16) tmem_ld16(base + (sub * RH + rr) * SPAD + c16 * 16, v[rr][c16]);
        tmem_ld_wait();
        // the accumulators are in registers: hand the buffer back before the stores
        tc_fence_before_sync();
        gsync();
        if (lead) mbar_arrive(&bars.buf_free[g]);
#pragma unroll
        for (int rr = 0; rr < RH; ++rr) {
          const int64_t row = u * R + sub * RH + rr;
          int8_t* dst = out + row * out_rs + jrow;
          if (row < rows) {
#pragma unroll
            for (int c16 = 0; c16 < SPAD / 16; ++c16) {
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int c = c16 * 16 + e;
                if (c < S) {
                  const float y = __uint_as_float(v[rr][c16][e]) * scale128;
                  int qv;
                  asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(qv) : "f"(y + copysignf(0.5f, y)));
                  dst[c * 128] = (int8_t)qv;
                }
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

__device__ unsigned long long g_neg12[12], g_neg20[20], g_neg28[28], g_neg40[40];

template <int S, int SPAD, int R>
int launch_one(const qb_hadamard_quant_args* a, const unsigned long long* masks, cudaStream_t st) {
  constexpr int N1 = R * S;
  constexpr int kStageBytes = 2 * N1 * 128;
  constexpr int kSmem = kOffX + kStages * kStageBytes + (int)sizeof(HadBars) + 1024;
  CUtensorMap tm;
  // byte view of x: rows * S lines of 256 bytes
  int rc = encode_tmap_2d_u8(&tm, a->x, (uint64_t)a->rows * S, 256, 256, N1, 128);
  if (rc != QB_OK) return rc;
  auto kern = hadamard_tc_kernel<S, SPAD, R>;
  static PerDeviceOnce attr_done;
  if (attr_done.first()) QB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "hadamard: device status word unavailable");
  const int64_t units = ceil_div(a->rows, R);
  const unsigned grid = (unsigned)std::min<int64_t>(units, sm_count());
  launch_dependent(kern, dim3(grid), dim3(kThreadsH), (size_t)kSmem, st, tm, a->out, a->out_row_stride, a->rows, a->scale * 128.0f, masks, status,
                   early_overlap() ? 1 : 0);
  QB_LAUNCH_OK("hadamard_tc_kernel");
  return QB_OK;
}

int upload_masks() {
  static bool done[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return QB_OK;
  QB_CUDA_OK(cudaMemcpyToSymbol(g_neg12, kHadNeg12, sizeof(unsigned long long) * 12));
  QB_CUDA_OK(cudaMemcpyToSymbol(g_neg20, kHadNeg20, sizeof(unsigned long long) * 20));
  QB_CUDA_OK(cudaMemcpyToSymbol(g_neg28, kHadNeg28, sizeof(unsigned long long) * 28));
  QB_CUDA_OK(cudaMemcpyToSymbol(g_neg40, kHadNeg40, sizeof(unsigned long long) * 40));
  if (dev < 64) done[dev] = true;
  return QB_OK;
}

template <typename T> const unsigned long long* symbol_ptr(T& sym) {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, sym) == cudaSuccess ? static_cast<const unsigned long long*>(p) : nullptr;
}

}  // namespace

// Tensor-core path of qb_hadamard_quant; QB_ERR_UNSUPPORTED when the shape or layout is not eligible.
int hadamard_tc_launch(const qb_hadamard_quant_args* a, cudaStream_t st) {
  if (a->in_dtype != 0 || a->dim % 128 != 0) return QB_ERR_UNSUPPORTED;               // fp16 rows of S * 128 elements
  if (a->x_row_stride != a->dim || !aligned(a->x, 16)) return QB_ERR_UNSUPPORTED;     // contiguous rows (one 2-D byte view)
  if (a->rows * (int64_t)(a->dim / 128) >= (1LL << 31)) return QB_ERR_UNSUPPORTED;
  const int s = a->dim / 128;
  if (a->special > 1) {
    if (s != a->special) return QB_ERR_UNSUPPORTED;   // special * 2^k with 2^k != 128
    int rc = upload_masks();
    if (rc != QB_OK) return rc;
    switch (s) {
      case 12: return launch_one<12, 16, 8>(a, symbol_ptr(g_neg12), st);
      case 20: return launch_one<20, 32, 4>(a, symbol_ptr(g_neg20), st);
      case 28: return launch_one<28, 32, 4>(a, symbol_ptr(g_neg28), st);
      case 40: return launch_one<40, 48, 2>(a, symbol_ptr(g_neg40), st);
    }
    return QB_ERR_UNSUPPORTED;
  }
  switch (s) {   // Sylvester: H_(s * 128) = H_s (x) H_128
    case 2: return launch_one<2, 16, 8>(a, nullptr, st);
    case 4: return launch_one<4, 16, 8>(a, nullptr, st);
    case 8: return launch_one<8, 16, 8>(a, nullptr, st);
    case 16: return launch_one<16, 16, 8>(a, nullptr, st);
    case 32: return launch_one<32, 32, 4>(a, nullptr, st);
    case 64: return launch_one<64, 64, 2>(a, nullptr, st);
  }
  return QB_ERR_UNSUPPORTED;
}

}  // namespace qb
