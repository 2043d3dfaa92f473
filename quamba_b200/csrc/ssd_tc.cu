// Mamba2 SSD chunk scan on the Blackwell tensor cores (headdim 64, d_state 128).
//
// One CTA owns one (batch, head) pair and walks the sequence in blocks of T = 128 tokens, carrying
// the 64 x 128 SSM state in registers (fp32), so nothing but inputs and outputs ever touches HBM:
//
//   CB    = C . B^T                         128 x 128 x 128   tcgen05 f16 (integer-valued operands: exact)
//   D1    = C . s                           128 x  64 x 128   state entering the block, fp16 copy
//   S_loc = B^T . (x * w)                   128 x  64 x 128   w_l = dt_l 2^(r - a_l)
//   D2    = Lm . x                          128 x  64 x 128   Lm[m,k] = CB[m,k] 2^(a_m - a_k) dt_k, k <= m
//   y[m,p]   = sC 2^(a_m) D1 + sx[p] (D2 + D x)            s <- 2^r s + sB sx[p] S_loc
//
// a_l is the running sum of dt*A*log2(e) inside the block and r its last value, so every exponent
// is <= 0.  Two small preparation kernels run first: one widens B and C (shared by all heads of a
// group) to fp16 once -- values stay the raw integers, scales are applied in the epilogues -- the
// other evaluates softplus / the running sums and leaves, per (batch, head, block), the vectors
// a[128], bk[128] = a - log2(dt) - log2(sC sB) and ec[128] (column factors of the off-diagonal
// 32 x 32 chunks of Lm: there 2^(a_m - bk_k) = 2^(a_m - a_end(chunk)) * ec[k], two multiplies
// instead of an ex2 per element; the diagonal chunks keep the exact per-element exponent).  When D
// has one value per head it is added on the diagonal of Lm, so the output step needs no x.
// Every CTA TMA-loads 128-byte-swizzled B / C tiles that serve as K-major operands (CB, D1) and as
// the MN-major A operand of S_loc without any reshuffling, plus the 1.5 KB of vectors.  x is read
// straight from global memory by the thread that converts it (int8 -> fp16 with integer / half
// ALU ops only).
//
// 640 threads: warp 0 issues TMA, warp 1 issues the MMAs and owns TMEM; warps 4..11 (group A) turn
// CB(j) into the Lm tile; warps 12..19 (group B) write the x operands of block k, then the output
// of block k - 1 (accumulators -> registers -> 4 x 4 shuffle transpose -> 64-byte row pieces straight
// to global memory), then fold S_loc(k) into the state they keep in registers.  TMEM (512 columns):
// CB and D1 double-buffered, D2, S.  Every barrier is waited on by each of its consumers once per
// phase and in order, no phase can complete twice before a consumer has looked at it, and all waits
// are bounded.  Two lessons are built into the code: setmaxnreg.inc blocks without a time limit when
// the pool is short (the 40 / 64 / 152 split leaves room for the allocation granularity), and the
// B / C stage is handed back to the TMA producer only at the end of an iteration (see below).
#include "tc_common.cuh"

namespace qb {

#ifdef QB_TRACE
__device__ long long g_trace[2][64][16];
#define TRACE(role, j, slot) do { if (blockIdx.x == 0 && (j) < 64) g_trace[role][j][slot] = clock64(); } while (0)
#else
#define TRACE(role, j, slot) do { } while (0)
#endif

#ifdef QB_DUMP
__device__ float* g_dump = nullptr;
#endif

namespace {
using namespace tc;

constexpr int T = 128, P = 64, N = 128;
// Warpgroup 0 (warps 0..3): warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..3 idle.
// Warpgroups 1..2 (warps 4..11) = compute group A, warpgroups 3..4 (warps 12..19) = compute group B.
// Registers are rebalanced between the warpgroups with setmaxnreg (the kernel launches at 96 per thread).
constexpr int kThreads = 640;
constexpr int kLead = 128;                     // first compute thread
constexpr int kRegsCtl = 40, kRegsA = 64, kRegsB = 152;

constexpr int kAtom = T * 128;                 // 16 KB: 128 rows x 128 bytes
constexpr int kOffB16 = 0;                     // 2 stages x 2 atoms
constexpr int kOffC16 = 4 * kAtom;             // 2 stages x 2 atoms
constexpr int kOffLm = 8 * kAtom;              // 2 atoms, unused since Lm lives in tensor memory (kept: tile offsets unchanged)
constexpr int kOffXraw = 10 * kAtom;           // 1 atom
constexpr int kOffXw = 11 * kAtom;             // 1 atom
constexpr int kOffS16 = 12 * kAtom;            // 1 atom
constexpr int kOffMisc = 13 * kAtom;           // vectors + barriers
constexpr int kMiscBytes = 4096;
constexpr int kSmemBytes = kOffMisc + kMiscBytes + 1024;
constexpr int kAbVecs = 3;                     // a[128], bk[128], ec[128] per block, fp32
constexpr int kAbBytes = kAbVecs * T * 4;

// CB is double-buffered (block j in buffer j & 1) so that C.B^T of the next block is computed while the Lm tile of the
// current one is still being built from the other buffer.
// D1 (the carried-in term C S_prev) is double-buffered as well: GEMM2(j) only needs the state of block j - 1, so it is
// issued while the x operands of block j are still being prepared and the tensor pipe would otherwise idle.
constexpr uint32_t kColCB = 0, kColD1 = 128, kColD2 = 192, kColS = 256, kColCB1 = 320, kColD1b = 448, kTmemCols = 512;

struct Misc {
  // per stage: a (inclusive running sum of dt*A*log2e), bk (+inf where dt == 0), ec (column factor of the off-diagonal
  // 32 x 32 chunks of Lm, see ssd_dt_kernel).  Both compute groups release a
  // stage right after their last read of it (group B copies what it needs into registers at the top of a block).
  float ab[2][kAbVecs * T];
  float sx[P];         // x scale per channel
  float dsx[P];        // D * sx per channel
  float sbx[P];        // sB * sx per channel
  float dfold;         // D of this head when it is one value per head (added on the diagonal of Lm), else 0
  uint64_t bc_full[2], bc_empty[2], ab_empty[2];
  uint64_t cb_ready[2], s_ready, y_ready, d1_ready, xops_ready, lm_ready, s16_ready, y_free;  // cb_ready / s_ready: one per TMEM buffer
  uint32_t tmem_slot;
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc does not fit");

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
template <int R> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R)); }
template <int R> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R)); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Four int8 in one word -> two half2 holding the same integers, without any conversion instruction:
// bias each byte to unsigned, splice it under the exponent byte 0x64 (1024 + b) and subtract 1152.
__device__ __forceinline__ void s8x4_to_h2x2(uint32_t word, __half2& lo, __half2& hi) {
  const uint32_t t = word ^ 0x80808080u;
  const uint32_t u0 = __byte_perm(t, 0x64646464u, 0x5140);
  const uint32_t u1 = __byte_perm(t, 0x64646464u, 0x7362);
  const __half2 k = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
  lo = __hsub2(*reinterpret_cast<const __half2*>(&u0), k);
  hi = __hsub2(*reinterpret_cast<const __half2*>(&u1), k);
}
// A load the compiler may not move: the x rows of the NEXT block are requested at the top of the current
// block so that their latency is covered by a whole block of work.
__device__ __forceinline__ uint4 ldg_nc_now(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<const uint32_t*>(&v); }

// 4 x 4 transpose of 16-byte pieces across the four lanes of a quad (lanes 4q .. 4q + 3): on entry lane i holds the
// pieces c[0..3] of "its" row; on exit lane i holds piece i of the rows of lanes 4q + 0 .. 4q + 3, in c[0..3].
__device__ __forceinline__ uint4 shfl_xor_u4(uint4 v, int m) {
  v.x = __shfl_xor_sync(0xffffffffu, v.x, m); v.y = __shfl_xor_sync(0xffffffffu, v.y, m);
  v.z = __shfl_xor_sync(0xffffffffu, v.z, m); v.w = __shfl_xor_sync(0xffffffffu, v.w, m);
  return v;
}
__device__ __forceinline__ void quad_transpose(uint4 (&c)[4], int lane) {
  const bool odd = (lane & 1) != 0, hi = (lane & 2) != 0;
  {
    const uint4 r0 = shfl_xor_u4(odd ? c[0] : c[1], 1);
    const uint4 r1 = shfl_xor_u4(odd ? c[2] : c[3], 1);
    if (odd) { c[0] = r0; c[2] = r1; } else { c[1] = r0; c[3] = r1; }
  }
  {
    const uint4 r0 = shfl_xor_u4(hi ? c[0] : c[2], 2);
    const uint4 r1 = shfl_xor_u4(hi ? c[1] : c[3], 2);
    if (hi) { c[0] = r0; c[1] = r1; } else { c[2] = r0; c[3] = r1; }
  }
}

// One K = 128 contraction as eight K = 16 instructions.  The descriptors come in as two 32-bit words each and a K step
// is one add on the low word: the issuing thread must spend only a handful of instructions per MMA, or the tensor pipe
// waits for it (48 to 64 cycles of tensor work per instruction here).
//   K-major operand (two 64-element atoms along K):   address = base + (ks / 4) * 16 KB + (ks % 4) * 32
//   MN-major operand (rows are K):                    address = base + ks * 16 rows * 128 B
template <bool kAMn, bool kBMn>
__device__ __forceinline__ void issue_gemm(uint32_t d_tmem, SmemDesc a, SmemDesc b, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t ao = kAMn ? ks * 2048 : (ks >> 2) * kAtom + (ks & 3) * 32;
    const uint32_t bo = kBMn ? ks * 2048 : (ks >> 2) * kAtom + (ks & 3) * 32;
    umma_f16(d_tmem, desc_advance(a, ao), desc_advance(b, bo), idesc, ks != 0 ? 1u : 0u);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
ssd_tc_kernel(const __grid_constant__ CUtensorMap tm_b16, const __grid_constant__ CUtensorMap tm_c16, qb_ssd_args a,
              const float* __restrict__ ab_ws, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Misc& ms = *reinterpret_cast<Misc*>(smem + kOffMisc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / a.nheads, h = blockIdx.x % a.nheads;
  const int hpg = a.nheads / a.ngroups;
  const int g = h / hpg;
  const int nb = (a.seqlen + T - 1) / T;
  const float sB = a.grouped ? a.B_scale[g] : a.B_scale[0];
  const float sC = a.grouped ? a.C_scale[g] : a.C_scale[0];

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&ms.bc_full[s], 1); mbar_init(&ms.bc_empty[s], 1); mbar_init(&ms.ab_empty[s], 2); }
    mbar_init(&ms.cb_ready[0], 1); mbar_init(&ms.cb_ready[1], 1); mbar_init(&ms.s_ready, 1); mbar_init(&ms.y_ready, 1); mbar_init(&ms.d1_ready, 1);
    mbar_init(&ms.xops_ready, 1); mbar_init(&ms.lm_ready, 1); mbar_init(&ms.s16_ready, 1); mbar_init(&ms.y_free, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_b16);
    prefetch_tensormap(&tm_c16);
  }
  if (warp == 1) {
    tmem_alloc(&ms.tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (threadIdx.x >= kLead && threadIdx.x < kLead + P) {
    const int p = threadIdx.x - kLead;
    float sx;
    if (!a.grouped) {
      sx = a.x_scales[0];
    } else {
      const int hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, h % hpg);
      const int dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, p);
      sx = a.x_scales[(g * a.nhead_groups + hg) * a.ndim_groups + dg];
    }
    float dv = 0.0f;
    if (a.D != nullptr) dv = (*a.D_scale) * (float)(a.D_has_hdim ? a.D[h * P + p] : a.D[h]);
    ms.sx[p] = sx;
    ms.dsx[p] = dv * sx;
    ms.sbx[p] = sB * sx;
    if (p == 0) ms.dfold = (a.D != nullptr && !a.D_has_hdim) ? (*a.D_scale) * (float)a.D[h] : 0.0f;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ms.tmem_slot;

  if (warp < 4) reg_dec<kRegsCtl>();
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const float* ab_src = ab_ws + ((int64_t)b * a.nheads + h) * nb * (kAbVecs * T);
      for (int j = 0; j < nb; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&ms.bc_empty[st], par, status, QB_ERR_TIMEOUT)) break;
        if (!mbar_wait(&ms.ab_empty[st], par, status, QB_ERR_TIMEOUT)) break;
        mbar_arrive_expect_tx(&ms.bc_full[st], 4 * kAtom + kAbBytes);
        uint8_t* dB = smem + kOffB16 + st * 2 * kAtom;
        uint8_t* dC = smem + kOffC16 + st * 2 * kAtom;
        bulk_load(ms.ab[st], ab_src + (int64_t)j * (kAbVecs * T), kAbBytes, &ms.bc_full[st]);
        tma_load_4d(dB, &tm_b16, &ms.bc_full[st], 0, g, j * T, b);
        tma_load_4d(dB + kAtom, &tm_b16, &ms.bc_full[st], 64, g, j * T, b);
        tma_load_4d(dC, &tm_c16, &ms.bc_full[st], 0, g, j * T, b);
        tma_load_4d(dC + kAtom, &tm_c16, &ms.bc_full[st], 64, g, j * T, b);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t id_cb = make_idesc(1, 0, 0, 0, 0, 128, 128);  // C (K-major) x B (K-major)
      constexpr uint32_t id_kn = make_idesc(1, 0, 0, 0, 1, 128, 64);   // K-major A x MN-major B
      constexpr uint32_t id_mn = make_idesc(1, 0, 0, 1, 1, 128, 64);   // MN-major A x MN-major B
      // descriptor words of every operand tile, built once (stage 1 of B / C is 2 atoms further)
      const SmemDesc dBk = make_smem_desc2(smem_u32(smem + kOffB16), 16, 1024, kSwizzle128B);      // B, K-major (CB)
      const SmemDesc dBm = make_smem_desc2(smem_u32(smem + kOffB16), kAtom, 1024, kSwizzle128B);   // B, MN-major A of GEMM4
      const SmemDesc dCk = make_smem_desc2(smem_u32(smem + kOffC16), 16, 1024, kSwizzle128B);      // C, K-major
      const SmemDesc dXraw = make_smem_desc2(smem_u32(smem + kOffXraw), 16, 1024, kSwizzle128B);
      const SmemDesc dXw = make_smem_desc2(smem_u32(smem + kOffXw), 16, 1024, kSwizzle128B);
      const SmemDesc dS16 = make_smem_desc2(smem_u32(smem + kOffS16), 16, 1024, kSwizzle128B);
      bool ok = mbar_wait(&ms.bc_full[0], 0, status, QB_ERR_TIMEOUT);
      if (ok) {
        tc_fence_after_sync();
        issue_gemm<false, false>(tmem + kColCB, dCk, dBk, id_cb);
        umma_commit(&ms.cb_ready[0]);
      }
      for (int j = 0; j < nb && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = j & 1;
        const SmemDesc bBm = desc_advance(dBm, st * 2 * kAtom), bC = desc_advance(dCk, st * 2 * kAtom);
        if (j > 0) {
          // GEMM2(j): D1[j & 1] = C(j) S_prev.  Needs the fp16 state of block j - 1; the buffer was last read by the
          // output step of block j - 2, whose y_free this thread observed before GEMM3(j - 1).  s16_ready also says that
          // the state update of block j - 1 has read the S accumulator, which GEMM4(j) overwrites below.
          ok = mbar_wait(&ms.s16_ready, (j - 1) & 1, status, QB_ERR_TIMEOUT);
          if (!ok) break;
          tc_fence_after_sync();
          TRACE(1, j, 0);
          issue_gemm<false, true>(tmem + (st ? kColD1b : kColD1), bC, dS16, id_kn);
          umma_commit(&ms.d1_ready);   // the state tile may be rewritten once this has fired
        }
        // GEMM4(j): local state of the block, S = (x w)^T B
        ok = mbar_wait(&ms.xops_ready, ph, status, QB_ERR_TIMEOUT);
        if (!ok) break;
        tc_fence_after_sync();
        TRACE(1, j, 1);
        issue_gemm<true, true>(tmem + kColS, bBm, dXw, id_mn);
        umma_commit(&ms.s_ready);
        // GEMM3(j) overwrites D2: the output step of block j - 1 must have loaded it
        if (j > 0) {
          ok = mbar_wait(&ms.y_free, (j - 1) & 1, status, QB_ERR_TIMEOUT);
          if (!ok) break;
        }
        // GEMM3(j): D2 = Lm X
        ok = mbar_wait(&ms.lm_ready, ph, status, QB_ERR_TIMEOUT);
        if (!ok) break;
        tc_fence_after_sync();
        TRACE(1, j, 2);
        {
          const uint32_t lm = tmem + (st ? kColCB1 : kColCB);   // packed fp16 Lm, 8 columns per K = 16 step
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_f16_ta(tmem + kColD2, lm + ks * 8, desc_advance(dXraw, ks * 2048), id_kn, ks != 0 ? 1u : 0u);
        }
        umma_commit(&ms.y_ready);
        TRACE(1, j, 3);
        if (j + 1 < nb) {
          // C.B^T of the next block into the other CB buffer (group A released it when it signalled lm_ready(j - 1)).
          // Issued after GEMM3(j) on purpose: it then runs while group B prepares the x operands of block j + 1 and the
          // tensor pipe would otherwise idle; ahead of GEMM3(j) it only delays the output of block j.
          const int sn = (j + 1) & 1;
          ok = mbar_wait(&ms.bc_full[sn], ((j + 1) >> 1) & 1, status, QB_ERR_TIMEOUT);
          if (!ok) break;
          tc_fence_after_sync();
          issue_gemm<false, false>(tmem + (sn ? kColCB1 : kColCB), desc_advance(dCk, sn * 2 * kAtom), desc_advance(dBk, sn * 2 * kAtom), id_cb);
          umma_commit(&ms.cb_ready[sn]);
        }
        // Release the B/C stage of block j last.  Its readers were CB(j), GEMM4(j) and GEMM2(j); releasing it right
        // after GEMM2(j) let the refill for block j + 2 run concurrently with GEMM3(j), and with that timing results
        // were not reproducible from run to run.  The refill has a whole block of slack, so nothing is lost here.
        umma_commit(&ms.bc_empty[st]);
      }
    }
  } else if (warp >= 4) {
    // ---------------- compute warps ----------------
    // Two groups of eight warps run concurrently on different parts of the pipeline:
    //   group A (warps 4..11)  builds Lm for block j as soon as CB(j) is ready and GEMM3(j-1) has released the tile;
    //   group B (warps 12..19) per step k: x operands of block k, output of block k - 1, state of block k.
    // Inside a group a thread owns one row (TMEM lane) and one half of the columns.
    const int cw = warp - 4;
    const int grp = cw >> 3;           // 0 = A, 1 = B
    const int q = warp & 3;            // TMEM lane quarter this warp may touch
    const int hsel = (cw >> 2) & 1;    // column half
    const int row = q * 32 + lane;
    const uint32_t tlane = (uint32_t)(q * 32) << 16;
    const int sw = row & 7;
    const bool lead = (threadIdx.x == kLead + grp * 256);
    auto gsync = [&]() {
      if (grp == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
    };
    // One thread of the group polls the mbarrier, the others park at the group's hardware barrier, which
    // also ANDs the outcome so that a timed-out wait makes the whole group leave its loop together.
    auto gwait = [&](uint64_t* bar, uint32_t parity) -> bool {
      uint32_t ok = 1;
      if (lead) ok = mbar_wait(bar, parity, status, QB_ERR_TIMEOUT) ? 1u : 0u;
      uint32_t r;
      if (grp == 0)
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(r) : "r"(ok) : "memory");
      else
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 2, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(r) : "r"(ok) : "memory");
      return r != 0;
    };

    // Several mbarriers, one group barrier: the lead thread waits for each in turn.
    auto gwait3 = [&](uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1, uint64_t* b2, uint32_t p2) -> bool {
      uint32_t ok = 1;
      if (lead) {
        ok = mbar_wait(b0, p0, status, QB_ERR_TIMEOUT) ? 1u : 0u;
        if (ok && b1 != nullptr) ok = mbar_wait(b1, p1, status, QB_ERR_TIMEOUT) ? 1u : 0u;
        if (ok && b2 != nullptr) ok = mbar_wait(b2, p2, status, QB_ERR_TIMEOUT) ? 1u : 0u;
      }
      uint32_t r;
      if (grp == 0)
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(r) : "r"(ok) : "memory");
      else
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 2, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(r) : "r"(ok) : "memory");
      return r != 0;
    };

    if (grp == 0) {
      reg_dec<kRegsA>();
      // ================= group A: Lm[t, s] = CB[t, s] 2^(a_t - bk_s) for s <= t (+ D on the diagonal) =================
      const float dfold = ms.dfold;
      for (int j = 0; j < nb; ++j) {
        const int st = j & 1;
        // the vectors of this block have landed and CB(j) is in TMEM buffer j & 1.  Lm(j) overwrites that buffer, which
        // GEMM3(j - 2) read long before CB(j) was issued into it, so nothing else has to be waited for.
        if (!gwait3(&ms.bc_full[st], (j >> 1) & 1, &ms.cb_ready[st], (j >> 1) & 1, nullptr, 0)) break;
        tc_fence_after_sync();
        if (lead) TRACE(0, j, 3);
        const float* av = ms.ab[st];
        const float* bkv = av + T;
        const float a_row = av[row];
        // Lm goes back into tensor memory, packed fp16, over the first 64 columns of the CB buffer it is computed from,
        // and GEMM3 reads it from there as its A operand: 32 KB of shared-memory stores and 32 KB of MMA operand reads
        // per block never happen.  Chunk c (fp32 columns 32c .. 32c + 31) becomes columns 16c .. 16c + 15.  The first
        // pass (chunks 0 and 1) writes columns 0 .. 31, which hold chunk 0's fp32 data, so a group barrier separates the
        // loads of that pass from its stores; the second pass (chunks 2, 3) writes columns 32 .. 63 = chunk 1's data,
        // consumed in the first pass.
        const uint32_t cbcol = tmem + tlane + ((j & 1) ? kColCB1 : kColCB);
#pragma unroll 1
        for (int i = 0; i < 2; ++i) {
          const int c = hsel + 2 * i;  // 32-column chunk of k
          uint32_t o[16];
          if (c > q) {  // entirely above the diagonal for every row of this warp
#pragma unroll
            for (int u = 0; u < 16; ++u) o[u] = 0u;
            if (i == 0) { gsync(); tc_fence_after_sync(); }
          } else {
            uint32_t cb[32];
            tmem_ld_32x32(cbcol + 32 * c, cb);
            if (c == q) {
              // diagonal chunk: exact exponent per element, the k <= m mask (k - 32c <= lane), and the skip weight D
              // on the diagonal itself (y = sx (Lm + D I) x) when D has one value per head
              tmem_ld_wait();
              if (i == 0) { tc_fence_before_sync(); gsync(); tc_fence_after_sync(); }
              const float4* bk4 = reinterpret_cast<const float4*>(bkv + 32 * c);
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const float4 bb = bk4[u];
                const int t0 = 4 * u;
                float e0 = __uint_as_float(cb[t0 + 0]) * fast_exp2(a_row - bb.x);
                float e1 = __uint_as_float(cb[t0 + 1]) * fast_exp2(a_row - bb.y);
                float e2 = __uint_as_float(cb[t0 + 2]) * fast_exp2(a_row - bb.z);
                float e3 = __uint_as_float(cb[t0 + 3]) * fast_exp2(a_row - bb.w);
                e0 = t0 + 0 < lane ? e0 : (t0 + 0 == lane ? e0 + dfold : 0.0f);
                e1 = t0 + 1 < lane ? e1 : (t0 + 1 == lane ? e1 + dfold : 0.0f);
                e2 = t0 + 2 < lane ? e2 : (t0 + 2 == lane ? e2 + dfold : 0.0f);
                e3 = t0 + 3 < lane ? e3 : (t0 + 3 == lane ? e3 + dfold : 0.0f);
                o[2 * u] = pack_h2(e0, e1);
                o[2 * u + 1] = pack_h2(e2, e3);
              }
            } else {
              // chunk below the diagonal: 2^(a_t - bk_s) = 2^(a_t - m) * ec[s], m = a at the end of chunk c
              const float e_row = fast_exp2(a_row - av[32 * c + 31]);
              tmem_ld_wait();
              if (i == 0) { tc_fence_before_sync(); gsync(); tc_fence_after_sync(); }
              const float4* ec4 = reinterpret_cast<const float4*>(av + 2 * T + 32 * c);
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const float4 ee = ec4[u];
                const int t0 = 4 * u;
                const float e0 = __uint_as_float(cb[t0 + 0]) * (e_row * ee.x);
                const float e1 = __uint_as_float(cb[t0 + 1]) * (e_row * ee.y);
                const float e2 = __uint_as_float(cb[t0 + 2]) * (e_row * ee.z);
                const float e3 = __uint_as_float(cb[t0 + 3]) * (e_row * ee.w);
                o[2 * u] = pack_h2(e0, e1);
                o[2 * u + 1] = pack_h2(e2, e3);
              }
            }
          }
          tmem_st16(cbcol + 16 * c, o);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        gsync();
        if (lead) { mbar_arrive(&ms.lm_ready); mbar_arrive(&ms.ab_empty[st]); TRACE(0, j, 4); }
      }
    } else {
      reg_inc<kRegsB>();
      // ================= group B: x operands of block k, output of block k - 1, state of block k =================
      const float lscb = fast_log2(sC * sB);
      const bool d_per_channel = a.D != nullptr && a.D_has_hdim;   // then the skip term is added here, from a re-read of x
      const int8_t* xrow_base = a.x + (int64_t)b * a.x_sb + (int64_t)h * a.x_sh + 32 * hsel;
      __half* out_base = static_cast<__half*>(a.out) + ((int64_t)b * a.seqlen * a.nheads + h) * P + 32 * hsel + 8 * (lane & 3);
      const int64_t out_pitch = (int64_t)a.nheads * P;
      float s_reg[32];
#pragma unroll
      for (int t = 0; t < 32; ++t) s_reg[t] = 0.0f;
      uint4 xn0 = make_uint4(0, 0, 0, 0), xn1 = make_uint4(0, 0, 0, 0);
      if (row < a.seqlen) {
        const uint4* src = reinterpret_cast<const uint4*>(xrow_base + (int64_t)row * a.x_sl);
        xn0 = ldg_nc_now(src); xn1 = ldg_nc_now(src + 1);
      }
      float e_prev = 0.0f;   // sC 2^(a_row) of the previous block: weight of its carried-in term
      float r_tot = 0.0f;
      for (int k = 0; k <= nb; ++k) {
        const int st = k & 1;
        if (k < nb) {
          // ---- x(k) -> fp16 operands: raw, and scaled by w_l = dt_l 2^(r - a_l) = 2^(r - bk_l - lscb) (0 where dt_l = 0).
          // The raw tile is free once GEMM3(k-1) is done (y_ready); the scaled tile was released by GEMM4(k-1),
          // whose completion this group observed before its previous state update.
          const int l = k * T + row;
          const uint4 xq0 = xn0, xq1 = xn1;
          if (l + T < a.seqlen) {  // the x rows of the next block: a whole block of work covers their latency
            const uint4* src = reinterpret_cast<const uint4*>(xrow_base + (int64_t)(l + T) * a.x_sl);
            xn0 = ldg_nc_now(src); xn1 = ldg_nc_now(src + 1);
          } else {
            xn0 = make_uint4(0, 0, 0, 0); xn1 = make_uint4(0, 0, 0, 0);
          }
          if (lead) TRACE(1, k, 4);
          // int8 -> fp16 happens before the wait: only the stores depend on the tiles being free
          uint4 xr[4];
          {
            const uint32_t xwd[8] = {xq0.x, xq0.y, xq0.z, xq0.w, xq1.x, xq1.y, xq1.z, xq1.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              __half2 r0, r1, r2, r3;
              s8x4_to_h2x2(xwd[2 * c], r0, r1);
              s8x4_to_h2x2(xwd[2 * c + 1], r2, r3);
              xr[c] = make_uint4(h2_bits(r0), h2_bits(r1), h2_bits(r2), h2_bits(r3));
            }
          }
          if (!gwait3(&ms.bc_full[st], (k >> 1) & 1, k > 0 ? &ms.y_ready : nullptr, (k - 1) & 1, nullptr, 0)) break;
          if (lead) TRACE(1, k, 13);
          const float* av = ms.ab[st];
          const float a_row = av[row];
          r_tot = av[T - 1];
          const __half2 w2 = __float2half2_rn(fast_exp2(r_tot - av[T + row] - lscb));
          const float e_now = k > 0 ? sC * fast_exp2(a_row) : 0.0f;
          {
            uint8_t* rowp_raw = smem + kOffXraw + row * 128;
            uint8_t* rowp_w = smem + kOffXw + row * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int chunk = ((4 * hsel + c) ^ sw) << 4;
              const uint4 v = xr[c];
              *reinterpret_cast<uint4*>(rowp_raw + chunk) = v;
              *reinterpret_cast<uint4*>(rowp_w + chunk) =
                  make_uint4(h2_bits(__hmul2(*reinterpret_cast<const __half2*>(&v.x), w2)),
                             h2_bits(__hmul2(*reinterpret_cast<const __half2*>(&v.y), w2)),
                             h2_bits(__hmul2(*reinterpret_cast<const __half2*>(&v.z), w2)),
                             h2_bits(__hmul2(*reinterpret_cast<const __half2*>(&v.w), w2)));
            }
          }
          fence_proxy_async_smem();
          gsync();
          if (lead) { mbar_arrive(&ms.xops_ready); mbar_arrive(&ms.ab_empty[st]); TRACE(1, k, 5); }
          // swap: e_prev must describe block k - 1 in the output step below, block k afterwards
          const float t = e_prev; e_prev = e_now;
          if (k > 0) {
            // ---- output of block k - 1 (weight t) ----
#define QB_SSD_OUTPUT_STEP(EW)                                                                                               \
            {                                                                                                                \
              const int jj = k - 1;                                                                                          \
              tc_fence_after_sync();                                                                                         \
              uint32_t d2[32], d1[32];                                                                                       \
              tmem_ld_32x32(tmem + tlane + kColD2 + 32 * hsel, d2);                                                          \
              if (jj > 0) tmem_ld_32x32(tmem + tlane + ((jj & 1) ? kColD1b : kColD1) + 32 * hsel, d1);                       \
              tmem_ld_wait();                                                                                                \
              tc_fence_before_sync();                                                                                        \
              gsync();                                                                                                       \
              if (lead) { mbar_arrive(&ms.y_free); TRACE(1, jj, 9); } /* both accumulators are in registers */               \
              const float4* sx4 = reinterpret_cast<const float4*>(ms.sx + 32 * hsel);                                        \
              uint4 c4[4];                                                                                                   \
              _Pragma("unroll") for (int t8 = 0; t8 < 4; ++t8) {                                                             \
                uint32_t o[4];                                                                                               \
                _Pragma("unroll") for (int v = 0; v < 2; ++v) {                                                              \
                  const int t4 = 2 * t8 + v;                                                                                 \
                  const float4 sx = sx4[t4];                                                                                 \
                  float y0 = sx.x * __uint_as_float(d2[4 * t4 + 0]);                                                         \
                  float y1 = sx.y * __uint_as_float(d2[4 * t4 + 1]);                                                         \
                  float y2 = sx.z * __uint_as_float(d2[4 * t4 + 2]);                                                         \
                  float y3 = sx.w * __uint_as_float(d2[4 * t4 + 3]);                                                         \
                  if (jj > 0) {                                                                                              \
                    y0 = fmaf(EW, __uint_as_float(d1[4 * t4 + 0]), y0);                                                      \
                    y1 = fmaf(EW, __uint_as_float(d1[4 * t4 + 1]), y1);                                                      \
                    y2 = fmaf(EW, __uint_as_float(d1[4 * t4 + 2]), y2);                                                      \
                    y3 = fmaf(EW, __uint_as_float(d1[4 * t4 + 3]), y3);                                                      \
                  }                                                                                                          \
                  if (d_per_channel) {                                                                                       \
                    const int lr = jj * T + row;                                                                             \
                    uint32_t xw = 0;                                                                                         \
                    if (lr < a.seqlen) xw = __ldg(reinterpret_cast<const uint32_t*>(xrow_base + (int64_t)lr * a.x_sl) + t4); \
                    const float4 dx = reinterpret_cast<const float4*>(ms.dsx + 32 * hsel)[t4];                               \
                    __half2 h01, h23;                                                                                        \
                    s8x4_to_h2x2(xw, h01, h23);                                                                              \
                    const float2 x01 = __half22float2(h01), x23 = __half22float2(h23);                                       \
                    y0 = fmaf(dx.x, x01.x, y0); y1 = fmaf(dx.y, x01.y, y1);                                                  \
                    y2 = fmaf(dx.z, x23.x, y2); y3 = fmaf(dx.w, x23.y, y3);                                                  \
                  }                                                                                                          \
                  o[2 * v] = pack_h2(y0, y1);                                                                                \
                  o[2 * v + 1] = pack_h2(y2, y3);                                                                            \
                }                                                                                                            \
                c4[t8] = make_uint4(o[0], o[1], o[2], o[3]);                                                                 \
              }                                                                                                              \
              /* 4 x 4 transpose of 16-byte pieces inside each quad of lanes: afterwards lane i of a quad holds piece i of  \
                 the quad's four rows, so one store instruction writes 64 contiguous bytes per row */                        \
              quad_transpose(c4, lane);                                                                                      \
              const int r0 = jj * T + (row & ~3);                                                                            \
              _Pragma("unroll") for (int m = 0; m < 4; ++m)                                                                  \
                if (r0 + m < a.seqlen) *reinterpret_cast<uint4*>(out_base + (int64_t)(r0 + m) * out_pitch) = c4[m];          \
            }
            QB_SSD_OUTPUT_STEP(t)
          }
        } else {
          if (!gwait(&ms.y_ready, (nb - 1) & 1)) break;
          QB_SSD_OUTPUT_STEP(e_prev)
          break;
        }
#undef QB_SSD_OUTPUT_STEP

        // ---- state: s <- 2^r s + sB sx S_loc ; publish its fp16 copy for the next block -----------
        // GEMM4(k) done; GEMM2(k) done, so the fp16 state tile it read may be rewritten
        if (!gwait3(&ms.s_ready, k & 1, k > 0 ? &ms.d1_ready : nullptr, (k - 1) & 1, nullptr, 0)) break;
        tc_fence_after_sync();
        if (lead) TRACE(1, k, 6);
        {
          const float dec = fast_exp2(r_tot);
          uint32_t sl[32];
          tmem_ld_32x32(tmem + tlane + kColS + 32 * hsel, sl);
          tmem_ld_wait();
          const float4* sb4 = reinterpret_cast<const float4*>(ms.sbx + 32 * hsel);
#pragma unroll
          for (int t4 = 0; t4 < 8; ++t4) {
            const float4 sc = sb4[t4];
            s_reg[4 * t4 + 0] = fmaf(dec, s_reg[4 * t4 + 0], sc.x * __uint_as_float(sl[4 * t4 + 0]));
            s_reg[4 * t4 + 1] = fmaf(dec, s_reg[4 * t4 + 1], sc.y * __uint_as_float(sl[4 * t4 + 1]));
            s_reg[4 * t4 + 2] = fmaf(dec, s_reg[4 * t4 + 2], sc.z * __uint_as_float(sl[4 * t4 + 2]));
            s_reg[4 * t4 + 3] = fmaf(dec, s_reg[4 * t4 + 3], sc.w * __uint_as_float(sl[4 * t4 + 3]));
          }
          if (k + 1 < nb) {
            uint8_t* dst = smem + kOffS16 + row * 128;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              *reinterpret_cast<uint4*>(dst + (((4 * hsel + u) ^ sw) << 4)) =
                  make_uint4(pack_h2(s_reg[8 * u], s_reg[8 * u + 1]), pack_h2(s_reg[8 * u + 2], s_reg[8 * u + 3]),
                             pack_h2(s_reg[8 * u + 4], s_reg[8 * u + 5]), pack_h2(s_reg[8 * u + 6], s_reg[8 * u + 7]));
            }
          }
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        gsync();
        if (lead && k + 1 < nb) mbar_arrive(&ms.s16_ready);   // also: the S accumulator has been read
        if (lead) TRACE(1, k, 7);

        // ---- final state -> int8 after the last block -----------------------------------------------------
        if (k + 1 == nb) {
          int hg = 0;
          if (a.grouped) hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, h % hpg);
          int8_t* fs = a.final_states + ((int64_t)b * a.nheads + h) * P * N + row;
#pragma unroll
          for (int t = 0; t < 32; ++t) {  // fully unrolled: s_reg must never be indexed dynamically
            const int p = 32 * hsel + t;
            float ss;
            if (!a.grouped) {
              ss = a.ssm_state_scale[0];
            } else {
              const int dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, p);
              ss = a.ssm_state_scale[((int64_t)(g * a.nhead_groups + hg) * a.ndim_groups + dg) * N + row];
            }
            const float fin = __half2float(__float2half_rn(s_reg[t]));
            fs[(int64_t)p * N] = (int8_t)rint_s8(fin / ss);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// B, C int8 (B, L, G, N) -> fp16 [B][L][G][N] contiguous (values unchanged).
__global__ void ssd_widen_bc_kernel(const int8_t* __restrict__ Bq, int64_t B_sb, int64_t B_sl, int64_t B_sg,
                                    const int8_t* __restrict__ Cq, int64_t C_sb, int64_t C_sl, int64_t C_sg,
                                    __half* __restrict__ B16, __half* __restrict__ C16, int batch, int seqlen, int ngroups) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 16-element piece
  const int pieces = N / 16;
  const int64_t total = (int64_t)batch * seqlen * ngroups * pieces;
  if (idx >= total) return;
  const int pc = (int)(idx % pieces);
  const int gg = (int)((idx / pieces) % ngroups);
  const int l = (int)((idx / ((int64_t)pieces * ngroups)) % seqlen);
  const int bb = (int)(idx / ((int64_t)pieces * ngroups * seqlen));
  auto widen = [&](const int8_t* src, __half* dst) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
    __half2 o[8];
    s8x4_to_h2x2(v.x, o[0], o[1]);
    s8x4_to_h2x2(v.y, o[2], o[3]);
    s8x4_to_h2x2(v.z, o[4], o[5]);
    s8x4_to_h2x2(v.w, o[6], o[7]);
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(h2_bits(o[0]), h2_bits(o[1]), h2_bits(o[2]), h2_bits(o[3]));
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(h2_bits(o[4]), h2_bits(o[5]), h2_bits(o[6]), h2_bits(o[7]));
  };
  const int64_t o16 = (((int64_t)bb * seqlen + l) * ngroups + gg) * N + pc * 16;
  widen(Bq + bb * B_sb + l * B_sl + gg * B_sg + pc * 16, B16 + o16);
  widen(Cq + bb * C_sb + l * C_sl + gg * C_sg + pc * 16, C16 + o16);
}

// Per (batch, head, 128-token block): dt = clamp(softplus(s_dt q + bias)); a = inclusive running sum of
// dt * A * log2(e) inside the block; bk = a - log2(dt) - log2(sC sB) (+inf where dt == 0, i.e. past the
// end of the sequence).  One warp per block, four tokens per lane.
__global__ void ssd_dt_kernel(qb_ssd_args a, float* __restrict__ ab_ws, int nb) {
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t units = (int64_t)a.batch * a.nheads * nb;
  if (unit >= units) return;
  const int j = (int)(unit % nb);
  const int h = (int)((unit / nb) % a.nheads);
  const int b = (int)(unit / ((int64_t)nb * a.nheads));
  const int g = h / (a.nheads / a.ngroups);
  const float A2 = -__expf((*a.A_scale) * (float)a.A_log[h]) * 1.4426950408889634f;
  const float s_dt = *a.dt_scale;
  const float bias = a.dt_bias != nullptr ? __half2float(static_cast<const __half*>(a.dt_bias)[h]) : 0.0f;
  const float lscb = fast_log2((a.grouped ? a.C_scale[g] : a.C_scale[0]) * (a.grouped ? a.B_scale[g] : a.B_scale[0]));
  const int8_t* dtp = a.dt + (int64_t)b * a.dt_sb + h;
  float dt[4], cs[4];
  float run = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int l = j * T + lane * 4 + i;
    float v = 0.0f;
    if (l < a.seqlen) {
      v = fmaf(s_dt, (float)dtp[(int64_t)l * a.dt_sl], bias);
      if (a.dt_softplus) v = softplus_f(v);
      v = fminf(fmaxf(v, a.dt_min), a.dt_max);
    }
    dt[i] = v;
    run += v * A2;
    cs[i] = run;
  }
  float incl = run;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float u = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += u;
  }
  const float pre = incl - run;
  float* dst = ab_ws + unit * (kAbVecs * T);
  float4 av, bv;
  float* ap = reinterpret_cast<float*>(&av);
  float* bp = reinterpret_cast<float*>(&bv);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ap[i] = pre + cs[i];
    bp[i] = dt[i] > 0.0f ? ap[i] - fast_log2(dt[i]) - lscb : __int_as_float(0x7f800000);
  }
  // ec[s] = 2^(m - bk[s]) with m = a at the end of the 32-token chunk of s (<= a[s], so the exponent is <= log2 of
  // dt sC sB: no overflow).  For a row t of a LATER chunk, Lm[t, s] = CB[t, s] 2^(a[t] - m) ec[s], both factors <= 1.
  const float m = __shfl_sync(0xffffffffu, ap[3], (lane & ~7) | 7);
  float4 ev;
  float* ep = reinterpret_cast<float*>(&ev);
#pragma unroll
  for (int i = 0; i < 4; ++i) ep[i] = fast_exp2(m - bp[i]);
  reinterpret_cast<float4*>(dst)[lane] = av;
  reinterpret_cast<float4*>(dst + T)[lane] = bv;
  reinterpret_cast<float4*>(dst + 2 * T)[lane] = ev;
}

int64_t align256l(int64_t v) { return (v + 255) & ~(int64_t)255; }

}  // namespace

bool ssd_tc_eligible(const qb_ssd_args* a) {
  if (a->headdim != P || a->dstate != N || a->z != nullptr) return false;
  if (!aligned(a->x, 16) || a->x_sl % 16 != 0 || a->x_sb % 16 != 0 || a->x_sh % 16 != 0) return false;
  if (!aligned(a->Bm, 16) || !aligned(a->Cm, 16) || a->B_sl % 16 || a->B_sb % 16 || a->B_sg % 16 || a->C_sl % 16 ||
      a->C_sb % 16 || a->C_sg % 16)
    return false;
  if (!aligned(a->out, 16)) return false;
  return true;
}

int64_t ssd_tc_workspace_bytes(int B, int L, int H, int G) {
  const int64_t nb = (L + T - 1) / T;
  return 2 * align256l((int64_t)B * L * G * N * 2) + align256l((int64_t)B * H * nb * kAbVecs * T * 4);
}

int ssd_tc_launch(const qb_ssd_args* a, cudaStream_t st) {
  const int64_t half_bytes = align256l((int64_t)a->batch * a->seqlen * a->ngroups * N * 2);
  const int nb = (int)ceil_div(a->seqlen, T);
  __half* B16 = reinterpret_cast<__half*>(static_cast<char*>(a->workspace));
  __half* C16 = reinterpret_cast<__half*>(static_cast<char*>(a->workspace) + half_bytes);
  float* ab_ws = reinterpret_cast<float*>(static_cast<char*>(a->workspace) + 2 * half_bytes);
  {
    const int64_t total = (int64_t)a->batch * a->seqlen * a->ngroups * (N / 16);
    ssd_widen_bc_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(a->Bm, a->B_sb, a->B_sl, a->B_sg, a->Cm, a->C_sb,
                                                                       a->C_sl, a->C_sg, B16, C16, a->batch, a->seqlen,
                                                                       a->ngroups);
    QB_LAUNCH_OK("ssd_widen_bc_kernel");
    const int64_t units = (int64_t)a->batch * a->nheads * nb;
    ssd_dt_kernel<<<(unsigned)ceil_div(units, 4), 128, 0, st>>>(*a, ab_ws, nb);
    QB_LAUNCH_OK("ssd_dt_kernel");
  }
  CUtensorMap tb, tcm;
  const uint64_t dims[4] = {(uint64_t)N, (uint64_t)a->ngroups, (uint64_t)a->seqlen, (uint64_t)a->batch};
  const uint64_t strides[3] = {(uint64_t)N * 2, (uint64_t)a->ngroups * N * 2, (uint64_t)a->seqlen * a->ngroups * N * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
  int rc = encode_tmap_f16_4d(&tb, B16, dims, strides, box);
  if (rc != QB_OK) return rc;
  rc = encode_tmap_f16_4d(&tcm, C16, dims, strides, box);
  if (rc != QB_OK) return rc;
  static bool attr_set[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 64 || !attr_set[dev]) {
    QB_CUDA_OK(cudaFuncSetAttribute(ssd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    if (dev < 64) attr_set[dev] = true;
  }
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "device status word unavailable");
  ssd_tc_kernel<<<(unsigned)(a->batch * a->nheads), kThreads, kSmemBytes, st>>>(tb, tcm, *a, ab_ws, status);
  QB_LAUNCH_OK("ssd_tc_kernel");
  return QB_OK;
}

}  // namespace qb

#ifdef QB_DUMP
extern "C" int qb_debug_set_dump(float* p) {  // development builds only
  return cudaMemcpyToSymbol(qb::g_dump, &p, sizeof(p)) == cudaSuccess ? 0 : -1;
}
#endif
#ifdef QB_TRACE
extern "C" int qb_debug_read_trace(long long* out) {  // 2 x 64 x 16 clock64 stamps of CTA 0 (development builds only)
  return cudaMemcpyFromSymbol(out, qb::g_trace, sizeof(qb::g_trace)) == cudaSuccess ? 0 : -1;
}
#endif
