// Mamba2 SSD chunk scan on the Blackwell tensor cores (headdim 64, d_state 128).
//
// The sequence of one (batch, head) pair is walked in blocks of T = 128 tokens with the 64 x 128 SSM state carried in
// registers (fp32), so nothing but inputs and outputs ever touches HBM.  Per block:
//
//   CB    = C . B^T                         128 x 128 x 128   tcgen05 f16 (integer-valued operands: exact)
//   D1    = C . s                           128 x  64 x 128   state entering the block, fp16 copy
//   S_loc = B^T . (x * w)                   128 x  64 x 128   w_l = dt_l 2^(r - a_l)
//   D2    = Lm . x                          128 x  64 x 128   Lm[m,k] = CB[m,k] 2^(a_m - a_k) dt_k, k <= m
//   y[m,p]   = sC 2^(a_m) D1 + sx[p] (D2 + D x)            s <- 2^r s + sB sx[p] S_loc
//
// a_l is the running sum of dt*A*log2(e) inside the block and r its last value, so every exponent is <= 0.  One small
// preparation kernel runs first: some of its blocks widen B and C (shared by all heads of a group) to fp16 once -- values
// stay the raw integers, scales are applied in the epilogues -- the others evaluate softplus / the running sums and leave, per
// (batch, head, block), the vectors a[128], bk[128] = a - log2(dt) - log2(sC sB) and ec[128] (column factors of the
// off-diagonal 32 x 32 chunks of Lm: there 2^(a_m - bk_k) = 2^(a_m - a_end(chunk)) * ec[k], two multiplies instead of
// an ex2 per element; the diagonal chunks keep the exact per-element exponent).  When D has one value per head it is
// added on the diagonal of Lm, so the output step needs no x.
//
// The kernel is persistent: one CTA per SM, and the (batch, head, block) list is cut into equal contiguous ranges, one
// per CTA, so that the SMs finish together whatever the number of pairs (320 pairs on 148 SMs would otherwise run as
// three waves of which the last is 16 % full).  A range covers the tail of one pair, whole pairs, and the head of
// another.  A CTA runs the head part FIRST (it depends on nothing) and hands the fp32 state after it to the next CTA
// through global memory (release / acquire on a flag); it runs its own tail part LAST, by which time the previous CTA
// has long published the state it needs.  A head part never waits, so the scheme cannot deadlock; the wait is bounded
// all the same.  The arithmetic per pair is the same sequence of operations wherever the cut falls, so results do not
// depend on the number of SMs.
//
// 640 threads.  Warp 3: one thread serves the TMA queues (loads of 128-byte-swizzled B / C tiles that serve as K-major
// operands of CB and D1 and as the MN-major A operand of S_loc without reshuffling, the int8 x tile, the vectors and the
// per-pair constants; and the output store of each block).  Warp 1 issues the MMAs and owns TMEM.  Warps 0 and 2 turn
// the int8 x tile of block k + 1 into the two fp16 operand tiles (raw, and scaled by w) while the compute warps are
// still on block k: that work needs no tensor memory.  Warps 4..19 compute; all 16 walk the same three phases per
// block, a thread owning one row (TMEM lane) and one quarter of the columns:
//   P2  CB(k) -> Lm(k), written back to tensor memory as packed fp16 (A operand)  -> GEMM3(k) = D2, then CB(k+1)
//   P3  state update from S_loc(k), fp16 copy of the state to shared memory      -> GEMM2(k+1) = D1
//   P4  y(k) from D2(k), D1(k): to a swizzled staging tile, stored by warp 3 with one TMA store
// so every GEMM runs while the compute warps are busy with the next phase, and program order plus the group barriers
// of each phase is what frees each buffer (noted at each wait).  The warps are kept in lock step on purpose: variants
// in which they synchronised through mbarriers only and drifted apart (each thread polling, or one barrier per phase
// with per-warp arrivals) were 10 to 30 % slower although they wait less -- with every warp in the same phase the
// unrolled code of that phase is fetched once for all of them.  Every mbarrier completes exactly once per block, is
// waited on by each consumer once per phase and in order, and all waits are bounded.  The B / C stage is handed back to
// the TMA producer only at the end of an MMA iteration.
#include "tc_common.cuh"

namespace qb {

namespace {
using namespace tc;

constexpr int T = 128, P = 64, N = 128;
// Warps 0 and 2: x operands; warp 1: MMA issuer; warp 3: TMA loads and stores.  Warps 4..19 compute.
constexpr int kThreads = 640;                  // 4 control warps + 16 compute warps (a 21st warp would cap registers at 80)
constexpr int kLead = 128;                     // first compute thread
constexpr int kCompute = kThreads - kLead;     // 512

constexpr int kAtom = T * 128;                 // 16 KB: 128 rows x 128 bytes
constexpr int kOffB16 = 0;                     // 2 stages x 2 atoms
constexpr int kOffC16 = 4 * kAtom;             // 2 stages x 2 atoms
constexpr int kOffXraw = 8 * kAtom;            // 1 atom
constexpr int kOffXw = 9 * kAtom;              // 1 atom
constexpr int kOffS16 = 10 * kAtom;            // 1 atom
constexpr int kOffY = 11 * kAtom;              // output staging: the fp16 y tile of a block, 128 rows x 128 bytes, swizzled
constexpr int kOffX8 = 12 * kAtom;             // 2 stages x 8 KB: the int8 x tile of a block (128 rows x 64 bytes)
constexpr int kXBytes = T * P;
constexpr int kOffMisc = 13 * kAtom;           // vectors + barriers
constexpr int kMiscBytes = 8192;
constexpr int kSmemBytes = kOffMisc + kMiscBytes + 1024;
constexpr int kAbVecs = 3;                     // a[128], bk[128], ec[128] per block, fp32
constexpr int kAbBytes = kAbVecs * T * 4;
constexpr int kHandoffFloats = kCompute * 16;  // one fp32 state (64 x 128) per CTA, thread-major
// Per (batch, head) constants, written by the preparation kernel and delivered with every block's stage, so that moving
// on to another pair costs the compute warps nothing: sx[64], D sx[64], sB sx[64], then the scalars below.
constexpr int kHcFloats = 256, kHcBytes = kHcFloats * 4;
constexpr int kHcSx = 0, kHcDsx = 64, kHcSbx = 128, kHcDfold = 192, kHcSC = 193, kHcLscb = 194, kHcStateScale = 195;

// Tensor memory: CB (fp32), Lm (packed fp16, 64 columns), D2, S, and D1 double-buffered (GEMM2(k+1) is issued while the
// output step of block k still has D1(k) to read).
constexpr uint32_t kColCB = 0, kColLm = 128, kColD2 = 192, kColS = 256, kColD1 = 320, kColD1b = 384, kTmemCols = 512;

struct Misc {
  float ab[2][kAbVecs * T];   // per stage: a, bk, ec of the block (see ssd_dt)
  float hc[2][kHcFloats];     // per stage: the constants of the block's (batch, head) pair (kHc* offsets)
  uint64_t bc_full[2], bc_empty[2], ab_empty[2];
  uint64_t cb_ready, xops_ready, s_ready, lm_ready, y_ready, s16_ready, d1_ready;
  uint64_t y_full, y_empty;   // output staging tile: written by the 16 compute warps, stored (and released) by warp 2
  uint32_t tmem_slot;
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc does not fit");

// The work of one CTA: blocks [s, e) of the list (pair-major, block-minor), as up to three kinds of item.
struct Plan {
  int n_items;      // head part + whole pairs + tail part
  int total;        // blocks in all items
  int head_unit, head_len;     // head part: blocks [0, head_len) of head_unit (0 = none); runs first, publishes its state
  int whole_first, n_whole;    // whole pairs (strided by whole_step)
  int whole_step;
  int tail_unit, tail_from;    // tail part: blocks [tail_from, nb) of tail_unit (tail_from = 0: none); runs last
};
struct Item { int unit, jb, je; bool has_init, publish; };

__device__ __forceinline__ Plan make_plan(int cta, int grid, int units, int nb, int split) {
  Plan p;
  if (!split) {   // whole pairs only, round robin
    p.head_len = 0; p.tail_from = 0; p.head_unit = p.tail_unit = 0;
    p.whole_first = cta; p.whole_step = grid;
    p.n_whole = cta < units ? (units - cta + grid - 1) / grid : 0;
  } else {
    const long long tb = (long long)units * nb;
    const long long s = tb * cta / grid, e = tb * (cta + 1) / grid;
    const int us = (int)(s / nb), js = (int)(s % nb), ue = (int)(e / nb), je = (int)(e % nb);
    p.tail_unit = us; p.tail_from = js;
    p.head_unit = ue; p.head_len = je;
    p.whole_first = js != 0 ? us + 1 : us; p.whole_step = 1;
    p.n_whole = ue - p.whole_first;   // >= 0 because a range is at least nb blocks long
  }
  p.n_items = p.n_whole + (p.head_len != 0) + (p.tail_from != 0);
  p.total = p.n_whole * nb + p.head_len + (p.tail_from != 0 ? nb - p.tail_from : 0);
  return p;
}
__device__ __forceinline__ Item get_item(const Plan& p, int idx, int nb) {
  Item im;
  if (p.head_len != 0) {
    if (idx == 0) { im.unit = p.head_unit; im.jb = 0; im.je = p.head_len; im.has_init = false; im.publish = true; return im; }
    --idx;
  }
  if (idx < p.n_whole) { im.unit = p.whole_first + idx * p.whole_step; im.jb = 0; im.je = nb; im.has_init = false; im.publish = false; return im; }
  im.unit = p.tail_unit; im.jb = p.tail_from; im.je = nb; im.has_init = true; im.publish = false;
  return im;
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
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
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
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

// kDPerChannel: D has one value per (head, channel) and is added in the output step (from a re-read of x); the common
// case (one value per head, folded into the diagonal of Lm) compiles without that code.
template <bool kDPerChannel>
__global__ void __launch_bounds__(kThreads, 1)
ssd_tc_kernel(const __grid_constant__ CUtensorMap tm_b16, const __grid_constant__ CUtensorMap tm_c16,
              const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_out, qb_ssd_args a,
              const float* __restrict__ ab_ws, const float* __restrict__ hc_ws, float* __restrict__ handoff, int* __restrict__ flags, int split, int* status,
              int early) {
  if (early) grid_dependency_launch();   // the kernel after this one may get resident and run its prologue as CTAs here finish
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Misc& ms = *reinterpret_cast<Misc*>(smem + kOffMisc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hpg = a.nheads / a.ngroups;
  const int nb = (a.seqlen + T - 1) / T;
  const Plan plan = make_plan((int)blockIdx.x, (int)gridDim.x, a.batch * a.nheads, nb, split);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&ms.bc_full[s], 1); mbar_init(&ms.bc_empty[s], 1); mbar_init(&ms.ab_empty[s], 1); }
    mbar_init(&ms.cb_ready, 1); mbar_init(&ms.xops_ready, 2); mbar_init(&ms.s_ready, 1); mbar_init(&ms.lm_ready, 1);
    mbar_init(&ms.y_ready, 1); mbar_init(&ms.s16_ready, 1); mbar_init(&ms.d1_ready, 1);
    mbar_init(&ms.y_full, 16); mbar_init(&ms.y_empty, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_b16);
    prefetch_tensormap(&tm_c16);
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(&ms.tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ms.tmem_slot;
  // The kernel is launched as a programmatic dependent of the preparation kernel: everything above overlaps its tail;
  // from here on its results (widened B / C, vectors, constants, cleared flags) are read.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 3) {
    // ---------------- TMA: loads and output stores ----------------
    // One thread serves two queues in an event loop of non-blocking tests: the loads of block k + 2 as soon as its stage
    // has been released (by the MMA issuer and by the compute warps), and the store of block k as soon as the compute
    // warps have filled the staging tile (one TMA store per block; rows past the end of the sequence are clipped by the
    // hardware; the tile is handed back once the store has read it).
    if (lane == 0) {
      struct Cursor { int ii, j, it; Item im; };
      auto start = [&](Cursor& c) { c.ii = 0; c.it = 0; if (plan.n_items > 0) { c.im = get_item(plan, 0, nb); c.j = c.im.jb; } };
      auto step = [&](Cursor& c) {
        ++c.it;
        if (++c.j >= c.im.je) { if (++c.ii < plan.n_items) { c.im = get_item(plan, c.ii, nb); c.j = c.im.jb; } }
      };
      Cursor ld, stc;
      start(ld); start(stc);
      long long t_last = clock64();
      while (stc.it < plan.total) {
        bool progress = false;
        if (ld.it < plan.total) {
          const int st = ld.it & 1;
          const uint32_t par = ((ld.it >> 1) & 1) ^ 1;
          if (mbar_test_wait(&ms.bc_empty[st], par) && mbar_test_wait(&ms.ab_empty[st], par)) {
            const int b = ld.im.unit / a.nheads, h = ld.im.unit % a.nheads, g = h / hpg;
            const float* ab_src = ab_ws + ((int64_t)ld.im.unit * nb + ld.j) * (kAbVecs * T);
            mbar_arrive_expect_tx(&ms.bc_full[st], 4 * kAtom + kAbBytes + kXBytes + kHcBytes);
            uint8_t* dB = smem + kOffB16 + st * 2 * kAtom;
            uint8_t* dC = smem + kOffC16 + st * 2 * kAtom;
            bulk_load(ms.ab[st], ab_src, kAbBytes, &ms.bc_full[st]);
            bulk_load(ms.hc[st], hc_ws + (int64_t)ld.im.unit * kHcFloats, kHcBytes, &ms.bc_full[st]);
            tma_load_4d(dB, &tm_b16, &ms.bc_full[st], 0, g, ld.j * T, b);
            tma_load_4d(dB + kAtom, &tm_b16, &ms.bc_full[st], 64, g, ld.j * T, b);
            tma_load_4d(dC, &tm_c16, &ms.bc_full[st], 0, g, ld.j * T, b);
            tma_load_4d(dC + kAtom, &tm_c16, &ms.bc_full[st], 64, g, ld.j * T, b);
            tma_load_4d(smem + kOffX8 + st * kXBytes, &tm_x, &ms.bc_full[st], 0, h, ld.j * T, b);   // rows past the end read as 0
            step(ld);
            progress = true;
          }
        }
        if (mbar_test_wait(&ms.y_full, stc.it & 1)) {
          tma_store_4d(&tm_out, smem + kOffY, 0, stc.im.unit % a.nheads, stc.j * T, stc.im.unit / a.nheads);
          bulk_commit();
          bulk_wait_read<0>();
          mbar_arrive(&ms.y_empty);
          step(stc);
          progress = true;
        }
        if (progress) {
          t_last = clock64();
        } else {
          __nanosleep(64);
          if (clock64() - t_last > kWaitBudgetCycles) { atomicCAS(status, 0, QB_ERR_TIMEOUT); break; }   // bounded like every wait
        }
      }
      bulk_wait_all<0>();   // every store is complete before the CTA exits
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && plan.total > 0) {
      constexpr uint32_t id_cb = make_idesc(1, 0, 0, 0, 0, 128, 128);  // C (K-major) x B (K-major)
      constexpr uint32_t id_kn = make_idesc(1, 0, 0, 0, 1, 128, 64);   // K-major (or tensor-memory) A x MN-major B
      constexpr uint32_t id_mn = make_idesc(1, 0, 0, 1, 1, 128, 64);   // MN-major A x MN-major B
      // descriptor words of every operand tile, built once (stage 1 of B / C is 2 atoms further)
      const SmemDesc dBk = make_smem_desc2(smem_u32(smem + kOffB16), 16, 1024, kSwizzle128B);      // B, K-major (CB)
      const SmemDesc dBm = make_smem_desc2(smem_u32(smem + kOffB16), kAtom, 1024, kSwizzle128B);   // B, MN-major A of GEMM4
      const SmemDesc dCk = make_smem_desc2(smem_u32(smem + kOffC16), 16, 1024, kSwizzle128B);      // C, K-major
      const SmemDesc dXraw = make_smem_desc2(smem_u32(smem + kOffXraw), 16, 1024, kSwizzle128B);
      const SmemDesc dXw = make_smem_desc2(smem_u32(smem + kOffXw), 16, 1024, kSwizzle128B);
      const SmemDesc dS16 = make_smem_desc2(smem_u32(smem + kOffS16), 16, 1024, kSwizzle128B);
      bool ok = mbar_wait_spin(&ms.bc_full[0], 0, status, QB_ERR_TIMEOUT);
      if (ok) {
        tc_fence_after_sync();
        issue_gemm<false, false>(tmem + kColCB, dCk, dBk, id_cb);
        umma_commit(&ms.cb_ready);
      }
      int it = 0;
      for (int ii = 0; ii < plan.n_items && ok; ++ii) {
        const Item im = get_item(plan, ii, nb);
        for (int j = im.jb; j < im.je; ++j, ++it) {
          const int st = it & 1;
          const uint32_t ph = it & 1;
          const bool use_d1 = j > im.jb || im.has_init;
          // GEMM2(it): D1[it & 1] = C(it) S_prev.  s16_ready says that the fp16 state entering this block is in shared
          // memory (nothing to multiply when a pair starts from the zero state), that the compute warps have read the
          // S accumulator of the previous block (GEMM4 below overwrites it) and, by program order, D1[it & 1] of two
          // blocks ago.
          ok = mbar_wait_spin(&ms.s16_ready, ph, status, QB_ERR_TIMEOUT);
          if (!ok) break;
          tc_fence_after_sync();
          if (use_d1) issue_gemm<false, true>(tmem + (st ? kColD1b : kColD1), desc_advance(dCk, st * 2 * kAtom), dS16, id_kn);
          umma_commit(&ms.d1_ready);   // the fp16 state tile may be rewritten once this has fired
          // GEMM4(it): local state of the block, S = B^T (x w)
          ok = mbar_wait_spin(&ms.xops_ready, ph, status, QB_ERR_TIMEOUT);
          if (!ok) break;
          tc_fence_after_sync();
          issue_gemm<true, true>(tmem + kColS, desc_advance(dBm, st * 2 * kAtom), dXw, id_mn);
          umma_commit(&ms.s_ready);
          // GEMM3(it): D2 = Lm X, Lm from tensor memory.  lm_ready also says (program order of the compute warps) that
          // the output step of the previous block has read D2.
          ok = mbar_wait_spin(&ms.lm_ready, ph, status, QB_ERR_TIMEOUT);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_f16_ta(tmem + kColD2, tmem + kColLm + ks * 8, desc_advance(dXraw, ks * 2048), id_kn, ks != 0 ? 1u : 0u);
          umma_commit(&ms.y_ready);
          if (it + 1 < plan.total) {
            // C.B^T of the next block (of this pair or the next one): the compute warps have finished reading CB(it)
            const int sn = (it + 1) & 1;
            ok = mbar_wait_spin(&ms.bc_full[sn], ((it + 1) >> 1) & 1, status, QB_ERR_TIMEOUT);
            if (!ok) break;
            tc_fence_after_sync();
            issue_gemm<false, false>(tmem + kColCB, desc_advance(dCk, sn * 2 * kAtom), desc_advance(dBk, sn * 2 * kAtom), id_cb);
            umma_commit(&ms.cb_ready);
          }
          // Release the B/C stage of this block last.  Its readers were CB(it), GEMM2(it) and GEMM4(it); releasing it
          // earlier let the refill run concurrently with the remaining MMAs of the block, and with that timing results
          // were not reproducible from run to run.  The refill has a whole block of slack, so nothing is lost here.
          umma_commit(&ms.bc_empty[st]);
        }
      }
    }
  } else if (warp == 0 || warp == 2) {
    // ---------------- x operands ----------------
    // x(k) -> the two fp16 operand tiles: raw (B of GEMM3) and scaled by w_l = dt_l 2^(r - a_l) = 2^(r - bk_l - lscb) (B of
    // GEMM4; 0 where dt_l = 0).  This needs no tensor memory, so one warp outside the 16 compute warps does it a block
    // ahead of them: the tiles may be rewritten once GEMM4 and GEMM3 of the previous block are complete, and the
    // deadlines (GEMM4 / GEMM3 of this block) lie a whole Lm phase later.  Two warps share the tile, 64 rows each; both
    // sit on the scheduler whose compute warps have the least Lm work.
    const int xhalf = warp == 2 ? 8 : 0;
    int it = 0;
    bool ok = true;
    for (int ii = 0; ii < plan.n_items && ok; ++ii) {
      const Item im = get_item(plan, ii, nb);
      for (int j = im.jb; j < im.je; ++j, ++it) {
        const int st = it & 1;
        ok = mbar_wait(&ms.bc_full[st], (it >> 1) & 1, status, QB_ERR_TIMEOUT);                 // x tile, vectors, constants
        if (ok && it > 0) ok = mbar_wait(&ms.s_ready, (it - 1) & 1, status, QB_ERR_TIMEOUT);     // GEMM4 of the previous block
        if (ok && it > 0) ok = mbar_wait(&ms.y_ready, (it - 1) & 1, status, QB_ERR_TIMEOUT);     // GEMM3 of the previous block
        if (!ok) break;
        const float* av = ms.ab[st];
        const float base = av[T - 1] - ms.hc[st][kHcLscb];
        const uint8_t* xs = smem + kOffX8 + st * kXBytes;
        const int piece = lane & 3;
#pragma unroll 4
        for (int i = xhalf; i < xhalf + 8; ++i) {
          const int r = 8 * i + (lane >> 2);      // a warp reads 512 contiguous bytes of the tile per step
          const uint4 xq = *reinterpret_cast<const uint4*>(xs + r * P + piece * 16);
          const uint32_t xwd[4] = {xq.x, xq.y, xq.z, xq.w};
          const __half2 w2 = __float2half2_rn(fast_exp2(base - av[T + r]));
          uint8_t* rowp_raw = smem + kOffXraw + r * 128;
          uint8_t* rowp_w = smem + kOffXw + r * 128;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            __half2 r0, r1, r2, r3;
            s8x4_to_h2x2(xwd[2 * c], r0, r1);
            s8x4_to_h2x2(xwd[2 * c + 1], r2, r3);
            const int chunk = ((2 * piece + c) ^ (r & 7)) << 4;
            *reinterpret_cast<uint4*>(rowp_raw + chunk) = make_uint4(h2_bits(r0), h2_bits(r1), h2_bits(r2), h2_bits(r3));
            *reinterpret_cast<uint4*>(rowp_w + chunk) = make_uint4(h2_bits(__hmul2(r0, w2)), h2_bits(__hmul2(r1, w2)),
                                                                   h2_bits(__hmul2(r2, w2)), h2_bits(__hmul2(r3, w2)));
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ms.xops_ready);
      }
    }
  } else if (warp >= 4) {
    // ---------------- compute warps ----------------
    const int cw = warp - 4;
    const int q = warp & 3;            // TMEM lane quarter this warp may touch
    const int sub = cw >> 2;           // quarter of the columns: channels 16 sub .. 16 sub + 15, chunk sub of Lm
    const int row = q * 32 + lane;
    const int ctid = threadIdx.x - kLead;
    const uint32_t tlane = (uint32_t)(q * 32) << 16;
    const int sw = row & 7;
    const bool lead = (threadIdx.x == kLead);
    auto gsync = [&]() { asm volatile("bar.sync 1, 512;" ::: "memory"); };
    auto gand = [&](uint32_t ok) -> bool {   // group barrier that ANDs a flag: a timed-out wait makes all warps leave together
      uint32_t r;
      asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 512, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                   : "=r"(r) : "r"(ok) : "memory");
      return r != 0;
    };
    // One thread polls the mbarrier(s), the others park at the group's hardware barrier.
    auto gwait = [&](uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1) -> bool {
      uint32_t ok = 1;
      if (lead) {
        ok = mbar_wait(b0, p0, status, QB_ERR_TIMEOUT) ? 1u : 0u;
        if (ok && b1 != nullptr) ok = mbar_wait(b1, p1, status, QB_ERR_TIMEOUT) ? 1u : 0u;
      }
      return gand(ok);
    };
    float s_reg[16];
    auto store_s16 = [&]() {   // fp16 copy of this thread's 16 state values: row n, channels 16 sub .. (MN-major B of GEMM2)
      uint8_t* dst = smem + kOffS16 + row * 128;
#pragma unroll
      for (int u = 0; u < 2; ++u)
        *reinterpret_cast<uint4*>(dst + (((2 * sub + u) ^ sw) << 4)) =
            make_uint4(pack_h2(s_reg[8 * u], s_reg[8 * u + 1]), pack_h2(s_reg[8 * u + 2], s_reg[8 * u + 3]),
                       pack_h2(s_reg[8 * u + 4], s_reg[8 * u + 5]), pack_h2(s_reg[8 * u + 6], s_reg[8 * u + 7]));
    };
    constexpr bool d_per_channel = kDPerChannel;
    int it = 0;
    bool ok = true;
    for (int ii = 0; ii < plan.n_items && ok; ++ii) {
      const Item im = get_item(plan, ii, nb);
      const int b = im.unit / a.nheads, h = im.unit % a.nheads, g = h / hpg;
      const int8_t* xrow_base = a.x + (int64_t)b * a.x_sb + (int64_t)h * a.x_sh + 16 * sub;
      // The constants of the pair arrive with every block's stage, so nothing has to be set up here for a pair that
      // starts from the zero state: no barrier, no global loads, no cold code.
      if (im.has_init) {
        // the state after the head part of this pair, published by the previous CTA early in its life
        uint32_t got = 1;
        if (lead) {
          const long long t0 = clock64();
          for (;;) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + blockIdx.x) : "memory");
            if (v != 0) break;
            __nanosleep(256);
            if (clock64() - t0 > kWaitBudgetCycles) { atomicCAS(status, 0, QB_ERR_TIMEOUT); got = 0; break; }
          }
        }
        ok = gand(got);
        if (!ok) break;
        const float4* src = reinterpret_cast<const float4*>(handoff + (int64_t)blockIdx.x * kHandoffFloats);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float4 f = __ldcg(src + v * kCompute + ctid);
          s_reg[4 * v] = f.x; s_reg[4 * v + 1] = f.y; s_reg[4 * v + 2] = f.z; s_reg[4 * v + 3] = f.w;
        }
        store_s16();   // GEMM2 of the previous block has completed: the state step that followed it waited for d1_ready
        fence_proxy_async_smem();
        gsync();
      } else {
#pragma unroll
        for (int t = 0; t < 16; ++t) s_reg[t] = 0.0f;
      }
      // s16_ready also tells the MMA issuer that the S accumulator of the previous block has been read: every warp did
      // that before the barrier that opened its output step.
      if (lead) mbar_arrive(&ms.s16_ready);

      for (int j = im.jb; j < im.je; ++j, ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1;
        const bool use_d1 = j > im.jb || im.has_init;
        const int l = j * T + row;
        // The x operands of this block are written by warp 0.  Here: the vectors and constants have landed (bc_full) and
        // C.B^T of this block is in tensor memory (cb_ready).
        ok = gwait(&ms.bc_full[st], (it >> 1) & 1, &ms.cb_ready, ph);
        if (!ok) break;
        // The vectors and constants of the previous block are read up to the end of its output step, which every warp
        // has left by now; its B / C / x tiles were released by the MMA issuer.
        if (lead && it > 0) mbar_arrive(&ms.ab_empty[(it - 1) & 1]);
        const float* av = ms.ab[st];
        const float* hc = ms.hc[st];
        const float sC = hc[kHcSC], dfold = hc[kHcDfold];
        const float a_row = av[row];
        const float r_tot = av[T - 1];
        const float e_out = use_d1 ? sC * fast_exp2(a_row) : 0.0f;   // weight of the carried-in term in the output

        // ================= P2: Lm[t, s] = CB[t, s] 2^(a_t - bk_s) for s <= t (+ D on the diagonal), chunk sub =============
        // Written as packed fp16 into its own tensor-memory columns, which GEMM3 of the previous block has finished
        // reading (its output step waited for y_ready).
        tc_fence_after_sync();
        {
          // Work split inside a lane quarter q (rows 32q .. 32q + 31, four warps): the chunks c < q lie below the
          // diagonal and cost two multiplies per element, the chunk c = q holds the diagonal and costs an ex2 and the
          // mask per element, the chunks c > q are zero.  Warp `sub` takes the whole chunk c = sub when it is below the
          // diagonal, and every warp takes eight columns (8 sub .. 8 sub + 7) of the diagonal chunk, so that the
          // expensive chunk is shared by four warps instead of being one warp's critical path.
          uint32_t dg[8];
          tmem_ld_32x8(tmem + tlane + kColCB + 32 * q + 8 * sub, dg);
          if (sub < q) {
            const int c = sub;
            uint32_t cb[32], o[16];
            tmem_ld_32x32(tmem + tlane + kColCB + 32 * c, cb);
            // chunk below the diagonal: 2^(a_t - bk_s) = 2^(a_t - m) * ec[s], m = a at the end of chunk c
            const float e_row = fast_exp2(a_row - av[32 * c + 31]);
            tmem_ld_wait();
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
            tmem_st16(tmem + tlane + kColLm + 16 * c, o);
          } else {
            tmem_ld_wait();
            if (sub > q) {  // this warp's own chunk is entirely above the diagonal
              uint32_t z[16];
#pragma unroll
              for (int u = 0; u < 16; ++u) z[u] = 0u;
              tmem_st16(tmem + tlane + kColLm + 16 * sub, z);
            }
          }
          {
            // eight columns of the diagonal chunk: exact exponent per element, the k <= m mask (k - 32q <= lane), and the
            // skip weight D on the diagonal itself (y = sx (Lm + D I) x) when D has one value per head
            const float4* bk4 = reinterpret_cast<const float4*>(av + T + 32 * q + 8 * sub);
            uint32_t o[4];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const float4 bb = bk4[u];
              const int t0 = 8 * sub + 4 * u;
              float e0 = __uint_as_float(dg[4 * u + 0]) * fast_exp2(a_row - bb.x);
              float e1 = __uint_as_float(dg[4 * u + 1]) * fast_exp2(a_row - bb.y);
              float e2 = __uint_as_float(dg[4 * u + 2]) * fast_exp2(a_row - bb.z);
              float e3 = __uint_as_float(dg[4 * u + 3]) * fast_exp2(a_row - bb.w);
              e0 = t0 + 0 < lane ? e0 : (t0 + 0 == lane ? e0 + dfold : 0.0f);
              e1 = t0 + 1 < lane ? e1 : (t0 + 1 == lane ? e1 + dfold : 0.0f);
              e2 = t0 + 2 < lane ? e2 : (t0 + 2 == lane ? e2 + dfold : 0.0f);
              e3 = t0 + 3 < lane ? e3 : (t0 + 3 == lane ? e3 + dfold : 0.0f);
              o[2 * u] = pack_h2(e0, e1);
              o[2 * u + 1] = pack_h2(e2, e3);
            }
            tmem_st4(tmem + tlane + kColLm + 16 * q + 4 * sub, o);
          }
        }
        tmem_st_wait();
        tc_fence_before_sync();
        gsync();
        if (lead) mbar_arrive(&ms.lm_ready);

        // ================= P3: state: s <- 2^r s + sB sx S_loc ; publish its fp16 copy for the next block ==============
        // s_ready: GEMM4(it) done.  d1_ready: GEMM2(it) done, so the fp16 state tile it read may be rewritten.
        ok = gwait(&ms.s_ready, ph, &ms.d1_ready, ph);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t d1[16];   // C.S of this block, complete since GEMM2 (d1_ready): fetched here, one TMEM round trip early
        {
          const float dec = fast_exp2(r_tot);
          uint32_t sl[16];
          tmem_ld_32x16(tmem + tlane + kColS + 16 * sub, sl);
          if (use_d1) tmem_ld_32x16(tmem + tlane + (st ? kColD1b : kColD1) + 16 * sub, d1);
          tmem_ld_wait();
          const float4* sb4 = reinterpret_cast<const float4*>(hc + kHcSbx + 16 * sub);
#pragma unroll
          for (int t4 = 0; t4 < 4; ++t4) {
            const float4 sc = sb4[t4];
            s_reg[4 * t4 + 0] = fmaf(dec, s_reg[4 * t4 + 0], sc.x * __uint_as_float(sl[4 * t4 + 0]));
            s_reg[4 * t4 + 1] = fmaf(dec, s_reg[4 * t4 + 1], sc.y * __uint_as_float(sl[4 * t4 + 1]));
            s_reg[4 * t4 + 2] = fmaf(dec, s_reg[4 * t4 + 2], sc.z * __uint_as_float(sl[4 * t4 + 2]));
            s_reg[4 * t4 + 3] = fmaf(dec, s_reg[4 * t4 + 3], sc.w * __uint_as_float(sl[4 * t4 + 3]));
          }
        }
        tc_fence_before_sync();
        if (j + 1 < im.je) {   // the next item prepares the tile itself (zero state or a state from another CTA)
          store_s16();
          fence_proxy_async_smem();
        }
        // One barrier closes the state step and opens the output step: the polling thread waits for GEMM3 of this block
        // (which never depends on the arrival below) and for the store of the previous block to have read the staging
        // tile, all warps meet, and then the fp16 state is announced to the MMA issuer.
        ok = gwait(&ms.y_ready, ph, it > 0 ? &ms.y_empty : nullptr, (it - 1) & 1);
        if (lead && j + 1 < im.je) mbar_arrive(&ms.s16_ready);
        if (!ok) break;

        // ================= P4: y(j) = sC 2^(a_m) D1 + sx (D2 + D x) ======================================================
        tc_fence_after_sync();
        {
          uint4 xq = make_uint4(0, 0, 0, 0);
          if (d_per_channel && l < a.seqlen) xq = ldg_nc_now(xrow_base + (int64_t)l * a.x_sl);   // own 16 channels of x
          uint32_t d2[16];
          tmem_ld_32x16(tmem + tlane + kColD2 + 16 * sub, d2);
          tmem_ld_wait();
          tc_fence_before_sync();
          const float4* sx4 = reinterpret_cast<const float4*>(hc + kHcSx + 16 * sub);
          const uint32_t xwd[4] = {xq.x, xq.y, xq.z, xq.w};
          uint4 c2[2];
#pragma unroll
          for (int t8 = 0; t8 < 2; ++t8) {
            uint32_t o[4];
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              const int t4 = 2 * t8 + v;
              const float4 sx = sx4[t4];
              float y0 = sx.x * __uint_as_float(d2[4 * t4 + 0]);
              float y1 = sx.y * __uint_as_float(d2[4 * t4 + 1]);
              float y2 = sx.z * __uint_as_float(d2[4 * t4 + 2]);
              float y3 = sx.w * __uint_as_float(d2[4 * t4 + 3]);
              if (use_d1) {
                y0 = fmaf(e_out, __uint_as_float(d1[4 * t4 + 0]), y0);
                y1 = fmaf(e_out, __uint_as_float(d1[4 * t4 + 1]), y1);
                y2 = fmaf(e_out, __uint_as_float(d1[4 * t4 + 2]), y2);
                y3 = fmaf(e_out, __uint_as_float(d1[4 * t4 + 3]), y3);
              }
              if (d_per_channel) {
                const float4 dx = reinterpret_cast<const float4*>(hc + kHcDsx + 16 * sub)[t4];
                __half2 h01, h23;
                s8x4_to_h2x2(xwd[t4], h01, h23);
                const float2 x01 = __half22float2(h01), x23 = __half22float2(h23);
                y0 = fmaf(dx.x, x01.x, y0); y1 = fmaf(dx.y, x01.y, y1);
                y2 = fmaf(dx.z, x23.x, y2); y3 = fmaf(dx.w, x23.y, y3);
              }
              o[2 * v] = pack_h2(y0, y1);
              o[2 * v + 1] = pack_h2(y2, y3);
            }
            c2[t8] = make_uint4(o[0], o[1], o[2], o[3]);
          }
          // This thread's 32 bytes of the row go to the staging tile (128-byte swizzle, as the tensor map expects); the
          // tile is free: the barrier that opened this step also waited for the previous block's store to have read it.
          {
            uint8_t* yrow = smem + kOffY + row * 128;
            *reinterpret_cast<uint4*>(yrow + (((2 * sub) ^ sw) << 4)) = c2[0];
            *reinterpret_cast<uint4*>(yrow + (((2 * sub + 1) ^ sw) << 4)) = c2[1];
            fence_proxy_async_smem();
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&ms.y_full);
        }
        if (!ok) break;
      }
      if (!ok) break;

      if (im.publish) {
        // ---- the state after the head part of a pair: to the CTA that runs the rest of it ------------------------
        float4* dst = reinterpret_cast<float4*>(handoff + (int64_t)(blockIdx.x + 1) * kHandoffFloats);
#pragma unroll
        for (int v = 0; v < 4; ++v)
          __stcg(dst + v * kCompute + ctid, make_float4(s_reg[4 * v], s_reg[4 * v + 1], s_reg[4 * v + 2], s_reg[4 * v + 3]));
        __threadfence();
        gsync();
        if (lead) {
          const int one = 1;
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flags + blockIdx.x + 1), "r"(one) : "memory");
        }
      } else {
        // ---- final state -> int8 after the last block ------------------------------------------------------------
        int hg = 0;
        if (a.grouped) hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, h % hpg);
        int8_t* fs = a.final_states + ((int64_t)b * a.nheads + h) * P * N + row;
#pragma unroll
        for (int t = 0; t < 16; ++t) {  // fully unrolled: s_reg must never be indexed dynamically
          const int p = 16 * sub + t;
          float ss;
          if (!a.grouped) {
            ss = ms.hc[(it - 1) & 1][kHcStateScale];   // the stage of the item's last block is still in place
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
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// B, C int8 (B, L, G, N) -> fp16 [B][L][G][N] contiguous (values unchanged).
__device__ __forceinline__ void ssd_widen_bc(int64_t block, const int8_t* __restrict__ Bq, int64_t B_sb, int64_t B_sl, int64_t B_sg,
                                             const int8_t* __restrict__ Cq, int64_t C_sb, int64_t C_sl, int64_t C_sg,
                                             __half* __restrict__ B16, __half* __restrict__ C16, int batch, int seqlen, int ngroups) {
  const int64_t idx = block * blockDim.x + threadIdx.x;  // one 16-element piece
  const int pieces = N / 16;
  const int64_t total = (int64_t)batch * seqlen * ngroups * pieces;
  if (idx >= total) return;
  const int pc = (int)(idx % pieces);
  const int gg = (int)((idx / pieces) % ngroups);
  const int l = (int)((idx / ((int64_t)pieces * ngroups)) % seqlen);
  const int bb = (int)(idx / ((int64_t)pieces * ngroups * seqlen));
  auto widen = [&](const int8_t* src, __half* dst) {
    const uint4 v = ld_act(reinterpret_cast<const uint4*>(src));     // conv output: an activation, read past L1
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
__device__ __forceinline__ void ssd_dt(int64_t block, const qb_ssd_args& a, float* __restrict__ ab_ws, float* __restrict__ hc_ws, int nb,
                                       int* __restrict__ flags, int nflags) {
  if (block == 0)   // the hand-off flags of the main kernel, which follows on the same stream
    for (int i = threadIdx.x; i < nflags; i += blockDim.x) flags[i] = 0;
  const int64_t unit = block * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t units = (int64_t)a.batch * a.nheads * nb;
  if (unit >= units) return;
  // heads vary fastest across the warps of a block: dt is (batch, seqlen, nheads) with the head innermost, so the eight
  // warps of a block read neighbouring bytes of the same sectors
  const int h = (int)(unit % a.nheads);
  const int j = (int)((unit / a.nheads) % nb);
  const int b = (int)(unit / ((int64_t)nb * a.nheads));
  const int g = h / (a.nheads / a.ngroups);
  const float A2 = -__expf((*a.A_scale) * (float)a.A_log[h]) * 1.4426950408889634f;
  const float s_dt = *a.dt_scale;
  const float bias = a.dt_bias != nullptr ? __half2float(static_cast<const __half*>(a.dt_bias)[h]) : 0.0f;
  const float sBg = a.grouped ? a.B_scale[g] : a.B_scale[0], sCg = a.grouped ? a.C_scale[g] : a.C_scale[0];
  const float lscb = fast_log2(sCg * sBg);
  if (j == 0) {
    // the constants of this (batch, head) pair: two channels per lane, the scalars by lane 0
    float* hc = hc_ws + ((int64_t)b * a.nheads + h) * kHcFloats;
    const int hpg = a.nheads / a.ngroups;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int p = lane + 32 * i;
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
      hc[kHcSx + p] = sx;
      hc[kHcDsx + p] = dv * sx;
      hc[kHcSbx + p] = sBg * sx;
    }
    if (lane == 0) {
      hc[kHcDfold] = (a.D != nullptr && !a.D_has_hdim) ? (*a.D_scale) * (float)a.D[h] : 0.0f;
      hc[kHcSC] = sCg;
      hc[kHcLscb] = lscb;
      hc[kHcStateScale] = a.grouped ? 1.0f : a.ssm_state_scale[0];
    }
  }
  const int8_t* dtp = a.dt + (int64_t)b * a.dt_sb + h;
  float dt[4], cs[4];
  float run = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int l = j * T + lane * 4 + i;
    float v = 0.0f;
    if (l < a.seqlen) {
      v = fmaf(s_dt, (float)ld_act(dtp + (int64_t)l * a.dt_sl), bias);
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
  float* dst = ab_ws + (((int64_t)b * a.nheads + h) * nb + j) * (kAbVecs * T);
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

// Both preparation steps in one launch (256 threads per block): the first widen_blocks blocks widen B and C, the rest
// evaluate the per-block vectors, eight (batch, head, block) units per block.
__global__ void __launch_bounds__(256) ssd_prep_kernel(qb_ssd_args a, __half* __restrict__ B16, __half* __restrict__ C16,
                                                       float* __restrict__ ab_ws, float* __restrict__ hc_ws, int nb,
                                                       int* __restrict__ flags, int nflags, int widen_blocks) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the main kernel may start its prologue
  asm volatile("griddepcontrol.wait;" ::: "memory");                // this kernel's inputs come from whatever ran before it
  if ((int)blockIdx.x < widen_blocks)
    ssd_widen_bc(blockIdx.x, a.Bm, a.B_sb, a.B_sl, a.B_sg, a.Cm, a.C_sb, a.C_sl, a.C_sg, B16, C16, a.batch, a.seqlen, a.ngroups);
  else
    ssd_dt((int64_t)blockIdx.x - widen_blocks, a, ab_ws, hc_ws, nb, flags, nflags);
}

int64_t align256l(int64_t v) { return (v + 255) & ~(int64_t)255; }
constexpr int kMaxCtas = 256;   // hand-off slots in the workspace (one per CTA of the persistent kernel)

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
  return 2 * align256l((int64_t)B * L * G * N * 2) + align256l((int64_t)B * H * nb * kAbVecs * T * 4) +
         align256l((int64_t)kMaxCtas * kHandoffFloats * 4) + align256l(kMaxCtas * 4) + align256l((int64_t)B * H * kHcBytes);
}

int ssd_tc_launch(const qb_ssd_args* a, cudaStream_t st) {
  const int64_t half_bytes = align256l((int64_t)a->batch * a->seqlen * a->ngroups * N * 2);
  const int nb = (int)ceil_div(a->seqlen, T);
  const int64_t ab_bytes = align256l((int64_t)a->batch * a->nheads * nb * kAbVecs * T * 4);
  char* ws = static_cast<char*>(a->workspace);
  __half* B16 = reinterpret_cast<__half*>(ws);
  __half* C16 = reinterpret_cast<__half*>(ws + half_bytes);
  float* ab_ws = reinterpret_cast<float*>(ws + 2 * half_bytes);
  float* handoff = reinterpret_cast<float*>(ws + 2 * half_bytes + ab_bytes);
  int* flags = reinterpret_cast<int*>(ws + 2 * half_bytes + ab_bytes + align256l((int64_t)kMaxCtas * kHandoffFloats * 4));
  float* hc_ws = reinterpret_cast<float*>(reinterpret_cast<char*>(flags) + align256l(kMaxCtas * 4));
  {
    const int64_t pieces = (int64_t)a->batch * a->seqlen * a->ngroups * (N / 16);
    const int64_t units = (int64_t)a->batch * a->nheads * nb;
    const int widen_blocks = (int)ceil_div(pieces, 256);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(widen_blocks + ceil_div(units, 8)));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // its launch overlaps the tail of the kernel before it
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QB_CUDA_OK(cudaLaunchKernelEx(&cfg, ssd_prep_kernel, *a, B16, C16, ab_ws, hc_ws, nb, flags, (int)kMaxCtas, widen_blocks));
  }
  CUtensorMap tb, tcm;
  const uint64_t dims[4] = {(uint64_t)N, (uint64_t)a->ngroups, (uint64_t)a->seqlen, (uint64_t)a->batch};
  const uint64_t strides[3] = {(uint64_t)N * 2, (uint64_t)a->ngroups * N * 2, (uint64_t)a->seqlen * a->ngroups * N * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
  int rc = encode_tmap_f16_4d(&tb, B16, dims, strides, box);
  if (rc != QB_OK) return rc;
  rc = encode_tmap_f16_4d(&tcm, C16, dims, strides, box);
  if (rc != QB_OK) return rc;
  CUtensorMap tx, tout;
  {
    // x int8 (P, H, L, B): one 128-row x 64-byte tile per block, unswizzled
    const uint64_t xd[4] = {(uint64_t)P, (uint64_t)a->nheads, (uint64_t)a->seqlen, (uint64_t)a->batch};
    const uint64_t xs[3] = {(uint64_t)a->x_sh, (uint64_t)a->x_sl, (uint64_t)a->x_sb};
    const uint32_t xb[4] = {(uint32_t)P, 1, (uint32_t)T, 1};
    rc = encode_tmap_4d(&tx, false, false, a->x, xd, xs, xb);
    if (rc != QB_OK) return rc;
    // out fp16 (P, H, L, B) contiguous: one 128-row x 64-channel tile per store, 128-byte swizzle on the shared-memory side
    const uint64_t od[4] = {(uint64_t)P, (uint64_t)a->nheads, (uint64_t)a->seqlen, (uint64_t)a->batch};
    const uint64_t os[3] = {(uint64_t)P * 2, (uint64_t)a->nheads * P * 2, (uint64_t)a->seqlen * a->nheads * P * 2};
    const uint32_t ob[4] = {(uint32_t)P, 1, (uint32_t)T, 1};
    rc = encode_tmap_4d(&tout, true, true, a->out, od, os, ob);
    if (rc != QB_OK) return rc;
  }
  static bool attr_set[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 64 || !attr_set[dev]) {
    QB_CUDA_OK(cudaFuncSetAttribute(ssd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    QB_CUDA_OK(cudaFuncSetAttribute(ssd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    if (dev < 64) attr_set[dev] = true;
  }
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "device status word unavailable");
  // One CTA per SM.  With at least as many (batch, head) pairs as CTAs the block list is cut into equal ranges (a range
  // is then at least one whole pair long, which is what the head-first / tail-last order of the kernel relies on);
  // with fewer, every CTA takes one whole pair.
  const int pairs = a->batch * a->nheads;
  const int ctas = std::min(std::min(sm_count(), kMaxCtas), pairs);
  const int split = pairs >= ctas && ctas == std::min(sm_count(), kMaxCtas) ? 1 : 0;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may begin while ssd_prep_kernel drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* ab_c = ab_ws;
    const float* hc_c = hc_ws;
    const int early = early_overlap() ? 1 : 0;
    if (a->D != nullptr && a->D_has_hdim) {
      QB_CUDA_OK(cudaLaunchKernelEx(&cfg, ssd_tc_kernel<true>, tb, tcm, tx, tout, *a, ab_c, hc_c, handoff, flags, split, status, early));
    } else {
      QB_CUDA_OK(cudaLaunchKernelEx(&cfg, ssd_tc_kernel<false>, tb, tcm, tx, tout, *a, ab_c, hc_c, handoff, flags, split, status, early));
    }
  }
  return QB_OK;
}

}  // namespace qb
