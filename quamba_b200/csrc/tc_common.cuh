// Blackwell (sm_100a) building blocks used by the tensor-core kernels: mbarriers with bounded
// waits, TMA tile loads (never multicast), TMEM allocation, tcgen05.mma / commit / ld, and the
// shared-memory matrix descriptors.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)
#include "common.cuh"

namespace qb {

// Device status word: a kernel whose bounded wait expires stores a code here and unwinds; the
// host reads it with qb_read_device_status().  0 = ok.  Kernels receive its address as an
// argument (device_status_ptr(), one word per device, owned by lib.cu).
int* device_status_ptr();

#ifdef __CUDACC__
namespace tc {

constexpr long long kWaitBudgetCycles = 2000000000LL;  // ~1 s at B200 clocks

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false (and a status code) if the phase does not complete within the budget.
// A waiting thread backs off between polls so that it does not compete for issue slots and for the
// shared-memory pipeline with the warps that are doing the work it waits for.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(32);
    }
    if (clock64() - t0 > kWaitBudgetCycles) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

// The same without the back-off, for a thread whose wake-up latency is on the critical path (an MMA issuer: one thread,
// and try_wait itself suspends it for a while, so it does not spin hot).
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitBudgetCycles) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

// 2-D TMA tile load, completion on an mbarrier of this CTA.  x = innermost coordinate.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Plain (untiled) bulk copies, 16-byte aligned addresses and size.  The load completes on an mbarrier of this CTA;
// stores are tracked by bulk groups of the issuing thread.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still read their shared-memory source / are still in flight.
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// The arrive happens when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.  kind: i8 (int32 accumulate) or f16 (fp32).
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors -------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address, leading / stride byte offsets (all in
// 16-byte units), descriptor version 1 (Blackwell), swizzle mode in bits 61..63.
enum Swizzle : uint64_t { kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6 };

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, Swizzle sw) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)sw << 61;
  return d;
}

// The same descriptor as two 32-bit words.  The issuing thread is a single warp whose dependent instructions cost
// several cycles each, and at 32 to 128 cycles of tensor work per tcgen05.mma a dozen instructions of descriptor
// arithmetic per MMA leave the tensor pipe waiting for the issuer (measured: 116 to 310 cycles per MMA with
// descriptors built per instruction, against 48 to 128 with the form below).  So: build the words once per tile,
// advance along K with ONE 32-bit add on the low word (the start-address field sits in bits 0..13 and never carries
// while the address stays inside shared memory), and let the asm block pair the words into the 64-bit operand.
struct SmemDesc { uint32_t lo, hi; };
__device__ __forceinline__ SmemDesc make_smem_desc2(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, Swizzle sw) {
  SmemDesc d;
  d.lo = ((smem_addr >> 4) & 0x3fff) | (((lbo_bytes >> 4) & 0x3fff) << 16);
  d.hi = ((sbo_bytes >> 4) & 0x3fff) | (1u << 14) | ((uint32_t)sw << 29);
  return d;
}
// byte_offset must be a multiple of 16
__device__ __forceinline__ SmemDesc desc_advance(SmemDesc d, uint32_t byte_offset) { d.lo += byte_offset >> 4; return d; }

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, SmemDesc a, SmemDesc b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, SmemDesc a, SmemDesc b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from tensor memory (fp16 packed two per 32-bit column: eight columns per K = 16 step)
__device__ __forceinline__ void umma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, SmemDesc b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor (32 bit).  c_format: 1 = f32, 2 = s32.  a/b format: kind::f16: 0 = f16,
// 1 = bf16; kind::i8: 0 = u8, 1 = s8.  major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_format, uint32_t a_format, uint32_t b_format, uint32_t a_major,
                                                  uint32_t b_major, uint32_t m, uint32_t n) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | (a_major << 15) | (b_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

}  // namespace tc
#endif  // __CUDACC__

// Host: encode a 2-D row-major byte tensor map (rows x cols bytes, row pitch in bytes) with a
// (box_rows x box_cols) box and 128-byte swizzle.  Returns QB_OK or an error.
int encode_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                      uint32_t box_rows, uint32_t box_cols);
// Host: 4-D fp16 tensor map, dims / box innermost first, strides (bytes) for dims 1..3, 128-byte swizzle.
int encode_tmap_f16_4d(CUtensorMap* out, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                       const uint32_t box[4]);
// Host: 4-D tensor map of fp16 or byte elements (dims / strides / box counted in elements resp. bytes as above), with
// 128-byte swizzle or none.
int encode_tmap_4d(CUtensorMap* out, bool f16, bool swizzle128, const void* base, const uint64_t dims[4],
                   const uint64_t strides_bytes[3], const uint32_t box[4]);

}  // namespace qb
