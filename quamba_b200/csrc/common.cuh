// Shared host/device helpers for the quamba_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/quamba_b200.h"

namespace qb {

// ---- host-side error reporting --------------------------------------------------------------
void set_error(const char* fmt, ...);

#define QB_REQUIRE(cond, code, ...)        \
  do {                                     \
    if (!(cond)) {                         \
      ::qb::set_error(__VA_ARGS__);        \
      return (code);                       \
    }                                      \
  } while (0)

#define QB_CUDA_OK(expr)                                                         \
  do {                                                                           \
    cudaError_t e__ = (expr);                                                    \
    if (e__ != cudaSuccess) {                                                    \
      ::qb::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));          \
      return QB_ERR_CUDA;                                                        \
    }                                                                            \
  } while (0)

#define QB_LAUNCH_OK(name)                                                       \
  do {                                                                           \
    cudaError_t e__ = cudaGetLastError();                                        \
    if (e__ != cudaSuccess) {                                                    \
      ::qb::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__)); \
      return QB_ERR_CUDA;                                                        \
    }                                                                            \
  } while (0)

#ifdef __CUDACC__
// Programmatic dependent launch, for the small kernels of a decode step whose cost is mostly the gap between launches:
// the kernel may be scheduled while its predecessor on the stream is still draining, and waits (grid_dependency_wait,
// before its first access to global memory) until that predecessor has completed and its writes are visible.  The
// error of a failed launch is picked up by QB_LAUNCH_OK like that of a <<<>>> launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the NEXT programmatic dependent on the stream be scheduled now: its CTAs then run up to their own
// grid_dependency_wait (set-up, prefetch of weights) while this kernel is still working.  Two conditions, both the
// caller's to guarantee (hence an explicit flag on the entry points that offer it):
//  * the whole grid is resident at once (the small kernels of a decode step): waiting dependents hold SM resources;
//  * the dependent reads what this kernel writes with loads that bypass L1 (__ldcg).  An SM's L1 is not invalidated
//    between a dependent's early start and its wait, so a cached (ld.global / __ldg) read after the wait can return a line
//    that the SM cached before this kernel overwrote it: a captured decode step produced garbage that way, while the same
//    launches issued one by one from the host, which never overlap, were correct.
__device__ __forceinline__ void grid_dependency_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Load of an ACTIVATION (anything a kernel earlier on the stream may have written): through L2, never from this SM's L1.
// Constants of a model (weights, scales, tables) keep their cached loads.
template <typename T>
__device__ __forceinline__ T ld_act(const T* p) { return __ldcg(p); }
__device__ __forceinline__ int8_t ld_act(const int8_t* p) { return (int8_t)__ldcg(reinterpret_cast<const signed char*>(p)); }
template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// qb_set_early_overlap: while on, the kernels of a prefill chain (norms, GEMMs, conv1d, SSD, Hadamard) execute
// grid_dependency_launch() as they start, so that the next programmatic launch on the stream gets its CTAs resident and its
// prologue done while this kernel still works.  Every kernel of this library that is launched as a programmatic dependent
// reads activations past L1 (ld_act() below, TMA or bulk copies), which is what makes that safe.
bool early_overlap();

// Cross-check switches (qb_set_path_override): each bit sends an op to its portable twin so that two implementations can be
// compared on one device.  Off by default; set explicitly through the C ABI, never read from the environment.
bool path_override(int bit);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

int sm_count();         // multiprocessors the kernels size their grids for: the device's count, capped by qb_set_sm_budget
int device_sm_count();  // multiprocessor count of the current device (cached per device)

// One-time-per-device guard for cudaFuncSetAttribute calls: kernel attributes belong to a device, so a process that
// drives several GPUs must set them on each.  Returns true the first time it is asked about the current device.
// (Two host threads asking at once may both get true: the attribute is then set twice to the same value, which is fine.)
struct PerDeviceOnce {
  bool done[64] = {};
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
};

// ---- device helpers ------------------------------------------------------------------------
#ifdef __CUDACC__

// x * sigmoid(x) with one MUFU op: sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5.
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float silu_fast(float v) {
  const float h = 0.5f * v;
  return fmaf(h, tanh_approx(h), h);
}
// v / (1 + exp(-v)) evaluated the long way (exp2 + divide): used where the result stays fp16.
__device__ __forceinline__ float silu_exact(float v) { return v / (1.0f + __expf(-v)); }

// 2^x on the MUFU pipe (flushes denormal results to zero).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// x <= 20 ? log1p(exp(x)) : x
__device__ __forceinline__ float softplus_f(float x) { return x <= 20.0f ? log1pf(__expf(x)) : x; }

// The same function on the MUFU pipe for the per-element paths: e = 2^(x log2 e); log1p(e) as ln2 * lg2(1 + e) for
// e >= 2^-7 and as the series e (1 - e/2 + e^2/3) below (the lg2 form loses relative accuracy when 1 + e rounds).
// Relative error <= ~3e-5 over the whole range, against 1e-7 for softplus_f.
__device__ __forceinline__ float softplus_fast(float x) {
  float e, l;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 1.4426950408889634f));
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(1.0f + e));
  const float big = l * 0.6931471805599453f;
  const float small = e * fmaf(e, fmaf(e, 0.3333333333f, -0.5f), 1.0f);
  const float r = e < 0.0078125f ? small : big;
  return x <= 20.0f ? r : x;
}

// v * sigmoid(v) with two MUFU ops (ex2, rcp): v / (1 + 2^(-v log2 e)).
__device__ __forceinline__ float silu_mufu(float v) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return v * r;
}

// C roundf (halves away from zero) followed by a clamp to int8, as one int.
__device__ __forceinline__ int round_away_s8(float v) {
  int r = __float2int_rz(v + copysignf(0.5f, v));
  return max(-128, min(127, r));
}
// rint (halves to even) + clamp.
__device__ __forceinline__ int rint_s8(float v) {
  int r = __float2int_rn(v);
  return max(-128, min(127, r));
}
// pack four already-clamped ints into one little-endian word of int8
__device__ __forceinline__ uint32_t pack4_s8(int a, int b, int c, int d) {
  return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)d << 24);
}

// pack four ints into one little-endian word of int8, each saturated to [-128, 127]
__device__ __forceinline__ uint32_t pack4_sat_s8(int a, int b, int c, int d) {
  uint32_t hi, r;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
  return r;
}

// Grouped ("group_heads") lookup: number of cumulative range ends <= idx, clamped to n-1.
__device__ __forceinline__ int group_lookup(const int32_t* range, int n, int idx) {
  int g = 0;
  for (int i = 0; i < n; ++i) g += (idx >= range[i]) ? 1 : 0;
  return min(g, n - 1);
}

#endif  // __CUDACC__

}  // namespace qb
