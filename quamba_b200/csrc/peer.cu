// The exchange step of a head-parallel layer over peer memory: regions shared through CUDA IPC, copy-engine puts, flags
// that only grow, a time-bounded wait, and the reduction of the received partial sums.
//
// Why copy engines and not stores from the GEMM's epilogue: at eight ranks the row-parallel out_proj of the 8B layer
// computes for about 0.3 ms and produces 1 GB of fp16 partial sums of which 7/8 leave the GPU, 1.2 ms of NVLink time.
// Stores from the epilogue would hold every multiprocessor for that long; a copy engine moves the same bytes while the
// next chunk's kernels have the whole GPU.
#include <string.h>

#include <algorithm>

#include "common.cuh"

namespace qb {
int* device_status_ptr();

struct FlagList {
  uint32_t* p[QB_MAX_PEERS];
};

// After the copies before it on the stream: one thread per flag, a system-scope fence and a store that a peer polls.
__global__ void peer_signal_kernel(FlagList f, int n, uint32_t value) {
  const int i = threadIdx.x;
  if (i < n && f.p[i] != nullptr) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.p[i]), "r"(value) : "memory");
  }
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// One warp; lane i polls flags[i] (local memory written by a peer) until flag - value >= 0 or the time limit passes.
// Once the status word holds an error (an earlier wait gave up, say) later waits return at once: a step whose peer has
// gone costs one time limit, not one per wait.
__global__ void peer_wait_kernel(const uint32_t* flags, int n, uint32_t value, uint64_t limit_ns, int* status) {
  const int i = threadIdx.x;
  bool ok = true;
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  if (i < n) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
      if ((int32_t)(v - value) >= 0) break;
      if (global_timer_ns() - t0 > limit_ns) { ok = false; break; }
      __nanosleep(256);
    }
  }
  if (!ok) atomicCAS(status, 0, 601);   // 601: a peer's flag did not arrive in time
  __threadfence_system();
}

// out = fp16(sum_p partials[p]), eight halves per thread and step, all partials of a step requested before the first add.
template <int NP>
__global__ void __launch_bounds__(256) sum_partials_kernel(const __half* __restrict__ x, int64_t stride, __half* __restrict__ out,
                                                           int64_t chunks) {
  grid_dependency_wait();
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
    uint4 r[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) r[p] = ld_act(reinterpret_cast<const uint4*>(x + p * stride) + c);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const __half2* h = reinterpret_cast<const __half2*>(&r[p]);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
    }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
    reinterpret_cast<uint4*>(out)[c] = o;
  }
}

// any count and alignment
__global__ void __launch_bounds__(256) sum_partials_generic_kernel(const __half* __restrict__ x, int np, int64_t stride,
                                                                   __half* __restrict__ out, int64_t n) {
  grid_dependency_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < np; ++p) acc += __half2float(ld_act(x + p * stride + i));
    out[i] = __float2half_rn(acc);
  }
}

}  // namespace qb

using namespace qb;

extern "C" int qb_peer_alloc(int64_t bytes, void** ptr, unsigned char handle[64]) {
  QB_REQUIRE(bytes > 0 && ptr != nullptr && handle != nullptr, QB_ERR_INVALID_ARG, "peer_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  QB_CUDA_OK(cudaMalloc(&p, (size_t)bytes));
  cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    set_error("peer_alloc: %s", cudaGetErrorString(e));
    return QB_ERR_CUDA;
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return QB_OK;
}

extern "C" int qb_peer_open(const unsigned char handle[64], void** ptr) {
  QB_REQUIRE(handle != nullptr && ptr != nullptr, QB_ERR_INVALID_ARG, "peer_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  QB_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return QB_OK;
}

extern "C" int qb_peer_close(void* ptr) {
  QB_REQUIRE(ptr != nullptr, QB_ERR_INVALID_ARG, "peer_close: null pointer");
  QB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return QB_OK;
}

extern "C" int qb_peer_free(void* ptr) {
  QB_REQUIRE(ptr != nullptr, QB_ERR_INVALID_ARG, "peer_free: null pointer");
  QB_CUDA_OK(cudaFree(ptr));
  return QB_OK;
}

extern "C" int qb_peer_put(const qb_peer_put_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "peer_put: null arguments");
  QB_REQUIRE(a->n >= 1 && a->n <= QB_MAX_PEERS && a->self >= 0 && a->self < a->n, QB_ERR_INVALID_ARG, "peer_put: n = %d, self = %d", a->n,
             a->self);
  QB_REQUIRE(a->bytes >= 0 && a->src_stride_bytes >= 0 && (a->bytes == 0 || a->src != nullptr), QB_ERR_INVALID_ARG, "peer_put: bad source");
  cudaStream_t st = (cudaStream_t)stream;
  cudaEvent_t ev = (cudaEvent_t)a->after_event;
  bool per_peer = false;
  for (int q = 0; q < a->n; ++q) per_peer = per_peer || a->stream_of[q] != nullptr;
  if (!per_peer) {
    FlagList f;
    bool any_flag = false;
    for (int q = 0; q < QB_MAX_PEERS; ++q) {
      f.p[q] = q < a->n ? a->flag[q] : nullptr;
      any_flag = any_flag || f.p[q] != nullptr;
    }
    if (ev != nullptr) QB_CUDA_OK(cudaStreamWaitEvent(st, ev, 0));
    if (a->bytes > 0) {
      for (int k = 1; k <= a->n; ++k) {
        const int q = (a->self + k) % a->n;      // own piece last
        if (a->dst[q] == nullptr) continue;
        const char* s = static_cast<const char*>(a->src) + (int64_t)q * a->src_stride_bytes;
        QB_CUDA_OK(cudaMemcpyAsync(a->dst[q], s, (size_t)a->bytes, cudaMemcpyDeviceToDevice, st));
      }
    }
    if (any_flag) {
      peer_signal_kernel<<<1, QB_MAX_PEERS, 0, st>>>(f, a->n, a->value);
      QB_LAUNCH_OK("peer_signal_kernel");
    }
    return QB_OK;
  }
  for (int k = 1; k <= a->n; ++k) {
    const int q = (a->self + k) % a->n;
    if (a->dst[q] == nullptr && a->flag[q] == nullptr) continue;
    cudaStream_t sq = a->stream_of[q] != nullptr ? (cudaStream_t)a->stream_of[q] : st;
    if (ev != nullptr) QB_CUDA_OK(cudaStreamWaitEvent(sq, ev, 0));
    if (a->bytes > 0 && a->dst[q] != nullptr) {
      const char* s = static_cast<const char*>(a->src) + (int64_t)q * a->src_stride_bytes;
      QB_CUDA_OK(cudaMemcpyAsync(a->dst[q], s, (size_t)a->bytes, cudaMemcpyDeviceToDevice, sq));
    }
    if (a->flag[q] != nullptr) {
      FlagList f = {};
      f.p[0] = a->flag[q];
      peer_signal_kernel<<<1, 32, 0, sq>>>(f, 1, a->value);
      QB_LAUNCH_OK("peer_signal_kernel");
    }
  }
  return QB_OK;
}

extern "C" int qb_peer_wait(const uint32_t* flags, int32_t n, uint32_t value, int32_t timeout_ms, void* stream) {
  QB_REQUIRE(flags != nullptr && n >= 1 && n <= 32 && timeout_ms > 0, QB_ERR_INVALID_ARG, "peer_wait: bad arguments");
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "device status word unavailable");
  peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, value, (uint64_t)timeout_ms * 1000000ull, status);
  QB_LAUNCH_OK("peer_wait_kernel");
  return QB_OK;
}

extern "C" int qb_sum_partials(const void* partials, int32_t n_partials, int64_t partial_stride, void* out, int64_t n, void* stream) {
  QB_REQUIRE(partials != nullptr && out != nullptr && n_partials >= 1 && n >= 0 && partial_stride >= 0, QB_ERR_INVALID_ARG,
             "sum_partials: bad arguments");
  if (n == 0) return QB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const __half* x = static_cast<const __half*>(partials);
  __half* o = static_cast<__half*>(out);
  const bool vec = n % 8 == 0 && partial_stride % 8 == 0 && aligned(x, 16) && aligned(o, 16);
  const int64_t work = vec ? n / 8 : n;
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(work, 256), (int64_t)sm_count() * 8);
#define QB_SUM_CASE(NP) \
  case NP: launch_dependent(sum_partials_kernel<NP>, dim3(grid), dim3(256), 0, st, x, partial_stride, o, work); break;
  if (vec && n_partials <= 8) {
    switch (n_partials) {
      QB_SUM_CASE(1) QB_SUM_CASE(2) QB_SUM_CASE(3) QB_SUM_CASE(4) QB_SUM_CASE(5) QB_SUM_CASE(6) QB_SUM_CASE(7) QB_SUM_CASE(8)
    }
  } else {
    launch_dependent(sum_partials_generic_kernel, dim3(grid), dim3(256), 0, st, x, (int)n_partials, partial_stride, o, n);
  }
#undef QB_SUM_CASE
  QB_LAUNCH_OK("sum_partials_kernel");
  return QB_OK;
}
