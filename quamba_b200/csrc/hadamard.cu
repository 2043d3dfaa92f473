// Fused Hadamard rotation + int8 quantisation for sm_100a.
//
// out[r, :] = sat_int8(roundf((H_dim x[r, :]) * scale)),  H_dim = H_special (x) H_{2^k}
// (element index = chunk * 2^k + j).  One CTA owns one row: the row is staged once in shared
// memory as fp32, the power-of-two part runs as in-register radix-8 butterflies over shared
// memory, the special 12/20/28/40 part is a dense +-1 product whose signs sit in constant
// memory (so each term is one FFMA with a constant-bank operand), and the result leaves as
// 16-byte int8 stores.  Global traffic is exactly one read and one write of the row.
#include <cstdlib>
#include "common.cuh"
#include "hadamard_tables.inc"

namespace qb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxDim = 32768;  // fp32 staging of one row must fit the CTA's shared memory budget

__constant__ float c_had12[12 * 12];
__constant__ float c_had20[20 * 20];
__constant__ float c_had28[28 * 28];
__constant__ float c_had40[40 * 40];

template <int S> struct HadTable;
template <> struct HadTable<12> { static __device__ __forceinline__ const float* get() { return c_had12; } };
template <> struct HadTable<20> { static __device__ __forceinline__ const float* get() { return c_had20; } };
template <> struct HadTable<28> { static __device__ __forceinline__ const float* get() { return c_had28; } };
template <> struct HadTable<40> { static __device__ __forceinline__ const float* get() { return c_had40; } };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

// One radix-2^R pass over bits [b0, b0+R) of the index, all `dim` elements of the row.
template <int R>
__device__ __forceinline__ void butterfly_pass(float* row, int dim, int b0) {
  constexpr int N = 1 << R;
  const int groups = dim >> R;
  const int lo_mask = (1 << b0) - 1;
  for (int g = threadIdx.x; g < groups; g += kThreads) {
    const int lo = g & lo_mask;
    const int hi = g >> b0;
    float* p = row + ((hi << (b0 + R)) | lo);
    float v[N];
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = p[k << b0];
#pragma unroll
    for (int s = 1; s < N; s <<= 1) {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        if ((k & s) == 0) {
          const float a = v[k], b = v[k | s];
          v[k] = a + b;
          v[k | s] = a - b;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < N; ++k) p[k << b0] = v[k];
  }
}

// Dense S x S +-1 product across the chunk index for every column j < p2.
// Two threads share a column when there are fewer columns than threads; each produces half of
// the S outputs.  Results go to `dst` (a second buffer) so that no thread overwrites inputs
// another thread still reads.
template <int S>
__device__ __forceinline__ void special_pass(const float* src, float* dst, int p2) {
  const float* tab = HadTable<S>::get();
  constexpr int kHalf = S / 2;
  for (int item = threadIdx.x; item < 2 * p2; item += kThreads) {
    const int j = item % p2;
    const int half = item / p2;
    float v[S];
#pragma unroll
    for (int c = 0; c < S; ++c) v[c] = src[c * p2 + j];
#pragma unroll
    for (int i = 0; i < kHalf; ++i) {
      const int row = half * kHalf + i;
      float acc = 0.0f;
#pragma unroll
      for (int c = 0; c < S; ++c) acc = fmaf(tab[row * S + c], v[c], acc);
      dst[row * p2 + j] = acc;
    }
  }
}

template <typename T, int S>
__global__ void __launch_bounds__(kThreads)
hadamard_quant_kernel(const T* __restrict__ x, int64_t x_rs, int8_t* __restrict__ out, int64_t out_rs,
                      int dim, int log_p2, float scale, int vec_ok) {
  extern __shared__ __align__(16) float smem[];
  float* row = smem;
  float* row2 = smem + dim;  // only used when S > 1
  const int64_t r = blockIdx.x;
  const T* src = x + r * x_rs;
  constexpr int kPerLoad = 16 / sizeof(T);
  if (vec_ok) {
    for (int i = threadIdx.x * kPerLoad; i < dim; i += kThreads * kPerLoad) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + i));
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int k = 0; k < kPerLoad; ++k) row[i + k] = to_f32<T>(e[k]);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += kThreads) row[i] = to_f32<T>(src[i]);
  }
  __syncthreads();
  int b = 0;
  for (; b + 3 <= log_p2; b += 3) { butterfly_pass<3>(row, dim, b); __syncthreads(); }
  if (log_p2 - b == 2) { butterfly_pass<2>(row, dim, b); __syncthreads(); }
  if (log_p2 - b == 1) { butterfly_pass<1>(row, dim, b); __syncthreads(); }
  const float* res = row;
  if constexpr (S > 1) {
    special_pass<S>(row, row2, 1 << log_p2);
    __syncthreads();
    res = row2;
  }
  int8_t* dst = out + r * out_rs;
  if (vec_ok) {
    for (int i = threadIdx.x * 16; i < dim; i += kThreads * 16) {
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float4 f = *reinterpret_cast<const float4*>(res + i + 4 * k);
        w[k] = pack4_s8(round_away_s8(f.x * scale), round_away_s8(f.y * scale), round_away_s8(f.z * scale),
                        round_away_s8(f.w * scale));
      }
      *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += kThreads) dst[i] = (int8_t)round_away_s8(res[i] * scale);
  }
}

int upload_tables() {
  static bool done[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return QB_OK;
  auto expand = [](const unsigned long long* masks, int n, float* dst) {
    for (int i = 0; i < n; ++i)
      for (int j = 0; j < n; ++j) dst[i * n + j] = ((masks[i] >> j) & 1ULL) ? -1.0f : 1.0f;
  };
  static float t12[144], t20[400], t28[784], t40[1600];
  expand(kHadNeg12, 12, t12); expand(kHadNeg20, 20, t20); expand(kHadNeg28, 28, t28); expand(kHadNeg40, 40, t40);
  QB_CUDA_OK(cudaMemcpyToSymbol(c_had12, t12, sizeof(t12)));
  QB_CUDA_OK(cudaMemcpyToSymbol(c_had20, t20, sizeof(t20)));
  QB_CUDA_OK(cudaMemcpyToSymbol(c_had28, t28, sizeof(t28)));
  QB_CUDA_OK(cudaMemcpyToSymbol(c_had40, t40, sizeof(t40)));
  if (dev < 64) done[dev] = true;
  return QB_OK;
}

template <typename T, int S>
int launch(const qb_hadamard_quant_args* a, int log_p2, int vec_ok, cudaStream_t st) {
  const size_t smem = (size_t)a->dim * sizeof(float) * (S > 1 ? 2 : 1);
  auto kern = hadamard_quant_kernel<T, S>;
  if (smem > 48 * 1024) QB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)a->rows, kThreads, smem, st>>>(static_cast<const T*>(a->x), a->x_row_stride, a->out,
                                                  a->out_row_stride, a->dim, log_p2, a->scale, vec_ok);
  QB_LAUNCH_OK("hadamard_quant_kernel");
  return QB_OK;
}

template <typename T>
int dispatch_special(const qb_hadamard_quant_args* a, int log_p2, int vec_ok, cudaStream_t st) {
  switch (a->special) {
    case 1: return launch<T, 1>(a, log_p2, vec_ok, st);
    case 12: return launch<T, 12>(a, log_p2, vec_ok, st);
    case 20: return launch<T, 20>(a, log_p2, vec_ok, st);
    case 28: return launch<T, 28>(a, log_p2, vec_ok, st);
    case 40: return launch<T, 40>(a, log_p2, vec_ok, st);
  }
  set_error("hadamard: special order %d not in {1, 12, 20, 28, 40}", a->special);
  return QB_ERR_INVALID_ARG;
}

}  // namespace
}  // namespace qb

using namespace qb;

namespace qb { int hadamard_tc_launch(const qb_hadamard_quant_args* a, cudaStream_t st); }

extern "C" int qb_hadamard_quant(const qb_hadamard_quant_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->x && a->out, QB_ERR_INVALID_ARG, "hadamard_quant: null pointer");
  QB_REQUIRE(a->rows >= 0 && a->dim > 0, QB_ERR_INVALID_ARG, "hadamard_quant: bad shape");
  if (a->rows == 0) return QB_OK;
  QB_REQUIRE(a->special == 1 || a->special == 12 || a->special == 20 || a->special == 28 || a->special == 40,
             QB_ERR_INVALID_ARG, "hadamard: special order %d not in {1, 12, 20, 28, 40}", a->special);
  QB_REQUIRE(a->dim % a->special == 0, QB_ERR_INVALID_ARG, "hadamard: dim %d not divisible by %d", a->dim, a->special);
  const int p2 = a->dim / a->special;
  QB_REQUIRE((p2 & (p2 - 1)) == 0, QB_ERR_INVALID_ARG, "hadamard: dim / %d = %d is not a power of two", a->special, p2);
  QB_REQUIRE(a->dim * (a->special > 1 ? 2 : 1) <= kMaxDim, QB_ERR_TOO_LARGE, "hadamard: dim %d too large", a->dim);
  QB_REQUIRE(a->in_dtype >= 0 && a->in_dtype <= 2, QB_ERR_INVALID_ARG, "hadamard: in_dtype must be 0, 1 or 2");
  int log_p2 = 0;
  while ((1 << log_p2) < p2) ++log_p2;
  const int esz = a->in_dtype == 2 ? 4 : 2;
  const int vec_ok = (a->dim % 16 == 0) && aligned(a->x, 16) && aligned(a->out, 16) &&
                     ((a->x_row_stride * esz) % 16 == 0) && (a->out_row_stride % 16 == 0);
  cudaStream_t st = (cudaStream_t)stream;
  {  // tensor-core path (fp16 rows of S * 128 elements, contiguous); the kernels below are the general fallback
    if (!path_override(QB_PATH_HADAMARD_SIMT) && aligned(a->out, 1)) {
      const int rc = hadamard_tc_launch(a, st);
      if (rc != QB_ERR_UNSUPPORTED) return rc;
    }
  }
  if (a->special > 1) {
    int rc = upload_tables();
    if (rc != QB_OK) return rc;
  }
  switch (a->in_dtype) {
    case 0: return dispatch_special<__half>(a, log_p2, vec_ok, st);
    case 1: return dispatch_special<__nv_bfloat16>(a, log_p2, vec_ok, st);
    default: return dispatch_special<float>(a, log_p2, vec_ok, st);
  }
}
