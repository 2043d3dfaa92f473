// Token embedding gather for sm_100a: fp16 table, int8 table (W8O16) or packed int4 table (W4O16), fp16 rows out.
// One warp per token row; a lane converts one 16-byte chunk of the stored row per step and writes 16-byte chunks.
#include "common.cuh"

namespace qb {
namespace {

constexpr int kStatusTokenRange = 501;   // keep in step with qb_read_device_status (lib.cu)

// kind 0: fp16 (vocab, dim).  kind 1: int8 (vocab, dim) + fp16 scale per row: out = scale * half(q) in fp16.
// kind 2: int32 (vocab, dim / 8): nibble i of a word holds element [0, 2, 4, 6, 1, 3, 5, 7][i] of its eight values
// (value + 8); out = half(q - 8) * scale in fp16, the product the reference forms with hsub2 / hfma2 + hmul2.
template <int KIND>
__global__ void __launch_bounds__(256)
embedding_kernel(const void* __restrict__ table, const __half* __restrict__ scales, const int64_t* __restrict__ tokens,
                 __half* __restrict__ out, int64_t n_tokens, int dim, int vocab, int* __restrict__ status) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= n_tokens) return;
  int64_t id = ld_act(tokens + tok);       // written by the argmax of the step before when a decode graph feeds itself
  if (id < 0 || id >= vocab) {       // an out-of-range id reads row 0 and raises the status word instead of faulting
    if (lane == 0) atomicCAS(status, 0, kStatusTokenRange);
    id = 0;
  }
  __half* o = out + tok * dim;
  if (KIND == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __half*>(table) + id * dim);
    for (int c = lane; c < dim / 8; c += 32) reinterpret_cast<uint4*>(o)[c] = __ldg(src + c);
  } else if (KIND == 1) {
    const __half s = scales[id];
    const uint2* src = reinterpret_cast<const uint2*>(static_cast<const int8_t*>(table) + id * dim);
    for (int c = lane; c < dim / 8; c += 32) {
      const uint2 raw = __ldg(src + c);
      const uint32_t w[2] = {raw.x, raw.y};
      uint4 r;
      __half* rh = reinterpret_cast<__half*>(&r);
#pragma unroll
      for (int e = 0; e < 8; ++e) rh[e] = __hmul(s, __int2half_rn((int)(int8_t)(w[e >> 2] >> (8 * (e & 3)))));
      reinterpret_cast<uint4*>(o)[c] = r;
    }
  } else {
    const __half s = scales[id];
    const uint32_t* src = static_cast<const uint32_t*>(table) + id * (dim / 8);
    for (int c = lane; c < dim / 8; c += 32) {
      const uint32_t q = __ldg(src + c);
      uint4 r;
      __half* rh = reinterpret_cast<__half*>(&r);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int nib = (e >> 1) + 4 * (e & 1);      // element e sits in nibble [0, 4, 1, 5, 2, 6, 3, 7][e]
        rh[e] = __hmul(__int2half_rn((int)((q >> (4 * nib)) & 0xf) - 8), s);
      }
      reinterpret_cast<uint4*>(o)[c] = r;
    }
  }
}

// Greedy sampling: index of the largest logit of each row (the lowest index among equals), as int64.
// A row is scanned by kArgBlocks CTAs; each folds its slice into one 64-bit key -- the value mapped to an order-preserving
// unsigned integer in the high word, the bitwise complement of the index in the low word, so that the largest key is the
// largest value at the lowest index -- and publishes it with atomicMax on a per-row word of library-owned scratch; the
// last CTA to arrive (a ticket counter) writes the token and leaves both words zeroed for the next call.  Calls whose
// kernels overlap on the GPU (different streams) would share that scratch: issue them on one stream.
constexpr int kArgBlocks = 32;
constexpr int kArgMaxRows = 1024;
__device__ unsigned long long g_arg_key[kArgMaxRows];
__device__ unsigned int g_arg_count[kArgMaxRows];

__global__ void __launch_bounds__(256)
argmax_rows_kernel(const __half* __restrict__ logits, int64_t row_stride, int n, int64_t* __restrict__ out) {
  __shared__ unsigned long long skey[8];
  grid_dependency_wait();
  const int r = blockIdx.y;
  const __half* row = logits + (int64_t)r * row_stride;
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int j0 = blockIdx.x * per, j1 = min(n, j0 + per);
  unsigned long long best = 0ull;
  for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
    const uint32_t bits = __float_as_uint(__half2float(__ldcg(row + j)));     // L2 read: the producer may have let this kernel start early
    const uint32_t ord = bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);
    const unsigned long long key = ((unsigned long long)ord << 32) | (uint32_t)(~(uint32_t)j);
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long v = __shfl_xor_sync(0xffffffffu, best, o);
    best = v > best ? v : best;
  }
  if ((threadIdx.x & 31) == 0) skey[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) best = skey[i] > best ? skey[i] : best;
    atomicMax(&g_arg_key[r], best);
    __threadfence();
    const unsigned int ticket = atomicAdd(&g_arg_count[r], 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      const unsigned long long k = atomicExch(&g_arg_key[r], 0ull);
      g_arg_count[r] = 0u;
      out[r] = k == 0ull ? 0 : (int64_t)(uint32_t)(~(uint32_t)k);
    }
  }
}

}  // namespace

int* device_status_ptr();   // lib.cu: the per-device status word

}  // namespace qb

using namespace qb;

extern "C" int qb_embedding_lookup(const qb_embedding_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->table && a->tokens && a->out, QB_ERR_INVALID_ARG, "embedding_lookup: null pointer");
  QB_REQUIRE(a->kind >= 0 && a->kind <= 2, QB_ERR_INVALID_ARG, "embedding_lookup: kind must be 0 (fp16), 1 (int8) or 2 (int4)");
  QB_REQUIRE(a->kind == 0 || a->scales != nullptr, QB_ERR_INVALID_ARG, "embedding_lookup: a quantised table needs its scales");
  QB_REQUIRE(a->n_tokens >= 0 && a->dim > 0 && a->vocab > 0, QB_ERR_INVALID_ARG, "embedding_lookup: bad shape");
  QB_REQUIRE(a->dim % 8 == 0 && aligned(a->table, a->kind == 0 ? 16 : (a->kind == 1 ? 8 : 4)) && aligned(a->out, 16),
             QB_ERR_INVALID_ARG, "embedding_lookup: dim must be a multiple of 8 and the buffers aligned");
  if (a->n_tokens == 0) return QB_OK;
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "embedding_lookup: no device status word");
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((unsigned)ceil_div(a->n_tokens, 8)), block(256);
  const __half* sc = static_cast<const __half*>(a->scales);
  __half* out = static_cast<__half*>(a->out);
  if (a->kind == 0) launch_dependent(embedding_kernel<0>, grid, block, 0, st, a->table, sc, a->tokens, out, a->n_tokens, a->dim, a->vocab, status);
  else if (a->kind == 1) launch_dependent(embedding_kernel<1>, grid, block, 0, st, a->table, sc, a->tokens, out, a->n_tokens, a->dim, a->vocab, status);
  else launch_dependent(embedding_kernel<2>, grid, block, 0, st, a->table, sc, a->tokens, out, a->n_tokens, a->dim, a->vocab, status);
  QB_LAUNCH_OK("embedding_kernel");
  return QB_OK;
}

extern "C" int qb_argmax_rows(const void* logits, int64_t row_stride, int32_t rows, int32_t n, int64_t* out, void* stream) {
  QB_REQUIRE(logits != nullptr && out != nullptr, QB_ERR_INVALID_ARG, "argmax_rows: null pointer");
  QB_REQUIRE(rows >= 0 && n > 0 && row_stride >= n, QB_ERR_INVALID_ARG, "argmax_rows: bad shape");
  if (rows == 0) return QB_OK;
  QB_REQUIRE(rows <= kArgMaxRows, QB_ERR_TOO_LARGE, "argmax_rows: at most %d rows per call", kArgMaxRows);
  launch_dependent(argmax_rows_kernel, dim3((unsigned)kArgBlocks, (unsigned)rows), dim3(256), 0, (cudaStream_t)stream,
                   static_cast<const __half*>(logits), row_stride, n, out);
  QB_LAUNCH_OK("argmax_rows_kernel");
  return QB_OK;
}
