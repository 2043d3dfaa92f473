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
  if (gridDim.x <= 64) grid_dependency_launch();    // decode-sized: the next kernel may start its set-up already
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= n_tokens) return;
  int64_t id = tokens[tok];
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
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const __half* __restrict__ logits, int64_t row_stride, int n, int64_t* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  grid_dependency_wait();
  const __half* row = logits + (int64_t)blockIdx.x * row_stride;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float v = __half2float(row[j]);
    if (v > best || (v == best && j < idx)) { best = v; idx = j; }
  }
  auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, best, o);
    const int i = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(v, i, best, idx)) { best = v; idx = i; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    best = lane < (int)(blockDim.x >> 5) ? sv[lane] : -INFINITY;
    idx = lane < (int)(blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v = __shfl_xor_sync(0xffffffffu, best, o);
      const int i = __shfl_xor_sync(0xffffffffu, idx, o);
      if (better(v, i, best, idx)) { best = v; idx = i; }
    }
    if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
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
  launch_dependent(argmax_rows_kernel, dim3((unsigned)rows), dim3(1024), 0, (cudaStream_t)stream,
                   static_cast<const __half*>(logits), row_stride, n, out);
  QB_LAUNCH_OK("argmax_rows_kernel");
  return QB_OK;
}
