// W4A8 / W8A8 linears for sm_100a: weight preparation, the shared epilogue, and the portable
// integer tile kernel used for shapes the tensor-core path does not take (ragged K / N, tiny M).
#include "common.cuh"
#include "linear_epilogue.cuh"

namespace qb {
namespace {

// ---- Marlin-QQQ packed int4 -> int8 (N, K) ---------------------------------------------------
__constant__ int16_t c_wperm_group[1024];
__constant__ int16_t c_wperm_channel[1024];

void build_weight_perm(bool per_channel, int16_t* out) {
  // Position j of a permuted 1024-element row holds element perm[j] of the tile-major row
  // (16 k-rows x 64 columns = four 16x16 tiles): the mma.sync fragment order of the Ampere
  // kernel this format was designed for, then an 8-element interleave that depends on the
  // quantisation type.
  int16_t base[1024];
  int idx = 0;
  for (int i = 0; i < 32; ++i) {
    int16_t one[8];
    int o = 0;
    const int col = i / 4;
    for (int block = 0; block < 2; ++block)
      for (int row = 4 * (i % 4); row < 4 * (i % 4) + 4; ++row) one[o++] = (int16_t)(16 * row + col + 8 * block);
    for (int j = 0; j < 4; ++j)
      for (int e = 0; e < 8; ++e) base[idx++] = (int16_t)(one[e] + 256 * j);
  }
  static const int inter_group[8] = {0, 2, 4, 6, 1, 3, 5, 7};
  static const int inter_channel[8] = {4, 0, 5, 1, 6, 2, 7, 3};
  const int* inter = per_channel ? inter_channel : inter_group;
  for (int g = 0; g < 128; ++g)
    for (int e = 0; e < 8; ++e) out[g * 8 + e] = base[g * 8 + inter[e]];
}

int upload_perms() {
  static bool done[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return QB_OK;
  static int16_t pg[1024], pc[1024];
  build_weight_perm(false, pg);
  build_weight_perm(true, pc);
  QB_CUDA_OK(cudaMemcpyToSymbol(c_wperm_group, pg, sizeof(pg)));
  QB_CUDA_OK(cudaMemcpyToSymbol(c_wperm_channel, pc, sizeof(pc)));
  if (dev < 64) done[dev] = true;
  return QB_OK;
}

__global__ void w4a8_unpack_kernel(const int32_t* __restrict__ packed, const __half* __restrict__ s_group,
                                   int8_t* __restrict__ w8, int size_k, int size_n, int group_size) {
  // one thread per packed word: 8 nibbles
  const int words_per_row = size_n * 2;  // N*16/8
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)(size_k / 16) * words_per_row;
  if (idx >= total) return;
  const int r = (int)(idx / words_per_row);
  const int c = (int)(idx % words_per_row);
  const uint32_t word = (uint32_t)packed[idx];
  const bool per_channel = s_group == nullptr;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int pidx = c * 8 + i;
    const int blk = pidx >> 10, within = pidx & 1023;
    const int src = (per_channel ? c_wperm_channel[within] : c_wperm_group[within]) + (blk << 10);
    const int nt = src >> 8, kk = (src & 255) >> 4, nn = src & 15;
    const int k = r * 16 + kk, n = nt * 16 + nn;
    const int nib = (word >> (4 * i)) & 0xf;
    int v;
    if (per_channel) {
      v = ((nib ^ 8) - 8) * 16;  // signed nibble in the high half of the byte
    } else {
      // natural (k / group, n) -> stored position inside its 64-element block (8x8 transpose)
      const int64_t nat = (int64_t)(k / group_size) * size_n + n;
      const int off = (int)(nat & 63);
      const int64_t pos = (nat & ~(int64_t)63) + ((off & 7) << 3) + (off >> 3);
      const float s = __half2float(s_group[pos]);
      // fp16 fma((q - 8), s, 1152): exact product, one rounding (half to even) at integer
      // granularity; the low mantissa byte is 128 + result, wrapped to 8 bits.
      const int rr = __float2int_rn((float)(nib - 8) * s);
      v = ((rr + 128) & 0xff) - 128;
    }
    w8[(int64_t)n * size_k + k] = (int8_t)v;
  }
}

__global__ void unpermute_channel_scale_kernel(const float* __restrict__ s_channel, float* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int off = i & 31;
  const int pos = (i & ~31) + ((off >> 1) & 3) * 8 + 2 * (off >> 3) + (off & 1);
  out[i] = s_channel[pos];
}

// ---- portable integer tile kernel --------------------------------------------------------------
// C[m, n] = sum_k A[m, k] * W[n, k], both operands K-contiguous int8; 64 x 64 tile per CTA,
// 64 bytes of K per step, dp4a.
constexpr int GT = 64;
constexpr int GKW = 16;  // words of K per step

__global__ void __launch_bounds__(256)
gemm_s8_dp4a_kernel(const int8_t* __restrict__ A, int64_t lda, const int8_t* __restrict__ W, int64_t ldw,
                    int M, int N, int K, Epilogue ep) {
  __shared__ uint32_t As[GT][GKW + 1];
  __shared__ uint32_t Ws[GT][GKW + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 3) == 0) &&
                   ((reinterpret_cast<uintptr_t>(W) & 3) == 0);
  int acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += GKW * 4) {
    __syncthreads();
    for (int e = tid; e < GT * GKW; e += 256) {
      const int row = e / GKW, w = e % GKW;
      const int k = k0 + w * 4;
      uint32_t va = 0, vw = 0;
      if (vec) {
        if (m0 + row < M && k < K) va = *reinterpret_cast<const uint32_t*>(A + (int64_t)(m0 + row) * lda + k);
        if (n0 + row < N && k < K) vw = *reinterpret_cast<const uint32_t*>(W + (int64_t)(n0 + row) * ldw + k);
      } else {
        for (int j = 0; j < 4; ++j) {
          if (k + j < K) {
            if (m0 + row < M) va |= (uint32_t)(uint8_t)A[(int64_t)(m0 + row) * lda + k + j] << (8 * j);
            if (n0 + row < N) vw |= (uint32_t)(uint8_t)W[(int64_t)(n0 + row) * ldw + k + j] << (8 * j);
          }
        }
      }
      As[row][w] = va;
      Ws[row][w] = vw;
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < GKW; ++w) {
      int a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = (int)As[tm + i][w]; b[i] = (int)Ws[tn + i][w]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(a[i], b[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + tm + i, n = n0 + tn + j;
      if (m < M && n < N) ep.store(acc[i][j], m, n);
    }
}

// ---- skinny-M kernel (decode: M = batch of single tokens) --------------------------------------------------------
// HBM-bound on the weights: each warp streams kNW rows of W (K-contiguous int8) with 16-byte loads, every lane taking
// chunks 512 bytes apart, and multiplies them against up to MB rows of A (re-read through L1/L2, they are small).
// dp4a accumulation, shuffle reduction, the shared epilogue.
constexpr int kGemvWarps = 8;
constexpr int kNW = 2;

// L2 prefetch of weight rows n0 .. n0 + kNW - 1 (row_bytes each): issued ahead of the dependency wait.
__device__ __forceinline__ void prefetch_rows(const void* W, int64_t pitch, int n0, int N, int row_bytes) {
  const int lane = threadIdx.x & 31;
  for (int j = 0; j < kNW; ++j) {
    if (n0 + j >= N) break;
    const uint8_t* rowp = static_cast<const uint8_t*>(W) + (int64_t)(n0 + j) * pitch;
    for (int off = lane * 128; off < row_bytes; off += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + off));
  }
}

template <int MB>
__global__ void __launch_bounds__(kGemvWarps * 32, 3)
gemv_s8_kernel(const int8_t* __restrict__ A, int64_t lda, const int8_t* __restrict__ W, int64_t ldw, int M, int N, int K,
               Epilogue ep) {
  // launched as a programmatic dependent: this warp's first weight rows are requested from HBM before the wait for the
  // kernel that produces A
  prefetch_rows(W, ldw, (blockIdx.x * kGemvWarps + (threadIdx.x >> 5)) * kNW, N, K);
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int chunks = K / 16;
  // The grid is one wave of CTAs (three per SM); a warp walks its column pairs with the grid's stride.  One CTA per 16
  // columns was 664 CTAs for the 2.7B in_proj: 1.5 to 2.2 waves of very short CTAs.
  for (int n0 = (blockIdx.x * kGemvWarps + (threadIdx.x >> 5)) * kNW; n0 < N; n0 += (int)gridDim.x * kGemvWarps * kNW)
  for (int m0 = 0; m0 < M; m0 += MB) {
    int acc[MB][kNW];
#pragma unroll
    for (int i = 0; i < MB; ++i)
#pragma unroll
      for (int j = 0; j < kNW; ++j) acc[i][j] = 0;
#pragma unroll 2
    for (int c = lane; c < chunks; c += 32) {
      uint4 w[kNW];
#pragma unroll
      for (int j = 0; j < kNW; ++j) {
        const int n = min(n0 + j, N - 1);
        w[j] = __ldg(reinterpret_cast<const uint4*>(W + (int64_t)n * ldw) + c);
      }
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        const int m = min(m0 + i, M - 1);
        const uint4 a = ld_act(reinterpret_cast<const uint4*>(A + (int64_t)m * lda) + c);
#pragma unroll
        for (int j = 0; j < kNW; ++j) {
          int t = acc[i][j];
          t = __dp4a((int)a.x, (int)w[j].x, t);
          t = __dp4a((int)a.y, (int)w[j].y, t);
          t = __dp4a((int)a.z, (int)w[j].z, t);
          t = __dp4a((int)a.w, (int)w[j].w, t);
          acc[i][j] = t;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < MB; ++i)
#pragma unroll
      for (int j = 0; j < kNW; ++j) {
        int t = acc[i][j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0 && m0 + i < M && n0 + j < N) ep.store(t, m0 + i, n0 + j);
      }
  }
}

// ---- decode-sized product straight from 4-bit weights ------------------------------------------------------------
// Per-channel quantised W4A8 weights are 16 * s with s the signed nibble, so the int8 copy the other kernels stream
// carries only four bits of information per byte.  For weight-streaming shapes (M < 32) this kernel reads a nibble-packed
// copy instead: row n holds K / 2 bytes; 32-bit word i of a row covers k = 8 i .. 8 i + 7 with u[8 i + b] in the low and
// u[8 i + 4 + b] in the high nibble of byte b, u = s + 8 in 0..15, so that (word & 0x0f0f0f0f) and (word >> 4) & 0x0f0f0f0f
// line up with two consecutive words of the activation row for dp4a.  sum_k a s = sum_k a u - 8 sum_k a, times 16: the
// same integer the int8 path accumulates, hence bit-identical outputs.
__global__ void w4a8_pack_nibbles_kernel(const int8_t* __restrict__ w8, uint32_t* __restrict__ w4, int64_t words) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one output word = 8 weights
  if (i >= words) return;
  const uint2 v = *reinterpret_cast<const uint2*>(w8 + i * 8);
  uint32_t out = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int lo = ((int)(int8_t)(v.x >> (8 * b)) >> 4) + 8;   // 16 s -> s + 8
    const int hi = ((int)(int8_t)(v.y >> (8 * b)) >> 4) + 8;
    out |= (uint32_t)(lo | (hi << 4)) << (8 * b);
  }
  w4[i] = out;
}

template <int MB>
__global__ void __launch_bounds__(kGemvWarps * 32, 3)
gemv_s4_kernel(const int8_t* __restrict__ A, int64_t lda, const uint8_t* __restrict__ W4, int M, int N, int K, Epilogue ep) {
  prefetch_rows(W4, K / 2, (blockIdx.x * kGemvWarps + (threadIdx.x >> 5)) * kNW, N, K / 2);
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int chunks = K / 32;              // 16 bytes of weights = 32 values per lane and step
  const int64_t ldw = K / 2;
  for (int n0 = (blockIdx.x * kGemvWarps + (threadIdx.x >> 5)) * kNW; n0 < N; n0 += (int)gridDim.x * kGemvWarps * kNW)
  for (int m0 = 0; m0 < M; m0 += MB) {
    int acc[MB][kNW], sa[MB];
#pragma unroll
    for (int i = 0; i < MB; ++i) {
      sa[i] = 0;
#pragma unroll
      for (int j = 0; j < kNW; ++j) acc[i][j] = 0;
    }
#pragma unroll 2
    for (int c = lane; c < chunks; c += 32) {
      uint4 w[kNW];
#pragma unroll
      for (int j = 0; j < kNW; ++j) {
        const int n = min(n0 + j, N - 1);
        w[j] = __ldg(reinterpret_cast<const uint4*>(W4 + (int64_t)n * ldw) + c);
      }
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        const int m = min(m0 + i, M - 1);
        const uint4 a0 = ld_act(reinterpret_cast<const uint4*>(A + (int64_t)m * lda) + 2 * c);
        const uint4 a1 = ld_act(reinterpret_cast<const uint4*>(A + (int64_t)m * lda) + 2 * c + 1);
        const int av[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
        int s = sa[i];
#pragma unroll
        for (int t = 0; t < 8; ++t) s = __dp4a(av[t], 0x01010101, s);
        sa[i] = s;
#pragma unroll
        for (int j = 0; j < kNW; ++j) {
          const uint32_t ww[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
          int t = acc[i][j];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            t = __dp4a(av[2 * q], (int)(ww[q] & 0x0f0f0f0fu), t);
            t = __dp4a(av[2 * q + 1], (int)((ww[q] >> 4) & 0x0f0f0f0fu), t);
          }
          acc[i][j] = t;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < MB; ++i) {
      int s = sa[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
      for (int j = 0; j < kNW; ++j) {
        int t = acc[i][j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0 && m0 + i < M && n0 + j < N) ep.store(16 * (t - 8 * s), m0 + i, n0 + j);
      }
    }
  }
}

int launch_gemv(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int M, int N, int K, const Epilogue& ep,
                cudaStream_t st) {
  if (K % 16 != 0 || lda % 16 != 0 || ldw % 16 != 0 || !aligned(A, 16) || !aligned(W, 16)) return QB_ERR_UNSUPPORTED;
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(N, kGemvWarps * kNW), (int64_t)sm_count() * 3);
  if (M == 1) launch_dependent(gemv_s8_kernel<1>, dim3(grid), dim3(kGemvWarps * 32), 0, st, A, lda, W, ldw, M, N, K, ep);
  else if (M == 2) launch_dependent(gemv_s8_kernel<2>, dim3(grid), dim3(kGemvWarps * 32), 0, st, A, lda, W, ldw, M, N, K, ep);
  else if (M <= 4) launch_dependent(gemv_s8_kernel<4>, dim3(grid), dim3(kGemvWarps * 32), 0, st, A, lda, W, ldw, M, N, K, ep);
  else launch_dependent(gemv_s8_kernel<8>, dim3(grid), dim3(kGemvWarps * 32), 0, st, A, lda, W, ldw, M, N, K, ep);
  QB_LAUNCH_OK("gemv_s8_kernel");
  return QB_OK;
}

int launch_portable(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int M, int N, int K,
                    const Epilogue& ep, cudaStream_t st) {
  dim3 grid((unsigned)ceil_div(N, GT), (unsigned)ceil_div(M, GT));
  gemm_s8_dp4a_kernel<<<grid, 256, 0, st>>>(A, lda, W, ldw, M, N, K, ep);
  QB_LAUNCH_OK("gemm_s8_dp4a_kernel");
  return QB_OK;
}

}  // namespace

// Implemented in gemm_tc.cu: returns QB_ERR_UNSUPPORTED when the shape is not eligible.
int launch_tensor_core_gemm(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int M, int N, int K,
                            const Epilogue& ep, cudaStream_t st);

int run_gemm(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int M, int N, int K, const Epilogue& ep,
             cudaStream_t st) {
  if (M <= 8) {  // a few rows stream the weights once through dp4a; from nine rows on the tensor-core kernel with
                 // 64-column tiles and a TMA box of only the rows that exist is faster (batch-16 decode: 30 us -> see bench)
    const int rc = launch_gemv(A, lda, W, ldw, M, N, K, ep, st);
    if (rc != QB_ERR_UNSUPPORTED) return rc;
  }
  const int rc = launch_tensor_core_gemm(A, lda, W, ldw, M, N, K, ep, st);
  if (rc != QB_ERR_UNSUPPORTED) return rc;
  return launch_portable(A, lda, W, ldw, M, N, K, ep, st);
}

}  // namespace qb

using namespace qb;

extern "C" int qb_w4a8_unpack(const qb_w4a8_unpack_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->packed && a->s_channel && a->w8 && a->s_channel_nat, QB_ERR_INVALID_ARG,
             "w4a8_unpack: null pointer");
  QB_REQUIRE(a->size_k > 0 && a->size_n > 0, QB_ERR_INVALID_ARG, "w4a8_unpack: empty shape");
  QB_REQUIRE(a->size_k % 16 == 0, QB_ERR_INVALID_ARG, "size_k = %d is not divisible by tile_size = 16", a->size_k);
  QB_REQUIRE(a->size_n % 64 == 0, QB_ERR_INVALID_ARG, "size_n = %d is not divisible by 64", a->size_n);
  if (a->s_group != nullptr) {
    QB_REQUIRE(a->group_size == 128, QB_ERR_INVALID_ARG, "Unexpected groupsize = %d", a->group_size);
    QB_REQUIRE(a->size_k % a->group_size == 0, QB_ERR_INVALID_ARG, "size_k not divisible by groupsize");
  }
  int rc = upload_perms();
  if (rc != QB_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = (int64_t)(a->size_k / 16) * a->size_n * 2;
  w4a8_unpack_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(
      a->packed, static_cast<const __half*>(a->s_group), a->w8, a->size_k, a->size_n, a->group_size);
  QB_LAUNCH_OK("w4a8_unpack_kernel");
  unpermute_channel_scale_kernel<<<(unsigned)ceil_div(a->size_n, 256), 256, 0, st>>>(a->s_channel, a->s_channel_nat,
                                                                                     a->size_n);
  QB_LAUNCH_OK("unpermute_channel_scale_kernel");
  return QB_OK;
}

extern "C" int qb_w4a8_gemm(const qb_w4a8_gemm_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->a && a->w8 && a->s_channel_nat && a->s_tok && a->out, QB_ERR_INVALID_ARG,
             "w4a8_gemm: null pointer");
  QB_REQUIRE(a->m >= 0 && a->n > 0 && a->k > 0, QB_ERR_INVALID_ARG, "w4a8_gemm: bad shape");
  if (a->m == 0) return QB_OK;
  QB_REQUIRE(a->a_row_stride >= a->k, QB_ERR_INVALID_ARG, "w4a8_gemm: a_row_stride < k");
  QB_REQUIRE(a->out_row_stride >= (a->output_transpose ? a->m : a->n), QB_ERR_INVALID_ARG,
             "w4a8_gemm: out_row_stride too small");
  Epilogue ep{};
  ep.row_scale = a->s_tok; ep.row_per = a->s_tok_per_row;
  ep.col_scale = a->s_channel_nat; ep.col_per = 1;
  ep.out = a->out; ep.out_stride = a->out_row_stride;
  ep.out_kind = a->out_int8 ? kOutS8Rne : kOutF16;
  ep.transpose = a->output_transpose;
  return run_gemm(a->a, a->a_row_stride, a->w8, a->k, a->m, a->n, a->k, ep, (cudaStream_t)stream);
}

extern "C" int qb_w8a8_gemm(const qb_w8a8_gemm_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->a && a->b && a->out, QB_ERR_INVALID_ARG, "w8a8_gemm: null pointer");
  QB_REQUIRE(a->use_alpha || (a->a_scale && a->b_scale), QB_ERR_INVALID_ARG, "w8a8_gemm: null scale pointer");
  QB_REQUIRE(a->m >= 0 && a->n > 0 && a->k > 0, QB_ERR_INVALID_ARG, "w8a8_gemm: bad shape");
  if (a->m == 0) return QB_OK;
  QB_REQUIRE(a->out_dtype >= 0 && a->out_dtype <= 2, QB_ERR_INVALID_ARG, "w8a8_gemm: unsupported output type");
  QB_REQUIRE(a->a_row_stride >= a->k && a->b_col_stride >= a->k && a->out_row_stride >= a->n, QB_ERR_INVALID_ARG,
             "w8a8_gemm: stride smaller than the extent");
  Epilogue ep{};
  ep.row_scale = a->a_scale; ep.row_per = a->a_scale_per_row;
  ep.col_scale = a->b_scale; ep.col_per = a->b_scale_per_col;
  ep.use_alpha = a->use_alpha; ep.alpha = a->alpha;
  ep.out = a->out; ep.out_stride = a->out_row_stride;
  ep.out_kind = a->out_dtype == 0 ? (a->round_half_away ? kOutS8Away : kOutS8Rne) : (a->out_dtype == 1 ? kOutF16 : kOutBF16);
  ep.transpose = 0;
  return run_gemm(a->a, a->a_row_stride, a->b, a->b_col_stride, a->m, a->n, a->k, ep, (cudaStream_t)stream);
}

extern "C" int qb_w4a8_pack_nibbles(const int8_t* w8, uint8_t* w4, int32_t n, int32_t k, void* stream) {
  QB_REQUIRE(w8 != nullptr && w4 != nullptr && n > 0 && k > 0, QB_ERR_INVALID_ARG, "w4a8_pack_nibbles: null pointer or empty shape");
  QB_REQUIRE(k % 8 == 0 && aligned(w8, 8) && aligned(w4, 4), QB_ERR_INVALID_ARG, "w4a8_pack_nibbles: k must be a multiple of 8");
  const int64_t words = (int64_t)n * k / 8;
  w4a8_pack_nibbles_kernel<<<(unsigned)ceil_div(words, 256), 256, 0, (cudaStream_t)stream>>>(w8, reinterpret_cast<uint32_t*>(w4), words);
  QB_LAUNCH_OK("w4a8_pack_nibbles_kernel");
  return QB_OK;
}

extern "C" int qb_w4a8_gemv_s4(const qb_w4a8_gemv_s4_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->a && a->w4 && a->s_channel_nat && a->s_tok && a->out, QB_ERR_INVALID_ARG, "w4a8_gemv_s4: null pointer");
  QB_REQUIRE(a->m > 0 && a->m < 32 && a->n > 0 && a->k > 0, QB_ERR_INVALID_ARG, "w4a8_gemv_s4: m must be in 1..31");
  QB_REQUIRE(a->k % 32 == 0 && a->a_row_stride % 16 == 0 && a->a_row_stride >= a->k && aligned(a->a, 16) && aligned(a->w4, 16),
             QB_ERR_INVALID_ARG, "w4a8_gemv_s4: k must be a multiple of 32 and the rows 16-byte aligned");
  QB_REQUIRE(a->out_row_stride >= (a->output_transpose ? a->m : a->n), QB_ERR_INVALID_ARG, "w4a8_gemv_s4: out_row_stride too small");
  Epilogue ep{};
  ep.row_scale = a->s_tok; ep.row_per = a->s_tok_per_row;
  ep.col_scale = a->s_channel_nat; ep.col_per = 1;
  ep.out = a->out; ep.out_stride = a->out_row_stride;
  ep.out_kind = a->out_int8 ? kOutS8Rne : kOutF16;
  ep.transpose = a->output_transpose;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(a->n, kGemvWarps * kNW), (int64_t)sm_count() * 3);
  const int M = a->m;
  if (M == 1) launch_dependent(gemv_s4_kernel<1>, dim3(grid), dim3(kGemvWarps * 32), 0, st, a->a, a->a_row_stride, a->w4, M, a->n, a->k, ep);
  else if (M == 2) launch_dependent(gemv_s4_kernel<2>, dim3(grid), dim3(kGemvWarps * 32), 0, st, a->a, a->a_row_stride, a->w4, M, a->n, a->k, ep);
  else if (M <= 4) launch_dependent(gemv_s4_kernel<4>, dim3(grid), dim3(kGemvWarps * 32), 0, st, a->a, a->a_row_stride, a->w4, M, a->n, a->k, ep);
  else launch_dependent(gemv_s4_kernel<8>, dim3(grid), dim3(kGemvWarps * 32), 0, st, a->a, a->a_row_stride, a->w4, M, a->n, a->k, ep);
  QB_LAUNCH_OK("gemv_s4_kernel");
  return QB_OK;
}
