// Fused kernels of the Mamba2 decode step for small batches (sm_100a).
//
// A decode step of one layer is seven tiny ops in the reference (block norm, in_proj, conv update, state update, gated
// norm, Hadamard + quantise, out_proj), each far below the launch-to-launch gap of a captured graph.  Four launches do
// the same work here:
//   1. qb_decode_norm_linear: residual add + RMSNorm + int8 quantise (re-done by every CTA in shared memory, it is 5 KB of
//      input) -> weight-streaming W4A8 product -> optional conv1d update of the xBC columns in the product's epilogue
//      (the warp that owns an output column also owns that channel's conv window).
//   2. the state update (qb_sscan_update, unchanged).
//   3. qb_decode_gate_had_quant: y * silu(z) -> grouped RMSNorm -> Hadamard rotation -> int8 quantise, one CTA per block
//      of 128 outputs; the out_proj product then runs as the ordinary weight-streaming kernel (a fourth launch).
// Arithmetic, rounding and operation order are those of the separate kernels (norm.cu, hadamard.cu, conv1d.cu,
// linear.cu), so results agree with the unfused path to the same tolerances.
#include <algorithm>
#include "common.cuh"
#include "tc_common.cuh"
#include "hadamard_tables.inc"

namespace qb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
// Output columns per warp and pass (NW) and 16-byte weight chunks a lane requests per column before it uses any (NB).
// SH = 0: 2 x 5, any k up to 8192.  SH = 1: 5 x 3 for wide products of short columns (at most 96 chunks per column): the
// 2.7B in_proj is 4.5 columns per resident warp, i.e. three dependent passes of two columns for a quarter of the warps and
// two for the rest -- or ONE pass of five for all of them; what a pass costs is its chain of round trips, not its bytes.
template <int SH> struct Shape { static constexpr int NW = SH ? 5 : 2; static constexpr int NB = SH ? 3 : 5; };
constexpr int kMaxRows = 4;         // batch rows a launch takes


__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum_f(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < kWarps; ++i) r += red[i];
  return r;
}
__device__ __forceinline__ float s8f(uint32_t w_biased, int k) {      // byte k of (w ^ 0x80808080) as a float
  return __uint_as_float(__byte_perm(w_biased, 0x4B000000u, 0x7650 + k)) - 8388736.0f;
}

// Weight formats a launch can stream (the template parameter WM of the kernels):
//   0  int8 (n, k): the expansion qb_w4a8_unpack makes
//   1  nibbles (n, k / 2) of a per-channel weight: value + 8, the int8 weight is 16 x the value
//   2  nibbles (n, k / 2) of a group-128 weight: the raw 4-bit codes, with s_grp (n, k / 128) fp16 group scales; the int8
//      weight (q - 8) * s_group rounded half to even is rebuilt in registers, two at a time in fp16 arithmetic, exactly as
//      the reference's kernel does it (marlin_qqq_gemm_kernel.cuh:136-178: one fp16 fma against 1152)
struct Linear {
  const __half* s_grp;     // format 2 only
  const uint8_t* w;        // int8 (n, k) rows, or a nibble copy (n, k / 2)
  const float* s_ch;       // channel scales in natural order
  const float* s_tok;      // input scale, one element
  void* out;
  int64_t out_stride;
  int n, k, out_int8;
};

// The conv1d update done in the product's epilogue for columns [c0, c0 + dim) of the output.
struct ConvEpi {
  int8_t* state;           // element (b, c, w) at b * sb + c * sd + w * sw
  int64_t sb, sd, sw;
  const int8_t* weight;    // (dim, 4)
  const int8_t* bias;      // (dim) or null
  int8_t* dst[3];          // x (B, x_dim), Bm, Cm (B, gn)
  const float* out_scale[3];
  float scale_in[3], scale_bias[3];
  int c0, dim, end0, end1;  // column of channel 0; segment ends in channels
  int enabled;
};

// dot products of the int8 rows in shared memory (MB rows of k bytes) with weight columns n0 .. n0 + kNW - 1.
// A lane loads kNB weight chunks per column BEFORE it uses any (clamped addresses, so the loads need no branches): at the
// model's sizes that is the lane's whole share of a column in one round trip to L2 instead of one round trip per chunk.

// One 32-bit word of format 2 (byte b: code of k = b in the low, of k = 4 + b in the high nibble) -> the int8 weights of
// k = 0..3 and of k = 4..7.  (1024 + q) - 1032 = q - 8 is exact in fp16; fma(q - 8, s, 1152) rounds the exact product once,
// at integer granularity, and leaves 128 + result in the low mantissa byte.
__device__ __forceinline__ void dequant8_group(uint32_t w, __half2 s2, uint32_t& lo4, uint32_t& hi4) {
  const __half2 k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));
  const __half2 k1152 = __half2half2(__ushort_as_half((unsigned short)0x6480));
  uint32_t p[4] = {(w & 0x000f000fu) | 0x64006400u, ((w >> 8) & 0x000f000fu) | 0x64006400u,
                   ((w >> 4) & 0x000f000fu) | 0x64006400u, ((w >> 12) & 0x000f000fu) | 0x64006400u};
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 v = __hfma2(__hsub2(*reinterpret_cast<const __half2*>(&p[i]), k1032), s2, k1152);
    r[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  lo4 = __byte_perm(r[0], r[1], 0x6240) ^ 0x80808080u;
  hi4 = __byte_perm(r[2], r[3], 0x6240) ^ 0x80808080u;
}

template <int MB, int S4, int SH>
__device__ __forceinline__ void dot_columns(const Linear& L, const int8_t* sA, int n0, int lane, int (&acc)[MB][Shape<SH>::NW],
                                            const uint8_t* sw = nullptr) {
  // sw: this warp's kNW weight rows staged in shared memory by a bulk copy (first pass), or null: read them from global
  constexpr int kNW = Shape<SH>::NW, kNB = Shape<SH>::NB;
  int sa[MB];
#pragma unroll
  for (int i = 0; i < MB; ++i) {
    sa[i] = 0;
#pragma unroll
    for (int j = 0; j < kNW; ++j) acc[i][j] = 0;
  }
  const int chunks = S4 ? L.k / 32 : L.k / 16;          // 16-byte weight chunks per column
  const int64_t ldw = S4 ? L.k / 2 : L.k;
  const uint4* wrow[kNW];
#pragma unroll
  for (int j = 0; j < kNW; ++j) wrow[j] = reinterpret_cast<const uint4*>(L.w + (int64_t)min(n0 + j, L.n - 1) * ldw);
  const int groups = L.k / 128;
  for (int c0 = lane; c0 < chunks; c0 += 32 * kNB) {
    uint4 w[kNW][kNB];
    unsigned short sg[kNW][kNB];     // format 2: the group scale of each chunk (a chunk is 32 codes of one group)
#pragma unroll
    for (int b = 0; b < kNB; ++b) {
      const int c = min(c0 + 32 * b, chunks - 1);
#pragma unroll
      for (int j = 0; j < kNW; ++j) {
        w[j][b] = sw != nullptr ? *(reinterpret_cast<const uint4*>(sw + (int64_t)j * ldw) + c) : __ldg(wrow[j] + c);
        if (S4 == 2) sg[j][b] = __ldg(reinterpret_cast<const unsigned short*>(L.s_grp) + (int64_t)min(n0 + j, L.n - 1) * groups + (c >> 2));
      }
    }
#pragma unroll
    for (int b = 0; b < kNB; ++b) {
      const int c = c0 + 32 * b;
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < MB; ++i) {
          if (!S4) {
            const uint4 a = *(reinterpret_cast<const uint4*>(sA + (int64_t)i * L.k) + c);
#pragma unroll
            for (int j = 0; j < kNW; ++j) {
              int t = acc[i][j];
              t = __dp4a((int)a.x, (int)w[j][b].x, t); t = __dp4a((int)a.y, (int)w[j][b].y, t);
              t = __dp4a((int)a.z, (int)w[j][b].z, t); t = __dp4a((int)a.w, (int)w[j][b].w, t);
              acc[i][j] = t;
            }
          } else if (S4 == 2) {
            // handled below, once per chunk for all rows
          } else {
            const uint4 a0 = *(reinterpret_cast<const uint4*>(sA + (int64_t)i * L.k) + 2 * c);
            const uint4 a1 = *(reinterpret_cast<const uint4*>(sA + (int64_t)i * L.k) + 2 * c + 1);
            const int av[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
            int sum = sa[i];
#pragma unroll
            for (int t = 0; t < 8; ++t) sum = __dp4a(av[t], 0x01010101, sum);
            sa[i] = sum;
#pragma unroll
            for (int j = 0; j < kNW; ++j) {
              const uint32_t ww[4] = {w[j][b].x, w[j][b].y, w[j][b].z, w[j][b].w};
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
        if (S4 == 2) {
#pragma unroll
          for (int j = 0; j < kNW; ++j) {
            const __half2 s2 = __half2half2(__ushort_as_half(sg[j][b]));
            const uint32_t ww[4] = {w[j][b].x, w[j][b].y, w[j][b].z, w[j][b].w};
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) dequant8_group(ww[q], s2, lo[q], hi[q]);
#pragma unroll
            for (int i = 0; i < MB; ++i) {
              const uint4 a0 = *(reinterpret_cast<const uint4*>(sA + (int64_t)i * L.k) + 2 * c);
              const uint4 a1 = *(reinterpret_cast<const uint4*>(sA + (int64_t)i * L.k) + 2 * c + 1);
              const int av[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
              int t = acc[i][j];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                t = __dp4a(av[2 * q], (int)lo[q], t);
                t = __dp4a(av[2 * q + 1], (int)hi[q], t);
              }
              acc[i][j] = t;
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MB; ++i) {
    const int s = S4 == 1 ? warp_sum_i(sa[i]) : 0;
#pragma unroll
    for (int j = 0; j < kNW; ++j) {
      const int t = warp_sum_i(acc[i][j]);
      acc[i][j] = S4 == 1 ? 16 * (t - 8 * s) : t;      // format 1: nibbles hold value + 8, the int8 weight is 16 x the value
    }
  }
}

// What a finishing lane needs beyond the accumulator.  Everything in it is either constant or was written by the previous
// decode STEP (the conv window), never by the kernel just before this one, so it is loaded ahead of the dependency wait.
struct FinishPre {
  float s_ch, s_tok, so, bias_term;
  int w0, w1, w2;          // the three newest samples of the conv window
  int wt;                  // four conv taps, packed
  int seg;                 // -1: not a conv column
};

__device__ __forceinline__ FinishPre finish_prefetch(const Linear& L, const ConvEpi& cv, int m, int n) {
  FinishPre f;
  f.s_ch = __ldg(L.s_ch + n);
  f.s_tok = __ldg(L.s_tok);
  f.seg = -1;
  const int c = n - cv.c0;
  if (L.out_int8 && cv.enabled && c >= 0 && c < cv.dim) {
    const int s = c < cv.end0 ? 0 : (c < cv.end1 ? 1 : 2);
    f.seg = s;
    const int8_t* st = cv.state + (int64_t)m * cv.sb + (int64_t)c * cv.sd;
    f.w0 = __ldcg(reinterpret_cast<const signed char*>(st) + cv.sw);      // rewritten every step: L2 reads
    f.w1 = __ldcg(reinterpret_cast<const signed char*>(st) + 2 * cv.sw);
    f.w2 = __ldcg(reinterpret_cast<const signed char*>(st) + 3 * cv.sw);
    f.wt = *reinterpret_cast<const int*>(cv.weight + (int64_t)c * 4);
    f.so = __ldg(cv.out_scale[s]);
    f.bias_term = cv.bias != nullptr ? cv.scale_bias[s] * (float)cv.bias[c] : 0.0f;
  }
  return f;
}

// scale, convert and store one output element; when the column is a conv channel, run that channel's decode step
__device__ __forceinline__ void finish(const Linear& L, const ConvEpi& cv, const FinishPre& f, int acc, int m, int n) {
  const float r = ((float)acc * f.s_ch) * f.s_tok;
  if (!L.out_int8) {
    static_cast<__half*>(L.out)[(int64_t)m * L.out_stride + n] = __float2half_rn(r);
    return;
  }
  const int q = rint_s8(r);
  if (f.seg < 0) {
    static_cast<int8_t*>(L.out)[(int64_t)m * L.out_stride + n] = (int8_t)q;
    return;
  }
  const int c = n - cv.c0, s = f.seg;
  int8_t* st = cv.state + (int64_t)m * cv.sb + (int64_t)c * cv.sd;
  st[0] = (int8_t)f.w0; st[cv.sw] = (int8_t)f.w1; st[2 * cv.sw] = (int8_t)f.w2; st[3 * cv.sw] = (int8_t)q;
  const int win = (f.w0 & 0xff) | ((f.w1 & 0xff) << 8) | ((f.w2 & 0xff) << 16) | (q << 24);
  const float dot = (float)__dp4a(win, f.wt, 0);
  const int cbase = s == 0 ? 0 : (s == 1 ? cv.end0 : cv.end1);
  const int width = s == 0 ? cv.end0 : cv.end1 - cv.end0;
  float v = cv.scale_in[s] * dot + f.bias_term;
  v = silu_fast(v);
  cv.dst[s][(int64_t)m * width + (c - cbase)] = (int8_t)round_away_s8(v / f.so);
}

// Ask L2 for every weight row this warp will stream (all its passes).  Weights do not depend on the kernel before this
// one, so the call sits ahead of the dependency wait and of the shared-memory prologue: HBM delivers while the prologue
// computes, and each pass then costs a round trip to L2 instead of one to HBM.
template <int S4, int SH>
__device__ __forceinline__ void prefetch_first_columns(const Linear& L, bool skip_first) {
  constexpr int kNW = Shape<SH>::NW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_bytes = S4 ? L.k / 2 : L.k;
  const int stride = (int)gridDim.x * kWarps * kNW;
  for (int n0 = (blockIdx.x * kWarps + warp) * kNW + (skip_first ? stride : 0); n0 < L.n; n0 += stride) {
    for (int j = 0; j < kNW; ++j) {
      if (n0 + j >= L.n) break;
      const uint8_t* rowp = L.w + (int64_t)(n0 + j) * row_bytes;
      for (int64_t off = (int64_t)lane * 128; off < row_bytes; off += 32 * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(rowp + off));
    }
  }
}

// `pre`: the finishing lane's constants of the first pass, loaded by the caller before the dependency wait.
template <int MB, int S4, int SH>
__device__ __forceinline__ void stream_columns(const Linear& L, const ConvEpi& cv, const int8_t* sA, int rows, FinishPre pre,
                                               const uint8_t* sw, uint64_t* wbar, int* status) {
  constexpr int kNW = Shape<SH>::NW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = lane / kNW, j = lane % kNW;
  const int first = (blockIdx.x * kWarps + warp) * kNW;
  for (int n0 = first; n0 < L.n; n0 += (int)gridDim.x * kWarps * kNW) {
    const bool mine = lane < MB * kNW && i < rows && n0 + j < L.n;
    if (n0 != first && mine) pre = finish_prefetch(L, cv, i, n0 + j);
    int acc[MB][kNW];
    const bool staged = sw != nullptr && n0 == first;
    if (staged) tc::mbar_wait(wbar, 0, status, QB_ERR_TIMEOUT);      // the bulk copies of this warp's first rows have landed
    dot_columns<MB, S4, SH>(L, sA, n0, lane, acc, staged ? sw : nullptr);
    // lanes 0 .. MB * kNW - 1 finish one (row, column) each, so that the conv windows of a warp's columns move in parallel
    if (mine) {
      int v = 0;
#pragma unroll
      for (int ii = 0; ii < MB; ++ii)
#pragma unroll
        for (int jj = 0; jj < kNW; ++jj)
          if (ii == i && jj == j) v = acc[ii][jj];
      finish(L, cv, pre, v, i, n0 + j);
    }
  }
}

template <int MB, int SH>
__device__ __forceinline__ FinishPre first_pass_prefetch(const Linear& L, const ConvEpi& cv, int rows) {
  constexpr int kNW = Shape<SH>::NW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = lane / kNW, j = lane % kNW;
  const int n0 = (blockIdx.x * kWarps + warp) * kNW;
  FinishPre pre{};
  if (lane < MB * kNW && i < rows && n0 + j < L.n) pre = finish_prefetch(L, cv, i, n0 + j);
  return pre;
}

// ---- launch 1: residual add + RMSNorm + quantise -> product (+ conv update) -------------------------------------------
struct NormIn {
  const int8_t* a_int8;     // (rows, k) already quantised input (stride x_stride): the norm is skipped
  const __half* x;          // (rows, k)
  const void* residual;     // fp32 or fp16 (rows, k), nullable
  void* residual_out;       // nullable
  const __half* weight;     // (k)
  int64_t x_stride, res_stride, res_out_stride;
  int res_f32, res_out_f32, early_launch;
  int stage_w;              // the first pass's weight rows go to shared memory by bulk copies issued before the dependency wait
  float eps, out_scale;
};

template <int MB, int S4, int SH>
__global__ void __launch_bounds__(kThreads, 2)
decode_norm_linear_kernel(NormIn nin, Linear L, ConvEpi cv, int rows, int* status) {
  extern __shared__ __align__(16) uint8_t dsm[];
  __shared__ float red[kWarps];
  __shared__ __align__(8) uint64_t wbar[kWarps];
  int8_t* sA = reinterpret_cast<int8_t*>(dsm);                 // MB rows of k int8
  const int K = L.k;
  if (nin.early_launch) grid_dependency_launch();
  // The weights of this warp's first pass travel HBM -> shared memory as bulk copies that are in flight during the
  // dependency wait and the norm: the product then reads them at shared-memory latency instead of paying a round trip
  // to L2 (or HBM) after the activations are ready.  Later passes (wide products) are prefetched into L2 as before.
  constexpr int kNWs = Shape<SH>::NW;
  const int64_t row_bytes = S4 ? K / 2 : K;
  const uint8_t* sw = nullptr;
  if (nin.stage_w) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* sW = dsm + (((int64_t)MB * K + 15) & ~(int64_t)15);
    if (threadIdx.x == 0) {
      for (int w = 0; w < kWarps; ++w) tc::mbar_init(&wbar[w], 1);
      tc::fence_barrier_init();
    }
    __syncthreads();
    sw = sW + (int64_t)warp * kNWs * row_bytes;
    const int n0 = (blockIdx.x * kWarps + warp) * kNWs;
    if (lane == 0 && n0 < L.n) {
      const int cols = min(kNWs, L.n - n0);
      tc::mbar_arrive_expect_tx(&wbar[warp], (uint32_t)(cols * row_bytes));
      for (int j = 0; j < cols; ++j)
        tc::bulk_load(const_cast<uint8_t*>(sw) + (int64_t)j * row_bytes, L.w + (int64_t)(n0 + j) * row_bytes, (uint32_t)row_bytes, &wbar[warp]);
    }
  }
  prefetch_first_columns<S4, SH>(L, nin.stage_w != 0);
  const FinishPre pre = first_pass_prefetch<MB, SH>(L, cv, rows);
  const int chunks = K / 8;
  uint4 nw[4];               // the norm weights of this thread's chunks: constants, fetched ahead of the wait
  if (nin.a_int8 == nullptr) {
#pragma unroll
    for (int i = 0; i < 4; ++i) nw[i] = __ldg(reinterpret_cast<const uint4*>(nin.weight) + min(threadIdx.x + i * kThreads, chunks - 1));
  }
  grid_dependency_wait();
  if (nin.a_int8 != nullptr) {
    for (int m = 0; m < MB; ++m) {
      const int row = min(m, rows - 1);
      for (int c = threadIdx.x; c < K / 16; c += kThreads)
        *(reinterpret_cast<uint4*>(sA + (int64_t)m * K) + c) = __ldcg(reinterpret_cast<const uint4*>(nin.a_int8 + (int64_t)row * nin.x_stride) + c);
    }
    __syncthreads();
    stream_columns<MB, S4, SH>(L, cv, sA, rows, pre, sw, &wbar[threadIdx.x >> 5], status);
    return;
  }
  const float inv_scale = 1.0f / nin.out_scale;
  for (int m = 0; m < MB; ++m) {
    const int row = min(m, rows - 1);
    // a thread keeps its (at most four) chunks of eight values in registers between the two passes
    float v[4][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < chunks) {
        // x and the residual come from the kernels just before: L2 reads (__ldcg), see grid_dependency_launch
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(nin.x + (int64_t)row * nin.x_stride) + c);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); v[i][2 * e] = f.x; v[i][2 * e + 1] = f.y; }
        if (nin.residual != nullptr) {
          if (nin.res_f32) {
            const float4* r = reinterpret_cast<const float4*>(static_cast<const float*>(nin.residual) + (int64_t)row * nin.res_stride) + 2 * c;
            const float4 a = __ldcg(r), b = __ldcg(r + 1);
            v[i][0] += a.x; v[i][1] += a.y; v[i][2] += a.z; v[i][3] += a.w;
            v[i][4] += b.x; v[i][5] += b.y; v[i][6] += b.z; v[i][7] += b.w;
          } else {
            const uint4 rr = __ldcg(reinterpret_cast<const uint4*>(static_cast<const __half*>(nin.residual) + (int64_t)row * nin.res_stride) + c);
            const __half2* rh = reinterpret_cast<const __half2*>(&rr);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(rh[e]); v[i][2 * e] += f.x; v[i][2 * e + 1] += f.y; }
          }
        }
        if (nin.residual_out != nullptr && blockIdx.x == 0 && m < rows) {
          if (nin.res_out_f32) {
            float4* o = reinterpret_cast<float4*>(static_cast<float*>(nin.residual_out) + (int64_t)row * nin.res_out_stride) + 2 * c;
            o[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
            o[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
          } else {
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(v[i][2 * e], v[i][2 * e + 1]);
            *(reinterpret_cast<uint4*>(static_cast<__half*>(nin.residual_out) + (int64_t)row * nin.res_out_stride) + c) = o;
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += v[i][e] * v[i][e];
      }
    }
    const float rstd = 1.0f / sqrtf(block_sum(sum, red) / (float)K + nin.eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < chunks) {
        const __half2* wh = reinterpret_cast<const __half2*>(&nw[i]);
        int q[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 w2 = __half22float2(wh[e]);
          q[2 * e] = __float2int_rn(v[i][2 * e] * rstd * w2.x * inv_scale);
          q[2 * e + 1] = __float2int_rn(v[i][2 * e + 1] * rstd * w2.y * inv_scale);
        }
        uint2 o;
        o.x = pack4_sat_s8(q[0], q[1], q[2], q[3]);
        o.y = pack4_sat_s8(q[4], q[5], q[6], q[7]);
        *(reinterpret_cast<uint2*>(sA + (int64_t)m * K) + c) = o;
      }
    }
  }
  __syncthreads();
  stream_columns<MB, S4, SH>(L, cv, sA, rows, pre, sw, &wbar[threadIdx.x >> 5], status);
}

// ---- launch 3: gate, grouped RMSNorm, Hadamard rotation, quantise -> product -------------------------------------------
struct GateIn {
  const __half* y;          // (rows, d)
  const int8_t* z;          // (rows, d) with row stride z_stride
  const __half* weight;     // (d)
  int64_t y_stride, z_stride;
  int early_launch;
  int d, group_size, special, table;    // d = special_rows * 128; table: index into c_dec_neg, or -1 for Sylvester rows
  float z_scale, eps, had_scale;        // had_scale: (1 / sqrt(d)) / x_H_scale
};

// The gated norm + Hadamard + quantise of one row, spread over S = d / 128 CTAs of 128 threads: every CTA gates,
// normalises and runs the 128-point stage on the whole row (a few hundred instructions per thread, all in registers and
// shuffles), then produces ONE block of 128 outputs of the S-point stage (S multiply-adds per thread).  Doing the S-point
// stage for all S blocks in every CTA of the product kernel was tried first: 5 000 instructions per warp of serial
// prologue, 28 us for a 6.6 MB product.
constexpr int kHadThreads = 256;
constexpr int kHadWarps = kHadThreads / 32;
constexpr int kMaxRowsPerWarp = 8;       // d / 128 <= 64 rows of 128 over 8 warps

__constant__ unsigned long long c_dec_neg[4][40];     // row i of the order-12 / 20 / 28 / 40 matrix: bit j set <=> entry -1

__global__ void __launch_bounds__(kHadThreads)
decode_gate_had_quant_kernel(GateIn gin, int8_t* __restrict__ out, int64_t out_stride) {
  extern __shared__ __align__(16) uint8_t dsm[];
  __shared__ float gsum[64], rowsum[64];
  const int D = gin.d, S = D / 128;
  float* buf = reinterpret_cast<float*>(dsm);                         // d floats: the row after the 128-point stage
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y, iout = blockIdx.x;
  if (gin.early_launch) grid_dependency_launch();
  // constants first (norm weights, the sign row of this CTA's output block): they do not depend on the kernel before
  uint2 wr[kMaxRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kMaxRowsPerWarp; ++i)
    wr[i] = __ldg(reinterpret_cast<const uint2*>(gin.weight + min(warp + i * kHadWarps, S - 1) * 128) + lane);
  const unsigned long long neg = gin.table >= 0 ? c_dec_neg[gin.table][iout] : 0ull;
  grid_dependency_wait();
  // A warp owns rows r = warp, warp + 8, ... of the (S x 128) view; a lane holds four neighbours of each.
  float f[kMaxRowsPerWarp][4];
  uint2 yr[kMaxRowsPerWarp];
  uint32_t zr[kMaxRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kMaxRowsPerWarp; ++i) {
    const int r = min(warp + i * kHadWarps, S - 1);
    yr[i] = __ldcg(reinterpret_cast<const uint2*>(gin.y + (int64_t)row * gin.y_stride + r * 128) + lane);   // L2 reads:
    zr[i] = __ldcg(reinterpret_cast<const uint32_t*>(gin.z + (int64_t)row * gin.z_stride + r * 128) + lane); // see grid_dependency_launch
  }
#pragma unroll
  for (int i = 0; i < kMaxRowsPerWarp; ++i) {
    const int r = warp + i * kHadWarps;
    const __half2* h = reinterpret_cast<const __half2*>(&yr[i]);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    f[i][0] = a.x; f[i][1] = a.y; f[i][2] = b.x; f[i][3] = b.y;
    const uint32_t zw = zr[i] ^ 0x80808080u;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float hz = s8f(zw, e) * (0.5f * gin.z_scale);
      f[i][e] *= fmaf(hz, tanh_approx(hz), hz);           // y * silu(z)
      ss += f[i][e] * f[i][e];
    }
    if (r < S) {                                           // warp-uniform
      ss = warp_sum_f(ss);
      if (lane == 0) rowsum[r] = ss;
    }
  }
  __syncthreads();
  // group sums in a fixed order (no atomics: the result must not depend on which warp arrives first): warp g adds the
  // rows of group g, lane-strided partial sums then a shuffle tree
  {
    const int ngroups = D / gin.group_size, rows_per_group = gin.group_size / 128;
    for (int g = warp; g < ngroups; g += kHadWarps) {
      float t = 0.f;
      for (int r = lane; r < rows_per_group; r += 32) t += rowsum[g * rows_per_group + r];
      t = warp_sum_f(t);
      if (lane == 0) gsum[g] = t;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kMaxRowsPerWarp; ++i) {
    const int r = warp + i * kHadWarps;
    if (r < S) {
      // normalise and round to fp16 as the separate norm kernel stores it
      const float rstd = 1.0f / sqrtf(gsum[(r * 128) / gin.group_size] / (float)gin.group_size + gin.eps);
      const __half2* wh = reinterpret_cast<const __half2*>(&wr[i]);
      const float2 w0 = __half22float2(wh[0]), w1 = __half22float2(wh[1]);
      const float t0 = __half2float(__float2half_rn(f[i][0] * rstd * w0.x)), t1 = __half2float(__float2half_rn(f[i][1] * rstd * w0.y));
      const float t2 = __half2float(__float2half_rn(f[i][2] * rstd * w1.x)), t3 = __half2float(__float2half_rn(f[i][3] * rstd * w1.y));
      // H_128 along the row: strides 1 and 2 inside the lane, 4 .. 64 through shuffles
      const float e0 = t0 + t1, e1 = t0 - t1, e2 = t2 + t3, e3 = t2 - t3;
      float g[4] = {e0 + e2, e1 + e3, e0 - e2, e1 - e3};
#pragma unroll
      for (int mk = 1; mk < 32; mk <<= 1) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float o = __shfl_xor_sync(0xffffffffu, g[k], mk);
          g[k] = (lane & mk) ? o - g[k] : g[k] + o;
        }
      }
      *reinterpret_cast<float4*>(buf + r * 128 + 4 * lane) = make_float4(g[0], g[1], g[2], g[3]);
    }
  }
  __syncthreads();
  // output block iout of the S-point stage: threads (column, half of the terms); signs from the row's bit mask (order
  // 12 .. 40) or the Sylvester rule (power-of-two S); two partial sums per thread, combined through shared memory
  {
    const int col = threadIdx.x & 127, half = threadIdx.x >> 7;
    const int j0 = half * ((S + 1) / 2), j1 = min(S, j0 + (S + 1) / 2);
    float a0 = 0.f, a1 = 0.f;
    for (int j = j0; j < j1; j += 2) {
      const float b0 = buf[j * 128 + col];
      const float b1 = j + 1 < j1 ? buf[(j + 1) * 128 + col] : 0.f;
      const uint32_t s0 = gin.table >= 0 ? (uint32_t)((neg >> j) & 1ull) : (uint32_t)(__popc(iout & j) & 1);
      const uint32_t s1 = gin.table >= 0 ? (uint32_t)((neg >> (j + 1)) & 1ull) : (uint32_t)(__popc(iout & (j + 1)) & 1);
      a0 += __uint_as_float(__float_as_uint(b0) ^ (s0 << 31));
      a1 += __uint_as_float(__float_as_uint(b1) ^ (s1 << 31));
    }
    __syncthreads();                       // all reads of buf are done: its first 128 floats carry the upper half's sums
    if (half == 1) buf[col] = a0 + a1;
    __syncthreads();
    if (half == 0)
      out[(int64_t)row * out_stride + iout * 128 + col] = (int8_t)round_away_s8(((a0 + a1) + buf[col]) * gin.had_scale);
  }
}

int upload_tables() {
  static bool done[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return QB_OK;
  const unsigned long long* masks[4] = {kHadNeg12, kHadNeg20, kHadNeg28, kHadNeg40};
  const int order[4] = {12, 20, 28, 40};
  static unsigned long long hmask[4][40];
  for (int t = 0; t < 4; ++t)
    for (int i = 0; i < 40; ++i) hmask[t][i] = i < order[t] ? masks[t][i] : 0ull;
  QB_CUDA_OK(cudaMemcpyToSymbol(c_dec_neg, hmask, sizeof(hmask)));
  if (dev < 64) done[dev] = true;
  return QB_OK;
}

int fill_linear(Linear& L, const void* w, const float* s_ch, const float* s_tok, void* out, int64_t out_stride, int n, int k,
                int s4, int out_int8, const char* who) {
  QB_REQUIRE(w && s_ch && s_tok && out, QB_ERR_INVALID_ARG, "%s: null pointer", who);
  QB_REQUIRE(n > 0 && k > 0 && k % 32 == 0 && aligned(w, 16), QB_ERR_INVALID_ARG, "%s: k must be a multiple of 32 and the weights 16-byte aligned", who);
  QB_REQUIRE(out_stride >= n, QB_ERR_INVALID_ARG, "%s: out_row_stride smaller than n", who);
  L.w = static_cast<const uint8_t*>(w); L.s_ch = s_ch; L.s_tok = s_tok; L.out = out; L.out_stride = out_stride;
  L.n = n; L.k = k; L.out_int8 = out_int8;
  (void)s4;
  return QB_OK;
}

unsigned grid_for(int n, int ctas_per_sm, int nw) {
  return (unsigned)std::min<int64_t>(ceil_div(n, kWarps * nw), (int64_t)sm_count() * ctas_per_sm);
}

template <typename K>
int opt_in_smem(K kernel, size_t bytes) {
  // per device and per kernel: the attribute is set on every launch that needs it (a cheap host-side call)
  if (bytes > 48 * 1024) QB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return QB_OK;
}

}  // namespace
}  // namespace qb

using namespace qb;

#define QB_LAUNCH_ONE(KERNEL, MBV, WMV, grid, smem, st, ...)                                                             \
  { if (sh__) { rc__ = opt_in_smem(KERNEL<MBV, WMV, 1>, smem); if (rc__ == QB_OK) launch_dependent(KERNEL<MBV, WMV, 1>, grid, dim3(kThreads), smem, st, __VA_ARGS__); } \
    else { rc__ = opt_in_smem(KERNEL<MBV, WMV, 0>, smem); if (rc__ == QB_OK) launch_dependent(KERNEL<MBV, WMV, 0>, grid, dim3(kThreads), smem, st, __VA_ARGS__); } }
#define QB_DISPATCH_WM(KERNEL, MBV, wm, grid, smem, st, ...)                                                             \
  if (wm == 2) QB_LAUNCH_ONE(KERNEL, MBV, 2, grid, smem, st, __VA_ARGS__)                                                 \
  else if (wm == 1) QB_LAUNCH_ONE(KERNEL, MBV, 1, grid, smem, st, __VA_ARGS__)                                            \
  else QB_LAUNCH_ONE(KERNEL, MBV, 0, grid, smem, st, __VA_ARGS__)
#define QB_DISPATCH_MB_S4(KERNEL, rows, wm, sh, grid, smem, st, ...)                                                      \
  do {                                                                                                                    \
    int rc__ = QB_OK;                                                                                                     \
    const int sh__ = (sh);                                                                                                \
    if (rows == 1) { QB_DISPATCH_WM(KERNEL, 1, wm, grid, smem, st, __VA_ARGS__) }                                         \
    else if (rows == 2) { QB_DISPATCH_WM(KERNEL, 2, wm, grid, smem, st, __VA_ARGS__) }                                    \
    else { QB_DISPATCH_WM(KERNEL, 4, wm, grid, smem, st, __VA_ARGS__) }                                                   \
    if (rc__ != QB_OK) return rc__;                                                                                       \
  } while (0)

extern "C" int qb_decode_norm_linear(const qb_decode_norm_linear_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && ((a->x && a->norm_weight) || a->a_int8), QB_ERR_INVALID_ARG, "decode_norm_linear: null pointer");
  QB_REQUIRE(a->rows >= 1 && a->rows <= kMaxRows, QB_ERR_UNSUPPORTED, "decode_norm_linear: 1 to %d rows", kMaxRows);
  QB_REQUIRE(a->k <= 8192 && a->k % 32 == 0, QB_ERR_UNSUPPORTED, "decode_norm_linear: k must be a multiple of 32, at most 8192");
  QB_REQUIRE(a->a_int8 != nullptr || a->norm_out_scale != 0.0f, QB_ERR_INVALID_ARG, "decode_norm_linear: the norm's output scale is zero");
  QB_REQUIRE(a->a_int8 == nullptr || (aligned(a->a_int8, 16) && a->x_row_stride % 16 == 0), QB_ERR_INVALID_ARG,
             "decode_norm_linear: int8 input rows must be 16-byte aligned");
  QB_REQUIRE(a->a_int8 != nullptr || (aligned(a->x, 16) && a->x_row_stride % 8 == 0 && aligned(a->norm_weight, 16)) &&
             (a->residual == nullptr || (aligned(a->residual, 16) && a->residual_row_stride % 8 == 0)) &&
             (a->residual_out == nullptr || (aligned(a->residual_out, 16) && a->residual_out_row_stride % 8 == 0)),
             QB_ERR_INVALID_ARG, "decode_norm_linear: rows must be 16-byte aligned");
  Linear L{};
  int rc = fill_linear(L, a->w, a->s_channel_nat, a->s_tok, a->out, a->out_row_stride, a->n, a->k, a->w_is_s4, a->out_int8,
                       "decode_norm_linear");
  if (rc != QB_OK) return rc;
  NormIn nin{};
  nin.a_int8 = a->a_int8;
  nin.x = static_cast<const __half*>(a->x); nin.residual = a->residual; nin.residual_out = a->residual_out;
  nin.weight = static_cast<const __half*>(a->norm_weight);
  nin.x_stride = a->x_row_stride; nin.res_stride = a->residual_row_stride; nin.res_out_stride = a->residual_out_row_stride;
  nin.res_f32 = a->residual_is_f32; nin.res_out_f32 = a->residual_out_is_f32; nin.eps = a->eps; nin.out_scale = a->norm_out_scale;
  nin.early_launch = a->early_launch;
  ConvEpi cv{};
  if (a->conv_state != nullptr) {
    QB_REQUIRE(a->out_int8 && a->conv_weight && a->conv_x && a->conv_B && a->conv_C && a->x_out_scale && a->B_out_scale && a->C_out_scale,
               QB_ERR_INVALID_ARG, "decode_norm_linear: the conv epilogue needs an int8 product and all conv pointers");
    QB_REQUIRE(a->conv_dim == a->conv_x_dim + 2 * a->conv_gn && a->conv_col0 >= 0 && a->conv_col0 + a->conv_dim <= a->n,
               QB_ERR_INVALID_ARG, "decode_norm_linear: conv channels out of the product's columns");
    cv.enabled = 1; cv.state = a->conv_state; cv.sb = a->conv_state_sb; cv.sd = a->conv_state_sd; cv.sw = a->conv_state_sw;
    cv.weight = a->conv_weight; cv.bias = a->conv_bias; cv.dst[0] = a->conv_x; cv.dst[1] = a->conv_B; cv.dst[2] = a->conv_C;
    cv.out_scale[0] = a->x_out_scale; cv.out_scale[1] = a->B_out_scale; cv.out_scale[2] = a->C_out_scale;
    cv.scale_in[0] = a->conv_scale_in_x; cv.scale_in[1] = a->conv_scale_in_B; cv.scale_in[2] = a->conv_scale_in_C;
    cv.scale_bias[0] = a->conv_scale_bias_x; cv.scale_bias[1] = a->conv_scale_bias_B; cv.scale_bias[2] = a->conv_scale_bias_C;
    cv.c0 = a->conv_col0; cv.dim = a->conv_dim; cv.end0 = a->conv_x_dim; cv.end1 = a->conv_x_dim + a->conv_gn;
  }
  const int mb = a->rows <= 2 ? a->rows : 4;
  size_t smem = (size_t)mb * a->k;
  // five columns per warp in one pass when the columns are short (at most 96 chunks) and two per warp would take more
  // than one pass of the resident warps
  const int chunks = a->w_is_s4 != 0 ? a->k / 32 : a->k / 16;
  const int sh = chunks <= 96 && (int64_t)a->n > (int64_t)sm_count() * 2 * kWarps * 2 ? 1 : 0;
  const dim3 grid(grid_for(a->n, 2, sh ? 5 : 2));
  // first-pass weights staged in shared memory when two CTAs of the kernel still fit an SM with them
  const size_t row_bytes = a->w_is_s4 != 0 ? (size_t)a->k / 2 : (size_t)a->k;
  const size_t stage_bytes = (size_t)kWarps * (sh ? 5 : 2) * row_bytes;
  const size_t smem_staged = ((smem + 15) & ~(size_t)15) + stage_bytes;
  nin.stage_w = row_bytes % 16 == 0 && smem_staged <= 100 * 1024 ? 1 : 0;
  if (nin.stage_w) smem = smem_staged;
  int* status = device_status_ptr();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "decode_norm_linear: device status word unavailable");
  cudaStream_t st = (cudaStream_t)stream;
  const int rows = a->rows;
  const int wm = a->w_is_s4 == 0 ? 0 : (a->s_group_nat != nullptr ? 2 : 1);
  if (wm == 2) {
    QB_REQUIRE(a->k % 128 == 0 && aligned(a->s_group_nat, 2), QB_ERR_INVALID_ARG, "decode_norm_linear: group scales need k to be a multiple of 128");
    L.s_grp = static_cast<const __half*>(a->s_group_nat);
  }
  QB_DISPATCH_MB_S4(decode_norm_linear_kernel, mb, wm, sh, grid, smem, st, nin, L, cv, rows, status);
  QB_LAUNCH_OK("decode_norm_linear_kernel");
  return QB_OK;
}

extern "C" int qb_decode_gate_had_quant(const qb_decode_gate_had_quant_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->y && a->z && a->norm_weight && a->out, QB_ERR_INVALID_ARG, "decode_gate_had_quant: null pointer");
  QB_REQUIRE(a->rows >= 1 && a->rows <= 65535, QB_ERR_INVALID_ARG, "decode_gate_had_quant: bad row count");
  QB_REQUIRE(a->d > 0 && a->d % 128 == 0, QB_ERR_UNSUPPORTED, "decode_gate_had_quant: d must be a multiple of 128");
  const int S = a->d / 128;
  int table = -1;
  if (S == 12 || S == 20 || S == 28 || S == 40) table = S == 12 ? 0 : (S == 20 ? 1 : (S == 28 ? 2 : 3));
  else QB_REQUIRE(S >= 1 && S <= 64 && (S & (S - 1)) == 0, QB_ERR_UNSUPPORTED, "decode_gate_had_quant: d / 128 must be 12, 20, 28, 40 or a power of two <= 64");
  QB_REQUIRE(a->group_size > 0 && a->d % a->group_size == 0 && a->group_size % 128 == 0 && a->d / a->group_size <= 64, QB_ERR_UNSUPPORTED,
             "decode_gate_had_quant: the norm group size must be a multiple of 128 that divides d");
  QB_REQUIRE(aligned(a->y, 8) && a->y_row_stride % 4 == 0 && aligned(a->z, 4) && a->z_row_stride % 4 == 0 && aligned(a->norm_weight, 8) &&
             a->out_row_stride >= a->d, QB_ERR_INVALID_ARG, "decode_gate_had_quant: rows must be 8-byte aligned (z: 4)");
  int rc = upload_tables();
  if (rc != QB_OK) return rc;
  GateIn gin{};
  gin.y = static_cast<const __half*>(a->y); gin.z = a->z; gin.weight = static_cast<const __half*>(a->norm_weight);
  gin.y_stride = a->y_row_stride; gin.z_stride = a->z_row_stride; gin.d = a->d; gin.group_size = a->group_size; gin.special = S;
  gin.table = table; gin.z_scale = a->z_scale; gin.eps = a->eps; gin.had_scale = a->had_scale; gin.early_launch = a->early_launch;
  launch_dependent(decode_gate_had_quant_kernel, dim3((unsigned)S, (unsigned)a->rows), dim3(kHadThreads), (size_t)a->d * 4,
                   (cudaStream_t)stream, gin, a->out, a->out_row_stride);
  QB_LAUNCH_OK("decode_gate_had_quant_kernel");
  return QB_OK;
}
