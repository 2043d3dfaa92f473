// Quantised RMSNorm (+ residual add) and gated, grouped RMSNorm for sm_100a.
//
// Both are one streaming pass: a normalised segment (a row, or one group of a row) is held in registers by
// 32 * WPR threads (16-byte loads, eight fp16 values per chunk), reduced with shuffles (and one shared-memory
// hop when several warps share a segment), scaled, and written as int8 (static or per-token scale) or fp16.
// Arithmetic follows the reference's Triton kernels: fp32 throughout, rstd = 1 / sqrt(mean(x^2) + eps),
// y = x * rstd * w (+ b), int8 = clamp(rint(y / scale)).
#include "common.cuh"

namespace qb {
namespace {

enum { kOutS8Static = 0, kOutS8Dynamic = 1, kOutF16 = 2 };

struct NormParams {
  const __half* x;
  const void* residual;
  void* residual_out;
  const int8_t* z;
  const __half* w;
  const __half* bias;
  void* y;
  float* dyn_scale;
  int64_t x_stride, res_stride, res_out_stride, z_stride, y_stride;
  int M, N, ngroups;      // N: elements per normalised segment
  int res_f32, res_out_f32, out_kind, gate_first, rms, pad_zero;
  int early;              // let the next programmatic launch start while this kernel runs (early_overlap())
  int n_partials, own_index;       // > 1: x is the fp16-rounded fp32 sum of n_partials inputs
  int64_t partial_stride;          // partial p at x + p * partial_stride, p == own_index at own (when given)
  const __half* own;
  float eps, out_scale, z_scale;
};

constexpr int kCH = 8;           // 16-byte chunks per thread, at most
constexpr int kNormWarps = 8;    // warps per CTA (16 when one segment needs 16 warps)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduction over the WPR warps of one segment.  Every thread of the CTA calls it (segments past the end carry
// neutral values), so the barrier is CTA-wide.
template <int WPR, bool MAX>
__device__ __forceinline__ float seg_reduce(float v, float* red, int warp, int lane) {
  v = MAX ? warp_max(v) : warp_sum(v);
  if (WPR == 1) return v;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int base = (warp / WPR) * WPR;
  float r = red[base];
#pragma unroll
  for (int i = 1; i < WPR; ++i) r = MAX ? fmaxf(r, red[base + i]) : r + red[base + i];
  return r;
}

// int8 -> float without a conversion instruction: byte k of w (biased by 128) under the exponent of 2^23.
__device__ __forceinline__ float s8_to_float(uint32_t w_biased, int k) {
  const uint32_t bits = __byte_perm(w_biased, 0x4B000000u, 0x7650 + k);   // {b_k, 0x00, 0x00, 0x4B}
  return __uint_as_float(bits) - 8388736.0f;                                // 2^23 + 128
}

// GATE: 0 no gate, 1 x * silu(z) before the norm, 2 y * silu(z) after it.  CH: 16-byte chunks per thread.
// Every global load of the segment is issued before the first use (clamped addresses, no branches around the loads),
// so a thread has all its chunks in flight at once.
template <int WPR, int GATE, int CH>
__global__ void __launch_bounds__((WPR > kNormWarps ? WPR : kNormWarps) * 32)
norm_quant_kernel(const NormParams p) {
  constexpr int WARPS = WPR > kNormWarps ? WPR : kNormWarps;
  constexpr int T = 32 * WPR;                 // threads per segment
  __shared__ float red[WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t units = (int64_t)p.M * p.ngroups;
  const int64_t unit_raw = (int64_t)blockIdx.x * (WARPS / WPR) + warp / WPR;
  const bool live = unit_raw < units;
  const int64_t unit = live ? unit_raw : units - 1;
  const int row = (int)(unit / p.ngroups), grp = (int)(unit % p.ngroups);
  const int t = (warp % WPR) * 32 + lane;
  const int chunks = p.N >> 3;
  const int64_t col0 = (int64_t)grp * p.N;
  int cc[CH];
  bool on[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) { const int c = t + i * T; on[i] = c < chunks; cc[i] = on[i] ? c : chunks - 1; }

  if (p.early) grid_dependency_launch();
  // weights do not depend on the kernel before this one: fetch them ahead of the dependency wait
  uint4 wr[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) wr[i] = __ldg(reinterpret_cast<const uint4*>(p.w + col0) + cc[i]);
  grid_dependency_wait();

  uint4 xr[CH];
  uint2 zr[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) xr[i] = ld_act(reinterpret_cast<const uint4*>(p.x + (int64_t)row * p.x_stride + col0) + cc[i]);
  if (GATE != 0) {
#pragma unroll
    for (int i = 0; i < CH; ++i) zr[i] = ld_act(reinterpret_cast<const uint2*>(p.z + (int64_t)row * p.z_stride + col0) + cc[i]);
  }
  if (GATE == 0 && p.n_partials > 1) {
    float xs[CH][8];
#pragma unroll 1
    for (int s = 0; s < p.n_partials; ++s) {
      const __half* base = (s == p.own_index && p.own != nullptr) ? p.own : p.x + (int64_t)s * p.partial_stride;
      uint4 t[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) t[i] = ld_act(reinterpret_cast<const uint4*>(base + (int64_t)row * p.x_stride + col0) + cc[i]);
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const __half2* h = reinterpret_cast<const __half2*>(&t[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          xs[i][2 * e] = s == 0 ? f.x : xs[i][2 * e] + f.x;
          xs[i][2 * e + 1] = s == 0 ? f.y : xs[i][2 * e + 1] + f.y;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      __half2* h = reinterpret_cast<__half2*>(&xr[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(xs[i][2 * e], xs[i][2 * e + 1]);
    }
  }
  float v[CH][8];
  if (GATE == 0 && p.residual != nullptr && p.res_f32) {
    float4 ra[CH], rb[CH];
    const float4* r = reinterpret_cast<const float4*>(static_cast<const float*>(p.residual) + (int64_t)row * p.res_stride + col0);
#pragma unroll
    for (int i = 0; i < CH; ++i) { ra[i] = ld_act(r + 2 * cc[i]); rb[i] = ld_act(r + 2 * cc[i] + 1); }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      v[i][0] = ra[i].x; v[i][1] = ra[i].y; v[i][2] = ra[i].z; v[i][3] = ra[i].w;
      v[i][4] = rb[i].x; v[i][5] = rb[i].y; v[i][6] = rb[i].z; v[i][7] = rb[i].w;
    }
  } else if (GATE == 0 && p.residual != nullptr) {
    uint4 rr[CH];
    const uint4* r = reinterpret_cast<const uint4*>(static_cast<const __half*>(p.residual) + (int64_t)row * p.res_stride + col0);
#pragma unroll
    for (int i = 0; i < CH; ++i) rr[i] = ld_act(r + cc[i]);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const __half2* rh = reinterpret_cast<const __half2*>(&rr[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(rh[e]); v[i][2 * e] = f.x; v[i][2 * e + 1] = f.y; }
    }
  } else {
#pragma unroll
    for (int i = 0; i < CH; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
  }
  float sum = 0.f;
  float gate[GATE == 2 ? CH : 1][8];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const __half2* h = reinterpret_cast<const __half2*>(&xr[i]);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); v[i][2 * e] += f.x; v[i][2 * e + 1] += f.y; }
    if (GATE == 0 && p.residual_out != nullptr && live && on[i]) {
      if (p.res_out_f32) {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.residual_out) + (int64_t)row * p.res_out_stride + col0) + 2 * cc[i];
        o[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
        o[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
      } else {
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(v[i][2 * e], v[i][2 * e + 1]);
        *(reinterpret_cast<uint4*>(static_cast<__half*>(p.residual_out) + (int64_t)row * p.res_out_stride + col0) + cc[i]) = o;
      }
    }
    if (GATE != 0) {
      const uint32_t zw[2] = {zr[i].x ^ 0x80808080u, zr[i].y ^ 0x80808080u};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float hz = s8_to_float(zw[e >> 2], e & 3) * (0.5f * p.z_scale);      // z / 2
        const float sg = fmaf(hz, tanh_approx(hz), hz);                               // z * sigmoid(z)
        if (GATE == 1) v[i][e] *= sg; else gate[GATE == 2 ? i : 0][e] = sg;
      }
    }
    if (on[i]) {
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += p.rms ? v[i][e] * v[i][e] : v[i][e];
    }
  }
  const float inv_n = 1.0f / (float)p.N;
  float mean = 0.f, var;
  if (p.rms) {
    var = seg_reduce<WPR, false>(sum, red, warp, lane) * inv_n;
  } else {
    mean = seg_reduce<WPR, false>(sum, red, warp, lane) * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i)
      if (on[i]) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float d = v[i][e] - mean; sq += d * d; }
      }
    var = seg_reduce<WPR, false>(sq, red, warp, lane) * inv_n;
  }
  const float rstd = 1.0f / sqrtf(var + p.eps);

  float mx = p.pad_zero ? 0.f : -INFINITY;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const __half2* wh = reinterpret_cast<const __half2*>(&wr[i]);
    uint4 br = make_uint4(0, 0, 0, 0);
    if (p.bias != nullptr) br = __ldg(reinterpret_cast<const uint4*>(p.bias + col0) + cc[i]);
    const __half2* bh = reinterpret_cast<const __half2*>(&br);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 w2 = __half22float2(wh[e]);
      float y0 = (v[i][2 * e] - mean) * rstd * w2.x;
      float y1 = (v[i][2 * e + 1] - mean) * rstd * w2.y;
      if (p.bias != nullptr) { const float2 b2 = __half22float2(bh[e]); y0 += b2.x; y1 += b2.y; }
      if (GATE == 2) { y0 *= gate[GATE == 2 ? i : 0][2 * e]; y1 *= gate[GATE == 2 ? i : 0][2 * e + 1]; }
      v[i][2 * e] = y0; v[i][2 * e + 1] = y1;
      if (on[i]) mx = fmaxf(mx, fmaxf(y0, y1));
    }
  }
  float inv_scale = 0.f;
  if (p.out_kind == kOutS8Static) {
    inv_scale = 1.0f / p.out_scale;
  } else if (p.out_kind == kOutS8Dynamic) {
    const float scale = seg_reduce<WPR, true>(mx, red, warp, lane) / 127.0f;
    if (live && t == 0) p.dyn_scale[(int64_t)grp * p.M + row] = scale;
    inv_scale = 1.0f / scale;
  }
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    if (live && on[i]) {
      if (p.out_kind == kOutF16) {
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(v[i][2 * e], v[i][2 * e + 1]);
        *(reinterpret_cast<uint4*>(static_cast<__half*>(p.y) + (int64_t)row * p.y_stride + col0) + cc[i]) = o;
      } else {
        int q[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) q[e] = __float2int_rn(v[i][e] * inv_scale);
        uint2 o;
        o.x = pack4_sat_s8(q[0], q[1], q[2], q[3]);
        o.y = pack4_sat_s8(q[4], q[5], q[6], q[7]);
        *(reinterpret_cast<uint2*>(static_cast<int8_t*>(p.y) + (int64_t)row * p.y_stride + col0) + cc[i]) = o;
      }
    }
  }
}

// Any segment length and alignment: one CTA per segment, three strided passes over global memory.
__global__ void __launch_bounds__(256) norm_quant_generic_kernel(const NormParams p) {
  __shared__ float red[8];
  if (p.early) grid_dependency_launch();
  grid_dependency_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x / p.ngroups, grp = blockIdx.x % p.ngroups;
  const int64_t col0 = (int64_t)grp * p.N;
  auto load = [&](int j, float& zsig) {
    float x = __half2float(ld_act(p.x + (int64_t)row * p.x_stride + col0 + j));
    if (p.n_partials > 1) {
      float acc = 0.f;
      for (int s = 0; s < p.n_partials; ++s) {
        const __half* base = (s == p.own_index && p.own != nullptr) ? p.own : p.x + (int64_t)s * p.partial_stride;
        acc += __half2float(ld_act(base + (int64_t)row * p.x_stride + col0 + j));
      }
      x = __half2float(__float2half_rn(acc));
    }
    if (p.residual != nullptr)
      x += p.res_f32 ? ld_act(static_cast<const float*>(p.residual) + (int64_t)row * p.res_stride + col0 + j)
                     : __half2float(ld_act(static_cast<const __half*>(p.residual) + (int64_t)row * p.res_stride + col0 + j));
    zsig = 1.f;
    if (p.z != nullptr) {
      const float zf = (float)ld_act(p.z + (int64_t)row * p.z_stride + col0 + j) * p.z_scale;
      zsig = zf * (1.0f / (1.0f + __expf(-zf)));
      if (p.gate_first) x *= zsig;
    }
    return x;
  };
  auto reduce = [&](float v, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < 8; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    return r;
  };
  float s = 0.f, zsig;
  for (int j = threadIdx.x; j < p.N; j += 256) {
    const float x = load(j, zsig);
    if (p.residual_out != nullptr) {
      if (p.res_out_f32) static_cast<float*>(p.residual_out)[(int64_t)row * p.res_out_stride + col0 + j] = x;
      else static_cast<__half*>(p.residual_out)[(int64_t)row * p.res_out_stride + col0 + j] = __float2half_rn(x);
    }
    s += p.rms ? x * x : x;
  }
  const float inv_n = 1.0f / (float)p.N;
  float mean = 0.f, var;
  if (p.rms) {
    var = reduce(s, false) * inv_n;
  } else {
    mean = reduce(s, false) * inv_n;
    float sq = 0.f;
    for (int j = threadIdx.x; j < p.N; j += 256) { const float d = load(j, zsig) - mean; sq += d * d; }
    var = reduce(sq, false) * inv_n;
  }
  const float rstd = 1.0f / sqrtf(var + p.eps);
  auto value = [&](int j) {
    float zg;
    float y = (load(j, zg) - mean) * rstd * __half2float(p.w[col0 + j]);
    if (p.bias != nullptr) y += __half2float(p.bias[col0 + j]);
    if (p.z != nullptr && !p.gate_first) y *= zg;
    return y;
  };
  float scale = p.out_scale;
  if (p.out_kind == kOutS8Dynamic) {
    float mx = p.pad_zero ? 0.f : -INFINITY;
    for (int j = threadIdx.x; j < p.N; j += 256) mx = fmaxf(mx, value(j));
    scale = reduce(mx, true) / 127.0f;
    if (threadIdx.x == 0) p.dyn_scale[(int64_t)grp * p.M + row] = scale;
  }
  for (int j = threadIdx.x; j < p.N; j += 256) {
    const float y = value(j);
    if (p.out_kind == kOutF16) static_cast<__half*>(p.y)[(int64_t)row * p.y_stride + col0 + j] = __float2half_rn(y);
    else static_cast<int8_t*>(p.y)[(int64_t)row * p.y_stride + col0 + j] = (int8_t)rint_s8(__fdiv_rn(y, scale));
  }
}

template <int WPR, int CH>
void launch_norm(const NormParams& p, int64_t units, cudaStream_t st) {
  constexpr int WARPS = WPR > kNormWarps ? WPR : kNormWarps;
  const dim3 grid((unsigned)ceil_div(units, WARPS / WPR)), block(WARPS * 32);
  if (p.z == nullptr) launch_dependent(norm_quant_kernel<WPR, 0, CH>, grid, block, 0, st, p);
  else if (p.gate_first) launch_dependent(norm_quant_kernel<WPR, 1, CH>, grid, block, 0, st, p);
  else launch_dependent(norm_quant_kernel<WPR, 2, CH>, grid, block, 0, st, p);
}

template <int WPR>
void launch_norm_ch(const NormParams& p, int64_t units, int ch, cudaStream_t st) {
  if (ch <= 1) launch_norm<WPR, 1>(p, units, st);
  else if (ch <= 2) launch_norm<WPR, 2>(p, units, st);
  else if (ch <= 3) launch_norm<WPR, 3>(p, units, st);
  else if (ch <= 4) launch_norm<WPR, 4>(p, units, st);
  else if (ch <= 5) launch_norm<WPR, 5>(p, units, st);
  else if (ch <= 6) launch_norm<WPR, 6>(p, units, st);
  else launch_norm<WPR, 8>(p, units, st);
}

int run_norm(const NormParams& p, cudaStream_t st) {
  const int64_t units = (int64_t)p.M * p.ngroups;
  if (units == 0) return QB_OK;
  bool vec = p.N % 8 == 0 && p.N <= 8 * kCH * 32 * 16 && aligned(p.x, 16) && p.x_stride % 8 == 0 && aligned(p.w, 16) &&
             aligned(p.y, 16) && p.y_stride % 16 == 0 && (p.bias == nullptr || aligned(p.bias, 16));
  if (p.residual) vec = vec && aligned(p.residual, 16) && p.res_stride % 8 == 0;
  if (p.residual_out) vec = vec && aligned(p.residual_out, 16) && p.res_out_stride % 8 == 0;
  if (p.z) vec = vec && aligned(p.z, 8) && p.z_stride % 8 == 0;
  if (p.n_partials > 1) vec = vec && p.partial_stride % 8 == 0 && (p.own == nullptr || aligned(p.own, 16));
  if (!vec) {
    QB_REQUIRE(units < (1ll << 31), QB_ERR_TOO_LARGE, "norm: too many rows");
    launch_dependent(norm_quant_generic_kernel, dim3((unsigned)units), dim3(256), 0, st, p);
    QB_LAUNCH_OK("norm_quant_generic_kernel");
    return QB_OK;
  }
  const int chunks = p.N / 8;
  // Warps per segment: the fewest that keep a thread at four chunks or less (five or six chunks cost 116 registers and
  // left two CTAs per SM: the 2560-wide block norm took 13.3 us against 11.7 us with three chunks per thread), more when
  // there are few segments (decode), down to two chunks per thread, to shorten the dependent chain.
  int wpr = 1;
  while (wpr < 16 && wpr * 32 * 4 < chunks) wpr *= 2;
  while (wpr < 8 && wpr * 64 < chunks && units * (2 * wpr) <= (int64_t)sm_count() * 2 * kNormWarps) wpr *= 2;
  const int ch = (int)ceil_div(chunks, wpr * 32);
  switch (wpr) {
    case 1: launch_norm_ch<1>(p, units, ch, st); break;
    case 2: launch_norm_ch<2>(p, units, ch, st); break;
    case 4: launch_norm_ch<4>(p, units, ch, st); break;
    case 8: launch_norm_ch<8>(p, units, ch, st); break;
    default: launch_norm_ch<16>(p, units, ch, st); break;
  }
  QB_LAUNCH_OK("norm_quant_kernel");
  return QB_OK;
}

int check_and_run(const qb_rmsnorm_args* a, bool gated, void* stream) {
  const char* who = gated ? "rmsnorm_gated" : "rmsnorm_quant";
  QB_REQUIRE(a != nullptr && a->x && a->weight && a->out, QB_ERR_INVALID_ARG, "%s: null pointer", who);
  QB_REQUIRE(a->rows >= 0 && a->group_size > 0 && a->ngroups > 0, QB_ERR_INVALID_ARG, "%s: bad shape", who);
  QB_REQUIRE(a->out_kind >= 0 && a->out_kind <= 2, QB_ERR_INVALID_ARG, "%s: out_kind must be 0, 1 or 2", who);
  QB_REQUIRE(a->out_kind != kOutS8Dynamic || a->dyn_scale != nullptr, QB_ERR_INVALID_ARG, "%s: per-token scales need dyn_scale", who);
  QB_REQUIRE(a->out_kind != kOutS8Static || a->out_scale != 0.0f, QB_ERR_INVALID_ARG, "%s: static output scale is zero", who);
  QB_REQUIRE((int64_t)a->group_size * 2 < 65536, QB_ERR_UNSUPPORTED, "This layer norm doesn't support feature dim >= 64KB.");
  const int64_t width = (int64_t)a->group_size * a->ngroups;
  QB_REQUIRE(a->x_row_stride >= width && a->out_row_stride >= width, QB_ERR_INVALID_ARG, "%s: row stride smaller than the row", who);
  if (gated) {
    QB_REQUIRE(a->residual == nullptr && a->residual_out == nullptr, QB_ERR_INVALID_ARG, "%s: takes no residual", who);
    QB_REQUIRE(a->z == nullptr || a->z_row_stride >= width, QB_ERR_INVALID_ARG, "%s: z row stride smaller than the row", who);
  } else {
    QB_REQUIRE(a->z == nullptr && a->ngroups == 1, QB_ERR_INVALID_ARG, "%s: takes no gate and one group", who);
    QB_REQUIRE(a->residual == nullptr || a->residual_row_stride >= width, QB_ERR_INVALID_ARG, "%s: residual row stride smaller than the row", who);
    QB_REQUIRE(a->residual_out == nullptr || a->residual_out_row_stride >= width, QB_ERR_INVALID_ARG,
               "%s: residual_out row stride smaller than the row", who);
  }
  NormParams p{};
  p.x = static_cast<const __half*>(a->x); p.residual = a->residual; p.residual_out = a->residual_out; p.z = a->z;
  p.w = static_cast<const __half*>(a->weight); p.bias = static_cast<const __half*>(a->bias); p.y = a->out; p.dyn_scale = a->dyn_scale;
  p.x_stride = a->x_row_stride; p.res_stride = a->residual_row_stride; p.res_out_stride = a->residual_out_row_stride;
  p.z_stride = a->z_row_stride; p.y_stride = a->out_row_stride;
  p.M = a->rows; p.N = a->group_size; p.ngroups = a->ngroups;
  p.res_f32 = a->residual_is_f32; p.res_out_f32 = a->residual_out_is_f32; p.out_kind = a->out_kind;
  p.gate_first = a->z != nullptr && !a->norm_before_gate; p.rms = a->is_rms_norm != 0;
  // The reference reduces max(y) over a power-of-two block whose padding lanes hold 0.
  p.pad_zero = (a->group_size & (a->group_size - 1)) != 0;
  p.eps = a->eps; p.out_scale = a->out_scale; p.z_scale = a->z_scale;
  // a dynamic-scale norm writes the per-row scales the next product reads through L1: no early start after it
  p.early = early_overlap() && a->dyn_scale == nullptr ? 1 : 0;
  QB_REQUIRE(a->n_partials >= 0 && a->n_partials <= 64 && (a->n_partials <= 1 || !gated), QB_ERR_INVALID_ARG,
             "%s: n_partials = %d (the gated norm takes one input)", who, a->n_partials);
  QB_REQUIRE(a->n_partials <= 1 || (a->partial_stride >= 0 && a->own_index >= -1 && a->own_index < a->n_partials), QB_ERR_INVALID_ARG,
             "%s: bad partial layout", who);
  p.n_partials = a->n_partials; p.own_index = a->own_index; p.partial_stride = a->partial_stride;
  p.own = a->n_partials > 1 ? static_cast<const __half*>(a->own_partial) : nullptr;
  return run_norm(p, (cudaStream_t)stream);
}

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qb_rmsnorm_quant(const qb_rmsnorm_args* a, void* stream) { return check_and_run(a, false, stream); }
extern "C" int qb_rmsnorm_gated(const qb_rmsnorm_args* a, void* stream) { return check_and_run(a, true, stream); }
