// int8 causal depthwise conv1d (+bias, SiLU, int8 requantisation) for sm_100a.
//
// Both layouts are pure streaming passes (1 byte in, 1 byte out per element), so the kernels
// are organised around coalesced loads/stores and keep the arithmetic per element to one
// byte-permute (window slide), one dp4a (the <=4 taps), one fma, one tanh.approx (SiLU) and the
// rounding.
//
//   channel-last  (Quamba2 xBC, and Quamba1 when the channel stride is 1): a thread owns 4
//                 adjacent channels (one 32-bit word; a warp moves one 128-byte line per time
//                 step) and walks TL consecutive time steps, keeping each channel's last four
//                 samples packed in one register.
//   sequence-last (Quamba1 (B, D, L) with L contiguous): a thread owns 16 adjacent time steps
//                 of one (batch, channel) row; windows are funnel shifts of adjacent words.
#include "common.cuh"

namespace qb {
namespace {

constexpr int kVec = 16;  // channels (or time steps) per thread = one 16-byte access

struct ClSegments {
  // Three output segments [0, end0), [end0, end1), [end1, dim) of the channel axis.
  int8_t* dst[3];
  int64_t dst_sb[3];
  int64_t dst_sl[3];
  int end0, end1;
  float scale_in[3];    // scale_w * scale_x per segment
  float scale_bias[3];  // bias scale per segment
  const float* out_scales[3];  // out_scales[0] == nullptr => out_scale_value (scale by value)
  float out_scale_value;
  // grouped x scales (segment 0 only)
  const int32_t* head_group_range;
  const int32_t* dim_group_range;
  int nhead_groups, ndim_groups, headdim, x_group_size, d_state;
  int grouped;
};

// weight bytes (C, W) -> one word whose byte i multiplies window byte i (= x[l-3+i])
__device__ __forceinline__ int pack_taps(const int8_t* w, int width) {
  uint32_t r = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int tap = i - (4 - width);
    const uint32_t v = tap >= 0 ? (uint32_t)(uint8_t)w[tap] : 0u;
    r |= v << (8 * i);
  }
  return (int)r;
}

constexpr int kCh = 4;       // channels per thread in the channel-last kernel = one 32-bit word
constexpr int kClBlock = 256;

// Channel-last layout.  A thread owns 4 adjacent channels (a warp reads / writes one 128-byte line per time step) and
// walks `tl` consecutive steps; byte i of win[j] = x[l-3+i] of channel j.  Per output the arithmetic is
//   prmt (slide window), dp4a into the bit pattern of 1.5*2^23 (so the sum is already a float: no I2F),
//   one subtraction, h = a/2 and hv = a/(2*s_out) as two FMAs, tanh, v = hv*tanh(h) + hv, round, convert;
// four results are packed with two saturating cvt.pack instructions.
template <bool kSilu>
__global__ void __launch_bounds__(kClBlock)
conv1d_channel_last_kernel(const int8_t* __restrict__ in, int64_t in_sb, int64_t in_sl,
                           const int8_t* __restrict__ weight, const int8_t* __restrict__ bias,
                           ClSegments seg, int batch, int dim, int seqlen, int width, int tl, int nseg, int early) {
  if (early) grid_dependency_launch();
  const int cv = dim / kCh;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)batch * nseg * cv;
  if (idx >= total) return;
  const int vec = (int)(idx % cv);
  const int sg = (int)((idx / cv) % nseg);
  const int b = (int)(idx / ((int64_t)cv * nseg));
  const int c0 = vec * kCh;
  const int s = c0 < seg.end0 ? 0 : (c0 < seg.end1 ? 1 : 2);
  const int cbase = s == 0 ? 0 : (s == 1 ? seg.end0 : seg.end1);

  int wpk[kCh];
  float hb[kCh], hsi[kCh], hbi[kCh];
  const float hs = 0.5f * seg.scale_in[s];
#pragma unroll
  for (int j = 0; j < kCh; ++j) {
    const int c = c0 + j;
    wpk[j] = pack_taps(weight + (int64_t)c * width, width);
    hb[j] = bias != nullptr ? 0.5f * seg.scale_bias[s] * (float)bias[c] : 0.0f;
    float so;
    if (seg.out_scales[0] == nullptr) {
      so = seg.out_scale_value;
    } else if (!seg.grouped) {
      so = seg.out_scales[s][0];
    } else if (s == 0) {
      const int g = c / seg.x_group_size;
      const int head = (c % seg.x_group_size) / seg.headdim;
      const int d = c % seg.headdim;
      const int hg = group_lookup(seg.head_group_range + g * seg.nhead_groups, seg.nhead_groups, head);
      const int dg = group_lookup(seg.dim_group_range + (g * seg.nhead_groups + hg) * seg.ndim_groups,
                                  seg.ndim_groups, d);
      so = seg.out_scales[0][(g * seg.nhead_groups + hg) * seg.ndim_groups + dg];
    } else {
      so = seg.out_scales[s][(c - cbase) / seg.d_state];
    }
    const float inv = 1.0f / so;
    hsi[j] = hs * inv;
    hbi[j] = hb[j] * inv;
  }

  const int l0 = sg * tl;
  const int l1 = min(seqlen, l0 + tl);
  const int8_t* src = in + (int64_t)b * in_sb + c0;
  int8_t* dst = seg.dst[s] + (int64_t)b * seg.dst_sb[s] + (c0 - cbase);
  const int64_t dsl = seg.dst_sl[s];

  // launched as a programmatic dependent: taps, bias and scales above are constants and were fetched while the kernel
  // before this one may still have been running; the input is read from here on, past L1 (ld_act)
  grid_dependency_wait();
  uint32_t win[kCh];
#pragma unroll
  for (int j = 0; j < kCh; ++j) win[j] = 0;
#pragma unroll
  for (int h = 3; h >= 1; --h) {
    const int l = l0 - h;
    const uint32_t r = l >= 0 ? ld_act(reinterpret_cast<const uint32_t*>(src + (int64_t)l * in_sl)) : 0u;
#pragma unroll
    for (int j = 0; j < kCh; ++j) win[j] = __byte_perm(win[j], r, 0x0321 | ((4 + j) << 12));
  }

  constexpr int kUnroll = 8;
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: int bits 0x4B400000 + n read back as the float kMagic + n
  const int8_t* p = src + (int64_t)l0 * in_sl;
  int8_t* o = dst + (int64_t)l0 * dsl;
  for (int l = l0; l < l1; l += kUnroll) {
    uint32_t rows[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      rows[u] = (l + u < l1) ? ld_act(reinterpret_cast<const uint32_t*>(p + (int64_t)u * in_sl)) : 0u;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int q[kCh];
#pragma unroll
      for (int j = 0; j < kCh; ++j) {
        win[j] = __byte_perm(win[j], rows[u], 0x0321 | ((4 + j) << 12));
        const float f = __int_as_float(__dp4a((int)win[j], wpk[j], 0x4B400000)) - kMagic;
        const float hv = fmaf(f, hsi[j], hbi[j]);
        float v;
        if (kSilu) {
          const float h = fmaf(f, hs, hb[j]);
          v = fmaf(hv, tanh_approx(h), hv);
        } else {
          v = hv + hv;
        }
        q[j] = __float2int_rz(v + copysignf(0.5f, v));
      }
      if (l + u < l1) *reinterpret_cast<uint32_t*>(o + (int64_t)u * dsl) = pack4_sat_s8(q[0], q[1], q[2], q[3]);
    }
    p += (int64_t)kUnroll * in_sl;
    o += (int64_t)kUnroll * dsl;
  }
}

// Sequence-last layout.  One thread = 16 consecutive time steps of one (b, d) row.
__global__ void __launch_bounds__(128)
conv1d_seq_last_kernel(const int8_t* __restrict__ in, int64_t in_sb, int64_t in_sd,
                       int8_t* __restrict__ out, int64_t out_sb, int64_t out_sd,
                       const int8_t* __restrict__ weight, const int8_t* __restrict__ bias,
                       int batch, int dim, int seqlen, int width, float scale_in, float scale_bias,
                       float scale_out, int silu, int vec_ok) {
  const int nv = (seqlen + kVec - 1) / kVec;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)batch * dim * nv;
  if (idx >= total) return;
  const int v = (int)(idx % nv);
  const int d = (int)((idx / nv) % dim);
  const int b = (int)(idx / ((int64_t)nv * dim));
  const int8_t* src = in + (int64_t)b * in_sb + (int64_t)d * in_sd;
  int8_t* dst = out + (int64_t)b * out_sb + (int64_t)d * out_sd;
  const int l0 = v * kVec;
  const int wpk = pack_taps(weight + (int64_t)d * width, width);
  const float hs_in = 0.5f * scale_in;
  const float hb = bias != nullptr ? 0.5f * scale_bias * (float)bias[d] : 0.0f;
  const float inv_out = 1.0f / scale_out;

  uint32_t w[5];  // w[0] = x[l0-4 .. l0-1], w[1..4] = x[l0 .. l0+15]
  const bool full = vec_ok && (l0 + kVec <= seqlen);
  if (full) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(src + l0));
    w[1] = r.x; w[2] = r.y; w[3] = r.z; w[4] = r.w;
    w[0] = l0 > 0 ? __ldg(reinterpret_cast<const uint32_t*>(src + l0 - 4)) : 0u;
  } else {
#pragma unroll
    for (int i = 0; i < 5; ++i) {
      uint32_t t = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int l = l0 - 4 + i * 4 + k;
        const uint32_t byte = (l >= 0 && l < seqlen) ? (uint32_t)(uint8_t)src[l] : 0u;
        t |= byte << (8 * k);
      }
      w[i] = t;
    }
  }
  uint32_t ow[4];
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    int q[4];
#pragma unroll
    for (int off = 0; off < 4; ++off) {
      const uint32_t window = off == 3 ? w[wi + 1] : __funnelshift_r(w[wi], w[wi + 1], 8 * (off + 1));
      const int acc = __dp4a((int)window, wpk, 0);
      const float h = fmaf((float)acc, hs_in, hb);
      const float y = silu ? fmaf(h, tanh_approx(h), h) : 2.0f * h;
      q[off] = round_away_s8(y * inv_out);
    }
    ow[wi] = pack4_s8(q[0], q[1], q[2], q[3]);
  }
  if (full) {
    *reinterpret_cast<uint4*>(dst + l0) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  } else {
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      if (l0 + i < seqlen) dst[l0 + i] = (int8_t)((ow[i >> 2] >> (8 * (i & 3))) & 0xff);
    }
  }
}

// Decode step, both flavours: one thread per (batch, channel).
struct UpdSegments {
  int8_t* dst[3];
  int64_t dst_sb[3];
  int64_t dst_sd[3];
  int end0, end1;
  float scale_in[3];
  float scale_bias[3];
  const float* out_scales[3];
  float out_scale_value;  // used when out_scales[0] == nullptr (Quamba1: scale by value)
  const int32_t* head_group_range;
  const int32_t* dim_group_range;
  int nhead_groups, ndim_groups, headdim, x_group_size, d_state;
  int grouped;
};

// Output scale lookup, bias, SiLU, re-quantisation and store of one (batch, channel) of a decode step.
__device__ __forceinline__ void update_finish(float acc, int b, int c, const int8_t* __restrict__ bias, const UpdSegments& seg, int silu) {
  const int s = c < seg.end0 ? 0 : (c < seg.end1 ? 1 : 2);
  const int cbase = s == 0 ? 0 : (s == 1 ? seg.end0 : seg.end1);
  float so;
  if (seg.out_scales[0] == nullptr) {
    so = seg.out_scale_value;
  } else if (!seg.grouped) {
    so = seg.out_scales[s][0];
  } else if (s == 0) {
    const int g = c / seg.x_group_size;
    const int head = (c % seg.x_group_size) / seg.headdim;
    const int d = c % seg.headdim;
    const int hg = group_lookup(seg.head_group_range + g * seg.nhead_groups, seg.nhead_groups, head);
    const int dg = group_lookup(seg.dim_group_range + (g * seg.nhead_groups + hg) * seg.ndim_groups,
                                seg.ndim_groups, d);
    so = seg.out_scales[0][(g * seg.nhead_groups + hg) * seg.ndim_groups + dg];
  } else {
    so = seg.out_scales[s][(c - cbase) / seg.d_state];
  }
  float v = seg.scale_in[s] * acc + (bias != nullptr ? seg.scale_bias[s] * (float)bias[c] : 0.0f);
  if (silu) v = silu_fast(v);
  seg.dst[s][(int64_t)b * seg.dst_sb[s] + (int64_t)(c - cbase) * seg.dst_sd[s]] = (int8_t)round_away_s8(v / so);
}

__global__ void __launch_bounds__(128)
conv1d_update_kernel(const int8_t* __restrict__ x, int64_t x_sb, int64_t x_sd,
                     int8_t* __restrict__ state, int64_t st_sb, int64_t st_sd, int64_t st_sw,
                     const int8_t* __restrict__ weight, const int8_t* __restrict__ bias,
                     UpdSegments seg, int batch, int dim, int width, int silu) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)batch * dim) return;
  const int c = (int)(idx % dim);
  const int b = (int)(idx / dim);
  int8_t* st = state + (int64_t)b * st_sb + (int64_t)c * st_sd;
  float acc = 0.0f;
  // shift left by one, append x, accumulate the dot product in the same pass
  for (int i = 0; i < width; ++i) {
    const int8_t v = (i < width - 1) ? st[(int64_t)(i + 1) * st_sw] : x[(int64_t)b * x_sb + (int64_t)c * x_sd];
    st[(int64_t)i * st_sw] = v;
    acc += (float)weight[(int64_t)c * width + i] * (float)v;
  }
  update_finish(acc, b, c, bias, seg, silu);
}

// The common layout -- width 4, state (batch, dim, 4) contiguous -- as one 32-bit word per channel: the window slides by
// a funnel shift, the four taps are one dp4a, state and weight accesses are one coalesced word per thread.
__global__ void __launch_bounds__(256)
conv1d_update_w4_kernel(const int8_t* __restrict__ x, int64_t x_sb, int64_t x_sd, uint32_t* __restrict__ state, int64_t st_sb_words,
                        const uint32_t* __restrict__ weight, const int8_t* __restrict__ bias, UpdSegments seg, int batch, int dim,
                        int silu) {
  grid_dependency_wait();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)batch * dim) return;
  const int c = (int)(idx % dim);
  const int b = (int)(idx / dim);
  uint32_t* st = state + (int64_t)b * st_sb_words + c;
  const uint32_t xv = (uint32_t)(uint8_t)ld_act(x + (int64_t)b * x_sb + (int64_t)c * x_sd);
  const uint32_t win = (ld_act(st) >> 8) | (xv << 24);   // drop the oldest sample, append the new one
  *st = win;
  const float acc = (float)__dp4a((int)win, (int)__ldg(weight + c), 0);
  update_finish(acc, b, c, bias, seg, silu);
}

bool update_w4_ok(int width, const void* state, int64_t sb, int64_t sd, int64_t sw, const void* weight) {
  return width == 4 && sw == 1 && sd == 4 && sb % 4 == 0 && aligned(state, 4) && aligned(weight, 4);
}

int pick_tl(int64_t rows_of_vectors, int seqlen) {
  // The time tile that fills ONE wave: at 64 registers an SM holds four 256-thread CTAs, and a grid of 1.1 waves runs
  // as long as one of 2 (a 672-CTA launch on 592 slots spent half its time on the last 80 CTAs).  So: as many segments
  // as fit in one wave, tiles rounded up to the unroll factor; larger problems than one wave take whole sequences.
  const int64_t wave_threads = (int64_t)sm_count() * 4 * kClBlock;
  int64_t nseg = wave_threads / rows_of_vectors;
  if (nseg < 1) nseg = 1;
  int tl = (int)ceil_div((int64_t)seqlen, nseg);
  tl = (tl + 7) & ~7;
  return tl < 8 ? 8 : tl;
}

int launch_channel_last(const int8_t* in, int64_t in_sb, int64_t in_sl, const int8_t* weight, const int8_t* bias,
                        const ClSegments& seg, int batch, int dim, int seqlen, int width, int silu, cudaStream_t stream) {
  const int cv = dim / kCh;
  const int tl = pick_tl((int64_t)batch * cv, seqlen);
  const int nseg = (int)ceil_div(seqlen, tl);
  const int64_t total = (int64_t)batch * nseg * cv;
  const unsigned grid = (unsigned)ceil_div(total, kClBlock);
  const int early = early_overlap() ? 1 : 0;
  if (silu) {
    launch_dependent(conv1d_channel_last_kernel<true>, dim3(grid), dim3(kClBlock), 0, stream, in, in_sb, in_sl, weight, bias, seg, batch,
                     dim, seqlen, width, tl, nseg, early);
  } else {
    launch_dependent(conv1d_channel_last_kernel<false>, dim3(grid), dim3(kClBlock), 0, stream, in, in_sb, in_sl, weight, bias, seg, batch,
                     dim, seqlen, width, tl, nseg, early);
  }
  QB_LAUNCH_OK("conv1d_channel_last_kernel");
  return QB_OK;
}

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qb_quamba2_conv1d_fwd(const qb_quamba2_conv1d_fwd_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "quamba2_conv1d_fwd: null args");
  QB_REQUIRE(a->xBC && a->x && a->Bm && a->Cm && a->weight && a->x_scales && a->B_scales && a->C_scales,
             QB_ERR_INVALID_ARG, "quamba2_conv1d_fwd: null tensor pointer");
  QB_REQUIRE(a->batch > 0 && a->dim > 0 && a->seqlen > 0, QB_ERR_INVALID_ARG, "quamba2_conv1d_fwd: empty shape");
  QB_REQUIRE(a->width >= 2 && a->width <= 4, QB_ERR_INVALID_ARG,
             "causal_conv1d only supports width between 2 and 4");
  const int gn = a->d_state * a->n_groups;
  QB_REQUIRE(a->x_dim + 2 * gn == a->dim, QB_ERR_INVALID_ARG, "x_dim + 2*d_state*n_groups must be equal to total dim");
  QB_REQUIRE(a->x_headdim > 0 && a->x_dim % a->x_headdim == 0, QB_ERR_INVALID_ARG, "x_dim must be divided by x_headdim");
  QB_REQUIRE(a->x_dim % kVec == 0 && gn % kVec == 0, QB_ERR_INVALID_ARG,
             "x_dim and d_state*n_groups must be multiples of 16");
  QB_REQUIRE(a->xBC_sl % kVec == 0 && a->xBC_sb % kVec == 0 && aligned(a->xBC, 16) && aligned(a->x, 16) &&
                 aligned(a->Bm, 16) && aligned(a->Cm, 16),
             QB_ERR_INVALID_ARG, "channel-last conv needs 16-byte aligned rows (strides multiple of 16)");
  const bool grouped = a->head_group_range != nullptr && a->dim_group_range != nullptr;
  QB_REQUIRE(grouped || (a->head_group_range == nullptr && a->dim_group_range == nullptr), QB_ERR_INVALID_ARG,
             "x_head_group_range and x_dim_group_range must be both null or both set");
  QB_REQUIRE(!grouped || (a->nhead_groups > 0 && a->ndim_groups > 0 && a->x_dim % a->n_groups == 0),
             QB_ERR_INVALID_ARG, "grouped scales need nhead_groups, ndim_groups > 0");
  ClSegments seg{};
  seg.dst[0] = a->x; seg.dst[1] = a->Bm; seg.dst[2] = a->Cm;
  seg.dst_sb[0] = (int64_t)a->seqlen * a->x_dim; seg.dst_sl[0] = a->x_dim;
  seg.dst_sb[1] = seg.dst_sb[2] = (int64_t)a->seqlen * gn; seg.dst_sl[1] = seg.dst_sl[2] = gn;
  seg.end0 = a->x_dim; seg.end1 = a->x_dim + gn;
  seg.scale_in[0] = a->scale_wx * a->scale_x; seg.scale_in[1] = a->scale_wB * a->scale_B; seg.scale_in[2] = a->scale_wC * a->scale_C;
  seg.scale_bias[0] = a->scale_bx; seg.scale_bias[1] = a->scale_bB; seg.scale_bias[2] = a->scale_bC;
  seg.out_scales[0] = a->x_scales; seg.out_scales[1] = a->B_scales; seg.out_scales[2] = a->C_scales;
  seg.head_group_range = a->head_group_range; seg.dim_group_range = a->dim_group_range;
  seg.nhead_groups = a->nhead_groups; seg.ndim_groups = a->ndim_groups; seg.headdim = a->x_headdim;
  seg.x_group_size = a->x_dim / a->n_groups; seg.d_state = a->d_state; seg.grouped = grouped ? 1 : 0;
  return launch_channel_last(a->xBC, a->xBC_sb, a->xBC_sl, a->weight, a->bias, seg, a->batch, a->dim, a->seqlen, a->width,
                             a->silu, (cudaStream_t)stream);
}

extern "C" int qb_causal_conv1d_fwd(const qb_conv1d_fwd_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->x && a->out && a->weight, QB_ERR_INVALID_ARG, "causal_conv1d_fwd: null pointer");
  QB_REQUIRE(a->batch > 0 && a->dim > 0 && a->seqlen > 0, QB_ERR_INVALID_ARG, "causal_conv1d_fwd: empty shape");
  QB_REQUIRE(a->width >= 2 && a->width <= 4, QB_ERR_INVALID_ARG,
             "causal_conv1d only supports width between 2 and 4");
  QB_REQUIRE(a->x_sl == 1 || a->x_sd == 1, QB_ERR_INVALID_ARG, "x must be contiguous in seqlen or in channels");
  const bool channel_last = a->x_sd == 1 && a->x_sl > 1;
  if (channel_last) {
    QB_REQUIRE(a->out_sd == 1, QB_ERR_INVALID_ARG, "out must have the layout of x");
    QB_REQUIRE(a->dim % kVec == 0 && a->x_sl % kVec == 0 && a->x_sb % kVec == 0 && a->out_sl % kVec == 0 &&
                   a->out_sb % kVec == 0 && aligned(a->x, 16) && aligned(a->out, 16),
               QB_ERR_INVALID_ARG,
               "causal_conv1d with channel last layout requires dim and strides to be multiples of 16");
    ClSegments seg{};
    for (int i = 0; i < 3; ++i) {
      seg.dst[i] = a->out; seg.dst_sb[i] = a->out_sb; seg.dst_sl[i] = a->out_sl;
      seg.scale_in[i] = a->scale_w * a->scale_x; seg.scale_bias[i] = a->scale_b;
      seg.out_scales[i] = nullptr;
    }
    seg.out_scale_value = a->scale_out;
    seg.end0 = seg.end1 = a->dim;
    return launch_channel_last(a->x, a->x_sb, a->x_sl, a->weight, a->bias, seg, a->batch, a->dim, a->seqlen, a->width,
                               a->silu, (cudaStream_t)stream);
  }
  QB_REQUIRE(a->out_sl == 1, QB_ERR_INVALID_ARG, "out must have the layout of x");
  const int vec_ok = (a->seqlen % kVec == 0) && (a->x_sd % kVec == 0) && (a->x_sb % kVec == 0) && (a->out_sd % kVec == 0) &&
                     (a->out_sb % kVec == 0) && aligned(a->x, 16) && aligned(a->out, 16);
  const int64_t total = (int64_t)a->batch * a->dim * ceil_div(a->seqlen, kVec);
  conv1d_seq_last_kernel<<<(unsigned)ceil_div(total, 128), 128, 0, (cudaStream_t)stream>>>(
      a->x, a->x_sb, a->x_sd, a->out, a->out_sb, a->out_sd, a->weight, a->bias, a->batch, a->dim, a->seqlen, a->width,
      a->scale_w * a->scale_x, a->scale_b, a->scale_out, a->silu, vec_ok);
  QB_LAUNCH_OK("conv1d_seq_last_kernel");
  return QB_OK;
}

extern "C" int qb_causal_conv1d_update(const qb_conv1d_update_args* a, void* stream) {
  QB_REQUIRE(a != nullptr && a->x && a->conv_state && a->out && a->weight, QB_ERR_INVALID_ARG,
             "causal_conv1d_update: null pointer");
  QB_REQUIRE(a->batch > 0 && a->dim > 0, QB_ERR_INVALID_ARG, "causal_conv1d_update: empty shape");
  QB_REQUIRE(a->width >= 2 && a->width <= 4, QB_ERR_INVALID_ARG,
             "causal_conv1d only supports width between 2 and 4");
  UpdSegments seg{};
  for (int i = 0; i < 3; ++i) {
    seg.dst[i] = a->out; seg.dst_sb[i] = a->out_sb; seg.dst_sd[i] = a->out_sd;
    seg.scale_in[i] = a->scale_w * a->scale_x; seg.scale_bias[i] = a->scale_b;
    seg.out_scales[i] = nullptr;
  }
  seg.out_scale_value = a->scale_out;
  seg.end0 = seg.end1 = a->dim;
  const int64_t total = (int64_t)a->batch * a->dim;
  if (update_w4_ok(a->width, a->conv_state, a->state_sb, a->state_sd, a->state_sw, a->weight)) {
    launch_dependent(conv1d_update_w4_kernel, dim3((unsigned)ceil_div(total, 256)), dim3(256), 0, (cudaStream_t)stream,
                     a->x, a->x_sb, a->x_sd, reinterpret_cast<uint32_t*>(a->conv_state), a->state_sb / 4,
                     reinterpret_cast<const uint32_t*>(a->weight), a->bias, seg, a->batch, a->dim, a->silu);
    QB_LAUNCH_OK("conv1d_update_w4_kernel");
    return QB_OK;
  }
  conv1d_update_kernel<<<(unsigned)ceil_div(total, 128), 128, 0, (cudaStream_t)stream>>>(
      a->x, a->x_sb, a->x_sd, a->conv_state, a->state_sb, a->state_sd, a->state_sw, a->weight, a->bias, seg,
      a->batch, a->dim, a->width, a->silu);
  QB_LAUNCH_OK("conv1d_update_kernel");
  return QB_OK;
}

extern "C" int qb_quamba2_conv1d_update(const qb_quamba2_conv1d_update_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "quamba2_conv1d_update: null args");
  QB_REQUIRE(a->xBC && a->conv_state && a->x && a->Bm && a->Cm && a->weight && a->x_scales && a->B_scales && a->C_scales,
             QB_ERR_INVALID_ARG, "quamba2_conv1d_update: null tensor pointer");
  QB_REQUIRE(a->batch > 0 && a->dim > 0, QB_ERR_INVALID_ARG, "quamba2_conv1d_update: empty shape");
  QB_REQUIRE(a->width == 4, QB_ERR_INVALID_ARG, "causal_conv1d only supports width = 4");
  const int gn = a->d_state * a->n_groups;
  QB_REQUIRE(a->x_dim + 2 * gn == a->dim, QB_ERR_INVALID_ARG, "x_dim + 2*d_state*n_groups must be equal to total dim");
  QB_REQUIRE(a->x_headdim > 0 && a->x_dim % a->x_headdim == 0, QB_ERR_INVALID_ARG, "x_dim must be divided by x_headdim");
  const bool grouped = a->head_group_range != nullptr && a->dim_group_range != nullptr;
  QB_REQUIRE(grouped || (a->head_group_range == nullptr && a->dim_group_range == nullptr), QB_ERR_INVALID_ARG,
             "x_head_group_range and x_dim_group_range must be both null or both set");
  QB_REQUIRE(!grouped || (a->nhead_groups > 0 && a->ndim_groups > 0 && a->x_dim % a->n_groups == 0),
             QB_ERR_INVALID_ARG, "grouped scales need nhead_groups, ndim_groups > 0");
  UpdSegments seg{};
  seg.dst[0] = a->x; seg.dst[1] = a->Bm; seg.dst[2] = a->Cm;
  seg.dst_sb[0] = a->x_dim; seg.dst_sb[1] = seg.dst_sb[2] = gn;
  seg.dst_sd[0] = seg.dst_sd[1] = seg.dst_sd[2] = 1;
  seg.end0 = a->x_dim; seg.end1 = a->x_dim + gn;
  seg.scale_in[0] = a->scale_wx * a->scale_x; seg.scale_in[1] = a->scale_wB * a->scale_B; seg.scale_in[2] = a->scale_wC * a->scale_C;
  seg.scale_bias[0] = a->scale_bx; seg.scale_bias[1] = a->scale_bB; seg.scale_bias[2] = a->scale_bC;
  seg.out_scales[0] = a->x_scales; seg.out_scales[1] = a->B_scales; seg.out_scales[2] = a->C_scales;
  seg.head_group_range = a->head_group_range; seg.dim_group_range = a->dim_group_range;
  seg.nhead_groups = a->nhead_groups; seg.ndim_groups = a->ndim_groups; seg.headdim = a->x_headdim;
  seg.x_group_size = a->x_dim / a->n_groups; seg.d_state = a->d_state; seg.grouped = grouped ? 1 : 0;
  const int64_t total = (int64_t)a->batch * a->dim;
  if (update_w4_ok(a->width, a->conv_state, a->state_sb, a->state_sd, a->state_sw, a->weight)) {
    launch_dependent(conv1d_update_w4_kernel, dim3((unsigned)ceil_div(total, 256)), dim3(256), 0, (cudaStream_t)stream,
                     a->xBC, a->xBC_sb, (int64_t)1, reinterpret_cast<uint32_t*>(a->conv_state), a->state_sb / 4,
                     reinterpret_cast<const uint32_t*>(a->weight), a->bias, seg, a->batch, a->dim, a->silu);
    QB_LAUNCH_OK("conv1d_update_w4_kernel");
    return QB_OK;
  }
  conv1d_update_kernel<<<(unsigned)ceil_div(total, 128), 128, 0, (cudaStream_t)stream>>>(
      a->xBC, a->xBC_sb, 1, a->conv_state, a->state_sb, a->state_sd, a->state_sw, a->weight, a->bias, seg,
      a->batch, a->dim, a->width, a->silu);
  QB_LAUNCH_OK("conv1d_update_kernel");
  return QB_OK;
}
