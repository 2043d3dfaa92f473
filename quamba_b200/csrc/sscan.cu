// Mamba1 int8 selective scan (prefill) and the single-step state update (decode) for sm_100a.
//
// Forward: one thread owns one (batch, channel) row and carries its N states in registers while
// it walks the sequence; a CTA of 64 rows stages 64-step tiles of u / delta / z (int8, coalesced
// 16-byte loads along L) and of B / C (shared by every row of the group, converted to fp32 once
// per tile) in shared memory.  The output is written directly in the (B, L, D) layout the
// out-projection consumes, so the reference's separate transpose pass does not exist here.
//
// Update: eight lanes share one (batch, head, channel) row of the int8 state (16 bytes each),
// the y reduction is a 3-step shuffle.
#include <algorithm>
#include "common.cuh"
#include "tc_common.cuh"

namespace qb {
namespace {

// (b, d) rows per CTA == threads per CTA: 64 for every state width that is built
constexpr int rows_per_cta(int /*dstate*/) { return 64; }
constexpr int kTile = 64;    // time steps per shared-memory tile
constexpr int kRowPad = 68;  // bytes per staged int8 row: 17 words, conflict-free column reads
constexpr int kChunk = 2048; // the reference stores the state after every 2048 steps

constexpr float kLog2e = 1.4426950408889634f;

template <int N, int kRows>
__global__ void __launch_bounds__(kRows)
sscan_fwd_kernel(qb_sscan_fwd_args a, int has_z, int vec_ok) {
  __shared__ __align__(16) int8_t s_u[kRows * kRowPad];
  __shared__ __align__(16) int8_t s_dt[kRows * kRowPad];
  __shared__ __align__(16) int8_t s_z[kRows * kRowPad];
  __shared__ __align__(16) float s_B[kTile * N];
  __shared__ __align__(16) float s_C[kTile * N];

  const int tid = threadIdx.x;
  const int tiles_d = (a.dim + kRows - 1) / kRows;
  const int b = blockIdx.x / tiles_d;
  const int d0 = (blockIdx.x % tiles_d) * kRows;
  const int d = d0 + tid;
  const bool row_ok = d < a.dim;
  const int dd = row_ok ? d : a.dim - 1;
  const int group = d0 / (a.dim / a.n_groups);
  const int nchunks = (a.seqlen + kChunk - 1) / kChunk;

  const float s_u_ = *a.u_scale, s_d_ = *a.delta_scale, s_B_ = *a.B_scale, s_C_ = *a.C_scale;
  const float s_A_ = *a.A_scale, s_st = *a.ssm_state_scale;
  const float s_z_ = has_z ? *a.z_scale : 0.0f;
  const float Dv = a.D != nullptr ? (*a.D_scale) * (float)a.D[dd] : 0.0f;
  const float bias = a.delta_bias != nullptr ? (*a.delta_bias_scale) * (float)a.delta_bias[dd] : 0.0f;
  float A2[N], h[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    A2[n] = -__expf(s_A_ * (float)a.A_log[(int64_t)dd * N + n]) * kLog2e;
    h[n] = 0.0f;
  }
  const int8_t* u_b = a.u + (int64_t)b * a.u_sb;
  const int8_t* dt_b = a.delta + (int64_t)b * a.delta_sb;
  const int8_t* z_b = has_z ? a.z + (int64_t)b * a.z_sb : nullptr;
  const int8_t* B_b = a.Bm + (int64_t)b * a.B_sb + (int64_t)group * a.B_sg;
  const int8_t* C_b = a.Cm + (int64_t)b * a.C_sb + (int64_t)group * a.C_sg;
  __half* out = static_cast<__half*>(a.out) + (int64_t)b * a.seqlen * a.dim + d;
  int8_t* xs = a.x_states + ((int64_t)b * a.dim + dd) * nchunks * N;

  // stage one 16-byte piece (or its in-range bytes) of a row into a padded shared row
  auto stage = [&](const int8_t* base, int64_t row_stride, int8_t* dst, int l0) {
    // kRows rows x 4 pieces of 16 steps; one thread per row -> 4 iterations
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int item = it * kRows + tid;
      const int r = item >> 2, piece = item & 3;
      const int rr = min(d0 + r, a.dim - 1);
      const int l = l0 + piece * 16;
      const int8_t* src = base + (int64_t)rr * row_stride + l;
      uint32_t w[4] = {0, 0, 0, 0};
      if (vec_ok && l + 16 <= a.seqlen) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
      } else {
        for (int k = 0; k < 16; ++k)
          if (l + k < a.seqlen) w[k >> 2] |= (uint32_t)(uint8_t)src[k] << (8 * (k & 3));
      }
      uint32_t* o = reinterpret_cast<uint32_t*>(dst + r * kRowPad + piece * 16);
      o[0] = w[0]; o[1] = w[1]; o[2] = w[2]; o[3] = w[3];
    }
  };
  auto stage_bc = [&](const int8_t* base, int64_t sn, float scale, float* dst, int l0) {
    // N rows x 4 pieces of 16 steps
    for (int item = tid; item < N * 4; item += kRows) {
      const int n = item >> 2, piece = item & 3;
      const int l = l0 + piece * 16;
      const int8_t* src = base + (int64_t)n * sn + l;
      __align__(16) int8_t v[16];
      if (vec_ok && l + 16 <= a.seqlen) {
        *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(src));
      } else {
        for (int k = 0; k < 16; ++k) v[k] = (l + k < a.seqlen) ? src[k] : (int8_t)0;
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) dst[(piece * 16 + k) * N + n] = scale * (float)v[k];
    }
  };

  for (int l0 = 0; l0 < a.seqlen; l0 += kTile) {
    __syncthreads();
    stage(u_b, a.u_sd, s_u, l0);
    stage(dt_b, a.delta_sd, s_dt, l0);
    if (has_z) stage(z_b, a.z_sd, s_z, l0);
    stage_bc(B_b, a.B_sn, s_B_, s_B, l0);
    stage_bc(C_b, a.C_sn, s_C_, s_C, l0);
    __syncthreads();
    const int steps = min(kTile, a.seqlen - l0);
    const uint32_t* ru = reinterpret_cast<const uint32_t*>(s_u + tid * kRowPad);
    const uint32_t* rd = reinterpret_cast<const uint32_t*>(s_dt + tid * kRowPad);
    const uint32_t* rz = reinterpret_cast<const uint32_t*>(s_z + tid * kRowPad);
    for (int t4 = 0; t4 < steps; t4 += 4) {
      const uint32_t wu = ru[t4 >> 2], wd = rd[t4 >> 2];
      const uint32_t wz = has_z ? rz[t4 >> 2] : 0u;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int t = t4 + k;
        if (t < steps) {
          // int8 -> float without a conversion instruction: the biased byte spliced into the mantissa of 2^15
          const float u = s_u_ * (__uint_as_float(__byte_perm(wu ^ 0x80808080u, 0x47000000u, 0x7404 | (k << 4))) - 32896.0f);
          float delta = fmaf(s_d_, __uint_as_float(__byte_perm(wd ^ 0x80808080u, 0x47000000u, 0x7404 | (k << 4))) - 32896.0f, bias);
          if (a.delta_softplus) delta = softplus_fast(delta);
          const float du = delta * u;
          float y4[4] = {Dv * u, 0.0f, 0.0f, 0.0f};  // four partial sums: the y chain is not one serial dependency
          const float4* Bt = reinterpret_cast<const float4*>(s_B + t * N);
          const float4* Ct = reinterpret_cast<const float4*>(s_C + t * N);
#pragma unroll
          for (int n4 = 0; n4 < N / 4; ++n4) {
            const float4 bv = Bt[n4], cv = Ct[n4];
            const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
            const float cc[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int n = n4 * 4 + j;
              h[n] = fmaf(fast_exp2(delta * A2[n]), h[n], bb[j] * du);
              y4[j] = fmaf(h[n], cc[j], y4[j]);
            }
          }
          float y = (y4[0] + y4[1]) + (y4[2] + y4[3]);
          if (has_z) {
            const float z = s_z_ * (__uint_as_float(__byte_perm(wz ^ 0x80808080u, 0x47000000u, 0x7404 | (k << 4))) - 32896.0f);
            y = y * silu_mufu(z);
          }
          const int l = l0 + t;
          if (row_ok) out[(int64_t)l * a.dim] = __float2half_rn(y);
          if (((l + 1) % kChunk == 0 || l == a.seqlen - 1) && row_ok) {
            int8_t* dst = xs + (int64_t)(l / kChunk) * N;
#pragma unroll
            for (int n = 0; n < N; ++n) dst[n] = (int8_t)round_away_s8(h[n] / s_st);
          }
        }
      }
    }
  }
}

// ---- decode step -----------------------------------------------------------------------------
// 8 lanes per (b, h, p) row; lane j owns states n = 16*j + 128*i .. (16-byte pieces).
__global__ void __launch_bounds__(128)
sscan_update_kernel(qb_sscan_update_args a) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid >> 3;
  const int sub = (int)(gid & 7);
  const int64_t rows = (int64_t)a.batch * a.nheads * a.headdim;
  const bool active = row < rows;
  const int64_t rr = active ? row : rows - 1;
  const int p = (int)(rr % a.headdim);
  const int hd = (int)((rr / a.headdim) % a.nheads);
  const int b = (int)(rr / ((int64_t)a.headdim * a.nheads));
  const int hpg = a.nheads / a.ngroups;
  const int g = hd / hpg;

  int hg = 0, dg = 0;
  float xs, Bs, Cs;
  if (a.grouped) {
    hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, hd % hpg);
    dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, p);
    xs = a.x_scales[(g * a.nhead_groups + hg) * a.ndim_groups + dg];
    Bs = a.B_scale[g];
    Cs = a.C_scale[g];
  } else {
    xs = a.x_scales[0];
    Bs = a.B_scale[0];
    Cs = a.C_scale[0];
  }
  const float* st_scale = a.grouped
      ? a.state_scale + ((int64_t)(g * a.nhead_groups + hg) * a.ndim_groups + dg) * a.dstate
      : nullptr;
  const float st_scale0 = a.grouped ? 0.0f : a.state_scale[0];

  const float x = xs * (float)a.x[(int64_t)b * a.x_sb + (int64_t)hd * a.x_sh + p];
  float dt = (*a.dt_scale) * (float)a.dt[(int64_t)b * a.dt_sb + (int64_t)hd * a.dt_sh + (int64_t)p * a.dt_sp];
  if (a.dt_bias != nullptr) {
    const int64_t bi = (int64_t)hd * a.bias_sh + (int64_t)p * a.bias_sp;
    if (a.dt_bias_is_half) dt += __half2float(static_cast<const __half*>(a.dt_bias)[bi]);
    else dt += (*a.dt_bias_scale) * (float)static_cast<const int8_t*>(a.dt_bias)[bi];
  }
  if (a.dt_softplus) dt = softplus_f(dt);
  const float sA = *a.A_scale;
  const float dtx = dt * x;
  const int8_t* Aq = a.A_log + (int64_t)hd * a.A_sh + (int64_t)p * a.A_sp;
  const int8_t* Bq = a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg;
  const int8_t* Cq = a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg;
  int8_t* st = a.state + (int64_t)b * a.state_sb + (int64_t)hd * a.state_sh + (int64_t)p * a.state_sp;
  const bool vec = (a.dstate % 16 == 0) && ((reinterpret_cast<uintptr_t>(st) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(Bq) & 15) == 0) && ((reinterpret_cast<uintptr_t>(Cq) & 15) == 0);
  float y = 0.0f;
  for (int n0 = sub * 16; n0 < a.dstate; n0 += 128) {
    __align__(16) int8_t sv[16], bv[16], cv[16];
    if (vec) {
      *reinterpret_cast<uint4*>(sv) = *reinterpret_cast<const uint4*>(st + n0);
      *reinterpret_cast<uint4*>(bv) = __ldg(reinterpret_cast<const uint4*>(Bq + n0));
      *reinterpret_cast<uint4*>(cv) = __ldg(reinterpret_cast<const uint4*>(Cq + n0));
    } else {
      for (int k = 0; k < 16; ++k) {
        const bool ok = n0 + k < a.dstate;
        sv[k] = ok ? st[n0 + k] : (int8_t)0;
        bv[k] = ok ? Bq[n0 + k] : (int8_t)0;
        cv[k] = ok ? Cq[n0 + k] : (int8_t)0;
      }
    }
    __align__(16) int8_t qo[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int n = n0 + k;
      const bool ok = n < a.dstate;
      const int nn = ok ? n : 0;
      const float ss = a.grouped ? st_scale[nn] : st_scale0;
      const float A = -__expf(sA * (float)Aq[(int64_t)nn * a.A_sn]);
      const float s = fmaf(ss * (float)sv[k], __expf(A * dt), (Bs * (float)bv[k]) * dtx);
      qo[k] = (int8_t)rint_s8(s / ss);
      if (ok) y = fmaf(s, Cs * (float)cv[k], y);
    }
    if (active) {
      if (vec) {
        *reinterpret_cast<uint4*>(st + n0) = *reinterpret_cast<const uint4*>(qo);
      } else {
        for (int k = 0; k < 16; ++k)
          if (n0 + k < a.dstate) st[n0 + k] = qo[k];
      }
    }
  }
  y += __shfl_xor_sync(0xffffffffu, y, 1);
  y += __shfl_xor_sync(0xffffffffu, y, 2);
  y += __shfl_xor_sync(0xffffffffu, y, 4);
  if (active && sub == 0) {
    if (a.D != nullptr) y = fmaf(x, (*a.D_scale) * (float)a.D[(int64_t)hd * a.D_sh + (int64_t)p * a.D_sp], y);
    if (a.z != nullptr) {
      const float z = (*a.z_scale) * (float)a.z[(int64_t)b * a.z_sb + (int64_t)hd * a.z_sh + p];
      y *= silu_exact(z);
    }
    static_cast<__half*>(a.out)[(int64_t)b * a.out_sb + (int64_t)hd * a.out_sh + p] = __float2half_rn(y);
  }
}


// Streaming form of the decode step for the common layouts (dstate a multiple of 16, 16-byte aligned state rows, all
// rows of a CTA in one (batch, SSD group)).  LANES lanes share one (b, h, p) row, each owning 16-byte pieces of the
// int8 state.  B and C are converted and scaled once per CTA into shared memory, exp(A_scale * q) comes from a
// 256-entry table (A_log is int8), the int8 state is widened with a byte permute into the mantissa of 2^15 (no
// integer-to-float conversion instruction), and the new state is rounded and packed four at a time.
template <int LANES>
__global__ void __launch_bounds__(256)
sscan_update_stream_kernel(qb_sscan_update_args a, int iters) {
  constexpr int ROWS = 256 / LANES;
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ __align__(16) float sB[256];
  __shared__ __align__(16) float sC[256];
  __shared__ float sLut[256];  // -exp(A_scale * q) * log2(e), q = index - 128
  const int tid = threadIdx.x;
  const int64_t rows = (int64_t)a.batch * a.nheads * a.headdim;
  const int64_t rows_per_b = (int64_t)a.nheads * a.headdim;
  const int64_t row0 = (int64_t)blockIdx.x * ROWS;
  const int hpg = a.nheads / a.ngroups;
  const int b = (int)(row0 / rows_per_b);
  const int g = (int)(((row0 % rows_per_b) / a.headdim) / hpg);
  {
    const float Bs = a.grouped ? a.B_scale[g] : a.B_scale[0];
    const float Cs = a.grouped ? a.C_scale[g] : a.C_scale[0];
    const int8_t* Bq = a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg;
    const int8_t* Cq = a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg;
    if (tid < a.dstate) {
      sB[tid] = Bs * (float)Bq[tid];
      sC[tid] = Cs * (float)Cq[tid];
    }
    sLut[tid] = -__expf((*a.A_scale) * (float)(tid - 128)) * kLog2e;
  }
  __syncthreads();
  const int64_t row = row0 + tid / LANES;
  const int sub = tid % LANES;
  if (row >= rows) return;
  const int p = (int)(row % a.headdim);
  const int hd = (int)((row / a.headdim) % a.nheads);

  float xs, ss0 = 0.0f;
  const float* ssn = nullptr;
  if (a.grouped) {
    const int hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, hd % hpg);
    const int dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, p);
    xs = a.x_scales[(g * a.nhead_groups + hg) * a.ndim_groups + dg];
    ssn = a.state_scale + ((int64_t)(g * a.nhead_groups + hg) * a.ndim_groups + dg) * a.dstate;
  } else {
    xs = a.x_scales[0];
    ss0 = a.state_scale[0];
  }
  const float x = xs * (float)a.x[(int64_t)b * a.x_sb + (int64_t)hd * a.x_sh + p];
  float dt = (*a.dt_scale) * (float)a.dt[(int64_t)b * a.dt_sb + (int64_t)hd * a.dt_sh + (int64_t)p * a.dt_sp];
  if (a.dt_bias != nullptr) {
    const int64_t bi = (int64_t)hd * a.bias_sh + (int64_t)p * a.bias_sp;
    if (a.dt_bias_is_half) dt += __half2float(static_cast<const __half*>(a.dt_bias)[bi]);
    else dt += (*a.dt_bias_scale) * (float)static_cast<const int8_t*>(a.dt_bias)[bi];
  }
  if (a.dt_softplus) dt = softplus_f(dt);
  const float dtx = dt * x;
  const int8_t* Aq = a.A_log + (int64_t)hd * a.A_sh + (int64_t)p * a.A_sp;
  const bool tied = a.A_sn == 0;
  const float dA_tied = tied ? fast_exp2(sLut[(int)Aq[0] + 128] * dt) : 0.0f;
  const float inv0 = a.grouped ? 0.0f : 1.0f / ss0;
  int8_t* st = a.state + (int64_t)b * a.state_sb + (int64_t)hd * a.state_sh + (int64_t)p * a.state_sp;

  float y = 0.0f;
  for (int it = 0; it < iters; ++it) {
    const int n0 = (it * LANES + sub) * 16;
    const uint4 raw = *reinterpret_cast<const uint4*>(st + n0);
    const uint32_t w[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
    uint32_t ow[4];
#pragma unroll
    for (int k4 = 0; k4 < 4; ++k4) {
      const float4 bf = *reinterpret_cast<const float4*>(sB + n0 + 4 * k4);
      const float4 cf = *reinterpret_cast<const float4*>(sC + n0 + 4 * k4);
      const float bb[4] = {bf.x, bf.y, bf.z, bf.w};
      const float cc[4] = {cf.x, cf.y, cf.z, cf.w};
      float ssv[4] = {ss0, ss0, ss0, ss0}, inv[4] = {inv0, inv0, inv0, inv0};
      if (a.grouped) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(ssn + n0 + 4 * k4));
        ssv[0] = t.x; ssv[1] = t.y; ssv[2] = t.z; ssv[3] = t.w;
#pragma unroll
        for (int k = 0; k < 4; ++k) inv[k] = __frcp_rn(ssv[k]);
      }
      int q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // bytes [0, v + 128, 0, 0x47] read as a float = 32768 + (v + 128)
        const float sv = __uint_as_float(__byte_perm(w[k4], 0x47000000u, 0x7404 | (k << 4))) - 32896.0f;
        float dA = dA_tied;
        if (!tied) dA = fast_exp2(sLut[(int)Aq[(int64_t)(n0 + 4 * k4 + k) * a.A_sn] + 128] * dt);
        const float snew = fmaf(bb[k], dtx, (ssv[k] * sv) * dA);
        q[k] = __float2int_rn(snew * inv[k]);
        y = fmaf(snew, cc[k], y);
      }
      ow[k4] = pack4_sat_s8(q[0], q[1], q[2], q[3]);
    }
    *reinterpret_cast<uint4*>(st + n0) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
#pragma unroll
  for (int m = 1; m < LANES; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
  if (sub == 0) {
    if (a.D != nullptr) y = fmaf(x, (*a.D_scale) * (float)a.D[(int64_t)hd * a.D_sh + (int64_t)p * a.D_sp], y);
    if (a.z != nullptr) {
      const float z = (*a.z_scale) * (float)a.z[(int64_t)b * a.z_sb + (int64_t)hd * a.z_sh + p];
      y *= silu_exact(z);
    }
    static_cast<__half*>(a.out)[(int64_t)b * a.out_sb + (int64_t)hd * a.out_sh + p] = __float2half_rn(y);
  }
}


// Low-latency form for decode steps with few (batch, head) pairs (one token of one to a few sequences): one CTA per
// pair, a thread owns 32 consecutive states of one row.  What makes a small decode kernel slow is not bandwidth but the
// chain of dependent round trips to memory, so everything that the kernel before this one on the stream cannot have
// written -- the state itself (last written by the previous decode step), A, D, dt_bias and the scales -- is loaded
// BEFORE the dependency wait; after it come one round of loads (x, dt, B, C), the arithmetic of the streaming kernel
// above, and the stores.  d_state 128, per-tensor scales, A / dt / D tied across the head.
__global__ void __launch_bounds__(256)
sscan_update_small_kernel(qb_sscan_update_args a) {
  constexpr float kLog2e = 1.4426950408889634f;
  if (a.early_launch) grid_dependency_launch();
  const int hd = blockIdx.x, b = blockIdx.y;
  const int sub = threadIdx.x & 3, n0 = sub * 32;
  const int g = hd / (a.nheads / a.ngroups);
  const float xs = __ldg(a.x_scales), ss = __ldg(a.state_scale), dts = __ldg(a.dt_scale), As = __ldg(a.A_scale);
  const float Bs = __ldg(a.B_scale), Cs = __ldg(a.C_scale);
  const float Dv = a.D != nullptr ? __ldg(a.D_scale) * (float)a.D[(int64_t)hd * a.D_sh] : 0.0f;
  float bias = 0.0f;
  if (a.dt_bias != nullptr) {
    const int64_t bi = (int64_t)hd * a.bias_sh;
    bias = a.dt_bias_is_half ? __half2float(static_cast<const __half*>(a.dt_bias)[bi])
                             : __ldg(a.dt_bias_scale) * (float)static_cast<const int8_t*>(a.dt_bias)[bi];
  }
  const float nA = -__expf(As * (float)a.A_log[(int64_t)hd * a.A_sh]) * kLog2e;
  const float inv = 1.0f / ss;
  for (int p = threadIdx.x >> 2; p < a.headdim; p += 64) {
    int8_t* st = a.state + (int64_t)b * a.state_sb + (int64_t)hd * a.state_sh + (int64_t)p * a.state_sp + n0;
    // the state changes every step and is read once: L2 reads, so that no line an SM cached in an earlier step is served
    const uint4 raw0 = __ldcg(reinterpret_cast<const uint4*>(st)), raw1 = __ldcg(reinterpret_cast<const uint4*>(st + 16));
    grid_dependency_wait();       // (a no-op from the second row tile on)
    // inputs written by the kernel before this one: L2 reads (__ldcg), see grid_dependency_launch
    const float x = xs * (float)__ldcg(reinterpret_cast<const signed char*>(a.x) + (int64_t)b * a.x_sb + (int64_t)hd * a.x_sh + p);
    float dt = dts * (float)__ldcg(reinterpret_cast<const signed char*>(a.dt) + (int64_t)b * a.dt_sb + (int64_t)hd * a.dt_sh) + bias;
    const uint4 bq0 = __ldcg(reinterpret_cast<const uint4*>(a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg + n0));
    const uint4 bq1 = __ldcg(reinterpret_cast<const uint4*>(a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg + n0 + 16));
    const uint4 cq0 = __ldcg(reinterpret_cast<const uint4*>(a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg + n0));
    const uint4 cq1 = __ldcg(reinterpret_cast<const uint4*>(a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg + n0 + 16));
    if (a.dt_softplus) dt = softplus_f(dt);
    const float dtx = dt * x, dA = fast_exp2(nA * dt);
    const uint32_t sw[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
    const uint32_t bw[8] = {bq0.x, bq0.y, bq0.z, bq0.w, bq1.x, bq1.y, bq1.z, bq1.w};
    const uint32_t cw[8] = {cq0.x, cq0.y, cq0.z, cq0.w, cq1.x, cq1.y, cq1.z, cq1.w};
    uint32_t ow[8];
    float y = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      int q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float sv = (float)(int8_t)(sw[w] >> (8 * k));
        const float bb = Bs * (float)(int8_t)(bw[w] >> (8 * k));
        const float cc = Cs * (float)(int8_t)(cw[w] >> (8 * k));
        const float snew = fmaf(bb, dtx, (ss * sv) * dA);
        q[k] = __float2int_rn(snew * inv);
        y = fmaf(snew, cc, y);
      }
      ow[w] = pack4_sat_s8(q[0], q[1], q[2], q[3]);
    }
    *reinterpret_cast<uint4*>(st) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    *reinterpret_cast<uint4*>(st + 16) = make_uint4(ow[4], ow[5], ow[6], ow[7]);
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    if (sub == 0) {
      if (a.D != nullptr) y = fmaf(x, Dv, y);
      static_cast<__half*>(a.out)[(int64_t)b * a.out_sb + (int64_t)hd * a.out_sh + p] = __float2half_rn(y);
    }
  }
}

// Pipelined form of the streaming decode step for a fully contiguous state (B, H, P, N): the state is a flat matrix of
// rows, so a tile of consecutive rows is one contiguous 8 KB block.  A persistent CTA walks a contiguous range of tiles
// through a four-slot shared-memory ring: bulk-copy loads run two tiles ahead (completion on an mbarrier), the tile is
// updated in place in shared memory, and a bulk-copy store drains it while the next tile is computed.  Memory-level
// parallelism is therefore set by the ring, not by registers.  LPR = 16-byte pieces per state row (dstate = 16 * LPR).
constexpr int kUpdTileBytes = 8192;
constexpr int kUpdSlots = 4;
constexpr int kStatusUpdateLoad = 301;

// Warp-autonomous variant for the Mamba2 decode shape (d_state 128, A tied across the state, per-tensor scales): every
// warp owns a ring of four 2 KB slots and walks its own list of 16-row tiles -- bulk load two tiles ahead, update in
// place, bulk store -- so no CTA-wide barrier exists after the set-up (the 256-thread kernel below spends a third of
// its stall cycles at its two __syncthreads per tile).  Lane l covers the 16 states n0 = 16 (l & 7) of the rows
// (l >> 3) + 4 e, e = 0..3; the row scalars (x, dt, exp2(A dt), ...) are computed once by lanes 0..15 and passed round
// by shuffles; the eight lanes of a row reduce y by shuffles.
constexpr int kWTileRows = 16, kWTileBytes = kWTileRows * 128, kWSlots = 4;
__global__ void __launch_bounds__(256, 3)
sscan_update_warp_kernel(qb_sscan_update_args a, int tiles, int* status) {
  using namespace tc;
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(128) uint8_t ring_all[];
  __shared__ __align__(8) uint64_t full_all[8][kWSlots];
  grid_dependency_wait();     // launched as a programmatic dependent (launch_dependent)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* ring = ring_all + warp * (kWSlots * kWTileBytes);
  uint64_t* full = full_all[warp];
  const int gw = blockIdx.x * 8 + warp, nw = gridDim.x * 8;
  const int per = tiles / nw, extra = tiles % nw;            // contiguous tiles per warp: neighbours share (batch, head)
  const int t_begin = gw * per + min(gw, extra);
  const int t_end = t_begin + per + (gw < extra ? 1 : 0);
  if (t_begin >= t_end) return;
  if (lane == 0) {
    for (int i = 0; i < kWSlots; ++i) mbar_init(&full[i], 1);
    fence_barrier_init();
  }
  __syncwarp();
  auto issue_load = [&](int t) {
    const int slot = (t - t_begin) & (kWSlots - 1);
    mbar_arrive_expect_tx(&full[slot], kWTileBytes);
    bulk_load(ring + slot * kWTileBytes, a.state + (int64_t)t * kWTileBytes, kWTileBytes, &full[slot]);
  };
  if (lane == 0) {
    issue_load(t_begin);
    if (t_begin + 1 < t_end) issue_load(t_begin + 1);
  }
  const int hpg = a.nheads / a.ngroups;
  const float ss0 = a.state_scale[0];
  const float xs0 = a.x_scales[0];
  const float dt_scale = *a.dt_scale;
  const float A_scale = *a.A_scale;
  const float bias_scale = (a.dt_bias != nullptr && !a.dt_bias_is_half) ? *a.dt_bias_scale : 0.0f;
  const float D_scale = a.D != nullptr ? *a.D_scale : 0.0f;
  const float z_scale = a.z != nullptr ? *a.z_scale : 0.0f;
  const int n0 = (lane & 7) * 16;
  const int tiles_per_head = a.headdim / kWTileRows;
  float bb[16], cc[16];
  int cur_bg = -1;
  // row scalars of one tile, held by lanes 0..15 (lane = row)
  struct Row { float x, dtx, dA, dsk; int hd, p; };
  auto row_prepare = [&](int t) -> Row {
    Row r{0.f, 0.f, 0.f, 0.f, 0, 0};
    const int head_lin = t / tiles_per_head;                  // (batch, head) index
    const int b = head_lin / a.nheads, hd = head_lin % a.nheads;
    const int p = (t % tiles_per_head) * kWTileRows + (lane & 15);
    r.hd = hd; r.p = p;
    if (lane < 16) {
      const float x = xs0 * (float)ld_act(a.x + (int64_t)b * a.x_sb + (int64_t)hd * a.x_sh + p);
      float bias = 0.0f;
      if (a.dt_bias != nullptr) {
        const int64_t bi = (int64_t)hd * a.bias_sh + (int64_t)p * a.bias_sp;
        bias = a.dt_bias_is_half ? __half2float(static_cast<const __half*>(a.dt_bias)[bi])
                                 : bias_scale * (float)static_cast<const int8_t*>(a.dt_bias)[bi];
      }
      float dt = fmaf(dt_scale, (float)ld_act(a.dt + (int64_t)b * a.dt_sb + (int64_t)hd * a.dt_sh + (int64_t)p * a.dt_sp), bias);
      if (a.dt_softplus) dt = softplus_f(dt);
      const float A2 = -__expf(A_scale * (float)a.A_log[(int64_t)hd * a.A_sh + (int64_t)p * a.A_sp]) * kLog2e;
      r.x = x;
      r.dtx = dt * x;
      r.dA = fast_exp2(A2 * dt);
      r.dsk = a.D != nullptr ? x * D_scale * (float)a.D[(int64_t)hd * a.D_sh + (int64_t)p * a.D_sp] : 0.0f;
    }
    return r;
  };
  Row nxt = row_prepare(t_begin);
  for (int t = t_begin; t < t_end; ++t) {
    const int k = t - t_begin;
    const int slot = k & (kWSlots - 1);
    const Row cur = nxt;
    if (t + 1 < t_end) nxt = row_prepare(t + 1);              // global loads in flight during this tile's arithmetic
    const int head_lin = t / tiles_per_head;
    const int b = head_lin / a.nheads, hd = head_lin % a.nheads;
    const int g = hd / hpg;
    if (b * a.ngroups + g != cur_bg) {                        // warp-uniform: this lane's slices of B and C
      cur_bg = b * a.ngroups + g;
      const float Bs = a.B_scale[0] / ss0, Cs = a.C_scale[0] * ss0;
      const uint4 bq = ld_act(reinterpret_cast<const uint4*>(a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg + n0));
      const uint4 cq = ld_act(reinterpret_cast<const uint4*>(a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg + n0));
      const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w}, cw[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        bb[i] = Bs * (float)(int8_t)(bw[i >> 2] >> (8 * (i & 3)));
        cc[i] = Cs * (float)(int8_t)(cw[i >> 2] >> (8 * (i & 3)));
      }
    }
    if (!mbar_wait(&full[slot], (uint32_t)((k / kWSlots) & 1), status, kStatusUpdateLoad)) break;   // all lanes wait on it
    uint8_t* tile = ring + slot * kWTileBytes;
    float ykeep = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = (lane >> 3) + 4 * e;                      // row of this piece inside the tile
      const float dtx = __shfl_sync(0xffffffffu, cur.dtx, r);
      const float dA = __shfl_sync(0xffffffffu, cur.dA, r);
      uint4* cell = reinterpret_cast<uint4*>(tile + r * 128 + n0);
      const uint4 rawst = *cell;
      const uint32_t w[4] = {rawst.x ^ 0x80808080u, rawst.y ^ 0x80808080u, rawst.z ^ 0x80808080u, rawst.w ^ 0x80808080u};
      uint32_t ow[4];
      float y = 0.0f;
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        int q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // bytes [0, v + 128, 0, 0x47] read as a float = 32768 + (v + 128); v is the state in units of its scale
          const float sv = __uint_as_float(__byte_perm(w[k4], 0x47000000u, 0x7404 | (j << 4))) - 32896.0f;
          const float v = fmaf(bb[4 * k4 + j], dtx, sv * dA);   // new state / state_scale
          q[j] = __float2int_rn(v);
          y = fmaf(v, cc[4 * k4 + j], y);
        }
        ow[k4] = pack4_sat_s8(q[0], q[1], q[2], q[3]);
      }
      *cell = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += __shfl_xor_sync(0xffffffffu, y, 4);
      // the lane that prepared row r (lane r) keeps its y: rows 4 e + (lane >> 3) live in lanes 8 (r & 3) .. of this step
      const float yrow = __shfl_sync(0xffffffffu, y, ((lane & 3) << 3));
      if ((lane >> 2) == e && lane < 16) ykeep = yrow;        // lane = 4 e + (lane & 3)
    }
    fence_proxy_async_smem();   // the tile was rewritten through the generic proxy; the bulk store reads it through the async one
    __syncwarp();
    if (lane == 0) {
      bulk_store(a.state + (int64_t)t * kWTileBytes, tile, kWTileBytes);
      bulk_commit();
      bulk_wait_read<1>();      // every store but the newest has finished reading its slot
      if (t + 2 < t_end) issue_load(t + 2);
    }
    if (lane < 16) {            // y of row `lane`: D skip term, z gate, fp16 store
      float y = ykeep + cur.dsk;
      if (a.z != nullptr) {
        const float z = z_scale * (float)ld_act(a.z + (int64_t)b * a.z_sb + (int64_t)cur.hd * a.z_sh + cur.p);
        y *= silu_exact(z);
      }
      static_cast<__half*>(a.out)[(int64_t)b * a.out_sb + (int64_t)cur.hd * a.out_sh + cur.p] = __float2half_rn(y);
    }
  }
  if (lane == 0) bulk_wait_all<0>();
}

template <int LPR, bool kTied, bool kGrouped>
__global__ void __launch_bounds__(256)
sscan_update_bulk_kernel(qb_sscan_update_args a, int tiles, int tiles_per_cta, int* status) {
  using namespace tc;
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr int kDstate = 16 * LPR;
  constexpr int kTileRows = kUpdTileBytes / kDstate;
  constexpr int kRowIters = (kTileRows + 255) / 256;  // rows a thread prepares per tile
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(16) float sB[256];   // B[n] * B_scale (/ state_scale when it is one number)
  __shared__ __align__(16) float sC[256];   // C[n] * C_scale (* state_scale when it is one number)
  __shared__ float sLut[256];               // -exp(A_scale * q) * log2(e), q = index - 128
  // per-row scalars, double-buffered: tile k uses buffer k & 1 while buffer (k + 1) & 1 is filled for the next tile
  __shared__ float rX[2][kTileRows], rDtx[2][kTileRows], rDt[2][kTileRows], rdA[2][kTileRows], rY[2][kTileRows];
  __shared__ int rScaleOfs[2][kTileRows];   // grouped scales: offset of the row's [dstate] state-scale vector
  __shared__ __align__(8) uint64_t full[kUpdSlots];
  grid_dependency_wait();   // launched as a programmatic dependent (launch_dependent)
  const int tid = threadIdx.x;
  const int t_begin = blockIdx.x * tiles_per_cta;
  const int t_end = min(tiles, t_begin + tiles_per_cta);
  if (t_begin >= t_end) return;
  if (tid == 0) {
    for (int i = 0; i < kUpdSlots; ++i) mbar_init(&full[i], 1);
    fence_barrier_init();
  }
  sLut[tid] = -__expf((*a.A_scale) * (float)(tid - 128)) * kLog2e;
  __syncthreads();
  auto issue_load = [&](int t) {
    const int slot = (t - t_begin) & (kUpdSlots - 1);
    mbar_arrive_expect_tx(&full[slot], kUpdTileBytes);
    bulk_load(ring + slot * kUpdTileBytes, a.state + (int64_t)t * kUpdTileBytes, kUpdTileBytes, &full[slot]);
  };
  if (tid == 0) {
    issue_load(t_begin);
    if (t_begin + 1 < t_end) issue_load(t_begin + 1);
  }
  const int hpg = a.nheads / a.ngroups;
  const float ss0 = kGrouped ? 1.0f : a.state_scale[0];
  const float dt_scale = *a.dt_scale;
  const float bias_scale = (a.dt_bias != nullptr && !a.dt_bias_is_half) ? *a.dt_bias_scale : 0.0f;
  const int n0 = (tid % LPR) * 16;    // both pieces of a thread, in every tile, cover the same 16 states
  float bb[16], cc[16];               // this thread's slice of sB / sC, refreshed when (batch, group) changes

  struct Coord { int b, hd0, p0; };   // (batch, head, row-in-head) of a tile's first row
  auto advance = [&](Coord c) {       // the next tile's first row: no 64-bit division in the tile loop
    c.p0 += kTileRows;
    while (c.p0 >= a.headdim) { c.p0 -= a.headdim; ++c.hd0; }
    while (c.hd0 >= a.nheads) { c.hd0 -= a.nheads; ++c.b; }
    return c;
  };
  Coord cur;
  {
    const int64_t rows_per_b = (int64_t)a.nheads * a.headdim;
    const int64_t row0 = (int64_t)t_begin * kTileRows;
    cur.b = (int)(row0 / rows_per_b);
    const int rem = (int)(row0 % rows_per_b);
    cur.hd0 = rem / a.headdim;
    cur.p0 = rem % a.headdim;
  }

  // Raw inputs of the rows this thread prepares (global loads issued early, consumed after the tile's arithmetic).
  struct RowRaw { int hd, p, xq, dtq, aq; float bias; };
  auto rows_fetch = [&](const Coord& c, RowRaw (&raw)[kRowIters]) {
#pragma unroll
    for (int i = 0; i < kRowIters; ++i) {
      const int r = tid + i * 256;
      if (r < kTileRows) {
        const unsigned pr = (unsigned)(c.p0 + r);
        const int hd = c.hd0 + (int)(pr / (unsigned)a.headdim);
        const int p = (int)(pr % (unsigned)a.headdim);
        raw[i].hd = hd; raw[i].p = p;
        raw[i].xq = ld_act(a.x + (int64_t)c.b * a.x_sb + (int64_t)hd * a.x_sh + p);
        raw[i].dtq = ld_act(a.dt + (int64_t)c.b * a.dt_sb + (int64_t)hd * a.dt_sh + (int64_t)p * a.dt_sp);
        raw[i].aq = kTied ? (int)a.A_log[(int64_t)hd * a.A_sh + (int64_t)p * a.A_sp] : 0;
        raw[i].bias = 0.0f;
        if (a.dt_bias != nullptr) {
          const int64_t bi = (int64_t)hd * a.bias_sh + (int64_t)p * a.bias_sp;
          raw[i].bias = a.dt_bias_is_half ? __half2float(static_cast<const __half*>(a.dt_bias)[bi])
                                          : bias_scale * (float)static_cast<const int8_t*>(a.dt_bias)[bi];
        }
      }
    }
  };
  auto rows_finish = [&](const Coord& c, const RowRaw (&raw)[kRowIters], int buf) {
#pragma unroll
    for (int i = 0; i < kRowIters; ++i) {
      const int r = tid + i * 256;
      if (r < kTileRows) {
        float xs;
        if (kGrouped) {
          const int g = c.hd0 / hpg;
          const int hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, raw[i].hd % hpg);
          const int dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, raw[i].p);
          const int cell = (g * a.nhead_groups + hg) * a.ndim_groups + dg;
          xs = a.x_scales[cell];
          rScaleOfs[buf][r] = cell * a.dstate;
        } else {
          xs = a.x_scales[0];
        }
        const float x = xs * (float)raw[i].xq;
        float dt = fmaf(dt_scale, (float)raw[i].dtq, raw[i].bias);
        if (a.dt_softplus) dt = softplus_f(dt);
        rX[buf][r] = x;
        rDt[buf][r] = dt;
        rDtx[buf][r] = dt * x;
        if (kTied) rdA[buf][r] = fast_exp2(sLut[raw[i].aq + 128] * dt);
      }
    }
  };
  // y of a finished tile: D skip term, z gate, fp16 store, one thread per row
  auto rows_store = [&](const Coord& c, int buf) {
    for (int r = tid; r < kTileRows; r += 256) {
      const unsigned pr = (unsigned)(c.p0 + r);
      const int hd = c.hd0 + (int)(pr / (unsigned)a.headdim);
      const int p = (int)(pr % (unsigned)a.headdim);
      float y = rY[buf][r];
      if (a.D != nullptr) y = fmaf(rX[buf][r], (*a.D_scale) * (float)a.D[(int64_t)hd * a.D_sh + (int64_t)p * a.D_sp], y);
      if (a.z != nullptr) {
        const float z = (*a.z_scale) * (float)ld_act(a.z + (int64_t)c.b * a.z_sb + (int64_t)hd * a.z_sh + p);
        y *= silu_exact(z);
      }
      static_cast<__half*>(a.out)[(int64_t)c.b * a.out_sb + (int64_t)hd * a.out_sh + p] = __float2half_rn(y);
    }
  };

  RowRaw raw[kRowIters];
  rows_fetch(cur, raw);
  rows_finish(cur, raw, 0);
  int cur_bg = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int k = t - t_begin;
    const int slot = k & (kUpdSlots - 1);
    const int buf = k & 1;
    const Coord nxt = advance(cur);
    const bool has_next = t + 1 < t_end;
    if (has_next) rows_fetch(nxt, raw);  // in flight during this tile's arithmetic
    const int g = cur.hd0 / hpg;
    const bool restage = cur.b * a.ngroups + g != cur_bg;  // block-uniform: the tile enters a new (batch, group)
    if (restage) {
      cur_bg = cur.b * a.ngroups + g;
      if (tid < kDstate) {
        const float Bs = kGrouped ? a.B_scale[g] : a.B_scale[0];
        const float Cs = kGrouped ? a.C_scale[g] : a.C_scale[0];
        sB[tid] = Bs * (float)ld_act(a.Bm + (int64_t)cur.b * a.B_sb + (int64_t)g * a.B_sg + tid) / ss0;
        sC[tid] = Cs * (float)ld_act(a.Cm + (int64_t)cur.b * a.C_sb + (int64_t)g * a.C_sg + tid) * ss0;
      }
    }
    __syncthreads();  // row scalars of this tile (written last iteration) and sB / sC are visible
    if (restage) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 bf = *reinterpret_cast<const float4*>(sB + n0 + 4 * i);
        const float4 cf = *reinterpret_cast<const float4*>(sC + n0 + 4 * i);
        bb[4 * i] = bf.x; bb[4 * i + 1] = bf.y; bb[4 * i + 2] = bf.z; bb[4 * i + 3] = bf.w;
        cc[4 * i] = cf.x; cc[4 * i + 1] = cf.y; cc[4 * i + 2] = cf.z; cc[4 * i + 3] = cf.w;
      }
    }
    const bool ok = mbar_wait(&full[slot], (uint32_t)((k / kUpdSlots) & 1), status, kStatusUpdateLoad);
    if (!ok) break;  // every thread waits on the same barrier, so all leave together
    uint8_t* tile = ring + slot * kUpdTileBytes;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int piece = tid + e * 256;
      const int r = piece / LPR;
      uint4* cell = reinterpret_cast<uint4*>(tile + piece * 16);
      const uint4 rawst = *cell;
      const uint32_t w[4] = {rawst.x ^ 0x80808080u, rawst.y ^ 0x80808080u, rawst.z ^ 0x80808080u, rawst.w ^ 0x80808080u};
      const float dtx = rDtx[buf][r];
      const float dA_row = kTied ? rdA[buf][r] : 0.0f;
      const float dt = kTied ? 0.0f : rDt[buf][r];
      const int8_t* Aq = nullptr;
      if (!kTied) {
        const unsigned pr = (unsigned)(cur.p0 + r);
        Aq = a.A_log + (int64_t)(cur.hd0 + (int)(pr / (unsigned)a.headdim)) * a.A_sh +
             (int64_t)(pr % (unsigned)a.headdim) * a.A_sp + (int64_t)n0 * a.A_sn;
      }
      const float* ssn = kGrouped ? a.state_scale + rScaleOfs[buf][r] + n0 : nullptr;
      uint32_t ow[4];
      float y = 0.0f;
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        float bs[4], cs[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { bs[j] = bb[4 * k4 + j]; cs[j] = cc[4 * k4 + j]; }
        if (kGrouped) {  // per-state scales: fold them into this piece's B and C values
          const float4 sc = __ldg(reinterpret_cast<const float4*>(ssn + 4 * k4));
          const float sv4[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { bs[j] *= __frcp_rn(sv4[j]); cs[j] *= sv4[j]; }
        }
        int q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // bytes [0, v + 128, 0, 0x47] read as a float = 32768 + (v + 128); v is the state in units of its scale
          const float sv = __uint_as_float(__byte_perm(w[k4], 0x47000000u, 0x7404 | (j << 4))) - 32896.0f;
          float dA = dA_row;
          if (!kTied) dA = fast_exp2(sLut[(int)Aq[(int64_t)(4 * k4 + j) * a.A_sn] + 128] * dt);
          const float v = fmaf(bs[j], dtx, sv * dA);  // new state / state_scale
          q[j] = __float2int_rn(v);
          y = fmaf(v, cs[j], y);
        }
        ow[k4] = pack4_sat_s8(q[0], q[1], q[2], q[3]);
      }
      *cell = make_uint4(ow[0], ow[1], ow[2], ow[3]);
#pragma unroll
      for (int m = 1; m < LPR; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
      if (piece % LPR == 0) rY[buf][r] = y;
    }
    if (has_next) rows_finish(nxt, raw, buf ^ 1);
    fence_proxy_async_smem();  // the tile was rewritten through the generic proxy; the bulk store reads it through the async one
    __syncthreads();
    if (tid == 0) {
      bulk_store(a.state + (int64_t)t * kUpdTileBytes, tile, kUpdTileBytes);
      bulk_commit();
      bulk_wait_read<1>();  // every store but the newest has finished reading its slot
      if (t + 2 < t_end) issue_load(t + 2);
    }
    rows_store(cur, buf);  // buffer `buf` is next written two iterations from now, after two more barriers
    cur = nxt;
  }
  if (tid == 0) bulk_wait_all<0>();
}

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qb_sscan_fwd(const qb_sscan_fwd_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "sscan_fwd: null args");
  QB_REQUIRE(a->u && a->delta && a->Bm && a->Cm && a->A_log && a->out && a->x_states, QB_ERR_INVALID_ARG,
             "sscan_fwd: null tensor pointer");
  QB_REQUIRE(a->u_scale && a->delta_scale && a->B_scale && a->C_scale && a->A_scale && a->ssm_state_scale,
             QB_ERR_INVALID_ARG, "sscan_fwd: null scale pointer");
  QB_REQUIRE(a->D == nullptr || a->D_scale != nullptr, QB_ERR_INVALID_ARG, "sscan_fwd: D without D_scale");
  QB_REQUIRE(a->z == nullptr || a->z_scale != nullptr, QB_ERR_INVALID_ARG, "sscan_fwd: z without z_scale");
  QB_REQUIRE(a->delta_bias == nullptr || a->delta_bias_scale != nullptr, QB_ERR_INVALID_ARG,
             "sscan_fwd: delta_bias without its scale");
  QB_REQUIRE(a->batch > 0 && a->dim > 0 && a->seqlen > 0 && a->n_groups > 0, QB_ERR_INVALID_ARG, "sscan_fwd: empty shape");
  QB_REQUIRE(a->dstate <= 256, QB_ERR_INVALID_ARG, "quant_sscan only supports state dimension <= 256");
  QB_REQUIRE(a->dim % a->n_groups == 0, QB_ERR_INVALID_ARG, "sscan_fwd: dim not divisible by n_groups");
  const int kRows = rows_per_cta(a->dstate);
  QB_REQUIRE(a->n_groups == 1 || (a->dim / a->n_groups) % kRows == 0, QB_ERR_UNSUPPORTED,
             "sscan_fwd: channels per group must be a multiple of %d", kRows);
  const int vec_ok = aligned(a->u, 16) && aligned(a->delta, 16) && (a->z == nullptr || aligned(a->z, 16)) &&
                     aligned(a->Bm, 16) && aligned(a->Cm, 16) && a->u_sd % 16 == 0 && a->u_sb % 16 == 0 &&
                     a->delta_sd % 16 == 0 && a->delta_sb % 16 == 0 && a->z_sd % 16 == 0 && a->z_sb % 16 == 0 &&
                     a->B_sn % 16 == 0 && a->B_sg % 16 == 0 && a->B_sb % 16 == 0 && a->C_sn % 16 == 0 &&
                     a->C_sg % 16 == 0 && a->C_sb % 16 == 0;
  const int tiles_d = (int)ceil_div(a->dim, kRows);
  const unsigned grid = (unsigned)(a->batch * tiles_d);
  cudaStream_t st = (cudaStream_t)stream;
  const int has_z = a->z != nullptr;
  switch (a->dstate) {
    case 8: sscan_fwd_kernel<8, rows_per_cta(8)><<<grid, kRows, 0, st>>>(*a, has_z, vec_ok); break;
    case 16: sscan_fwd_kernel<16, rows_per_cta(16)><<<grid, kRows, 0, st>>>(*a, has_z, vec_ok); break;
    case 32: sscan_fwd_kernel<32, rows_per_cta(32)><<<grid, kRows, 0, st>>>(*a, has_z, vec_ok); break;
    case 64: sscan_fwd_kernel<64, rows_per_cta(64)><<<grid, kRows, 0, st>>>(*a, has_z, vec_ok); break;
    default:
      set_error("sscan_fwd: dstate %d not built (8, 16, 32, 64 are)", a->dstate);
      return QB_ERR_UNSUPPORTED;
  }
  QB_LAUNCH_OK("sscan_fwd_kernel");
  return QB_OK;
}

extern "C" int qb_sscan_update(const qb_sscan_update_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "sscan_update: null args");
  QB_REQUIRE(a->state && a->x && a->dt && a->A_log && a->Bm && a->Cm && a->out, QB_ERR_INVALID_ARG,
             "sscan_update: null tensor pointer");
  QB_REQUIRE(a->x_scales && a->dt_scale && a->A_scale && a->state_scale && a->B_scale && a->C_scale,
             QB_ERR_INVALID_ARG, "sscan_update: null scale pointer");
  QB_REQUIRE(a->D == nullptr || a->D_scale != nullptr, QB_ERR_INVALID_ARG, "sscan_update: D without D_scale");
  QB_REQUIRE(a->z == nullptr || a->z_scale != nullptr, QB_ERR_INVALID_ARG, "sscan_update: z without z_scale");
  QB_REQUIRE(a->dt_bias == nullptr || a->dt_bias_is_half || a->dt_bias_scale != nullptr, QB_ERR_INVALID_ARG,
             "sscan_update: int8 dt_bias without its scale");
  QB_REQUIRE(a->batch > 0 && a->nheads > 0 && a->headdim > 0 && a->dstate > 0 && a->ngroups > 0,
             QB_ERR_INVALID_ARG, "sscan_update: empty shape");
  QB_REQUIRE(a->nheads % a->ngroups == 0, QB_ERR_INVALID_ARG, "nheads must be divisible by ngroups");
  QB_REQUIRE(!a->grouped || (a->head_group_range && a->dim_group_range && a->nhead_groups > 0 && a->ndim_groups > 0),
             QB_ERR_INVALID_ARG, "sscan_update: grouped scales need the range tables");
  // warp-autonomous kernel: the Mamba2 decode shape (d_state 128, A tied across the state, per-tensor scales), fully
  // few (batch, head) pairs: the low-latency kernel, one CTA per pair
  if (a->dstate == 128 && a->A_sn == 0 && a->A_sp == 0 && a->dt_sp == 0 && !a->grouped && a->z == nullptr && a->headdim % 64 == 0 &&
      (a->D == nullptr || a->D_sp == 0) && (a->dt_bias == nullptr || a->bias_sp == 0) && a->state_sp % 16 == 0 && a->state_sh % 16 == 0 &&
      a->state_sb % 16 == 0 && aligned(a->state, 16) && aligned(a->Bm, 16) && aligned(a->Cm, 16) && a->B_sb % 16 == 0 && a->B_sg % 16 == 0 &&
      a->C_sb % 16 == 0 && a->C_sg % 16 == 0 && (int64_t)a->batch * a->nheads <= (int64_t)sm_count() * 4 && a->batch <= 65535 &&
      !path_override(QB_PATH_UPDATE_CTA_TILES)) {
    launch_dependent(sscan_update_small_kernel, dim3((unsigned)a->nheads, (unsigned)a->batch), dim3(256), 0, (cudaStream_t)stream, *a);
    QB_LAUNCH_OK("sscan_update_small_kernel");
    return QB_OK;
  }
  QB_REQUIRE(!a->early_launch, QB_ERR_UNSUPPORTED,
             "sscan_update: early_launch is only offered on the one-CTA-per-head decode kernel, which this call is not eligible for");
  // contiguous state, 16-row tiles inside one head
  if (a->dstate == 128 && a->A_sn == 0 && !a->grouped && a->headdim % kWTileRows == 0 && aligned(a->state, 16) &&
      a->state_sp == a->dstate && a->state_sh == (int64_t)a->headdim * a->dstate &&
      a->state_sb == (int64_t)a->nheads * a->headdim * a->dstate && aligned(a->Bm, 16) && aligned(a->Cm, 16) &&
      a->B_sb % 16 == 0 && a->B_sg % 16 == 0 && a->C_sb % 16 == 0 && a->C_sg % 16 == 0 &&
      !path_override(QB_PATH_UPDATE_CTA_TILES)) {
    int* status = device_status_ptr();
    QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "sscan_update: device status word unavailable");
    static PerDeviceOnce wattr;
    const size_t wsmem = (size_t)8 * kWSlots * kWTileBytes;
    if (wattr.first())
      QB_CUDA_OK(cudaFuncSetAttribute(sscan_update_warp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem));
    const int64_t rows = (int64_t)a->batch * a->nheads * a->headdim;
    const int wtiles = (int)(rows / kWTileRows);
    const int wctas = (int)std::min<int64_t>(ceil_div(wtiles, 8), (int64_t)sm_count() * 3);
    launch_dependent(sscan_update_warp_kernel, dim3((unsigned)wctas), dim3(256), wsmem, (cudaStream_t)stream, *a, wtiles, status);
    QB_LAUNCH_OK("sscan_update_warp_kernel");
    return QB_OK;
  }
  // pipelined kernel: fully contiguous state, dstate in {16, 32, 64, 128, 256}, whole 8 KB tiles inside one (batch, group)
  {
    const int lpr = a->dstate / 16;
    const bool pow2 = a->dstate % 16 == 0 && lpr >= 1 && lpr <= 16 && (lpr & (lpr - 1)) == 0;
    const int64_t rows = (int64_t)a->batch * a->nheads * a->headdim;
    const int64_t rows_per_group = (int64_t)(a->nheads / a->ngroups) * a->headdim;
    if (pow2 && aligned(a->state, 16) && a->state_sp == a->dstate && a->state_sh == (int64_t)a->headdim * a->dstate &&
        a->state_sb == (int64_t)a->nheads * a->headdim * a->dstate && (!a->grouped || aligned(a->state_scale, 16)) &&
        rows_per_group % (kUpdTileBytes / a->dstate) == 0) {
      const int tiles = (int)(rows * a->dstate / kUpdTileBytes);
      const int ctas = (int)std::min<int64_t>(tiles, (int64_t)sm_count() * 3);
      const int tiles_per_cta = (int)ceil_div(tiles, ctas);
      const unsigned grid = (unsigned)ceil_div(tiles, tiles_per_cta);
      const size_t smem = (size_t)kUpdSlots * kUpdTileBytes;
      cudaStream_t st = (cudaStream_t)stream;
      int* status = device_status_ptr();
      QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "sscan_update: device status word unavailable");
      const bool tied = a->A_sn == 0;
      const bool grp = a->grouped != 0;
#define QB_UPD_LAUNCH(L)                                                                                           \
  do {                                                                                                             \
    static PerDeviceOnce attr_done; /* static + dynamic shared memory exceeds 48 KB for small dstate */          \
    if (attr_done.first()) {                                                                                       \
      QB_CUDA_OK(cudaFuncSetAttribute(sscan_update_bulk_kernel<L, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));   \
      QB_CUDA_OK(cudaFuncSetAttribute(sscan_update_bulk_kernel<L, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));    \
      QB_CUDA_OK(cudaFuncSetAttribute(sscan_update_bulk_kernel<L, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));  \
      QB_CUDA_OK(cudaFuncSetAttribute(sscan_update_bulk_kernel<L, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));   \
    }                                                                                                              \
    if (tied && !grp) launch_dependent(sscan_update_bulk_kernel<L, true, false>, dim3(grid), dim3(256), smem, st, *a, tiles, tiles_per_cta, status);      \
    else if (tied && grp) launch_dependent(sscan_update_bulk_kernel<L, true, true>, dim3(grid), dim3(256), smem, st, *a, tiles, tiles_per_cta, status);   \
    else if (!grp) launch_dependent(sscan_update_bulk_kernel<L, false, false>, dim3(grid), dim3(256), smem, st, *a, tiles, tiles_per_cta, status);        \
    else launch_dependent(sscan_update_bulk_kernel<L, false, true>, dim3(grid), dim3(256), smem, st, *a, tiles, tiles_per_cta, status);                   \
  } while (0)
      switch (lpr) {
        case 1: QB_UPD_LAUNCH(1); break;
        case 2: QB_UPD_LAUNCH(2); break;
        case 4: QB_UPD_LAUNCH(4); break;
        case 8: QB_UPD_LAUNCH(8); break;
        default: QB_UPD_LAUNCH(16); break;
      }
#undef QB_UPD_LAUNCH
      QB_LAUNCH_OK("sscan_update_bulk_kernel");
      return QB_OK;
    }
  }
  // streaming kernel: 16-byte pieces of aligned state rows, every CTA inside one (batch, SSD group)
  if (a->dstate % 16 == 0 && a->dstate <= 256 && aligned(a->state, 16) && a->state_sp % 16 == 0 && a->state_sh % 16 == 0 &&
      a->state_sb % 16 == 0 && (!a->grouped || aligned(a->state_scale, 16))) {
    const int pieces = a->dstate / 16;
    int lanes = 1;
    while (lanes < 8 && pieces % (2 * lanes) == 0) lanes *= 2;
    const int rows_per_cta = 256 / lanes;
    const int64_t rows_per_group = (int64_t)(a->nheads / a->ngroups) * a->headdim;
    if (rows_per_group % rows_per_cta == 0) {
      const int64_t rows = (int64_t)a->batch * a->nheads * a->headdim;
      const unsigned grid = (unsigned)(rows / rows_per_cta);
      const int iters = pieces / lanes;
      cudaStream_t st = (cudaStream_t)stream;
      switch (lanes) {
        case 1: sscan_update_stream_kernel<1><<<grid, 256, 0, st>>>(*a, iters); break;
        case 2: sscan_update_stream_kernel<2><<<grid, 256, 0, st>>>(*a, iters); break;
        case 4: sscan_update_stream_kernel<4><<<grid, 256, 0, st>>>(*a, iters); break;
        default: sscan_update_stream_kernel<8><<<grid, 256, 0, st>>>(*a, iters); break;
      }
      QB_LAUNCH_OK("sscan_update_stream_kernel");
      return QB_OK;
    }
  }
  const int64_t threads = (int64_t)a->batch * a->nheads * a->headdim * 8;
  sscan_update_kernel<<<(unsigned)ceil_div(threads, 128), 128, 0, (cudaStream_t)stream>>>(*a);
  QB_LAUNCH_OK("sscan_update_kernel");
  return QB_OK;
}
