// Mamba2 int8 SSD chunk scan with inter-chunk state passing for sm_100a.
//
// Stages (all on the caller's stream, scratch in the caller's workspace):
//   1. dt / dA cumsum per (batch, chunk, head)                          -> ws.dt, ws.dA   fp32
//   2. C B^T per (batch, chunk, group), exact (int8 products summed in fp32 stay < 2^24)
//                                                                       -> ws.CB         fp32
//   3. per-chunk states  S_c[p,n] = sum_l x[l,p] B[l,n] exp(dA_end - dA_l) dt_l
//                                                                       -> ws.states     fp32
//   4. inter-chunk recurrence s <- exp(dA_end) s + S_c; the state entering each chunk is kept in
//      fp16 (as the reference stores it), the last one is requantised to int8 (rint + clamp)
//                                                                       -> ws.prev fp16, final int8
//   5. y[m,p] = exp(dA_m) C[m,:] . prev[p,:] + sum_{k<=m} CB[m,k] exp(dA_m - dA_k) dt_k x[k,p]
//               + D x[m,p]   (optionally gated by z)                    -> out fp16
// Contraction operands are rounded to fp16 before multiplication and accumulated in fp32, which
// is what the reference's tensor-core dots do.
#include "common.cuh"

#include <stdlib.h>

namespace qb {
namespace {

constexpr int TM = 64, TN = 64, TK = 32;
constexpr int kThreads = 256;

struct Ws {
  float* dt;      // [B, nc, H, Q]
  float* dA;      // [B, nc, H, Q]  cumulative within the chunk
  float* CB;      // [B, nc, G, Q, Q]
  float* states;  // [B, nc, H, P, N]
  __half* prev;   // [B, nc, H, P, N]
};

__host__ __device__ inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

struct WsLayout {
  int64_t off_dt, off_dA, off_CB, off_states, off_prev, total;
};

WsLayout ws_layout(int B, int L, int H, int P, int G, int N, int Q) {
  const int64_t nc = (L + Q - 1) / Q;
  WsLayout w;
  int64_t o = 0;
  w.off_dt = o; o = align256(o + (int64_t)B * nc * H * Q * 4);
  w.off_dA = o; o = align256(o + (int64_t)B * nc * H * Q * 4);
  w.off_CB = o; o = align256(o + (int64_t)B * nc * G * Q * Q * 4);
  w.off_states = o; o = align256(o + (int64_t)B * nc * H * P * N * 4);
  w.off_prev = o; o = align256(o + (int64_t)B * nc * H * P * N * 2);
  w.total = o;
  return w;
}

__device__ __forceinline__ float f16r(float v) { return __half2float(__float2half_rn(v)); }

// ---- stage 1 ---------------------------------------------------------------------------------
__global__ void ssd_cumsum_kernel(qb_ssd_args a, Ws ws, int nc) {
  const int b = blockIdx.x / nc, c = blockIdx.x % nc;
  const int Q = a.chunk_size;
  for (int h = threadIdx.x; h < a.nheads; h += blockDim.x) {
    const float A = -__expf((*a.A_scale) * (float)a.A_log[h]);
    const float bias = a.dt_bias != nullptr ? __half2float(static_cast<const __half*>(a.dt_bias)[h]) : 0.0f;
    const float s_dt = *a.dt_scale;
    float* dt_o = ws.dt + (((int64_t)b * nc + c) * a.nheads + h) * Q;
    float* dA_o = ws.dA + (((int64_t)b * nc + c) * a.nheads + h) * Q;
    float cs = 0.0f;
    for (int q = 0; q < Q; ++q) {
      const int l = c * Q + q;
      float dt = 0.0f;
      if (l < a.seqlen) {
        dt = fmaf(s_dt, (float)a.dt[(int64_t)b * a.dt_sb + (int64_t)l * a.dt_sl + h], bias);
        if (a.dt_softplus) dt = softplus_f(dt);
        dt = fminf(fmaxf(dt, a.dt_min), a.dt_max);
      }
      cs += dt * A;
      dt_o[q] = dt;
      dA_o[q] = cs;
    }
  }
}

// ---- shared 64x64 tile contraction -----------------------------------------------------------
// acc[i][j] += sum_k A(m0+tm+i, k) * B(k, n0+tn+j), k in [kbeg, kend); A / B come from functors
// fa(m, k), fb(k, n) (tile-relative m, n; absolute k).  FAST_K_x selects which index consecutive
// threads walk when filling the tile so that the functor's global reads coalesce.
template <bool FAST_K_A, bool FAST_K_B, class FA, class FB>
__device__ __forceinline__ void tile_contract(float (&acc)[4][4], int kbeg, int kend, FA fa, FB fb,
                                              float (*As)[TM + 4], float (*Bs)[TN + 4]) {
  const int tid = threadIdx.x;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  for (int k0 = kbeg; k0 < kend; k0 += TK) {
    __syncthreads();
    for (int e = tid; e < TK * TM; e += kThreads) {
      const int kk = FAST_K_A ? (e % TK) : (e / TM);
      const int mm = FAST_K_A ? (e / TK) : (e % TM);
      As[kk][mm] = (k0 + kk < kend) ? fa(mm, k0 + kk) : 0.0f;
    }
    for (int e = tid; e < TK * TN; e += kThreads) {
      const int kk = FAST_K_B ? (e % TK) : (e / TN);
      const int nn = FAST_K_B ? (e / TK) : (e % TN);
      Bs[kk][nn] = (k0 + kk < kend) ? fb(k0 + kk, nn) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][tm]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tn]);
      const float aa[4] = {av.x, av.y, av.z, av.w};
      const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
    }
  }
}

// ---- stage 2: CB ------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
ssd_cb_kernel(qb_ssd_args a, Ws ws, int nc) {
  __shared__ __align__(16) float As[TK][TM + 4];
  __shared__ __align__(16) float Bs[TK][TN + 4];
  const int Q = a.chunk_size;
  const int tiles = Q / TM;
  const int mt = blockIdx.x / tiles, kt = blockIdx.x % tiles;
  if (kt > mt) return;  // only k <= m is ever read
  const int bcg = blockIdx.y;
  const int g = bcg % a.ngroups;
  const int c = (bcg / a.ngroups) % nc;
  const int b = bcg / (a.ngroups * nc);
  const int8_t* Cq = a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg;
  const int8_t* Bq = a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg;
  const int lbase = c * Q;
  float acc[4][4] = {};
  auto fa = [&](int m, int n) -> float {
    const int l = lbase + mt * TM + m;
    return l < a.seqlen ? (float)Cq[(int64_t)l * a.C_sl + n] : 0.0f;
  };
  auto fb = [&](int n, int k) -> float {
    const int l = lbase + kt * TN + k;
    return l < a.seqlen ? (float)Bq[(int64_t)l * a.B_sl + n] : 0.0f;
  };
  tile_contract<true, true>(acc, 0, a.dstate, fa, fb, As, Bs);
  const float sc = (a.grouped ? a.C_scale[g] : a.C_scale[0]) * (a.grouped ? a.B_scale[g] : a.B_scale[0]);
  float* cb = ws.CB + (((int64_t)b * nc + c) * a.ngroups + g) * Q * Q;
  const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 v = make_float4(acc[i][0] * sc, acc[i][1] * sc, acc[i][2] * sc, acc[i][3] * sc);
    *reinterpret_cast<float4*>(cb + (int64_t)(mt * TM + tm + i) * Q + kt * TN + tn) = v;
  }
}

__device__ __forceinline__ float x_scale_of(const qb_ssd_args& a, int h, int p) {
  if (!a.grouped) return a.x_scales[0];
  const int hpg = a.nheads / a.ngroups;
  const int g = h / hpg;
  const int hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, h % hpg);
  const int dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, p);
  return a.x_scales[(g * a.nhead_groups + hg) * a.ndim_groups + dg];
}

// ---- stage 3: per-chunk states -----------------------------------------------------------------
// grid: x = (P/64) * (N/64) tiles, y = b * nc * H
__global__ void __launch_bounds__(kThreads)
ssd_chunk_state_kernel(qb_ssd_args a, Ws ws, int nc) {
  __shared__ __align__(16) float As[TK][TM + 4];
  __shared__ __align__(16) float Bs[TK][TN + 4];
  __shared__ float s_w[1024];
  __shared__ float s_xs[TM];
  const int Q = a.chunk_size;
  const int ntn = a.dstate / TN;
  const int pt = blockIdx.x / ntn, nt = blockIdx.x % ntn;
  const int h = blockIdx.y % a.nheads;
  const int c = (blockIdx.y / a.nheads) % nc;
  const int b = blockIdx.y / (a.nheads * nc);
  const int g = h / (a.nheads / a.ngroups);
  const float* dt = ws.dt + (((int64_t)b * nc + c) * a.nheads + h) * Q;
  const float* dA = ws.dA + (((int64_t)b * nc + c) * a.nheads + h) * Q;
  const float dA_last = dA[Q - 1];
  const float sB = a.grouped ? a.B_scale[g] : a.B_scale[0];
  for (int q = threadIdx.x; q < Q; q += kThreads) s_w[q] = __expf(dA_last - dA[q]) * dt[q];
  if (threadIdx.x < TM) s_xs[threadIdx.x] = x_scale_of(a, h, pt * TM + threadIdx.x);
  __syncthreads();
  const int8_t* xq = a.x + (int64_t)b * a.x_sb + (int64_t)h * a.x_sh;
  const int8_t* Bq = a.Bm + (int64_t)b * a.B_sb + (int64_t)g * a.B_sg;
  const int lbase = c * Q;
  const int lim = min(Q, a.seqlen - lbase);
  float acc[4][4] = {};
  auto fa = [&](int p, int l) -> float {
    return f16r(s_xs[p] * (float)xq[(int64_t)(lbase + l) * a.x_sl + pt * TM + p]);
  };
  auto fb = [&](int l, int n) -> float {
    return f16r(sB * (float)Bq[(int64_t)(lbase + l) * a.B_sl + nt * TN + n] * s_w[l]);
  };
  tile_contract<false, false>(acc, 0, lim, fa, fb, As, Bs);
  float* st = ws.states + ((((int64_t)b * nc + c) * a.nheads + h) * a.headdim) * a.dstate;
  const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    *reinterpret_cast<float4*>(st + (int64_t)(pt * TM + tm + i) * a.dstate + nt * TN + tn) =
        make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  }
}

// ---- stage 4: inter-chunk recurrence ------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
ssd_state_passing_kernel(qb_ssd_args a, Ws ws, int nc) {
  const int PN = a.headdim * a.dstate;
  const int h = blockIdx.y, b = blockIdx.z;
  const int e = blockIdx.x * kThreads + threadIdx.x;
  if (e >= PN) return;
  const int p = e / a.dstate, n = e % a.dstate;
  const int Q = a.chunk_size;
  float s = 0.0f;
  for (int c = 0; c < nc; ++c) {
    const int64_t base = (((int64_t)b * nc + c) * a.nheads + h);
    ws.prev[base * PN + e] = __float2half_rn(s);
    const float dA_last = ws.dA[base * Q + Q - 1];
    s = fmaf(__expf(dA_last), s, ws.states[base * PN + e]);
  }
  float ss;
  if (!a.grouped) {
    ss = a.ssm_state_scale[0];
  } else {
    const int hpg = a.nheads / a.ngroups;
    const int g = h / hpg;
    const int hg = group_lookup(a.head_group_range + g * a.nhead_groups, a.nhead_groups, h % hpg);
    const int dg = group_lookup(a.dim_group_range + (g * a.nhead_groups + hg) * a.ndim_groups, a.ndim_groups, p);
    ss = a.ssm_state_scale[((int64_t)(g * a.nhead_groups + hg) * a.ndim_groups + dg) * a.dstate + n];
  }
  const float fin = __half2float(__float2half_rn(s));
  a.final_states[((int64_t)b * a.nheads + h) * PN + e] = (int8_t)rint_s8(fin / ss);
}

// ---- stage 5: output ----------------------------------------------------------------------------
// grid: x = (Q/64) m-tiles * (P/64) p-tiles, y = b * nc * H
__global__ void __launch_bounds__(kThreads)
ssd_chunk_scan_kernel(qb_ssd_args a, Ws ws, int nc) {
  __shared__ __align__(16) float As[TK][TM + 4];
  __shared__ __align__(16) float Bs[TK][TN + 4];
  __shared__ float s_dA[1024];
  __shared__ float s_dt[1024];
  __shared__ float s_xs[TN];
  const int Q = a.chunk_size;
  const int npt = a.headdim / TN;
  const int mt = blockIdx.x / npt, pt = blockIdx.x % npt;
  const int h = blockIdx.y % a.nheads;
  const int c = (blockIdx.y / a.nheads) % nc;
  const int b = blockIdx.y / (a.nheads * nc);
  const int g = h / (a.nheads / a.ngroups);
  const int lbase = c * Q;
  const int lim = min(Q, a.seqlen - lbase);
  if (mt * TM >= lim) return;
  const int64_t bch = ((int64_t)b * nc + c) * a.nheads + h;
  for (int q = threadIdx.x; q < Q; q += kThreads) {
    s_dA[q] = ws.dA[bch * Q + q];
    s_dt[q] = ws.dt[bch * Q + q];
  }
  if (threadIdx.x < TN) s_xs[threadIdx.x] = x_scale_of(a, h, pt * TN + threadIdx.x);
  __syncthreads();
  const float sC = a.grouped ? a.C_scale[g] : a.C_scale[0];
  const int8_t* Cq = a.Cm + (int64_t)b * a.C_sb + (int64_t)g * a.C_sg;
  const int8_t* xq = a.x + (int64_t)b * a.x_sb + (int64_t)h * a.x_sh;
  const __half* prev = ws.prev + bch * a.headdim * a.dstate;
  const float* cb = ws.CB + (((int64_t)b * nc + c) * a.ngroups + g) * Q * Q;
  const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;

  float acc[4][4] = {};
  {  // C . prev^T, scaled by exp(dA_m)
    auto fa = [&](int m, int n) -> float {
      const int l = lbase + mt * TM + m;
      return l < a.seqlen ? f16r(sC * (float)Cq[(int64_t)l * a.C_sl + n]) : 0.0f;
    };
    auto fb = [&](int n, int p) -> float { return __half2float(prev[(int64_t)(pt * TN + p) * a.dstate + n]); };
    tile_contract<true, true>(acc, 0, a.dstate, fa, fb, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float e = __expf(s_dA[mt * TM + tm + i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] *= e;
    }
  }
  {  // causal intra-chunk term
    auto fa = [&](int m, int k) -> float {
      const int mm = mt * TM + m;
      if (k > mm) return 0.0f;
      return f16r(cb[(int64_t)mm * Q + k] * __expf(s_dA[mm] - s_dA[k]) * s_dt[k]);
    };
    auto fb = [&](int k, int p) -> float {
      return f16r(s_xs[p] * (float)xq[(int64_t)(lbase + k) * a.x_sl + pt * TN + p]);
    };
    tile_contract<true, false>(acc, 0, min((mt + 1) * TM, lim), fa, fb, As, Bs);
  }
  __half* out = static_cast<__half*>(a.out) + ((int64_t)b * a.seqlen * a.nheads + h) * a.headdim;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = mt * TM + tm + i;
    const int l = lbase + m;
    if (l >= a.seqlen) continue;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = pt * TN + tn + j;
      v[j] = acc[i][j];
      if (a.D != nullptr) {
        const float Dv = (*a.D_scale) * (float)(a.D_has_hdim ? a.D[h * a.headdim + p] : a.D[h]);
        v[j] = fmaf(s_xs[tn + j] * (float)xq[(int64_t)l * a.x_sl + p], Dv, v[j]);
      }
      if (a.z != nullptr) {
        const float z = (*a.z_scale) * (float)a.z[(int64_t)b * a.z_sb + (int64_t)l * a.z_sl + (int64_t)h * a.z_sh + p];
        v[j] *= silu_exact(z);
      }
    }
    __half2* o = reinterpret_cast<__half2*>(out + (int64_t)l * a.nheads * a.headdim + pt * TN + tn);
    o[0] = __floats2half2_rn(v[0], v[1]);
    o[1] = __floats2half2_rn(v[2], v[3]);
  }
}

}  // namespace

// Tensor-core path (ssd_tc.cu): headdim 64, d_state 128, no z gate.
bool ssd_tc_eligible(const qb_ssd_args* a);
int64_t ssd_tc_workspace_bytes(int B, int L, int H, int G);
int ssd_tc_launch(const qb_ssd_args* a, cudaStream_t st);

namespace {
bool force_portable() {  // selects the five-stage path (used to cross-check the two on a device)
  return path_override(QB_PATH_SSD_PORTABLE);
}
int64_t total_workspace(int B, int L, int H, int P, int G, int N, int Q) {
  const int64_t a = ws_layout(B, L, H, P, G, N, Q).total;
  const int64_t b = ssd_tc_workspace_bytes(B, L, H, G);
  return a > b ? a : b;
}
}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int64_t qb_ssd_workspace_bytes(int32_t batch, int32_t seqlen, int32_t nheads, int32_t headdim,
                                          int32_t ngroups, int32_t dstate, int32_t chunk_size) {
  if (batch <= 0 || seqlen <= 0 || nheads <= 0 || headdim <= 0 || ngroups <= 0 || dstate <= 0 || chunk_size <= 0)
    return -1;
  return total_workspace(batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size);
}

extern "C" int qb_ssd_chunk_scan_fwd(const qb_ssd_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "ssd: null args");
  QB_REQUIRE(a->x && a->dt && a->Bm && a->Cm && a->A_log && a->out && a->final_states, QB_ERR_INVALID_ARG,
             "ssd: null tensor pointer");
  QB_REQUIRE(a->x_scales && a->dt_scale && a->A_scale && a->B_scale && a->C_scale && a->ssm_state_scale,
             QB_ERR_INVALID_ARG, "ssd: null scale pointer");
  QB_REQUIRE(a->D == nullptr || a->D_scale != nullptr, QB_ERR_INVALID_ARG, "ssd: D without D_scale");
  QB_REQUIRE(a->z == nullptr || a->z_scale != nullptr, QB_ERR_INVALID_ARG, "ssd: z without z_scale");
  QB_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->ngroups > 0, QB_ERR_INVALID_ARG, "ssd: empty shape");
  QB_REQUIRE(a->nheads % a->ngroups == 0, QB_ERR_INVALID_ARG, "ssd: nheads must be divisible by ngroups");
  QB_REQUIRE(a->headdim % TN == 0 && a->dstate % TN == 0 && a->chunk_size % TM == 0 && a->chunk_size <= 1024,
             QB_ERR_UNSUPPORTED, "ssd: headdim, dstate and chunk_size must be multiples of 64 (chunk <= 1024)");
  QB_REQUIRE(!a->grouped || (a->head_group_range && a->dim_group_range && a->nhead_groups > 0 && a->ndim_groups > 0),
             QB_ERR_INVALID_ARG, "ssd: grouped scales need the range tables");
  const WsLayout wl = ws_layout(a->batch, a->seqlen, a->nheads, a->headdim, a->ngroups, a->dstate, a->chunk_size);
  const int64_t need = total_workspace(a->batch, a->seqlen, a->nheads, a->headdim, a->ngroups, a->dstate, a->chunk_size);
  QB_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= need && aligned(a->workspace, 256),
             QB_ERR_INVALID_ARG, "ssd: workspace must be 256-byte aligned and hold %lld bytes", (long long)need);
  if (!force_portable() && ssd_tc_eligible(a)) return ssd_tc_launch(a, (cudaStream_t)stream);
  char* base = static_cast<char*>(a->workspace);
  Ws ws;
  ws.dt = reinterpret_cast<float*>(base + wl.off_dt);
  ws.dA = reinterpret_cast<float*>(base + wl.off_dA);
  ws.CB = reinterpret_cast<float*>(base + wl.off_CB);
  ws.states = reinterpret_cast<float*>(base + wl.off_states);
  ws.prev = reinterpret_cast<__half*>(base + wl.off_prev);
  const int Q = a->chunk_size;
  const int nc = (int)ceil_div(a->seqlen, Q);
  cudaStream_t st = (cudaStream_t)stream;
  ssd_cumsum_kernel<<<a->batch * nc, 128, 0, st>>>(*a, ws, nc);
  QB_LAUNCH_OK("ssd_cumsum_kernel");
  {
    dim3 grid((Q / TM) * (Q / TN), a->batch * nc * a->ngroups);
    ssd_cb_kernel<<<grid, kThreads, 0, st>>>(*a, ws, nc);
    QB_LAUNCH_OK("ssd_cb_kernel");
  }
  {
    dim3 grid((a->headdim / TM) * (a->dstate / TN), a->batch * nc * a->nheads);
    ssd_chunk_state_kernel<<<grid, kThreads, 0, st>>>(*a, ws, nc);
    QB_LAUNCH_OK("ssd_chunk_state_kernel");
  }
  {
    dim3 grid((unsigned)ceil_div((int64_t)a->headdim * a->dstate, kThreads), a->nheads, a->batch);
    ssd_state_passing_kernel<<<grid, kThreads, 0, st>>>(*a, ws, nc);
    QB_LAUNCH_OK("ssd_state_passing_kernel");
  }
  {
    dim3 grid((Q / TM) * (a->headdim / TN), a->batch * nc * a->nheads);
    ssd_chunk_scan_kernel<<<grid, kThreads, 0, st>>>(*a, ws, nc);
    QB_LAUNCH_OK("ssd_chunk_scan_kernel");
  }
  return QB_OK;
}

// ---- allocation-free variant -------------------------------------------------------------------
// Some callers of this library cannot hand over scratch memory at all: a host process that owns no
// CUDA allocator of its own (a plain C inference loop, a language binding without device-memory
// management) or a runtime whose memory pool is frozen once the model is loaded has nowhere to get
// the SSD workspace from, because obtaining one would mean calling cudaMalloc.  For them the
// scratch lives in this library's own device image: a fixed-size array that every GPU loading the
// library holds until the process exits.
namespace qb {
namespace {

constexpr int64_t kStaticScratchBytes = 48ll << 20;  // 48 MiB: one Mamba2-2.7B layer, batch 1, 2048 tokens
static __device__ __align__(256) unsigned char g_ssd_static_scratch[kStaticScratchBytes];

// In host code `g_ssd_static_scratch` is only a host-side handle; the address a kernel can use has
// to be asked for, once per device, with that device current.
// The per-device cache is written without a lock: two host threads making their first call on one device may both
// query the address and both store it; they store the same value, so the race is harmless.
int static_scratch_ptr(char** out) {
  static char* cached[64] = {};
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] != nullptr) {
    *out = cached[dev];
    return QB_OK;
  }
  char* p = nullptr;
  QB_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_ssd_static_scratch));
  QB_REQUIRE(p != nullptr, QB_ERR_CUDA, "ssd: the static scratch array has no device address");
  if (dev >= 0 && dev < 64) cached[dev] = p;
  *out = p;
  return QB_OK;
}

}  // namespace
}  // namespace qb

extern "C" int64_t qb_ssd_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int qb_ssd_chunk_scan_fwd_noalloc(const qb_ssd_args* a, void* stream) {
  QB_REQUIRE(a != nullptr, QB_ERR_INVALID_ARG, "ssd: null args");
  QB_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->ngroups > 0 && a->dstate > 0 &&
                 a->chunk_size > 0,
             QB_ERR_INVALID_ARG, "ssd: empty shape");
  const int64_t need =
      total_workspace(a->batch, a->seqlen, a->nheads, a->headdim, a->ngroups, a->dstate, a->chunk_size);
  QB_REQUIRE(need <= kStaticScratchBytes, QB_ERR_TOO_LARGE,
             "ssd (no-alloc): this shape needs %lld bytes of scratch, the built-in array holds %lld; "
             "use qb_ssd_chunk_scan_fwd with a caller-provided workspace",
             (long long)need, (long long)kStaticScratchBytes);
  char* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);
  if (rc != QB_OK) return rc;
  qb_ssd_args b = *a;
  b.workspace = scratch;
  b.workspace_bytes = kStaticScratchBytes;
  // Every stage fully rewrites the part of the scratch it later reads, so nothing has to be cleared
  // between calls even though the array keeps the previous call's contents.
  return qb_ssd_chunk_scan_fwd(&b, stream);
}
