// Epilogue shared by every integer GEMM kernel: int32 accumulator -> scaled fp32 -> output type.
//   r = (float(acc) * col_scale[n]) * row_scale[m]        (W4A8: acc * s_channel * s_tok;
//                                                          W8A8: a_scale * (b_scale * acc))
//   or r = alpha * float(acc) when use_alpha (the GEMV form with host scalars).
#pragma once
#include "common.cuh"

namespace qb {

enum OutKind { kOutS8Rne = 0, kOutF16 = 1, kOutBF16 = 2, kOutS8Away = 3 };

struct Epilogue {
  const float* row_scale;  // 1 element, or M when row_per
  const float* col_scale;  // 1 element, or N when col_per
  void* out;
  int64_t out_stride;  // elements between rows of out ((N, M) rows when transpose)
  float alpha;
  int row_per, col_per, use_alpha, out_kind, transpose;

#ifdef __CUDACC__
  __device__ __forceinline__ float scaled(int acc, int m, int n) const {
    const float f = (float)acc;
    if (use_alpha) return alpha * f;
    const float cs = col_scale[col_per ? n : 0];
    // (per-row scales come from the kernel that quantised the rows, through a cached load: that kernel therefore never
    // lets its successor start early, see run_norm)
    const float rs = row_scale[row_per ? m : 0];
    return (f * cs) * rs;
  }
  __device__ __forceinline__ int to_s8(float r) const {
    return out_kind == kOutS8Away ? round_away_s8(r) : rint_s8(r);
  }
  __device__ __forceinline__ void store(int acc, int m, int n) const {
    const float r = scaled(acc, m, n);
    const int64_t idx = transpose ? (int64_t)n * out_stride + m : (int64_t)m * out_stride + n;
    switch (out_kind) {
      case kOutF16: static_cast<__half*>(out)[idx] = __float2half_rn(r); break;
      case kOutBF16: static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(r); break;
      default: static_cast<int8_t*>(out)[idx] = (int8_t)to_s8(r); break;
    }
  }
#endif
};

}  // namespace qb
