"""CPU restatement of the W4A8 / W8A8 linears (test infrastructure only).

Pinned: the packed-int4 layout, the permuted scale layouts and the dequantised
reference weights are checked against the reference's own packer
(quamba/marlin_utils.py imported on CPU; fixtures in tests/golden made by
tests/golden/make_linear_golden.py).  Integer accumulators are exact.

Follows
  quamba/marlin_utils.py:33-133, :139-279                    packed format (restated as an inverse)
  csrc/linear/marlin_qqq_gemm_kernel.cuh:127-178, :541-567   int4 -> int8 dequantisation
  csrc/linear/marlin_qqq_gemm_kernel.cuh:743-749             fp16 epilogue  acc * s_ch * s_tok
  csrc/linear/marlin_qqq_gemm_kernel_o8.cuh:107-116          int8 epilogue (cvt.rni, saturating)
  csrc/linear/quant_linear_fwd_kernel.cuh:83-109             W8A8 epilogue a_s * (b_s * acc)
  csrc/linear/quant_linear_fwd_gemv_kernel.cuh:27-61         per-column-scale GEMV, roundf + clamp
"""
import numpy as np
import torch

from .quant import round_half_away

TILE = 16


def weight_perm(per_channel: bool) -> np.ndarray:
    """The 1024-entry permutation applied to each row of the (K/16, N*16) tile-major matrix
    before nibble packing (quamba/marlin_utils.py:75-105)."""
    perm = []
    for i in range(32):
        col = i // 4
        one = [16 * row + col + 8 * block for block in (0, 1) for row in range(4 * (i % 4), 4 * (i % 4) + 4)]
        for j in range(4):
            perm.extend(p + 256 * j for p in one)
    perm = np.array(perm)
    inter = np.array([4, 0, 5, 1, 6, 2, 7, 3] if per_channel else [0, 2, 4, 6, 1, 3, 5, 7])
    return perm.reshape(-1, 8)[:, inter].ravel()


def scale_perms():
    """(group-scale perm of 64, channel-scale perm of 32), quamba/marlin_utils.py:108-117."""
    sp = [i + 8 * j for i in range(8) for j in range(8)]
    sps = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]
    return np.array(sp), np.array(sps)


def unpack_weight(packed: torch.Tensor, size_k: int, size_n: int, per_channel: bool) -> torch.Tensor:
    """packed int32 (K/16, N*16/8) -> nibbles (K, N): 0..15 (per-group) or signed -8..7 (per-channel)."""
    p = packed.cpu().numpy().astype(np.uint32)
    rows = size_k // TILE
    nib = np.zeros((rows, size_n * TILE), dtype=np.int64)
    for i in range(8):
        nib[:, i::8] = (p >> (4 * i)) & 0xF
    perm = weight_perm(per_channel)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(perm.size)
    nib = nib.reshape(-1, perm.size)[:, inv].reshape(rows, size_n * TILE)
    q = nib.reshape(rows, size_n // TILE, TILE, TILE).transpose(0, 2, 1, 3).reshape(size_k, size_n)
    if per_channel:
        q = np.where(q >= 8, q - 16, q)
    return torch.from_numpy(q.astype(np.int64))


def unpermute_scales(s_group: torch.Tensor, s_channel: torch.Tensor, size_n: int, per_channel: bool):
    """Undo w4a8_permute_scales (quamba/marlin_utils.py:120-133).  Returns natural-order
    (s_group fp16 (K/g, N) or None, s_channel fp32 (N,))."""
    sp, sps = scale_perms()
    inv_sps = np.empty_like(sps)
    inv_sps[sps] = np.arange(sps.size)
    sc = s_channel.reshape(-1, sps.size)[:, torch.from_numpy(inv_sps)].reshape(size_n)
    if per_channel or s_group is None or s_group.numel() == 0:
        return None, sc
    inv_sp = np.empty_like(sp)
    inv_sp[sp] = np.arange(sp.size)
    sg = s_group.reshape(-1, sp.size)[:, torch.from_numpy(inv_sp)].reshape(-1, size_n)
    return sg, sc


def dequant_to_int8(q: torch.Tensor, s_group_nat, group_size: int) -> torch.Tensor:
    """The int8 weights the GEMM multiplies with.
    per-group  : fp16 fma((q-8), s_group, 1152) -> low mantissa byte ^ 0x80, i.e. the product rounded
                 half-to-even to an integer, wrapped to 8 bits (marlin_qqq_gemm_kernel.cuh:136-178);
    per-channel: the signed nibble placed in the high half of the byte = 16 * q (:127-132)."""
    if s_group_nat is None:
        return (q * 16).to(torch.int64)
    K, N = q.shape
    sg = s_group_nat.to(torch.float16).double().repeat_interleave(group_size, dim=0)   # (K, N)
    prod = (q - 8).double() * sg                                                          # exact
    r = torch.round(prod)                                                                 # half to even
    return ((r.to(torch.int64) + 128) % 256) - 128


def int_matmul(a_int8: torch.Tensor, w_int: torch.Tensor) -> torch.Tensor:
    """Exact integer GEMM (M,K) x (K,N) -> int64 via fp64 BLAS (|acc| << 2^53)."""
    return torch.round(a_int8.double() @ w_int.double()).to(torch.int64)


def _f32(v):
    return torch.as_tensor(v, dtype=torch.float32)


def cvt_rni_sat_s8(x: torch.Tensor) -> torch.Tensor:
    return torch.clamp(torch.round(x), -128, 127).to(torch.int8)


def w4a8_gemm(a_int8, packed, s_tok, s_channel, s_group, size_n, size_k, out_int8: bool,
              output_transpose: bool = False, return_acc: bool = False):
    """quant_linear_cuda.w4a8o16_gemm / w4a8o8_gemm on the packed buffers exactly as the module
    stores them.  s_tok: 1 element (per tensor) or M elements (per row)."""
    per_channel = s_group is None or s_group.numel() == 0
    q = unpack_weight(packed, size_k, size_n, per_channel)
    sg, sc = unpermute_scales(s_group, s_channel.float(), size_n, per_channel)
    group = size_k if per_channel else size_k // sg.shape[0]
    w8 = dequant_to_int8(q, sg, group)
    acc = int_matmul(a_int8, w8)
    st = _f32(s_tok).reshape(-1)
    st = st.reshape(-1, 1) if st.numel() > 1 else st.reshape(1, 1)
    res = (acc.float() * sc.float()[None, :]) * st                # fp32, same operation order
    out = cvt_rni_sat_s8(res) if out_int8 else res.to(torch.float16)
    if output_transpose:
        out = out.t().contiguous()
    return (out, acc) if return_acc else out


def w8a8_gemm(a_int8, w_kn_int8, a_scales, b_scales, out_dtype, return_acc: bool = False):
    """quant_linear_cuda.cutlass_scaled_mm_dq: D = cvt(a_s * (b_s * float(acc))).
    a (M,K) int8; w (K,N) int8; a_scales 1 or M elements; b_scales 1 or N elements.
    int8 output: round half to even, saturating (the CUTLASS converter's rounding at exact ties is
    third-party code that is absent here: parity unpinned at ties)."""
    acc = int_matmul(a_int8, w_kn_int8.to(torch.int64))
    As = _f32(a_scales).reshape(-1)
    Bs = _f32(b_scales).reshape(-1)
    As = As.reshape(-1, 1) if As.numel() > 1 else As.reshape(1, 1)
    Bs = Bs.reshape(1, -1) if Bs.numel() > 1 else Bs.reshape(1, 1)
    res = As * (Bs * acc.float())
    out = cvt_rni_sat_s8(res) if out_dtype == torch.int8 else res.to(out_dtype)
    return (out, acc) if return_acc else out


def w8a8_gemv_alpha(w_nk_int8, x_1k_int8, alpha, out_dtype):
    """quant_linear_cuda.cutlass_scaled_mv_dq(c, W(n,k), x(1,k), alpha, beta=0): alpha * acc."""
    acc = int_matmul(x_1k_int8, w_nk_int8.t().to(torch.int64))
    res = _f32(alpha) * acc.float()
    return cvt_rni_sat_s8(res) if out_dtype == torch.int8 else res.to(out_dtype)


def w8a8o8_gemv(w_nk_int8, x_1k_int8, scale_w_n, scale_x):
    """quant_linear_cuda.w8a8o8_gemv: int8(clamp(roundf(s_w[n] * s_x * acc)))."""
    acc = int_matmul(x_1k_int8, w_nk_int8.t().to(torch.int64))
    scale = _f32(scale_w_n).reshape(1, -1) * _f32(scale_x).reshape(-1)[0]
    return torch.clamp(round_half_away(scale * acc.float()), -128, 127).to(torch.int8)
