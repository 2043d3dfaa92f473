"""CPU restatement of the quantised RMSNorm kernels (test infrastructure only).

Follows quamba/triton/quant_norm.py:68-132 (``_qlayer_norm_fwd_1pass_kernel``: residual add, RMS / layer
norm, static or per-token int8 output) and quamba/triton/quant_normgated.py:11-83 (grouped norm with an
int8 gate, fp16 or int8 output).  Pinned: tests/golden/norm_*.npz hold the outputs of those two Triton
kernels executed in Triton interpreter mode (tests/golden/make_norm_golden.py), with libdevice.rint
replaced by an equivalent round-half-to-even.
"""
import torch


def _next_pow2(n):
    return 1 << (n - 1).bit_length()


def _quant(y, static_out_scale, n):
    """int8 = clamp(rint(y / scale)); scale static, or max(y) / 127 per row where the maximum also covers the
    zero padding of the power-of-two block (quant_norm.py:123-129)."""
    if static_out_scale is not None:
        scale = torch.tensor(static_out_scale, dtype=torch.float32)
        return torch.clamp(torch.round(y / scale), -128, 127).to(torch.int8), None
    mx = y.amax(dim=-1)
    if _next_pow2(n) != n:
        mx = mx.clamp(min=0.0)
    scale = mx / 127.0
    return torch.clamp(torch.round(y / scale[..., None]), -128, 127).to(torch.int8), scale


def qlayer_norm_fwd(x, weight, bias, eps, residual=None, static_out_scale=None, residual_dtype=None, is_rms_norm=True):
    """quant_norm.py:134-206.  x (M, N) fp16; returns (y int8, residual_out, per_token_scale or None)."""
    M, N = x.shape
    h = x.float()
    if residual is not None:
        residual_dtype = residual.dtype
        h = h + residual.float()
    store = residual is not None or (residual_dtype is not None and residual_dtype != x.dtype)
    residual_out = h.to(residual_dtype if residual_dtype is not None else x.dtype) if store else x
    if is_rms_norm:
        mean = 0.0
        var = (h * h).sum(-1, keepdim=True) / N
    else:
        mean = h.sum(-1, keepdim=True) / N
        var = ((h - mean) ** 2).sum(-1, keepdim=True) / N
    rstd = 1.0 / torch.sqrt(var + eps)
    y = (h - mean) * rstd * weight.float()
    if bias is not None:
        y = y + bias.float()
    q, scale = _quant(y, static_out_scale, N)
    return q, residual_out, scale


def qlayer_normgated_fwd(x, weight, bias, eps, q_z=None, z_scale=None, static_out_scale=None, use_float16_output=False,
                         group_size=None, norm_before_gate=True, is_rms_norm=True):
    """quant_normgated.py:85-132.  x (M, N) fp16, q_z (M, N) int8; returns (out, per_token_scale (ngroups * M) or None)."""
    M, N = x.shape
    group_size = group_size or N
    G = N // group_size
    h = x.float().reshape(M, G, group_size)
    gate = None
    if q_z is not None:
        z = q_z.float().reshape(M, G, group_size) * z_scale
        gate = z * torch.sigmoid(z)
        if not norm_before_gate:
            h = h * gate
    if is_rms_norm:
        mean = 0.0
        var = (h * h).sum(-1, keepdim=True) / group_size
    else:
        mean = h.sum(-1, keepdim=True) / group_size
        var = ((h - mean) ** 2).sum(-1, keepdim=True) / group_size
    rstd = 1.0 / torch.sqrt(var + eps)
    y = (h - mean) * rstd * weight.float().reshape(G, group_size)
    if bias is not None:
        y = y + bias.float().reshape(G, group_size)
    if gate is not None and norm_before_gate:
        y = y * gate
    if use_float16_output:
        return y.reshape(M, N).to(torch.float16), None
    q, scale = _quant(y, static_out_scale, group_size)
    if scale is not None:
        scale = scale.t().contiguous().reshape(-1)       # stored as [group * M + row]
    return q.reshape(M, N), scale
