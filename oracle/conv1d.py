"""CPU restatement of the int8 causal conv1d kernels (test infrastructure only).

Parity unpinned: the reference implements these only as CUDA kernels; this file
follows their arithmetic line by line and is checked for self-consistency
(fwd == repeated update; closed-form cases).

Follows
  csrc/causal_conv1d/quant_causal_conv1d_fwd_kernel.cuh:57-158   (Quamba1 fwd)
  csrc/causal_conv1d/quant_causal_conv1d_update_kernel.cuh:34-75 (Quamba1 update)
  csrc/causal_conv1d/quamba2_conv1d_fwd_kernel.cuh:163-271       (Quamba2 fwd)
  csrc/causal_conv1d/quamba2_conv1d_update_kernel.cuh:62-146     (Quamba2 update)
"""
import torch
import torch.nn.functional as F

from .quant import to_int8_rhaz, expand_x_scales


def _silu(v):
    # out / (1 + expf(-out)), quant_causal_conv1d_fwd_kernel.cuh:141
    return v / (1.0 + torch.exp(-v))


def _int_conv(q_x, q_w):
    """Exact integer depthwise causal conv. q_x int8 (B, C, L), q_w int8 (C, W) -> fp32 (B, C, L).
    Sum over w of w[c, w] * x[c, l - (W-1-w)] with zero left padding."""
    B, C, L = q_x.shape
    W = q_w.shape[1]
    x = F.pad(q_x.float(), (W - 1, 0))
    out = torch.zeros(B, C, L, dtype=torch.float32)
    for w in range(W):
        out += q_w[:, w].float()[None, :, None] * x[:, :, w:w + L]
    return out


def quant_causal_conv1d_fwd(q_x, scale_x, q_w, scale_w, scale_out, scale_b, q_bias=None, silu=True):
    """Quamba1 conv: q_x int8 (B, D, L) (any strides), returns int8 (B, D, L).
    out = scale_w*scale_x*acc + scale_b*bias ; silu ; roundf(out/scale_out) clamp."""
    acc = _int_conv(q_x, q_w)
    scale_wx = torch.tensor(scale_w, dtype=torch.float32) * torch.tensor(scale_x, dtype=torch.float32)
    out = scale_wx * acc
    if q_bias is not None:
        out = out + (q_bias.float() * torch.tensor(scale_b, dtype=torch.float32))[None, :, None]
    if silu:
        out = _silu(out)
    return to_int8_rhaz(out / torch.tensor(scale_out, dtype=torch.float32))


def quant_causal_conv1d_update(q_x, conv_state, scale_x, q_w, scale_w, scale_out, scale_b, q_bias=None, silu=True):
    """Quamba1 decode step. q_x int8 (B, D); conv_state int8 (B, D, W) shifted in place.
    Returns int8 (B, D)."""
    W = q_w.shape[1]
    conv_state[:, :, :-1] = conv_state[:, :, 1:].clone()
    conv_state[:, :, -1] = q_x
    acc = (conv_state.float() * q_w.float()[None]).sum(-1)
    out = torch.tensor(scale_w, dtype=torch.float32) * torch.tensor(scale_x, dtype=torch.float32) * acc
    if q_bias is not None:
        out = out + q_bias.float()[None] * torch.tensor(scale_b, dtype=torch.float32)
    if silu:
        out = _silu(out)
    return to_int8_rhaz(out / torch.tensor(scale_out, dtype=torch.float32))


def _segment_tables(x_dim, headdim, d_state, n_groups, sx, sB, sC, swx, swB, swC, sbx, sbB, sbC,
                    x_scales, B_scales, C_scales, head_group_range, dim_group_range):
    """Per-channel (scale_in, scale_bias, scale_out) of the concatenated [x | B | C] tensor."""
    gn = d_state * n_groups
    f = lambda v: torch.tensor(v, dtype=torch.float32)
    scale_in = torch.cat([(f(swx) * f(sx)).expand(x_dim), (f(swB) * f(sB)).expand(gn), (f(swC) * f(sC)).expand(gn)])
    scale_bias = torch.cat([f(sbx).expand(x_dim), f(sbB).expand(gn), f(sbC).expand(gn)])
    nheads = x_dim // headdim
    xs = expand_x_scales(x_scales, head_group_range, dim_group_range, nheads, headdim, n_groups).reshape(-1)
    if head_group_range is None:
        Bs = B_scales.float().reshape(-1)[0].expand(gn)
        Cs = C_scales.float().reshape(-1)[0].expand(gn)
    else:
        Bs = B_scales.float().reshape(-1).repeat_interleave(d_state)
        Cs = C_scales.float().reshape(-1).repeat_interleave(d_state)
    scale_out = torch.cat([xs, Bs, Cs])
    return scale_in, scale_bias, scale_out


def quamba2_conv1d_fwd(q_xBC, sx, sB, sC, x_dim, headdim, d_state, n_groups,
                       head_group_range, dim_group_range, x_scales, B_scales, C_scales,
                       q_w, swx, swB, swC, q_bias, sbx, sbB, sbC, silu=True):
    """Quamba2 conv on q_xBC int8 (B, C_conv, L).  Returns (x (B,x_dim,L), B (B,GN,L), C (B,GN,L)) int8.
    out = scale_in*acc + scale_bias*bias (fwd_kernel.cuh:232-240), silu, roundf(out/scale_out)."""
    gn = d_state * n_groups
    scale_in, scale_bias, scale_out = _segment_tables(
        x_dim, headdim, d_state, n_groups, sx, sB, sC, swx, swB, swC, sbx, sbB, sbC,
        x_scales, B_scales, C_scales, head_group_range, dim_group_range)
    acc = _int_conv(q_xBC, q_w)
    out = scale_in[None, :, None] * acc
    if q_bias is not None:
        out = out + (scale_bias * q_bias.float())[None, :, None]
    if silu:
        out = _silu(out)
    q = to_int8_rhaz(out / scale_out[None, :, None])
    return q[:, :x_dim], q[:, x_dim:x_dim + gn], q[:, x_dim + gn:]


def quamba2_conv1d_update(q_xBC, conv_state, sx, sB, sC, x_dim, headdim, d_state, n_groups,
                          head_group_range, dim_group_range, x_scales, B_scales, C_scales,
                          q_w, swx, swB, swC, q_bias, sbx, sbB, sbC, silu=True):
    """Quamba2 decode step. q_xBC int8 (B, C_conv); conv_state int8 (B, C_conv, W) updated in place.
    out = scale_bias*bias + sum_w scale_in*w*x (update_kernel.cuh:138-141)."""
    gn = d_state * n_groups
    scale_in, scale_bias, scale_out = _segment_tables(
        x_dim, headdim, d_state, n_groups, sx, sB, sC, swx, swB, swC, sbx, sbB, sbC,
        x_scales, B_scales, C_scales, head_group_range, dim_group_range)
    conv_state[:, :, :-1] = conv_state[:, :, 1:].clone()
    conv_state[:, :, -1] = q_xBC
    acc = (conv_state.float() * q_w.float()[None]).sum(-1)
    out = scale_in[None] * acc
    if q_bias is not None:
        out = out + (scale_bias * q_bias.float())[None]
    if silu:
        out = _silu(out)
    q = to_int8_rhaz(out / scale_out[None])
    return q[:, :x_dim], q[:, x_dim:x_dim + gn], q[:, x_dim + gn:]
