"""Quantisation helpers shared by the oracle modules (test infrastructure only).

Follows quamba/quant_utils.py:16-27 (per-tensor absmax) and the rounding modes
used at each requantisation site of the reference kernels.
"""
import torch


def quantize_per_tensor_absmax(w: torch.Tensor, n_bits: int = 8, clip_ratio: float = 1.0):
    """quamba/quant_utils.py:16-27: scale = max|w| (>=1e-5) / qmax, round half to
    even (torch.round), clamp to [qmin, qmax].  Returns (int8 tensor, fp32 0-d scale)."""
    q_max = 2 ** (n_bits - 1) - 1
    q_min = -2 ** (n_bits - 1)
    w = w.float()
    w_max = w.abs().amax().clamp(min=1e-5)
    if clip_ratio < 1.0:
        w_max = w_max * clip_ratio
    scale = (w_max / q_max).float()
    q = torch.clamp(torch.round(w / scale), q_min, q_max).to(torch.int8)
    return q, scale


def round_half_away(x: torch.Tensor) -> torch.Tensor:
    """C ``roundf``: halves round away from zero (conv, Mamba1 scan state, Hadamard)."""
    return torch.sign(x) * torch.floor(torch.abs(x) + 0.5)


def to_int8_rhaz(x: torch.Tensor) -> torch.Tensor:
    """clamp(int(roundf(x)), -128, 127) as at quant_causal_conv1d_fwd_kernel.cuh:149-150."""
    return torch.clamp(round_half_away(x), -128, 127).to(torch.int8)


def to_int8_rne(x: torch.Tensor) -> torch.Tensor:
    """clamp(rint(x), -128, 127): round half to even (Triton kernels, cvt.rni)."""
    return torch.clamp(torch.round(x), -128, 127).to(torch.int8)


def softplus_ref(x: torch.Tensor) -> torch.Tensor:
    """x <= 20 ? log1p(exp(x)) : x, as at quant_sscan_fwd_kernel.cuh:159-161."""
    return torch.where(x <= 20.0, torch.log1p(torch.exp(torch.clamp(x, max=20.0))), x)


def inv_softplus(dt: torch.Tensor) -> torch.Tensor:
    """dt + log(-expm1(-dt)): the bias initialisation used by the Mamba mixers."""
    return dt + torch.log(-torch.expm1(-dt))


def group_index_tables(head_group_range, dim_group_range, nheads_per_group, headdim):
    """Expand the cumulative range tables of the grouped ("group_heads") scheme.

    head_group_range: int32 [G, HG] cumulative head ends inside one SSD group.
    dim_group_range:  int32 [G, HG, DG] cumulative channel ends inside a head.
    Returns (hg_idx [G, heads_per_group], dg_idx [G, heads_per_group, headdim]) as
    long tensors -- the same lookup the kernels do with ``sum(idx >= range)``
    (quamba/triton/quant_chunk_state.py:202-214)."""
    G, HG = head_group_range.shape
    DG = dim_group_range.shape[2]
    heads = torch.arange(nheads_per_group)
    dims = torch.arange(headdim)
    hg_idx = (heads[None, :, None] >= head_group_range[:, None, :].long()).sum(-1)      # [G, hpg]
    hg_idx = hg_idx.clamp(max=HG - 1)
    dgr = torch.gather(dim_group_range.long(), 1, hg_idx[:, :, None].expand(G, nheads_per_group, DG))
    dg_idx = (dims[None, None, :, None] >= dgr[:, :, None, :]).sum(-1).clamp(max=DG - 1)  # [G, hpg, P]
    return hg_idx, dg_idx


def expand_x_scales(x_scales, head_group_range, dim_group_range, nheads, headdim, ngroups):
    """Per-channel fp32 scale [nheads, headdim] from x_scales [G, HG, DG] (or 1-element)."""
    x_scales = x_scales.float()
    if head_group_range is None:
        return x_scales.reshape(-1)[0].expand(nheads, headdim).clone()
    hpg = nheads // ngroups
    hg_idx, dg_idx = group_index_tables(head_group_range, dim_group_range, hpg, headdim)
    g = torch.arange(ngroups)[:, None, None].expand(ngroups, hpg, headdim)
    out = x_scales[g, hg_idx[:, :, None].expand_as(g), dg_idx]
    return out.reshape(nheads, headdim).contiguous()


def expand_state_scales(state_scale, head_group_range, dim_group_range, nheads, headdim, ngroups, dstate):
    """Per-element fp32 scale [nheads, headdim, dstate] from [G, HG, DG, N] (or 1-element)."""
    state_scale = state_scale.float()
    if head_group_range is None:
        return state_scale.reshape(-1)[0].expand(nheads, headdim, dstate).clone()
    hpg = nheads // ngroups
    hg_idx, dg_idx = group_index_tables(head_group_range, dim_group_range, hpg, headdim)
    g = torch.arange(ngroups)[:, None, None].expand(ngroups, hpg, headdim)
    out = state_scale[g, hg_idx[:, :, None].expand_as(g), dg_idx]          # [G, hpg, P, N]
    return out.reshape(nheads, headdim, dstate).contiguous()
