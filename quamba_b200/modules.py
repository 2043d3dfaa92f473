"""Module-level mirror of the reference's quantized mixer layers.

Each class keeps the reference's name, constructor arguments, buffer names / shapes / dtypes and the extra
float entries its state-dict hooks add, so a checkpoint written by the reference loads here and vice versa:

  QCausalConv1D, Quamb2Conv1D      quamba/qConvLayer.py:11-131, 134-340
  QSScan                           quamba/qSelectiveScan.py:76-203
  Quamba2ChunkScan                 quamba/qChunkScan.py:17-246
  QHadamard                        quamba/qHadamard.py:8-38
  W4A8B16O16Linear, W4A8B8O8Linear, W4A8B8O8LinearParallel,
  W8A8B8O8Linear, W8A8B8O8LinearParallel, W8A8B16O16Linear
                                   quamba/qLinearLayer.py:139-823

``forward`` / ``update`` / ``to_seqlen_last`` run the CUDA entry points in :mod:`quamba_b200.ops`; there is no
CPU execution path.  Construction, ``from_fp16`` and state-dict round trips work without a GPU (buffers are
then created on the CPU), which is what the host-side tests use.
"""
import math
from functools import partial

import torch
import torch.nn as nn

from . import ops
from .packing import w4a8_quantize

__all__ = ["QCausalConv1D", "Quamb2Conv1D", "QSScan", "Quamba2ChunkScan", "QHadamard", "W4A8B16O16Linear",
           "W4A8B8O8Linear", "W4A8B8O8LinearParallel", "W8A8B8O8Linear", "W8A8B8O8LinearParallel",
           "W8A8B16O16Linear", "quantize_tensor_per_tensor_absmax"]


def _dev(device=None):
    if device is not None:
        return torch.device(device)
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


@torch.no_grad()
def quantize_tensor_per_tensor_absmax(w, n_bits=8, clip_ratio=1.0):
    """Symmetric per-tensor quantisation: returns (rounded values as float, fp32 scale tensor)
    (quamba/quant_utils.py:16-28)."""
    q_max = 2 ** (n_bits - 1) - 1
    w_max = w.abs().amax().clamp(min=1e-5)
    if clip_ratio < 1.0:
        w_max = w_max * clip_ratio
    scale = w_max / q_max
    return torch.clamp(torch.round(w / scale), -q_max - 1, q_max), scale.float()


def _as_float(v):
    return v.item() if torch.is_tensor(v) else v


class _FloatStateMixin:
    """Python-float attributes that travel in the state dict next to the buffers."""
    _float_state = ()

    def _install_float_state(self):
        self._register_state_dict_hook(self._store_floats)
        self._register_load_state_dict_pre_hook(self._load_floats)

    def _float_names(self):
        return self._float_state

    @staticmethod
    def _store_floats(module, state_dict, prefix, local_metadata):
        for name in module._float_names():
            state_dict[prefix + name] = getattr(module, name)
        return state_dict

    def _load_floats(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        for name in self._float_names():
            setattr(self, name, state_dict.pop(prefix + name))


# ------------------------------------------------------------------------------------------------ conv1d

def _check_depthwise(in_channels, out_channels, groups, kernel_size):
    assert in_channels == out_channels == groups, "only depthwise convolution (in == out == groups) is supported"
    if isinstance(kernel_size, tuple):
        assert len(kernel_size) == 1, "only a 1-D kernel_size is supported"
        kernel_size = kernel_size[0]
    return kernel_size


class QCausalConv1D(_FloatStateMixin, nn.Module):
    """int8 depthwise causal conv1d + SiLU with one scale per tensor (Quamba1)."""
    _float_state = ("weight_scale", "bias_scale", "input_scale", "output_scale")

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 device=None, **kwargs):
        super().__init__()
        kernel_size = _check_depthwise(in_channels, out_channels, groups, kernel_size)
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, kernel_size
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups
        dev = _dev(device)
        self.register_buffer("weight", torch.empty((in_channels, kernel_size), dtype=torch.int8, device=dev))
        if bias is not None:
            self.register_buffer("bias", torch.empty((in_channels,), dtype=torch.int8, device=dev))
        else:
            self.bias = None
        self.weight_scale = self.bias_scale = self.input_scale = self.output_scale = 0.0
        self._install_float_state()

    @classmethod
    def from_fp16(cls, originalLayer: nn.Conv1d, input_scale=1.0, output_scale=1.0):
        dev = originalLayer.weight.device
        q = cls(originalLayer.in_channels, originalLayer.out_channels, originalLayer.kernel_size, originalLayer.stride,
                originalLayer.padding, originalLayer.dilation, originalLayer.groups, originalLayer.bias, device=dev)
        q.input_scale, q.output_scale = _as_float(input_scale), _as_float(output_scale)
        w8, ws = quantize_tensor_per_tensor_absmax(originalLayer.weight.detach().clone(), 8)
        q.weight = w8.to(torch.int8).squeeze(1).contiguous().to(dev)
        q.weight_scale = ws.item()
        if originalLayer.bias is not None:
            b8, bs = quantize_tensor_per_tensor_absmax(originalLayer.bias.detach().clone(), 8)
            q.bias = b8.to(torch.int8).contiguous().to(dev)
            q.bias_scale = bs.item()
        else:
            q.bias, q.bias_scale = None, 1.0
        return q

    @torch.no_grad()
    def forward(self, x):
        return ops.quant_causal_conv1d_cuda.fwd(x, self.input_scale, self.weight, self.weight_scale, self.output_scale,
                                                self.bias_scale, self.bias, None, None, None, True)

    @torch.no_grad()
    def update(self, x, conv_state):
        """One decode step; conv_state is shifted in place."""
        return ops.quant_causal_conv1d_cuda.update(x, conv_state, self.input_scale, self.weight, self.weight_scale,
                                                   self.output_scale, self.bias_scale, self.bias, True)

    def __repr__(self):
        return (f"QCausalConv1D({self.out_channels}, {self.in_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride})")


class Quamb2Conv1D(_FloatStateMixin, nn.Module):
    """int8 depthwise causal conv1d + SiLU over the concatenated [x | B | C] channels with separate input,
    weight and bias scales per segment, grouped output scales for x and per-ssd-group scales for B, C."""

    def __init__(self, x_dim, x_headdim, d_state, n_groups, x_nhead_group, x_ndim_group, in_channels, out_channels,
                 kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True, device=None, **kwargs):
        super().__init__()
        self.x_dim, self.x_headdim, self.d_state, self.n_groups = x_dim, x_headdim, d_state, n_groups
        self.x_nhead_group, self.x_ndim_group = x_nhead_group, x_ndim_group
        kernel_size = _check_depthwise(in_channels, out_channels, groups, kernel_size)
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, kernel_size
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups
        self.x_scale = self.B_scale = self.C_scale = 0.0
        self.wx_scale = self.wB_scale = self.wC_scale = 0.0
        dev = _dev(device)
        self.register_buffer("weight", torch.empty((in_channels, kernel_size), dtype=torch.int8, device=dev))
        if bias is not None:
            self.register_buffer("bias", torch.empty((in_channels,), dtype=torch.int8, device=dev))
            self.bx_scale = self.bB_scale = self.bC_scale = 0.0
        else:
            self.bias = None
            self.bx_scale = self.bB_scale = self.bC_scale = None
        self._install_float_state()
        if x_nhead_group > 0 and x_ndim_group > 0:
            self.register_buffer("x_head_group_range",
                                 torch.empty((n_groups, x_nhead_group), dtype=torch.int32, device=dev))
            self.register_buffer("x_dim_group_range",
                                 torch.empty((n_groups, x_nhead_group, x_ndim_group), dtype=torch.int32, device=dev))
            self.register_buffer("x_out_scales",
                                 torch.empty((n_groups, x_nhead_group, x_ndim_group), dtype=torch.float32, device=dev))
        elif x_nhead_group == 0 and x_ndim_group == 0:
            self.x_head_group_range = self.x_dim_group_range = None
            self.register_buffer("x_out_scales", torch.empty((1,), dtype=torch.float32, device=dev))
        else:
            raise ValueError("x_nhead_group and x_ndim_group must be both zero or both non-zero")
        self.register_buffer("B_out_scales", torch.empty((n_groups,), dtype=torch.float32, device=dev))
        self.register_buffer("C_out_scales", torch.empty((n_groups,), dtype=torch.float32, device=dev))

    def _float_names(self):
        names = ("x_scale", "B_scale", "C_scale", "wx_scale", "wB_scale", "wC_scale")
        return names + (("bx_scale", "bB_scale", "bC_scale") if self.bias is not None else ())

    def _segments(self):
        bc = self.d_state * self.n_groups
        return (self.x_dim, bc, bc)

    @classmethod
    def from_fp16(cls, originalLayer: nn.Conv1d, x_dim, x_headdim, d_state, n_groups, x_scale, B_scale, C_scale,
                  x_out_scales, B_out_scales, C_out_scales, x_head_group_range, x_dim_group_range):
        if (x_head_group_range is None) != (x_dim_group_range is None):
            raise ValueError("x_head_group_range and x_dim_group_range must be both None or both not None")
        if x_head_group_range is not None:
            assert x_head_group_range.dim() == 2, "x_head_group_range must be [n_ssd_group, x_nhead_group]"
            assert x_dim_group_range.dim() == 3, "x_dim_group_range must be [n_ssd_group, x_nhead_group, n_dim_group]"
            nhg, ndg = x_head_group_range.shape[1], x_dim_group_range.shape[2]
        else:
            nhg = ndg = 0
        dev = originalLayer.weight.device
        q = cls(x_dim, x_headdim, d_state, n_groups, nhg, ndg, originalLayer.in_channels, originalLayer.out_channels,
                originalLayer.kernel_size, originalLayer.stride, originalLayer.padding, originalLayer.dilation,
                originalLayer.groups, originalLayer.bias, device=dev)
        q.x_scale, q.B_scale, q.C_scale = _as_float(x_scale), _as_float(B_scale), _as_float(C_scale)
        q.x_head_group_range = None if x_head_group_range is None else x_head_group_range.to(dev)
        q.x_dim_group_range = None if x_dim_group_range is None else x_dim_group_range.to(dev)
        q.x_out_scales, q.B_out_scales, q.C_out_scales = (t.to(dev) for t in (x_out_scales, B_out_scales, C_out_scales))

        def split_quant(t):
            parts, scales, start = [], [], 0
            for n in q._segments():
                p8, s = quantize_tensor_per_tensor_absmax(t[start:start + n].contiguous(), 8)
                parts.append(p8.to(torch.int8))
                scales.append(s.item())
                start += n
            return torch.cat(parts, dim=0).contiguous(), scales

        q.weight, (q.wx_scale, q.wB_scale, q.wC_scale) = split_quant(
            originalLayer.weight.detach().clone().float().squeeze(1))
        if originalLayer.bias is not None:
            q.bias, (q.bx_scale, q.bB_scale, q.bC_scale) = split_quant(originalLayer.bias.detach().clone().float())
        else:
            q.bias = None
            q.bx_scale = q.bB_scale = q.bC_scale = None
        return q

    def _common(self):
        return (self.x_scale, self.B_scale, self.C_scale, self.x_dim, self.x_headdim, self.d_state, self.n_groups,
                self.x_head_group_range, self.x_dim_group_range, self.x_out_scales, self.B_out_scales,
                self.C_out_scales, self.weight, self.wx_scale, self.wB_scale, self.wC_scale, self.bias, self.bx_scale,
                self.bB_scale, self.bC_scale, None, None, None, True)

    @torch.no_grad()
    def forward(self, xBC):
        return ops.quamba2_conv1d_cuda.fwd(xBC, *self._common())

    @torch.no_grad()
    def update(self, xBC, conv_state):
        """One decode step; conv_state is shifted in place."""
        return ops.quamba2_conv1d_cuda.update(xBC, conv_state, *self._common())

    def __repr__(self):
        return (f"Quamb2Conv1D({self.out_channels}, {self.in_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride})")


# ------------------------------------------------------------------------------------------------ Hadamard

def _is_pow2(n):
    return n > 0 and (n & (n - 1)) == 0


def get_qhad_fn(dim):
    """(transform, special order, 1/sqrt(dim)) for a row length (quamba/hadamard_utils.py:33-48)."""
    had_scale = 1.0 / math.sqrt(dim)
    if dim % 12 == 0:
        assert _is_pow2(dim // 12)
        return ops.quant_hadamard.fast_hadamard_transform_12N, 12, had_scale
    if dim % 40 == 0:
        assert _is_pow2(dim // 40)
        return ops.quant_hadamard.fast_hadamard_transform_40N, 40, had_scale
    assert _is_pow2(dim)
    return ops.quant_hadamard.fast_hadamard_transform, 2, had_scale


class QHadamard(_FloatStateMixin, nn.Module):
    """Normalised Hadamard transform of the last dimension fused with int8 quantisation."""
    _float_state = ("x_H_scale",)

    def __init__(self, dim, x_H_scale=1.0, blocks=1):
        """``blocks`` > 1 rotates each of ``blocks`` equal slices of the last dimension on its own (the block-diagonal
        I_blocks (x) H_{dim / blocks}), which is what lets out_proj be cut row-wise across GPUs; 1 is the reference's
        layer."""
        super().__init__()
        assert dim % blocks == 0
        self.dim, self.blocks = dim, blocks
        self.x_H_scale = x_H_scale
        self.transform_fn, self.N, self.had_scale = get_qhad_fn(dim // blocks)
        self._install_float_state()

    @torch.no_grad()
    def forward(self, x):
        scale = self.had_scale / self.x_H_scale
        if self.blocks == 1:
            return self.transform_fn(x, scale)
        shape = x.shape
        return self.transform_fn(x.reshape(-1, self.dim // self.blocks), scale).reshape(shape)

    def __repr__(self):
        return f"QHadamard(dim={self.dim})" if self.blocks == 1 else f"QHadamard(dim={self.dim}, blocks={self.blocks})"


# ------------------------------------------------------------------------------------------------ Mamba1 scan

@torch.no_grad()
def _quant_weight_absmax(w, n_bits=8):
    """(quamba/qSelectiveScan.py:13-19): scale clamp is applied to the max, not to the scale."""
    q_max = 2 ** (n_bits - 1) - 1
    scale = w.abs().max().clamp(min=1e-5) / q_max
    return torch.round(w / scale), scale


def quant_selective_scan_fn(u, scale_u, delta, scale_delta, A, scale_A, B, scale_B, C, scale_C, ssm_state_scale,
                            D=None, scale_D=None, z=None, scale_z=None, delta_bias=None, scale_delta_bias=None,
                            delta_softplus=False, return_last_state=False):
    """int8 selective scan; with return_last_state also the final state (batch, dim, dstate)
    (quamba/qSelectiveScan.py:22-73)."""
    def last_contig(t):
        return t if t is None or t.stride(-1) == 1 else t.contiguous()
    u, delta, B, C, z = map(last_contig, (u, delta, B, C, z))
    if D is not None:
        D = D.contiguous()
    if B.dim() == 3:
        B = B.unsqueeze(1)
    if C.dim() == 3:
        C = C.unsqueeze(1)
    out, x = ops.quant_sscan_cuda.fwd(u, scale_u, delta, scale_delta, A, scale_A, B, scale_B, C, scale_C,
                                      ssm_state_scale, D, scale_D, z, scale_z, delta_bias, scale_delta_bias,
                                      delta_softplus)
    return (out, x[:, :, -1, :]) if return_last_state else out


class QSScan(nn.Module):
    """Mamba1 selective scan with int8 inputs, int8 A_log / D / dt_bias and an int8 state (W8A8B8O8)."""
    _scale_names = ("u_scale", "dt_scale", "B_scale", "C_scale", "z_scale", "ssm_state_scale")

    def __init__(self, d_state, d_inner, delta_softplus=True, device=None):
        super().__init__()
        dev = _dev(device)
        self.delta_softplus = delta_softplus
        one = partial(torch.tensor, 1.0, device=dev, dtype=torch.float32)
        self.register_buffer("dt_bias", torch.empty((d_inner,), device=dev, dtype=torch.int8))
        self.register_buffer("dt_bias_scale", one())
        self.register_buffer("A_log", torch.empty((d_inner, d_state), device=dev, dtype=torch.int8))
        self.register_buffer("A_scale", one())
        self.register_buffer("D", torch.empty((d_inner,), device=dev, dtype=torch.int8))
        self.register_buffer("D_scale", one())
        for name in self._scale_names:
            self.register_buffer(name, one())

    @classmethod
    def from_fp16(cls, d_state, d_inner, A_log, D=None, dt_bias=None, delta_softplus=True, ssm_state_scale=1.0,
                  u_scale=1.0, dt_scale=1.0, B_scale=1.0, C_scale=1.0, z_scale=1.0):
        q = cls(d_state, d_inner, device=A_log.device)

        def f32(v):
            return torch.as_tensor(v, dtype=torch.float32, device=A_log.device)

        a8, a_s = _quant_weight_absmax(A_log.detach().clone())
        q.A_log, q.A_scale = a8.to(torch.int8), a_s.float()
        if D is not None:
            d8, d_s = _quant_weight_absmax(D.detach().clone())
            q.D, q.D_scale = d8.to(torch.int8), d_s.float()
        else:
            q.D = None
        if dt_bias is not None:
            b8, b_s = _quant_weight_absmax(dt_bias.detach().clone())
            q.dt_bias, q.dt_bias_scale = b8.to(torch.int8), b_s.float()
        else:
            q.dt_bias, q.dt_bias_scale = None, f32(0.0)
        q.u_scale, q.dt_scale, q.B_scale, q.C_scale = f32(u_scale), f32(dt_scale), f32(B_scale), f32(C_scale)
        q.z_scale, q.ssm_state_scale = f32(z_scale), f32(ssm_state_scale)
        q.delta_softplus = delta_softplus
        return q

    @torch.no_grad()
    def forward(self, u, dt, B, C, z=None, return_last_state=False):
        """u, dt, z: int8 (batch, d_inner, L); B, C: int8 (batch, d_state, L).  Returns fp16 y when z is given
        (the gate is applied in floating point), else int8-compatible output as the extension defines."""
        has_D, has_b = self.D is not None, self.dt_bias is not None
        return quant_selective_scan_fn(
            u, self.u_scale[None], dt, self.dt_scale[None], self.A_log, self.A_scale[None], B, self.B_scale[None],
            C, self.C_scale[None], ssm_state_scale=self.ssm_state_scale[None],
            D=self.D if has_D else None, scale_D=self.D_scale[None] if has_D else None,
            z=z, scale_z=self.z_scale[None],
            delta_bias=self.dt_bias if has_b else None, scale_delta_bias=self.dt_bias_scale[None] if has_b else None,
            delta_softplus=self.delta_softplus, return_last_state=return_last_state)

    @torch.no_grad()
    def update(self, ssm_state, u, dt, B, C, z=None):
        """One decode step; ssm_state (int8) is updated in place and returned with y."""
        has_D, has_b = self.D is not None, self.dt_bias is not None
        y = ops.quant_sscan_update_triton(
            ssm_state, u, self.u_scale[None], dt, self.dt_scale[None], self.A_log, self.A_scale[None],
            self.ssm_state_scale[None], B, self.B_scale[None], C, self.C_scale[None],
            self.D if has_D else None, self.D_scale[None] if has_D else None,
            z, self.z_scale[None] if z is not None else None,
            self.dt_bias if has_b else None, self.dt_bias_scale[None] if has_b else None, self.delta_softplus)
        return y, ssm_state

    def __repr__(self):
        return "QSScan()"


# ------------------------------------------------------------------------------------------------ Mamba2 SSD

class Quamba2ChunkScan(nn.Module):
    """Mamba2 SSD chunk scan (prefill) and single-token state update (decode) on int8 x / dt / B / C with an
    int8 A_log and D, fp16 dt_bias, and either per-tensor or head/dim-grouped x and state scales."""

    def __init__(self, d_ssm, headdim, d_state, ngroups, D_has_hdim, chunk_size, nhead_groups=0, ndim_groups=0,
                 delta_softplus=True, quant_dt=True, quant_B=True, quant_C=True, quant_z=False,
                 dt_limit=(0.0, float("inf")), device=None, **kwargs):
        super().__init__()
        dev = _dev(device)
        self.d_ssm, self.headdim, self.d_state, self.ngroups = d_ssm, headdim, d_state, ngroups
        self.D_has_hdim, self.chunk_size = D_has_hdim, chunk_size
        self.nhead_groups, self.ndim_groups = nhead_groups, ndim_groups
        self.delta_softplus, self.dt_limit = delta_softplus, dt_limit
        nheads = d_ssm // headdim

        def buf(name, shape, dtype=torch.float32):
            self.register_buffer(name, torch.empty(shape, dtype=dtype, device=dev))

        buf("dt_bias", nheads, torch.float16)
        buf("A_log", nheads, torch.int8)
        buf("A_log_scale", [])
        buf("D", d_ssm if D_has_hdim else nheads, torch.int8)
        buf("D_scale", [])
        for name, flag in (("dt", quant_dt), ("z", quant_z)):
            if flag:
                buf(f"{name}_scale", [])
            else:
                setattr(self, f"{name}_scale", None)
        if nhead_groups > 0 and ndim_groups > 0:
            buf("ssm_state_scale", [ngroups, nhead_groups, ndim_groups, d_state])
            buf("x_scales", [ngroups, nhead_groups, ndim_groups])
            buf("x_head_group_range", [ngroups, nhead_groups], torch.int32)
            buf("x_dim_group_range", [ngroups, nhead_groups, ndim_groups], torch.int32)
            bc_shape = [ngroups]
        elif nhead_groups == 0 and ndim_groups == 0:
            buf("ssm_state_scale", [1])
            buf("x_scales", [1])
            self.x_head_group_range = self.x_dim_group_range = None
            bc_shape = [1]
        else:
            raise ValueError("nhead_groups and ndim_groups must be both 0 or both not 0")
        for name, flag in (("B", quant_B), ("C", quant_C)):
            if flag:
                buf(f"{name}_scale", bc_shape)
            else:
                setattr(self, f"{name}_scale", None)

    @property
    def grouped(self):
        if (self.x_head_group_range is None) != (self.x_dim_group_range is None):
            raise ValueError("x_head_group_range and x_dim_group_range must be both None or both not None")
        return self.x_head_group_range is not None

    @classmethod
    def from_fp16(cls, d_ssm, headdim, d_state, ngroups, x_scales, x_head_group_range, x_dim_group_range, A_log,
                  chunk_size, ssm_state_scale, D=None, D_has_hdim=False, dt_bias=None, delta_softplus=True,
                  dt_scale=None, B_scale=None, C_scale=None, z_scale=None, dt_limit=(0.0, float("inf"))):
        nhg = x_head_group_range.shape[1] if x_head_group_range is not None else 0
        ndg = x_dim_group_range.shape[2] if x_dim_group_range is not None else 0
        dev = A_log.device
        q = cls(d_ssm, headdim, d_state, ngroups, D_has_hdim, chunk_size, nhg, ndg, delta_softplus,
                dt_limit=dt_limit, device=dev)
        a8, a_s = quantize_tensor_per_tensor_absmax(A_log, 8)
        q.A_log, q.A_log_scale = a8.to(torch.int8), a_s.float().to(dev)
        if x_head_group_range is not None and x_dim_group_range is not None:
            q.ssm_state_scale = cls.get_ssm_state_scales(ssm_state_scale, ngroups, nhg, ndg, d_state, dev)
        else:
            q.ssm_state_scale = ssm_state_scale.float().to(dev)
        if D is not None:
            d8, d_s = quantize_tensor_per_tensor_absmax(D, 8)
            q.D, q.D_scale = d8.to(torch.int8), d_s.float().to(dev)
        else:
            q.D = None
        q.dt_bias = dt_bias.to(torch.float16) if dt_bias is not None else None
        for name, s in (("dt_scale", dt_scale), ("B_scale", B_scale), ("C_scale", C_scale), ("z_scale", z_scale)):
            setattr(q, name, s.float() if s is not None else None)
        q.x_scales = x_scales.float().to(dev)
        q.x_head_group_range = None if x_head_group_range is None else x_head_group_range.to(dev)
        q.x_dim_group_range = None if x_dim_group_range is None else x_dim_group_range.to(dev)
        return q

    @staticmethod
    def get_ssm_state_scales(scales, ngroups, n_head_groups, n_dim_groups, dstates, device):
        """Calibration hands the grouped state scales over either as a tensor
        [ngroups, n_head_groups, n_dim_groups, dstate] or as nested lists of
        (head group size, dim group sizes, [n_dim_groups, dstate] scales) per ssd group."""
        if not isinstance(scales, list):
            return scales.to(device)
        out = torch.empty((ngroups, n_head_groups, n_dim_groups, dstates), device=device)
        for g in range(ngroups):
            for i, (_, _, ch_scales) in enumerate(scales[g]):
                out[g, i] = ch_scales.to(device)
        return out

    def _D_2d(self, expand):
        """D as (h, p) when it has one value per channel, else (h,) or its stride-0 expansion to (h, p)."""
        if self.D is None:
            return None
        if self.D_has_hdim:
            return self.D.reshape(-1, self.headdim)
        return self.D[:, None].expand(-1, self.headdim) if expand else self.D

    def _fixed_args(self):
        return dict(dt_scale=self.dt_scale, q_A_log=self.A_log, A_log_scale=self.A_log_scale,
                    ssm_state_scale=self.ssm_state_scale, B_scale=self.B_scale, C_scale=self.C_scale)

    @torch.no_grad()
    def forward(self, x, dt, B, C, z=None, return_final_states=False):
        """x int8 (b, L, h, p); dt int8 (b, L, h); B, C int8 (b, L, g, n); z int8 or None.  y is fp16."""
        kw = dict(q_x=x, q_dt=dt, q_B=B, q_C=C, q_z=z, z_scale=self.z_scale if z is not None else None,
                  q_D=self._D_2d(False), D_scale=self.D_scale, chunk_size=self.chunk_size, dt_bias=self.dt_bias,
                  initial_states=None, seq_idx=None, cu_seqlens=None, dt_softplus=self.delta_softplus,
                  dt_limit=self.dt_limit, mm_dtype=torch.float16, **self._fixed_args())
        if self.grouped:
            y, final_states = ops._quamba2_mamba_chunk_scan_combined_fwd(
                x_scales=self.x_scales, x_head_group_range=self.x_head_group_range,
                x_dim_group_range=self.x_dim_group_range, **kw)
        else:
            y, final_states = ops._quant_mamba_chunk_scan_combined_fwd(x_scale=self.x_scales, **kw)
        return (y, final_states) if return_final_states else y

    @torch.no_grad()
    def update(self, ssm_state, x, dt, B, C, z=None):
        """One decode step: x int8 (b, h*p), dt int8 (b, h), B, C int8 (b, g*n); ssm_state int8 (b, h, p, n) is
        updated in place."""
        p, n = self.headdim, self.d_state
        b = x.shape[0]
        kw = dict(state=ssm_state, q_x=x.reshape(b, -1, p), q_dt=dt.unsqueeze(-1).expand(-1, -1, p),
                  q_B=B.reshape(b, self.ngroups, n), q_C=C.reshape(b, self.ngroups, n), q_z=z,
                  z_scale=self.z_scale if z is not None else None,
                  q_D=self._D_2d(True),
                  D_scale=self.D_scale if self.D is not None else None,
                  dt_bias=self.dt_bias[:, None].expand(-1, p) if self.dt_bias is not None else None,
                  dt_softplus=self.delta_softplus, **self._fixed_args())
        kw["q_A_log"] = self.A_log[:, None, None].expand(-1, p, n)
        if self.grouped:
            return ops.quamba2_sscan_update_triton(x_scales=self.x_scales, x_head_group_range=self.x_head_group_range,
                                                   x_dim_group_range=self.x_dim_group_range, **kw)
        return ops.quant_sscan_update_triton(x_scale=self.x_scales, **kw)

    def __repr__(self):
        return "QChunkScan()"


# ------------------------------------------------------------------------------------------------ W4A8 linears

_MARLIN_MIN_THREAD_N = 64
_MARLIN_MAX_PARALLEL = 16


class _W4A8Base(nn.Module):
    """int8 activations x Marlin-QQQ packed int4 weights.  ``weight`` int32 (K/16, 2N), ``s_group`` fp16
    (K/128, N), ``s_channel`` fp32 (1, N) and the scalar ``input_scale`` are buffers; ``workspace`` is kept for
    state-dict compatibility (the reference's kernel uses it as a lock array; the kernels here do not)."""
    _out_int8 = False

    def __init__(self, in_features, out_features, group_size=128, device=None, **kwargs):
        super().__init__()
        dev = _dev(device)
        self.bias = None
        self.in_features, self.out_features = in_features, out_features
        self.size_k = in_features
        self.pad_out = (64 - out_features % 64) % 64
        self.size_n = out_features + self.pad_out
        self.max_par = _MARLIN_MAX_PARALLEL
        self.register_buffer("workspace", torch.zeros(self.size_n // _MARLIN_MIN_THREAD_N * _MARLIN_MAX_PARALLEL,
                                                      dtype=torch.int, device=dev))
        self.register_buffer("weight", torch.empty((self.size_k // 16, self.size_n * 16 // 8), dtype=torch.int32,
                                                   device=dev))
        self.register_buffer("input_scale", torch.empty((), dtype=torch.float32, device=dev))
        self.register_buffer("s_channel", torch.empty((1, self.size_n), dtype=torch.float32, device=dev))
        self.register_buffer("s_group", torch.empty((self.size_k // group_size, self.size_n), dtype=torch.float16,
                                                    device=dev))

    @classmethod
    def _pack_from(cls, originalLayer, input_scale, out_scales):
        assert input_scale.numel() == 1, "only a per-tensor input scale is supported"
        assert originalLayer.bias is None, "bias is not supported"
        bits, group_scale = 4, None
        group_size = 128 if originalLayer.in_features > 128 else -1
        # a float layer may ask for per-output-channel int4 (group -1) with a ``w4_group_size`` attribute
        group_size = getattr(originalLayer, "w4_group_size", group_size)
        if getattr(originalLayer, "apply_gptq", False):        # a GPTQ-processed layer carries its own grid
            bits, group_size = originalLayer.bits, originalLayer.group_size
            group_scale = originalLayer.group_scale.to(torch.float16)
        assert bits == 4, "only 4-bit weights are supported"
        if group_size not in (-1, 128):
            raise ValueError("Only groupsize -1 and 128 are supported.")
        dev = originalLayer.weight.device
        q = cls(originalLayer.in_features, originalLayer.out_features, group_size=128, device=dev)
        W = originalLayer.weight.detach()                       # (N, K), possibly already fake-quantised
        ch_scale = (W.abs().amax(dim=1, keepdim=True) / 127.0).reshape(1, -1).float()
        w_ref, packed, s_group, s_channel = w4a8_quantize(
            W.to(torch.float16).t().contiguous(), bits, group_size, group_scale, ch_scale,
            out_scales=out_scales, pad_out=q.pad_out)
        q.size_k, q.size_n = w_ref.shape
        q.weight, q.input_scale = packed.to(dev), input_scale.to(dev).float().reshape(())
        q.s_group, q.s_channel = s_group.to(dev), s_channel.to(dev)
        return q

    def prepared(self):
        """The streaming copies of this layer's weight (:class:`quamba_b200.ops.W4A8Prepared`), owned by the
        module: built on first use, rebuilt when a buffer is replaced (``.to()``, ``load_state_dict``) or written
        in place, freed with the module.  ``release_prepared()`` drops them early."""
        prep = self.__dict__.get("_prep")
        if prep is None or prep.stale(self.weight, self.s_channel, self.s_group):
            prep = ops.prepare_w4a8_weight(self.weight, self.s_channel, self.s_group, self.size_n, self.size_k)
            self.__dict__["_prep"] = prep
        return prep

    def release_prepared(self, w8=True, w4=True):
        prep = self.__dict__.get("_prep")
        if prep is not None:
            prep.release(w8, w4)

    def _gemm(self, x2, transpose):
        return ops.w4a8_linear(x2, self.prepared(), self.input_scale, transpose, self._out_int8)

    @torch.no_grad()
    def forward(self, x):
        lead = x.shape[:-1]
        y = self._gemm(x.reshape(-1, x.shape[-1]).contiguous(), False)
        if self.pad_out:
            y = y[:, :-self.pad_out]
        return y.reshape(*lead, -1)

    @torch.no_grad()
    def to_seqlen_last(self, x):
        """(B, L, K) -> (B, N, L) view of a (N, B*L) result: the sequence stays the unit-stride dimension,
        which is what the conv1d forward wants."""
        lead = x.shape[:-1]
        y = self._gemm(x.reshape(-1, x.shape[-1]), True)
        if self.pad_out:
            y = y[:-self.pad_out, :]
        return y.view(-1, *lead).transpose(0, 1)

    def __repr__(self):
        return f"{type(self).__name__}(in_features={self.in_features}, out_features={self.out_features})"


class W4A8B16O16Linear(_W4A8Base):
    """fp16 output."""

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear, input_scale: torch.Tensor):
        return cls._pack_from(originalLayer, input_scale, None)


class W4A8B8O8Linear(_W4A8Base):
    """int8 output; the output scale is folded into s_channel."""
    _out_int8 = True

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear, input_scale: torch.Tensor, output_scale: torch.Tensor):
        assert output_scale.numel() == 1, "only a per-tensor output scale is supported"
        return cls._pack_from(originalLayer, input_scale, output_scale)


class W4A8B8O8LinearParallel(_W4A8Base):
    """int8 output with one output scale per column segment (x | B | C | dt ... produced by one projection)."""
    _out_int8 = True

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear, input_scale: torch.Tensor, output_scales, out_split_dims):
        assert sum(out_split_dims) == originalLayer.out_features
        assert len(out_split_dims) == len(output_scales)
        per_col = torch.cat([torch.as_tensor(s).reshape(-1)[:1].float().cpu().repeat(d)
                             for d, s in zip(out_split_dims, output_scales)])
        return cls._pack_from(originalLayer, input_scale, per_col)

    to_seqlen_last = None


# ------------------------------------------------------------------------------------------------ W8A8 linears

class _W8A8Base(nn.Module):
    """int8 activations x int8 weights.  ``weight`` is the (K, N_pad) transpose view of a row-major (N_pad, K)
    matrix; ``a`` and ``b`` are the activation-side and weight-side fp32 scales."""
    _b_per_column = False
    _out_dtype = None           # None: same as the input (int8)

    def __init__(self, in_features, out_features, device=None):
        super().__init__()
        dev = _dev(device)
        self.bias = None
        self.in_features, self.out_features = in_features, out_features
        self.pad_out = (16 - out_features % 16) % 16
        n_pad = out_features + self.pad_out
        self.register_buffer("weight", torch.empty_strided((in_features, n_pad), stride=(1, in_features),
                                                           dtype=torch.int8, device=dev))
        self.register_buffer("a", torch.empty((1, 1), dtype=torch.float32, device=dev))
        self.register_buffer("b", torch.empty((1, n_pad if self._b_per_column else 1), dtype=torch.float32, device=dev))

    def _set_weight(self, w8_float):
        """w8_float: (N, K) rounded values."""
        if self.pad_out:
            w8_float = nn.functional.pad(w8_float, (0, 0, 0, self.pad_out)).contiguous()
        self.weight = w8_float.to(torch.int8).t()

    def _matvec(self, y, x2):
        ops.quant_linear_cuda.cutlass_scaled_mv_dq(y, self.weight.t(), x2, self.alpha, 0.0)

    @torch.no_grad()
    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = torch.empty((x2.shape[0], self.out_features + self.pad_out), dtype=self._out_dtype or x.dtype,
                        device=x.device)
        if x2.shape[0] == 1:
            self._matvec(y, x2)
        else:
            ops.quant_linear_cuda.cutlass_scaled_mm_dq(y, x2, self.weight, self.a, self.b)
        if self.pad_out:
            y = y[:, :-self.pad_out]
        return y.reshape(*lead, -1)

    def __repr__(self):
        return f"{type(self).__name__}(in_features={self.in_features}, out_features={self.out_features})"


class _AlphaMixin(_FloatStateMixin):
    _float_state = ("alpha",)


class W8A8B8O8Linear(_AlphaMixin, _W8A8Base):
    """int8 output, per-tensor scales: y = rint(a * b * (x @ W^T)) with a = s_in / s_out, b = s_w."""

    def __init__(self, in_features, out_features, device=None):
        super().__init__(in_features, out_features, device)
        self.alpha = 0.0
        self._install_float_state()

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear, input_scale: float = 1.0, output_scale: float = 1.0):
        dev = originalLayer.weight.device
        q = cls(originalLayer.in_features, originalLayer.out_features, device=dev)
        w8, ws = quantize_tensor_per_tensor_absmax(originalLayer.weight.detach(), 8)
        q._set_weight(w8)
        s_in, s_out = _as_float(input_scale), _as_float(output_scale)
        q.a = torch.tensor([[s_in / s_out]], dtype=torch.float32, device=dev)
        q.b = ws.reshape(1, 1).to(dev)
        q.alpha = (ws * s_in / s_out).item()
        return q

    @torch.no_grad()
    def to_seqlen_last(self, x):
        """(B, L, K) -> (B, N, L) view of a (N, B*L) int8 result."""
        B, L, D = x.shape
        x2 = x.reshape(-1, D)
        pad_in = (16 - x2.shape[0] % 16) % 16                   # output rows must stay 16-byte aligned
        if pad_in:
            x2 = nn.functional.pad(x2, (0, 0, pad_in, 0))
        y = torch.empty((self.out_features + self.pad_out, x2.shape[0]), dtype=x.dtype, device=x.device)
        ops.quant_linear_cuda.cutlass_scaled_mm_dq(y, self.weight.t(), x2.t(), self.b, self.a)
        if self.pad_out:
            y = y[:-self.pad_out]
        if pad_in:
            y = y[:, pad_in:]
        return y.reshape(-1, B, L).transpose(0, 1) if pad_in else y.view(-1, B, L).transpose(0, 1)


class W8A8B8O8LinearParallel(_W8A8Base):
    """int8 output with a weight scale and an output scale per column segment: b[n] = s_w(seg) / s_out(seg)."""
    _b_per_column = True

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear, input_scale: float, output_scales: list, out_split_dims: list):
        assert sum(out_split_dims) == originalLayer.out_features
        assert len(out_split_dims) == len(output_scales)
        dev = originalLayer.weight.device
        q = cls(originalLayer.in_features, originalLayer.out_features, device=dev)
        parts, col_scales, start = [], [], 0
        W = originalLayer.weight.detach()
        for dim, s_out in zip(out_split_dims, output_scales):
            w8, ws = quantize_tensor_per_tensor_absmax(W[start:start + dim], 8)
            parts.append(w8)
            col_scales += [ws.item() / _as_float(s_out)] * dim
            start += dim
        col_scales += [0.0] * q.pad_out
        q._set_weight(torch.cat(parts, dim=0))
        q.a = torch.tensor([[_as_float(input_scale)]], dtype=torch.float32, device=dev)
        q.b = torch.tensor([col_scales], dtype=torch.float32, device=dev)
        return q

    def _matvec(self, y, x2):
        ops.quant_linear_cuda.w8a8o8_gemv(y, self.weight.t(), x2, self.b, self.a)


class W8A8B16O16Linear(_AlphaMixin, _W8A8Base):
    """fp16 output, per-tensor scales: y = a * b * (x @ W^T) with a = s_in, b = s_w."""
    _out_dtype = torch.float16

    def __init__(self, in_features, out_features, device=None):
        super().__init__(in_features, out_features, device)
        self.alpha = 0.0
        self._install_float_state()

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear, input_scale: float = 1.0):
        dev = originalLayer.weight.device
        q = cls(originalLayer.in_features, originalLayer.out_features, device=dev)
        w8, ws = quantize_tensor_per_tensor_absmax(originalLayer.weight.detach(), 8)
        q._set_weight(w8)
        s_in = _as_float(input_scale)
        q.a = torch.tensor([[s_in]], dtype=torch.float32, device=dev)
        q.b = ws.reshape(1, 1).to(dev)
        q.alpha = (ws * s_in).item()
        return q
