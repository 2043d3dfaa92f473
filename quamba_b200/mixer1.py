"""Quantized Mamba1 mixers W8A8QMamba / W4A8QMamba with the reference's constructor arguments, sub-module names, scale
keys and cache layout (quamba/qMambaLayer.py:512-756 and :759-1003), composed from this package's modules:

    in_proj (int8 out, written sequence-last) -> x | z -> QCausalConv1D -> x_proj -> dt | B | C -> dt_proj (sequence-last)
    -> QSScan (int8 scan, gate z) -> QHadamard (or QAct) -> out_proj (fp16)

The decode caches are int8: conv_state (batch, d_inner, d_conv) and ssm_state (batch, d_inner, d_state).
"""
import copy
import math

import torch
import torch.nn as nn

from .modules import (QCausalConv1D, QHadamard, QSScan, W4A8B8O8Linear, W4A8B16O16Linear, W8A8B8O8Linear, W8A8B16O16Linear,
                      _FloatStateMixin)

__all__ = ["QAct", "W8A8QMamba", "W4A8QMamba"]


class QAct(_FloatStateMixin, nn.Module):
    """Per-tensor int8 quantisation without a rotation, the reference's alternative to QHadamard
    (quamba/qActLayer.py:4-28): clamp(x / scale) cast to int8 (the cast truncates toward zero, as there)."""
    _float_state = ("scale",)

    def __init__(self, scale):
        super().__init__()
        self.scale = scale
        self._install_float_state()

    @torch.no_grad()
    def forward(self, x):
        return (x / self.scale).clamp(min=-128, max=127).to(torch.int8)

    def __repr__(self):
        return "QAct()"


def _item(v):
    return v.item() if torch.is_tensor(v) else float(v)


class _QMamba(nn.Module):
    _in_cls = _x_cls = _out_cls = None          # linear classes of in_proj, x_proj, out_proj (dt_proj is W8A8 in both mixers)

    def __init__(self, d_model, d_state=16, d_conv=4, expand=2, dt_rank="auto", dt_min=0.001, dt_max=0.1, dt_init="random",
                 dt_scale=1.0, dt_init_floor=1e-4, conv_bias=True, bias=False, use_had_transform=True, use_fast_path=True,
                 layer_idx=None, device=None, dtype=None):
        super().__init__()
        assert bias is False, "Only support bias=False for now"
        self.d_model, self.d_state, self.d_conv, self.expand = d_model, d_state, d_conv, expand
        self.d_inner = int(expand * d_model)
        self.dt_rank = math.ceil(d_model / 16) if dt_rank == "auto" else dt_rank
        self.use_fast_path, self.layer_idx, self.activation = use_fast_path, layer_idx, "silu"
        self.in_proj = self._new_linear(self._in_cls, d_model, self.d_inner * 2, device)
        self.conv1d = QCausalConv1D(self.d_inner, self.d_inner, d_conv, groups=self.d_inner, padding=d_conv - 1, bias=conv_bias,
                                    device=device)
        self.x_proj = self._new_linear(self._x_cls, self.d_inner, self.dt_rank + 2 * d_state, device)
        self.dt_proj = W8A8B8O8Linear(self.dt_rank, self.d_inner, device=device)
        self.selective_scan = QSScan(d_state=d_state, d_inner=self.d_inner, delta_softplus=True, device=device)
        self.had = QHadamard(self.d_inner, x_H_scale=1.0) if use_had_transform else QAct(scale=1.0)
        self.out_proj = self._new_linear(self._out_cls, self.d_inner, d_model, device)

    @staticmethod
    def _new_linear(cls, k, n, device):
        if issubclass(cls, (W4A8B8O8Linear, W4A8B16O16Linear)):
            return cls(k, n, group_size=128, device=device)
        return cls(k, n, device=device)

    @classmethod
    def _linear_from(cls, lin_cls, layer, input_scale, output_scale=None):
        w4 = issubclass(lin_cls, (W4A8B8O8Linear, W4A8B16O16Linear))
        s_in = torch.as_tensor(input_scale, dtype=torch.float32) if w4 else _item(input_scale)
        if output_scale is None:
            return lin_cls.from_fp16(copy.deepcopy(layer), s_in)
        s_out = torch.as_tensor(output_scale, dtype=torch.float32) if w4 else _item(output_scale)
        return lin_cls.from_fp16(copy.deepcopy(layer), s_in, s_out)

    @classmethod
    @torch.no_grad()
    def from_fp16(cls, originalLayer, act_scales, use_had_transform=True):
        """``originalLayer``: a float Mamba1 mixer with in_proj, conv1d, x_proj, dt_proj (bias kept apart in
        ``dt_proj_bias``), A_log, D, out_proj; ``act_scales``: the reference's tap names -> scale."""
        o, s = originalLayer, act_scales
        dev = o.out_proj.weight.device
        q = cls(d_model=o.d_model, d_state=o.d_state, d_conv=o.d_conv, expand=o.expand, dt_rank=o.dt_rank,
                use_had_transform=use_had_transform, use_fast_path=False, layer_idx=o.layer_idx, device=dev)
        q.in_proj = cls._linear_from(cls._in_cls, o.in_proj, s["in_proj:input"], s["in_proj:output"])
        q.conv1d = QCausalConv1D.from_fp16(copy.deepcopy(o.conv1d), input_scale=_item(s["in_proj:output"]),
                                           output_scale=_item(s["x_proj:input"]))
        q.x_proj = cls._linear_from(cls._x_cls, o.x_proj, s["x_proj:input"], s["x_proj:output"])
        # dt_proj reads x_proj's int8 output as it is (no requantisation in between); its bias lives in the scan
        q.dt_proj = W8A8B8O8Linear.from_fp16(copy.deepcopy(o.dt_proj), _item(s["x_proj:output"]), _item(s["dt_proj:output"]))
        q.selective_scan = QSScan.from_fp16(o.d_state, o.d_inner, o.A_log.detach().clone(), D=o.D.detach().clone(),
                                            dt_bias=o.dt_proj_bias.detach().clone(), delta_softplus=True,
                                            ssm_state_scale=s["ssm_state_act:input"], u_scale=s["x_proj:input"],
                                            dt_scale=s["dt_proj:output"], B_scale=s["x_proj:output"], C_scale=s["x_proj:output"],
                                            z_scale=s["in_proj:output"])
        if use_had_transform:
            q.had.x_H_scale = _item(s["out_proj:input"])
        else:
            q.had.scale = _item(s["out_proj:input"])
        q.out_proj = cls._linear_from(cls._out_cls, o.out_proj, s["out_proj:input"])
        return q.to(dev)

    @torch.no_grad()
    def forward(self, hidden_states, inference_params=None):
        """hidden_states int8 (B, L, d_model) -> fp16 (B, L, d_model); with ``inference_params`` the caches are filled
        (prefill) or one token is decoded (seqlen_offset > 0)."""
        batch, seqlen, _ = hidden_states.shape
        conv_state = ssm_state = None
        if inference_params is not None:
            conv_state, ssm_state = self._get_states_from_cache(inference_params, batch)
            if inference_params.seqlen_offset > 0:
                return self.step(hidden_states, conv_state, ssm_state)[0]
        xz = self.in_proj.to_seqlen_last(hidden_states)                 # (B, 2 d_inner, L) int8, L contiguous
        x, z = xz.chunk(2, dim=1)
        if conv_state is not None:                                        # the last d_conv inputs of every channel
            conv_state.copy_(nn.functional.pad(x, (self.d_conv - seqlen, 0)) if seqlen < self.d_conv else x[..., -self.d_conv:])
        x = self.conv1d(x)                                                # (B, d_inner, L) int8
        x_dbl = self.x_proj(x.transpose(1, 2).contiguous())               # (B, L, dt_rank + 2 N) int8
        dt, B, C = torch.split(x_dbl, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        dt = self.dt_proj.to_seqlen_last(dt.contiguous())                 # (B, d_inner, L) int8
        B, C = B.transpose(1, 2).contiguous(), C.transpose(1, 2).contiguous()
        y = self.selective_scan(x, dt, B, C, z=z, return_last_state=ssm_state is not None)
        if ssm_state is not None:
            y, last = y
            ssm_state.copy_(last)
        return self.out_proj(self.had(y))

    @torch.no_grad()
    def step(self, hidden_states, conv_state, ssm_state):
        assert hidden_states.shape[1] == 1, "Only support decoding with 1 token at a time for now"
        xz = self.in_proj(hidden_states.squeeze(1))                       # (B, 2 d_inner) int8
        x, z = xz.chunk(2, dim=-1)
        x = self.conv1d.update(x.contiguous(), conv_state)
        x_dbl = self.x_proj(x)
        dt, B, C = torch.split(x_dbl, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        dt = self.dt_proj(dt.contiguous())
        y, ssm_state = self.selective_scan.update(ssm_state, x.contiguous(), dt, B.contiguous(), C.contiguous(), z=z.contiguous())
        out = self.out_proj(self.had(y))
        return out.unsqueeze(1), conv_state, ssm_state

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        dev = self.out_proj.weight.device
        return (torch.zeros(batch_size, self.d_inner, self.d_conv, device=dev, dtype=torch.int8),
                torch.zeros(batch_size, self.d_inner, self.d_state, device=dev, dtype=torch.int8))

    def _get_states_from_cache(self, inference_params, batch_size, initialize_states=False):
        assert self.layer_idx is not None
        cache = inference_params.key_value_memory_dict
        if self.layer_idx not in cache:
            cache[self.layer_idx] = self.allocate_inference_cache(batch_size, 0)
        elif initialize_states:
            for t in cache[self.layer_idx]:
                t.zero_()
        return cache[self.layer_idx]


class W8A8QMamba(_QMamba):
    _in_cls, _x_cls, _out_cls = W8A8B8O8Linear, W8A8B8O8Linear, W8A8B16O16Linear


class W4A8QMamba(_QMamba):
    _in_cls, _x_cls, _out_cls = W4A8B8O8Linear, W4A8B8O8Linear, W4A8B16O16Linear
