"""Quantized Mamba2 mixers W4A8QMamba2 / W8A8QMamba2 with the reference's constructor arguments, sub-module
names (``in_proj``, ``conv1d``, ``qchunk_scan``, ``norm``, ``had``, ``out_proj``), ``forward`` / ``step`` /
``allocate_inference_cache`` (quamba/qMamba2.py:735-1068, :1071-1406).  Every tensor op of ``forward`` and ``step``
is one of this package's CUDA entry points; what remains here is views (``split`` of in_proj's int8 output) and
the copy of the last ``d_conv`` inputs into the conv state.
"""
import copy

import torch
import torch.nn as nn

from .modules import (QHadamard, Quamb2Conv1D, Quamba2ChunkScan, W4A8B8O8LinearParallel, W4A8B16O16Linear,
                      W8A8B8O8LinearParallel, W8A8B16O16Linear)
from .norm import QRMSNormGated

__all__ = ["W4A8QMamba2", "W8A8QMamba2", "get_group_params"]


def get_group_params(scales, ngroups, device):
    """x_conv_out scales as calibration hands them over: a tensor (per-tensor scale) or, per ssd group, a list of
    (head group size, dim group sizes, scales) -> cumulative range tables + [G, HG, DG] scales
    (quamba/qMamba2.py:42-66)."""
    if not isinstance(scales, list):
        return None, None, scales.to(device)
    hgr, dgr, out = [], [], []
    for g in range(ngroups):
        hs = torch.stack([s[0] for s in scales[g]], dim=0).to(device)
        ds = torch.stack([s[1] for s in scales[g]], dim=0).to(device)
        hgr.append(torch.cumsum(hs, dim=0).to(torch.int32))
        dgr.append(torch.cumsum(ds, dim=1).to(torch.int32))
        out.append(torch.stack([s[2] for s in scales[g]], dim=0))
    return torch.stack(hgr, 0), torch.stack(dgr, 0), torch.stack(out, 0)


class _QMamba2(nn.Module):
    _in_proj_cls = None
    _out_proj_cls = None
    _linear_kwargs = {}

    def __init__(self, d_model, d_state=128, d_conv=4, conv_init=None, expand=2, headdim=64, d_ssm=None, ngroups=1,
                 A_init_range=(1, 16), D_has_hdim=False, rmsnorm=True, norm_before_gate=False, use_had_transform=True,
                 dt_min=0.001, dt_max=0.1, dt_init_floor=1e-4, dt_limit=(0.0, float("inf")), bias=False, conv_bias=True,
                 chunk_size=256, use_mem_eff_path=True, layer_idx=None, process_group=None, sequence_parallel=True,
                 device=None, dtype=None, x_nhead_group=4, x_ndim_group=4):
        super().__init__()
        kw = {"device": device}
        self.d_model, self.d_state, self.d_conv, self.conv_init, self.expand = d_model, d_state, d_conv, conv_init, expand
        assert process_group is None, "Only support process_group=None for now"
        self.process_group, self.sequence_parallel = None, sequence_parallel
        self.world_size, self.local_rank = 1, 0
        self.d_inner = expand * d_model
        self.headdim = headdim
        self.d_ssm = self.d_inner if d_ssm is None else d_ssm
        self.ngroups = ngroups
        assert self.d_ssm % headdim == 0
        self.nheads = self.d_ssm // headdim
        self.D_has_hdim, self.rmsnorm, self.norm_before_gate = D_has_hdim, rmsnorm, norm_before_gate
        self.dt_limit, self.activation, self.chunk_size = dt_limit, "silu", chunk_size
        self.use_mem_eff_path, self.layer_idx = use_mem_eff_path, layer_idx
        assert bias is False, "Only support bias=False for now"
        # Order: [z, x, B, C, dt]
        d_in_proj = 2 * self.d_inner + 2 * ngroups * d_state + self.nheads
        self.in_proj = self._in_proj_cls(d_model, d_in_proj, **self._linear_kwargs, **kw)
        conv_dim = self.d_ssm + 2 * ngroups * d_state
        self.conv1d = Quamb2Conv1D(self.d_ssm, headdim, d_state, ngroups, x_nhead_group, x_ndim_group, conv_dim, conv_dim,
                                   d_conv, groups=conv_dim, padding=d_conv - 1, bias=True, **kw)
        self.qchunk_scan = Quamba2ChunkScan(self.d_ssm, headdim, d_state, ngroups, D_has_hdim, chunk_size, x_nhead_group,
                                            x_ndim_group, delta_softplus=True, dt_limit=dt_limit, **kw)
        assert rmsnorm, "Only support Mamba2 block with rmsnorm"
        self.norm = QRMSNormGated(self.d_ssm, eps=1e-5, norm_before_gate=norm_before_gate, group_size=self.d_ssm // ngroups,
                                  use_float16_output=True, **kw)
        assert use_had_transform, "the out_proj input is always Hadamard-rotated here"
        self.had = QHadamard(self.d_inner, x_H_scale=1.0)
        self.out_proj = self._out_proj_cls(self.d_inner, d_model, **self._linear_kwargs, **kw)

    # ---- construction from a float layer + calibrated activation scales (qMamba2.py:826-917) --------------------
    @classmethod
    def _make_linears(cls, layer, act_scales, split_dims):
        raise NotImplementedError

    @classmethod
    def from_fp16(cls, originalLayer, act_scales, use_had_transform=True):
        o = originalLayer
        dev = o.conv1d.weight.device
        hgr, dgr, x_out_scales = get_group_params(act_scales["x_conv_out:input"], o.ngroups, dev)
        nhg = 0 if hgr is None else hgr.shape[1]
        ndg = 0 if dgr is None else dgr.shape[2]
        q = cls(d_model=o.d_model, d_state=o.d_state, d_conv=o.d_conv, conv_init=getattr(o, "conv_init", None),
                expand=o.expand, headdim=o.headdim, d_ssm=o.d_ssm, ngroups=o.ngroups, rmsnorm=o.rmsnorm,
                norm_before_gate=o.norm_before_gate, use_had_transform=use_had_transform, dt_limit=o.dt_limit,
                chunk_size=o.chunk_size, use_mem_eff_path=False, layer_idx=o.layer_idx, device=dev,
                x_nhead_group=nhg, x_ndim_group=ndg)
        split_dims = [q.d_ssm, q.d_ssm, q.ngroups * q.d_state, q.ngroups * q.d_state, q.nheads]
        q.in_proj, q.out_proj = cls._make_linears(o, act_scales, split_dims)
        q.conv1d = Quamb2Conv1D.from_fp16(copy.deepcopy(o.conv1d), q.d_ssm, q.headdim, q.d_state, q.ngroups,
                                          act_scales["x_conv_in:output"], act_scales["B_conv_in:output"],
                                          act_scales["C_conv_in:output"], x_out_scales, act_scales["B_conv_out:input"],
                                          act_scales["C_conv_out:input"], hgr, dgr)
        q.qchunk_scan = Quamba2ChunkScan.from_fp16(
            q.d_ssm, q.headdim, q.d_state, q.ngroups, x_out_scales, hgr, dgr, o.A_log, o.chunk_size, D=o.D,
            D_has_hdim=q.D_has_hdim, dt_bias=o.dt_bias, delta_softplus=True, dt_scale=act_scales["dt_act:output"],
            B_scale=act_scales["B_conv_out:input"], C_scale=act_scales["C_conv_out:input"],
            ssm_state_scale=act_scales["ssm_state_act:input"], dt_limit=o.dt_limit)
        q.norm = QRMSNormGated.from_fp16(o.norm, z_scale=act_scales["z_act:output"].item(), use_float16_output=True)
        q.had = QHadamard(q.d_inner, x_H_scale=act_scales["out_proj:input"].item(), blocks=getattr(o, "had_blocks", 1))
        return q

    # ---- prefill (qMamba2.py:920-994) ------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, u, seqlen=None, seq_idx=None, cu_seqlens=None, inference_params=None):
        """u int8: (batch, seqlen, d_model), or (batch * seqlen, d_model) with ``seqlen`` given.  Returns fp16 of the
        same shape."""
        seqlen_og = seqlen
        if seqlen is None:
            batch, seqlen, _ = u.shape
        else:
            batch = u.shape[0] // seqlen
        conv_state = ssm_state = None
        if inference_params is not None:
            conv_state, ssm_state = self._get_states_from_cache(inference_params, batch)
            if inference_params.seqlen_offset > 0:
                out, _, _ = self.step(u, conv_state, ssm_state)
                return out
        zxbcdt = self.in_proj(u)
        if seqlen_og is not None:
            zxbcdt = zxbcdt.view(batch, seqlen, -1)
        gn = self.ngroups * self.d_state
        z, xBC, dt = torch.split(zxbcdt, [self.d_ssm, self.d_ssm + 2 * gn, self.nheads], dim=-1)
        if conv_state is not None:
            # the last d_conv inputs, zero-padded on the left when the prompt is shorter
            xBC_t = xBC.transpose(1, 2)
            conv_state.copy_(nn.functional.pad(xBC_t, (self.d_conv - xBC_t.shape[-1], 0)))
        x, B, C = self.conv1d(xBC.transpose(1, 2))
        x = x.transpose(1, 2).unflatten(-1, (self.nheads, self.headdim))
        B = B.transpose(1, 2).unflatten(-1, (self.ngroups, self.d_state))
        C = C.transpose(1, 2).unflatten(-1, (self.ngroups, self.d_state))
        y = self.qchunk_scan(x, dt, B, C, z=None, return_final_states=ssm_state is not None)
        if ssm_state is not None:
            y, last_state = y
            if cu_seqlens is not None:
                raise NotImplementedError("Not implemented for cu_seqlens yet")
            ssm_state.copy_(last_state)
        y = self.norm(y.flatten(-2), z)
        if seqlen_og is not None:
            y = y.flatten(0, 1)
        return self.out_proj(self.had(y))

    # ---- decode (qMamba2.py:997-1020) ------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, hidden_states, conv_state, ssm_state):
        assert hidden_states.shape[1] == 1, "Only support decoding with 1 token at a time for now"
        zxbcdt = self.in_proj(hidden_states.squeeze(1))
        gn = self.ngroups * self.d_state
        z, xBC, dt = torch.split(zxbcdt, [self.d_ssm, self.d_ssm + 2 * gn, self.nheads], dim=-1)
        x, B, C = self.conv1d.update(xBC, conv_state)
        y = self.qchunk_scan.update(ssm_state, x, dt, B, C, z=None)
        y = self.norm(y.flatten(-2), z)
        out = self.out_proj(self.had(y))
        return out.unsqueeze(1), conv_state, ssm_state

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        dev = self.out_proj.weight.device
        conv_state = torch.zeros(batch_size, self.d_conv, self.conv1d.weight.shape[0], device=dev,
                                 dtype=torch.int8).transpose(1, 2)
        ssm_state = torch.zeros(batch_size, self.nheads, self.headdim, self.d_state, device=dev, dtype=torch.int8)
        return conv_state, ssm_state

    def _get_states_from_cache(self, inference_params, batch_size, initialize_states=False):
        assert self.layer_idx is not None
        cache = inference_params.key_value_memory_dict
        if self.layer_idx not in cache:
            # int8 states: the kernels update both caches in place in int8 (the reference allocates its ssm state
            # here as float16 and then copies the int8 final state into it)
            cache[self.layer_idx] = self.allocate_inference_cache(batch_size, 0)
        elif initialize_states:
            for t in cache[self.layer_idx]:
                t.zero_()
        return cache[self.layer_idx]


class W4A8QMamba2(_QMamba2):
    _in_proj_cls = W4A8B8O8LinearParallel
    _out_proj_cls = W4A8B16O16Linear
    _linear_kwargs = {"group_size": 128}

    @classmethod
    def _make_linears(cls, o, act_scales, split_dims):
        in_proj = W4A8B8O8LinearParallel.from_fp16(
            copy.deepcopy(o.in_proj), act_scales["in_proj:input"],
            [act_scales["z_act:input"], act_scales["x_conv_in:input"], act_scales["B_conv_in:input"],
             act_scales["C_conv_in:input"], act_scales["dt_act:input"]], split_dims)
        out_proj = W4A8B16O16Linear.from_fp16(copy.deepcopy(o.out_proj), act_scales["out_proj:input"])
        return in_proj, out_proj


class W8A8QMamba2(_QMamba2):
    _in_proj_cls = W8A8B8O8LinearParallel
    _out_proj_cls = W8A8B16O16Linear

    @classmethod
    def _make_linears(cls, o, act_scales, split_dims):
        in_proj = W8A8B8O8LinearParallel.from_fp16(
            copy.deepcopy(o.in_proj), act_scales["in_proj:input"].item(),
            [act_scales[k].item() for k in ("z_act:input", "x_conv_in:input", "B_conv_in:input", "C_conv_in:input",
                                            "dt_act:input")], split_dims)
        out_proj = W8A8B16O16Linear.from_fp16(copy.deepcopy(o.out_proj), act_scales["out_proj:input"].item())
        return in_proj, out_proj
