"""Extension-level API of the reference, served by the B200 library.

Each namespace below has the name and the call signatures of one compiled extension
(or Triton entry point) of the reference, so the quantized modules and the parity tests
read the same way; underneath, every call marshals raw device pointers into the C ABI of
``libquamba_b200.so`` on torch's current stream.  Outputs are allocated here through
torch's caching allocator exactly as the reference's bindings do.  There is no fallback
path: a missing library or a rejected argument raises ``RuntimeError``.

Reference interfaces mirrored (paths inside the reference project):
  quant_sscan_cuda.fwd                      csrc/selective_scan/quant_sscan.cpp:122-270
  quant_causal_conv1d_cuda.fwd / .update    csrc/causal_conv1d/quant_causal_conv1d.cpp:77-231
  quamba2_conv1d_cuda.fwd / .update         csrc/causal_conv1d/quamba2_conv1d.cpp:122-385
  quant_hadamard.fast_hadamard_transform*   csrc/hadamard/quant_hadamard.cpp:72-294
  quant_linear_cuda.*                       csrc/linear/quant_linear.cpp:62-75
  _quant_/_quamba2_mamba_chunk_scan_combined_fwd   quamba/triton/quant_ssd_combined.py:11-166
  quant_/quamba2_sscan_update_triton        quamba/triton/selective_state_update.py:129-478
  _qlayer_norm_fwd / _qlayer_normgated_fwd  quamba/triton/quant_norm.py:134-206, quant_normgated.py:85-132
  quant_embedding_cuda.*                    csrc/embedding/quant_embedding_kernel.cuh:87-139, :207-260
"""
import math

import ctypes
import weakref

import torch

from . import _lib

__all__ = ["quant_sscan_cuda", "quant_causal_conv1d_cuda", "quamba2_conv1d_cuda", "quant_hadamard",
           "quant_linear_cuda", "_quant_mamba_chunk_scan_combined_fwd", "_quamba2_mamba_chunk_scan_combined_fwd",
           "quant_sscan_update_triton", "quamba2_sscan_update_triton", "prepare_w4a8_weight", "_qlayer_norm_fwd",
           "_qlayer_normgated_fwd", "quant_embedding_cuda"]


def _p(t):
    return None if t is None else t.data_ptr()


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _req(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _cuda_i8(t, name):
    _req(t.is_cuda, f"{name} must be a CUDA tensor")
    _req(t.dtype == torch.int8, f"{name} must be int8")


def _scale_t(t, name, device):
    _req(t is not None, f"{name} is required")
    _req(t.is_cuda and t.dtype == torch.float32, f"{name} must be a float32 CUDA tensor")
    return t


def _run(fn, args, ref_tensor):
    with torch.cuda.device(ref_tensor.device):
        _lib.call(fn, args, _stream(ref_tensor))


# ------------------------------------------------------------------------------------------------
class quant_causal_conv1d_cuda:
    @staticmethod
    def fwd(x, scale_x, weight, scale_w, scale_out, scale_b, bias=None, seq_idx=None, initial_states=None,
            final_states_out=None, silu_activation=True):
        _cuda_i8(x, "x"); _cuda_i8(weight, "weight")
        _req(x.dim() == 3, "x must be (batch, dim, seqlen)")
        batch, dim, seqlen = x.shape
        width = weight.shape[-1]
        _req(tuple(weight.shape) == (dim, width), "weight must have shape (dim, width)")
        _req(x.stride(2) == 1 or x.stride(1) == 1, "x must be contiguous in seqlen or in channels")
        if bias is not None:
            _cuda_i8(bias, "bias"); _req(tuple(bias.shape) == (dim,) and bias.stride(-1) == 1, "bias must have shape (dim,)")
        if seq_idx is not None:
            raise RuntimeError("No implementation for seq_idx")
        if initial_states is not None:
            raise RuntimeError("No implementation for initial_states")
        if final_states_out is not None:
            raise RuntimeError("No implementation for final_states_out")
        out = torch.empty_like(x)
        w = weight.contiguous()
        args = _lib.make("qb_conv1d_fwd_args", x=_p(x), out=_p(out), weight=_p(w), bias=_p(bias),
                         x_sb=x.stride(0), x_sd=x.stride(1), x_sl=x.stride(2),
                         out_sb=out.stride(0), out_sd=out.stride(1), out_sl=out.stride(2),
                         batch=batch, dim=dim, seqlen=seqlen, width=width, scale_x=float(scale_x),
                         scale_w=float(scale_w), scale_out=float(scale_out), scale_b=float(scale_b),
                         silu=int(bool(silu_activation)))
        _run("qb_causal_conv1d_fwd", args, x)
        return out

    @staticmethod
    def update(x, conv_state, scale_x, weight, scale_w, scale_out, scale_b, bias=None, silu_activation=True):
        _cuda_i8(x, "x"); _cuda_i8(conv_state, "conv_state"); _cuda_i8(weight, "weight")
        batch, dim = x.shape
        width = weight.shape[-1]
        _req(tuple(conv_state.shape) == (batch, dim, width), "conv_state must have shape (batch, dim, width)")
        _req(tuple(weight.shape) == (dim, width), "weight must have shape (dim, width)")
        out = torch.empty_like(x)
        w = weight.contiguous()
        args = _lib.make("qb_conv1d_update_args", x=_p(x), conv_state=_p(conv_state), out=_p(out), weight=_p(w),
                         bias=_p(bias), x_sb=x.stride(0), x_sd=x.stride(1), state_sb=conv_state.stride(0),
                         state_sd=conv_state.stride(1), state_sw=conv_state.stride(2), out_sb=out.stride(0),
                         out_sd=out.stride(1), batch=batch, dim=dim, width=width, scale_x=float(scale_x),
                         scale_w=float(scale_w), scale_out=float(scale_out), scale_b=float(scale_b),
                         silu=int(bool(silu_activation)))
        _run("qb_causal_conv1d_update", args, x)
        return out


# ------------------------------------------------------------------------------------------------
def _q2_common(x_dim, x_headdim, d_state, n_groups, hgr, dgr, x_scales, B_scales, C_scales):
    nhg = ndg = 0
    if hgr is not None and dgr is not None:
        _req(hgr.dtype == torch.int32 and dgr.dtype == torch.int32, "group ranges must be int32")
        _req(hgr.shape[0] == n_groups and dgr.shape[0] == n_groups,
             "x_head_group_range.shape[0] / x_dim_group_range.shape[0] must equal the number of groups")
        nhg, ndg = hgr.shape[1], dgr.shape[2]
        _req(dgr.shape[1] == nhg, "x_dim_group_range.shape[1] must equal the number of head groups")
        _req(x_scales.numel() == n_groups * nhg * ndg, "number of x scales must equal the number of groups")
        _req(B_scales.numel() == n_groups and C_scales.numel() == n_groups,
             "number of B / C scales must equal the number of SSD groups")
        hgr, dgr = hgr.contiguous(), dgr.contiguous()
    else:
        _req(hgr is None and dgr is None, "x_head_group_range and x_dim_group_range must be both None or both set")
        _req(x_scales.numel() == 1 and B_scales.numel() == 1 and C_scales.numel() == 1,
             "number of x / B / C scales must be equal to 1")
    return hgr, dgr, nhg, ndg


class quamba2_conv1d_cuda:
    @staticmethod
    def fwd(xBC, scale_x, scale_B, scale_C, x_dim, x_headdim, d_state, n_groups, x_head_group_range,
            x_dim_group_range, x_scales, B_scales, C_scales, weight, scale_wx, scale_wB, scale_wC, bias,
            scale_bx, scale_bB, scale_bC, seq_idx=None, initial_states=None, final_states_out=None,
            silu_activation=True):
        _cuda_i8(xBC, "xBC"); _cuda_i8(weight, "weight")
        batch, dim, seqlen = xBC.shape
        width = weight.shape[-1]
        _req(tuple(weight.shape) == (dim, width), "weight must have shape (dim, width)")
        _req(xBC.stride(1) == 1 and xBC.stride(2) > 1, "only support channel_last")
        if bias is not None:
            _cuda_i8(bias, "bias"); _req(tuple(bias.shape) == (dim,), "bias must have shape (dim,)")
        if seq_idx is not None:
            raise RuntimeError("No implementation for seq_idx")
        if initial_states is not None:
            raise RuntimeError("No implementation for initial_states")
        if final_states_out is not None:
            raise RuntimeError("No implementation for final_states_out")
        hgr, dgr, nhg, ndg = _q2_common(x_dim, x_headdim, d_state, n_groups, x_head_group_range, x_dim_group_range,
                                        x_scales, B_scales, C_scales)
        gn = d_state * n_groups
        x = torch.empty((batch, seqlen, x_dim), dtype=torch.int8, device=xBC.device)
        Bo = torch.empty((batch, seqlen, gn), dtype=torch.int8, device=xBC.device)
        Co = torch.empty((batch, seqlen, gn), dtype=torch.int8, device=xBC.device)
        w = weight.contiguous()
        args = _lib.make("qb_quamba2_conv1d_fwd_args", xBC=_p(xBC), x=_p(x), Bm=_p(Bo), Cm=_p(Co), weight=_p(w),
                         bias=_p(bias), head_group_range=_p(hgr), dim_group_range=_p(dgr),
                         x_scales=_p(x_scales), B_scales=_p(B_scales), C_scales=_p(C_scales),
                         xBC_sb=xBC.stride(0), xBC_sl=xBC.stride(2), batch=batch, dim=dim, seqlen=seqlen, width=width,
                         x_dim=x_dim, x_headdim=x_headdim, d_state=d_state, n_groups=n_groups, nhead_groups=nhg,
                         ndim_groups=ndg, scale_x=float(scale_x), scale_B=float(scale_B), scale_C=float(scale_C),
                         scale_wx=float(scale_wx), scale_wB=float(scale_wB), scale_wC=float(scale_wC),
                         scale_bx=float(scale_bx or 0.0), scale_bB=float(scale_bB or 0.0),
                         scale_bC=float(scale_bC or 0.0), silu=int(bool(silu_activation)))
        _run("qb_quamba2_conv1d_fwd", args, xBC)
        return [x.transpose(1, 2), Bo.transpose(1, 2), Co.transpose(1, 2)]

    @staticmethod
    def update(xBC, conv_state, scale_x, scale_B, scale_C, x_dim, x_headdim, d_state, n_groups, x_head_group_range,
               x_dim_group_range, x_scales, B_scales, C_scales, weight, scale_wx, scale_wB, scale_wC, bias,
               scale_bx, scale_bB, scale_bC, seq_idx=None, initial_states=None, final_states_out=None,
               silu_activation=True):
        _cuda_i8(xBC, "xBC"); _cuda_i8(conv_state, "conv_state"); _cuda_i8(weight, "weight")
        batch, dim = xBC.shape
        width = weight.shape[-1]
        _req(tuple(conv_state.shape) == (batch, dim, width), "conv_state must have shape (batch, dim, width)")
        _req(xBC.stride(1) == 1, "xBC must be contiguous in channels")
        hgr, dgr, nhg, ndg = _q2_common(x_dim, x_headdim, d_state, n_groups, x_head_group_range, x_dim_group_range,
                                        x_scales, B_scales, C_scales)
        gn = d_state * n_groups
        x = torch.empty((batch, x_dim), dtype=torch.int8, device=xBC.device)
        Bo = torch.empty((batch, gn), dtype=torch.int8, device=xBC.device)
        Co = torch.empty((batch, gn), dtype=torch.int8, device=xBC.device)
        w = weight.contiguous()
        args = _lib.make("qb_quamba2_conv1d_update_args", xBC=_p(xBC), conv_state=_p(conv_state), x=_p(x), Bm=_p(Bo),
                         Cm=_p(Co), weight=_p(w), bias=_p(bias), head_group_range=_p(hgr), dim_group_range=_p(dgr),
                         x_scales=_p(x_scales), B_scales=_p(B_scales), C_scales=_p(C_scales), xBC_sb=xBC.stride(0),
                         state_sb=conv_state.stride(0), state_sd=conv_state.stride(1), state_sw=conv_state.stride(2),
                         batch=batch, dim=dim, width=width, x_dim=x_dim, x_headdim=x_headdim, d_state=d_state,
                         n_groups=n_groups, nhead_groups=nhg, ndim_groups=ndg, scale_x=float(scale_x),
                         scale_B=float(scale_B), scale_C=float(scale_C), scale_wx=float(scale_wx),
                         scale_wB=float(scale_wB), scale_wC=float(scale_wC), scale_bx=float(scale_bx or 0.0),
                         scale_bB=float(scale_bB or 0.0), scale_bC=float(scale_bC or 0.0),
                         silu=int(bool(silu_activation)))
        _run("qb_quamba2_conv1d_update", args, xBC)
        return [x, Bo, Co]


# ------------------------------------------------------------------------------------------------
_IN_DTYPE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _hadamard(x, scale, special):
    _req(x.is_cuda, "x must be a CUDA tensor")
    _req(x.dtype in _IN_DTYPE, "x must be fp16, bf16 or fp32")
    shape = x.shape
    dim = shape[-1]
    x2 = x.reshape(-1, dim)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
    args = _lib.make("qb_hadamard_quant_args", x=_p(x2), out=_p(out), x_row_stride=x2.stride(0),
                     out_row_stride=out.stride(0), rows=x2.shape[0], dim=dim, special=special,
                     in_dtype=_IN_DTYPE[x.dtype], scale=float(scale))
    _run("qb_hadamard_quant", args, x)
    return out.reshape(shape)


class quant_hadamard:
    fast_hadamard_transform = staticmethod(lambda x, scale: _hadamard(x, scale, 1))
    fast_hadamard_transform_12N = staticmethod(lambda x, scale: _hadamard(x, scale, 12))
    fast_hadamard_transform_20N = staticmethod(lambda x, scale: _hadamard(x, scale, 20))
    fast_hadamard_transform_28N = staticmethod(lambda x, scale: _hadamard(x, scale, 28))
    fast_hadamard_transform_40N = staticmethod(lambda x, scale: _hadamard(x, scale, 40))


# ------------------------------------------------------------------------------------------------
class quant_sscan_cuda:
    @staticmethod
    def fwd(u, scale_u, delta, scale_delta, A, scale_A, B, scale_B, C, scale_C, scale_ssm_state, D=None,
            scale_D=None, z=None, scale_z=None, delta_bias=None, scale_delta_bias=None, delta_softplus=False):
        for t, n in ((u, "u"), (delta, "delta"), (A, "A"), (B, "B"), (C, "C")):
            _cuda_i8(t, n)
        _req(u.dim() == 3, "u must be (batch, dim, seqlen)")
        batch, dim, seqlen = u.shape
        dstate = A.shape[1]
        _req(B.dim() >= 3 and C.dim() >= 3, "Must be input-dependent B and C")
        if B.dim() == 3:
            B = B.unsqueeze(1)
        if C.dim() == 3:
            C = C.unsqueeze(1)
        n_groups = B.shape[1]
        _req(dstate <= 256, "quant_sscan only supports state dimension <= 256")
        _req(tuple(delta.shape) == (batch, dim, seqlen), "delta must have the shape of u")
        _req(tuple(A.shape) == (dim, dstate), "A must be (dim, dstate)")
        _req(tuple(B.shape) == (batch, n_groups, dstate, seqlen), "B must be (batch, n_groups, dstate, seqlen)")
        _req(tuple(C.shape) == (batch, n_groups, dstate, seqlen), "C must be (batch, n_groups, dstate, seqlen)")
        for t, n in ((u, "u"), (delta, "delta"), (B, "B"), (C, "C")):
            _req(t.stride(-1) == 1 or t.size(-1) == 1, f"{n} must be contiguous in seqlen")
        for s, n in ((scale_u, "scale_u"), (scale_delta, "scale_delta"), (scale_A, "scale_A"), (scale_B, "scale_B"),
                     (scale_C, "scale_C"), (scale_ssm_state, "scale_ssm_state")):
            _scale_t(s, n, u.device); _req(s.numel() == 1, f"{n} must have 1 element")
        if z is not None:
            _cuda_i8(z, "z"); _req(tuple(z.shape) == (batch, dim, seqlen) and z.stride(-1) == 1, "z must match u")
            _scale_t(scale_z, "scale_z", u.device)
        A = A.contiguous()
        n_chunks = (seqlen + 2047) // 2048
        out = torch.empty((batch, seqlen, dim), dtype=torch.float16, device=u.device)
        x = torch.empty((batch, dim, n_chunks, dstate), dtype=torch.int8, device=u.device)
        args = _lib.make(
            "qb_sscan_fwd_args", u=_p(u), delta=_p(delta), z=_p(z), Bm=_p(B), Cm=_p(C), A_log=_p(A),
            D=_p(D), delta_bias=_p(delta_bias), u_scale=_p(scale_u), delta_scale=_p(scale_delta),
            z_scale=_p(scale_z) if z is not None else None, B_scale=_p(scale_B), C_scale=_p(scale_C), A_scale=_p(scale_A),
            D_scale=_p(scale_D) if D is not None else None,
            delta_bias_scale=_p(scale_delta_bias) if delta_bias is not None else None,
            ssm_state_scale=_p(scale_ssm_state), out=_p(out), x_states=_p(x),
            u_sb=u.stride(0), u_sd=u.stride(1), delta_sb=delta.stride(0), delta_sd=delta.stride(1),
            z_sb=z.stride(0) if z is not None else 0, z_sd=z.stride(1) if z is not None else 0,
            B_sb=B.stride(0), B_sg=B.stride(1), B_sn=B.stride(2), C_sb=C.stride(0), C_sg=C.stride(1), C_sn=C.stride(2),
            batch=batch, dim=dim, seqlen=seqlen, dstate=dstate, n_groups=n_groups,
            delta_softplus=int(bool(delta_softplus)))
        _run("qb_sscan_fwd", args, u)
        return [out, x]


# ------------------------------------------------------------------------------------------------
# Programmatic early launch between the kernels of a fused decode step: the kernels named in the header's early_launch note
# read their producer's output past L1, so each may let its successor start while it runs.  The switch is on only inside
# QuambaMixerModel.decode_step_fused, whose launch sequence consists of exactly those kernels.
_EARLY = False


class early_dependents:
    def __enter__(self):
        global _EARLY
        self.prev, _EARLY = _EARLY, True

    def __exit__(self, *exc):
        global _EARLY
        _EARLY = self.prev


def _update(state, q_x, x_scales, hgr, dgr, q_dt, dt_scale, q_A_log, A_log_scale, ssm_state_scale, q_B, B_scale,
            q_C, C_scale, q_D, D_scale, q_z, z_scale, dt_bias, dt_bias_scale, dt_softplus, grouped):
    has_heads = state.dim() > 3
    if state.dim() == 3:
        state = state.unsqueeze(1)
    if q_x.dim() == 2:
        q_x = q_x.unsqueeze(1)
    if q_dt.dim() == 2:
        q_dt = q_dt.unsqueeze(1)
    if q_A_log.dim() == 2:
        q_A_log = q_A_log.unsqueeze(0)
    if q_B.dim() == 2:
        q_B = q_B.unsqueeze(1)
    if q_C.dim() == 2:
        q_C = q_C.unsqueeze(1)
    if q_D is not None and q_D.dim() == 1:
        q_D = q_D.unsqueeze(0)
    if q_z is not None and q_z.dim() == 2:
        q_z = q_z.unsqueeze(1)
    if dt_bias is not None and dt_bias.dim() == 1:
        dt_bias = dt_bias.unsqueeze(0)
    ngroups = q_B.shape[1]
    batch, nheads, dim, dstate = state.shape
    _req(q_x.is_cuda, "q_x must be a CUDA tensor")
    _req(tuple(q_x.shape) == (batch, nheads, dim), "q_x must have shape (batch, nheads, dim)")
    _req(q_dt.shape == q_x.shape, "q_dt must have the shape of q_x")
    _req(tuple(q_A_log.shape) == (nheads, dim, dstate), "q_A_log must have shape (nheads, dim, dstate)")
    _req(nheads % ngroups == 0, "nheads must be divisible by ngroups")
    _req(tuple(q_B.shape) == (batch, ngroups, dstate) and q_C.shape == q_B.shape, "q_B / q_C must be (batch, ngroups, dstate)")
    _req(state.stride(-1) == 1 and q_x.stride(-1) == 1 and q_B.stride(-1) == 1 and q_C.stride(-1) == 1,
         "state, x, B, C must be contiguous in their last dim")
    if grouped:
        _req(x_scales.numel() == ngroups * hgr.shape[1] * dgr.shape[2], "x_scales must be [G, HG, DG]")
        _req(B_scale.numel() == ngroups and C_scale.numel() == ngroups, "B / C scales must be [G]")
    else:
        _req(B_scale.numel() == 1 and C_scale.numel() == 1, "B / C scales must have 1 element")
    if q_D is not None:
        _req(tuple(q_D.shape) == (nheads, dim), "q_D must have shape (nheads, dim)")
    if q_z is not None:
        _req(q_z.shape == q_x.shape and q_z.stride(-1) == 1, "q_z must have the shape of q_x")
    bias_is_half = 0
    if dt_bias is not None:
        _req(tuple(dt_bias.shape) == (nheads, dim), "dt_bias must have shape (nheads, dim)")
        if dt_bias.dtype == torch.int8:
            _req(dt_bias_scale is not None, "int8 dt_bias needs dt_bias_scale")
        else:
            _req(dt_bias.dtype == torch.float16, "dt_bias must be int8 (with a scale) or float16")
            bias_is_half = 1
    out = torch.empty(q_x.shape, dtype=torch.float16, device=q_x.device)
    args = _lib.make(
        "qb_sscan_update_args", state=_p(state), x=_p(q_x), dt=_p(q_dt), A_log=_p(q_A_log), Bm=_p(q_B), Cm=_p(q_C),
        D=_p(q_D), z=_p(q_z), dt_bias=_p(dt_bias), x_scales=_p(x_scales), dt_scale=_p(dt_scale),
        A_scale=_p(A_log_scale), state_scale=_p(ssm_state_scale), B_scale=_p(B_scale), C_scale=_p(C_scale),
        D_scale=_p(D_scale) if q_D is not None else None, z_scale=_p(z_scale) if q_z is not None else None,
        dt_bias_scale=_p(dt_bias_scale) if (dt_bias is not None and not bias_is_half) else None,
        head_group_range=_p(hgr), dim_group_range=_p(dgr), out=_p(out),
        state_sb=state.stride(0), state_sh=state.stride(1), state_sp=state.stride(2),
        x_sb=q_x.stride(0), x_sh=q_x.stride(1), dt_sb=q_dt.stride(0), dt_sh=q_dt.stride(1), dt_sp=q_dt.stride(2),
        A_sh=q_A_log.stride(0), A_sp=q_A_log.stride(1), A_sn=q_A_log.stride(2),
        B_sb=q_B.stride(0), B_sg=q_B.stride(1), C_sb=q_C.stride(0), C_sg=q_C.stride(1),
        D_sh=q_D.stride(0) if q_D is not None else 0, D_sp=q_D.stride(1) if q_D is not None else 0,
        z_sb=q_z.stride(0) if q_z is not None else 0, z_sh=q_z.stride(1) if q_z is not None else 0,
        bias_sh=dt_bias.stride(0) if dt_bias is not None else 0, bias_sp=dt_bias.stride(1) if dt_bias is not None else 0,
        out_sb=out.stride(0), out_sh=out.stride(1), batch=batch, nheads=nheads, headdim=dim, dstate=dstate,
        ngroups=ngroups, grouped=int(grouped), nhead_groups=hgr.shape[1] if grouped else 0,
        ndim_groups=dgr.shape[2] if grouped else 0, dt_bias_is_half=bias_is_half, dt_softplus=int(bool(dt_softplus)),
        early_launch=int(_EARLY))
    _run("qb_sscan_update", args, q_x)
    return out if has_heads else out.squeeze(1)


def quant_sscan_update_triton(state, q_x, x_scale, q_dt, dt_scale, q_A_log, A_log_scale, ssm_state_scale, q_B, B_scale,
                              q_C, C_scale, q_D=None, D_scale=None, q_z=None, z_scale=None, dt_bias=None,
                              dt_bias_scale=None, dt_softplus=False):
    """state int8 (batch, dim, dstate) or (batch, nheads, dim, dstate), updated in place; returns out fp16."""
    return _update(state, q_x, x_scale, None, None, q_dt, dt_scale, q_A_log, A_log_scale, ssm_state_scale, q_B, B_scale,
                   q_C, C_scale, q_D, D_scale, q_z, z_scale, dt_bias, dt_bias_scale, dt_softplus, grouped=False)


def quamba2_sscan_update_triton(state, q_x, x_scales, x_head_group_range, x_dim_group_range, q_dt, dt_scale, q_A_log,
                                A_log_scale, ssm_state_scale, q_B, B_scale, q_C, C_scale, q_D=None, D_scale=None,
                                q_z=None, z_scale=None, dt_bias=None, dt_softplus=False):
    """Grouped-scale variant: x_scales [G,HG,DG], ssm_state_scale [G,HG,DG,N], B/C scales [G]."""
    _req(x_head_group_range.dtype == torch.int32 and x_dim_group_range.dtype == torch.int32, "group ranges must be int32")
    return _update(state, q_x, x_scales, x_head_group_range.contiguous(), x_dim_group_range.contiguous(), q_dt, dt_scale,
                   q_A_log, A_log_scale, ssm_state_scale.contiguous(), q_B, B_scale, q_C, C_scale, q_D, D_scale, q_z,
                   z_scale, dt_bias, None, dt_softplus, grouped=True)


# ------------------------------------------------------------------------------------------------
def _ssd(q_x, x_scales, hgr, dgr, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale, ssm_state_scale,
         chunk_size, q_D, D_scale, q_z, z_scale, dt_bias, initial_states, seq_idx, cu_seqlens, dt_softplus, dt_limit,
         grouped):
    batch, seqlen, nheads, headdim = q_x.shape
    _, _, ngroups, dstate = q_B.shape
    _req(nheads % ngroups == 0, "nheads must be divisible by ngroups")
    for t, n in ((q_x, "q_x"), (q_B, "q_B"), (q_dt, "q_dt"), (q_A_log, "q_A_log"), (q_C, "q_C")):
        _cuda_i8(t, n)
    _req(tuple(q_B.shape) == (batch, seqlen, ngroups, dstate) and q_C.shape == q_B.shape, "q_B / q_C shape mismatch")
    _req(tuple(q_dt.shape) == (batch, seqlen, nheads), "q_dt must be (batch, seqlen, nheads)")
    _req(tuple(q_A_log.shape) == (nheads,), "q_A_log must be (nheads,)")
    if initial_states is not None:
        raise NotImplementedError("Only supports initial_states=None")
    if seq_idx is not None:
        raise NotImplementedError("Only supports seq_idx=None")
    if cu_seqlens is not None:
        raise NotImplementedError("Only supports `cu_seqlens=None`")
    if q_B.stride(-1) != 1:
        q_B = q_B.contiguous()
    if q_C.stride(-1) != 1:
        q_C = q_C.contiguous()
    if q_x.stride(-1) != 1:
        q_x = q_x.contiguous()
    if q_dt.stride(-1) != 1:
        q_dt = q_dt.contiguous()
    if q_z is not None:
        _req(q_z.shape == q_x.shape, "q_z must have the shape of q_x")
        if q_z.stride(-1) != 1:
            q_z = q_z.contiguous()
    d_has_hdim = 0
    if q_D is not None:
        _req(tuple(q_D.shape) in ((nheads, headdim), (nheads,)), "q_D must be (nheads, headdim) or (nheads,)")
        d_has_hdim = int(q_D.dim() == 2)
        q_D = q_D.contiguous()
    if dt_bias is not None:
        _req(tuple(dt_bias.shape) == (nheads,), "dt_bias must be (nheads,)")
        dt_bias = dt_bias.to(torch.float16).contiguous()
    if grouped:
        _req(x_scales.numel() == ngroups * hgr.shape[1] * dgr.shape[2], "x_scales must be [G, HG, DG]")
        _req(B_scale.numel() == ngroups and C_scale.numel() == ngroups, "B / C scales must be [G]")
        _req(tuple(ssm_state_scale.shape) == (ngroups, hgr.shape[1], dgr.shape[2], dstate),
             "ssm_state_scale must be [G, HG, DG, N]")
    else:
        _req(x_scales.numel() == 1 and B_scale.numel() == 1 and C_scale.numel() == 1, "scales must have 1 element")
    out = torch.empty((batch, seqlen, nheads, headdim), dtype=torch.float16, device=q_x.device)
    final_states = torch.empty((batch, nheads, headdim, dstate), dtype=torch.int8, device=q_x.device)
    ws_bytes = _lib.lib().qb_ssd_workspace_bytes(batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size)
    _req(ws_bytes > 0, "invalid SSD shape")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q_x.device)
    args = _lib.make(
        "qb_ssd_args", x=_p(q_x), dt=_p(q_dt), Bm=_p(q_B), Cm=_p(q_C), A_log=_p(q_A_log), D=_p(q_D), z=_p(q_z),
        dt_bias=_p(dt_bias), x_scales=_p(x_scales), dt_scale=_p(dt_scale), A_scale=_p(A_log_scale), B_scale=_p(B_scale),
        C_scale=_p(C_scale), D_scale=_p(D_scale) if q_D is not None else None,
        z_scale=_p(z_scale) if q_z is not None else None, ssm_state_scale=_p(ssm_state_scale),
        head_group_range=_p(hgr), dim_group_range=_p(dgr), out=_p(out), final_states=_p(final_states),
        workspace=_p(ws), workspace_bytes=ws_bytes,
        x_sb=q_x.stride(0), x_sl=q_x.stride(1), x_sh=q_x.stride(2), dt_sb=q_dt.stride(0), dt_sl=q_dt.stride(1),
        B_sb=q_B.stride(0), B_sl=q_B.stride(1), B_sg=q_B.stride(2), C_sb=q_C.stride(0), C_sl=q_C.stride(1),
        C_sg=q_C.stride(2), z_sb=q_z.stride(0) if q_z is not None else 0, z_sl=q_z.stride(1) if q_z is not None else 0,
        z_sh=q_z.stride(2) if q_z is not None else 0, batch=batch, seqlen=seqlen, nheads=nheads, headdim=headdim,
        ngroups=ngroups, dstate=dstate, chunk_size=chunk_size, grouped=int(grouped),
        nhead_groups=hgr.shape[1] if grouped else 0, ndim_groups=dgr.shape[2] if grouped else 0,
        D_has_hdim=d_has_hdim, dt_softplus=int(bool(dt_softplus)), dt_min=float(dt_limit[0]),
        dt_max=float(min(dt_limit[1], 3.0e38)))
    _run("qb_ssd_chunk_scan_fwd", args, q_x)
    return out, final_states


def _quant_mamba_chunk_scan_combined_fwd(q_x, x_scale, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale,
                                         ssm_state_scale, chunk_size, q_D=None, D_scale=None, q_z=None, z_scale=None,
                                         dt_bias=None, initial_states=None, seq_idx=None, cu_seqlens=None,
                                         dt_softplus=False, dt_limit=(0.0, float("inf")), mm_dtype=torch.float16):
    return _ssd(q_x, x_scale, None, None, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale,
                ssm_state_scale, chunk_size, q_D, D_scale, q_z, z_scale, dt_bias, initial_states, seq_idx, cu_seqlens,
                dt_softplus, dt_limit, grouped=False)


def _quamba2_mamba_chunk_scan_combined_fwd(q_x, x_scales, x_head_group_range, x_dim_group_range, q_dt, dt_scale,
                                           q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale, ssm_state_scale,
                                           chunk_size, q_D=None, D_scale=None, q_z=None, z_scale=None, dt_bias=None,
                                           initial_states=None, seq_idx=None, cu_seqlens=None, dt_softplus=False,
                                           dt_limit=(0.0, float("inf")), mm_dtype=torch.float16):
    _req(x_head_group_range.dim() == 2, "x_head_group_range must have shape [n_ssd_group, x_nhead_group]")
    _req(x_dim_group_range.dim() == 3, "x_dim_group_range must have shape [n_ssd_group, x_nhead_group, n_dim_group]")
    _req(x_head_group_range.dtype == torch.int32 and x_dim_group_range.dtype == torch.int32, "group ranges must be int32")
    return _ssd(q_x, x_scales, x_head_group_range.contiguous(), x_dim_group_range.contiguous(), q_dt, dt_scale, q_A_log,
                A_log_scale, q_B, B_scale, q_C, C_scale, ssm_state_scale.contiguous(), chunk_size, q_D, D_scale, q_z,
                z_scale, dt_bias, initial_states, seq_idx, cu_seqlens, dt_softplus, dt_limit, grouped=True)


# ------------------------------------------------------------------------------------------------
class W4A8Prepared:
    """The streaming copies of one Marlin-QQQ packed weight, owned by whoever prepared it (a linear module keeps
    one; nothing global holds it).  ``sc`` fp32 (N) channel scales in natural order; ``w8`` int8 (N, K) the values
    the reference kernel multiplies with; ``w4`` uint8 (N, K / 2) nibble copy of a per-channel weight for
    decode-sized calls.  ``w8`` and ``w4`` are built on first use and can be dropped with :meth:`release`."""

    def __init__(self, b_q_weight, s_ch, s_group, size_n, size_k):
        _req(b_q_weight.is_cuda and b_q_weight.dtype == torch.int32, "b_q_weight must be an int32 CUDA tensor")
        _req(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_size = 16")
        _req(b_q_weight.shape[0] == size_k // 16, "Shape mismatch: b_q_weight.size(0) != size_k / tile_size")
        _req(b_q_weight.shape[1] == size_n * 2, "Shape mismatch: b_q_weight.size(1) != size_n * tile_size / pack_factor")
        _req(s_ch.numel() == size_n, f"Shape mismatch: s_ch.numel() = {s_ch.numel()}, size_n = {size_n}")
        self.per_channel = s_group.numel() == 0
        self.group = -1 if self.per_channel else size_k // s_group.shape[0]
        _req(self.group in (-1, 128), f"Unexpected groupsize = {self.group}")
        if not self.per_channel:
            _req(s_group.dtype == torch.float16 and s_group.shape[1] == size_n, "s_group must be fp16 (K/128, N)")
        # weak references: the prepared copies must not keep a deleted layer's buffers alive
        self._src = tuple(weakref.ref(t) for t in (b_q_weight, s_ch, s_group))
        self.size_n, self.size_k = size_n, size_k
        self.versions = (b_q_weight._version, s_ch._version, s_group._version)
        self.w8 = self.w4 = self.sc = self.w4g = self.sg_nat = None

    def stale(self, b_q_weight, s_ch, s_group):
        live = tuple(r() for r in self._src)
        return (live[0] is not b_q_weight or live[1] is not s_ch or live[2] is not s_group
                or self.versions != (b_q_weight._version, s_ch._version, s_group._version))

    def _unpack(self):
        packed, s_ch, s_group = (r() for r in self._src)
        _req(packed is not None and s_ch is not None and s_group is not None, "the packed weight was freed")
        dev = packed.device
        w8 = torch.empty((self.size_n, self.size_k), dtype=torch.int8, device=dev)
        sc = torch.empty((self.size_n,), dtype=torch.float32, device=dev)
        args = _lib.make("qb_w4a8_unpack_args", packed=_p(packed.contiguous()),
                         s_group=None if self.per_channel else _p(s_group.contiguous()),
                         s_channel=_p(s_ch.contiguous().float()), w8=_p(w8), s_channel_nat=_p(sc),
                         size_k=self.size_k, size_n=self.size_n, group_size=self.group if self.group > 0 else self.size_k)
        _run("qb_w4a8_unpack", args, packed)
        return w8, sc

    def need_w8(self):
        if self.w8 is None:
            self.w8, self.sc = self._unpack()
        return self.w8

    def need_w4(self):
        """Nibble copy (per-channel weights only); the int8 expansion it is built from is not kept unless it
        already exists."""
        if self.w4 is None:
            w8 = self.w8
            if w8 is None:
                w8, self.sc = self._unpack()
            w4 = torch.empty((self.size_n, self.size_k // 2), dtype=torch.uint8, device=w8.device)
            with torch.cuda.device(w8.device):
                f = _lib.lib().qb_w4a8_pack_nibbles
                f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
                _lib.check(f(w8.data_ptr(), w4.data_ptr(), self.size_n, self.size_k, ctypes.c_void_p(_stream(w8))))
            self.w4 = w4
        return self.w4

    def need_w4g(self):
        """Group-128 weights as the decode kernels stream them: (codes, scales) with ``codes`` uint8 (N, K / 2), the raw
        4-bit codes in the nibble layout of :meth:`need_w4` (byte b of 32-bit word i of a row: k = 8 i + b low, k = 8 i + 4 + b
        high), and ``scales`` fp16 (N, K / 128), the group scales in natural order.  Built once, from the packed buffer."""
        if self.w4g is None:
            from . import packing
            packed, s_ch, s_group = (r() for r in self._src)
            _req(packed is not None and s_ch is not None and s_group is not None, "the packed weight was freed")
            _req(not self.per_channel, "need_w4g is for group-quantised weights")
            q = packing.unpack_int4(packed, self.size_k, self.size_n, False)                 # (K, N) codes 0..15
            sg, sc = packing.unpermute_scales(s_group, s_ch, self.size_n, False)             # (K / 128, N), (1, N)
            qt = q.t().contiguous().to(torch.uint8).view(self.size_n, self.size_k // 8, 2, 4)
            self.w4g = (qt[:, :, 0, :] | (qt[:, :, 1, :] << 4)).reshape(self.size_n, self.size_k // 2).contiguous()
            self.sg_nat = sg.t().contiguous().to(torch.float16)
            if self.sc is None:
                self.sc = sc.reshape(-1).float().contiguous()
        return self.w4g, self.sg_nat

    def release(self, w8=True, w4=True):
        if w8:
            self.w8 = None
        if w4:
            self.w4 = self.w4g = self.sg_nat = None

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w8, self.w4, self.sc, self.w4g, self.sg_nat) if t is not None)


def prepare_w4a8_weight(b_q_weight, s_ch, s_group, size_n, size_k):
    """Wrap a Marlin-QQQ packed weight for the B200 kernels.  The caller owns the result (and with it the
    streaming copies); nothing is cached globally."""
    return W4A8Prepared(b_q_weight, s_ch, s_group, size_n, size_k)


# Extension-level calls receive raw tensors on every call.  Their prepared copies are remembered per weight
# OBJECT (id of the packed tensor, checked against a weak reference, dropped by a finalizer when the tensor
# dies), so an address re-used by the allocator can never hit another weight's entry.
_W4A8_BY_ID = {}


def _prepared_for(b_q_weight, s_ch, s_group, size_n, size_k):
    key = id(b_q_weight)
    hit = _W4A8_BY_ID.get(key)
    if hit is not None and not hit.stale(b_q_weight, s_ch, s_group) and (hit.size_n, hit.size_k) == (size_n, size_k):
        return hit
    prep = W4A8Prepared(b_q_weight, s_ch, s_group, size_n, size_k)
    _W4A8_BY_ID[key] = prep
    weakref.finalize(b_q_weight, _W4A8_BY_ID.pop, key, None)
    return prep


def _w4a8(a, prep, s_tok, size_m, size_n, size_k, output_transpose, out_int8):
    _cuda_i8(a, "a")
    _req(a.dim() == 2 and a.stride(1) == 1, "a must be a row-major (m, k) matrix")
    _req(size_m == a.shape[0], f"Shape mismatch: a.size(0) = {a.shape[0]}, size_m = {size_m}")
    _req(size_k == a.shape[1], f"Shape mismatch: a.size(1) = {a.shape[1]}, size_k = {size_k}")
    _req(s_tok.numel() in (1, size_m), f"s_tok.numel() = {s_tok.numel()} is not 1 or equal to size_m = {size_m}")
    _scale_t(s_tok, "s_tok", a.device)
    dt = torch.int8 if out_int8 else torch.float16
    shape = (size_n, size_m) if output_transpose else (size_m, size_n)
    out = torch.empty(shape, dtype=dt, device=a.device)
    if size_m == 0:
        return out
    common = dict(s_tok=_p(s_tok), out=_p(out), a_row_stride=a.stride(0), out_row_stride=out.stride(0), m=size_m, n=size_n,
                  k=size_k, s_tok_per_row=int(s_tok.numel() != 1), out_int8=int(out_int8),
                  output_transpose=int(bool(output_transpose)))
    if (0 < size_m <= 8 and prep.per_channel and size_k % 32 == 0 and a.stride(0) % 16 == 0 and a.data_ptr() % 16 == 0):
        # a few rows on per-channel weights: stream the nibble copy (half the bytes, identical results); from nine rows on
        # the tensor-core kernel on the int8 copy is faster than re-streaming the weights for every eight rows
        w4 = prep.need_w4()
        args = _lib.make("qb_w4a8_gemv_s4_args", a=_p(a), w4=_p(w4), s_channel_nat=_p(prep.sc), **common)
        _run("qb_w4a8_gemv_s4", args, a)
        return out
    w8 = prep.need_w8()
    args = _lib.make("qb_w4a8_gemm_args", a=_p(a), w8=_p(w8), s_channel_nat=_p(prep.sc), **common)
    _run("qb_w4a8_gemm", args, a)
    return out


def w4a8_linear(a, prep, s_tok, output_transpose=False, out_int8=False):
    """The W4A8 product on a weight prepared once with :func:`prepare_w4a8_weight` (what the linear modules call)."""
    return _w4a8(a, prep, s_tok, a.shape[0], prep.size_n, prep.size_k, output_transpose, out_int8)


_OUT_DTYPE = {torch.int8: 0, torch.float16: 1, torch.bfloat16: 2}


class quant_linear_cuda:
    @staticmethod
    def w4a8o16_gemm(a, b_q_weight, s_tok, s_ch, s_group, workspace, size_m, size_n, size_k, output_transpose=False):
        prep = _prepared_for(b_q_weight, s_ch, s_group, size_n, size_k)
        return _w4a8(a, prep, s_tok, size_m, size_n, size_k, output_transpose, False)

    @staticmethod
    def w4a8o8_gemm(a, b_q_weight, s_tok, s_ch, s_group, workspace, size_m, size_n, size_k, output_transpose=False):
        prep = _prepared_for(b_q_weight, s_ch, s_group, size_n, size_k)
        return _w4a8(a, prep, s_tok, size_m, size_n, size_k, output_transpose, True)

    @staticmethod
    def cutlass_scaled_mm_dq(c, a, b, a_scales, b_scales):
        """c (M,N) = cvt(a_scales * (b_scales * (a (M,K) @ b (K,N)))), a row-major, b column-major."""
        _cuda_i8(a, "a"); _cuda_i8(b, "b")
        _req(a.dim() == 2 and b.dim() == 2 and c.dim() == 2, "a, b, c must be matrices")
        _req(c.shape[0] == a.shape[0] and a.shape[1] == b.shape[0] and b.shape[1] == c.shape[1], "shape mismatch")
        _req(a_scales.numel() in (1, a.shape[0]) and b_scales.numel() in (1, b.shape[1]), "scale shape mismatch")
        _req(a.stride(1) == 1 and c.stride(1) == 1, "a and c must be row-major")
        _req(b.stride(0) == 1, "b must be column-major")
        _req(c.stride(0) % 16 == 0 and b.stride(1) % 16 == 0, "16 byte alignment of c rows and b columns")
        _req(c.dtype in _OUT_DTYPE, "unsupported output type")
        _scale_t(a_scales, "a_scales", a.device); _scale_t(b_scales, "b_scales", a.device)
        _req(a_scales.is_contiguous() and b_scales.is_contiguous(), "scales must be contiguous")
        m, k = a.shape
        n = b.shape[1]
        args = _lib.make("qb_w8a8_gemm_args", a=_p(a), b=_p(b), a_scale=_p(a_scales), b_scale=_p(b_scales), out=_p(c),
                         a_row_stride=a.stride(0), b_col_stride=b.stride(1), out_row_stride=c.stride(0), m=m, n=n, k=k,
                         a_scale_per_row=int(a_scales.numel() != 1), b_scale_per_col=int(b_scales.numel() != 1),
                         out_dtype=_OUT_DTYPE[c.dtype], use_alpha=0, round_half_away=0, alpha=0.0)
        _run("qb_w8a8_gemm", args, a)

    @staticmethod
    def cutlass_scaled_mv_dq(c, a, b, alpha, beta):
        """c (1,N) = cvt(alpha * (a (N,K) @ b (1,K)^T)); beta must be 0 (the reference never passes another value)."""
        _cuda_i8(a, "a"); _cuda_i8(b, "b")
        _req(a.dim() == 2 and b.dim() == 2 and c.dim() == 2, "a, b, c must be matrices")
        _req(c.shape[0] == b.shape[0] and a.shape[1] == b.shape[1] and a.shape[0] == c.shape[1], "shape mismatch")
        _req(a.stride(1) == 1 and b.stride(1) == 1 and c.stride(1) == 1, "a, b, c must be row-major")
        _req(float(beta) == 0.0, "beta != 0 is not supported")
        _req(c.dtype in _OUT_DTYPE, "unsupported output type")
        n, k = a.shape
        args = _lib.make("qb_w8a8_gemm_args", a=_p(b), b=_p(a), a_scale=None, b_scale=None, out=_p(c),
                         a_row_stride=b.stride(0), b_col_stride=a.stride(0), out_row_stride=c.stride(0), m=b.shape[0],
                         n=n, k=k, a_scale_per_row=0, b_scale_per_col=0, out_dtype=_OUT_DTYPE[c.dtype], use_alpha=1,
                         round_half_away=0, alpha=float(alpha))
        _run("qb_w8a8_gemm", args, a)

    @staticmethod
    def w8a8o8_gemv(c, a, b, scale_a, scale_b):
        """c (1,N) int8 = clamp(roundf(scale_a[n] * scale_b * (a (N,K) @ b (1,K)^T)))."""
        _cuda_i8(a, "a"); _cuda_i8(b, "b"); _cuda_i8(c, "c")
        n, k = a.shape
        _req(scale_a.numel() == n, f"Shape mismatch: scale_a.numel() = {scale_a.numel()}, size_n = {n}")
        _req(scale_b.numel() == 1, f"Shape mismatch: scale_b.numel() = {scale_b.numel()}")
        _req(c.shape[0] == b.shape[0] and a.shape[1] == b.shape[1] and a.shape[0] == c.shape[1], "shape mismatch")
        _req(a.stride(1) == 1 and b.stride(1) == 1 and c.stride(1) == 1, "a, b, c must be row-major")
        args = _lib.make("qb_w8a8_gemm_args", a=_p(b), b=_p(a), a_scale=_p(scale_b), b_scale=_p(scale_a.contiguous()),
                         out=_p(c), a_row_stride=b.stride(0), b_col_stride=a.stride(0), out_row_stride=c.stride(0),
                         m=b.shape[0], n=n, k=k, a_scale_per_row=0, b_scale_per_col=1, out_dtype=0, use_alpha=0,
                         round_half_away=1, alpha=0.0)
        _run("qb_w8a8_gemm", args, a)
        return c


# ------------------------------------------------------------------------------------------------
def _norm_call(fn, x, weight, bias, eps, residual, residual_out, q_z, z_scale, out, dyn, group_size, ngroups, out_kind,
               out_scale, norm_before_gate, is_rms_norm, partials=None):
    extra = {}
    if partials is not None:          # (n, stride in elements, index of the partial read from ``own``, own or None)
        n_p, stride_p, own_i, own = partials
        extra = dict(n_partials=n_p, partial_stride=stride_p, own_index=own_i if own is not None else -1, own_partial=_p(own))
    args = _lib.make(
        "qb_rmsnorm_args", x=_p(x), residual=_p(residual), residual_out=_p(residual_out), z=_p(q_z), weight=_p(weight),
        bias=_p(bias), out=_p(out), dyn_scale=_p(dyn), x_row_stride=x.stride(0),
        residual_row_stride=residual.stride(0) if residual is not None else 0,
        residual_out_row_stride=residual_out.stride(0) if residual_out is not None else 0,
        z_row_stride=q_z.stride(0) if q_z is not None else 0, out_row_stride=out.stride(0), rows=x.shape[0],
        group_size=group_size, ngroups=ngroups,
        residual_is_f32=int(residual is not None and residual.dtype == torch.float32),
        residual_out_is_f32=int(residual_out is not None and residual_out.dtype == torch.float32), out_kind=out_kind,
        norm_before_gate=int(bool(norm_before_gate)), is_rms_norm=int(bool(is_rms_norm)), eps=float(eps),
        out_scale=float(out_scale), z_scale=float(z_scale), **extra)
    _run(fn, args, x)


def _qlayer_norm_fwd(x, weight, bias, eps, residual=None, static_out_scale=None, residual_dtype=None, is_rms_norm=False,
                     partials=None, out=None):
    """quamba/triton/quant_norm.py:134-206: returns (y int8, residual_out, per_token_scale or None).  ``partials`` (not in
    the reference): (slots, own_index, own) with slots fp16 (n, M, N) -- the input is then the fp16-rounded fp32 sum of
    the n slots, slot ``own_index`` read from the (M, N) tensor ``own`` when that is given; ``x`` must be ``slots[0]``."""
    if partials is not None:
        slots, own_i, own = partials
        _req(slots.dim() == 3 and slots.dtype == torch.float16 and slots[0].is_contiguous() and x.data_ptr() == slots.data_ptr(),
             "partials: fp16 (n, M, N) slots with contiguous rows, x = slots[0]")
        _req(own is None or (own.shape == x.shape and own.dtype == torch.float16 and own.stride() == x.stride()),
             "partials: own piece must have the shape and strides of a slot")
        partials = (slots.shape[0], slots.stride(0), own_i, own)
    _req(x.is_cuda and x.dtype == torch.float16 and x.dim() == 2, "x must be a 2-D float16 CUDA tensor")
    _req(x.stride(-1) == 1, "x must be contiguous in its last dim")
    M, N = x.shape
    _req(tuple(weight.shape) == (N,) and weight.stride(-1) == 1 and weight.dtype == torch.float16, "weight must be fp16 (N,)")
    if bias is not None:
        _req(tuple(bias.shape) == (N,) and bias.stride(-1) == 1 and bias.dtype == torch.float16, "bias must be fp16 (N,)")
    if residual is not None:
        _req(residual.shape == x.shape and residual.stride(-1) == 1, "residual must have the shape of x")
        _req(residual.dtype in (torch.float16, torch.float32), "residual must be float16 or float32")
        residual_dtype = residual.dtype
    _req(N * x.element_size() < 65536, "This layer norm doesn't support feature dim >= 64KB.")
    if out is not None:               # not in the reference: the int8 rows land in a caller's buffer (rows contiguous)
        _req(out.dtype == torch.int8 and tuple(out.shape) == (M, N) and out.stride(-1) == 1 and out.device == x.device,
             "out must be an int8 (M, N) tensor on x's device, contiguous in its last dim")
    y = out if out is not None else torch.empty((M, N), dtype=torch.int8, device=x.device)
    residual_out = None
    if residual is not None or (residual_dtype is not None and residual_dtype != x.dtype):
        _req(residual_dtype in (torch.float16, torch.float32), "residual_dtype must be float16 or float32")
        residual_out = torch.empty((M, N), dtype=residual_dtype, device=x.device)
    static = bool(static_out_scale)       # the reference tests truthiness: None and 0.0 both mean per-token scales
    dyn = None if static else torch.empty((M,), dtype=torch.float32, device=x.device)
    if M > 0:
        _norm_call("qb_rmsnorm_quant", x, weight, bias, eps, residual, residual_out, None, 0.0, y, dyn, N, 1,
                   0 if static else 1, static_out_scale if static else 0.0, True, is_rms_norm, partials=partials)
    return y, (residual_out if residual_out is not None else x), dyn


def _qlayer_normgated_fwd(x, weight, bias, eps, q_z=None, z_scale=None, static_out_scale=None, use_float16_output=False,
                          group_size=None, norm_before_gate=True, is_rms_norm=False):
    """quamba/triton/quant_normgated.py:85-132: returns (out fp16 or int8, per_token_scale (ngroups * M))."""
    _req(x.is_cuda and x.dtype == torch.float16 and x.dim() == 2, "x must be a 2-D float16 CUDA tensor")
    _req(x.stride(-1) == 1, "x must be contiguous in its last dim")
    M, N = x.shape
    group_size = N if group_size is None else group_size
    _req(N % group_size == 0, "the feature dim must be divisible by group_size")
    ngroups = N // group_size
    if q_z is not None:
        _cuda_i8(q_z, "q_z")
        _req(q_z.shape == x.shape and q_z.stride(-1) == 1, "q_z must have the shape of x")
        _req(z_scale is not None, "q_z needs z_scale")
    _req(tuple(weight.shape) == (N,) and weight.stride(-1) == 1 and weight.dtype == torch.float16, "weight must be fp16 (N,)")
    if bias is not None:
        _req(tuple(bias.shape) == (N,) and bias.stride(-1) == 1 and bias.dtype == torch.float16, "bias must be fp16 (N,)")
    _req(group_size * x.element_size() < 65536, "This layer norm doesn't support feature dim >= 64KB.")
    out = torch.empty((M, N), dtype=torch.float16 if use_float16_output else torch.int8, device=x.device)
    per_token = torch.empty((ngroups * M,), dtype=torch.float32, device=x.device)
    kind = 2 if use_float16_output else (0 if static_out_scale is not None else 1)
    if M > 0:
        _norm_call("qb_rmsnorm_gated", x, weight, bias, eps, None, None, q_z, z_scale or 0.0, out, per_token, group_size,
                   ngroups, kind, static_out_scale if kind == 0 else 0.0, norm_before_gate, is_rms_norm)
    return out, per_token


class quant_embedding_cuda:
    """csrc/embedding/quant_embedding.cpp: w4a16_embedding_lookup / w8a16_embedding_lookup (+ the fp16 table)."""

    @staticmethod
    def _lookup(input, weight, scale, kind, dim):
        _req(weight.dim() == 2 and weight.is_cuda, "weight must be a 2-D CUDA tensor")
        _req(input.dim() in (1, 2), "input must be a 1D or 2D tensor")
        _req(input.is_cuda and input.dtype == torch.int64, "input must be an int64 CUDA tensor")
        vocab = weight.shape[0]
        if kind:
            _req(scale.dim() == 1 and scale.is_cuda and scale.dtype == torch.float16 and scale.numel() == vocab,
                 "scale must be a float16 CUDA tensor with one entry per row")
        tokens = input.contiguous()
        out = torch.empty((*tokens.shape, dim), dtype=torch.float16, device=input.device)
        args = _lib.make("qb_embedding_args", table=_p(weight.contiguous()), scales=_p(scale) if kind else None,
                         tokens=_p(tokens), out=_p(out), n_tokens=tokens.numel(), dim=dim, vocab=vocab, kind=kind)
        _run("qb_embedding_lookup", args, input)
        return out

    @staticmethod
    def w4a16_embedding_lookup(input, weight, scale):
        _req(weight.dtype == torch.int32, "weight's dtype must be int32")
        return quant_embedding_cuda._lookup(input, weight, scale, 2, weight.shape[1] * 8)

    @staticmethod
    def w8a16_embedding_lookup(input, weight, scale):
        _req(weight.dtype == torch.int8, "weight's dtype must be int8")
        return quant_embedding_cuda._lookup(input, weight, scale, 1, weight.shape[1])

    @staticmethod
    def f16_embedding_lookup(input, weight):
        _req(weight.dtype == torch.float16, "weight's dtype must be float16")
        return quant_embedding_cuda._lookup(input, weight, None, 0, weight.shape[1])


def greedy_next_token(logits, out=None):
    """Row-wise argmax of fp16 logits (rows, vocab) -> int64 (rows); ``out`` lets a captured step write in place."""
    _req(logits.is_cuda and logits.dtype == torch.float16 and logits.dim() == 2 and logits.stride(1) == 1,
         "logits must be a 2-D float16 CUDA tensor, contiguous in its last dim")
    rows, n = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int64, device=logits.device)
    _req(out.dtype == torch.int64 and out.numel() == rows and out.is_contiguous(), "out must be int64 (rows,)")
    f = _lib.lib().qb_argmax_rows
    f.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    with torch.cuda.device(logits.device):
        _lib.check(f(logits.data_ptr(), logits.stride(0), rows, n, out.data_ptr(), ctypes.c_void_p(_stream(logits))))
    return out


# ------------------------------------------------------------------------------------------------
# Fused decode-step launches (1 to 4 rows).  ``prep`` is a W4A8Prepared; per-channel weights stream their nibble copy.
def _decode_weight(prep):
    """(weight copy, w_is_s4, group scales or None) for the decode kernels: nibbles for both weight formats."""
    if prep.per_channel and prep.size_k % 32 == 0:
        return prep.need_w4(), 1, None
    if not prep.per_channel and prep.size_k % 128 == 0 and GROUP_NIBBLES:
        w, sg = prep.need_w4g()
        return w, 1, sg
    return prep.need_w8(), 0, None


# Group-128 weights at decode: True streams the 4-bit codes + group scales and rebuilds the int8 weights in registers
# (half the bytes, bit-identical results, no int8 copy needed by a decode-only deployment); False streams the int8
# expansion.  Measured on the 2.7B model (batch 1): 1.86 ms per token from the codes against 1.53 ms from the expansion
# -- the decode step is bound by latency, not by bytes, and the ~2.4 instructions per weight of the fp16 rebuild sit on the
# critical path -- so the expansion is the default.
GROUP_NIBBLES = False


def decode_norm_linear(x, residual, norm_weight, eps, norm_out_scale, prep, s_tok, out_int8, residual_in_fp32=True, conv=None):
    """residual add + RMSNorm + quantise + W4A8 product for (rows, k) fp16 ``x``.  Returns (out (rows, n) int8 or fp16,
    residual_out).  ``conv``: dict(state, weight, bias, col0, x_dim, gn, scale_in, scale_bias, out_scales) runs the conv1d
    decode step on columns [col0, col0 + x_dim + 2 gn) in the epilogue and adds ``x``, ``B``, ``C`` int8 outputs to it."""
    rows, k = x.shape
    w, s4, sg = _decode_weight(prep)
    dt = torch.int8 if out_int8 else torch.float16
    out = torch.empty((rows, prep.size_n), dtype=dt, device=x.device)
    res_dtype = residual.dtype if residual is not None else (torch.float32 if residual_in_fp32 else torch.float16)
    residual_out = torch.empty((rows, k), dtype=res_dtype, device=x.device)
    kw = {}
    if conv is not None:
        st = conv["state"]
        conv["x"] = torch.empty((rows, conv["x_dim"]), dtype=torch.int8, device=x.device)
        conv["B"] = torch.empty((rows, conv["gn"]), dtype=torch.int8, device=x.device)
        conv["C"] = torch.empty((rows, conv["gn"]), dtype=torch.int8, device=x.device)
        so = conv["out_scales"]
        kw = dict(conv_state=_p(st), conv_weight=_p(conv["weight"]), conv_bias=_p(conv["bias"]), conv_x=_p(conv["x"]),
                  conv_B=_p(conv["B"]), conv_C=_p(conv["C"]), x_out_scale=_p(so[0]), B_out_scale=_p(so[1]), C_out_scale=_p(so[2]),
                  conv_state_sb=st.stride(0), conv_state_sd=st.stride(1), conv_state_sw=st.stride(2), conv_col0=conv["col0"],
                  conv_dim=conv["x_dim"] + 2 * conv["gn"], conv_x_dim=conv["x_dim"], conv_gn=conv["gn"],
                  conv_scale_in_x=conv["scale_in"][0], conv_scale_in_B=conv["scale_in"][1], conv_scale_in_C=conv["scale_in"][2],
                  conv_scale_bias_x=conv["scale_bias"][0], conv_scale_bias_B=conv["scale_bias"][1],
                  conv_scale_bias_C=conv["scale_bias"][2])
    args = _lib.make("qb_decode_norm_linear_args", x=_p(x), residual=_p(residual), residual_out=_p(residual_out),
                     norm_weight=_p(norm_weight), w=_p(w), s_channel_nat=_p(prep.sc), s_group_nat=_p(sg), s_tok=_p(s_tok), out=_p(out),
                     x_row_stride=x.stride(0), residual_row_stride=residual.stride(0) if residual is not None else 0,
                     residual_out_row_stride=residual_out.stride(0), out_row_stride=out.stride(0), rows=rows, n=prep.size_n,
                     k=k, w_is_s4=s4, out_int8=int(out_int8), residual_is_f32=int(residual is not None and residual.dtype == torch.float32),
                     residual_out_is_f32=int(res_dtype == torch.float32), eps=float(eps), norm_out_scale=float(norm_out_scale),
                     early_launch=int(_EARLY), **kw)
    _run("qb_decode_norm_linear", args, x)
    return out, residual_out


def decode_linear(a, prep, s_tok, out_int8=False):
    """Decode-sized W4A8 product of int8 rows ``a`` (1 to 4 rows) on the low-latency kernel: (rows, n) fp16 or int8."""
    rows, k = a.shape
    w, s4, sg = _decode_weight(prep)
    out = torch.empty((rows, prep.size_n), dtype=torch.int8 if out_int8 else torch.float16, device=a.device)
    args = _lib.make("qb_decode_norm_linear_args", a_int8=_p(a), w=_p(w), s_channel_nat=_p(prep.sc), s_group_nat=_p(sg), s_tok=_p(s_tok), out=_p(out),
                     x_row_stride=a.stride(0), out_row_stride=out.stride(0), rows=rows, n=prep.size_n, k=k, w_is_s4=s4,
                     out_int8=int(out_int8), early_launch=int(_EARLY))
    _run("qb_decode_norm_linear", args, a)
    return out


def decode_gate_had_quant(y, z, z_scale, norm_weight, eps, group_size, had_scale):
    """y (rows, d) fp16, z (rows, d) int8 (a strided view is fine) -> gate, grouped RMSNorm, Hadamard rotation, int8:
    QRMSNormGated (fp16 output) followed by QHadamard in one launch.  Returns (rows, d) int8."""
    rows, d = y.shape
    out = torch.empty((rows, d), dtype=torch.int8, device=y.device)
    args = _lib.make("qb_decode_gate_had_quant_args", y=_p(y), z=_p(z), norm_weight=_p(norm_weight), out=_p(out),
                     y_row_stride=y.stride(0), z_row_stride=z.stride(0), out_row_stride=out.stride(0), rows=rows, d=d,
                     group_size=group_size, z_scale=float(z_scale), eps=float(eps), had_scale=float(had_scale),
                     early_launch=int(_EARLY))
    _run("qb_decode_gate_had_quant", args, y)
    return out
