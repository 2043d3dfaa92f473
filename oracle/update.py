"""CPU restatement of the single-step (decode) state update (test infrastructure only).

Pinned against the reference's pure-torch ``selective_state_update_ref``
(quamba/triton/selective_state_update.py:481-542) on dequantised inputs; the
int8 state requantisation follows the Triton kernels.

Follows
  quamba/triton/selective_state_update.py:83-126   (Mamba1 / per-tensor scales)
  quamba/triton/selective_state_update.py:303-362  (Quamba2: grouped x scales, [G,HG,DG,N] state scales)
"""
import torch

from .quant import softplus_ref, to_int8_rne, expand_x_scales, expand_state_scales


def sscan_update(state_q, q_x, x_scale_hp, q_dt, s_dt, q_A_log, s_A, state_scale_hpn,
                 q_B, s_B_g, q_C, s_C_g, q_D=None, s_D=None, q_z=None, s_z=None,
                 dt_bias=None, s_dt_bias=None, dt_softplus=True, requant_mult=1e2):
    """Generic form.  state_q int8 (B, H, P, N) updated IN PLACE.
    q_x (B,H,P) int8 with per-channel scale x_scale_hp (H,P); q_dt int8 broadcastable to (B,H,P);
    q_A_log int8 broadcastable to (H,P,N); q_B,q_C int8 (B,G,N) with per-group scales (G,);
    q_D int8 broadcastable to (H,P); dt_bias broadcastable to (H,P): int8 with s_dt_bias, or
    float (added unscaled) when s_dt_bias is None.  Returns out fp16 (B,H,P) and the
    un-requantised fp32 state."""
    f = lambda v: torch.as_tensor(v, dtype=torch.float32)
    Bsz, H, P, N = state_q.shape
    G = q_B.shape[1]
    x = x_scale_hp.float()[None] * q_x.float()
    state = state_scale_hpn.float()[None] * state_q.float()
    dt = f(s_dt) * q_dt.float().expand(Bsz, H, P)
    if dt_bias is not None:
        if s_dt_bias is not None:
            dt = dt + (f(s_dt_bias) * dt_bias.float()).expand(H, P)[None]
        else:
            dt = dt + dt_bias.float().expand(H, P)[None]
    if dt_softplus:
        dt = softplus_ref(dt)
    A = -torch.exp(f(s_A) * q_A_log.float().expand(H, P, N))
    dA = torch.exp(A[None] * dt[..., None])
    Bv = (f(s_B_g).reshape(-1, 1) * q_B.float()).repeat_interleave(H // G, dim=1)   # (B,H,N)
    Cv = (f(s_C_g).reshape(-1, 1) * q_C.float()).repeat_interleave(H // G, dim=1)
    dB = Bv[:, :, None, :] * dt[..., None]
    state = state * dA + dB * x[..., None]
    m = torch.tensor(requant_mult, dtype=torch.float32)
    state_q.copy_(to_int8_rne((state * m) / (state_scale_hpn.float()[None] * m)))
    out = (state * Cv[:, :, None, :]).sum(-1)
    if q_D is not None:
        out = out + x * (f(s_D) * q_D.float().expand(H, P))[None]
    if q_z is not None:
        z = f(s_z) * q_z.float()
        out = out * z * torch.sigmoid(z)
    return out.to(torch.float16), state


def quant_sscan_update(state_q, q_x, s_x, q_dt, s_dt, q_A_log, s_A, s_state, q_B, s_B, q_C, s_C,
                       q_D=None, s_D=None, q_z=None, s_z=None, dt_bias=None, s_dt_bias=None,
                       dt_softplus=True):
    """Per-tensor-scale variant (quant_sscan_update_triton).  Accepts the Mamba1 shapes
    (state (B,D,N), x (B,D), A_log (D,N), B/C (B,N), D (D)) or the headed ones."""
    has_heads = state_q.dim() == 4
    st = state_q if has_heads else state_q.unsqueeze(1)
    x = q_x if has_heads else q_x.unsqueeze(1)
    dt = q_dt if has_heads else q_dt.unsqueeze(1)
    A = q_A_log if has_heads else q_A_log.unsqueeze(0)
    Bq = q_B if q_B.dim() == 3 else q_B.unsqueeze(1)
    Cq = q_C if q_C.dim() == 3 else q_C.unsqueeze(1)
    Dq = None if q_D is None else (q_D if q_D.dim() == 2 else q_D.unsqueeze(0))
    z = None if q_z is None else (q_z if has_heads else q_z.unsqueeze(1))
    bias = None if dt_bias is None else (dt_bias if dt_bias.dim() == 2 else dt_bias.unsqueeze(0))
    Bsz, H, P, N = st.shape
    G = Bq.shape[1]
    f = lambda v: torch.as_tensor(v, dtype=torch.float32).reshape(-1)[0]
    out, state = sscan_update(
        st, x, f(s_x).expand(H, P), dt, s_dt, A, s_A, f(s_state).expand(H, P, N),
        Bq, f(s_B).expand(G), Cq, f(s_C).expand(G), Dq, s_D, z, s_z, bias, s_dt_bias, dt_softplus, 1e2)
    return (out if has_heads else out.squeeze(1)), state


def quamba2_sscan_update(state_q, q_x, x_scales, head_group_range, dim_group_range, q_dt, s_dt,
                         q_A_log, s_A, state_scale, q_B, s_B, q_C, s_C, q_D=None, s_D=None,
                         q_z=None, s_z=None, dt_bias=None, dt_softplus=True):
    """Grouped variant (quamba2_sscan_update_triton): state (B,H,P,N), x (B,H,P), dt (B,H,P) (tied
    across P), A_log (H,P,N) tied, B/C (B,G,N), scales x [G,HG,DG], state [G,HG,DG,N], B/C [G]."""
    Bsz, H, P, N = state_q.shape
    G = q_B.shape[1]
    xs = expand_x_scales(x_scales, head_group_range, dim_group_range, H, P, G)
    ss = expand_state_scales(state_scale, head_group_range, dim_group_range, H, P, G, N)
    return sscan_update(state_q, q_x, xs, q_dt, s_dt, q_A_log, s_A, ss, q_B, s_B.reshape(-1), q_C,
                        s_C.reshape(-1), q_D, s_D, q_z, s_z, dt_bias, None, dt_softplus, 1e6)
