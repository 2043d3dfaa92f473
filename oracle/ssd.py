"""CPU restatement of the Mamba2 int8 SSD chunk scan (test infrastructure only).

Pinned: ``chunk_scan_faithful`` is compared stage by stage with the reference's
own Triton kernels run in interpreter mode on CPU (fixtures in tests/golden, made
by tests/golden/make_ssd_golden.py).  ``chunk_scan_ideal`` is the plain per-token
recurrence (the role of the SSD reference) that the chunked form must agree with.

Follows
  quamba/triton/quant_chunk_cumsum.py:56-70          dt, dA cumsum
  quamba/triton/quant_chunk_state.py:74-96, :202-262 per-chunk states (fp16 operands, fp32 acc)
  quamba/triton/quant_state_passing.py:60-83         inter-chunk recurrence, fp16 storage
  quamba/triton/quant_bmm_chunk.py:60-79             C B^T per chunk
  quamba/triton/quant_chunk_scan.py:90-171, :254-414 output
  quamba/triton/quant_ssm_states.py:32-45, :90-121   final state -> int8 (rint)
  quamba/triton/quant_ssd_combined.py:61-77, :146-162 glue
"""
import math

import torch

from .quant import softplus_ref, to_int8_rne, expand_x_scales, expand_state_scales


def _h(x):
    """Round to fp16 and come back (the ``.to(mm_dtype)`` before every tl.dot)."""
    return x.to(torch.float16).float()


def _prep(q_x, x_scales, hgr, dgr, q_dt, s_dt, q_A_log, s_A, q_B, s_B, q_C, s_C, dt_bias,
          dt_softplus, dt_limit, chunk):
    f = lambda v: torch.as_tensor(v, dtype=torch.float32)
    Bsz, L, H, P = q_x.shape
    G, N = q_B.shape[2], q_B.shape[3]
    nc = math.ceil(L / chunk)
    Lp = nc * chunk
    xs = expand_x_scales(f(x_scales), hgr, dgr, H, P, G)                      # (H, P)
    dt = f(s_dt).reshape(()) * q_dt.float()                                    # (B, L, H)
    if dt_bias is not None:
        dt = dt + dt_bias.float()[None, None, :]
    if dt_softplus:
        dt = softplus_ref(dt)
    dt = torch.clamp(dt, dt_limit[0], dt_limit[1])
    dt = torch.nn.functional.pad(dt, (0, 0, 0, Lp - L))                        # zero beyond seqlen
    A = -torch.exp(f(s_A).reshape(()) * q_A_log.float())                       # (H,)
    dt = dt.reshape(Bsz, nc, chunk, H)
    dA_cs = torch.cumsum(dt * A[None, None, None, :], dim=2)                   # (B, nc, Q, H)
    pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, 0, 0, Lp - L))
    x = pad(xs[None, None] * q_x.float()).reshape(Bsz, nc, chunk, H, P)
    sB = f(s_B).reshape(-1)
    sC = f(s_C).reshape(-1)
    sB = sB.expand(G) if sB.numel() == 1 else sB
    sC = sC.expand(G) if sC.numel() == 1 else sC
    Bm = pad(sB[None, None, :, None] * q_B.float()).reshape(Bsz, nc, chunk, G, N)
    Cm = pad(sC[None, None, :, None] * q_C.float()).reshape(Bsz, nc, chunk, G, N)
    return xs, dt, A, dA_cs, x, Bm, Cm, nc, Lp


def chunk_scan_faithful(q_x, x_scales, head_group_range, dim_group_range, q_dt, s_dt, q_A_log, s_A,
                        q_B, s_B, q_C, s_C, state_scale, chunk_size, q_D=None, s_D=None,
                        q_z=None, s_z=None, dt_bias=None, dt_softplus=True,
                        dt_limit=(0.0, float("inf")), return_intermediates=False):
    """q_x int8 (B,L,H,P); q_dt int8 (B,L,H); q_B,q_C int8 (B,L,G,N); q_A_log int8 (H);
    q_D int8 (H) or (H,P); dt_bias float (H).  x_scales 1-element or [G,HG,DG]; state_scale
    1-element or [G,HG,DG,N]; s_B/s_C 1-element or [G].
    Returns y fp16 (B,L,H,P), final_states int8 (B,H,P,N) [, dict of intermediates]."""
    f = lambda v: torch.as_tensor(v, dtype=torch.float32)
    Bsz, L, H, P = q_x.shape
    G, N = q_B.shape[2], q_B.shape[3]
    Q = chunk_size
    xs, dt, A, dA_cs, x, Bm, Cm, nc, Lp = _prep(q_x, x_scales, head_group_range, dim_group_range, q_dt, s_dt,
                                                q_A_log, s_A, q_B, s_B, q_C, s_C, dt_bias, dt_softplus,
                                                dt_limit, Q)
    rep = H // G
    Bh = Bm.repeat_interleave(rep, dim=3)                                      # (B,nc,Q,H,N)
    Ch = Cm.repeat_interleave(rep, dim=3)
    # chunk states: fp16(x) . fp16(B * exp(dA_last - dA_l) * dt_l)
    w = torch.exp(dA_cs[:, :, -1:, :] - dA_cs) * dt                            # (B,nc,Q,H)
    states = torch.einsum("bclhp,bclhn->bchpn", _h(x), _h(Bh * w[..., None]))  # fp32
    # state passing (carried state stored fp16 per chunk)
    s = torch.zeros(Bsz, H, P, N)
    prev = torch.empty(Bsz, nc, H, P, N)
    for c in range(nc):
        prev[:, c] = _h(s)
        s = torch.exp(dA_cs[:, c, -1, :])[:, :, None, None] * s + states[:, c]
    final_f16 = _h(s)
    # C B^T per group
    CB = torch.einsum("bcmgn,bckgn->bcgmk", Cm, Bm)                            # (B,nc,G,Q,Q)
    CBh = CB.repeat_interleave(rep, dim=2)                                     # (B,nc,H,Q,Q)
    # output
    acc = torch.einsum("bcmhn,bchpn->bcmhp", _h(Ch), prev) * torch.exp(dA_cs)[..., None]
    dAm = dA_cs.permute(0, 1, 3, 2)                                            # (B,nc,H,Q)
    decay = torch.exp(dAm[..., :, None] - dAm[..., None, :])                   # (B,nc,H,m,k)
    Lmat = CBh * decay * dt.permute(0, 1, 3, 2)[..., None, :]
    mask = torch.tril(torch.ones(Q, Q, dtype=torch.bool))
    Lmat = torch.where(mask, Lmat, torch.zeros(()))
    acc = acc + torch.einsum("bchmk,bckhp->bcmhp", _h(Lmat), _h(x))
    if q_D is not None:
        Dv = f(s_D).reshape(()) * q_D.float()
        Dv = Dv[:, None] if Dv.dim() == 1 else Dv
        acc = acc + x * Dv[None, None, None]
    acc = acc.reshape(Bsz, Lp, H, P)[:, :L]
    out_x = acc
    if q_z is not None:
        z = f(s_z).reshape(()) * q_z.float()
        acc = acc * z * torch.sigmoid(z)
    y = acc.to(torch.float16)
    ss = expand_state_scales(f(state_scale), head_group_range, dim_group_range, H, P, G, N)
    m = torch.tensor(1e2 if head_group_range is None else 1e6)
    final_q = to_int8_rne((final_f16 * m) / (ss[None] * m))
    if return_intermediates:
        return y, final_q, dict(dt=dt, dA_cs=dA_cs, states=states, prev_states=prev, final_f16=final_f16,
                                CB=CB, out_x=out_x)
    return y, final_q


def chunk_scan_ideal(q_x, x_scales, head_group_range, dim_group_range, q_dt, s_dt, q_A_log, s_A,
                     q_B, s_B, q_C, s_C, q_D=None, s_D=None, q_z=None, s_z=None, dt_bias=None,
                     dt_softplus=True, dt_limit=(0.0, float("inf")), dtype=torch.float64):
    """Dequantise, then the plain per-token recurrence h <- exp(dt A) h + dt B x, y = C h + D x.
    Returns y (B,L,H,P) and the final state (B,H,P,N), both in ``dtype``."""
    f = lambda v: torch.as_tensor(v, dtype=torch.float32)
    Bsz, L, H, P = q_x.shape
    G, N = q_B.shape[2], q_B.shape[3]
    xs, dt, A, _, x, Bm, Cm, nc, Lp = _prep(q_x, x_scales, head_group_range, dim_group_range, q_dt, s_dt,
                                           q_A_log, s_A, q_B, s_B, q_C, s_C, dt_bias, dt_softplus,
                                           dt_limit, L)
    rep = H // G
    dt = dt.reshape(Bsz, L, H).to(dtype)
    x = x.reshape(Bsz, L, H, P).to(dtype)
    Bh = Bm.reshape(Bsz, L, G, N).repeat_interleave(rep, dim=2).to(dtype)
    Ch = Cm.reshape(Bsz, L, G, N).repeat_interleave(rep, dim=2).to(dtype)
    A = A.to(dtype)
    h = torch.zeros(Bsz, H, P, N, dtype=dtype)
    y = torch.empty(Bsz, L, H, P, dtype=dtype)
    for l in range(L):
        dA = torch.exp(dt[:, l] * A[None])                                     # (B,H)
        h = dA[:, :, None, None] * h + (dt[:, l, :, None] * x[:, l])[..., None] * Bh[:, l, :, None, :]
        y[:, l] = torch.einsum("bhpn,bhn->bhp", h, Ch[:, l])
    if q_D is not None:
        Dv = (f(s_D).reshape(()) * q_D.float()).to(dtype)
        Dv = Dv[:, None] if Dv.dim() == 1 else Dv
        y = y + x * Dv[None, None]
    if q_z is not None:
        z = (f(s_z).reshape(()) * q_z.float()).to(dtype)
        y = y * z * torch.sigmoid(z)
    return y, h
