"""Seeded input generators shared by the CPU and GPU tests (shapes and value ranges of the
benchmark configurations; synthetic stand-ins for calibration data)."""
import math

import numpy as np
import torch

GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"


def q8(x):
    """Per-tensor symmetric int8: scale = max|x| / 127, round half to even, clamp."""
    s = (x.abs().amax().clamp(min=1e-5) / 127).float()
    return torch.clamp(torch.round(x / s), -128, 127).to(torch.int8), s.reshape(1)


def load_golden(name):
    return {k: torch.from_numpy(v) for k, v in np.load(GOLDEN / name).items()}


def inv_softplus(dt):
    return dt + torch.log(-torch.expm1(-dt))


def make_conv2_case(Bsz, L, H, P, G, N, W=4, grouped=False, seed=0, row_stride=None):
    """Quamba2 conv inputs: returns dict with xBC int8 channel-last view (B, C, L) etc."""
    g = torch.Generator().manual_seed(seed)
    x_dim, gn = H * P, G * N
    C = x_dim + 2 * gn
    S = row_stride or C
    buf = torch.zeros(Bsz, L, S, dtype=torch.int8)
    segs = [(0, x_dim), (x_dim, x_dim + gn), (x_dim + gn, C)]
    in_scales = []
    for a, b in segs:
        q, s = q8(torch.randn(Bsz, L, b - a, generator=g))
        buf[:, :, a:b] = q
        in_scales.append(float(s))
    w = torch.randn(C, W, generator=g) * 0.2
    bias = torch.randn(C, generator=g) * 0.02
    qw = torch.empty(C, W, dtype=torch.int8)
    qb = torch.empty(C, dtype=torch.int8)
    w_scales, b_scales = [], []
    for a, b in segs:
        q, s = q8(w[a:b]); qw[a:b] = q; w_scales.append(float(s))
        q, s = q8(bias[a:b]); qb[a:b] = q; b_scales.append(float(s))
    xBC = buf[:, :, :C].transpose(1, 2)  # (B, C, L), strides (L*S, 1, S)
    if grouped:
        hpg = H // G
        HG, DG = min(4, hpg), 4
        hgr = torch.tensor([[(i + 1) * hpg // HG for i in range(HG)]] * G, dtype=torch.int32)
        dgr = torch.tensor([[[(i + 1) * P // DG for i in range(DG)]] * HG] * G, dtype=torch.int32)
        x_scales = (torch.rand(G, HG, DG, generator=g) * 0.02 + 0.01).float()
        B_scales = (torch.rand(G, generator=g) * 0.02 + 0.01).float()
        C_scales = (torch.rand(G, generator=g) * 0.02 + 0.01).float()
    else:
        hgr = dgr = None
        x_scales = torch.tensor([0.02]); B_scales = torch.tensor([0.015]); C_scales = torch.tensor([0.017])
    return dict(xBC=xBC, sx=in_scales[0], sB=in_scales[1], sC=in_scales[2], x_dim=x_dim, headdim=P, d_state=N,
                n_groups=G, hgr=hgr, dgr=dgr, x_scales=x_scales, B_scales=B_scales, C_scales=C_scales, weight=qw,
                swx=w_scales[0], swB=w_scales[1], swC=w_scales[2], bias=qb, sbx=b_scales[0], sbB=b_scales[1],
                sbC=b_scales[2])


def make_ssd_case(Bsz, L, H, P, G, N, Q, grouped=False, seed=0, with_z=False, d_has_hdim=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Bsz, L, H, P, generator=g)
    dt0 = torch.rand(H, generator=g) * 0.099 + 0.001
    c = dict(chunk=Q)
    c["q_dt"], c["s_dt"] = q8(torch.randn(Bsz, L, H, generator=g))
    c["dt_bias"] = inv_softplus(dt0).to(torch.float16)
    c["q_A_log"], c["s_A"] = q8(torch.log(torch.rand(H, generator=g) * 15 + 1))
    Dv = 1 + 0.1 * torch.randn((H, P) if d_has_hdim else (H,), generator=g)
    c["q_D"], c["s_D"] = q8(Dv)
    Bm = torch.randn(Bsz, L, G, N, generator=g)
    Cm = torch.randn(Bsz, L, G, N, generator=g)
    if grouped:
        hpg = H // G
        HG, DG = min(4, hpg), 4
        c["hgr"] = torch.tensor([[(i + 1) * hpg // HG for i in range(HG)]] * G, dtype=torch.int32)
        c["dgr"] = torch.tensor([[[(i + 1) * P // DG for i in range(DG)]] * HG] * G, dtype=torch.int32)
        xs = torch.empty(G, HG, DG)
        qx = torch.empty(Bsz, L, H, P, dtype=torch.int8)
        xv, qv = x.view(Bsz, L, G, hpg, P), qx.view(Bsz, L, G, hpg, P)
        for gi in range(G):
            for hg in range(HG):
                for dg in range(DG):
                    hs = slice(hg * hpg // HG, (hg + 1) * hpg // HG)
                    ds = slice(dg * P // DG, (dg + 1) * P // DG)
                    qv[:, :, gi, hs, ds], s = q8(xv[:, :, gi, hs, ds])
                    xs[gi, hg, dg] = s
        c["q_x"], c["x_scales"] = qx, xs
        c["q_B"] = torch.empty(Bsz, L, G, N, dtype=torch.int8); c["q_C"] = torch.empty_like(c["q_B"])
        c["s_B"] = torch.empty(G); c["s_C"] = torch.empty(G)
        for gi in range(G):
            c["q_B"][:, :, gi], s = q8(Bm[:, :, gi]); c["s_B"][gi] = s
            c["q_C"][:, :, gi], s = q8(Cm[:, :, gi]); c["s_C"][gi] = s
        c["state_scale"] = (torch.rand(G, HG, DG, N, generator=g) * 0.01 + 0.005).float()
    else:
        c["hgr"] = c["dgr"] = None
        c["q_x"], c["x_scales"] = q8(x)
        c["q_B"], c["s_B"] = q8(Bm)
        c["q_C"], c["s_C"] = q8(Cm)
        c["state_scale"] = torch.tensor([0.01])
    if with_z:
        c["q_z"], c["s_z"] = q8(torch.randn(Bsz, L, H, P, generator=g))
    else:
        c["q_z"] = c["s_z"] = None
    return c


def make_sscan_case(Bsz, D, L, N, G=1, seed=0, with_z=True):
    """The recipe of the reference's scan test (quamba/tests/test_qsscan.py): u, z, delta_raw, B, C ~ N(0,1) -> per-tensor int8; A = -[1..N]."""
    g = torch.Generator().manual_seed(seed)
    c = {}
    c["q_u"], c["s_u"] = q8(torch.randn(Bsz, D, L, generator=g))
    c["q_delta"], c["s_delta"] = q8(torch.randn(Bsz, D, L, generator=g))
    if with_z:
        c["q_z"], c["s_z"] = q8(torch.randn(Bsz, D, L, generator=g))
    else:
        c["q_z"] = c["s_z"] = None
    c["q_B"], c["s_B"] = q8(torch.randn(Bsz, G, N, L, generator=g))
    c["q_C"], c["s_C"] = q8(torch.randn(Bsz, G, N, L, generator=g))
    dt0 = torch.rand(D, generator=g) * 0.099 + 0.001
    c["q_bias"], c["s_bias"] = q8(inv_softplus(dt0))
    c["q_A"], c["s_A"] = q8(torch.log(torch.arange(1, N + 1).float()).repeat(D, 1))
    c["q_D"], c["s_D"] = q8(torch.ones(D))
    c["s_state"] = torch.tensor([0.05])
    return c


def allclose_report(a, b, rtol, atol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    return bool(not bad.any()), f"max err {err.max().item():.4g}, violations {int(bad.sum())}/{bad.numel()}, ref max {b.abs().max().item():.4g}"
