#!/usr/bin/env python
"""Generate tests/golden/update_ref.npz with the REFERENCE's pure-torch
``selective_state_update_ref`` (quamba/triton/selective_state_update.py:481-542).

    python tests/golden/make_update_golden.py /path/to/reference

The file is imported by path with a stub for the un-vendored
``mamba_ssm.ops.triton.softplus`` (only the Triton kernels in that file use it).
Inputs are seeded int8 tensors + scales; the reference is fed their dequantised
values, and its fp32 state / output are stored for one Mamba1-shaped and one
Mamba2-shaped step.
"""
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: %s <path to the reference checkout>" % sys.argv[0])
REF = Path(sys.argv[1])
OUT = Path(__file__).resolve().parent


def load_ref():
    sp = types.ModuleType("mamba_ssm.ops.triton.softplus")
    sp.softplus = lambda x: x
    for name in ("mamba_ssm", "mamba_ssm.ops", "mamba_ssm.ops.triton"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["mamba_ssm.ops.triton.softplus"] = sp
    spec = importlib.util.spec_from_file_location("ref_ssu", REF / "quamba" / "triton" / "selective_state_update.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.selective_state_update_ref


def q8(x):
    s = x.abs().amax().clamp(min=1e-5) / 127
    return torch.clamp(torch.round(x / s), -128, 127).to(torch.int8), s.float().reshape(1)


def main():
    ref = load_ref()
    out = {}
    # Mamba1 shaped: state (B, D, N)
    torch.manual_seed(0)
    Bsz, D, N = 3, 96, 16
    qs, ss = q8(torch.randn(Bsz, D, N))
    qx, sx = q8(torch.randn(Bsz, D))
    qdt, sdt = q8(torch.randn(Bsz, D))
    qz, sz = q8(torch.randn(Bsz, D))
    qB, sB = q8(torch.randn(Bsz, N))
    qC, sC = q8(torch.randn(Bsz, N))
    qA, sA = q8(torch.log(torch.arange(1, N + 1).float()).repeat(D, 1))
    qD, sD = q8(torch.ones(D) + 0.1 * torch.randn(D))
    dt0 = torch.rand(D) * 0.099 + 0.001
    qb, sb = q8(dt0 + torch.log(-torch.expm1(-dt0)))
    state = ss * qs.float()
    y = ref(state, sx * qx.float(), sdt * qdt.float(), -torch.exp(sA * qA.float()), sB * qB.float(), sC * qC.float(),
            D=sD * qD.float(), z=sz * qz.float(), dt_bias=sb * qb.float(), dt_softplus=True)
    out.update(m1_state_q=qs, m1_s_state=ss, m1_q_x=qx, m1_s_x=sx, m1_q_dt=qdt, m1_s_dt=sdt, m1_q_z=qz, m1_s_z=sz,
               m1_q_B=qB, m1_s_B=sB, m1_q_C=qC, m1_s_C=sC, m1_q_A=qA, m1_s_A=sA, m1_q_D=qD, m1_s_D=sD,
               m1_q_bias=qb, m1_s_bias=sb, m1_ref_state=state, m1_ref_y=y)
    # Mamba2 shaped: state (B, H, P, N), dt / A / bias tied across P
    torch.manual_seed(1)
    Bsz, H, P, N, G = 2, 8, 32, 64, 2
    qs, ss = q8(torch.randn(Bsz, H, P, N))
    qx, sx = q8(torch.randn(Bsz, H, P))
    qdt, sdt = q8(torch.randn(Bsz, H))
    qB, sB = q8(torch.randn(Bsz, G, N))
    qC, sC = q8(torch.randn(Bsz, G, N))
    qA, sA = q8(torch.log(torch.rand(H) * 15 + 1))
    qD, sD = q8(torch.ones(H) + 0.1 * torch.randn(H))
    dt0 = torch.rand(H) * 0.099 + 0.001
    bias = (dt0 + torch.log(-torch.expm1(-dt0))).to(torch.float16)
    state = ss * qs.float()
    A = -torch.exp(sA * qA.float())
    y = ref(state, sx * qx.float(), (sdt * qdt.float())[..., None].expand(Bsz, H, P),
            A[:, None, None].expand(H, P, N), sB * qB.float(), sC * qC.float(),
            D=(sD * qD.float())[:, None].expand(H, P), z=None,
            dt_bias=bias.float()[:, None].expand(H, P), dt_softplus=True)
    out.update(m2_state_q=qs, m2_s_state=ss, m2_q_x=qx, m2_s_x=sx, m2_q_dt=qdt, m2_s_dt=sdt,
               m2_q_B=qB, m2_s_B=sB, m2_q_C=qC, m2_s_C=sC, m2_q_A=qA, m2_s_A=sA, m2_q_D=qD, m2_s_D=sD,
               m2_bias=bias, m2_ref_state=state, m2_ref_y=y)
    np.savez_compressed(OUT / "update_ref.npz", **{k: v.numpy() for k, v in out.items()})
    print("wrote", OUT / "update_ref.npz")


if __name__ == "__main__":
    main()
