#!/usr/bin/env python
"""Generate tests/golden/ssd_*.npz by running the REFERENCE's own Triton SSD kernels on CPU.

Run in a container where the reference checkout is mounted:

    TRITON_INTERPRET=1 python tests/golden/make_ssd_golden.py /path/to/reference

The reference's Python wrappers insist on CUDA tensors, so the @triton.jit functions
underneath the autotuner are launched directly (``kernel.fn[grid](...)``) with explicit
block sizes, in Triton interpreter mode, with the argument order of the wrappers in
quamba/triton/quant_{chunk_cumsum,chunk_state,state_passing,bmm_chunk,chunk_scan}.py.
``mamba_ssm.ops.triton.softplus`` (un-vendored third party) is replaced by a stub whose
arithmetic is the one the reference's CUDA twin states (x <= 20 ? log1p(exp(x)) : x,
csrc/selective_scan/quant_sscan_fwd_kernel.cuh:159-161).
The final-state int8 quantisation kernel uses libdevice.rint, which the interpreter
cannot run; its fp16 input (the final state) is stored instead.
"""
import math
import os
import sys
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch
import triton
import triton.language as tl

if len(sys.argv) < 2:
    raise SystemExit("usage: %s <path to the reference checkout>" % sys.argv[0])
REF = Path(sys.argv[1])
OUT = Path(__file__).resolve().parent


@triton.jit
def _softplus_stub(dt):
    return tl.where(dt <= 20.0, tl.log(tl.exp(dt) + 1.0), dt)


def _install_stubs():
    m = types.ModuleType("mamba_ssm")
    ops = types.ModuleType("mamba_ssm.ops")
    tr = types.ModuleType("mamba_ssm.ops.triton")
    sp = types.ModuleType("mamba_ssm.ops.triton.softplus")
    sp.softplus = _softplus_stub
    sys.modules.update({"mamba_ssm": m, "mamba_ssm.ops": ops, "mamba_ssm.ops.triton": tr,
                        "mamba_ssm.ops.triton.softplus": sp})


def _load(name):
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_" + name, REF / "quamba" / "triton" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def q8(x):
    s = x.abs().amax().clamp(min=1e-5) / 127
    return torch.clamp(torch.round(x / s), -128, 127).to(torch.int8), s.float().reshape(1)


def run_case(tag, Bsz, L, H, P, G, N, Q, grouped, seed, slim=False):
    torch.manual_seed(seed)
    cum, cst, spz, bmm, csc = (_load(n) for n in ("quant_chunk_cumsum", "quant_chunk_state", "quant_state_passing",
                                                   "quant_bmm_chunk", "quant_chunk_scan"))
    nc = math.ceil(L / Q)
    x = torch.randn(Bsz, L, H, P)
    dt_raw = torch.randn(Bsz, L, H)
    dt0 = torch.rand(H) * (0.1 - 0.001) + 0.001
    dt_bias = (dt0 + torch.log(-torch.expm1(-dt0))).to(torch.float16)
    A_log = torch.log(torch.rand(H) * 15 + 1)
    Bm = torch.randn(Bsz, L, G, N)
    Cm = torch.randn(Bsz, L, G, N)
    D = 1 + 0.1 * torch.randn(H)
    q_dt, s_dt = q8(dt_raw)
    q_A, s_A = q8(A_log)
    q_D, s_D = q8(D)
    if grouped:
        HG, DG = 2, 2
        hpg = H // G
        hgr = torch.tensor([[hpg // 2, hpg]] * G, dtype=torch.int32)
        dgr = torch.tensor([[[P // 2, P]] * HG] * G, dtype=torch.int32)
        xs = torch.empty(G, HG, DG)
        q_x = torch.empty(Bsz, L, H, P, dtype=torch.int8)
        xv = x.reshape(Bsz, L, G, hpg, P)
        for g in range(G):
            for hg in range(HG):
                for dg in range(DG):
                    h0, h1 = hg * hpg // 2, (hg + 1) * hpg // 2
                    d0, d1 = dg * P // 2, (dg + 1) * P // 2
                    blk = xv[:, :, g, h0:h1, d0:d1]
                    qq, ss = q8(blk)
                    xs[g, hg, dg] = ss
                    q_x.view(Bsz, L, G, hpg, P)[:, :, g, h0:h1, d0:d1] = qq
        q_B = torch.empty(Bsz, L, G, N, dtype=torch.int8)
        q_C = torch.empty(Bsz, L, G, N, dtype=torch.int8)
        s_B = torch.empty(G)
        s_C = torch.empty(G)
        for g in range(G):
            q_B[:, :, g], sb = q8(Bm[:, :, g])
            q_C[:, :, g], sc = q8(Cm[:, :, g])
            s_B[g], s_C[g] = sb, sc
    else:
        hgr = dgr = None
        q_x, xs = q8(x)
        q_B, s_B = q8(Bm)
        q_C, s_C = q8(Cm)

    # T1 cumsum (quant_chunk_cumsum.py:73-93)
    dt_out = torch.empty(Bsz, H, nc, Q)
    dA_cs = torch.empty(Bsz, H, nc, Q)
    BH = 2
    cum._quant_chunk_cumsum_fwd_kernel.fn[(Bsz, nc, triton.cdiv(H, BH))](
        q_dt, s_dt, q_A, s_A, dt_bias, dt_out, dA_cs, Bsz, L, H, Q, 0.0, float("inf"),
        q_dt.stride(0), q_dt.stride(1), q_dt.stride(2), q_A.stride(0), dt_bias.stride(0),
        dt_out.stride(0), dt_out.stride(2), dt_out.stride(1), dt_out.stride(3),
        dA_cs.stride(0), dA_cs.stride(2), dA_cs.stride(1), dA_cs.stride(3),
        True, HAS_DT_BIAS=True, BLOCK_SIZE_H=BH, BLOCK_SIZE_CHUNK=triton.next_power_of_2(Q))

    # T2 chunk state (quant_chunk_state.py:106-147 / :265-330)
    states = torch.empty(Bsz, nc, H, P, N)
    BM, BN, BK = 32, 32, 32
    grid = (triton.cdiv(P, BM) * triton.cdiv(N, BN), Bsz * nc, H)
    common = (P, N, Q, Bsz, L, H // G,
              q_x.stride(0), q_x.stride(1), q_x.stride(2), q_x.stride(3),
              q_B.stride(0), q_B.stride(1), q_B.stride(2), q_B.stride(3),
              states.stride(0), states.stride(1), states.stride(2), states.stride(3), states.stride(4),
              dt_out.stride(0), dt_out.stride(2), dt_out.stride(1), dt_out.stride(3),
              dA_cs.stride(0), dA_cs.stride(2), dA_cs.stride(1), dA_cs.stride(3), 0, 0)
    if grouped:
        cst._quamba2_chunk_state_fwd_kernel.fn[grid](
            q_x, xs, hgr, dgr, q_B, s_B, states, dt_out, dA_cs, None, *common,
            nhead_groups=2, ndim_groups=2, USE_FLOA32_MM=False, HAS_SEQ_IDX=False,
            BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK)
    else:
        cst._quant_chunk_state_fwd_kernel.fn[grid](
            q_x, xs, q_B, s_B, states, dt_out, dA_cs, None, *common,
            USE_FLOA32_MM=False, HAS_SEQ_IDX=False, BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK)

    # T3 state passing (quant_state_passing.py:86-115), carried states stored fp16
    dim = P * N
    st_flat = states.reshape(Bsz, nc, H, dim)
    dA_last = dA_cs[:, :, :, -1]
    prev = torch.empty(Bsz, nc, H, dim, dtype=torch.float16)
    final = torch.empty(Bsz, H, dim, dtype=torch.float16)
    BS = 256
    spz._quant_state_passing_fwd_kernel.fn[(triton.cdiv(dim, BS), Bsz, H)](
        st_flat, prev, final, dA_last, None, None, dim, nc, 0, 0,
        st_flat.stride(0), st_flat.stride(1), st_flat.stride(2), st_flat.stride(3),
        prev.stride(0), prev.stride(1), prev.stride(2), prev.stride(3),
        final.stride(0), final.stride(1), final.stride(2),
        dA_last.stride(0), dA_last.stride(2), dA_last.stride(1), 0, 0, 0, 0, 0,
        HAS_INITSTATES=False, HAS_SEQ_IDX=False, BLOCK_SIZE=BS)
    prev5 = prev.reshape(Bsz, nc, H, P, N)

    # T4 C B^T (quant_bmm_chunk.py:82-137 / :209-260), fp32 dot
    CB = torch.empty(Bsz, nc, G, Q, Q)
    grid = (triton.cdiv(Q, BM) * triton.cdiv(Q, BN), Bsz, nc * G)
    kern = bmm._quamba2_bmm_chunk_fwd_kernel if grouped else bmm._quant_bmm_chunk_fwd_kernel
    kern.fn[grid](
        q_C, s_C, q_B, s_B, CB, None, L, Q, N, G,
        q_C.stride(0), q_C.stride(1), q_C.stride(2), q_C.stride(3),
        q_B.stride(0), q_B.stride(1), q_B.stride(2), q_B.stride(3),
        CB.stride(0), CB.stride(1), CB.stride(2), CB.stride(3), CB.stride(4), 0, 0,
        False, tl.float32, HAS_SEQ_IDX=False, BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK)

    # T5 chunk scan (quant_chunk_scan.py:174-233 / :419-494)
    out = torch.empty(Bsz, L, H, P, dtype=torch.float16)
    grid = (triton.cdiv(Q, BM) * triton.cdiv(P, BN), Bsz * nc, H)
    tail = (Q, P, N, Bsz, L, H // G,
            CB.stride(0), CB.stride(1), CB.stride(2), CB.stride(3), CB.stride(4),
            q_x.stride(0), q_x.stride(1), q_x.stride(2), q_x.stride(3), 0, 0, 0, 0,
            out.stride(0), out.stride(1), out.stride(2), out.stride(3),
            dt_out.stride(0), dt_out.stride(2), dt_out.stride(1), dt_out.stride(3),
            dA_cs.stride(0), dA_cs.stride(2), dA_cs.stride(1), dA_cs.stride(3), 0, 0,
            q_C.stride(0), q_C.stride(1), q_C.stride(2), q_C.stride(3),
            prev5.stride(0), prev5.stride(1), prev5.stride(2), prev5.stride(3), prev5.stride(4),
            q_D.stride(0))
    meta = dict(IS_CAUSAL=True, HAS_D=True, D_HAS_HDIM=False, HAS_Z=False, HAS_SEQ_IDX=False,
                USE_FLOA32_MM=False, BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK,
                BLOCK_SIZE_DSTATE=max(triton.next_power_of_2(N), 16), IS_TRITON_22=True)
    if grouped:
        csc._quamba2_chunk_scan_fwd_kernel.fn[grid](
            CB, q_x, xs, hgr, dgr, None, None, out, None, dt_out, dA_cs, None, q_C, s_C, prev5, q_D, s_D,
            *tail, nhead_groups=2, ndim_groups=2, **meta)
    else:
        csc._quant_chunk_scan_fwd_kernel.fn[grid](
            CB, q_x, xs, None, None, out, None, dt_out, dA_cs, None, q_C, s_C, prev5, q_D, s_D,
            *tail, **meta)

    save = dict(q_x=q_x, x_scales=xs, q_dt=q_dt, s_dt=s_dt, q_A_log=q_A, s_A=s_A, q_B=q_B, s_B=s_B, q_C=q_C,
                s_C=s_C, q_D=q_D, s_D=s_D, dt_bias=dt_bias, chunk=torch.tensor(Q),
                ref_dt=dt_out, ref_dA_cs=dA_cs, ref_states=states, ref_prev_states=prev5,
                ref_final_f16=final.reshape(Bsz, H, P, N), ref_CB=CB, ref_out=out)
    if grouped:
        save.update(head_group_range=hgr, dim_group_range=dgr)
    if slim:        # keep the fixture small: inputs, the cumulative sums, the outputs
        for k in ("ref_states", "ref_prev_states", "ref_CB"):
            save.pop(k)
    np.savez_compressed(OUT / f"ssd_{tag}.npz", **{k: v.numpy() for k, v in save.items()})
    print("wrote", OUT / f"ssd_{tag}.npz")


if __name__ == "__main__":
    _install_stubs()
    run_case("pertensor", Bsz=2, L=96, H=4, P=64, G=1, N=64, Q=64, grouped=False, seed=0)
    run_case("grouped", Bsz=1, L=128, H=8, P=64, G=2, N=64, Q=64, grouped=True, seed=1)
    # headdim 64, d_state 128, chunk 256: the shape family the tensor-core SSD kernel serves (ragged length: 300 = 256 + 44)
    # (three chunks, five 128-token blocks, ragged tail: 600 = 256 + 256 + 88)
    run_case("n128", Bsz=1, L=600, H=2, P=64, G=1, N=128, Q=256, grouped=False, seed=2, slim=True)
