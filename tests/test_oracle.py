"""CPU tests: the oracle against the committed golden vectors and its own invariants."""
import math

import pytest
import torch

from oracle import conv1d as oconv, hadamard as ohad, linear as olin, quant as oq, ssd as ossd, sscan as osscan, update as oupd
from helpers import load_golden, make_conv2_case, make_ssd_case, make_sscan_case, q8


# ---- SSD: faithful oracle vs the reference's Triton kernels (interpreter-mode golden) -------------
@pytest.mark.parametrize("tag", ["pertensor", "grouped", "n128"])
def test_ssd_oracle_matches_reference_triton(tag):
    g = load_golden(f"ssd_{tag}.npz")
    hgr, dgr = g.get("head_group_range"), g.get("dim_group_range")
    G, N = g["q_B"].shape[2:]
    ss = torch.ones(1) if hgr is None else torch.ones(G, 2, 2, N)
    y, _, im = ossd.chunk_scan_faithful(g["q_x"], g["x_scales"], hgr, dgr, g["q_dt"], g["s_dt"], g["q_A_log"], g["s_A"],
                                        g["q_B"], g["s_B"], g["q_C"], g["s_C"], ss, int(g["chunk"]), g["q_D"], g["s_D"],
                                        None, None, g["dt_bias"], True, return_intermediates=True)
    assert torch.allclose(im["dt"].permute(0, 3, 1, 2), g["ref_dt"], atol=1e-6)
    assert torch.allclose(im["dA_cs"].permute(0, 3, 1, 2), g["ref_dA_cs"], rtol=1e-6, atol=1e-4)
    if "ref_states" in g:       # the d_state-128 fixture stores inputs, cumulative sums and outputs only
        assert torch.allclose(im["states"], g["ref_states"], rtol=1e-4, atol=1e-4)
        assert torch.allclose(im["prev_states"], g["ref_prev_states"].float(), rtol=2e-3, atol=2e-4)
        assert torch.allclose(im["CB"], g["ref_CB"], rtol=1e-5, atol=1e-4)
    assert torch.allclose(im["final_f16"], g["ref_final_f16"].float(), rtol=2e-3, atol=2e-4)
    assert torch.allclose(y.float(), g["ref_out"].float(), rtol=2e-3, atol=4e-3)


@pytest.mark.parametrize("tag", ["pertensor", "grouped", "n128"])
def test_ssd_ideal_recurrence_agrees_with_reference(tag):
    g = load_golden(f"ssd_{tag}.npz")
    hgr, dgr = g.get("head_group_range"), g.get("dim_group_range")
    yi, hi = ossd.chunk_scan_ideal(g["q_x"], g["x_scales"], hgr, dgr, g["q_dt"], g["s_dt"], g["q_A_log"], g["s_A"],
                                   g["q_B"], g["s_B"], g["q_C"], g["s_C"], g["q_D"], g["s_D"], None, None, g["dt_bias"], True)
    # fp16 tolerance: 1e-2 relative + 1e-3 of the output's largest magnitude absolute
    ref = g["ref_out"].float()
    assert ((yi.float() - ref).abs() <= 1e-3 * ref.abs().max() + 1e-2 * ref.abs()).all()
    assert torch.allclose(hi.float(), g["ref_final_f16"].float(), rtol=1e-2, atol=2e-3)


def test_ssd_ragged_and_z_chunked_equals_sequential():
    c = make_ssd_case(2, 200, 4, 64, 2, 64, 64, grouped=True, seed=3, with_z=True, d_has_hdim=True)
    y, fq = ossd.chunk_scan_faithful(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"],
                                     c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["state_scale"], 64, c["q_D"], c["s_D"],
                                     c["q_z"], c["s_z"], c["dt_bias"], True)
    yi, hi = ossd.chunk_scan_ideal(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"],
                                   c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["q_D"], c["s_D"], c["q_z"], c["s_z"], c["dt_bias"], True)
    ref = yi.float()
    assert ((y.float() - ref).abs() <= 1e-3 * ref.abs().max() + 1e-2 * ref.abs()).all()
    ss = oq.expand_state_scales(c["state_scale"], c["hgr"], c["dgr"], 4, 64, 2, 64)
    want = torch.clamp(hi.float() / ss[None], -128, 127)
    assert ((fq.float() - want).abs() <= 1.0 + 1e-2 * want.abs()).all()


# ---- W4A8: the checker's inverse of the reference packer ------------------------------------------
@pytest.mark.parametrize("tag", ["g128", "g128_pad", "perchannel"])
def test_linear_unpack_matches_reference_packer(tag):
    g = load_golden(f"linear_w4a8_{tag}.npz")
    K, N0 = g["w"].shape
    pad = int(g["pad_out"])
    N = N0 + pad
    per_channel = int(g["group"]) == -1
    q = olin.unpack_weight(g["packed"], K, N, per_channel)
    qw = torch.nn.functional.pad(g["q_w"].long(), (0, pad))
    assert torch.equal(q, qw)
    sg, sc = olin.unpermute_scales(g["s_group"], g["s_channel"].float(), N, per_channel)
    sc_raw = g["s_channel_raw"].reshape(-1).float()
    if float(g["out_scale"]) > 0:
        sc_raw = sc_raw / float(g["out_scale"])
    sc_raw = torch.cat([sc_raw, torch.full((pad,), 1e-6)])
    assert torch.equal(sc, sc_raw)
    if not per_channel:
        assert torch.equal(sg, torch.nn.functional.pad(g["s_group_raw"], (0, pad)))
    w8 = olin.dequant_to_int8(q, sg, 128)
    back = sc_raw * (float(g["out_scale"]) if float(g["out_scale"]) > 0 else 1.0)
    err = ((w8.float() * back[None]) - g["w_ref"]).abs() / back[None]
    assert err[:, :N0].max() <= 1.1  # the reference's w_ref and its kernel's int8 weight differ by <= 1 step


def test_linear_epilogues():
    g = load_golden("linear_w4a8_g128.npz")
    K, N = g["w"].shape
    a, s_a = q8(torch.randn(37, K, generator=torch.Generator().manual_seed(5)))
    o16, acc = olin.w4a8_gemm(a, g["packed"], s_a, g["s_channel"], g["s_group"], N, K, out_int8=False, return_acc=True)
    want = (a.float() * s_a) @ g["w_ref"]
    assert torch.allclose(o16.float(), want, rtol=2e-2, atol=2e-2 * want.abs().max())
    o8 = olin.w4a8_gemm(a, g["packed"], s_a * 40, g["s_channel"], g["s_group"], N, K, out_int8=True)
    assert o8.dtype == torch.int8 and o8.float().abs().max() > 10
    t = olin.w4a8_gemm(a, g["packed"], s_a, g["s_channel"], g["s_group"], N, K, out_int8=False, output_transpose=True)
    assert torch.equal(t, o16.t())
    w = torch.randint(-127, 128, (K, 48), dtype=torch.int8)
    r = olin.w8a8_gemm(a, w, torch.tensor([0.01]), torch.rand(48) * 0.01, torch.int8)
    assert r.shape == (37, 48)
    v = olin.w8a8o8_gemv(w.t().contiguous(), a[:1], torch.rand(48) * 0.001, torch.tensor([0.02]))
    assert v.shape == (1, 48)


# ---- state update: against the reference's pure-torch selective_state_update_ref --------------------
def test_update_oracle_matches_reference_torch():
    g = load_golden("update_ref.npz")
    st = g["m1_state_q"].clone()
    y, s = oupd.quant_sscan_update(st, g["m1_q_x"], g["m1_s_x"], g["m1_q_dt"], g["m1_s_dt"], g["m1_q_A"], g["m1_s_A"],
                                   g["m1_s_state"], g["m1_q_B"], g["m1_s_B"], g["m1_q_C"], g["m1_s_C"], g["m1_q_D"],
                                   g["m1_s_D"], g["m1_q_z"], g["m1_s_z"], g["m1_q_bias"], g["m1_s_bias"], True)
    assert torch.allclose(s.squeeze(1), g["m1_ref_state"], atol=1e-5)
    assert torch.allclose(y.float(), g["m1_ref_y"], rtol=2e-3, atol=2e-3)
    want_q = torch.clamp(torch.round(g["m1_ref_state"] / g["m1_s_state"]), -128, 127)
    assert (st.float() - want_q).abs().max() <= 1
    st2 = g["m2_state_q"].clone()
    H, P, N = 8, 32, 64
    y2, s2 = oupd.quant_sscan_update(st2, g["m2_q_x"], g["m2_s_x"], g["m2_q_dt"][..., None].expand(2, H, P), g["m2_s_dt"],
                                     g["m2_q_A"][:, None, None].expand(H, P, N), g["m2_s_A"], g["m2_s_state"], g["m2_q_B"],
                                     g["m2_s_B"], g["m2_q_C"], g["m2_s_C"], g["m2_q_D"][:, None].expand(H, P), g["m2_s_D"],
                                     None, None, g["m2_bias"][:, None].expand(H, P), None, True)
    assert torch.allclose(s2, g["m2_ref_state"], atol=1e-5)
    assert torch.allclose(y2.float(), g["m2_ref_y"], rtol=2e-3, atol=1e-2)


# ---- conv: forward == repeated decode steps; closed form ---------------------------------------------
@pytest.mark.parametrize("grouped", [False, True])
def test_conv2_forward_equals_repeated_update(grouped):
    c = make_conv2_case(2, 11, 4, 64, 1 if not grouped else 2, 64, grouped=grouped, seed=1)
    args = (c["sx"], c["sB"], c["sC"], c["x_dim"], c["headdim"], c["d_state"], c["n_groups"], c["hgr"], c["dgr"],
            c["x_scales"], c["B_scales"], c["C_scales"], c["weight"], c["swx"], c["swB"], c["swC"], c["bias"], c["sbx"],
            c["sbB"], c["sbC"])
    x, Bm, Cm = oconv.quamba2_conv1d_fwd(c["xBC"], *args)
    state = torch.zeros(2, c["xBC"].shape[1], 4, dtype=torch.int8)
    for l in range(11):
        xs, Bs, Cs = oconv.quamba2_conv1d_update(c["xBC"][:, :, l].contiguous(), state, *args)
        assert (xs.int() - x[:, :, l].int()).abs().max() <= 1
        assert (Bs.int() - Bm[:, :, l].int()).abs().max() <= 1
        assert (Cs.int() - Cm[:, :, l].int()).abs().max() <= 1


def test_conv1_identity_kernel():
    x = torch.randint(-100, 100, (2, 8, 19), dtype=torch.int8)
    w = torch.zeros(8, 4, dtype=torch.int8); w[:, 3] = 1
    y = oconv.quant_causal_conv1d_fwd(x, 0.5, w, 1.0, 0.5, 1.0, None, silu=False)
    assert torch.equal(y, x)
    w2 = torch.zeros(8, 3, dtype=torch.int8); w2[:, 0] = 1
    y2 = oconv.quant_causal_conv1d_fwd(x, 1.0, w2, 1.0, 1.0, 1.0, None, silu=False)
    assert torch.equal(y2[:, :, 2:], x[:, :, :-2]) and (y2[:, :, :2] == 0).all()


# ---- Hadamard ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dim", [64, 1536, 2560, 3584, 5120])
def test_hadamard_matrix_is_orthogonal(dim):
    special = {1536: 12, 2560: 20, 3584: 28, 5120: 40}.get(dim)
    H = ohad.hadamard_matrix(dim, special)
    if dim <= 2560:
        assert torch.equal(H @ H.t(), dim * torch.eye(dim, dtype=torch.float64))
    else:
        v = torch.randn(3, dim, dtype=torch.float64)
        assert torch.allclose((v @ H.t()) @ H / dim, v, atol=1e-9)
    assert ohad.split_dim(5120) == (40, 128) and ohad.split_dim(1536) == (12, 128) and ohad.split_dim(8192) == (1, 8192)


def test_hadamard_quant_flags_overflow():
    x = torch.ones(1, 64) * 100
    q, ovf = ohad.quant_hadamard(x, 1.0)
    assert ovf[0, 0] and q[0, 0] == 127 and not ovf[0, 1:].any()


# ---- Mamba1 scan -----------------------------------------------------------------------------------------
def test_sscan_oracle_last_state_feeds_update():
    c = make_sscan_case(1, 32, 40, 16, seed=2)
    y, x, h = osscan.quant_sscan_fwd(c["q_u"], c["s_u"], c["q_delta"], c["s_delta"], c["q_A"], c["s_A"], c["q_B"], c["s_B"],
                                     c["q_C"], c["s_C"], c["s_state"], c["q_D"], c["s_D"], c["q_z"], c["s_z"], c["q_bias"],
                                     c["s_bias"], True)
    assert y.shape == (1, 40, 32) and x.shape == (1, 32, 1, 16)
    # scanning the first 39 steps and then taking one decode step reproduces the 40th output
    L = 39
    y39, x39, h39 = osscan.quant_sscan_fwd(c["q_u"][..., :L], c["s_u"], c["q_delta"][..., :L], c["s_delta"], c["q_A"], c["s_A"],
                                           c["q_B"][..., :L], c["s_B"], c["q_C"][..., :L], c["s_C"], c["s_state"], c["q_D"],
                                           c["s_D"], c["q_z"][..., :L], c["s_z"], c["q_bias"], c["s_bias"], True)
    assert torch.equal(y39, y[:, :L])
    fine = torch.tensor([1e-6])  # a state scale fine enough not to matter
    st = torch.zeros(1, 32, 16, dtype=torch.int8)
    out, _ = oupd.sscan_update(st.unsqueeze(1), c["q_u"][:, None, :, L], c["s_u"].expand(1, 32), c["q_delta"][:, None, :, L],
                               c["s_delta"], c["q_A"][None], c["s_A"], torch.ones(1, 32, 16), c["q_B"][:, :, :, L],
                               c["s_B"], c["q_C"][:, :, :, L], c["s_C"], c["q_D"][None], c["s_D"], c["q_z"][:, None, :, L],
                               c["s_z"], c["q_bias"][None], c["s_bias"], True)
    # with a zero int8 state the step only sees the input term; add the carried part by hand
    A = -torch.exp(c["s_A"] * c["q_A"].float())
    delta = oq.softplus_ref(c["s_delta"] * c["q_delta"][:, :, L].float() + c["s_bias"] * c["q_bias"].float())
    carried = (h39 * torch.exp(delta[..., None] * A[None]) * (c["s_C"] * c["q_C"][:, 0, :, L].float())[:, None, :]).sum(-1)
    z = c["s_z"] * c["q_z"][:, :, L].float()
    want = y[:, L].float()
    got = out.float().squeeze(1) + carried * z * torch.sigmoid(z)
    assert torch.allclose(got, want, rtol=1e-2, atol=1e-2)
