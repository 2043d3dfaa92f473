"""Module-level mirror (quamba_b200.modules): host logic on CPU, forwards on the GPU against the oracle.

The CPU part checks what a checkpoint depends on: buffer names / shapes / dtypes, the float entries added
to the state dict, the int4 packer against vectors made with the reference's own packer, and that a state
dict round-trips.  The GPU part drives forward / update / to_seqlen_last and compares with the CPU oracle
fed with the module's own buffers."""
import pytest
import torch
import torch.nn as nn

from helpers import allclose_report, load_golden, make_conv2_case, make_ssd_case, make_sscan_case, q8
from oracle import conv1d as oconv, hadamard as ohad, linear as olin, ssd as ossd, sscan as osscan, update as oupd
from quamba_b200 import modules as M
from quamba_b200.packing import w4a8_quantize

DEV = "cuda"


def _lsb(got, want, max_lsb=1, max_frac=0.02):
    d = (got.cpu().int() - want.int()).abs()
    assert d.max().item() <= max_lsb, f"max diff {d.max().item()} LSB"
    assert (d > 0).float().mean().item() <= max_frac


def _fp16(got, want, rtol=1e-2, atol_rel=1e-3):
    want = want.float()
    ok, msg = allclose_report(got.cpu(), want, rtol, atol_rel * want.abs().max().item())
    assert ok, msg


def _roundtrip(mod, fresh):
    sd = mod.state_dict()
    fresh.load_state_dict(sd)
    sd2 = fresh.state_dict()
    assert sd.keys() == sd2.keys()
    for k in sd:
        if torch.is_tensor(sd[k]):
            assert torch.equal(sd[k], sd2[k]), k
        else:
            assert sd[k] == sd2[k], k
    return sd


# ------------------------------------------------------------------------------------------- CPU: host logic
@pytest.mark.parametrize("tag", ["g128", "g128_pad", "perchannel"])
def test_packer_equals_reference_packer(tag):
    g = load_golden(f"linear_w4a8_{tag}.npz")
    os_ = float(g["out_scale"])
    outs = None if os_ == 0 else torch.full((g["w"].shape[1],), os_)
    w_ref, packed, sg, sc = w4a8_quantize(g["w"].clone(), 4, int(g["group"]), out_scales=outs, pad_out=int(g["pad_out"]))
    assert torch.equal(packed, g["packed"])
    assert torch.equal(sg, g["s_group"]) and torch.equal(sc, g["s_channel"])
    assert torch.equal(w_ref.float(), g["w_ref"])


def test_packer_roundtrips_through_the_oracle_unpacker():
    torch.manual_seed(3)
    w = (torch.randn(256, 192) * 0.05).half()
    w_ref, packed, sg, sc = w4a8_quantize(w, 4, 128)
    q = olin.unpack_weight(packed, 256, 192, per_channel=False)
    sgn, scn = olin.unpermute_scales(sg, sc, 192, per_channel=False)
    w8 = olin.dequant_to_int8(q, sgn, 128)
    # the fp16 group-scale arithmetic of the kernel may land one int8 step from the packer's own int8 view
    err = (w8.float() * scn.reshape(1, -1) - w_ref.float()).abs() / scn.reshape(1, -1)
    assert err.max().item() <= 1.1 and (err > 0.5).float().mean().item() < 0.05


def test_conv_modules_state_dict_and_from_fp16():
    torch.manual_seed(0)
    conv = nn.Conv1d(96, 96, 4, groups=96, padding=3, bias=True)
    q = M.QCausalConv1D.from_fp16(conv, input_scale=0.02, output_scale=0.03)
    assert q.weight.dtype == torch.int8 and q.weight.shape == (96, 4) and q.bias.shape == (96,)
    assert abs(q.weight_scale - conv.weight.abs().max().item() / 127) < 1e-7
    sd = _roundtrip(q, M.QCausalConv1D(96, 96, 4, groups=96, device="cpu"))
    assert {"weight", "bias", "weight_scale", "bias_scale", "input_scale", "output_scale"} == set(sd)

    H, P, G, N = 4, 64, 2, 32
    d = H * P + 2 * G * N
    conv2 = nn.Conv1d(d, d, 4, groups=d, padding=3, bias=True)
    hgr = torch.tensor([[1, 2]] * G, dtype=torch.int32)
    dgr = torch.tensor([[[16, 32, 48, 64]] * 2] * G, dtype=torch.int32)
    q2 = M.Quamb2Conv1D.from_fp16(conv2, H * P, P, N, G, torch.tensor(0.02), torch.tensor(0.03), torch.tensor(0.04),
                                  torch.rand(G, 2, 4) * 0.1, torch.rand(G) * 0.1, torch.rand(G) * 0.1, hgr, dgr)
    assert (q2.x_nhead_group, q2.x_ndim_group) == (2, 4)
    # each segment has its own weight scale, and its largest weight maps to +-127
    for lo, hi in ((0, H * P), (H * P, H * P + G * N), (H * P + G * N, d)):
        assert q2.weight[lo:hi].abs().max().item() == 127
    sd = _roundtrip(q2, M.Quamb2Conv1D(H * P, P, N, G, 2, 4, d, d, 4, groups=d, device="cpu"))
    assert {"x_scale", "B_scale", "C_scale", "wx_scale", "wB_scale", "wC_scale", "bx_scale", "bB_scale", "bC_scale",
            "weight", "bias", "x_head_group_range", "x_dim_group_range", "x_out_scales", "B_out_scales",
            "C_out_scales"} == set(sd)
    with pytest.raises(ValueError):
        M.Quamb2Conv1D(H * P, P, N, G, 2, 0, d, d, 4, groups=d, device="cpu")
    with pytest.raises(AssertionError):
        M.QCausalConv1D(8, 16, 4, groups=8, device="cpu")


def test_scan_modules_state_dict_and_from_fp16():
    torch.manual_seed(1)
    D, N = 64, 16
    A_log = torch.log(torch.arange(1, N + 1).float()).repeat(D, 1)
    t = torch.tensor
    q = M.QSScan.from_fp16(N, D, A_log.clone(), D=torch.ones(D), dt_bias=torch.randn(D), ssm_state_scale=t(0.05),
                           u_scale=t(0.02), dt_scale=t(0.03), B_scale=t(0.04), C_scale=t(0.05), z_scale=t(0.06))
    assert q.A_log.dtype == torch.int8 and q.A_log.abs().max().item() == 127
    assert set(q.state_dict()) == {"dt_bias", "dt_bias_scale", "A_log", "A_scale", "D", "D_scale", "u_scale",
                                   "dt_scale", "B_scale", "C_scale", "z_scale", "ssm_state_scale"}
    _roundtrip(q, M.QSScan(N, D, device="cpu"))

    H, P, G, N2 = 8, 64, 2, 128
    hgr = torch.tensor([[2, 4]] * G, dtype=torch.int32)
    dgr = torch.tensor([[[16, 32, 48, 64]] * 2] * G, dtype=torch.int32)
    cs = M.Quamba2ChunkScan.from_fp16(H * P, P, N2, G, torch.rand(G, 2, 4), hgr, dgr, torch.rand(H) + 0.5, 256,
                                      torch.rand(G, 2, 4, N2), D=torch.ones(H), dt_bias=torch.randn(H),
                                      dt_scale=t(0.02), B_scale=torch.rand(G), C_scale=torch.rand(G), z_scale=None)
    assert cs.grouped and (cs.nhead_groups, cs.ndim_groups) == (2, 4)
    assert cs.ssm_state_scale.shape == (G, 2, 4, N2) and cs.dt_bias.dtype == torch.float16
    assert cs.z_scale is None and "z_scale" not in cs.state_dict()
    _roundtrip(cs, M.Quamba2ChunkScan(H * P, P, N2, G, False, 256, 2, 4, device="cpu"))
    nested = [[(2, [16] * 4, torch.full((4, N2), float(g * 2 + i))) for i in range(2)] for g in range(G)]
    ss = M.Quamba2ChunkScan.get_ssm_state_scales(nested, G, 2, 4, N2, "cpu")
    assert ss.shape == (G, 2, 4, N2) and ss[1, 1, 3, 5] == 3.0

    pt = M.Quamba2ChunkScan.from_fp16(H * P, P, N2, 1, t([0.02]), None, None, torch.rand(H) + 0.5, 256, t([0.01]),
                                      D=torch.ones(H), dt_bias=None, dt_scale=t(0.02), B_scale=t([0.1]),
                                      C_scale=t([0.1]))
    assert not pt.grouped and pt.dt_bias is None and pt.x_scales.shape == (1,)
    with pytest.raises(ValueError):
        M.Quamba2ChunkScan(H * P, P, N2, G, False, 256, 2, 0, device="cpu")


def test_hadamard_module_picks_the_transform_by_dim():
    assert M.QHadamard(5120).N == 40 and M.QHadamard(1536).N == 12 and M.QHadamard(2048).N == 2
    with pytest.raises(AssertionError):
        M.QHadamard(1000)
    h = M.QHadamard(1024, x_H_scale=0.5)
    sd = _roundtrip(h, M.QHadamard(1024))
    assert sd == {"x_H_scale": 0.5}


def test_linear_modules_state_dict_and_from_fp16():
    torch.manual_seed(2)
    lin = nn.Linear(256, 200, bias=False)
    a = M.W4A8B16O16Linear.from_fp16(lin, torch.tensor(0.02))
    assert a.pad_out == 56 and a.size_n == 256 and a.size_k == 256
    assert a.weight.shape == (16, 512) and a.weight.dtype == torch.int32
    assert a.s_group.shape == (2, 256) and a.s_group.dtype == torch.float16 and a.s_channel.shape == (1, 256)
    assert set(a.state_dict()) == {"workspace", "weight", "input_scale", "s_channel", "s_group"}
    _roundtrip(a, M.W4A8B16O16Linear(256, 200, device="cpu"))
    # folding an output scale divides the channel scales, and nothing else changes
    b = M.W4A8B8O8Linear.from_fp16(lin, torch.tensor(0.02), torch.tensor(0.5))
    assert torch.equal(b.weight, a.weight) and torch.equal(b.s_group, a.s_group)
    _, sc_a = olin.unpermute_scales(a.s_group, a.s_channel, 256, False)
    _, sc_b = olin.unpermute_scales(b.s_group, b.s_channel, 256, False)
    assert torch.allclose(sc_b[:200], sc_a[:200] / 0.5)
    c = M.W4A8B8O8LinearParallel.from_fp16(lin, torch.tensor(0.02), [torch.tensor(0.5), torch.tensor(0.25)], [128, 72])
    _, sc_c = olin.unpermute_scales(c.s_group, c.s_channel, 256, False)
    assert torch.allclose(sc_c[:128], sc_a[:128] / 0.5) and torch.allclose(sc_c[128:200], sc_a[128:200] / 0.25)
    small = M.W4A8B16O16Linear.from_fp16(nn.Linear(128, 64, bias=False), torch.tensor(1.0))
    assert small.s_group.numel() == 0                                   # K <= 128: per-channel quantisation
    with pytest.raises(AssertionError):
        M.W4A8B16O16Linear.from_fp16(nn.Linear(256, 64, bias=True), torch.tensor(1.0))

    lin8 = nn.Linear(96, 50, bias=False)
    d = M.W8A8B8O8Linear.from_fp16(lin8, 0.02, 0.04)
    assert d.weight.shape == (96, 64) and d.weight.stride() == (1, 96) and d.pad_out == 14
    assert torch.all(d.weight[:, 50:] == 0)
    ws = lin8.weight.abs().max().item() / 127
    assert abs(d.alpha - ws * 0.02 / 0.04) < 1e-9 and abs(d.a.item() - 0.5) < 1e-7 and abs(d.b.item() - ws) < 1e-9
    sd = _roundtrip(d, M.W8A8B8O8Linear(96, 50, device="cpu"))
    assert set(sd) == {"weight", "a", "b", "alpha"}
    e = M.W8A8B8O8LinearParallel.from_fp16(lin8, 0.02, [0.5, 0.25], [20, 30])
    assert e.b.shape == (1, 64) and torch.all(e.b[0, 50:] == 0)
    assert e.weight[:, :20].abs().max() == 127 and e.weight[:, 20:50].abs().max() == 127
    f = M.W8A8B16O16Linear.from_fp16(lin8, 0.02)
    assert abs(f.alpha - ws * 0.02) < 1e-9 and set(f.state_dict()) == {"weight", "a", "b", "alpha"}


def test_forward_without_a_gpu_fails_loudly():
    q = M.QCausalConv1D(16, 16, 4, groups=16, device="cpu")
    q.weight.zero_(); q.bias.zero_()
    q.weight_scale = q.bias_scale = q.input_scale = q.output_scale = 1.0
    with pytest.raises(Exception):
        q(torch.zeros(1, 16, 8, dtype=torch.int8))


# ------------------------------------------------------------------------------------------- GPU: forwards
gpu = pytest.mark.gpu


@gpu
def test_qcausalconv_forward_and_update():
    torch.manual_seed(0)
    D, L, Bsz = 128, 70, 2
    conv = nn.Conv1d(D, D, 4, groups=D, padding=3, bias=True)
    x, sx = q8(torch.randn(Bsz, D, L))
    q = M.QCausalConv1D.from_fp16(conv, input_scale=sx, output_scale=0.02).to(DEV)
    y = q(x.to(DEV))
    want = oconv.quant_causal_conv1d_fwd(x, sx, q.weight.cpu(), q.weight_scale, 0.02, q.bias_scale, q.bias.cpu())
    _lsb(y, want)
    # the result de-quantises to the floating-point layer's output within quantisation error
    ref = torch.nn.functional.silu(conv(x.float() * sx)[..., :L]).detach()
    assert (y.cpu().float() * 0.02 - ref.clamp(-2.56, 2.54)).abs().max() < 0.08
    state = torch.zeros(Bsz, D, 4, dtype=torch.int8, device=DEV)
    for t in range(6):
        yt = q.update(x[:, :, t].contiguous().to(DEV), state)
        _lsb(yt, want[:, :, t])


@gpu
@pytest.mark.parametrize("grouped", [False, True])
def test_quamb2conv_forward_and_update(grouped):
    H, P, G, N, L, Bsz = 8, 64, 2 if grouped else 1, 64, 45, 2      # per-tensor scales need a single SSD group
    c = make_conv2_case(Bsz, L, H, P, G, N, grouped=grouped, seed=11)
    d = c["xBC"].shape[1]
    q = M.Quamb2Conv1D(c["x_dim"], P, N, G, c["hgr"].shape[1] if grouped else 0, c["dgr"].shape[2] if grouped else 0,
                       d, d, 4, groups=d, device=DEV)
    q.weight.copy_(c["weight"]); q.bias.copy_(c["bias"])
    q.x_scale, q.B_scale, q.C_scale = c["sx"], c["sB"], c["sC"]
    q.wx_scale, q.wB_scale, q.wC_scale = c["swx"], c["swB"], c["swC"]
    q.bx_scale, q.bB_scale, q.bC_scale = c["sbx"], c["sbB"], c["sbC"]
    q.x_out_scales.copy_(c["x_scales"]); q.B_out_scales.copy_(c["B_scales"]); q.C_out_scales.copy_(c["C_scales"])
    if grouped:
        q.x_head_group_range.copy_(c["hgr"]); q.x_dim_group_range.copy_(c["dgr"])
    want = oconv.quamba2_conv1d_fwd(c["xBC"], c["sx"], c["sB"], c["sC"], c["x_dim"], P, N, G, c["hgr"], c["dgr"],
                                    c["x_scales"], c["B_scales"], c["C_scales"], c["weight"], c["swx"], c["swB"],
                                    c["swC"], c["bias"], c["sbx"], c["sbB"], c["sbC"])
    xBC = c["xBC"].transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    got = q(xBC)
    for g_, w_ in zip(got, want):
        _lsb(g_, w_)
    state = torch.zeros(Bsz, d, 4, dtype=torch.int8, device=DEV)
    for t in range(5):
        xs, Bs, Cs = q.update(c["xBC"][:, :, t].contiguous().to(DEV), state)
        for g_, w_ in zip((xs, Bs, Cs), want):
            _lsb(g_.reshape(Bsz, -1), w_[:, :, t].reshape(Bsz, -1))


@gpu
@pytest.mark.parametrize("dim", [2048, 5120, 1536])
def test_qhadamard_forward(dim):
    torch.manual_seed(dim)
    x = torch.randn(3, 7, dim).half()
    h = M.QHadamard(dim, x_H_scale=0.03).to(DEV)
    y = h(x.to(DEV))
    want, _ = ohad.quant_hadamard(x.float().reshape(-1, dim), h.had_scale / 0.03, None if h.N == 2 else h.N)
    assert y.shape == x.shape and y.dtype == torch.int8
    _lsb(y.reshape(-1, dim), want)


@gpu
def test_qsscan_forward_and_update():
    Bsz, D, L, N = 2, 128, 40, 16
    c = make_sscan_case(Bsz, D, L, N, seed=5)
    t = torch.tensor
    q = M.QSScan(N, D, device=DEV)
    for name, v in (("A_log", c["q_A"]), ("D", c["q_D"]), ("dt_bias", c["q_bias"])):
        getattr(q, name).copy_(v)
    for name, v in (("A_scale", c["s_A"]), ("D_scale", c["s_D"]), ("dt_bias_scale", c["s_bias"]), ("u_scale", c["s_u"]),
                    ("dt_scale", c["s_delta"]), ("B_scale", c["s_B"]), ("C_scale", c["s_C"]), ("z_scale", c["s_z"]),
                    ("ssm_state_scale", c["s_state"])):
        getattr(q, name).copy_(t(float(torch.as_tensor(v).reshape(-1)[0])))
    d = lambda v: v.to(DEV)
    y, last = q(d(c["q_u"]), d(c["q_delta"]), d(c["q_B"][:, 0]), d(c["q_C"][:, 0]), z=d(c["q_z"]), return_last_state=True)
    y_ref, x_ref, _ = osscan.quant_sscan_fwd(c["q_u"], c["s_u"], c["q_delta"], c["s_delta"], c["q_A"], c["s_A"], c["q_B"],
                                             c["s_B"], c["q_C"], c["s_C"], c["s_state"], c["q_D"], c["s_D"], c["q_z"],
                                             c["s_z"], c["q_bias"], c["s_bias"], True)
    _fp16(y, y_ref)
    _lsb(last, x_ref[:, :, -1, :])
    state = torch.zeros(Bsz, D, N, dtype=torch.int8)
    want_state = state.clone()
    st_dev = state.to(DEV)
    for tk in range(4):
        args = (c["q_u"][:, :, tk], c["q_delta"][:, :, tk], c["q_B"][:, 0, :, tk], c["q_C"][:, 0, :, tk])
        out, st2 = q.update(st_dev, *(d(a.contiguous()) for a in args), z=d(c["q_z"][:, :, tk].contiguous()))
        assert st2 is st_dev
        want, _ = oupd.quant_sscan_update(want_state, args[0], c["s_u"], args[1], c["s_delta"], c["q_A"], c["s_A"],
                                                   c["s_state"], args[2], c["s_B"], args[3], c["s_C"], c["q_D"], c["s_D"],
                                                   c["q_z"][:, :, tk], c["s_z"], c["q_bias"], c["s_bias"], True)
        _fp16(out, want, rtol=2e-2, atol_rel=2e-3)
        _lsb(st_dev, want_state, max_frac=0.03)
        st_dev.copy_(want_state)


@gpu
@pytest.mark.parametrize("grouped,dh", [(False, False), (True, False), (False, True)])
def test_chunkscan_forward_and_update(grouped, dh):
    Bsz, L, H, P, G, N, Q = 2, 300, 8, 64, 2 if grouped else 1, 128, 256
    c = make_ssd_case(Bsz, L, H, P, G, N, Q, grouped=grouped, seed=21, with_z=False, d_has_hdim=dh)
    q = M.Quamba2ChunkScan(H * P, P, N, G, dh, Q, c["hgr"].shape[1] if grouped else 0,
                           c["dgr"].shape[2] if grouped else 0, device=DEV)
    q.A_log.copy_(c["q_A_log"]); q.A_log_scale.copy_(torch.as_tensor(c["s_A"]).reshape(()))
    q.D.copy_(c["q_D"].reshape(-1)); q.D_scale.copy_(torch.as_tensor(c["s_D"]).reshape(()))
    q.dt_bias.copy_(c["dt_bias"]); q.dt_scale.copy_(torch.as_tensor(c["s_dt"]).reshape(()))
    q.x_scales.copy_(torch.as_tensor(c["x_scales"]).reshape(q.x_scales.shape))
    q.B_scale.copy_(torch.as_tensor(c["s_B"]).reshape(q.B_scale.shape))
    q.C_scale.copy_(torch.as_tensor(c["s_C"]).reshape(q.C_scale.shape))
    q.ssm_state_scale.copy_(c["state_scale"])
    if grouped:
        q.x_head_group_range.copy_(c["hgr"]); q.x_dim_group_range.copy_(c["dgr"])
    d = lambda v: v.to(DEV)
    y, fs = q(d(c["q_x"]), d(c["q_dt"]), d(c["q_B"]), d(c["q_C"]), return_final_states=True)
    y_ref, fq_ref = ossd.chunk_scan_faithful(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"],
                                             c["s_A"], c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["state_scale"], Q, c["q_D"],
                                             c["s_D"], None, None, c["dt_bias"], True)
    _fp16(y, y_ref)
    _lsb(fs, fq_ref, max_frac=0.02)
    assert torch.equal(q(d(c["q_x"]), d(c["q_dt"]), d(c["q_B"]), d(c["q_C"])), y)

    # decode: continue from the prefill state with one token
    x1, dt1 = c["q_x"][:, 0].reshape(Bsz, -1), c["q_dt"][:, 0]
    B1, C1 = c["q_B"][:, 0].reshape(Bsz, -1), c["q_C"][:, 0].reshape(Bsz, -1)
    st = fq_ref.clone().to(DEV)
    out = q.update(st, d(x1), d(dt1), d(B1), d(C1))
    A3 = c["q_A_log"][:, None, None].expand(-1, P, N)
    D2 = c["q_D"] if dh else c["q_D"][:, None].expand(-1, P)
    b2 = c["dt_bias"][:, None].expand(-1, P)
    dt3 = dt1[:, :, None].expand(-1, -1, P)
    want_st = fq_ref.clone()                                     # the oracle updates its int8 state in place
    if grouped:
        want, _ = oupd.quamba2_sscan_update(want_st, c["q_x"][:, 0], c["x_scales"], c["hgr"], c["dgr"], dt3,
                                                  c["s_dt"], A3, c["s_A"], c["state_scale"], c["q_B"][:, 0], c["s_B"],
                                                  c["q_C"][:, 0], c["s_C"], D2, c["s_D"], None, None, b2, True)
    else:
        want, _ = oupd.quant_sscan_update(want_st, c["q_x"][:, 0], c["x_scales"], dt3, c["s_dt"], A3, c["s_A"],
                                                c["state_scale"], c["q_B"][:, 0], c["s_B"], c["q_C"][:, 0], c["s_C"], D2,
                                                c["s_D"], None, None, b2, None, True)
    _fp16(out, want, rtol=2e-2, atol_rel=2e-3)
    _lsb(st, want_st, max_frac=0.03)


def _int8_act(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return q8(torch.randn(*shape, generator=g))


@gpu
@pytest.mark.parametrize("K,N", [(256, 200), (768, 1536), (128, 64)])
def test_w4a8_modules(K, N):
    torch.manual_seed(K + N)
    lin = nn.Linear(K, N, bias=False)
    x, sx = _int8_act((2, 33, K), 1)
    fp = (x.float() * sx) @ lin.weight.detach().t()
    o16 = M.W4A8B16O16Linear.from_fp16(lin, torch.tensor(sx)).to(DEV)
    y = o16(x.to(DEV))
    want = olin.w4a8_gemm(x.reshape(-1, K), o16.weight.cpu(), o16.input_scale.cpu(), o16.s_channel.cpu(),
                          o16.s_group.cpu(), o16.size_n, K, out_int8=False)[:, :N]
    assert y.shape == (2, 33, N) and y.dtype == torch.float16
    _fp16(y.reshape(-1, N), want, rtol=2e-3, atol_rel=1e-4)
    # 4-bit weights: the layer output stays within ~15 % of the full-precision product in RMS
    assert ((y.cpu().float() - fp).norm() / fp.norm()).item() < 0.2
    yt = o16.to_seqlen_last(x.to(DEV))
    assert yt.shape == (2, N, 33) and yt.stride(-1) == 1
    assert torch.equal(yt.transpose(1, 2), y)

    s_out = fp.abs().max().item() / 127
    o8 = M.W4A8B8O8Linear.from_fp16(lin, torch.tensor(sx), torch.tensor(s_out)).to(DEV)
    y8 = o8(x.to(DEV))
    want8 = olin.w4a8_gemm(x.reshape(-1, K), o8.weight.cpu(), o8.input_scale.cpu(), o8.s_channel.cpu(), o8.s_group.cpu(),
                           o8.size_n, K, out_int8=True)[:, :N]
    assert y8.dtype == torch.int8
    _lsb(y8.reshape(-1, N), want8, max_frac=0.002)
    assert torch.equal(o8.to_seqlen_last(x.to(DEV)).transpose(1, 2), y8)

    split = [N // 4, N - N // 4]
    scales = [torch.tensor(s_out), torch.tensor(2 * s_out)]
    par = M.W4A8B8O8LinearParallel.from_fp16(lin, torch.tensor(sx), scales, split).to(DEV)
    yp = par(x.to(DEV)).cpu()
    _lsb(yp[..., :split[0]], y8.cpu()[..., :split[0]], max_frac=0.002)
    half = torch.clamp(torch.round(fp[..., split[0]:] / (2 * s_out)), -128, 127)
    assert (yp[..., split[0]:].float() - half).abs().mean() < 8            # same quantity on the coarser grid
    # one token (decode)
    y1 = o8(x[:1, :1].to(DEV))
    assert torch.equal(y1, y8[:1, :1])


@gpu
@pytest.mark.parametrize("K,N", [(96, 50), (768, 1536)])
def test_w8a8_modules(K, N):
    torch.manual_seed(K)
    lin = nn.Linear(K, N, bias=False)
    x, sx = _int8_act((2, 19, K), 2)
    fp = (x.float() * sx) @ lin.weight.detach().t()
    s_out = fp.abs().max().item() / 127
    o8 = M.W8A8B8O8Linear.from_fp16(lin, sx, s_out).to(DEV)
    y8 = o8(x.to(DEV))
    want = olin.w8a8_gemm(x.reshape(-1, K), o8.weight.cpu(), o8.a.cpu(), o8.b.cpu(), torch.int8)[:, :N]
    assert y8.shape == (2, 19, N) and y8.dtype == torch.int8
    _lsb(y8.reshape(-1, N), want, max_frac=0.002)
    assert (y8.cpu().float() * s_out - fp).abs().max() < 3 * s_out
    yt = o8.to_seqlen_last(x.to(DEV))                                      # 38 rows: exercises the row padding
    assert yt.shape == (2, N, 19) and yt.stride(-1) == 1
    _lsb(yt.transpose(1, 2).reshape(-1, N), want, max_frac=0.002)
    y1 = o8(x[:1, :1].to(DEV))                                             # matrix-vector path (alpha)
    want1 = olin.w8a8_gemv_alpha(o8.weight.cpu().t(), x[0, :1], o8.alpha, torch.int8)[:, :N]
    _lsb(y1.reshape(1, N), want1, max_frac=0.01)

    o16 = M.W8A8B16O16Linear.from_fp16(lin, sx).to(DEV)
    y16 = o16(x.to(DEV))
    want16 = olin.w8a8_gemm(x.reshape(-1, K), o16.weight.cpu(), o16.a.cpu(), o16.b.cpu(), torch.float16)[:, :N]
    _fp16(y16.reshape(-1, N), want16, rtol=2e-3, atol_rel=1e-4)
    _fp16(o16(x[:1, :1].to(DEV)).reshape(1, N), want16[:1], rtol=2e-3, atol_rel=1e-4)

    split = [N // 2, N - N // 2]
    par = M.W8A8B8O8LinearParallel.from_fp16(lin, sx, [s_out, 2 * s_out], split).to(DEV)
    yp = par(x.to(DEV))
    wantp = olin.w8a8_gemm(x.reshape(-1, K), par.weight.cpu(), par.a.cpu(), par.b.cpu(), torch.int8)[:, :N]
    _lsb(yp.reshape(-1, N), wantp, max_frac=0.002)
    y1p = par(x[:1, :1].to(DEV))
    want1p = olin.w8a8o8_gemv(par.weight.cpu().t(), x[0, :1], par.b.cpu(), par.a.cpu())[:, :N]
    _lsb(y1p.reshape(1, N), want1p, max_frac=0.01)
