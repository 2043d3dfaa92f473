"""GPU parity tests: every call goes through the C ABI (ctypes -> libquamba_b200.so) and is compared
with the CPU oracle on the same seeded inputs, or with the committed golden vectors.

Tolerances: re-quantised int8 activations within +-1 LSB; integer GEMM results exact; fp16 scan / SSD
outputs within 1e-2 relative + 1e-3 absolute, the absolute term measured on the output's scale
(1e-3 * max|ref|; outputs here have max|ref| of 3 to 30, and the achieved absolute error is printed by the
reference-golden tests)."""
import pytest
import torch

from helpers import allclose_report, load_golden, make_conv2_case, make_ssd_case, make_sscan_case, q8
from oracle import conv1d as oconv, hadamard as ohad, linear as olin, ssd as ossd, sscan as osscan, update as oupd

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ops():
    from quamba_b200 import ops as o
    return o


def dev(t):
    return None if t is None else t.to(DEV)


def assert_lsb(got, want, max_lsb=1, max_frac=0.02):
    d = (got.cpu().int() - want.int()).abs()
    assert d.max().item() <= max_lsb, f"max diff {d.max().item()} LSB"
    assert (d > 0).float().mean().item() <= max_frac, f"{(d > 0).float().mean().item():.4f} of elements differ"


def assert_fp16(got, want, rtol=1e-2, atol_rel=1e-3):
    want = want.float()
    ok, msg = allclose_report(got.cpu(), want, rtol, atol_rel * want.abs().max().item())
    assert ok, msg


# ---- conv1d ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("Bsz,L,H,P,G,N,grouped,stride", [
    (2, 37, 4, 64, 1, 64, False, None), (1, 130, 8, 64, 2, 64, True, None), (2, 64, 4, 64, 1, 128, False, 768),
    (1, 1, 2, 64, 1, 64, False, None), (1, 300, 16, 64, 8, 16, True, 1344)])
def test_quamba2_conv_fwd(Bsz, L, H, P, G, N, grouped, stride):
    c = make_conv2_case(Bsz, L, H, P, G, N, grouped=grouped, seed=L, row_stride=stride)
    want = oconv.quamba2_conv1d_fwd(c["xBC"], c["sx"], c["sB"], c["sC"], c["x_dim"], P, N, G, c["hgr"], c["dgr"], c["x_scales"],
                                    c["B_scales"], c["C_scales"], c["weight"], c["swx"], c["swB"], c["swC"], c["bias"], c["sbx"],
                                    c["sbB"], c["sbC"])
    S = c["xBC"].stride(2)
    buf = torch.zeros(Bsz, L, S, dtype=torch.int8)
    buf[:, :, :c["xBC"].shape[1]] = c["xBC"].transpose(1, 2)
    xBC = buf.to(DEV)[:, :, :c["xBC"].shape[1]].transpose(1, 2)
    got = ops().quamba2_conv1d_cuda.fwd(xBC, c["sx"], c["sB"], c["sC"], c["x_dim"], P, N, G, dev(c["hgr"]), dev(c["dgr"]),
                                        dev(c["x_scales"]), dev(c["B_scales"]), dev(c["C_scales"]), dev(c["weight"]), c["swx"],
                                        c["swB"], c["swC"], dev(c["bias"]), c["sbx"], c["sbB"], c["sbC"], None, None, None, True)
    for g_, w_ in zip(got, want):
        assert g_.shape == w_.shape and g_.stride(1) == 1
        assert_lsb(g_, w_)


def test_quamba2_conv_update_matches_fwd_and_oracle():
    c = make_conv2_case(3, 9, 4, 64, 2, 64, grouped=True, seed=4)
    C = c["xBC"].shape[1]
    args = (c["sx"], c["sB"], c["sC"], c["x_dim"], 64, 64, 2)
    tail = (c["weight"], c["swx"], c["swB"], c["swC"], c["bias"], c["sbx"], c["sbB"], c["sbC"])
    state_ref = torch.zeros(3, C, 4, dtype=torch.int8)
    state = torch.zeros(3, 4, C, dtype=torch.int8, device=DEV).transpose(1, 2)   # (B, C, 4) backed by (B, 4, C)
    for l in range(9):
        xl = c["xBC"][:, :, l].contiguous()
        want = oconv.quamba2_conv1d_update(xl, state_ref, *args, c["hgr"], c["dgr"], c["x_scales"], c["B_scales"], c["C_scales"], *tail)
        got = ops().quamba2_conv1d_cuda.update(xl.to(DEV), state, *args, dev(c["hgr"]), dev(c["dgr"]), dev(c["x_scales"]),
                                               dev(c["B_scales"]), dev(c["C_scales"]), *[dev(t) if torch.is_tensor(t) else t for t in tail],
                                               None, None, None, True)
        for g_, w_ in zip(got, want):
            assert_lsb(g_, w_, max_frac=0.05)
        assert torch.equal(state.cpu(), state_ref)


@pytest.mark.parametrize("Bsz,D,L,W,layout", [(2, 48, 33, 4, "seq"), (1, 64, 256, 4, "seq"), (2, 32, 100, 3, "seq"),
                                               (1, 16, 7, 2, "seq"), (2, 64, 50, 4, "chan"), (1, 128, 257, 3, "chan")])
def test_quamba1_conv_fwd(Bsz, D, L, W, layout):
    g = torch.Generator().manual_seed(L)
    x, sx = q8(torch.randn(Bsz, D, L, generator=g))
    w, sw = q8(torch.randn(D, W, generator=g) * 0.3)
    b, sb = q8(torch.randn(D, generator=g) * 0.1)
    want = oconv.quant_causal_conv1d_fwd(x, float(sx), w, float(sw), 0.03, float(sb), b, True)
    xd = x.to(DEV)
    if layout == "chan":
        xd = x.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    got = ops().quant_causal_conv1d_cuda.fwd(xd, float(sx), w.to(DEV), float(sw), 0.03, float(sb), b.to(DEV), None, None, None, True)
    assert got.stride() == xd.stride()
    assert_lsb(got, want)
    got_nb = ops().quant_causal_conv1d_cuda.fwd(xd, float(sx), w.to(DEV), float(sw), 0.03, float(sb), None, None, None, None, False)
    assert_lsb(got_nb, oconv.quant_causal_conv1d_fwd(x, float(sx), w, float(sw), 0.03, float(sb), None, False))


def test_quamba1_conv_update():
    g = torch.Generator().manual_seed(1)
    x, sx = q8(torch.randn(4, 96, generator=g))
    w, sw = q8(torch.randn(96, 4, generator=g) * 0.3)
    b, sb = q8(torch.randn(96, generator=g) * 0.1)
    st = torch.randint(-128, 128, (4, 96, 4), dtype=torch.int8, generator=g)
    st_ref = st.clone()
    want = oconv.quant_causal_conv1d_update(x, st_ref, float(sx), w, float(sw), 0.02, float(sb), b, True)
    std = st.to(DEV)
    got = ops().quant_causal_conv1d_cuda.update(x.to(DEV), std, float(sx), w.to(DEV), float(sw), 0.02, float(sb), b.to(DEV), True)
    assert_lsb(got, want, max_frac=0.05)
    assert torch.equal(std.cpu(), st_ref)


def test_conv_rejects_what_the_reference_rejects():
    x = torch.zeros(1, 16, 8, dtype=torch.int8, device=DEV)
    w5 = torch.zeros(16, 5, dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError, match="width between 2 and 4"):
        ops().quant_causal_conv1d_cuda.fwd(x, 1.0, w5, 1.0, 1.0, 1.0)
    with pytest.raises(RuntimeError, match="seq_idx"):
        ops().quant_causal_conv1d_cuda.fwd(x, 1.0, w5[:, :4].contiguous(), 1.0, 1.0, 1.0, None, torch.zeros(1))


# ---- Hadamard ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,dim,special,dtype", [(5, 1024, 1, torch.float16), (3, 5120, 40, torch.float16),
                                                      (2, 1536, 12, torch.float16), (2, 2560, 20, torch.bfloat16),
                                                      (1, 3584, 28, torch.float32), (4, 8192, 1, torch.float16),
                                                      (7, 64, 1, torch.float16), (2, 96, 12, torch.float16)])
def test_hadamard_quant(rows, dim, special, dtype):
    x = (torch.randn(rows, dim, generator=torch.Generator().manual_seed(dim)) * 2).to(dtype)
    scale = (1.0 / dim ** 0.5) / 0.03
    want, _ = ohad.quant_hadamard(x.float(), scale, special)
    fn = {1: "fast_hadamard_transform", 12: "fast_hadamard_transform_12N", 20: "fast_hadamard_transform_20N",
          28: "fast_hadamard_transform_28N", 40: "fast_hadamard_transform_40N"}[special]
    got = getattr(ops().quant_hadamard, fn)(x.to(DEV), scale)
    assert got.dtype == torch.int8 and got.shape == x.shape
    assert_lsb(got, want)


@pytest.mark.parametrize("rows,dim,special", [(19, 5120, 40), (9, 1536, 12), (6, 2560, 20), (5, 3584, 28), (11, 256, 1), (3, 512, 1),
                                              (17, 2048, 1), (5, 4096, 1), (300, 5120, 40)])
def test_hadamard_tensor_core_path(rows, dim, special):
    """fp16 rows of S * 128 elements take the tcgen05 path (odd row counts exercise the ragged last unit); the result must
    match the oracle and the SIMT kernel (selected with the library's path override)."""
    x = (torch.randn(rows, dim, generator=torch.Generator().manual_seed(rows + dim)) * 3).to(torch.float16)
    scale = (1.0 / dim ** 0.5) / 0.05
    want, _ = ohad.quant_hadamard(x.float(), scale, special)
    fn = {1: "fast_hadamard_transform", 12: "fast_hadamard_transform_12N", 20: "fast_hadamard_transform_20N",
          28: "fast_hadamard_transform_28N", 40: "fast_hadamard_transform_40N"}[special]
    got = getattr(ops().quant_hadamard, fn)(x.to(DEV), scale)
    assert_lsb(got, want, max_frac=0.002)
    from quamba_b200 import _lib as qlib
    with qlib.path_override(qlib.PATH_HADAMARD_SIMT):
        simt = getattr(ops().quant_hadamard, fn)(x.to(DEV), scale)
    assert_lsb(got, simt.cpu(), max_frac=0.002)
    ops()._lib.read_device_status(torch.cuda.current_stream().cuda_stream)


def test_hadamard_saturates():
    x = torch.full((1, 128), 50.0, dtype=torch.float16)
    got = ops().quant_hadamard.fast_hadamard_transform(x.to(DEV), 1.0).cpu()
    assert got[0, 0] == 127 and (got[0, 1:] == 0).all()


# ---- Mamba1 scan --------------------------------------------------------------------------------------
@pytest.mark.parametrize("Bsz,D,L,N,with_z", [(1, 1536, 512, 16, True), (2, 100, 33, 16, True), (1, 64, 2100, 16, False),
                                               (2, 128, 64, 32, True)])
def test_sscan_fwd(Bsz, D, L, N, with_z):
    c = make_sscan_case(Bsz, D, L, N, seed=L, with_z=with_z)
    y_ref, x_ref, h_ref = osscan.quant_sscan_fwd(c["q_u"], c["s_u"], c["q_delta"], c["s_delta"], c["q_A"], c["s_A"], c["q_B"],
                                                 c["s_B"], c["q_C"], c["s_C"], c["s_state"], c["q_D"], c["s_D"], c["q_z"],
                                                 c["s_z"], c["q_bias"], c["s_bias"], True)
    out, x = ops().quant_sscan_cuda.fwd(dev(c["q_u"]), dev(c["s_u"]), dev(c["q_delta"]), dev(c["s_delta"]), dev(c["q_A"]),
                                        dev(c["s_A"]), dev(c["q_B"]), dev(c["s_B"]), dev(c["q_C"]), dev(c["s_C"]), dev(c["s_state"]),
                                        dev(c["q_D"]), dev(c["s_D"]), dev(c["q_z"]), dev(c["s_z"]), dev(c["q_bias"]), dev(c["s_bias"]), True)
    assert out.shape == (Bsz, L, D) and out.dtype == torch.float16 and out.is_contiguous()
    assert x.shape == x_ref.shape
    assert_fp16(out, y_ref)
    assert_lsb(x, x_ref, max_frac=0.05)
    # the dequantised last state against the fp32 reference state
    last = x[:, :, -1, :].cpu().float() * c["s_state"]
    assert (last - torch.clamp(h_ref, -128 * 0.05, 127 * 0.05)).abs().max() <= 0.05 * 1.01


# ---- state update ----------------------------------------------------------------------------------------
def test_update_mamba1_against_reference_torch_golden():
    g = load_golden("update_ref.npz")
    st = g["m1_state_q"].clone().to(DEV)
    out = ops().quant_sscan_update_triton(st, dev(g["m1_q_x"]), dev(g["m1_s_x"]), dev(g["m1_q_dt"]), dev(g["m1_s_dt"]), dev(g["m1_q_A"]),
                                          dev(g["m1_s_A"]), dev(g["m1_s_state"]), dev(g["m1_q_B"]), dev(g["m1_s_B"]), dev(g["m1_q_C"]),
                                          dev(g["m1_s_C"]), dev(g["m1_q_D"]), dev(g["m1_s_D"]), dev(g["m1_q_z"]), dev(g["m1_s_z"]),
                                          dev(g["m1_q_bias"]), dev(g["m1_s_bias"]), True)
    assert_fp16(out, g["m1_ref_y"])
    want_q = torch.clamp(torch.round(g["m1_ref_state"] / g["m1_s_state"]), -128, 127).to(torch.int8)
    assert_lsb(st, want_q, max_frac=0.02)


def test_update_mamba2_tied_and_grouped():
    g = load_golden("update_ref.npz")
    H, P, N = 8, 32, 64
    st = g["m2_state_q"].clone().to(DEV)
    dt = dev(g["m2_q_dt"])[..., None].expand(2, H, P)
    A = dev(g["m2_q_A"])[:, None, None].expand(H, P, N)
    Dq = dev(g["m2_q_D"])[:, None].expand(H, P)
    bias = dev(g["m2_bias"])[:, None].expand(H, P)
    out = ops().quant_sscan_update_triton(st, dev(g["m2_q_x"]), dev(g["m2_s_x"]), dt, dev(g["m2_s_dt"]), A, dev(g["m2_s_A"]),
                                          dev(g["m2_s_state"]), dev(g["m2_q_B"]), dev(g["m2_s_B"]), dev(g["m2_q_C"]), dev(g["m2_s_C"]),
                                          Dq, dev(g["m2_s_D"]), None, None, bias, None, True)
    assert_fp16(out, g["m2_ref_y"])
    want_q = torch.clamp(torch.round(g["m2_ref_state"] / g["m2_s_state"]), -128, 127).to(torch.int8)
    assert_lsb(st, want_q, max_frac=0.02)
    # grouped scales, against the oracle
    gen = torch.Generator().manual_seed(9)
    G, HG, DG = 2, 2, 4
    hgr = torch.tensor([[2, 4]] * G, dtype=torch.int32)
    dgr = torch.tensor([[[8, 16, 24, 32]] * HG] * G, dtype=torch.int32)
    xs = torch.rand(G, HG, DG, generator=gen) * 0.02 + 0.01
    ss = torch.rand(G, HG, DG, N, generator=gen) * 0.01 + 0.005
    sB = torch.rand(G, generator=gen) * 0.02 + 0.01
    sC = torch.rand(G, generator=gen) * 0.02 + 0.01
    st_ref = g["m2_state_q"].clone()
    y_ref, _ = oupd.quamba2_sscan_update(st_ref, g["m2_q_x"], xs, hgr, dgr, g["m2_q_dt"][..., None].expand(2, H, P), g["m2_s_dt"],
                                         g["m2_q_A"][:, None, None].expand(H, P, N), g["m2_s_A"], ss, g["m2_q_B"], sB, g["m2_q_C"], sC,
                                         g["m2_q_D"][:, None].expand(H, P), g["m2_s_D"], None, None, g["m2_bias"][:, None].expand(H, P), True)
    st2 = g["m2_state_q"].clone().to(DEV)
    out2 = ops().quamba2_sscan_update_triton(st2, dev(g["m2_q_x"]), dev(xs), dev(hgr), dev(dgr), dt, dev(g["m2_s_dt"]), A, dev(g["m2_s_A"]),
                                             dev(ss), dev(g["m2_q_B"]), dev(sB), dev(g["m2_q_C"]), dev(sC), Dq, dev(g["m2_s_D"]), None, None,
                                             bias, True)
    assert_fp16(out2, y_ref)
    assert_lsb(st2, st_ref, max_frac=0.02)


# ---- SSD --------------------------------------------------------------------------------------------------
def _run_ssd(c, grouped):
    o = ops()
    if grouped:
        return o._quamba2_mamba_chunk_scan_combined_fwd(
            dev(c["q_x"]), dev(c["x_scales"]), dev(c["hgr"]), dev(c["dgr"]), dev(c["q_dt"]), dev(c["s_dt"]), dev(c["q_A_log"]), dev(c["s_A"]),
            dev(c["q_B"]), dev(c["s_B"]), dev(c["q_C"]), dev(c["s_C"]), dev(c["state_scale"]), c["chunk"], dev(c["q_D"]), dev(c["s_D"]),
            dev(c.get("q_z")), dev(c.get("s_z")), dev(c["dt_bias"]), None, None, None, True)
    return o._quant_mamba_chunk_scan_combined_fwd(
        dev(c["q_x"]), dev(c["x_scales"]), dev(c["q_dt"]), dev(c["s_dt"]), dev(c["q_A_log"]), dev(c["s_A"]), dev(c["q_B"]), dev(c["s_B"]),
        dev(c["q_C"]), dev(c["s_C"]), dev(c["state_scale"]), c["chunk"], dev(c["q_D"]), dev(c["s_D"]), dev(c.get("q_z")), dev(c.get("s_z")),
        dev(c["dt_bias"]), None, None, None, True)


@pytest.mark.parametrize("tag", ["pertensor", "grouped", "n128"])
def test_ssd_against_reference_triton_golden(tag):
    """Outputs of the reference's own Triton kernels (interpreter mode).  "n128" (headdim 64, d_state 128, chunk 256, 600
    tokens) is the shape family of the tensor-core kernel, the other two reach the portable path."""
    g = load_golden(f"ssd_{tag}.npz")
    grouped = tag == "grouped"
    G, N = g["q_B"].shape[2:]
    c = dict(q_x=g["q_x"], x_scales=g["x_scales"], hgr=g.get("head_group_range"), dgr=g.get("dim_group_range"), q_dt=g["q_dt"],
             s_dt=g["s_dt"], q_A_log=g["q_A_log"], s_A=g["s_A"], q_B=g["q_B"], s_B=g["s_B"], q_C=g["q_C"], s_C=g["s_C"],
             state_scale=torch.full((G, 2, 2, N), 0.01) if grouped else torch.tensor([0.01]), chunk=int(g["chunk"]), q_D=g["q_D"],
             s_D=g["s_D"], dt_bias=g["dt_bias"])
    y, fs = _run_ssd(c, grouped)
    assert_fp16(y, g["ref_out"])
    err = (y.cpu().float() - g["ref_out"].float()).abs().max().item()
    print(f"ssd_{tag}: max |y - reference| = {err:.3e} with max |reference| = {g['ref_out'].float().abs().max().item():.3f}")
    want_q = torch.clamp(torch.round(g["ref_final_f16"].float() / 0.01), -128, 127).to(torch.int8)
    assert_lsb(fs, want_q, max_frac=0.02)


@pytest.mark.parametrize("Bsz,L,H,P,G,N,Q,grouped,with_z,dh", [
    (2, 200, 4, 64, 2, 64, 64, True, True, True), (1, 512, 8, 64, 1, 128, 256, False, False, False),
    (1, 100, 2, 64, 1, 128, 128, False, True, False), (2, 256, 16, 64, 8, 128, 256, True, False, False)])
def test_ssd_against_oracle(Bsz, L, H, P, G, N, Q, grouped, with_z, dh):
    c = make_ssd_case(Bsz, L, H, P, G, N, Q, grouped=grouped, seed=L + H, with_z=with_z, d_has_hdim=dh)
    y_ref, fq_ref = ossd.chunk_scan_faithful(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"],
                                             c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["state_scale"], Q, c["q_D"], c["s_D"], c["q_z"],
                                             c["s_z"], c["dt_bias"], True)
    y_id, _ = ossd.chunk_scan_ideal(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"], c["q_B"],
                                    c["s_B"], c["q_C"], c["s_C"], c["q_D"], c["s_D"], c["q_z"], c["s_z"], c["dt_bias"], True,
                                    dtype=torch.float32)
    y, fs = _run_ssd(c, grouped)
    assert y.shape == (Bsz, L, H, P) and fs.shape == (Bsz, H, P, N)
    assert_fp16(y, y_ref)
    assert_fp16(y, y_id)
    assert_lsb(fs, fq_ref, max_frac=0.02)


@pytest.mark.parametrize("Bsz,L,H,G,grouped,dh", [(1, 50, 2, 1, False, False), (2, 333, 4, 2, True, True), (1, 128, 3, 1, False, False),
                                                  (1, 1000, 8, 8, True, False), (3, 129, 2, 2, False, True)])
def test_ssd_tensor_core_path_against_oracle(Bsz, L, H, G, grouped, dh):
    """headdim 64 / d_state 128 / no z: the tcgen05 kernel (128-token blocks, state kept on chip)."""
    P, N, Q = 64, 128, 256
    c = make_ssd_case(Bsz, L, H, P, G, N, Q, grouped=grouped, seed=L, d_has_hdim=dh)
    y_ref, fq_ref = ossd.chunk_scan_faithful(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"],
                                             c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["state_scale"], Q, c["q_D"], c["s_D"], None, None,
                                             c["dt_bias"], True)
    y_id, h_id = ossd.chunk_scan_ideal(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"], c["q_B"],
                                       c["s_B"], c["q_C"], c["s_C"], c["q_D"], c["s_D"], None, None, c["dt_bias"], True, dtype=torch.float32)
    y, fs = _run_ssd(c, grouped)
    torch.cuda.synchronize()
    from quamba_b200 import _lib
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
    assert_fp16(y, y_id)
    assert_fp16(y, y_ref)
    assert_lsb(fs, fq_ref, max_frac=0.03)


def test_ssd_tensor_core_path_equals_portable_path_on_device():
    """Same inputs through both CUDA paths at a layer-sized shape (batch 1 of the benchmark configuration)."""
    c = make_ssd_case(1, 2048, 80, 64, 1, 128, 256, seed=7)
    y_tc, f_tc = _run_ssd(c, False)
    from quamba_b200 import _lib as qlib
    with qlib.path_override(qlib.PATH_SSD_PORTABLE):
        y_pt, f_pt = _run_ssd(c, False)
    torch.cuda.synchronize()
    assert_fp16(y_tc, y_pt.cpu())
    assert_lsb(f_tc, f_pt.cpu(), max_frac=0.03)


# ---- linears ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["g128", "g128_pad", "perchannel"])
@pytest.mark.parametrize("M", [1, 5, 16, 89, 256])
def test_w4a8_gemm_with_reference_packed_weights(tag, M):
    g = load_golden(f"linear_w4a8_{tag}.npz")
    K = g["w"].shape[0]
    N = g["s_channel"].numel()
    a, s_a = q8(torch.randn(M, K, generator=torch.Generator().manual_seed(M)))
    ws = torch.zeros(N // 64 * 16, dtype=torch.int32, device=DEV)
    o = ops().quant_linear_cuda
    want16, acc = olin.w4a8_gemm(a, g["packed"], s_a, g["s_channel"], g["s_group"], N, K, out_int8=False, return_acc=True)
    got16 = o.w4a8o16_gemm(a.to(DEV), dev(g["packed"]), dev(s_a), dev(g["s_channel"]), dev(g["s_group"]), ws, M, N, K, False)
    assert got16.dtype == torch.float16 and got16.shape == (M, N)
    assert torch.equal(got16.cpu(), want16), (got16.cpu().float() - want16.float()).abs().max()
    gotT = o.w4a8o16_gemm(a.to(DEV), dev(g["packed"]), dev(s_a), dev(g["s_channel"]), dev(g["s_group"]), ws, M, N, K, True)
    assert gotT.shape == (N, M) and torch.equal(gotT.cpu(), want16.t())
    s_big = s_a * 30
    want8 = olin.w4a8_gemm(a, g["packed"], s_big, g["s_channel"], g["s_group"], N, K, out_int8=True)
    got8 = o.w4a8o8_gemm(a.to(DEV), dev(g["packed"]), dev(s_big), dev(g["s_channel"]), dev(g["s_group"]), ws, M, N, K, False)
    assert torch.equal(got8.cpu(), want8)
    s_row = (torch.rand(M) * 0.02 + 0.01)
    want_row = olin.w4a8_gemm(a, g["packed"], s_row, g["s_channel"], g["s_group"], N, K, out_int8=False)
    got_row = o.w4a8o16_gemm(a.to(DEV), dev(g["packed"]), dev(s_row), dev(g["s_channel"]), dev(g["s_group"]), ws, M, N, K, False)
    if M > 1:
        assert torch.equal(got_row.cpu(), want_row)


@pytest.mark.parametrize("M,K,N", [(1, 768, 1536), (89, 768, 1536), (1024, 2560, 256), (130, 160, 320), (64, 5120, 192)])
def test_w8a8_gemm_and_gemv(M, K, N):
    gen = torch.Generator().manual_seed(M + K)
    a = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
    w_nk = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=gen)
    b = w_nk.to(DEV).t()                       # (K, N) column-major, as the modules store it
    o = ops().quant_linear_cuda
    a_s = torch.tensor([[0.002]]); b_s = torch.tensor([[0.003]])
    for dt in (torch.int8, torch.float16, torch.bfloat16):
        c = torch.empty(M, N, dtype=dt, device=DEV)
        o.cutlass_scaled_mm_dq(c, a.to(DEV), b, dev(a_s), dev(b_s))
        want = olin.w8a8_gemm(a, w_nk.t(), a_s, b_s, dt)
        assert torch.equal(c.cpu(), want), dt
    b_col = (torch.rand(1, N, generator=gen) * 0.004 + 0.001)
    c = torch.empty(M, N, dtype=torch.int8, device=DEV)
    o.cutlass_scaled_mm_dq(c, a.to(DEV), b, dev(a_s), dev(b_col))
    assert torch.equal(c.cpu(), olin.w8a8_gemm(a, w_nk.t(), a_s, b_col, torch.int8))
    a_row = (torch.rand(M, 1, generator=gen) * 0.004 + 0.001)
    c16 = torch.empty(M, N, dtype=torch.float16, device=DEV)
    o.cutlass_scaled_mm_dq(c16, a.to(DEV), b, dev(a_row), dev(b_col))
    assert torch.equal(c16.cpu(), olin.w8a8_gemm(a, w_nk.t(), a_row, b_col, torch.float16))
    if M == 1:
        cv = torch.empty(1, N, dtype=torch.float16, device=DEV)
        o.cutlass_scaled_mv_dq(cv, w_nk.to(DEV), a.to(DEV), 6e-6, 0.0)
        assert torch.equal(cv.cpu(), olin.w8a8_gemv_alpha(w_nk, a, 6e-6, torch.float16))
        c8 = torch.empty(1, N, dtype=torch.int8, device=DEV)
        sw = (torch.rand(N, generator=gen) * 0.002 + 0.001)
        o.w8a8o8_gemv(c8, w_nk.to(DEV), a.to(DEV), dev(sw), dev(torch.tensor([0.01])))
        assert_lsb(c8, olin.w8a8o8_gemv(w_nk, a, sw, torch.tensor([0.01])), max_frac=0.01)


def test_to_seqlen_last_operand_swap():
    """The W8A8 'seqlen last' form: D (N, M) = W^T (N, K) . X^T (K, M) with the scale roles swapped."""
    gen = torch.Generator().manual_seed(3)
    M, K, N = 48, 256, 128
    x = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
    w_nk = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=gen)
    a_s = torch.tensor([[0.002]]); b_s = torch.tensor([[0.003]])
    y = torch.empty(N, M, dtype=torch.int8, device=DEV)
    ops().quant_linear_cuda.cutlass_scaled_mm_dq(y, w_nk.to(DEV), x.to(DEV).t(), dev(b_s), dev(a_s))
    want = olin.w8a8_gemm(w_nk, x.t(), b_s, a_s, torch.int8)
    assert torch.equal(y.cpu(), want)


def test_no_device_wait_timed_out():
    from quamba_b200 import _lib
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)


# ---- state update: the kernels behind qb_sscan_update (warp-autonomous, pipelined bulk-copy, streaming, generic) -----
@pytest.mark.parametrize("Bsz,H,P,G,N,grouped,layout", [
    (3, 8, 64, 1, 128, False, "contig"),     # Mamba2 decode shape: warp-autonomous kernel (16-row tiles)
    (7, 5, 48, 1, 128, False, "contig"),     # the same kernel: three tiles per head, 105 tiles over the warps
    (4, 6, 32, 2, 128, False, "contig"),     # the same kernel: two SSD groups
    (2, 8, 64, 2, 128, True, "contig"),      # pipelined, grouped scales
    (2, 4, 64, 1, 256, False, "contig"),     # pipelined, 16 pieces per row
    (5, 1, 1024, 1, 16, False, "contig"),    # pipelined, Mamba1 shape (one piece per row), A not tied
    (2, 8, 64, 1, 128, False, "padded"),     # rows 16-byte aligned but not contiguous -> streaming kernel
    (2, 1, 256, 1, 16, False, "contig"),     # too few rows per group for a tile -> streaming kernel
    (2, 3, 24, 1, 40, False, "contig"),      # dstate not a multiple of 16 -> generic kernel
])
def test_update_kernel_variants_against_oracle(Bsz, H, P, G, N, grouped, layout):
    gen = torch.Generator().manual_seed(Bsz * 1000 + N)
    ri8 = lambda *s: torch.randint(-127, 128, s, generator=gen, dtype=torch.int32).to(torch.int8)
    state = ri8(Bsz, H, P, N)
    x, dt, Bm, Cm = ri8(Bsz, H, P), ri8(Bsz, H, P), ri8(Bsz, G, N), ri8(Bsz, G, N)
    tied = H > 1
    A = ri8(H)[:, None, None].expand(H, P, N) if tied else ri8(H, P, N)
    Dq, bias = ri8(H, P), (torch.rand(H, P, generator=gen) * 2 - 4).half()
    s_dt, s_A, s_D = torch.tensor(0.02), torch.tensor(0.015), torch.tensor(0.01)
    zq, s_z = (ri8(Bsz, H, P), torch.tensor(0.03)) if Bsz == 4 else (None, None)     # one case runs with the z gate
    if grouped:
        HG, DG = 2, 4
        hgr = torch.tensor([[H // G // 2, H // G]] * G, dtype=torch.int32)
        dgr = torch.tensor([[[P // 4, P // 2, 3 * P // 4, P]] * HG] * G, dtype=torch.int32)
        xs = torch.rand(G, HG, DG, generator=gen) * 0.02 + 0.01
        ss = torch.rand(G, HG, DG, N, generator=gen) * 0.01 + 0.005
        sB, sC = torch.rand(G, generator=gen) * 0.02 + 0.01, torch.rand(G, generator=gen) * 0.02 + 0.01
        st_ref = state.clone()
        y_ref, _ = oupd.quamba2_sscan_update(st_ref, x, xs, hgr, dgr, dt, s_dt, A, s_A, ss, Bm, sB, Cm, sC, Dq, s_D, None, None, bias, True)
    else:
        xs, ss, sB, sC = torch.tensor([0.02]), torch.tensor([0.01]), torch.tensor([0.015]), torch.tensor([0.017])
        st_ref = state.clone()
        y_ref, _ = oupd.quant_sscan_update(st_ref, x, xs, dt, s_dt, A, s_A, ss, Bm, sB, Cm, sC, Dq, s_D, zq, s_z, bias, None, True)
    if layout == "padded":
        buf = torch.zeros(Bsz, H, P, N + 16, dtype=torch.int8, device=DEV)
        st = buf[..., :N]
        st.copy_(state)
    else:
        st = state.clone().to(DEV)
    A_dev = dev(A.contiguous()) if not tied else dev(A[:, 0, 0].contiguous())[:, None, None].expand(H, P, N)
    if grouped:
        out = ops().quamba2_sscan_update_triton(st, dev(x), dev(xs), dev(hgr), dev(dgr), dev(dt), dev(s_dt), A_dev, dev(s_A), dev(ss),
                                                dev(Bm), dev(sB), dev(Cm), dev(sC), dev(Dq), dev(s_D), None, None, dev(bias), True)
    else:
        out = ops().quant_sscan_update_triton(st, dev(x), dev(xs), dev(dt), dev(s_dt), A_dev, dev(s_A), dev(ss), dev(Bm), dev(sB),
                                              dev(Cm), dev(sC), dev(Dq), dev(s_D), dev(zq), dev(s_z), dev(bias), None, True)
    assert_fp16(out, y_ref)
    assert_lsb(st, st_ref, max_frac=0.02)
    ops()._lib.read_device_status(torch.cuda.current_stream().cuda_stream)      # raises if a device-side wait timed out


# ---- large GEMMs: the persistent tensor-core kernel (needs at least one 128 x 256 tile per SM; the tile width it then
# uses, 192 or 256 columns, depends on the shape: the cases below reach both) ---------------------------
@pytest.mark.parametrize("M,K,N,out_dtype", [(2000, 528, 3024, torch.int8), (2048, 1024, 5120, torch.float16),
                                             (4100, 272, 2304, torch.int8), (2048, 512, 2560, torch.float16),
                                             (2048, 256, 10576, torch.int8), (8192, 128, 2560, torch.float16)])
def test_w8a8_gemm_large_against_exact_float_matmul(M, K, N, out_dtype):
    """|acc| <= K * 127^2 < 2^24 for K <= 1040, so an fp32 matmul of the int8 values is exact and serves as the accumulator
    reference at sizes the CPU oracle would take minutes for; the epilogue is then restated with the oracle's operation order."""
    g = torch.Generator().manual_seed(M + N)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int32).to(torch.int8).to(DEV)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int32).to(torch.int8).to(DEV)   # (N, K) K-contiguous
    a_s = (torch.rand(M, 1, generator=g) * 0.01 + 0.001).to(DEV)
    b_s = (torch.rand(1, N, generator=g) * 0.01 + 0.001).to(DEV)
    acc = a.float() @ w.float().t()
    assert acc.abs().max().item() < 2 ** 24
    res = a_s * (b_s * acc)
    want = torch.clamp(torch.round(res), -128, 127).to(torch.int8) if out_dtype == torch.int8 else res.to(torch.float16)
    c = torch.empty((M, N), dtype=out_dtype, device=DEV)
    ops().quant_linear_cuda.cutlass_scaled_mm_dq(c, a, w.t(), a_s.reshape(-1), b_s.reshape(-1))
    if out_dtype == torch.int8:
        d = (c.int() - want.int()).abs()
        assert d.max().item() <= 1 and (d > 0).float().mean().item() < 1e-4    # fp32 product order at exact ties only
    else:
        assert torch.equal(c, want)
    ops()._lib.read_device_status(torch.cuda.current_stream().cuda_stream)
