"""GPU tests at the benchmark's full sizes, where the CPU oracle would take minutes: properties that hold whatever the
size and that pin down exactly the things a large launch does differently from a small one (how work is cut across SMs,
tile edges, wave boundaries).

* batch independence, bit for bit: the rows of a batched call equal the same rows run one at a time.  For the SSD kernel
  this is the check that the result does not depend on where the (batch, head, block) list is cut between CTAs: batch 4
  is 320 pairs cut into 148 ranges with a state hand-off at every cut, batch 1 is 80 whole pairs.
* causality, bit for bit: changing the tail of a sequence leaves the outputs of the head untouched.
* the tensor-core path against the portable path on the device, at the full batch.
"""
import pytest
import torch

from helpers import make_conv2_case, make_ssd_case, make_sscan_case

pytestmark = pytest.mark.gpu
DEV = "cuda"

# configs[1] of the baseline: batch 4, seqlen 2048, 80 heads of 64, one group, d_state 128, chunk 256
B, L, H, P, G, N, Q = 4, 2048, 80, 64, 1, 128, 256


def ops():
    from quamba_b200 import ops as o
    return o


def dev(t):
    return None if t is None else t.to(DEV)


def run_ssd(c, sl=slice(None)):
    y, fs = ops()._quant_mamba_chunk_scan_combined_fwd(
        dev(c["q_x"][sl]), dev(c["x_scales"]), dev(c["q_dt"][sl]), dev(c["s_dt"]), dev(c["q_A_log"]), dev(c["s_A"]), dev(c["q_B"][sl]),
        dev(c["s_B"]), dev(c["q_C"][sl]), dev(c["s_C"]), dev(c["state_scale"]), c["chunk"], dev(c["q_D"]), dev(c["s_D"]), None, None,
        dev(c["dt_bias"]), None, None, None, True)
    torch.cuda.synchronize()
    from quamba_b200 import _lib
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
    return y, fs


def test_ssd_full_size_is_independent_of_how_the_work_is_cut():
    c = make_ssd_case(B, L, H, P, G, N, Q, seed=11)
    y4, f4 = run_ssd(c)
    assert y4.shape == (B, L, H, P) and f4.shape == (B, H, P, N)
    assert torch.isfinite(y4.float()).all()
    for b in range(B):
        y1, f1 = run_ssd(c, slice(b, b + 1))
        assert torch.equal(y4[b], y1[0]), f"batch row {b}: outputs differ between the batched and the single call"
        assert torch.equal(f4[b], f1[0]), f"batch row {b}: final states differ"
    # twice the same launch: bit-identical (no dependence on the timing between CTAs)
    y4b, f4b = run_ssd(c)
    assert torch.equal(y4, y4b) and torch.equal(f4, f4b)


def test_ssd_full_size_every_pair_against_the_oracle():
    """The benchmarked launch itself (320 (batch, head) pairs cut into 148 ranges, a state hand-off at every cut) against
    the CPU oracle run pair by pair: every pair of the full problem, so every cut position is covered.  fp16 outputs within
    1e-2 relative + 1e-3 x the pair's largest |reference|; final int8 states within 1 LSB.  The largest absolute error is
    printed next to the largest |reference| (the bound is relative to the output range, not 1e-3 absolute)."""
    from oracle import ssd as ossd
    c = make_ssd_case(B, L, H, P, G, N, Q, seed=11)
    y, fs = run_ssd(c)
    y, fs = y.cpu().float(), fs.cpu().int()
    worst_abs, worst_rel_to_max, ref_max = 0.0, 0.0, 0.0
    for b in range(B):
        for h in range(H):
            want_y, want_f = ossd.chunk_scan_faithful(
                c["q_x"][b:b + 1, :, h:h + 1], c["x_scales"], None, None, c["q_dt"][b:b + 1, :, h:h + 1], c["s_dt"], c["q_A_log"][h:h + 1],
                c["s_A"], c["q_B"][b:b + 1], c["s_B"], c["q_C"][b:b + 1], c["s_C"], c["state_scale"], Q, c["q_D"][h:h + 1], c["s_D"], None,
                None, c["dt_bias"][h:h + 1], True)
            w = want_y[0, :, 0].float()
            err = (y[b, :, h] - w).abs()
            assert (err <= 1e-3 * w.abs().max() + 1e-2 * w.abs()).all(), f"pair ({b}, {h}): max err {err.max().item():.4g} of {w.abs().max().item():.4g}"
            assert (fs[b, h] - want_f[0, 0].int()).abs().max() <= 1, f"pair ({b}, {h}): final state"
            worst_abs = max(worst_abs, err.max().item())
            worst_rel_to_max = max(worst_rel_to_max, (err.max() / w.abs().max()).item())
            ref_max = max(ref_max, w.abs().max().item())
    print(f"ssd full size, 320 pairs: max |y - oracle| = {worst_abs:.3e} (largest |oracle| {ref_max:.2f}); "
          f"worst pair: {worst_rel_to_max:.2e} of its largest |oracle|")


def test_ssd_full_size_is_causal():
    c = make_ssd_case(B, L, H, P, G, N, Q, seed=12)
    y, _ = run_ssd(c)
    c2 = dict(c)
    cut = 1152                                     # a multiple of the kernel's 128-token block
    for k in ("q_x", "q_dt", "q_B", "q_C"):
        t = c[k].clone()
        t[:, cut:] = torch.roll(t[:, cut:], 1, dims=0)          # the tails of the batch rows change places
        c2[k] = t
    y2, _ = run_ssd(c2)
    assert torch.equal(y[:, :cut], y2[:, :cut])
    assert not torch.equal(y[:, cut:], y2[:, cut:])


def test_ssd_full_size_tensor_core_path_equals_portable_path():
    c = make_ssd_case(B, L, H, P, G, N, Q, seed=13)
    y_tc, f_tc = run_ssd(c)
    from quamba_b200 import _lib as qlib
    with qlib.path_override(qlib.PATH_SSD_PORTABLE):
        y_pt, f_pt = run_ssd(c)
    err = (y_tc.float() - y_pt.float()).abs()
    tol = 1e-2 * y_pt.float().abs() + 1e-3 * y_pt.float().abs().max()
    assert (err <= tol).all(), f"max err {err.max().item()}"
    d = (f_tc.int() - f_pt.int()).abs()
    assert d.max().item() <= 1 and (d > 0).float().mean().item() <= 0.03


@pytest.mark.parametrize("Bsz,Ls,Hs", [(8, 300, 80), (64, 100, 16), (2, 700, 80), (5, 1025, 37)])
def test_ssd_range_cuts_at_other_shapes(Bsz, Ls, Hs):
    """More (batch, head) pairs than SMs with 1, 3, 6 and 9 blocks per pair: the equal ranges then start and end in the
    middle of pairs at other places than in the benchmark shape (one block per pair: no cut inside a pair at all)."""
    c = make_ssd_case(Bsz, Ls, Hs, P, G, N, Q, seed=Ls)
    y_tc, f_tc = run_ssd(c)
    y_1, f_1 = run_ssd(c, slice(Bsz - 1, Bsz))          # fewer pairs than SMs: whole pairs per CTA
    assert torch.equal(y_tc[Bsz - 1], y_1[0]) and torch.equal(f_tc[Bsz - 1], f_1[0])
    from quamba_b200 import _lib as qlib
    with qlib.path_override(qlib.PATH_SSD_PORTABLE):
        y_pt, f_pt = run_ssd(c)
    err = (y_tc.float() - y_pt.float()).abs()
    tol = 1e-2 * y_pt.float().abs() + 1e-3 * y_pt.float().abs().max()
    assert (err <= tol).all(), f"max err {err.max().item()}"
    d = (f_tc.int() - f_pt.int()).abs()
    assert d.max().item() <= 1 and (d > 0).float().mean().item() <= 0.03


def test_ssd_range_cuts_with_grouped_scales_and_per_channel_D():
    """192 pairs (more than SMs, so ranges are cut inside pairs), four SSD groups with grouped scale tables, D per channel
    (the output step then re-reads x), 700 tokens (the last block of every pair is ragged)."""
    Bsz, Ls, Hs, Gs = 6, 700, 32, 4
    c = make_ssd_case(Bsz, Ls, Hs, P, Gs, N, Q, grouped=True, seed=77, d_has_hdim=True)

    def run(sl=slice(None)):
        y, fs = ops()._quamba2_mamba_chunk_scan_combined_fwd(
            dev(c["q_x"][sl]), dev(c["x_scales"]), dev(c["hgr"]), dev(c["dgr"]), dev(c["q_dt"][sl]), dev(c["s_dt"]), dev(c["q_A_log"]),
            dev(c["s_A"]), dev(c["q_B"][sl]), dev(c["s_B"]), dev(c["q_C"][sl]), dev(c["s_C"]), dev(c["state_scale"]), c["chunk"],
            dev(c["q_D"]), dev(c["s_D"]), None, None, dev(c["dt_bias"]), None, None, None, True)
        torch.cuda.synchronize()
        from quamba_b200 import _lib
        _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
        return y, fs

    y_tc, f_tc = run()
    y_1, f_1 = run(slice(2, 3))
    assert torch.equal(y_tc[2], y_1[0]) and torch.equal(f_tc[2], f_1[0])
    from quamba_b200 import _lib as qlib
    with qlib.path_override(qlib.PATH_SSD_PORTABLE):
        y_pt, f_pt = run()
    err = (y_tc.float() - y_pt.float()).abs()
    tol = 1e-2 * y_pt.float().abs() + 1e-3 * y_pt.float().abs().max()
    assert (err <= tol).all(), f"max err {err.max().item()}"
    d = (f_tc.int() - f_pt.int()).abs()
    assert d.max().item() <= 1 and (d > 0).float().mean().item() <= 0.03


def run_conv(c, xBC):
    o = ops().quamba2_conv1d_cuda.fwd(dev(xBC), c["sx"], c["sB"], c["sC"], c["x_dim"], P, N, G, dev(c["hgr"]), dev(c["dgr"]),
                                      dev(c["x_scales"]), dev(c["B_scales"]), dev(c["C_scales"]), dev(c["weight"]), c["swx"], c["swB"],
                                      c["swC"], dev(c["bias"]), c["sbx"], c["sbB"], c["sbC"], None, None, None, True)
    torch.cuda.synchronize()
    return o


def test_conv_full_size_batch_independence_and_causality():
    c = make_conv2_case(B, L, H, P, G, N, seed=21)
    x, Bm, Cm = run_conv(c, c["xBC"])
    assert x.shape == (B, H * P, L) and Bm.shape == (B, G * N, L)
    for b in (0, B - 1):
        x1, B1, C1 = run_conv(c, c["xBC"][b:b + 1])
        assert torch.equal(x[b], x1[0]) and torch.equal(Bm[b], B1[0]) and torch.equal(Cm[b], C1[0])
    # a change at step t reaches outputs t .. t + width - 1 and nothing before
    t = 1000
    xBC2 = c["xBC"].clone()
    xBC2[:, :, t] = torch.roll(xBC2[:, :, t], 1, dims=0)
    x2, B2, C2 = run_conv(c, xBC2)
    assert torch.equal(x[:, :, :t], x2[:, :, :t]) and torch.equal(x[:, :, t + 4:], x2[:, :, t + 4:])
    assert torch.equal(Cm[:, :, :t], C2[:, :, :t]) and torch.equal(Cm[:, :, t + 4:], C2[:, :, t + 4:])


def test_sscan_full_size_batch_independence_and_causality():
    # the Mamba1 layer shape of the baseline's scan benchmark, batch 4 to keep the test short
    Bs, D, Ls, Ns = 4, 5120, 1024, 16
    c = make_sscan_case(Bs, D, Ls, Ns, seed=31)

    def run(sl=slice(None), mod=None):
        t = {k: (mod[k] if mod and k in mod else c[k]) for k in ("q_u", "q_delta", "q_B", "q_C", "q_z")}
        out, x = ops().quant_sscan_cuda.fwd(dev(t["q_u"][sl]), dev(c["s_u"]), dev(t["q_delta"][sl]), dev(c["s_delta"]), dev(c["q_A"]),
                                            dev(c["s_A"]), dev(t["q_B"][sl]), dev(c["s_B"]), dev(t["q_C"][sl]), dev(c["s_C"]),
                                            dev(c["s_state"]), dev(c["q_D"]), dev(c["s_D"]), dev(t["q_z"][sl]), dev(c["s_z"]),
                                            dev(c["q_bias"]), dev(c["s_bias"]), True)
        torch.cuda.synchronize()
        return out, x

    out, x = run()
    assert out.shape == (Bs, Ls, D) and torch.isfinite(out.float()).all()
    out1, x1 = run(slice(2, 3))
    assert torch.equal(out[2], out1[0]) and torch.equal(x[2], x1[0])
    cut = 700
    mod = {}
    for k in ("q_u", "q_delta", "q_B", "q_C", "q_z"):
        t = c[k].clone()
        t[..., cut:] = torch.roll(t[..., cut:], 1, dims=0)
        mod[k] = t
    out2, _ = run(mod=mod)
    assert torch.equal(out[:, :cut], out2[:, :cut]) and not torch.equal(out[:, cut:], out2[:, cut:])


def test_hadamard_full_size_rows_are_independent():
    torch.manual_seed(41)
    rows, dim = 8192, 5120
    x = torch.randn(rows, dim, dtype=torch.float16, device=DEV)
    y = ops().quant_hadamard.fast_hadamard_transform_40N(x, 0.4)
    perm = torch.randperm(rows, device=DEV)
    yp = ops().quant_hadamard.fast_hadamard_transform_40N(x[perm].contiguous(), 0.4)
    assert torch.equal(y[perm], yp)
    # H (-x) = -(H x) survives rounding half away from zero and symmetric saturation
    yn = ops().quant_hadamard.fast_hadamard_transform_40N((-x).contiguous(), 0.4)
    sat = (y == -128) | (yn == -128)
    assert torch.equal(yn[~sat], (-y.int()[~sat]).to(torch.int8)) and sat.float().mean().item() < 1e-3
