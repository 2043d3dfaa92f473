"""GPU parity against the REFERENCE's own CUDA kernels, compiled for sm_100a from the reference checkout by
oracle/build_ref.py into oracle/_ref/ (checker binaries, never part of the product).  Every test runs the reference
extension and this package's entry point on the same device tensors:

    quant_sscan_cuda.fwd, quant_causal_conv1d_cuda.fwd / .update, quamba2_conv1d_cuda.fwd / .update,
    quant_hadamard.fast_hadamard_transform{,_12N,_40N}, quant_embedding_cuda.w4a16 / w8a16_embedding_lookup

Tolerances: int8 outputs +-1 LSB (the two sides differ in fast-math SiLU / exp and in summation order), fp16 scan outputs
1e-2 relative + 1e-3 of the output's largest magnitude, embeddings exact.  Skipped when the binaries are absent (they
are built where the reference checkout is mounted and travel with the tree)."""
import importlib.util
from pathlib import Path

import pytest
import torch

from helpers import make_conv2_case, make_sscan_case, q8

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


def ref(name):
    so = REF_DIR / name / f"{name}.so"
    if not so.exists():
        pytest.skip(f"{so} not built (python oracle/build_ref.py <reference checkout>)")
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def ops():
    from quamba_b200 import ops as o
    return o


def dev(t):
    return None if t is None else t.to(DEV)


def lsb(got, want, what, max_frac=0.02):
    d = (got.int() - want.int()).abs()
    frac = (d > 0).float().mean().item()
    assert d.max().item() <= 1 and frac <= max_frac, f"{what}: max diff {d.max().item()} LSB, {frac:.5f} of elements differ"
    return frac


@pytest.mark.parametrize("Bsz,D,L,N,with_z", [(1, 1536, 512, 16, True), (2, 256, 2300, 16, True), (1, 128, 33, 16, False)])
def test_mamba1_scan_against_reference_kernel(Bsz, D, L, N, with_z):
    r = ref("quant_sscan_cuda")
    c = {k: dev(v) for k, v in make_sscan_case(Bsz, D, L, N, seed=L, with_z=with_z).items()}
    args = (c["q_u"], c["s_u"], c["q_delta"], c["s_delta"], c["q_A"], c["s_A"], c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["s_state"],
            c["q_D"], c["s_D"], c["q_z"], c["s_z"], c["q_bias"], c["s_bias"], True)
    want_y, want_x = r.fwd(*args)
    got_y, got_x = ops().quant_sscan_cuda.fwd(*args)
    torch.cuda.synchronize()
    assert got_y.shape == want_y.shape and got_x.shape == want_x.shape
    w = want_y.float()
    err = (got_y.float() - w).abs()
    assert (err <= 1e-3 * w.abs().max() + 1e-2 * w.abs()).all(), f"max err {err.max().item():.4g} of {w.abs().max().item():.4g}"
    lsb(got_x, want_x, "scan states")
    print(f"sscan B{Bsz} D{D} L{L}: max |y - reference| {err.max().item():.3e}, max |reference| {w.abs().max().item():.3f}")


@pytest.mark.parametrize("Bsz,D,L,channel_last", [(2, 256, 1024, False), (1, 512, 333, False), (2, 384, 200, True)])
def test_quamba1_conv_against_reference_kernel(Bsz, D, L, channel_last):
    r = ref("quant_causal_conv1d_cuda")
    g = torch.Generator().manual_seed(L)
    x, sx = q8(torch.randn(Bsz, D, L, generator=g))
    w, sw = q8(torch.randn(D, 4, generator=g) * 0.2)
    b, sb = q8(torch.randn(D, generator=g) * 0.02)
    x = dev(x)
    if channel_last:
        x = x.transpose(1, 2).contiguous().transpose(1, 2)
    args = (x, float(sx), dev(w), float(sw), 0.02, float(sb), dev(b), None, None, None, True)
    want = r.fwd(*args)
    got = ops().quant_causal_conv1d_cuda.fwd(*args)
    assert got.stride() == want.stride()
    lsb(got, want, "conv fwd")
    # decode steps continue the sequence on both sides
    st_r = torch.zeros(Bsz, D, 4, dtype=torch.int8, device=DEV)
    st_g = st_r.clone()
    for t in range(6):
        xt = x[:, :, t].contiguous()
        wr = r.update(xt, st_r, float(sx), dev(w), float(sw), 0.02, float(sb), dev(b), True)
        gr = ops().quant_causal_conv1d_cuda.update(xt, st_g, float(sx), dev(w), float(sw), 0.02, float(sb), dev(b), True)
        lsb(gr, wr, f"conv update step {t}")
        assert torch.equal(st_r, st_g)


@pytest.mark.parametrize("Bsz,L,H,P,G,N,grouped", [(2, 257, 8, 64, 1, 128, False), (1, 512, 80, 64, 1, 128, False),
                                                   (1, 130, 8, 64, 2, 64, True), (2, 64, 16, 64, 8, 128, True)])
def test_quamba2_conv_against_reference_kernel(Bsz, L, H, P, G, N, grouped):
    r = ref("quamba2_conv1d_cuda")
    c = make_conv2_case(Bsz, L, H, P, G, N, grouped=grouped, seed=L + H)
    xBC = c["xBC"].transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    args = (xBC, c["sx"], c["sB"], c["sC"], c["x_dim"], P, N, G, dev(c["hgr"]), dev(c["dgr"]), dev(c["x_scales"]), dev(c["B_scales"]),
            dev(c["C_scales"]), dev(c["weight"]), c["swx"], c["swB"], c["swC"], dev(c["bias"]), c["sbx"], c["sbB"], c["sbC"], None, None,
            None, True)
    want = r.fwd(*args)
    got = ops().quamba2_conv1d_cuda.fwd(*args)
    for g_, w_, n in zip(got, want, "xBC"):
        assert g_.shape == w_.shape
        lsb(g_, w_, f"quamba2 conv fwd {n}")
    C = xBC.shape[1]
    st_r = torch.zeros(Bsz, 4, C, dtype=torch.int8, device=DEV).transpose(1, 2)
    st_g = st_r.clone().transpose(1, 2).contiguous().transpose(1, 2)
    for t in range(5):
        xt = xBC[:, :, t].contiguous()
        a2 = (xt,) + args[1:]
        wr = r.update(xt, st_r, *args[1:])
        gr = ops().quamba2_conv1d_cuda.update(xt, st_g, *args[1:])
        for g_, w_, n in zip(gr, wr, "xBC"):
            lsb(g_, w_, f"quamba2 conv update {n} step {t}")
        assert torch.equal(st_r, st_g)


@pytest.mark.parametrize("rows,dim,fn", [(64, 5120, "fast_hadamard_transform_40N"), (33, 1536, "fast_hadamard_transform_12N"),
                                         (128, 8192, "fast_hadamard_transform"), (7, 512, "fast_hadamard_transform"),
                                         (16, 2560, "fast_hadamard_transform_20N")])
def test_hadamard_against_reference_kernel(rows, dim, fn):
    r = ref("quant_hadamard")
    g = torch.Generator().manual_seed(dim + rows)
    x = torch.randn(rows, dim, generator=g).to(torch.float16).to(DEV)
    scale = (1.0 / dim ** 0.5) / 0.05           # results have a standard deviation of 20: none reaches 127, where the reference wraps
    want = getattr(r, fn)(x, scale)
    got = getattr(ops().quant_hadamard, fn)(x, scale)
    lsb(got, want, fn)


def test_embedding_against_reference_kernel():
    r = ref("quant_embedding_cuda")
    from oracle import embedding as oemb
    g = torch.Generator().manual_seed(0)
    table = torch.randn(300, 2560, generator=g) * 0.02
    ids = torch.randint(0, 300, (3, 40), generator=g).to(DEV)
    p4, s4 = oemb.pack_w4(table)
    assert torch.equal(ops().quant_embedding_cuda.w4a16_embedding_lookup(ids, dev(p4), dev(s4)),
                       r.w4a16_embedding_lookup(ids, dev(p4), dev(s4)))
    p8, s8 = oemb.pack_w8(table)
    assert torch.equal(ops().quant_embedding_cuda.w8a16_embedding_lookup(ids, dev(p8), dev(s8)),
                       r.w8a16_embedding_lookup(ids, dev(p8), dev(s8)))


def _time_us(fn, reps=20, warm=3):
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def test_speed_beside_the_reference_kernels():
    """The reference's kernels (compiled for sm_100a, unchanged) timed beside this package's at the per-layer shapes of
    the models they serve: same device tensors, eager launches through each side's Python binding, CUDA events, 20
    repetitions.  Both sides pay their own host-side launch path, so the small decode shapes compare bindings as much as
    kernels.  The table is printed (pytest -s) and written to $QB_REF_TIMING_JSON when that is set."""
    import json
    import os
    rows = {}
    # Quamba2 conv1d forward, B4 L2048 (80 heads x 64, one group, d_state 128)
    r = ref("quamba2_conv1d_cuda")
    c = make_conv2_case(4, 2048, 80, 64, 1, 128, grouped=False, seed=1)
    xBC = c["xBC"].transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    args = (xBC, c["sx"], c["sB"], c["sC"], c["x_dim"], 64, 128, 1, None, None, dev(c["x_scales"]), dev(c["B_scales"]), dev(c["C_scales"]),
            dev(c["weight"]), c["swx"], c["swB"], c["swC"], dev(c["bias"]), c["sbx"], c["sbB"], c["sbC"], None, None, None, True)
    rows["quamba2_conv1d fwd B4 L2048 C5376"] = (_time_us(lambda: r.fwd(*args)), _time_us(lambda: ops().quamba2_conv1d_cuda.fwd(*args)))
    # Hadamard 40 x 128 + quantise, 8192 rows
    r = ref("quant_hadamard")
    x = torch.randn(8192, 5120, generator=torch.Generator().manual_seed(0)).to(torch.float16).to(DEV)
    rows["hadamard_40N 8192 x 5120"] = (_time_us(lambda: r.fast_hadamard_transform_40N(x, 0.3)),
                                        _time_us(lambda: ops().quant_hadamard.fast_hadamard_transform_40N(x, 0.3)))
    # Mamba1 selective scan, B16 D5120 L1024 N16
    r = ref("quant_sscan_cuda")
    s = {k: dev(v) for k, v in make_sscan_case(16, 5120, 1024, 16, seed=2, with_z=True).items()}
    sargs = (s["q_u"], s["s_u"], s["q_delta"], s["s_delta"], s["q_A"], s["s_A"], s["q_B"], s["s_B"], s["q_C"], s["s_C"], s["s_state"],
             s["q_D"], s["s_D"], s["q_z"], s["s_z"], s["q_bias"], s["s_bias"], True)
    rows["sscan fwd B16 D5120 L1024 N16"] = (_time_us(lambda: r.fwd(*sargs), reps=5), _time_us(lambda: ops().quant_sscan_cuda.fwd(*sargs), reps=5))
    # Quamba1 conv1d forward, B16 D5120 L1024
    r = ref("quant_causal_conv1d_cuda")
    g = torch.Generator().manual_seed(3)
    xq, sx = q8(torch.randn(16, 5120, 1024, generator=g))
    w, sw = q8(torch.randn(5120, 4, generator=g) * 0.2)
    b, sb = q8(torch.randn(5120, generator=g) * 0.02)
    cargs = (dev(xq), float(sx), dev(w), float(sw), 0.02, float(sb), dev(b), None, None, None, True)
    rows["causal_conv1d fwd B16 D5120 L1024"] = (_time_us(lambda: r.fwd(*cargs)), _time_us(lambda: ops().quant_causal_conv1d_cuda.fwd(*cargs)))
    out = {k: {"reference_us": round(a, 2), "this_us": round(b_, 2), "speedup": round(a / b_, 2)} for k, (a, b_) in rows.items()}
    for k, v in out.items():
        print(f"{k:40s} reference {v['reference_us']:9.1f} us   this package {v['this_us']:9.1f} us   x{v['speedup']}")
        assert v["this_us"] > 0 and v["reference_us"] > 0
    if os.environ.get("QB_REF_TIMING_JSON"):
        with open(os.environ["QB_REF_TIMING_JSON"], "w") as f:
            json.dump(out, f, indent=1)
