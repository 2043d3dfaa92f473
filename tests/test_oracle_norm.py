"""CPU checks of the norm / embedding oracle against outputs of the reference's own code (tests/golden/norm_*.npz,
embedding_w4.npz: made by tests/golden/make_norm_golden.py), and of the host-side mirrors (modules, model shell,
calibration) that need no GPU."""
import numpy as np
import pytest
import torch

from helpers import load_golden
from oracle import embedding as oemb, model as omodel, norm as onorm
from quamba_b200 import calibrate as cal

STATIC = ["static_res32", "static_res16", "static_nores"]


def _lsb(got, want, max_frac=0.002):
    d = (got.int() - want.int()).abs()
    assert d.max().item() <= 1, f"max diff {d.max().item()} LSB"
    assert (d > 0).float().mean().item() <= max_frac, f"{(d > 0).float().mean().item():.5f} of elements differ"


@pytest.mark.parametrize("tag", STATIC + ["dynamic"])
def test_norm_oracle_matches_reference_triton_kernel(tag):
    g = load_golden(f"norm_{tag}.npz")
    static = float(g["static"]) or None
    res = g.get("res")
    y, res_out, scale = onorm.qlayer_norm_fwd(g["x"], g["w"], None, 1e-5, res, static_out_scale=static,
                                              residual_dtype=res.dtype if res is not None else None, is_rms_norm=True)
    _lsb(y, g["y"])
    if res is not None:
        assert torch.equal(res_out, g["res_out"])
    if static is None:
        torch.testing.assert_close(scale, g["dyn"], rtol=1e-5, atol=0)


@pytest.mark.parametrize("tag", ["f16_g1", "f16_g8", "f16_nbg", "s8_static", "s8_dynamic"])
def test_gated_norm_oracle_matches_reference_triton_kernel(tag):
    g = load_golden(f"norm_gated_{tag}.npz")
    f16 = g["y"].dtype == torch.float16
    static = float(g["static"]) or None
    y, scale = onorm.qlayer_normgated_fwd(g["x"], g["w"], None, 1e-5, q_z=g["qz"], z_scale=float(g["z_scale"]),
                                          static_out_scale=static, use_float16_output=f16, group_size=int(g["group_size"]),
                                          norm_before_gate=bool(g["norm_before_gate"]), is_rms_norm=True)
    if f16:
        torch.testing.assert_close(y.float(), g["y"].float(), rtol=2e-3, atol=1e-5)     # one fp16 ulp
    else:
        _lsb(y, g["y"])
        if static is None:
            torch.testing.assert_close(scale, g["dyn"], rtol=1e-5, atol=0)


def test_embedding_oracle_matches_reference_packer():
    g = load_golden("embedding_w4.npz")
    packed, scales = oemb.pack_w4(g["embed_w"])
    assert torch.equal(packed, g["packed"]) and torch.equal(scales, g["scales"])
    ids = torch.arange(g["packed"].shape[0])
    assert torch.equal(oemb.lookup_w4(ids, g["packed"], g["scales"]), g["rows"])


def test_embedding_module_packs_like_the_reference():
    from quamba_b200.embedding import W4O16Embedding, W8O16Embedding
    g = load_golden("embedding_w4.npz")
    emb = torch.nn.Embedding(*g["embed_w"].shape)
    emb.weight.data = g["embed_w"].clone()
    q = W4O16Embedding.from_fp16(emb)
    assert torch.equal(q.weight.data.cpu(), g["packed"]) and torch.equal(q.scales.cpu(), g["scales"])
    q8 = W8O16Embedding.from_fp16(emb)
    w8, s8 = oemb.pack_w8(g["embed_w"])
    assert torch.equal(q8.weight.data.cpu(), w8) and torch.equal(q8.scales.cpu(), s8)
    sd = q.state_dict()
    assert set(sd) == {"weight", "scales"} and sd["weight"].dtype == torch.int32


def _small_model(seed=0, group=None, n_layer=2):
    from quamba_b200 import calibrate as cal
    m = cal.Mamba2LMFloat(d_model=256, n_layer=n_layer, vocab_size=320, seed=seed, w4_group_size=group)
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, 320, (2, 48), generator=g) for _ in range(2)]
    return m, cal.calibrate(m, seqs), seqs


@pytest.mark.parametrize("group", [None, -1])
def test_calibrate_and_quantize_model_on_cpu(group, tmp_path):
    from quamba_b200 import calibrate as cal
    from quamba_b200.model import QuambaLMHeadModel
    m, scales, seqs = _small_model(group=group)
    assert len(scales) == 3 and "lm_head:input" in scales[-1]
    for k in ("in_proj:input", "x_conv_in:output", "x_conv_out:input", "ssm_state_act:input", "out_proj:input"):
        assert scales[0][k].numel() == 1 and scales[0][k].item() > 0
    q = cal.quantize_model(m, scales)
    mixer = q.backbone.layers[0].mixer
    assert (mixer.in_proj.s_group.numel() == 0) == (group == -1)
    # checkpoint round trip: save_pretrained -> from_pretrained (config.json + pytorch_model.bin, the reference's layout)
    q.save_pretrained(tmp_path)
    q2 = QuambaLMHeadModel.from_pretrained(tmp_path)
    assert set(q2.state_dict()) == set(q.state_dict())
    lo1 = omodel.model_forward(q, seqs[0])
    lo2 = omodel.model_forward(q2, seqs[0])
    assert torch.equal(lo1, lo2)
    # the quantized model tracks the float model it was made from
    lf = m(seqs[0])
    c = torch.corrcoef(torch.stack([lo1.float().flatten(), lf.flatten()]))[0, 1].item()
    assert c > (0.85 if group == -1 else 0.9), c


def test_oracle_decode_step_continues_the_prefill():
    m, scales, seqs = _small_model(seed=1)
    from quamba_b200 import calibrate as cal
    q = cal.quantize_model(m, scales)
    ids = seqs[0]
    states = {}
    lo = omodel.model_forward(q, ids[:, :-1], states=states)
    before = states[0][1].clone()
    step = omodel.model_step(q, ids[:, -1], states)
    assert states[0][1].abs().max().item() > 0 and not torch.equal(states[0][1], before)   # the int8 state moved on in place
    full = omodel.model_forward(q, ids)[:, -1]
    # the step starts from int8-rounded states, the prefill carries them in floating point
    assert (step.float() - full.float()).abs().max().item() < 0.05 * full.float().abs().max().item()


# ---- Mamba1 mixers and the W8A8 Mamba2 model on CPU ------------------------------------------------------------------------
@pytest.mark.parametrize("cls_name,tol", [("W8A8QMamba", 0.08), ("W4A8QMamba", 0.35)])
def test_mamba1_mixer_quantises_on_cpu_and_the_oracle_tracks_the_float_layer(cls_name, tol):
    """Float Mamba1 layer -> calibration -> W8A8QMamba / W4A8QMamba (buffers built on CPU) -> the oracle's composition of
    the Quamba1 ops stays within a quantisation-sized error of the float layer (4-bit weights of a 256-wide random layer
    are coarse: the bound reflects that), and a decode step from the prefill's caches equals the next token of a longer
    prefill up to +-1 LSB effects."""
    from quamba_b200 import mixer1
    g = torch.Generator().manual_seed(0)
    fl = cal.Mamba1Float(256, layer_idx=0, generator=g, w4_group_size=128)
    u = torch.randn(2, 33, 256, generator=g)
    s = cal.calibrate_mamba1(fl, [u])
    assert set(s) == {"in_proj:input", "in_proj:output", "x_proj:input", "x_proj:output", "dt_proj:output", "ssm_state_act:input",
                      "out_proj:input"}
    q = getattr(mixer1, cls_name).from_fp16(fl, s)
    u8 = (u / s["in_proj:input"]).round().clamp(-128, 127).to(torch.int8)
    with torch.no_grad():
        ref = fl(u)
    out, conv, ssm = omodel.mamba1_forward(q, u8, want_states=True)
    assert out.dtype == torch.float16 and conv.shape == (2, 512, 4) and ssm.shape == (2, 512, 16) and ssm.dtype == torch.int8
    err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < tol, f"oracle vs float layer: {err:.3f} of the largest output"
    head, conv_h, ssm_h = omodel.mamba1_forward(q, u8[:, :-1], want_states=True)
    step = omodel.mamba1_step(q, u8[:, -1], conv_h, ssm_h)      # moves both caches on in place
    assert torch.equal(conv_h, conv)
    assert (ssm_h.int() - ssm.int()).abs().max().item() <= 1
    d = (step.float() - out[:, -1].float()).abs().max().item() / out.float().abs().max().item()
    assert d < 0.05, f"decode step vs last prefill token: {d:.3f}"


def test_w8a8_mamba2_model_oracle_on_cpu():
    """quantize_model(w_bits=8) builds the reference's default layer class on CPU; the model oracle reads its W8A8 layers
    (GEMM form for several rows, the two GEMV forms for one) and tracks the float model."""
    from quamba_b200.mixer import W8A8QMamba2
    m = cal.Mamba2LMFloat(d_model=256, n_layer=2, vocab_size=320, seed=3)
    ids = torch.randint(0, 320, (1, 40), generator=torch.Generator().manual_seed(0))
    q = cal.quantize_model(m, cal.calibrate(m, [ids]), w_bits=8)
    assert isinstance(q.backbone.layers[0].mixer, W8A8QMamba2)
    st = {}
    lg = omodel.model_forward(q, ids, num_last_tokens=1, states=st)[:, -1]
    with torch.no_grad():
        ref = m(ids)[:, -1]
    assert (lg.float() - ref).abs().max().item() < 0.15 * ref.abs().max().item()
    nxt = omodel.model_step(q, lg.argmax(-1), st)
    assert nxt.shape == (1, 320) and torch.isfinite(nxt.float()).all()
