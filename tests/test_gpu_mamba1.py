"""GPU parity of the Mamba1 mixers W8A8QMamba / W4A8QMamba (in_proj -> conv1d -> x_proj -> dt_proj -> int8 selective scan ->
Hadamard -> out_proj, quamba/qMambaLayer.py:512-1003) against the CPU oracle's composition of the same ops: prefill with
cache fill, then decode steps that continue from the GPU's own int8 caches (so that +-1 LSB differences do not accumulate).
Tolerances: fp16 layer outputs within 1e-2 relative + 3e-2 of the largest |reference| on at least 98 % of the elements
(+-1 LSB flips of int8 activations propagate through four quantised products), conv cache bit-exact, ssm cache +-1 LSB."""
import copy

import pytest
import torch

from oracle import model as omodel

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, what, max_frac=0.02):
    want = want.float()
    err = (got.cpu().float() - want).abs()
    frac = (err > 3e-2 * want.abs().max() + 1e-2 * want.abs()).float().mean().item()
    assert frac <= max_frac, f"{what}: {frac:.4f} of elements outside tolerance, max err {err.max().item():.4g} of {want.abs().max().item():.4g}"


def _layer(cls_name, seed, d_model=256, use_had=True, L=70, batch=2):
    from quamba_b200 import calibrate as cal, mixer1
    g = torch.Generator().manual_seed(seed)
    fl = cal.Mamba1Float(d_model, layer_idx=0, generator=g, w4_group_size=128)
    u = torch.randn(batch, L, d_model, generator=g)
    s = cal.calibrate_mamba1(fl, [u])
    q = getattr(mixer1, cls_name).from_fp16(fl, s, use_had_transform=use_had)
    u8 = (u / s["in_proj:input"]).round().clamp(-128, 127).to(torch.int8)
    return q, u8


@pytest.mark.parametrize("cls_name,use_had,batch", [("W8A8QMamba", True, 2), ("W4A8QMamba", True, 2), ("W8A8QMamba", False, 1),
                                                    ("W4A8QMamba", True, 1)])
def test_mamba1_layer_prefill_and_decode_match_oracle(cls_name, use_had, batch):
    from quamba_b200 import _lib
    from quamba_b200.model import InferenceParams
    q, u8 = _layer(cls_name, seed=7 + batch, use_had=use_had, batch=batch)
    L = u8.shape[1]
    want, want_conv, want_ssm = omodel.mamba1_forward(q, u8[:, :L - 3], want_states=True)
    gq = copy.deepcopy(q).to(DEV)
    params = InferenceParams(max_seqlen=L, max_batch_size=batch)
    got = gq(u8[:, :L - 3].to(DEV), inference_params=params)
    torch.cuda.synchronize()
    _close(got, want, f"{cls_name} prefill")
    conv, ssm = params.key_value_memory_dict[0]
    assert torch.equal(conv.cpu(), want_conv), "conv cache after prefill"
    assert (ssm.cpu().int() - want_ssm.int()).abs().max().item() <= 1, "ssm cache after prefill"
    # the same layer without caches gives the same output
    assert torch.equal(gq(u8[:, :L - 3].to(DEV)), got)
    for t in range(L - 3, L):
        params.seqlen_offset = t
        cpu_conv, cpu_ssm = conv.cpu().clone(), ssm.cpu().clone()
        got_t = gq(u8[:, t:t + 1].to(DEV), inference_params=params)
        want_t = omodel.mamba1_step(q, u8[:, t], cpu_conv, cpu_ssm)
        _close(got_t[:, 0], want_t, f"{cls_name} decode step {t}")
        assert torch.equal(conv.cpu(), cpu_conv), f"conv cache after step {t}"
        assert (ssm.cpu().int() - cpu_ssm.int()).abs().max().item() <= 1, f"ssm cache after step {t}"
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)


def test_mamba1_layer_state_dict_round_trip():
    """The mixer's buffers and float scales survive state_dict -> a freshly constructed layer (the reference's checkpoint
    layout: module names in_proj, conv1d, x_proj, dt_proj, selective_scan, had, out_proj)."""
    from quamba_b200.mixer1 import W8A8QMamba
    q, u8 = _layer("W8A8QMamba", seed=3, batch=1, L=20)
    sd = q.state_dict()
    for name in ("in_proj.weight", "conv1d.weight", "x_proj.weight", "dt_proj.weight", "selective_scan.A_log", "out_proj.weight",
                 "had.x_H_scale"):
        assert name in sd, name
    fresh = W8A8QMamba(d_model=256, layer_idx=0, device="cpu")
    fresh.load_state_dict(sd)
    a = copy.deepcopy(q).to(DEV)(u8.to(DEV))
    b = fresh.to(DEV)(u8.to(DEV))
    assert torch.equal(a, b)


@pytest.mark.parametrize("w_bits", [8, 4])
def test_mamba1_model_prefill_and_graph_decode_match_oracle(w_bits):
    """A two-layer Mamba1 model in the model shell (block norms with fused residual add, final norm, head): graph-replayed
    prefill and three graph-replayed decode steps against the oracle; the decode graph also feeds the greedy token back."""
    from quamba_b200 import _lib, calibrate as cal, ops
    fm = cal.Mamba1LMFloat(d_model=256, n_layer=2, vocab_size=320, seed=5, w4_group_size=128)
    ids = torch.randint(0, 320, (2, 90), generator=torch.Generator().manual_seed(1))
    q = cal.quantize_mamba1_model(fm, [ids], w_bits=w_bits)
    want = omodel.model_forward(q, ids, num_last_tokens=1)[:, -1]
    gq = copy.deepcopy(q).to(DEV)
    pre = gq.capture_prefill(2, 90)
    pre.input_ids.copy_(ids)
    got = pre.replay()
    torch.cuda.synchronize()
    _close(got, want, "Mamba1 model prefill logits")
    params = pre.inference_params
    params.seqlen_offset = 90
    dec = gq.capture_decode(2, 128, inference_params=params)
    tok = ops.greedy_next_token(got.contiguous())
    for step in range(3):
        states = {k: tuple(t.cpu().clone() for t in v) for k, v in params.key_value_memory_dict.items()}
        dec.input_ids.copy_(tok[:, None])
        logits = dec.replay().clone()
        _close(logits, omodel.model_step(q, tok.cpu(), states), f"Mamba1 model decode step {step}")
        nxt = dec.input_ids[:, 0].clone()
        assert torch.equal(nxt.cpu(), logits.float().cpu().argmax(-1))
        tok = nxt
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
