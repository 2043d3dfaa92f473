"""GPU parity tests of the norm / embedding kernels, the Mamba2 mixer layer and the model shell, all through the C ABI.

Tolerances: int8 outputs within +-1 LSB of the reference-made golden vectors and of the CPU oracle; fp16 outputs
within one fp16 ulp (norms) or 1e-2 relative + 1e-3 absolute on the output's scale (layer and model outputs, where
+-1 LSB flips of intermediate int8 activations propagate)."""
import pytest
import torch

from helpers import load_golden
from oracle import embedding as oemb, model as omodel, norm as onorm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ops():
    from quamba_b200 import ops as o
    return o


def _lsb(got, want, max_frac=0.002):
    d = (got.cpu().int() - want.int()).abs()
    assert d.max().item() <= 1, f"max diff {d.max().item()} LSB"
    assert (d > 0).float().mean().item() <= max_frac, f"{(d > 0).float().mean().item():.5f} of elements differ"


@pytest.mark.parametrize("tag", ["static_res32", "static_res16", "static_nores", "dynamic"])
def test_rmsnorm_against_reference_triton_golden(tag):
    g = load_golden(f"norm_{tag}.npz")
    static = float(g["static"]) or None
    res = g.get("res")
    y, res_out, scale = ops()._qlayer_norm_fwd(g["x"].to(DEV), g["w"].to(DEV), None, 1e-5, None if res is None else res.to(DEV),
                                               static_out_scale=static, is_rms_norm=True)
    _lsb(y, g["y"])
    if res is not None:
        assert torch.equal(res_out.cpu(), g["res_out"])
    if static is None:
        torch.testing.assert_close(scale.cpu(), g["dyn"], rtol=1e-5, atol=0)


@pytest.mark.parametrize("tag", ["f16_g1", "f16_g8", "f16_nbg", "s8_static", "s8_dynamic"])
def test_gated_rmsnorm_against_reference_triton_golden(tag):
    g = load_golden(f"norm_gated_{tag}.npz")
    f16 = g["y"].dtype == torch.float16
    static = float(g["static"]) or None
    y, scale = ops()._qlayer_normgated_fwd(g["x"].to(DEV), g["w"].to(DEV), None, 1e-5, q_z=g["qz"].to(DEV),
                                           z_scale=float(g["z_scale"]), static_out_scale=static, use_float16_output=f16,
                                           group_size=int(g["group_size"]), norm_before_gate=bool(g["norm_before_gate"]),
                                           is_rms_norm=True)
    if f16:
        torch.testing.assert_close(y.cpu().float(), g["y"].float(), rtol=2e-3, atol=1e-5)
    else:
        _lsb(y, g["y"])
        if static is None:
            torch.testing.assert_close(scale.cpu(), g["dyn"], rtol=1e-5, atol=0)


@pytest.mark.parametrize("M,N,res_dtype,rms", [(1, 2560, torch.float32, True), (300, 2560, torch.float32, True),
                                               (7, 4096, torch.float16, True), (3, 20480, None, True),
                                               (5, 1000, torch.float32, True), (9, 77, torch.float16, False),
                                               (4, 768, torch.float16, False), (0, 256, None, True)])
def test_rmsnorm_shapes_against_oracle(M, N, res_dtype, rms):
    g = torch.Generator().manual_seed(M * 131 + N)
    x = torch.randn(M, N, generator=g).to(torch.float16)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.float16)
    res = None if res_dtype is None else (3 * torch.randn(M, N, generator=g)).to(res_dtype)
    want, want_res, _ = onorm.qlayer_norm_fwd(x, w, None, 1e-5, res, static_out_scale=0.02, residual_dtype=res_dtype, is_rms_norm=rms)
    got, got_res, _ = ops()._qlayer_norm_fwd(x.to(DEV), w.to(DEV), None, 1e-5, None if res is None else res.to(DEV),
                                             static_out_scale=0.02, is_rms_norm=rms)
    assert got.shape == want.shape
    if M:
        _lsb(got, want)
        assert torch.equal(got_res.cpu(), want_res)


def test_rmsnorm_strided_rows_and_gate_view():
    """The mixer hands the gate over as a column block of in_proj's output; the final norm gets the last rows only."""
    g = torch.Generator().manual_seed(5)
    M, N, S = 37, 1024, 2368
    buf = torch.randint(-128, 128, (M, S), generator=g, dtype=torch.int8)
    y = torch.randn(M, N, generator=g).to(torch.float16)
    w = torch.ones(N, dtype=torch.float16)
    want, _ = onorm.qlayer_normgated_fwd(y, w, None, 1e-5, q_z=buf[:, :N], z_scale=0.03, use_float16_output=True, group_size=256,
                                         norm_before_gate=False)
    got, _ = ops()._qlayer_normgated_fwd(y.to(DEV), w.to(DEV), None, 1e-5, q_z=buf.to(DEV)[:, :N], z_scale=0.03,
                                         use_float16_output=True, group_size=256, norm_before_gate=False, is_rms_norm=True)
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2e-3, atol=1e-5)


def test_norm_rejects_what_the_reference_rejects():
    x = torch.zeros(2, 40000, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="64KB"):
        ops()._qlayer_norm_fwd(x, torch.ones(40000, dtype=torch.float16, device=DEV), None, 1e-5, static_out_scale=0.1)


def test_embedding_lookup_all_kinds():
    g = load_golden("embedding_w4.npz")
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, g["packed"].shape[0], (3, 17), generator=gen)
    got = ops().quant_embedding_cuda.w4a16_embedding_lookup(ids.to(DEV), g["packed"].to(DEV), g["scales"].to(DEV))
    assert torch.equal(got.cpu(), g["rows"][ids])
    w8, s8 = oemb.pack_w8(g["embed_w"])
    got8 = ops().quant_embedding_cuda.w8a16_embedding_lookup(ids.to(DEV)[0], w8.to(DEV), s8.to(DEV))
    assert torch.equal(got8.cpu(), oemb.lookup_w8(ids[0], w8, s8))
    tab = g["embed_w"].to(torch.float16)
    got16 = ops().quant_embedding_cuda.f16_embedding_lookup(ids.to(DEV), tab.to(DEV))
    assert torch.equal(got16.cpu(), tab[ids])


def test_embedding_reports_bad_token_ids():
    from quamba_b200 import _lib
    g = load_golden("embedding_w4.npz")
    ids = torch.tensor([1, 10_000], device=DEV)
    ops().quant_embedding_cuda.w4a16_embedding_lookup(ids, g["packed"].to(DEV), g["scales"].to(DEV))
    with pytest.raises(RuntimeError, match="token id"):
        _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)        # cleared by the read


def test_greedy_next_token():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(5, 50288, generator=g).to(torch.float16)
    logits[2, 777] = logits[2, 4000] = 30.0          # a tie: the lower index wins
    got = ops().greedy_next_token(logits.to(DEV))
    want = logits.float().argmax(-1)
    want[2] = 777
    assert torch.equal(got.cpu(), want)
    padded = torch.zeros(5, 50304, dtype=torch.float16)
    padded[:, :50288] = logits
    assert torch.equal(ops().greedy_next_token(padded.to(DEV)[:, :50288]).cpu(), want)


# ---- layer and model --------------------------------------------------------------------------------------------------
def _small(seed, group, d_model=256, n_layer=2, vocab=320, L=300, batch=2, w_bits=4):
    from quamba_b200 import calibrate as cal
    m = cal.Mamba2LMFloat(d_model=d_model, n_layer=n_layer, vocab_size=vocab, seed=seed, w4_group_size=group)
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (batch, L), generator=g)
    q = cal.quantize_model(m, cal.calibrate(m, [ids]), w_bits=w_bits)
    return q, ids


def _close(got, want, what, atol_rel=1e-3, max_frac=0.0):
    want = want.float()
    err = (got.cpu().float() - want).abs()
    tol = atol_rel * want.abs().max() + 1e-2 * want.abs()
    frac = (err > tol).float().mean().item()
    assert frac <= max_frac, (f"{what}: {frac:.4f} of elements outside 1e-2 rel + {atol_rel:g} x max abs, max err "
                              f"{err.max().item():.4g} of {want.abs().max().item():.4g}")


@pytest.mark.parametrize("group", [None, -1])
def test_mixer_layer_stage_by_stage(group):
    """One W4A8QMamba2 layer on the GPU with every sub-module's output captured; each stage is then re-computed by the
    CPU oracle FROM THE GPU'S OWN INPUTS to that stage, so each comparison is at that op's tolerance (exact for the two
    GEMMs, +-1 LSB for conv and Hadamard-quant, fp16 for SSD and the gated norm) and nothing accumulates."""
    import copy
    from oracle import conv1d as oconv, hadamard as ohad, ssd as ossd
    from quamba_b200.model import InferenceParams
    q, ids = _small(3, group, n_layer=1, L=300)
    m = q.backbone.layers[0].mixer
    gm = copy.deepcopy(m).to(DEV)
    cap = {}
    for name in ("in_proj", "conv1d", "qchunk_scan", "norm", "had", "out_proj"):
        getattr(gm, name).register_forward_hook(lambda mod, inp, out, name=name: cap.__setitem__(name, (inp, out)))
    g = torch.Generator().manual_seed(9)
    b, l = 2, 300
    u = torch.randint(-127, 128, (b, l, 256), generator=g, dtype=torch.int8)
    params = InferenceParams(max_seqlen=l + 1, max_batch_size=b)
    got = gm(u.to(DEV), inference_params=params)
    cpu = lambda t: t.cpu() if torch.is_tensor(t) else t
    # in_proj: exact
    zx = cpu(cap["in_proj"][1])
    assert torch.equal(zx.reshape(b * l, -1), omodel._w4a8(m.in_proj, u.reshape(b * l, -1), True))
    # conv on the GPU's xBC: +-1 LSB
    xBC = cpu(cap["conv1d"][0][0])
    want_x, want_B, want_C = oconv.quamba2_conv1d_fwd(xBC, *omodel._conv_args(m.conv1d))
    gx, gB, gC = (cpu(t) for t in cap["conv1d"][1])
    for a_, w_ in ((gx, want_x), (gB, want_B), (gC, want_C)):
        _lsb(a_, w_, max_frac=0.02)
    # SSD on the GPU's conv outputs: fp16 tolerance, final state +-1 LSB
    sx, sdt, sB, sC = (cpu(t) for t in cap["qchunk_scan"][0][:4])
    s = m.qchunk_scan
    want_y, want_last = ossd.chunk_scan_faithful(sx, s.x_scales, None, None, sdt, s.dt_scale, s.A_log, s.A_log_scale, sB, s.B_scale, sC,
                                                 s.C_scale, s.ssm_state_scale, s.chunk_size, s.D, s.D_scale, None, None, s.dt_bias, True)
    gy, glast = (cpu(t) for t in cap["qchunk_scan"][1])
    _close(gy, want_y, "ssd y")
    assert (glast.int() - want_last.int()).abs().max().item() <= 1
    # gated norm on the GPU's y and z: one fp16 ulp
    ny, nz = (cpu(t) for t in cap["norm"][0])
    want_n, _ = onorm.qlayer_normgated_fwd(ny.reshape(b * l, -1), m.norm.weight, None, m.norm.eps, q_z=nz.reshape(b * l, -1),
                                           z_scale=m.norm.z_scale, use_float16_output=True, group_size=m.norm.group_size,
                                           norm_before_gate=False)
    torch.testing.assert_close(cpu(cap["norm"][1]).reshape(b * l, -1).float(), want_n.float(), rtol=2e-3, atol=1e-5)
    # Hadamard + quantise on the GPU's norm output: +-1 LSB
    want_h, _ = ohad.quant_hadamard(cpu(cap["had"][0][0]).reshape(b * l, -1), m.had.had_scale / m.had.x_H_scale)
    _lsb(cpu(cap["had"][1]).reshape(b * l, -1), want_h, max_frac=0.02)
    # out_proj on the GPU's int8 input: exact
    assert torch.equal(cpu(cap["out_proj"][1]).reshape(b * l, -1),
                       omodel._w4a8(m.out_proj, cpu(cap["out_proj"][0][0]).reshape(b * l, -1), False))
    # caches, and the whole layer against the oracle's own chain (+-1 LSB flips of int8 intermediates reach the output as
    # noise of a few 1e-3 of its range)
    want, conv_w, ssm_w = omodel.mixer_forward(m, u, want_states=True)
    _close(got, want, "layer output", atol_rel=1e-2)
    conv_g, ssm_g = params.key_value_memory_dict[0]
    assert torch.equal(conv_g.cpu(), conv_w)
    assert (ssm_g.cpu().int() - ssm_w.int()).abs().max().item() <= 1
    # one decode step: the oracle continues from the GPU's states
    u1 = torch.randint(-127, 128, (b, 256), generator=g, dtype=torch.int8)
    conv_c, ssm_c = conv_g.cpu().clone(), ssm_g.cpu().clone()
    want1 = omodel.mixer_step(m, u1, conv_c, ssm_c)
    params.seqlen_offset = l
    got1 = gm(u1.to(DEV)[:, None], inference_params=params)
    _close(got1[:, 0], want1, "decode step", atol_rel=1e-2)
    assert torch.equal(conv_g.cpu(), conv_c)
    assert (ssm_g.cpu().int() - ssm_c.int()).abs().max().item() <= 1


def test_model_prefill_and_graph_decode_match_oracle():
    import copy
    from quamba_b200 import _lib
    q, ids = _small(4, None, n_layer=2, L=200)
    states = {}
    want = omodel.model_forward(q, ids, num_last_tokens=1, states=states)[:, -1]
    gq = copy.deepcopy(q).to(DEV)
    runner = gq.capture_prefill(2, 200)
    runner.input_ids.copy_(ids)
    got = runner.replay()
    torch.cuda.synchronize()
    _close(got, want, "prefill logits", atol_rel=3e-2, max_frac=0.02)
    # decode from the prefill's caches under a CUDA graph; the oracle continues from the same (GPU) states
    params = runner.inference_params
    params.seqlen_offset = 200
    cpu_states = {k: tuple(t.cpu().clone() for t in v) for k, v in params.key_value_memory_dict.items()}
    dec = gq.capture_decode(2, 260, inference_params=params)
    tok = ops().greedy_next_token(got.contiguous())
    for _ in range(3):
        dec.input_ids.copy_(tok[:, None])
        logits = dec.replay().clone()
        want_step = omodel.model_step(q, tok.cpu(), cpu_states)
        _close(logits, want_step, "decode logits", atol_rel=3e-2, max_frac=0.02)
        nxt = dec.input_ids[:, 0].clone()
        assert torch.equal(nxt.cpu(), logits.float().cpu().argmax(-1))
        tok = nxt
        # keep the oracle on the GPU's int8 states so that +-1 LSB state differences do not accumulate across steps
        cpu_states = {k: tuple(t.cpu().clone() for t in v) for k, v in params.key_value_memory_dict.items()}
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("group", [None, -1])
def test_graph_replayed_prefill_equals_the_eager_prefill_bit_for_bit(group):
    """Eager launches are separated by host time and never overlap; a replayed graph runs the same launches back to back
    with each kernel's successor started early.  Equal logits and caches, bit for bit and over several replays on
    different prompts, is the check that no kernel reads what its predecessor has not finished writing (or a stale copy
    of it)."""
    import copy
    from quamba_b200.model import InferenceParams
    q, _ = _small(21, group, d_model=512, n_layer=3, vocab=640, L=64, batch=2)
    gq = copy.deepcopy(q).to(DEV)
    L = 700
    runner = gq.capture_prefill(2, L)
    g = torch.Generator().manual_seed(5)
    for rep in range(4):
        ids = torch.randint(0, 640, (2, L), generator=g).to(DEV)
        runner.input_ids.copy_(ids)
        got = runner.replay().clone()
        got_states = {k: tuple(t.clone() for t in v) for k, v in runner.inference_params.key_value_memory_dict.items()}
        params = InferenceParams(max_seqlen=L + 8, max_batch_size=2)
        want = gq(ids, inference_params=params, num_last_tokens=1).logits[:, -1]
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"replay {rep}: logits differ between the graph and the eager prefill"
        for k, v in params.key_value_memory_dict.items():
            assert torch.equal(got_states[k][0], v[0]) and torch.equal(got_states[k][1], v[1]), f"replay {rep}: layer {k} caches differ"
    import quamba_b200
    quamba_b200.check_device_status()


@pytest.mark.parametrize("batch", [1, 2])
def test_w8a8_model_prefill_and_graph_decode_match_oracle(batch):
    """The reference's default layer class, W8A8QMamba2 (W8 embedding, W8A8 head): prefill logits and three graph-replayed
    decode steps against the CPU oracle.  Batch 1 takes the single-row GEMV forms of the W8A8 linears, batch 2 the GEMM."""
    import copy
    from quamba_b200 import _lib
    from quamba_b200.mixer import W8A8QMamba2
    q, ids = _small(31 + batch, None, n_layer=2, L=150, batch=batch, w_bits=8)
    assert isinstance(q.backbone.layers[0].mixer, W8A8QMamba2)
    want = omodel.model_forward(q, ids, num_last_tokens=1)[:, -1]
    gq = copy.deepcopy(q).to(DEV)
    runner = gq.capture_prefill(batch, 150)
    runner.input_ids.copy_(ids)
    got = runner.replay()
    torch.cuda.synchronize()
    _close(got, want, "W8A8 prefill logits", atol_rel=3e-2, max_frac=0.02)
    params = runner.inference_params
    params.seqlen_offset = 150
    dec = gq.capture_decode(batch, 200, inference_params=params)
    tok = ops().greedy_next_token(got.contiguous())
    for _ in range(3):
        cpu_states = {k: tuple(t.cpu().clone() for t in v) for k, v in params.key_value_memory_dict.items()}
        dec.input_ids.copy_(tok[:, None])
        logits = dec.replay().clone()
        _close(logits, omodel.model_step(q, tok.cpu(), cpu_states), "W8A8 decode logits", atol_rel=3e-2, max_frac=0.02)
        tok = dec.input_ids[:, 0].clone()
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)


def test_generate_greedy_graph_equals_eager():
    import copy
    q, ids = _small(5, -1, n_layer=2, L=64, batch=1)
    gq = copy.deepcopy(q).to(DEV)
    a = gq.generate_greedy(ids.to(DEV), 8, use_graph=True)
    b = gq.generate_greedy(ids.to(DEV), 8, use_graph=False)
    assert a.shape == (1, 72) and torch.equal(a, b)


def test_rebuilt_layer_of_same_shape_uses_its_own_weights():
    """A freed layer's streaming weight copies must never serve a new layer that lands on the same addresses."""
    from quamba_b200.modules import W4A8B16O16Linear
    g = torch.Generator().manual_seed(0)
    x = torch.randint(-127, 128, (64, 256), generator=g, dtype=torch.int8).to(DEV)
    outs = []
    for seed in (1, 2):
        lin = torch.nn.Linear(256, 128, bias=False)
        lin.weight.data = torch.randn(128, 256, generator=torch.Generator().manual_seed(seed)) * 0.02
        ql = W4A8B16O16Linear.from_fp16(lin, torch.tensor(0.01)).to(DEV)
        y = ql(x)
        want = olin_ref(ql, x)
        assert torch.equal(y.cpu(), want)
        outs.append(y.cpu())
        del ql, y
        torch.cuda.synchronize()
    assert not torch.equal(outs[0], outs[1])


def olin_ref(ql, x):
    from oracle import linear as olin
    sg = ql.s_group.cpu() if ql.s_group.numel() else None
    return olin.w4a8_gemm(x.cpu(), ql.weight.cpu(), ql.input_scale.cpu().reshape(1), ql.s_channel.cpu(), sg, ql.size_n,
                          ql.size_k, False)[:, :ql.out_features]


@pytest.mark.parametrize("group,batch,nibbles", [(-1, 1, False), (None, 1, False), (-1, 2, False), (None, 3, False), (-1, 4, False),
                                                 (None, 2, True)])
def test_fused_decode_step_equals_the_op_by_op_step(group, batch, nibbles, monkeypatch):
    """The three-launch decode step against the seven-launch one on the same model, token and caches, and against the
    CPU oracle's step: conv state bit for bit, int8 ssm state +-1 LSB, logits within the model-level tolerance."""
    import copy
    import quamba_b200.model as qmodel
    from quamba_b200.model import InferenceParams
    monkeypatch.setattr(ops(), "GROUP_NIBBLES", nibbles)      # group-128 weights streamed as 4-bit codes in the fused step
    q, ids = _small(11 + batch, group, n_layer=2, L=40, batch=batch)
    gq = copy.deepcopy(q).to(DEV)
    params = InferenceParams(max_seqlen=64, max_batch_size=batch)
    first = gq(ids.to(DEV), inference_params=params, num_last_tokens=1).logits[:, -1]
    tok = ops().greedy_next_token(first.contiguous())
    params.seqlen_offset = 40
    base = {k: tuple(t.clone() for t in v) for k, v in params.key_value_memory_dict.items()}
    cpu_states = {k: tuple(t.cpu().clone() for t in v) for k, v in base.items()}
    assert gq.backbone._decode_fusable(batch, gq.lm_head)
    fused = gq(tok[:, None], inference_params=params).logits[:, -1].clone()
    fused_states = {k: tuple(t.clone() for t in v) for k, v in params.key_value_memory_dict.items()}
    for k, v in base.items():
        for dst, src in zip(params.key_value_memory_dict[k], v):
            dst.copy_(src)
    monkeypatch.setattr(qmodel, "_UNFUSED_DECODE", True)
    plain = gq(tok[:, None], inference_params=params).logits[:, -1].clone()
    want = omodel.model_step(q, tok.cpu(), cpu_states)
    _close(fused, plain.cpu(), "fused vs op-by-op logits", atol_rel=3e-2, max_frac=0.02)
    _close(fused, want, "fused vs oracle logits", atol_rel=3e-2, max_frac=0.02)
    for k in base:
        conv_f, ssm_f = fused_states[k]
        conv_p, ssm_p = params.key_value_memory_dict[k]
        if k == 0:      # the first layer sees identical inputs on both paths
            assert torch.equal(conv_f, conv_p)
            assert torch.equal(conv_f.cpu(), cpu_states[k][0])
            assert (ssm_f.int() - ssm_p.int()).abs().max().item() <= 1
        else:           # later layers inherit +-1 LSB differences of the layer before
            assert (conv_f.int() - conv_p.int()).abs().float().mean().item() < 0.05
            assert (ssm_f.int() - ssm_p.int()).abs().max().item() <= 2


@pytest.mark.parametrize("K,N,rows,out_int8", [(2560, 10624, 1, True), (5120, 2560, 1, False), (256, 320, 3, False),
                                               (1024, 4160, 4, True), (384, 128, 2, False)])
def test_decode_product_from_group128_nibbles_is_bit_identical(K, N, rows, out_int8):
    """Group-128 weights streamed as 4-bit codes + fp16 group scales, the int8 weights rebuilt in registers with the
    reference's fp16 fma, against (a) the same kernel on the int8 expansion qb_w4a8_unpack makes and (b) the large-M product
    entry point on that expansion: all three bit for bit."""
    from quamba_b200.modules import W4A8B8O8Linear, W4A8B16O16Linear
    o = ops()
    g = torch.Generator().manual_seed(K + N)
    lin = torch.nn.Linear(K, N, bias=False)
    lin.weight.data = torch.randn(N, K, generator=g) * 0.02 * (1 + 3 * torch.rand(N, 1, generator=g))
    cls = W4A8B8O8Linear if out_int8 else W4A8B16O16Linear
    ql = (cls.from_fp16(lin, torch.tensor(0.02), torch.tensor(0.05)) if out_int8 else cls.from_fp16(lin, torch.tensor(0.02))).to(DEV)
    prep = ql.prepared()
    assert not prep.per_channel
    a = torch.randint(-127, 128, (rows, K), generator=g, dtype=torch.int32).to(torch.int8).to(DEV)
    s_tok = ql.input_scale
    old = o.GROUP_NIBBLES
    try:
        o.GROUP_NIBBLES = True
        got = o.decode_linear(a, prep, s_tok, out_int8=out_int8)
        codes, scales = prep.need_w4g()
        assert codes.shape == (prep.size_n, K // 2) and scales.shape == (prep.size_n, K // 128)
        o.GROUP_NIBBLES = False
        from_int8 = o.decode_linear(a, prep, s_tok, out_int8=out_int8)
    finally:
        o.GROUP_NIBBLES = old
    big = o.w4a8_linear(a, prep, s_tok, out_int8=out_int8)
    torch.cuda.synchronize()
    assert torch.equal(got, from_int8)
    assert torch.equal(got, big)
