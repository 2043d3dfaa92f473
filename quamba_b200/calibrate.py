"""Float Mamba2 language model with activation taps, absmax calibration, and conversion to the quantized model.

This is the on-ramp that turns float weights into a :class:`quamba_b200.model.QuambaLMHeadModel`: the float layer
follows ``Mamba2Simple`` (quamba/qMamba2.py:70-330: same tap names), calibration follows ``run_quamba2_calibration``
(quamba/modelutils_mamba.py:235-372) with per-tensor min-max observers (quamba/observer.py:34-70: scale = absmax /
127), and the conversion follows ``quantize_fp16_model`` (modelutils_mamba.py:579-668).  It runs in plain torch on
whatever device the float model lives on; it is offline work, not part of the inference path.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .embedding import F16Embedding, W4O16Embedding, W8O16Embedding
from .hadamard_utils import hadamard_transform
from .mixer import W4A8QMamba2, W8A8QMamba2
from .model import QuambaConfig, QuambaLMHeadModel
from .modules import W4A8B16O16Linear, W8A8B16O16Linear
from .norm import QRMSNorm

__all__ = ["Mamba1Float", "Mamba1LMFloat", "Mamba2Float", "Mamba2LMFloat", "calibrate", "calibrate_mamba1", "quantize_model",
           "quantize_mamba1_model", "ssd_float"]


def ssd_float(x, dt, A, B, C, D, chunk_size=256, initial_state=None):
    """Chunked SSD in float: x (b, l, h, p), dt (b, l, h) after softplus, A (h) negative, B / C (b, l, g, n),
    D (h).  Returns (y (b, l, h, p), final state (b, h, p, n))."""
    b, l, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    rep = h // g
    state = x.new_zeros(b, h, p, n) if initial_state is None else initial_state.clone()
    ys = []
    for s in range(0, l, chunk_size):
        xc, dtc = x[:, s:s + chunk_size], dt[:, s:s + chunk_size]
        Bc = B[:, s:s + chunk_size].repeat_interleave(rep, dim=2)
        Cc = C[:, s:s + chunk_size].repeat_interleave(rep, dim=2)
        cs = torch.cumsum(dtc * A, dim=1)                                   # (b, q, h)
        q = xc.shape[1]
        decay = torch.exp(cs[:, :, None, :] - cs[:, None, :, :])             # (b, t, s, h)
        mask = torch.tril(torch.ones(q, q, dtype=torch.bool, device=x.device))[None, :, :, None]
        w = torch.where(mask, decay, torch.zeros_like(decay)) * dtc[:, None, :, :]
        cb = torch.einsum("bthn,bshn->btsh", Cc, Bc)
        y = torch.einsum("btsh,bshp->bthp", cb * w, xc)
        y = y + torch.einsum("bthn,bhpn->bthp", Cc, state) * torch.exp(cs)[..., None]
        tail = torch.exp(cs[:, -1:, :] - cs) * dtc                          # (b, q, h)
        state = state * torch.exp(cs[:, -1, :])[:, :, None, None] + torch.einsum("bshn,bsh,bshp->bhpn", Bc, tail, xc)
        ys.append(y)
    y = torch.cat(ys, dim=1) + x * D[None, None, :, None]
    return y, state


class RMSNormFloat(nn.Module):
    def __init__(self, dim, eps=1e-5, group_size=None, norm_before_gate=False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps, self.group_size, self.norm_before_gate = eps, group_size, norm_before_gate

    def forward(self, x, z=None):
        if z is not None and not self.norm_before_gate:
            x = x * F.silu(z)
        gs = self.group_size or x.shape[-1]
        xg = x.float().unflatten(-1, (-1, gs))
        y = (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + self.eps)).flatten(-2) * self.weight.float()
        if z is not None and self.norm_before_gate:
            y = y * F.silu(z)
        return y


class Mamba2Float(nn.Module):
    """Float Mamba2 mixer (the role of mamba_ssm's ``Mamba2`` wrapped by ``Mamba2Simple``) with the reference's tap
    points.  ``taps`` (dict name -> running absmax) is filled when given."""

    def __init__(self, d_model, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=256, layer_idx=None,
                 w4_group_size=None, had_blocks=1, generator=None, device=None):
        super().__init__()
        self.had_blocks = had_blocks        # block-diagonal out_proj rotation (head-parallel serving), 1 = one full rotation
        self.d_model, self.d_state, self.d_conv, self.expand, self.headdim = d_model, d_state, d_conv, expand, headdim
        self.d_inner = self.d_ssm = expand * d_model
        self.ngroups, self.nheads = ngroups, self.d_ssm // headdim
        self.rmsnorm, self.norm_before_gate, self.D_has_hdim = True, False, False
        self.dt_limit, self.chunk_size, self.layer_idx = (0.0, float("inf")), chunk_size, layer_idx
        rnd = lambda *shape: torch.randn(*shape, generator=generator, device=device)
        uni = lambda *shape: torch.rand(*shape, generator=generator, device=device)
        d_in_proj = 2 * self.d_inner + 2 * ngroups * d_state + self.nheads
        conv_dim = self.d_ssm + 2 * ngroups * d_state
        self.in_proj = nn.Linear(d_model, d_in_proj, bias=False, device=device)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=False, device=device)
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, d_conv, groups=conv_dim, padding=d_conv - 1, bias=True, device=device)
        with torch.no_grad():
            self.in_proj.weight.copy_(rnd(d_in_proj, d_model) * 0.02)
            self.out_proj.weight.copy_(rnd(d_model, self.d_inner) * 0.02)
            self.conv1d.weight.copy_(rnd(conv_dim, 1, d_conv) * 0.2)
            self.conv1d.bias.copy_(rnd(conv_dim) * 0.02)
        if w4_group_size is not None:
            self.in_proj.w4_group_size = self.out_proj.w4_group_size = w4_group_size
        dt0 = uni(self.nheads) * (0.1 - 0.001) + 0.001
        self.dt_bias = nn.Parameter(dt0 + torch.log(-torch.expm1(-dt0)))
        self.A_log = nn.Parameter(torch.log(uni(self.nheads) * 15 + 1))
        self.D = nn.Parameter(torch.ones(self.nheads, device=device))
        self.norm = RMSNormFloat(self.d_ssm, eps=1e-5, group_size=self.d_ssm // ngroups, norm_before_gate=False).to(device)

    @staticmethod
    def _tap(taps, name, t):
        if taps is not None:
            v = t.detach().abs().amax().float()
            taps[name] = torch.maximum(taps[name], v) if name in taps else v
        return t

    def forward(self, u, taps=None, state=None):
        """u (b, l, d_model) float.  ``state`` (dict) receives ``conv`` (b, conv_dim, d_conv) and ``ssm``."""
        tap = lambda name, t: self._tap(taps, name, t)
        gn = self.ngroups * self.d_state
        zxbcdt = self.in_proj(tap("in_proj:input", u))
        z, x, B, C, dt = torch.split(zxbcdt, [self.d_ssm, self.d_ssm, gn, gn, self.nheads], dim=-1)
        x, B, C = tap("x_conv_in", x), tap("B_conv_in", B), tap("C_conv_in", C)
        xBC = torch.cat([x, B, C], dim=-1)
        if state is not None:
            state["conv"] = F.pad(xBC.transpose(1, 2), (self.d_conv - xBC.shape[1], 0))
        xBC = F.silu(self.conv1d(xBC.transpose(1, 2))[..., :u.shape[1]].transpose(1, 2))
        x, B, C = torch.split(xBC, [self.d_ssm, gn, gn], dim=-1)
        x, B, C = tap("x_conv_out", x), tap("B_conv_out", B), tap("C_conv_out", C)
        dt, z = tap("dt_act", dt), tap("z_act", z)
        y, last = ssd_float(x.float().unflatten(-1, (self.nheads, self.headdim)), F.softplus(dt.float() + self.dt_bias.float()),
                            -torch.exp(self.A_log.float()), B.float().unflatten(-1, (self.ngroups, self.d_state)),
                            C.float().unflatten(-1, (self.ngroups, self.d_state)), self.D.float(), self.chunk_size)
        tap("ssm_state_act", last)
        if state is not None:
            state["ssm"] = last
        y = self.norm(y.flatten(-2), z.float())
        y = tap("out_proj:input", hadamard_transform(y.unflatten(-1, (self.had_blocks, -1))).flatten(-2))
        return self.out_proj(y.to(u.dtype))


class Mamba2LMFloat(nn.Module):
    """embedding -> [add, RMSNorm, Mamba2Float] x n_layer -> add, RMSNorm -> lm_head, random-initialised from a seed
    (N(0, 0.02) matrices, the mixer defaults above).  The head has its own matrix: a quantized embedding table and a
    quantized head cannot share storage, so the reference unties them before quantisation as well."""

    def __init__(self, d_model=2560, n_layer=64, vocab_size=50288, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1,
                 chunk_size=256, w4_group_size=None, had_blocks=1, seed=0, device=None, dtype=torch.float32):
        super().__init__()
        gen = torch.Generator(device=device or "cpu").manual_seed(seed)
        self.d_model, self.n_layer, self.vocab_size = d_model, n_layer, vocab_size
        self.ssm_cfg = dict(d_state=d_state, d_conv=d_conv, expand=expand, headdim=headdim, ngroups=ngroups,
                            chunk_size=chunk_size)
        self.embedding = nn.Embedding(vocab_size, d_model, device=device)
        self.lm_head = nn.Linear(d_model, vocab_size, bias=False, device=device)
        with torch.no_grad():
            self.embedding.weight.copy_(torch.randn(vocab_size, d_model, generator=gen, device=device) * 0.02)
            self.lm_head.weight.copy_(torch.randn(vocab_size, d_model, generator=gen, device=device) * 0.02)
        if w4_group_size is not None:
            self.lm_head.w4_group_size = w4_group_size
        self.norms = nn.ModuleList([RMSNormFloat(d_model).to(device) for _ in range(n_layer)])
        self.mixers = nn.ModuleList([Mamba2Float(d_model, layer_idx=i, w4_group_size=w4_group_size, had_blocks=had_blocks, generator=gen,
                                                 device=device, **self.ssm_cfg) for i in range(n_layer)])
        self.norm_f = RMSNormFloat(d_model).to(device)
        self.to(dtype)

    @torch.no_grad()
    def forward(self, input_ids, taps=None, states=None, num_last_tokens=0):
        """taps: list of n_layer + 1 dicts (the last one for the head) filled with running absmax values."""
        h = self.embedding(input_ids)
        residual = torch.zeros_like(h, dtype=torch.float32)
        for i, (norm, mixer) in enumerate(zip(self.norms, self.mixers)):
            residual = residual + h.float()
            st = None if states is None else states.setdefault(i, {})
            h = mixer(norm(residual).to(h.dtype), None if taps is None else taps[i], st)
        residual = residual + h.float()
        if num_last_tokens > 0:
            residual = residual[:, -num_last_tokens:]
        y = self.norm_f(residual).to(h.dtype)
        if taps is not None:
            Mamba2Float._tap(taps[-1], "lm_head:input", y)
        return self.lm_head(y)


@torch.no_grad()
def calibrate(model: Mamba2LMFloat, sequences):
    """Runs the float model over ``sequences`` (an iterable of int64 (b, l) batches) and returns the per-layer
    activation scales with the reference's key names (absmax / 127 each; the ``:input`` / ``:output`` pairs of an
    identity tap are the same tensor, so they share a value)."""
    taps = [dict() for _ in range(model.n_layer + 1)]
    for ids in sequences:
        model(ids, taps=taps)
    out = []
    for t in taps[:-1]:
        s = {k: (v / 127.0).clamp(min=1e-8).float().reshape(1) for k, v in t.items()}
        d = {"in_proj:input": s["in_proj:input"], "out_proj:input": s["out_proj:input"],
             "ssm_state_act:input": s["ssm_state_act"]}
        for name in ("x_conv_in", "B_conv_in", "C_conv_in", "x_conv_out", "B_conv_out", "C_conv_out", "dt_act", "z_act"):
            d[name + ":input"] = d[name + ":output"] = s[name]
        out.append(d)
    out.append({"lm_head:input": (taps[-1]["lm_head:input"] / 127.0).clamp(min=1e-8).float().reshape(1)})
    return out


@torch.no_grad()
def quantize_model(model: Mamba2LMFloat, act_scales, w_bits=4, quantize_embedding=True, device=None):
    """Float model + calibrated scales -> QuambaLMHeadModel (W4A8 or W8A8 mixers and head, W4 / W8 embedding)."""
    assert w_bits in (4, 8)
    dev = device or model.embedding.weight.device
    mixer_cls = W4A8QMamba2 if w_bits == 4 else W8A8QMamba2
    cfg = QuambaConfig(d_model=model.d_model, n_layer=0, vocab_size=model.vocab_size,
                       ssm_cfg=dict(layer=mixer_cls.__name__, **model.ssm_cfg), norm_cfg={"norm": "QRMSNorm"},
                       embedding_cfg={"layer": ("W4O16Embedding" if w_bits == 4 else "W8O16Embedding") if quantize_embedding
                                      else "Embedding"},
                       lm_head_cfg={"layer": "W4A8B16O16Linear" if w_bits == 4 else "W8A8B16O16Linear"})
    # build the shell without layers (no throw-away buffers), then attach the converted ones
    q = QuambaLMHeadModel(cfg, device="meta")
    cfg.n_layer = model.n_layer
    emb = model.embedding
    if quantize_embedding:
        q.backbone.embedding = (W4O16Embedding if w_bits == 4 else W8O16Embedding).from_fp16(emb)
    else:
        q.backbone.embedding = F16Embedding(emb.num_embeddings, emb.embedding_dim, device=dev)
        q.backbone.embedding.weight.data = emb.weight.detach().to(torch.float16)
    from .model import Block
    layers = []
    for i, (norm, mixer) in enumerate(zip(model.norms, model.mixers)):
        s = act_scales[i]
        blk = Block.__new__(Block)
        nn.Module.__init__(blk)
        blk.residual_in_fp32, blk.fused_add_norm, blk.layer_idx = True, True, i
        blk.norm = QRMSNorm.from_fp16(norm, output_scale=s["in_proj:input"].item())
        blk.mixer = mixer_cls.from_fp16(mixer, s)
        layers.append(blk)
    q.backbone.layers = nn.ModuleList(layers)
    head_scale = act_scales[-1]["lm_head:input"]
    q.backbone.norm_f = QRMSNorm.from_fp16(model.norm_f, output_scale=head_scale.item())
    if w_bits == 4:
        q.lm_head = W4A8B16O16Linear.from_fp16(model.lm_head, head_scale)
    else:
        q.lm_head = W8A8B16O16Linear.from_fp16(model.lm_head, head_scale.item())
    return q.to(dev) if str(dev) != str(emb.weight.device) else q


# ---- Mamba1 ---------------------------------------------------------------------------------------------------------------
class Mamba1Float(nn.Module):
    """Float Mamba1 mixer (the role of the reference's ``MambaSimple``) with its tap points: in_proj -> x | z -> causal
    conv1d + SiLU -> x_proj -> dt | B | C -> dt_proj (bias kept apart in ``dt_proj_bias``) -> selective scan with gate z ->
    Hadamard rotation -> out_proj.  ``taps`` (dict name -> running absmax) is filled when given."""

    def __init__(self, d_model, d_state=16, d_conv=4, expand=2, dt_rank="auto", layer_idx=None, w4_group_size=None,
                 generator=None, device=None):
        super().__init__()
        self.d_model, self.d_state, self.d_conv, self.expand, self.layer_idx = d_model, d_state, d_conv, expand, layer_idx
        self.d_inner = expand * d_model
        self.dt_rank = math.ceil(d_model / 16) if dt_rank == "auto" else dt_rank
        D, R, N = self.d_inner, self.dt_rank, d_state
        rnd = lambda *shape: torch.randn(*shape, generator=generator, device=device)
        uni = lambda *shape: torch.rand(*shape, generator=generator, device=device)
        self.in_proj = nn.Linear(d_model, 2 * D, bias=False, device=device)
        self.conv1d = nn.Conv1d(D, D, d_conv, groups=D, padding=d_conv - 1, bias=True, device=device)
        self.x_proj = nn.Linear(D, R + 2 * N, bias=False, device=device)
        self.dt_proj = nn.Linear(R, D, bias=False, device=device)
        self.out_proj = nn.Linear(D, d_model, bias=False, device=device)
        with torch.no_grad():
            self.in_proj.weight.copy_(rnd(2 * D, d_model) * 0.02)
            self.conv1d.weight.copy_(rnd(D, 1, d_conv) * 0.2)
            self.conv1d.bias.copy_(rnd(D) * 0.02)
            self.x_proj.weight.copy_(rnd(R + 2 * N, D) * 0.05)
            self.dt_proj.weight.copy_((uni(D, R) * 2 - 1) * R ** -0.5)
            self.out_proj.weight.copy_(rnd(d_model, D) * 0.02)
        if w4_group_size is not None:
            self.in_proj.w4_group_size = self.x_proj.w4_group_size = self.out_proj.w4_group_size = w4_group_size
        dt0 = uni(D) * (0.1 - 0.001) + 0.001
        self.dt_proj_bias = nn.Parameter(dt0 + torch.log(-torch.expm1(-dt0)))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, N + 1, dtype=torch.float32, device=device)).repeat(D, 1))
        self.D = nn.Parameter(torch.ones(D, device=device))

    def forward(self, u, taps=None, state=None):
        """u (b, l, d_model) float.  ``state`` (dict) receives ``conv`` (b, d_inner, d_conv) and ``ssm`` (b, d_inner, d_state)."""
        tap = lambda name, t: Mamba2Float._tap(taps, name, t)
        b, l, _ = u.shape
        R, N = self.dt_rank, self.d_state
        xz = tap("in_proj:output", self.in_proj(tap("in_proj:input", u)))
        x, z = xz.transpose(1, 2).chunk(2, dim=1)                               # (b, D, l)
        if state is not None:
            state["conv"] = F.pad(x, (self.d_conv - l, 0))
        x = tap("x_proj:input", F.silu(self.conv1d(x)[..., :l]))
        x_dbl = tap("x_proj:output", self.x_proj(x.transpose(1, 2)))           # (b, l, R + 2N)
        dt = tap("dt_proj:output", self.dt_proj(x_dbl[..., :R])).transpose(1, 2)   # (b, D, l), bias not added yet
        Bm, Cm = x_dbl[..., R:R + N].float(), x_dbl[..., R + N:].float()      # (b, l, N)
        delta = F.softplus(dt.float() + self.dt_proj_bias.float()[None, :, None])
        A = -torch.exp(self.A_log.float())
        h = torch.zeros(b, self.d_inner, N, dtype=torch.float32, device=u.device)
        xf = x.float()
        ys = []
        for t in range(l):
            dA = torch.exp(delta[:, :, t, None] * A)
            h = dA * h + (delta[:, :, t] * xf[:, :, t])[:, :, None] * Bm[:, t, None, :]
            ys.append((h * Cm[:, t, None, :]).sum(-1) + self.D.float() * xf[:, :, t])
        tap("ssm_state_act:input", h)
        if state is not None:
            state["ssm"] = h
        y = torch.stack(ys, dim=1) * F.silu(z.float()).transpose(1, 2)          # (b, l, D)
        y = tap("out_proj:input", hadamard_transform(y))
        return self.out_proj(y.to(u.dtype))


def calibrate_mamba1(layer: Mamba1Float, inputs):
    """Runs the float layer over ``inputs`` (an iterable of (b, l, d_model) float batches) and returns the activation scales
    under the reference's key names (absmax / 127)."""
    taps = {}
    with torch.no_grad():
        for u in inputs:
            layer(u, taps=taps)
    return {k: (v / 127.0).clamp(min=1e-8).float().reshape(1) for k, v in taps.items()}


class Mamba1LMFloat(nn.Module):
    """embedding -> [add, RMSNorm, Mamba1Float] x n_layer -> add, RMSNorm -> lm_head, random-initialised from a seed: the
    Mamba1 counterpart of :class:`Mamba2LMFloat` (same tap convention: one dict per layer plus one for the head)."""

    def __init__(self, d_model=2560, n_layer=64, vocab_size=50288, d_state=16, d_conv=4, expand=2, w4_group_size=None, seed=0,
                 device=None):
        super().__init__()
        g = torch.Generator(device=device).manual_seed(seed)
        self.d_model, self.n_layer, self.vocab_size = d_model, n_layer, vocab_size
        self.ssm_cfg = dict(d_state=d_state, d_conv=d_conv, expand=expand)
        self.embedding = nn.Embedding(vocab_size, d_model, device=device)
        self.lm_head = nn.Linear(d_model, vocab_size, bias=False, device=device)
        with torch.no_grad():
            self.embedding.weight.copy_(torch.randn(vocab_size, d_model, generator=g, device=device) * 0.02)
            self.lm_head.weight.copy_(torch.randn(vocab_size, d_model, generator=g, device=device) * 0.02)
        if w4_group_size is not None:
            self.lm_head.w4_group_size = w4_group_size
        self.mixers = nn.ModuleList([Mamba1Float(d_model, layer_idx=i, w4_group_size=w4_group_size, generator=g, device=device,
                                                 **self.ssm_cfg) for i in range(n_layer)])
        self.norms = nn.ModuleList([RMSNormFloat(d_model).to(device) for _ in range(n_layer)])
        self.norm_f = RMSNormFloat(d_model).to(device)

    @torch.no_grad()
    def forward(self, input_ids, taps=None):
        h = self.embedding(input_ids)
        residual = torch.zeros_like(h, dtype=torch.float32)
        for i, (norm, mixer) in enumerate(zip(self.norms, self.mixers)):
            residual = residual + h.float()
            h = mixer(norm(residual).to(h.dtype), None if taps is None else taps[i])
        residual = residual + h.float()
        y = self.norm_f(residual)
        if taps is not None:
            Mamba2Float._tap(taps[-1], "lm_head:input", y)
        return self.lm_head(y.to(h.dtype))


@torch.no_grad()
def quantize_mamba1_model(model: Mamba1LMFloat, sequences, w_bits=8, use_had_transform=True):
    """Calibrates the float Mamba1 model on ``sequences`` and returns a QuambaLMHeadModel with W8A8QMamba (or W4A8QMamba)
    mixers, QRMSNorm block norms with static output scales, an fp16 embedding and a W8A8 / W4A8 head."""
    from .mixer1 import W4A8QMamba, W8A8QMamba
    from .model import Block
    assert w_bits in (4, 8)
    taps = [dict() for _ in range(model.n_layer + 1)]
    for ids in sequences:
        model(ids, taps=taps)
    scales = [{k: (v / 127.0).clamp(min=1e-8).float().reshape(1) for k, v in t.items()} for t in taps]
    mixer_cls = W8A8QMamba if w_bits == 8 else W4A8QMamba
    dev = model.embedding.weight.device
    cfg = QuambaConfig(d_model=model.d_model, n_layer=0, vocab_size=model.vocab_size,
                       ssm_cfg=dict(layer=mixer_cls.__name__, **model.ssm_cfg), norm_cfg={"norm": "QRMSNorm"},
                       embedding_cfg={"layer": "Embedding"},
                       lm_head_cfg={"layer": "W8A8B16O16Linear" if w_bits == 8 else "W4A8B16O16Linear"})
    q = QuambaLMHeadModel(cfg, device="meta")
    cfg.n_layer = model.n_layer
    q.backbone.embedding = F16Embedding(model.vocab_size, model.d_model, device=dev)
    q.backbone.embedding.weight.data = model.embedding.weight.detach().to(torch.float16)
    layers = []
    for i, (norm, mixer) in enumerate(zip(model.norms, model.mixers)):
        blk = Block.__new__(Block)
        nn.Module.__init__(blk)
        blk.residual_in_fp32, blk.fused_add_norm, blk.layer_idx = True, True, i
        blk.norm = QRMSNorm.from_fp16(norm, output_scale=scales[i]["in_proj:input"].item())
        blk.mixer = mixer_cls.from_fp16(mixer, scales[i], use_had_transform=use_had_transform)
        layers.append(blk)
    q.backbone.layers = nn.ModuleList(layers)
    head_scale = scales[-1]["lm_head:input"]
    q.backbone.norm_f = QRMSNorm.from_fp16(model.norm_f, output_scale=head_scale.item())
    if w_bits == 8:
        q.lm_head = W8A8B16O16Linear.from_fp16(model.lm_head, head_scale.item())
    else:
        q.lm_head = W4A8B16O16Linear.from_fp16(model.lm_head, head_scale)
    return q
