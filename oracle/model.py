"""CPU restatement of the quantized Mamba2 layer and model (test infrastructure only): the composition of the
oracle's ops in the order of W4A8QMamba2.forward / .step (quamba/qMamba2.py:920-1020) and of the model shell
(QRMSNorm with fused residual add -> mixer, ..., norm_f -> lm_head).  The layer objects passed in are read by attribute
(buffers and float scales of the module classes); nothing of the product's execution path is called.
"""
import torch

from . import conv1d as oconv, hadamard as ohad, linear as olin, norm as onorm, ssd as ossd, update as oupd, embedding as oemb
from . import sscan as osscan


def _w4a8(lin, a_int8, out_int8):
    """The product of a quantized linear layer, read off its buffers: W4A8 (Marlin-QQQ packed weight, qLinearLayer.py:227-273,
    :370-414) or W8A8 (int8 weight with ``a`` / ``b`` scales; one row goes through the reference's GEMV forms,
    qLinearLayer.py:607-647, :725-742, :805-820)."""
    if hasattr(lin, "s_channel"):
        sg = lin.s_group if lin.s_group.numel() else None
        out = olin.w4a8_gemm(a_int8, lin.weight, lin.input_scale.reshape(1), lin.s_channel, sg, lin.size_n, lin.size_k, out_int8)
        return out[:, :lin.out_features]
    w_kn = lin.weight                                   # (K, N_pad) view of a row-major (N_pad, K) matrix
    out_dtype = torch.int8 if out_int8 else torch.float16
    if a_int8.shape[0] == 1:
        if lin.b.numel() > 1:                           # W8A8B8O8LinearParallel._matvec
            out = olin.w8a8o8_gemv(w_kn.t(), a_int8, lin.b, lin.a)
        else:                                           # cutlass_scaled_mv_dq with the folded alpha
            out = olin.w8a8_gemv_alpha(w_kn.t(), a_int8, lin.alpha, out_dtype)
    else:
        out = olin.w8a8_gemm(a_int8, w_kn, lin.a, lin.b, out_dtype)
    return out[:, :lin.out_features]


def _conv_args(c):
    return (c.x_scale, c.B_scale, c.C_scale, c.x_dim, c.x_headdim, c.d_state, c.n_groups, c.x_head_group_range,
            c.x_dim_group_range, c.x_out_scales, c.B_out_scales, c.C_out_scales, c.weight, c.wx_scale, c.wB_scale,
            c.wC_scale, c.bias, c.bx_scale, c.bB_scale, c.bC_scale)


def mixer_forward(m, u_int8, want_states=False):
    """u_int8 (b, l, d_model) -> fp16 (b, l, d_model) [, conv_state (b, conv_dim, d_conv) int8, ssm_state int8]."""
    b, l, _ = u_int8.shape
    gn = m.ngroups * m.d_state
    zxbcdt = _w4a8(m.in_proj, u_int8.reshape(b * l, -1), True).reshape(b, l, -1)
    z, xBC, dt = torch.split(zxbcdt, [m.d_ssm, m.d_ssm + 2 * gn, m.nheads], dim=-1)
    x, B, C = oconv.quamba2_conv1d_fwd(xBC.transpose(1, 2), *_conv_args(m.conv1d))
    s = m.qchunk_scan
    y, last = ossd.chunk_scan_faithful(
        x.transpose(1, 2).reshape(b, l, m.nheads, m.headdim), s.x_scales, s.x_head_group_range, s.x_dim_group_range, dt,
        s.dt_scale, s.A_log, s.A_log_scale, B.transpose(1, 2).reshape(b, l, m.ngroups, m.d_state), s.B_scale,
        C.transpose(1, 2).reshape(b, l, m.ngroups, m.d_state), s.C_scale, s.ssm_state_scale, s.chunk_size, s.D, s.D_scale,
        None, None, s.dt_bias, True, s.dt_limit)
    out = _gate_rotate_project(m, y.reshape(b * l, -1), z.reshape(b * l, -1)).reshape(b, l, -1)
    if not want_states:
        return out
    conv_state = torch.nn.functional.pad(xBC.transpose(1, 2), (m.d_conv - l, 0)).contiguous()
    return out, conv_state, last


def _gate_rotate_project(m, y16, z8):
    n = m.norm
    yn, _ = onorm.qlayer_normgated_fwd(y16, n.weight, None, n.eps, q_z=z8, z_scale=n.z_scale, use_float16_output=True,
                                       group_size=n.group_size, norm_before_gate=n.norm_before_gate, is_rms_norm=True)
    blocks = getattr(m.had, "blocks", 1)          # block-diagonal rotation: each slice of the row on its own
    q, _ = ohad.quant_hadamard(yn.reshape(-1, yn.shape[-1] // blocks), m.had.had_scale / m.had.x_H_scale)
    return _w4a8(m.out_proj, q.reshape(yn.shape), False)


def mixer_step(m, u_int8, conv_state, ssm_state):
    """One decode token: u_int8 (b, d_model); the two states are updated in place.  Returns fp16 (b, d_model)."""
    b = u_int8.shape[0]
    gn = m.ngroups * m.d_state
    zxbcdt = _w4a8(m.in_proj, u_int8, True)
    z, xBC, dt = torch.split(zxbcdt, [m.d_ssm, m.d_ssm + 2 * gn, m.nheads], dim=-1)
    x, B, C = oconv.quamba2_conv1d_update(xBC, conv_state, *_conv_args(m.conv1d))
    s = m.qchunk_scan
    p, n = m.headdim, m.d_state
    args = (x.reshape(b, m.nheads, p), s.x_scales)
    common = (dt[:, :, None].expand(-1, -1, p), s.dt_scale, s.A_log[:, None, None].expand(-1, p, n), s.A_log_scale,
              s.ssm_state_scale, B.reshape(b, m.ngroups, n), s.B_scale, C.reshape(b, m.ngroups, n), s.C_scale)
    D2 = s.D[:, None].expand(-1, p)
    bias = s.dt_bias[:, None].expand(-1, p)
    if s.x_head_group_range is None:
        y, _ = oupd.quant_sscan_update(ssm_state, *args, *common, D2, s.D_scale, None, None, bias.float(), None, True)
    else:
        y, _ = oupd.quamba2_sscan_update(ssm_state, *args, s.x_head_group_range, s.x_dim_group_range, *common, D2,
                                         s.D_scale, None, None, bias.float(), True)
    # (the int8 state was requantised in place; the second return value is the fp32 state the output was formed from)
    return _gate_rotate_project(m, y.reshape(b, -1), z.contiguous())


# ---- Mamba1 mixers (W8A8QMamba / W4A8QMamba, quamba/qMambaLayer.py:512-1003) ----------------------------------------------
def _mamba1_rotate_project(m, y16):
    if hasattr(m.had, "x_H_scale"):
        q, _ = ohad.quant_hadamard(y16.reshape(-1, y16.shape[-1]), m.had.had_scale / m.had.x_H_scale)
    else:                                                # QAct: clamp(x / scale), cast truncates (qActLayer.py:24)
        q = (y16.reshape(-1, y16.shape[-1]) / m.had.scale).clamp(min=-128, max=127).to(torch.int8)
    return _w4a8(m.out_proj, q, False)


def mamba1_forward(m, u_int8, want_states=False):
    """u_int8 (b, l, d_model) -> fp16 (b, l, d_model) [, conv_state (b, d_inner, d_conv) int8, ssm_state (b, d_inner, N) int8]
    in the order of W8A8QMamba.forward (qMambaLayer.py:903-940)."""
    b, l, _ = u_int8.shape
    R, N, D = m.dt_rank, m.d_state, m.d_inner
    xz = _w4a8(m.in_proj, u_int8.reshape(b * l, -1), True).reshape(b, l, 2 * D).transpose(1, 2)       # (b, 2D, l)
    x, z = xz[:, :D], xz[:, D:]
    c = m.conv1d
    conv_state = torch.nn.functional.pad(x, (m.d_conv - l, 0)).contiguous()
    x = oconv.quant_causal_conv1d_fwd(x, c.input_scale, c.weight, c.weight_scale, c.output_scale, c.bias_scale, c.bias, True)
    x_dbl = _w4a8(m.x_proj, x.transpose(1, 2).reshape(b * l, D), True)
    dt, Bq, Cq = torch.split(x_dbl, [R, N, N], dim=-1)
    dt = _w4a8(m.dt_proj, dt.contiguous(), True).reshape(b, l, D).transpose(1, 2)
    Bq = Bq.reshape(b, l, N).transpose(1, 2)[:, None]                                                 # (b, 1, N, l)
    Cq = Cq.reshape(b, l, N).transpose(1, 2)[:, None]
    sc = m.selective_scan
    y, xs, _ = osscan.quant_sscan_fwd(x, sc.u_scale, dt, sc.dt_scale, sc.A_log, sc.A_scale, Bq, sc.B_scale, Cq, sc.C_scale,
                                      sc.ssm_state_scale, sc.D, sc.D_scale, z, sc.z_scale, sc.dt_bias, sc.dt_bias_scale,
                                      sc.delta_softplus)
    out = _mamba1_rotate_project(m, y.reshape(b * l, D)).reshape(b, l, -1)
    return (out, conv_state, xs[:, :, -1, :].contiguous()) if want_states else out


def mamba1_step(m, u_int8, conv_state, ssm_state):
    """One decode token: u_int8 (b, d_model); conv_state (b, d_inner, d_conv) and ssm_state (b, d_inner, N) int8 are updated
    in place (qMambaLayer.py:942-962).  Returns fp16 (b, d_model)."""
    R, N, D = m.dt_rank, m.d_state, m.d_inner
    xz = _w4a8(m.in_proj, u_int8, True)
    x, z = xz[:, :D], xz[:, D:]
    c = m.conv1d
    x = oconv.quant_causal_conv1d_update(x, conv_state, c.input_scale, c.weight, c.weight_scale, c.output_scale, c.bias_scale, c.bias, True)
    x_dbl = _w4a8(m.x_proj, x, True)
    dt, Bq, Cq = torch.split(x_dbl, [R, N, N], dim=-1)
    dt = _w4a8(m.dt_proj, dt.contiguous(), True)
    sc = m.selective_scan
    y, _ = oupd.quant_sscan_update(ssm_state, x, sc.u_scale, dt, sc.dt_scale, sc.A_log, sc.A_scale, sc.ssm_state_scale, Bq.contiguous(),
                                   sc.B_scale, Cq.contiguous(), sc.C_scale, sc.D, sc.D_scale, z, sc.z_scale, sc.dt_bias,
                                   sc.dt_bias_scale, sc.delta_softplus)
    return _mamba1_rotate_project(m, y)


def _embed(e, ids):
    if e.weight.dtype == torch.int32:
        return oemb.lookup_w4(ids, e.weight.data, e.scales)
    if e.weight.dtype == torch.int8:
        return oemb.lookup_w8(ids, e.weight.data, e.scales)
    return e.weight.data[ids]


def model_forward(model, input_ids, num_last_tokens=0, states=None):
    """Prefill of a QuambaLMHeadModel-shaped object on CPU: logits fp16.  ``states`` (dict) receives each layer's
    (conv_state, ssm_state)."""
    bb = model.backbone
    h = _embed(bb.embedding, input_ids)
    b, l, d = h.shape
    residual = None
    for i, layer in enumerate(bb.layers):
        nq = layer.norm
        q, residual, _ = onorm.qlayer_norm_fwd(h.reshape(b * l, d), nq.weight, None, nq.eps, residual,
                                               static_out_scale=nq.output_scale, residual_dtype=torch.float32)
        fwd = mamba1_forward if hasattr(layer.mixer, "selective_scan") else mixer_forward
        if states is None:
            h = fwd(layer.mixer, q.reshape(b, l, d))
        else:
            h, cs, ss = fwd(layer.mixer, q.reshape(b, l, d), True)
            states[i] = (cs, ss)
    h, residual = h.reshape(b, l, d), residual.reshape(b, l, d)
    if num_last_tokens > 0:
        h, residual = h[:, -num_last_tokens:], residual[:, -num_last_tokens:]
    rows = h.shape[0] * h.shape[1]
    q, _, _ = onorm.qlayer_norm_fwd(h.reshape(rows, d), bb.norm_f.weight, None, bb.norm_f.eps, residual.reshape(rows, d),
                                    static_out_scale=bb.norm_f.output_scale, residual_dtype=torch.float32)
    return _w4a8(model.lm_head, q, False).reshape(b, -1, model.lm_head.out_features)


def model_step(model, token_ids, states):
    """One decode step on CPU: token_ids (b,), states from model_forward (updated in place).  Returns logits (b, V)."""
    bb = model.backbone
    h = _embed(bb.embedding, token_ids)
    residual = None
    for i, layer in enumerate(bb.layers):
        nq = layer.norm
        q, residual, _ = onorm.qlayer_norm_fwd(h, nq.weight, None, nq.eps, residual, static_out_scale=nq.output_scale,
                                               residual_dtype=torch.float32)
        h = (mamba1_step if hasattr(layer.mixer, "selective_scan") else mixer_step)(layer.mixer, q, *states[i])
    q, _, _ = onorm.qlayer_norm_fwd(h, bb.norm_f.weight, None, bb.norm_f.eps, residual, static_out_scale=bb.norm_f.output_scale,
                                    residual_dtype=torch.float32)
    return _w4a8(model.lm_head, q, False)


# ---- the dequantise-then-fp32 path (the role of the reference's float torch path on CPU) -------------------------------
def _deq_w4a8(lin):
    """Float (N, K) weight a W4A8 layer multiplies with, and its per-column output factor."""
    per_channel = lin.s_group.numel() == 0
    q = olin.unpack_weight(lin.weight, lin.size_k, lin.size_n, per_channel)
    sg, sc = olin.unpermute_scales(None if per_channel else lin.s_group, lin.s_channel.float(), lin.size_n, per_channel)
    group = lin.size_k if per_channel else lin.size_k // sg.shape[0]
    w8 = olin.dequant_to_int8(q, sg, group).float()                     # (K, N) integer values
    w = (w8 * sc.float()[None, :] * lin.input_scale.float()).t().contiguous()
    return w[:lin.out_features]


class FloatPath:
    """The quantized model's weights dequantised once to fp32; ``prefill`` / ``step`` then run plain float torch ops
    (F.linear, conv1d + SiLU, chunked SSD einsums, RMS norms, a dense Hadamard product) with activations kept in
    floating point.  This is the CPU baseline the benchmark times; building it is not part of the timed work."""

    def __init__(self, model, layers=None):
        bb = model.backbone
        ids = torch.arange(bb.embedding.weight.shape[0])
        self.table = _embed(bb.embedding, ids).float()
        self.layers = []
        for layer in list(bb.layers)[:layers]:
            m, s, c = layer.mixer, layer.mixer.qchunk_scan, layer.mixer.conv1d
            gn = m.ngroups * m.d_state
            seg = torch.cat([torch.full((n,), v) for n, v in ((m.d_ssm, c.wx_scale), (gn, c.wB_scale), (gn, c.wC_scale))])
            bseg = torch.cat([torch.full((n,), v) for n, v in ((m.d_ssm, c.bx_scale), (gn, c.bB_scale), (gn, c.bC_scale))])
            # in_proj's int8 outputs carry their output scales inside s_channel: multiply them back
            col = torch.cat([torch.full((n,), float(v)) for n, v in
                             ((m.d_ssm, layer.mixer.norm.z_scale), (m.d_ssm, c.x_scale), (gn, c.B_scale), (gn, c.C_scale),
                              (m.nheads, float(s.dt_scale)))])
            self.layers.append(dict(
                m=m, norm_w=layer.norm.weight.float(), norm_eps=layer.norm.eps, norm_scale=layer.norm.output_scale,
                w_in=_deq_w4a8(m.in_proj) * col[:, None], w_out=_deq_w4a8(m.out_proj),
                conv_w=c.weight.float() * seg[:, None], conv_b=c.bias.float() * bseg,
                A=-torch.exp(s.A_log.float() * s.A_log_scale), D=s.D.float() * s.D_scale, dt_bias=s.dt_bias.float(),
                gate_w=m.norm.weight.float(), H=ohad.hadamard_matrix(m.d_inner).float() / (m.d_inner ** 0.5)))
        self.norm_f_w, self.norm_f_eps = bb.norm_f.weight.float(), bb.norm_f.eps
        self.w_head = _deq_w4a8(model.lm_head)
        self.head_in_scale = float(bb.norm_f.output_scale)

    @staticmethod
    def _rms(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def prefill(self, input_ids, num_last_tokens=1):
        F = torch.nn.functional
        h = self.table[input_ids]
        residual = torch.zeros_like(h)
        b, l, _ = h.shape
        for p in self.layers:
            m = p["m"]
            gn = m.ngroups * m.d_state
            residual = residual + h
            # w_in already holds input_scale: feed it the activation in units of that scale
            u = self._rms(residual, p["norm_w"], p["norm_eps"]) / p["norm_scale"]
            zxbcdt = F.linear(u, p["w_in"])
            z, xBC, dt = torch.split(zxbcdt, [m.d_ssm, m.d_ssm + 2 * gn, m.nheads], dim=-1)
            xBC = F.silu(F.conv1d(xBC.transpose(1, 2), p["conv_w"][:, None, :], p["conv_b"], padding=m.d_conv - 1,
                                  groups=xBC.shape[-1])[..., :l].transpose(1, 2))
            x, B, C = torch.split(xBC, [m.d_ssm, gn, gn], dim=-1)
            y = _ssd_float(x.unflatten(-1, (m.nheads, m.headdim)), F.softplus(dt + p["dt_bias"]), p["A"],
                           B.unflatten(-1, (m.ngroups, m.d_state)), C.unflatten(-1, (m.ngroups, m.d_state)), p["D"],
                           m.chunk_size)
            gs = m.d_ssm // m.ngroups
            yg = (y.flatten(-2) * F.silu(z)).unflatten(-1, (-1, gs))
            yn = (yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + m.norm.eps)).flatten(-2) * p["gate_w"]
            rot = (yn @ p["H"].t()) / m.had.x_H_scale          # in units of out_proj's input scale
            h = F.linear(rot, p["w_out"])
        residual = residual + h
        if num_last_tokens > 0:
            residual = residual[:, -num_last_tokens:]
        y = self._rms(residual, self.norm_f_w, self.norm_f_eps) / self.head_in_scale
        return F.linear(y, self.w_head)


def _ssd_float(x, dt, A, B, C, D, chunk):
    b, l, h, p = x.shape
    rep = h // B.shape[2]
    state = x.new_zeros(b, h, p, B.shape[3])
    ys = []
    for s in range(0, l, chunk):
        xc, dtc = x[:, s:s + chunk], dt[:, s:s + chunk]
        Bc, Cc = B[:, s:s + chunk].repeat_interleave(rep, 2), C[:, s:s + chunk].repeat_interleave(rep, 2)
        cs = torch.cumsum(dtc * A, dim=1)
        q = xc.shape[1]
        keep = torch.tril(torch.ones(q, q, dtype=torch.bool))[None, :, :, None]
        w = torch.exp((cs[:, :, None, :] - cs[:, None, :, :]).masked_fill(~keep, -float("inf"))) * dtc[:, None, :, :]
        y = torch.einsum("btsh,bshp->bthp", torch.einsum("bthn,bshn->btsh", Cc, Bc) * w, xc)
        y = y + torch.einsum("bthn,bhpn->bthp", Cc, state) * torch.exp(cs)[..., None]
        tail = torch.exp(cs[:, -1:, :] - cs) * dtc
        state = state * torch.exp(cs[:, -1, :])[:, :, None, None] + torch.einsum("bshn,bsh,bshp->bhpn", Bc, tail, xc)
        ys.append(y)
    return torch.cat(ys, 1) + x * D[None, None, :, None]
