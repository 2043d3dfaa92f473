"""Per-kernel measurements behind ``bench.py --op NAME``: one JSON line per op with its own roofline.

Each op runs at the per-layer shape of the model configuration it belongs to (Mamba2-2.7B: d_model 2560, 80 heads x 64,
d_state 128; Mamba1-2.8B: d_inner 5120, d_state 16), through the public ops API, inputs resident in HBM.  Timing: the
call is captured into one CUDA graph per input set, the sets are replayed round-robin (enough sets that consecutive
replays cannot hit L2: their summed footprint exceeds twice the 126 MB L2), CUDA events on the replay stream.
"""
import json
import math
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
L2_BYTES = 126 * 2 ** 20


def _peaks():
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        p = json.loads(pk.read_text())
        return float(p.get("hbm_gbs", 6650.0)), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def _i8(shape, dev, gen, std=40.0):
    return (torch.randn(shape, device=dev, generator=gen) * std).round_().clamp_(-127, 127).to(torch.int8)


class _ScaleCache:
    """One-element fp32 device tensors by value, created before graph capture and reused inside it."""

    def __init__(self, dev):
        self.dev, self.t = dev, {}

    def __call__(self, v):
        if v not in self.t:
            self.t[v] = torch.tensor([v], device=self.dev)
        return self.t[v]


def _sets_for(footprint_bytes, cap=48):
    return max(2, min(cap, math.ceil(2.2 * L2_BYTES / max(footprint_bytes, 1))))


def time_graphs(make_call, nsets, steps, warmup, stream):
    """make_call(i) -> zero-argument callable running the op on input set i.  One CUDA graph holds one call per input
    set, back to back (as the ops sit in a model's captured step), so that a replay's launch cost is shared by nsets
    invocations; the figure returned is the time per invocation."""
    calls = [make_call(i) for i in range(nsets)]
    with torch.cuda.stream(stream):
        for c in calls:
            c()
        stream.synchronize()
        keep = []
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for c in calls:
                keep.append(c())
        for i in range(max(warmup, 3)):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        replays = max(1, -(-steps // nsets))
        e0.record(stream)
        for i in range(replays):
            g.replay()
        e1.record(stream)
        e1.synchronize()
    return e0.elapsed_time(e1) / (replays * nsets)


# ---------------------------------------------------------------------------------------------------------------------
def op_conv(dev, gen, ops):
    B, L, H, P, G, N, W = 4, 2048, 80, 64, 1, 128, 4
    C = H * P + 2 * G * N
    by = 2 * B * C * L + C * (W + 1)
    n = _sets_for(by)
    w, b = _i8((C, W), dev, gen), _i8((C,), dev, gen)
    sx, sB, sC = (torch.tensor([v], device=dev) for v in (0.02, 0.015, 0.017))
    xs = [_i8((B, L, C), dev, gen).transpose(1, 2) for _ in range(n)]

    def mk(i):
        return lambda: ops.quamba2_conv1d_cuda.fwd(xs[i], 0.03, 0.03, 0.03, H * P, P, N, G, None, None, sx, sB,
                                                   sC, w, 0.004, 0.004, 0.004, b, 0.0005, 0.0005, 0.0005, None, None,
                                                   None, True)
    return dict(workload=f"Quamba2 conv1d fwd B{B} L{L} C{C} W{W} channel-last", bytes=by, flops=0, nsets=n, make=mk,
                kernel="conv1d_channel_last_kernel", launches=1)


def op_conv_update(dev, gen, ops):
    B, H, P, G, N, W = 64, 80, 64, 1, 128, 4
    C = H * P + 2 * G * N
    by = B * C * (2 + 2 * W) + C * (W + 1)
    n = _sets_for(by)
    w, b = _i8((C, W), dev, gen), _i8((C,), dev, gen)
    sx, sB, sC = (torch.tensor([v], device=dev) for v in (0.02, 0.015, 0.017))
    xs = [_i8((B, C), dev, gen) for _ in range(n)]
    st = [_i8((B, C, W), dev, gen) for _ in range(n)]

    def mk(i):
        return lambda: ops.quamba2_conv1d_cuda.update(xs[i], st[i], 0.03, 0.03, 0.03, H * P, P, N, G, None, None, sx,
                                                      sB, sC, w, 0.004, 0.004, 0.004, b, 0.0005, 0.0005, 0.0005,
                                                      None, None, None, True)
    return dict(workload=f"Quamba2 conv1d decode step B{B} C{C} W{W}", bytes=by, flops=0, nsets=n, make=mk,
                kernel="conv1d_update_kernel", launches=1)


def op_hadamard(dev, gen, ops):
    M, D = 8192, 5120
    by = 3 * M * D
    n = _sets_for(by)
    xs = [torch.randn((M, D), device=dev, generator=gen, dtype=torch.float16) for _ in range(n)]

    def mk(i):
        return lambda: ops.quant_hadamard.fast_hadamard_transform_40N(xs[i], 1.0 / math.sqrt(D) / 0.03)
    return dict(workload=f"Hadamard(40 x 128) + int8 quantise, {M} rows x {D} fp16", bytes=by, flops=0, nsets=n, make=mk,
                kernel="hadamard_quant_kernel", launches=1)


def op_sscan(dev, gen, ops):
    B, D, L, N = 16, 5120, 1024, 16
    by = B * D * L * 5 + 2 * B * N * L + B * D * N + D * (N + 2)
    n = _sets_for(by, cap=3)
    A = _i8((D, N), dev, gen)
    Dv, bias = _i8((D,), dev, gen), _i8((D,), dev, gen)
    s = _ScaleCache(dev)
    sets = [dict(u=_i8((B, D, L), dev, gen), dt=_i8((B, D, L), dev, gen), z=_i8((B, D, L), dev, gen),
                 Bm=_i8((B, 1, N, L), dev, gen), Cm=_i8((B, 1, N, L), dev, gen)) for _ in range(n)]

    def mk(i):
        d = sets[i]
        return lambda: ops.quant_sscan_cuda.fwd(d["u"], s(0.03), d["dt"], s(0.03), A, s(0.02), d["Bm"], s(0.03), d["Cm"], s(0.03),
                                                s(0.05), Dv, s(0.01), d["z"], s(0.03), bias, s(0.03), True)
    return dict(workload=f"Mamba1 int8 selective scan fwd B{B} D{D} L{L} N{N} (Mamba1-2.8B layer, batch 16 x 1024)", bytes=by,
                flops=0, nsets=n, make=mk, kernel="sscan_fwd_kernel", launches=1)


def op_ssd(dev, gen, ops):
    B, L, H, P, G, N, Q = 4, 2048, 80, 64, 1, 128, 256
    by = B * L * (H * P + H + 2 * G * N) + 2 * B * L * H * P + B * H * P * N
    n = _sets_for(by)
    s = _ScaleCache(dev)
    A, Dv = _i8((H,), dev, gen), _i8((H,), dev, gen)
    bias = (torch.rand(H, device=dev, generator=gen) * 2 - 4).half()
    sets = [dict(x=_i8((B, L, H, P), dev, gen), dt=_i8((B, L, H), dev, gen), Bm=_i8((B, L, G, N), dev, gen),
                 Cm=_i8((B, L, G, N), dev, gen)) for _ in range(n)]

    def mk(i):
        d = sets[i]
        return lambda: ops._quant_mamba_chunk_scan_combined_fwd(d["x"], s(0.03), d["dt"], s(0.03), A, s(0.02), d["Bm"], s(0.03),
                                                                d["Cm"], s(0.03), s(0.01), Q, Dv, s(0.01), None, None, bias, None,
                                                                None, None, True)
    fl = 2 * B * H * L * 128 * (N + P + 2 * P)          # per 128-token block: C.B^T, Lm.X, C.S, Xw^T.B
    return dict(workload=f"Mamba2 int8 SSD chunk scan B{B} L{L} H{H} P{P} G{G} N{N} Q{Q}", bytes=by, flops=fl, nsets=n, make=mk,
                kernel="ssd_tc_kernel (+ ssd_prep_kernel)", launches=2)


def op_ssd_update(dev, gen, ops):
    B, H, P, G, N = 64, 80, 64, 1, 128
    by = 2 * B * H * P * N + B * (H * P * 3 + H + 2 * G * N)
    n = _sets_for(by)
    s = _ScaleCache(dev)
    A = _i8((H,), dev, gen)[:, None, None].expand(-1, P, N)
    Dv = _i8((H,), dev, gen)[:, None].expand(-1, P)
    bias = (torch.rand(H, device=dev, generator=gen) * 2 - 4).half()[:, None].expand(-1, P)
    sets = [dict(st=_i8((B, H, P, N), dev, gen), x=_i8((B, H, P), dev, gen), dt=_i8((B, H), dev, gen)[:, :, None].expand(-1, -1, P),
                 Bm=_i8((B, G, N), dev, gen), Cm=_i8((B, G, N), dev, gen)) for _ in range(n)]

    def mk(i):
        d = sets[i]
        return lambda: ops.quant_sscan_update_triton(d["st"], d["x"], s(0.03), d["dt"], s(0.03), A, s(0.02), s(0.01), d["Bm"],
                                                     s(0.03), d["Cm"], s(0.03), Dv, s(0.01), None, None, bias, None, True)
    return dict(workload=f"Mamba2 int8 state update (decode) B{B} H{H} P{P} N{N}", bytes=by, flops=0, nsets=n, make=mk,
                kernel="sscan_update_kernel", launches=1)


def _w4a8(dev, gen, ops, M, K, N, out_int8, tag, group=128):
    from quamba_b200.packing import w4a8_quantize
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(K, N, generator=g) * 0.02).half()
    _, packed, sg, sc = w4a8_quantize(w, 4, group)
    packed, sg, sc = packed.to(dev), sg.to(dev), sc.to(dev)
    by = M * K + K * N // 2 + M * N * (1 if out_int8 else 2)
    # The weights dominate the footprint of a decode-sized call: every input set then gets its own copy of them (the
    # int8 expansion the kernel streams is 2 bytes per packed byte), so that they come from HBM as they do in a model
    # whose layers each have their own weights, not from L2.
    n = _sets_for(by if M >= 32 else M * K + (K * N if group > 0 else K * N // 2) + M * N)
    packs = [packed] if M >= 4096 else [packed.clone() for _ in range(n)]
    xs = [_i8((M, K), dev, gen) for _ in range(n)]
    st = torch.tensor(0.03, device=dev)
    ws = torch.zeros(N // 64 * 16, dtype=torch.int32, device=dev)
    fn = ops.quant_linear_cuda.w4a8o8_gemm if out_int8 else ops.quant_linear_cuda.w4a8o16_gemm

    def mk(i):
        return lambda: fn(xs[i], packs[i % len(packs)], st, sc, sg, ws, M, N, K, False)
    return dict(workload=f"W4A8 GEMM {tag}: M{M} K{K} N{N}, int4 {'group-128' if group > 0 else 'per-channel'} weights, {'int8' if out_int8 else 'fp16'} out",
                bytes=by, flops=2 * M * N * K, nsets=n, make=mk, launches=1,
                kernel=("gemm_s8_tcgen05_persistent_kernel" if M >= 128 else "gemm_s8_tcgen05_kernel<64>" if M >= 32 else
                        "gemv_s4_kernel" if group < 0 else "gemv_s8_kernel"),
                note="weights unpacked to int8 once at first use (cached); the timed GEMM streams int8 weights")


def op_w4a8_in(dev, gen, ops):
    return _w4a8(dev, gen, ops, 8192, 2560, 10624, True, "Mamba2-2.7B in_proj, 4 x 2048 tokens")


def op_w4a8_out(dev, gen, ops):
    return _w4a8(dev, gen, ops, 8192, 5120, 2560, False, "Mamba2-2.7B out_proj, 4 x 2048 tokens")


def op_w4a8_in_b1(dev, gen, ops):
    return _w4a8(dev, gen, ops, 2048, 2560, 10624, True, "Mamba2-2.7B in_proj, 1 x 2048 tokens", group=-1)


def op_w4a8_out_b1(dev, gen, ops):
    return _w4a8(dev, gen, ops, 2048, 5120, 2560, False, "Mamba2-2.7B out_proj, 1 x 2048 tokens", group=-1)


def op_rmsnorm(dev, gen, ops):
    M, N = 2048, 2560
    by = M * N * (2 + 4 + 4 + 1)
    n = _sets_for(by)
    w = torch.ones(N, dtype=torch.float16, device=dev)
    xs = [torch.randn((M, N), device=dev, generator=gen).half() for _ in range(n)]
    rs = [torch.randn((M, N), device=dev, generator=gen) for _ in range(n)]

    def mk(i):
        return lambda: ops._qlayer_norm_fwd(xs[i], w, None, 1e-5, rs[i], static_out_scale=0.03, is_rms_norm=True)
    return dict(workload=f"QRMSNorm + residual add, Mamba2-2.7B block norm at 1 x 2048 tokens: M{M} N{N}, fp16 x, fp32 residual in and out, int8 out",
                bytes=by, flops=0, nsets=n, make=mk, kernel="norm_quant_kernel<2, 0, 5>", launches=1)


def op_rmsnorm_partials(dev, gen, ops):
    """The block norm of a head-parallel layer at eight ranks: sums the eight received fp16 slots of this rank's rows itself."""
    T, M, N = 8, 4096, 4096
    by = M * N * (2 * T + 4 + 4 + 1)
    n = _sets_for(by)
    w = torch.ones(N, dtype=torch.float16, device=dev)
    xs = [torch.randn((T, M, N), device=dev, generator=gen).half() for _ in range(n)]
    rs = [torch.randn((M, N), device=dev, generator=gen) for _ in range(n)]

    def mk(i):
        return lambda: ops._qlayer_norm_fwd(xs[i][0], w, None, 1e-5, rs[i], static_out_scale=0.03, is_rms_norm=True,
                                            partials=(xs[i], 0, None))
    return dict(workload=f"QRMSNorm + residual add over the sum of {T} partial inputs (head-parallel Mamba2-8B at eight ranks, one chunk's rows "
                         f"of one rank): M{M} N{N}, {T} fp16 slots, fp32 residual in and out, int8 out",
                bytes=by, flops=0, nsets=n, make=mk, kernel="norm_quant_kernel<4, 0, 4> (n_partials = 8)", launches=1)


def op_rmsnorm_gated(dev, gen, ops):
    M, N = 2048, 5120
    by = M * N * (2 + 1 + 2)
    n = _sets_for(by)
    w = torch.ones(N, dtype=torch.float16, device=dev)
    xs = [torch.randn((M, N), device=dev, generator=gen).half() for _ in range(n)]
    zs = [_i8((M, N), dev, gen) for _ in range(n)]

    def mk(i):
        return lambda: ops._qlayer_normgated_fwd(xs[i], w, None, 1e-5, q_z=zs[i], z_scale=0.02, use_float16_output=True,
                                                 group_size=N, norm_before_gate=False, is_rms_norm=True)
    return dict(workload=f"gated RMSNorm, Mamba2-2.7B at 1 x 2048 tokens: M{M} N{N}, fp16 x, int8 gate, fp16 out",
                bytes=by, flops=0, nsets=n, make=mk, kernel="norm_quant_kernel<4, 1, 5>", launches=1)


def op_w4a8_decode(dev, gen, ops):
    return _w4a8(dev, gen, ops, 1, 2560, 10624, True, "Mamba2-2.7B in_proj, one token")


def op_w4a8_decode_pc(dev, gen, ops):
    return _w4a8(dev, gen, ops, 1, 2560, 10624, True, "Mamba2-2.7B in_proj, one token", group=-1)


def op_w4a8_decode_b64(dev, gen, ops):
    return _w4a8(dev, gen, ops, 64, 2560, 10624, True, "Mamba2-2.7B in_proj, 64 sequences x one token")


def _decode_linear_layer(dev, K, N, seed):
    from quamba_b200.modules import W4A8B8O8Linear, W4A8B16O16Linear
    lin = torch.nn.Linear(K, N, bias=False)
    lin.weight.data = torch.randn(N, K, generator=torch.Generator().manual_seed(seed)) * 0.02
    lin.w4_group_size = -1
    return lin


def op_decode_in_proj(dev, gen, ops):
    """Launch 1 of the fused decode step at the 2.7B shape: residual add + RMSNorm + quantise + in_proj (nibble weights) +
    conv1d update in the epilogue, one token."""
    from quamba_b200.modules import W4A8B8O8Linear
    K, N, D, GN = 2560, 10576, 5120, 128
    import copy
    n = _sets_for(K * N // 2)
    first = W4A8B8O8Linear.from_fp16(_decode_linear_layer(dev, K, N, 0), torch.tensor(0.03), torch.tensor(0.05)).to(dev)
    layers = [first] + [copy.deepcopy(first) for _ in range(n - 1)]       # every set streams its own copy of the weights
    preps = [l.prepared() for l in layers]
    x = torch.randn((1, K), device=dev, generator=gen).half()
    res = torch.randn((1, K), device=dev, generator=gen)
    nw = torch.ones(K, dtype=torch.float16, device=dev)
    C = D + 2 * GN
    convs = []
    for i in range(n):
        st = torch.zeros((1, 4, C), dtype=torch.int8, device=dev).transpose(1, 2)
        convs.append(dict(state=st, weight=_i8((C, 4), dev, gen), bias=None, col0=D, x_dim=D, gn=GN, scale_in=(1e-4, 1e-4, 1e-4),
                          scale_bias=(0.0, 0.0, 0.0), out_scales=tuple(torch.tensor([0.02], device=dev) for _ in range(3))))

    def mk(i):
        return lambda: ops.decode_norm_linear(x, res, nw, 1e-5, 0.03, preps[i], layers[i].input_scale, True, True, convs[i])
    by = K * layers[0].size_n // 2 + K * 10 + layers[0].size_n
    return dict(workload=f"fused decode launch 1, Mamba2-2.7B: residual + RMSNorm + in_proj {K} -> {layers[0].size_n} (4-bit weights from HBM) + conv1d update, one token",
                bytes=by, flops=0, nsets=n, make=mk, kernel="decode_norm_linear_kernel<1, 1, 1>", launches=1)


def op_decode_out_proj(dev, gen, ops):
    from quamba_b200.modules import W4A8B16O16Linear
    K, N = 5120, 2560
    import copy
    n = _sets_for(K * N // 2)
    first = W4A8B16O16Linear.from_fp16(_decode_linear_layer(dev, K, N, 100), torch.tensor(0.03)).to(dev)
    layers = [first] + [copy.deepcopy(first) for _ in range(n - 1)]
    preps = [l.prepared() for l in layers]
    a = _i8((1, K), dev, gen)

    def mk(i):
        return lambda: ops.decode_linear(a, preps[i], layers[i].input_scale)
    return dict(workload=f"fused decode launch 4, Mamba2-2.7B: out_proj {K} -> {N} on int8 input (4-bit weights from HBM), one token",
                bytes=K * N // 2 + K + 2 * N, flops=0, nsets=n, make=mk, kernel="decode_norm_linear_kernel<1, 1, 0>", launches=1)


def op_decode_gate_had(dev, gen, ops):
    D = 5120
    n = 8
    ys = [torch.randn((1, D), device=dev, generator=gen).half() for _ in range(n)]
    zs = [_i8((1, D), dev, gen) for _ in range(n)]
    w = torch.ones(D, dtype=torch.float16, device=dev)

    def mk(i):
        return lambda: ops.decode_gate_had_quant(ys[i], zs[i], 0.02, w, 1e-5, D, (1.0 / D ** 0.5) / 0.05)
    return dict(workload=f"fused decode launch 3, Mamba2-2.7B: gate + RMSNorm + Hadamard (40 x 128) + int8 quantise of one row of {D}",
                bytes=D * (2 + 1 + 2 + 1), flops=0, nsets=n, make=mk, kernel="decode_gate_had_quant_kernel", launches=1,
                note="latency-bound: 36 KB of traffic; the figure of merit is the time, not the bandwidth")


def op_decode_update(dev, gen, ops):
    H, P, N = 80, 64, 128
    n = 8
    states = [_i8((1, H, P, N), dev, gen) for _ in range(n)]
    x = _i8((1, H, P), dev, gen)
    dt = _i8((1, H), dev, gen)
    Bm, Cm = _i8((1, 1, N), dev, gen), _i8((1, 1, N), dev, gen)
    A = _i8((H,), dev, gen)
    one = torch.tensor([0.02], device=dev)
    bias = torch.zeros((H,), dtype=torch.float16, device=dev)

    def mk(i):
        return lambda: ops.quant_sscan_update_triton(states[i], x, one, dt[:, :, None].expand(-1, -1, P), one, A[:, None, None].expand(-1, P, N), one,
                                                     one, Bm, one, Cm, one, None, None, None, None, bias[:, None].expand(-1, P), None, True)
    return dict(workload=f"fused decode launch 2, Mamba2-2.7B: int8 state update of one token, H{H} P{P} N{N} (one CTA per head)",
                bytes=2 * H * P * N + H * P * 3 + H + 2 * N, flops=0, nsets=n, make=mk, kernel="sscan_update_small_kernel", launches=1)


def op_w8a8(dev, gen, ops):
    M, K, N = 16384, 2560, 10240
    by = M * K + K * N + M * N
    n = _sets_for(by)
    w = _i8((N, K), dev, gen).t()
    xs = [_i8((M, K), dev, gen) for _ in range(n)]
    a, b = torch.tensor([[0.5]], device=dev), torch.tensor([[0.001]], device=dev)
    ys = [torch.empty((M, N), dtype=torch.int8, device=dev) for _ in range(n)]

    def mk(i):
        return lambda: ops.quant_linear_cuda.cutlass_scaled_mm_dq(ys[i], xs[i], w, a, b)
    return dict(workload=f"W8A8 GEMM Mamba1-2.8B in_proj, 16 x 1024 tokens: M{M} K{K} N{N}, int8 out", bytes=by,
                flops=2 * M * N * K, nsets=n, make=mk, kernel="gemm_s8_tcgen05_kernel", launches=1)


OPS = {"conv": op_conv, "conv_update": op_conv_update, "hadamard": op_hadamard, "sscan": op_sscan, "ssd": op_ssd,
       "ssd_update": op_ssd_update, "w4a8_in_proj": op_w4a8_in, "w4a8_out_proj": op_w4a8_out,
       "w4a8_in_proj_b1": op_w4a8_in_b1, "w4a8_out_proj_b1": op_w4a8_out_b1, "rmsnorm": op_rmsnorm, "rmsnorm_partials": op_rmsnorm_partials,
       "rmsnorm_gated": op_rmsnorm_gated, "w4a8_decode": op_w4a8_decode, "w4a8_decode_pc": op_w4a8_decode_pc, "w4a8_decode_b64": op_w4a8_decode_b64,
       "decode_in_proj": op_decode_in_proj, "decode_update": op_decode_update, "decode_gate_had": op_decode_gate_had,
       "decode_out_proj": op_decode_out_proj, "w8a8": op_w8a8}


def i8_peak():
    """The dense int8 rate of tcgen05.mma kind::i8 (qb_i8_mma_peak): a burst (about 5 ms) and a sustained run (about 2 s,
    under the power cap), next to the measured bf16 cuBLAS peak."""
    import ctypes
    from quamba_b200 import _lib
    f = _lib.lib().qb_i8_mma_peak
    f.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    for tag, groups, repeats in (("burst", 4096, 4), ("sustained", 65536, 100)):
        tops, ms = ctypes.c_double(), ctypes.c_double()
        _lib.check(f(groups, repeats, ctypes.c_void_p(st), ctypes.byref(tops), ctypes.byref(ms)))
        out[tag] = {"tops": tops.value, "ms": ms.value}
    _lib.read_device_status(st)
    hbm, bf16, src = _peaks()
    return {"op": "i8_peak", "metric": "int8_tensor_tops", "value": out["burst"]["tops"], "unit": "TOP/s", "n_gpus": 1,
            "higher_is_better": True, "data": "synthetic", "sustained_tops": out["sustained"]["tops"],
            "ms": {k: v["ms"] for k, v in out.items()}, "bf16_cublas_tflops": bf16, "ratio_to_bf16": out["burst"]["tops"] / bf16,
            "config": {"workload": "tcgen05.mma kind::i8 M128 N256 K32, operands resident in shared memory, one CTA per SM, "
                                   "two alternating TMEM accumulators, no loads and no epilogue"}}


def run(name, steps, warmup):
    """Returns the list of JSON-able result lines for ``name`` ('all' runs every op)."""
    from quamba_b200 import _lib, ops
    assert torch.cuda.is_available(), "needs a CUDA device; there is no CPU fallback"
    if name == "i8_peak":
        return [i8_peak()]
    dev = torch.device("cuda", 0)
    hbm, bf16, src = _peaks()
    i8_file = ROOT / "profiles" / "int8_mma_peak.json"      # a kernel timed alone: the burst figure
    int8_peak = float(json.loads(i8_file.read_text())["tops"]) if i8_file.exists() else 2.0 * bf16
    stream = torch.cuda.Stream(device=dev)
    out = []
    for nm in (list(OPS) if name == "all" else [name]):
        gen = torch.Generator(device=dev).manual_seed(0)
        spec = OPS[nm](dev, gen, ops)
        ms = time_graphs(spec["make"], spec["nsets"], steps, warmup, stream)
        _lib.read_device_status(stream.cuda_stream)
        gbs = spec["bytes"] / (ms * 1e-3) / 1e9
        tfl = spec["flops"] / (ms * 1e-3) / 1e12
        t_hbm, t_tc = spec["bytes"] / (hbm * 1e9), spec["flops"] / (int8_peak * 1e12)
        tensor_bound = nm.startswith("w") and t_tc > t_hbm
        roof = ({"bound": "tensor", "achieved": tfl, "peak": int8_peak, "unit": "TFLOP/s", "frac": tfl / int8_peak}
                if tensor_bound else {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm})
        roof.update(kernel=spec["kernel"], traffic=None, peak_source=src, algorithmic_bytes=spec["bytes"], flops=spec["flops"],
                    ms=ms)
        if tensor_bound:
            roof["peak_note"] = ("measured tcgen05 kind::i8 issue rate, burst (profiles/int8_mma_peak.json)" if i8_file.exists()
                                 else "2 x measured bf16 cuBLAS peak")
        line = {"op": nm, "metric": "kernel_time_ms", "value": ms, "unit": "ms", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3),
                "higher_is_better": False, "data": "synthetic", "config": {"workload": spec["workload"],
                                                                            "l2": f"{spec['nsets']} rotating input sets"},
                "gpu_launches": spec["launches"] * steps, "roofline": roof}
        if "note" in spec:
            line["config"]["note"] = spec["note"]
        out.append(line)
        del spec
        torch.cuda.empty_cache()
    return out
