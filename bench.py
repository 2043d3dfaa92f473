#!/usr/bin/env python
"""Benchmark: Quamba2 Mamba2-2.7B W4A8, prefill tok/s (L = 2048) and decode TPOT, on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --op NAME|all        # one kernel of the path on its own (bench_ops.py), one GPU
    python bench.py --op mixer_core      # the conv1d + SSD op-level configuration (bench_mixer_core.py)
    python bench.py --gpus N (N >= 2)    # head-parallel Mamba2-8B prefill, strong scaling (bench_parallel.py)

Workload (one "step" = one prefill): d_model 2560, 64 layers, expand 2 (80 heads x 64), ngroups 1, d_state 128,
d_conv 4, vocab 50288, random-init weights N(0, 0.02) quantized to int4 (per output channel; ``--group-size 128`` for
the per-group format), int8 activations with static per-tensor scales calibrated on 4 random sequences, batch 1,
2048 uniform-random token ids, then 256 greedy decode steps.  Prints ONE JSON line:

  value     prefill tokens/s, token ids resident on the device, the whole prefill replayed from one CUDA graph, CUDA
            events on the replay stream, max over ranks
  decode    TPOT: the decode step (embedding ... lm_head, greedy argmax, token fed back on the device) replayed 256 times
  e2e       the same prefill from token ids in pinned HOST memory to last-token logits in HOST memory
  roofline  the dominant kernel of the prefill (from a per-call CUDA-event trace of one eager prefill) against its roofline,
            with every entry point's share of the step
  cpu_baseline / --impl reference   the dequantise-then-fp32 torch path of oracle/ on the host cores, bounded sample
"""
import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

MODEL = dict(d_model=2560, n_layer=64, vocab_size=50288, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=256)
PROMPT, DECODE_TOKENS, CALIB_SEQS = 2048, 256, 4
WORKLOAD = ("configs[2]: Quamba2 Mamba2-2.7B W4A8 (d_model 2560, 64 layers, 80 heads x 64, ngroups 1, d_state 128, d_conv 4, "
            "vocab 50288), batch 1, prefill 2048 token ids, then 256 greedy decode tokens")


def peaks():
    pk = ROOT / "MEASURED_PEAKS.json"
    p = json.loads(pk.read_text()) if pk.exists() else {}
    out = dict(hbm=float(p.get("hbm_gbs", 6650.0)), bf16=float(p.get("bf16_tflops", 1590.0)), source="measured" if p else "fallback")
    i8 = ROOT / "profiles" / "int8_mma_peak.json"
    if i8.exists():         # written from a run of `bench.py --op i8_peak` (a tcgen05 kind::i8 issue-rate measurement)
        d = json.loads(i8.read_text())
        # the sustained figure: the GEMMs here are timed inside a step that runs for seconds under the power cap
        out["i8"], out["i8_burst"] = float(d["tops_sustained"]), float(d["tops"])
        out["i8_source"] = "measured tcgen05 kind::i8 issue rate, sustained (profiles/int8_mma_peak.json; burst %.0f)" % d["tops"]
    else:
        out["i8"], out["i8_source"] = 2.0 * out["bf16"], "2 x the measured bf16 cuBLAS peak"
    return out


def gemm_traffic():
    """DRAM bytes (read + written) per launch of the GEMM kernel at the prefill shapes, from the committed summary of an ncu
    launch list of this benchmark; (None, None) when the file is absent."""
    f = ROOT / "profiles" / "model_2p7b_w4a8_traffic.json"
    if not f.exists():
        return None, None
    t = json.loads(f.read_text())
    return t["dram_bytes_read_per_launch"] + t["dram_bytes_write_per_launch"], f"{t['source']} (captured {t['captured']})"


def model_flops_and_bytes(m, L, group_size):
    """Algorithmic int8 flops of one prefill and HBM bytes of one decode token (weights + states + head + embedding row)."""
    D, H, P, G, N = m["d_model"] * m["expand"], m["d_model"] * m["expand"] // m["headdim"], m["headdim"], m["ngroups"], m["d_state"]
    d_in_proj = 2 * D + 2 * G * N + H
    gemm = 2 * L * m["d_model"] * (d_in_proj + D)
    prefill_flops = m["n_layer"] * gemm + 2 * m["d_model"] * m["vocab_size"]
    wbytes = lambda k, n: k * n // 2 + 4 * n + (0 if group_size < 0 else (k // 128) * n * 2)
    layer = (wbytes(m["d_model"], d_in_proj) + wbytes(D, m["d_model"]) + 2 * H * P * N + 2 * 4 * (D + 2 * G * N) +
             2 * m["d_model"] * 4 + 2 * D)
    decode_bytes = m["n_layer"] * layer + wbytes(m["d_model"], m["vocab_size"]) + m["d_model"] // 2
    return prefill_flops, decode_bytes, gemm


# ---- the CPU arm -----------------------------------------------------------------------------------------------------------
def cpu_sample(layers=1, L=512, vocab=4096, model=None, prompt_desc="the 2048 prompt tokens (batch 1)"):
    """oracle/'s dequantise-then-fp32 path on a bounded sample: ``layers`` layers at full width over ``L`` tokens, scaled
    to all the model's layers (every layer has the same shapes), plus the final norm and the head on the last token
    (vocabulary cut to ``vocab`` rows to keep the set-up short; the head's share of a prefill is far below a percent)."""
    import torch
    from oracle import model as omodel
    from quamba_b200 import calibrate as cal
    torch.set_num_threads(os.cpu_count() or 1)
    model = model or MODEL
    cfg = dict(model, n_layer=layers, vocab_size=vocab)
    fm = cal.Mamba2LMFloat(**cfg, w4_group_size=-1, seed=0, device="cpu")
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, vocab, (1, L), generator=g)
    q = cal.quantize_model(fm, cal.calibrate(fm, [ids[:, :128]]))
    del fm
    fp = omodel.FloatPath(q)
    fp.prefill(ids[:, :64])
    t0 = time.perf_counter()
    fp.prefill(ids)
    t_all = time.perf_counter() - t0
    saved, fp.layers = fp.layers, []
    t0 = time.perf_counter()
    fp.prefill(ids)                                   # embedding + final norm + head only
    t_rest = time.perf_counter() - t0
    fp.layers = saved
    per_layer = (t_all - t_rest) / layers
    t_full = per_layer * model["n_layer"] + t_rest
    sample = (f"{layers} of the {model['n_layer']} layers at full width over {L} of {prompt_desc}, time scaled to {model['n_layer']} layers, "
              f"vocabulary cut to {vocab}; torch fp32 on dequantised weights")
    return L / t_full, t_full, sample


def run_reference(args, rank):
    if rank != 0:
        return
    workload = WORKLOAD
    if args.gpus >= 2 or args.model == "8b":      # the GPU arm then runs the head-parallel Mamba2-8B prefill: same workload here
        import bench_parallel as bp
        tok_s, t_full, sample = cpu_sample(model=bp.CFG8B, prompt_desc="the 32 x 4096 prompt tokens")
        workload = bp.WORKLOAD8B
    else:
        tok_s, t_full, sample = cpu_sample()
    cores = os.cpu_count() or 1
    line = {"impl": "reference", "metric": "prefill_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": 1,
            "warmup": 1, "ms_per_step": t_full * 1e3, "higher_is_better": True, "scaling": "weak" if workload == WORKLOAD else "strong",
            "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": workload, "sample": sample},
            "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- the GPU arm -----------------------------------------------------------------------------------------------------------
def build_model(dev, group_size, seed, n_layer):
    """Float model (fp16, torch) -> absmax calibration on 4 random sequences -> quantized model.  Offline work."""
    import torch
    from quamba_b200 import calibrate as cal
    cfg = dict(MODEL, n_layer=n_layer)
    fm = cal.Mamba2LMFloat(**cfg, w4_group_size=group_size, seed=seed, device=dev, dtype=torch.float16)
    g = torch.Generator(device=dev).manual_seed(seed + 1)
    seqs = [torch.randint(0, MODEL["vocab_size"], (1, PROMPT), generator=g, device=dev) for _ in range(CALIB_SEQS)]
    q = cal.quantize_model(fm, cal.calibrate(fm, seqs))
    del fm
    torch.cuda.empty_cache()
    return q


def trace_shares(run, stream):
    """One eager pass of ``run`` with a CUDA-event pair around every C-ABI call: {entry point: (calls, total ms)}.
    Eager launches are host-bound (the device would wait for the host between calls, and an event pair would then time the
    host's launch path, not the kernel), so the stream is first parked on a device-side delay twice as long as the host
    needs to enqueue the whole pass: the device then finds every launch already queued and the event pairs bracket
    kernel time only."""
    import torch
    from quamba_b200 import _lib
    sink = []
    with torch.cuda.stream(stream):
        run()
        stream.synchronize()
        _lib.set_call_trace([])                      # rehearsal with the tracing overhead, to size the delay
        h0 = time.perf_counter()
        run()
        host_ms = (time.perf_counter() - h0) * 1e3
        stream.synchronize()
        _lib.set_call_trace(sink)
        torch.cuda._sleep(int(2.0 * host_ms * 2.0e6))   # ~2 x 10^6 cycles per millisecond at the boost clock
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        run()
        t1.record(stream)
        _lib.set_call_trace(None)
        stream.synchronize()
    agg = {}
    for fn, e0, e1 in sink:
        c, ms = agg.get(fn, (0, 0.0))
        agg[fn] = (c + 1, ms + e0.elapsed_time(e1))
    return agg, t0.elapsed_time(t1)


def measure(model, args, dev, rank, world, group_size, batch=1, vocab=None):
    import torch
    import torch.distributed as dist
    from quamba_b200 import _lib, ops
    from quamba_b200.sharding import max_over_ranks
    steps, warmup = args.steps, max(args.warmup, 3)
    L, ntok = args.seqlen, args.decode_tokens

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    g = torch.Generator().manual_seed(1234 + rank)
    host_ids = [torch.randint(0, vocab or MODEL["vocab_size"], (batch, L), generator=g).pin_memory() for _ in range(3)]
    dev_ids = [t.to(dev) for t in host_ids]
    pre = model.capture_prefill(batch, L)
    st = pre.stream
    with torch.cuda.stream(st):
        for i in range(warmup):
            pre.input_ids.copy_(dev_ids[i % 3]); pre.replay()
    barrier()
    _lib.read_device_status(st.cuda_stream)

    # ---- timed region: K prefills, device timed ----
    from bench_mixer_core import ClockSampler
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(st):
        e0.record(st)
        for i in range(steps):
            pre.input_ids.copy_(dev_ids[i % 3], non_blocking=True); pre.replay()
        e1.record(st)
    barrier()
    ms_prefill = e0.elapsed_time(e1) / steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: pinned host token ids -> device -> prefill -> last-token logits in pinned host memory ----
    host_logits = torch.empty((batch, model.lm_head.out_features), dtype=torch.float16).pin_memory()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(st):
        e2.record(st)
        for i in range(steps):
            pre.input_ids.copy_(host_ids[i % 3], non_blocking=True)
            pre.replay()
            host_logits.copy_(pre.logits, non_blocking=True)
        e3.record(st)
    barrier()
    ms_e2e = e2.elapsed_time(e3) / steps

    # ---- decode: 256 greedy tokens from the prefill's caches, one CUDA graph per step ----
    params = pre.inference_params
    params.seqlen_offset = L
    dec = model.capture_decode(batch, L + ntok, inference_params=params)
    with torch.cuda.stream(st):
        dec.stream.wait_stream(st)
    with torch.cuda.stream(dec.stream):
        ops.greedy_next_token(pre.logits.contiguous(), out=dec.input_ids.view(-1))
        for _ in range(8):
            dec.replay()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dec.stream.synchronize()
    barrier()
    with torch.cuda.stream(dec.stream):
        d0.record(dec.stream)
        for _ in range(ntok):
            dec.replay()
        d1.record(dec.stream)
    barrier()
    tpot_ms = d0.elapsed_time(d1) / ntok
    _lib.read_device_status(dec.stream.cuda_stream)

    # ---- per entry point: CUDA events around every call of one eager prefill and one eager decode step ----
    pparams = type(params)(max_seqlen=L + 1, max_batch_size=batch, key_value_memory_dict=params.key_value_memory_dict)
    shares_p, eager_ms = trace_shares(lambda: model(dev_ids[0], inference_params=pparams, num_last_tokens=1), st)
    params.seqlen_offset = L
    tok = dec.input_ids.clone()
    shares_d, _ = trace_shares(lambda: model(tok, inference_params=params), st)
    ms_prefill, ms_e2e, tpot_ms = max_over_ranks([ms_prefill, ms_e2e, tpot_ms], device=dev)
    return dict(ms_prefill=ms_prefill, ms_e2e=ms_e2e, tpot_ms=tpot_ms, clocks=clocks, shares_p=shares_p, shares_d=shares_d,
                eager_ms=eager_ms, h2d=host_ids[0].numel() * 8, d2h=host_logits.numel() * 2, L=L, ntok=ntok)


def shares_table(agg):
    total = sum(ms for _, ms in agg.values()) or 1.0
    return {fn: {"calls": c, "ms": round(ms, 4), "share": round(ms / total, 4)} for fn, (c, ms) in
            sorted(agg.items(), key=lambda kv: -kv[1][1])}


def run_head_parallel(args, rank, local_rank, world, pk):
    """N >= 2 (or --model 8b): the head-parallel Mamba2-8B prefill, strong scaling, one all-reduce per layer."""
    import torch
    import bench_parallel as bp
    from quamba_b200 import _lib
    r = bp.run(args, rank, local_rank, world, layers=args.layers if args.layers != MODEL["n_layer"] else None)
    if rank != 0:
        return
    line = {
        "metric": "prefill_tok_per_s", "value": r["value"], "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": 3,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 (int4 weights, int8 activations, int32 accumulate; fp16 / fp32 scan and norm math)", "data": "synthetic",
        "config": {"workload": r["workload"] + ("" if r["layers"] == bp.CFG8B["n_layer"] else f" -- REDUCED to {r['layers']} layers (profiling case)"),
                   "weights": "int4 per output channel", "parallelism": f"head-parallel tp{world}: in_proj column-parallel by SSD group, "
                   "out_proj row-parallel, one exchange step per layer in chunks of sequences overlapped with compute: " + str(r["collective"]),
                   "l2": "131072 tokens per step: every activation tensor is far larger than the 126 MB L2",
                   "note": "at N = 1 bench.py reports the Mamba2-2.7B line (the metric's own configuration) and carries this workload's "
                           "single-GPU time in its head_parallel_8b key: that is the base of this strong-scaling curve"},
        "head_parallel_8b": r, "clocks": r.get("clocks"),
        "e2e": {"value": r["e2e_value"], "unit": "tok/s", "ms_per_step": r["e2e_ms_per_step"], "h2d_bytes_per_step": bp.BATCH * bp.PROMPT * 8,
                "d2h_bytes_per_step": bp.BATCH * bp.CFG8B["vocab_size"] * 2,
                "note": "every rank copies the token ids from pinned host memory and its last-token logits back to pinned host memory inside the timed region"},
        "gpu_launches": args.steps * r["layers"] * (bp.BATCH // r["chunk_sequences"]) * 8,
        "roofline": {"kernel": "gemm_s8_tcgen05 (in_proj + out_proj shards)", "bound": "tensor", "achieved": r["gemm_tops_per_gpu"], "peak": pk["i8"],
                     "unit": "TOP/s", "frac": r["gemm_tops_per_gpu"] / pk["i8"], "traffic": None, "peak_source": pk["i8_source"],
                     "note": "GEMM flops of the step per GPU over the compute-only step time (all kernels, no collective)"},
    }
    print(json.dumps(line), flush=True)


MAMBA1 = dict(d_model=2560, n_layer=64, vocab_size=50280, d_state=16, d_conv=4, expand=2)
WORKLOAD_MAMBA1 = ("configs[3]: Quamba Mamba1-2.8B W8A8 (d_model 2560, 64 layers, d_inner 5120, d_state 16, dt_rank 160, d_conv 4, "
                   "vocab 50280), batch 16, prefill 1024 token ids, then 128 greedy decode tokens")


def run_mamba1(args, dev, pk):
    """``--model mamba1``: the Mamba1-2.8B W8A8 model (int8 selective scan, Quamba1 conv1d, W8A8 linears, Hadamard), batch 16."""
    import torch
    from quamba_b200 import calibrate as cal
    layers = args.layers if args.layers != MODEL["n_layer"] else MAMBA1["n_layer"]
    fm = cal.Mamba1LMFloat(**dict(MAMBA1, n_layer=layers), seed=0, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    calib = [torch.randint(0, MAMBA1["vocab_size"], (1, 128), generator=g, device=dev) for _ in range(CALIB_SEQS)]
    model = cal.quantize_mamba1_model(fm, calib, w_bits=8)
    del fm
    torch.cuda.empty_cache()
    args.seqlen = 1024 if args.seqlen == PROMPT else args.seqlen
    args.decode_tokens = 128 if args.decode_tokens == DECODE_TOKENS else args.decode_tokens
    batch = 16
    r = measure(model, args, dev, 0, 1, -1, batch=batch, vocab=MAMBA1["vocab_size"])
    tokens = batch * r["L"]
    D, N, R_, d = MAMBA1["d_model"] * 2, MAMBA1["d_state"], 160, MAMBA1["d_model"]
    gemm_flops = layers * 2 * tokens * (d * 2 * D + D * (R_ + 2 * N) + R_ * D + D * d)
    scan_bytes = layers * (batch * D * r["L"] * 5 + 2 * batch * N * r["L"] + batch * D * N + D * (N + 2))
    sp = shares_table(r["shares_p"])
    line = {
        "metric": "prefill_tok_per_s", "value": tokens / (r["ms_prefill"] * 1e-3), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": r["ms_prefill"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 (int8 weights and activations, int32 accumulate; fp32 scan math)", "data": "synthetic",
        "config": {"workload": WORKLOAD_MAMBA1 if layers == MAMBA1["n_layer"] else f"REDUCED to {layers} layers: " + WORKLOAD_MAMBA1,
                   "l2": "every step streams all layers' int8 weights and 16 x 1024 tokens of activations: far beyond the 126 MB L2",
                   "graphs": "prefill and decode step replayed from CUDA graphs"},
        "decode": {"tpot_ms": r["tpot_ms"], "tokens": r["ntok"], "batch": batch, "tok_per_s": batch * 1e3 / r["tpot_ms"]},
        "e2e": {"value": tokens / (r["ms_e2e"] * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": args.steps * sum(v["calls"] for v in sp.values()),
        "roofline": {"shares_prefill": sp, "shares_decode_step": shares_table(r["shares_d"]),
                     "gemm_flops_per_step": gemm_flops, "gemm_tensor_bound_ms": gemm_flops / (pk["i8"] * 1e12) * 1e3,
                     "scan_algorithmic_bytes_per_step": scan_bytes, "scan_hbm_bound_ms": scan_bytes / (pk["hbm"] * 1e9) * 1e3},
        "eager_prefill_ms": r["eager_ms"], "clocks": r["clocks"],
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    if world > 1:
        # before the CUDA context exists: streams of one process on hardware queues of their own (a put queued behind another
        # stream's waiting kernel would keep a peer waiting in turn)
        os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        if args.comm_sms > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.comm_sms))
        # NCCL's kernels on a high-priority stream: their CTAs are placed ahead of the pending CTAs of the compute kernels, so
        # a collective starts as soon as SM slots free up instead of after the kernel that is draining
        opts = None
        if not os.environ.get("QB_NCCL_NORMAL_PRIORITY"):
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    pk = peaks()
    if world == 1 and args.model == "mamba1":
        run_mamba1(args, dev, pk)
        return
    if world > 1 or args.model == "8b":
        run_head_parallel(args, rank, local_rank, world, pk)
        if world > 1:
            dist.destroy_process_group()
        return
    model = build_model(dev, args.group_size, seed=rank, n_layer=args.layers)
    r = measure(model, args, dev, rank, world, args.group_size)
    extra = None
    if args.also_group128 and args.group_size != 128:
        del model
        torch.cuda.empty_cache()
        model = build_model(dev, 128, seed=rank, n_layer=args.layers)
        extra = measure(model, args, dev, rank, world, 128)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    m = dict(MODEL, n_layer=args.layers)
    flops, dbytes, gemm_flops_layer = model_flops_and_bytes(m, r["L"], args.group_size)
    tokens = r["L"] * world
    value = tokens / (r["ms_prefill"] * 1e-3)
    sp = shares_table(r["shares_p"])
    top = next(iter(sp))
    top_ms = sp[top]["ms"]
    if top in ("qb_w4a8_gemm", "qb_w8a8_gemm"):
        achieved = m["n_layer"] * gemm_flops_layer / (top_ms * 1e-3) / 1e12
        traffic, traffic_source = gemm_traffic()
        roof = {"kernel": "gemm_s8_tcgen05 (in_proj + out_proj of 64 layers)", "bound": "tensor", "achieved": achieved, "peak": pk["i8"],
                "unit": "TOP/s", "frac": achieved / pk["i8"], "traffic": traffic, "traffic_source": traffic_source, "peak_source": pk["i8_source"],
                "algorithmic_flops": m["n_layer"] * gemm_flops_layer, "ms": top_ms}
    else:
        roof = {"kernel": top, "bound": "hbm", "achieved": None, "peak": pk["hbm"], "unit": "GB/s", "frac": None, "traffic": None,
                "ms": top_ms}
    roof["shares_prefill"] = sp
    roof["shares_decode_step"] = shares_table(r["shares_d"])
    roof["model_tensor_bound_ms"] = flops / (pk["i8"] * 1e12) * 1e3
    reduced = args.layers != MODEL["n_layer"] or r["L"] != PROMPT
    line = {
        "metric": "prefill_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": r["ms_prefill"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 (int4 weights, int8 activations, int32 accumulate; fp16 / fp32 scan and norm math)", "data": "synthetic",
        "config": {"workload": WORKLOAD if not reduced else f"REDUCED (profiling case): {args.layers} layers, prompt {r['L']}; " + WORKLOAD,
                   "weights": "int4 per output channel" if args.group_size < 0 else "int4 group 128",
                   "l2": "every step streams 64 layers' weights (2.6 GB of int8 expansions) and rotates among 3 prompts: far beyond the 126 MB L2",
                   "sharding": "one prompt per GPU, no collective (replicas)" if world > 1 else "single GPU",
                   "graphs": "prefill and decode step replayed from CUDA graphs"},
        "decode": {"tpot_ms": r["tpot_ms"], "tokens": r["ntok"], "tok_per_s": world * 1e3 / r["tpot_ms"],
                   "hbm_bytes_per_token": dbytes, "hbm_bound_ms": dbytes / (pk["hbm"] * 1e9) * 1e3,
                   "frac_of_hbm_bound": dbytes / (pk["hbm"] * 1e9) * 1e3 / r["tpot_ms"]},
        "e2e": {"value": tokens / (r["ms_e2e"] * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": args.steps * sum(c + (c if fn == "qb_ssd_chunk_scan_fwd" else 0) for fn, (c, _) in r["shares_p"].items()),
        "roofline": roof, "eager_prefill_ms": r["eager_ms"], "clocks": r["clocks"],
    }
    if extra is not None:
        line["group128"] = {"value": tokens / (extra["ms_prefill"] * 1e-3), "unit": "tok/s", "tpot_ms": extra["tpot_ms"],
                            "e2e": tokens / (extra["ms_e2e"] * 1e-3), "shares_decode_step": shares_table(extra["shares_d"])}
    if world == 1 and not args.no_8b_base:
        # the single-GPU base of the head-parallel strong-scaling curve that bench.py --gpus N (N >= 2) reports
        try:
            del model
            torch.cuda.empty_cache()
            import bench_parallel as bp
            base_args = argparse.Namespace(steps=max(2, min(args.steps, 4)), warmup=1)
            line["head_parallel_8b"] = bp.run(base_args, 0, local_rank, 1)
        except Exception as e:      # never lose the main line to the extra measurement
            line["head_parallel_8b"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if world == 1 and not args.no_cpu_baseline:
        tok_s, t_full, sample = cpu_sample()
        line["cpu_baseline"] = {"value": tok_s, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--op", default=None, help="'mixer_core' (conv1d + SSD op-level line) or one kernel of bench_ops.OPS / 'all'")
    ap.add_argument("--batch", type=int, default=0, help="--op mixer_core only: sequences per GPU (reduced profiling case)")
    ap.add_argument("--group-size", type=int, default=-1, choices=[-1, 128], help="int4 weight format: per output channel or group 128")
    ap.add_argument("--also-group128", action="store_true", help="measure the group-128 weight format too (second model build)")
    ap.add_argument("--layers", type=int, default=MODEL["n_layer"], help="fewer layers = a reduced profiling case, flagged in config")
    ap.add_argument("--model", default="2.7b", choices=["2.7b", "8b", "mamba1"],
                    help="8b: the head-parallel Mamba2-8B prefill (always used for --gpus >= 2); mamba1: the Mamba1-2.8B W8A8 model, batch 16")
    ap.add_argument("--no-8b-base", action="store_true", help="skip the single-GPU Mamba2-8B measurement added to the 2.7B line")
    ap.add_argument("--comm-sms", type=int, default=16, help="--gpus >= 2: multiprocessors left to NCCL (compute grids use the rest); 0 = no split")
    ap.add_argument("--plain-allreduce", action="store_true", help="--gpus >= 2: one fp16 all-reduce per layer and a replicated block norm "
                    "instead of reduce-scatter + token-sharded norm + int8 all-gather")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="--gpus >= 2: who moves the bytes of the token-sharded layer exchange: NCCL reduce-scatter / all-gather kernels, or "
                    "copy-engine puts into peer memory with flags and bounded waits (quamba_b200/peer.py)")
    ap.add_argument("--peer-lag", type=int, default=0, help="--exchange peer: shard tasks of other chunks between a partial output and the "
                    "norm that consumes it (0: half the number of chunks)")
    ap.add_argument("--chunk-seqs", type=int, default=0, help="head-parallel prefill: sequences per chunk (0: 8 on several GPUs, 4 on one)")
    ap.add_argument("--seqlen", type=int, default=PROMPT)
    ap.add_argument("--decode-tokens", type=int, default=DECODE_TOKENS)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.op == "mixer_core":
        import bench_mixer_core
        bench_mixer_core.run(args)
    elif args.op is not None:
        import bench_ops
        for line in bench_ops.run(args.op, args.steps, args.warmup):
            print(json.dumps(line), flush=True)
    elif args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
