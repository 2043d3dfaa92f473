"""Op-level benchmark of the Mamba2 mixer core (conv1d + SSD chunk scan), reached as ``bench.py --op mixer_core``.

    python bench.py --op mixer_core [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the hot path over one batch of synthetic input:
int8 causal conv1d over xBC (+SiLU, requant, x/B/C split) followed by the int8 SSD chunk scan with
inter-chunk state passing, at the op configuration B4 L2048 H80 P64 G1 N128 Q256 W4 (the conv + SSD
shapes of one Mamba2-2.7B layer at batch 4).  Prints ONE JSON line (see the keys below).

  value     tokens/s with inputs resident in HBM (device-timed, CUDA events around CUDA-graph replays of the step, max over ranks)
  e2e       the same through the public ops API with pinned HOST buffers: H2D of the int8 inputs and
            D2H of y + final states inside the timed region
  roofline  SSD forward (the dominant part): algorithmic bytes / its CUDA-event time vs measured HBM peak
  cpu_baseline  the CPU oracle (torch fp32, all host threads) on a bounded sample, rank 0, N = 1 only
  --impl reference  times that CPU path alone (the reference has no CPU implementation of its own and
            its CUDA/Triton extensions cannot be installed offline; the oracle restates them)
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

CFG = dict(B=4, L=2048, H=80, P=64, G=1, N=128, Q=256, W=4)
WORKLOAD = ("configs[1]: Mamba2 int8 causal_conv1d + SSD chunk scan, batch 4, seqlen 2048, nheads 80, headdim 64, "
            "ngroups 1, d_state 128, chunk 256, d_conv 4")


def ssd_traffic(batch_rows):
    """dram__bytes_read.sum + dram__bytes_write.sum of one ssd_tc_kernel launch, from the committed summary of an ncu pass
    over this very benchmark (it grows with the number of (batch, head) pairs, hence scaled by batch rows).  Returns
    (bytes, source) or (None, None) when the summary file is absent."""
    import json
    from pathlib import Path
    f = Path(__file__).resolve().parent / "profiles" / "mixer_core_cfg2_traffic.json"
    if not f.exists():
        return None, None
    t = json.loads(f.read_text())
    per_row = (t["dram_bytes_read_per_launch"] + t["dram_bytes_write_per_launch"]) / t["batch_rows"]
    return per_row * batch_rows, f"{t['source']} (captured {t['captured']})"


def algorithmic_bytes():
    B, L, H, P, G, N, W = (CFG[k] for k in "BLHPGNW")
    C = H * P + 2 * G * N
    conv = 2 * B * C * L + C * (W + 1)
    ssd = B * L * (H * P + H + 2 * G * N) + 2 * B * L * H * P + B * H * P * N
    return conv, ssd


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(seed, B=None):
    from helpers import make_conv2_case, make_ssd_case
    B = B or CFG["B"]
    conv = make_conv2_case(B, CFG["L"], CFG["H"], CFG["P"], CFG["G"], CFG["N"], W=CFG["W"], seed=seed)
    ssd = make_ssd_case(B, CFG["L"], CFG["H"], CFG["P"], CFG["G"], CFG["N"], CFG["Q"], seed=seed + 100)
    return conv, ssd


def cpu_step(conv, ssd):
    """The CPU oracle's pass over one batch (dequantise -> fp32 torch)."""
    import torch
    from oracle import conv1d as oconv, ssd as ossd
    c = conv
    x, Bm, Cm = oconv.quamba2_conv1d_fwd(c["xBC"], c["sx"], c["sB"], c["sC"], c["x_dim"], CFG["P"], CFG["N"], CFG["G"], None, None,
                                         c["x_scales"], c["B_scales"], c["C_scales"], c["weight"], c["swx"], c["swB"], c["swC"],
                                         c["bias"], c["sbx"], c["sbB"], c["sbC"])
    Bsz, L = x.shape[0], x.shape[2]
    qx = x.transpose(1, 2).reshape(Bsz, L, CFG["H"], CFG["P"])
    qB = Bm.transpose(1, 2).reshape(Bsz, L, CFG["G"], CFG["N"])
    qC = Cm.transpose(1, 2).reshape(Bsz, L, CFG["G"], CFG["N"])
    s = ssd
    return ossd.chunk_scan_faithful(qx, c["x_scales"], None, None, s["q_dt"], s["s_dt"], s["q_A_log"], s["s_A"], qB, c["B_scales"], qC,
                                    c["C_scales"], s["state_scale"], CFG["Q"], s["q_D"], s["s_D"], None, None, s["dt_bias"], True)


def time_cpu(steps, warmup):
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    conv, ssd = make_inputs(0, B=1)  # bounded sample: one of the four sequences
    for _ in range(warmup):
        cpu_step(conv, ssd)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(conv, ssd)
    dt = (time.perf_counter() - t0) / steps
    return CFG["L"] / dt, dt, "1 of the 4 sequences (batch 1, seqlen 2048, all 80 heads)"


def run_reference(args, rank, world):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    tok_s, dt, sample = time_cpu(steps, min(args.warmup, 1))
    cores = os.cpu_count() or 1
    line = {"impl": "reference", "metric": "prefill_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
            "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run(args):
    """``args``: the namespace bench.py parsed (gpus, steps, warmup, impl, no_cpu_baseline, batch)."""
    global WORKLOAD
    if args.batch and args.batch != CFG["B"]:
        WORKLOAD = WORKLOAD.replace("batch 4", f"batch {args.batch} (REDUCED from 4: profiling case)")
        CFG["B"] = args.batch
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from quamba_b200 import ops, _lib
    from quamba_b200.sharding import max_over_ranks

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    steps = args.steps
    to = lambda t: None if t is None else t.to(dev)

    # ---- inputs: NSETS rotating sets so that consecutive steps never re-read L2-resident data ----
    NSETS = 3
    sets = []
    for i in range(NSETS):
        conv, ssd = make_inputs(1000 * rank + i)
        C = conv["xBC"].shape[1]
        host_xBC = conv["xBC"].transpose(1, 2).contiguous().pin_memory()       # (B, L, C) int8
        host_dt = ssd["q_dt"].contiguous().pin_memory()
        d = dict(conv=conv, ssd=ssd, host_xBC=host_xBC, host_dt=host_dt, xBC=host_xBC.to(dev).transpose(1, 2), q_dt=host_dt.to(dev),
                 weight=to(conv["weight"]), bias=to(conv["bias"]), x_scales=to(conv["x_scales"]), B_scales=to(conv["B_scales"]),
                 C_scales=to(conv["C_scales"]), s_dt=to(ssd["s_dt"]), q_A=to(ssd["q_A_log"]), s_A=to(ssd["s_A"]), q_D=to(ssd["q_D"]),
                 s_D=to(ssd["s_D"]), dt_bias=to(ssd["dt_bias"]), state_scale=to(ssd["state_scale"]))
        sets.append(d)
    B, L, H, P, G, N, Q = (CFG[k] for k in "BLHPGNQ")

    def conv_call(d, xBC):
        c = d["conv"]
        return ops.quamba2_conv1d_cuda.fwd(xBC, c["sx"], c["sB"], c["sC"], c["x_dim"], P, N, G, None, None, d["x_scales"], d["B_scales"],
                                           d["C_scales"], d["weight"], c["swx"], c["swB"], c["swC"], d["bias"], c["sbx"], c["sbB"],
                                           c["sbC"], None, None, None, True)

    def ssd_call(d, x, Bm, Cm, q_dt):
        qx = x.transpose(1, 2).reshape(B, L, H, P)
        qB = Bm.transpose(1, 2).reshape(B, L, G, N)
        qC = Cm.transpose(1, 2).reshape(B, L, G, N)
        return ops._quant_mamba_chunk_scan_combined_fwd(qx, d["x_scales"], q_dt, d["s_dt"], d["q_A"], d["s_A"], qB, d["B_scales"], qC,
                                                        d["C_scales"], d["state_scale"], Q, d["q_D"], d["s_D"], None, None, d["dt_bias"],
                                                        None, None, None, True)

    def step(d):
        x, Bm, Cm = conv_call(d, d["xBC"])
        return ssd_call(d, x, Bm, Cm, d["q_dt"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Everything below runs on one side stream (CUDA-graph capture needs a non-default stream).
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    for i in range(warmup):
        step(sets[i % NSETS])
    barrier()
    _lib.read_device_status(stream.cuda_stream)

    # ---- CUDA graphs: the step, and its two parts, captured once per input set so that the timed region
    # contains only device work (the Python/ctypes marshalling of each call is tens of microseconds) ----
    graphs, conv_graphs, ssd_graphs, keep = [], [], [], []
    for d in sets:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            keep.append(step(d))
        graphs.append(g)
        gc = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gc, stream=stream):
            xbc = conv_call(d, d["xBC"])
        conv_graphs.append(gc)
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs, stream=stream):
            keep.append(ssd_call(d, xbc[0], xbc[1], xbc[2], d["q_dt"]))
        ssd_graphs.append(gs)
        keep.append(xbc)
    for i in range(warmup):
        graphs[i % NSETS].replay()
    barrier()

    # ---- timed region: whole step, device timed ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for i in range(steps):
        graphs[i % NSETS].replay()
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-part timings for the roofline (same stream, CUDA events around K replays of each part) ----
    def time_graphs(gl):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(3):
            gl[i % NSETS].replay()
        a.record(stream)
        for i in range(steps):
            gl[i % NSETS].replay()
        b_.record(stream)
        b_.synchronize()
        return a.elapsed_time(b_) / steps
    conv_ms = time_graphs(conv_graphs)
    ssd_ms = time_graphs(ssd_graphs)

    # ---- end to end: pinned host inputs -> device -> hot path -> host outputs ----
    # Every step copies its own inputs from pinned host memory and its own outputs back; the three stages (H2D, the two
    # ops, D2H) run on three streams over two sets of buffers, so that the copies of neighbouring steps overlap with the
    # kernels and with each other (PCIe is full duplex).  The timed region ends when the last output has reached the host.
    NBUF = 2
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    slots = []
    for _ in range(NBUF):
        slots.append({
            "host_y": torch.empty((B, L, H, P), dtype=torch.float16).pin_memory(),
            "host_f": torch.empty((B, H, P, N), dtype=torch.int8).pin_memory(),
            "dxBC": torch.empty_like(sets[0]["host_xBC"], device=dev), "ddt": torch.empty_like(sets[0]["host_dt"], device=dev),
            "ev_in": torch.cuda.Event(), "ev_done": torch.cuda.Event(), "ev_out": torch.cuda.Event(), "y": None, "f": None})
    host_y, host_f = slots[0]["host_y"], slots[0]["host_f"]

    def e2e_run(n):
        for i in range(n):
            d, sl = sets[i % NSETS], slots[i % NBUF]
            with torch.cuda.stream(s_in):
                if i >= NBUF:
                    s_in.wait_event(sl["ev_done"])          # the kernels of step i - NBUF have read these input buffers
                sl["dxBC"].copy_(d["host_xBC"], non_blocking=True)
                sl["ddt"].copy_(d["host_dt"], non_blocking=True)
                sl["ev_in"].record(s_in)
            with torch.cuda.stream(stream):
                stream.wait_event(sl["ev_in"])
                if i >= NBUF:
                    stream.wait_event(sl["ev_out"])         # the outputs of step i - NBUF have left the device
                x, Bm, Cm = conv_call(d, sl["dxBC"].transpose(1, 2))
                sl["y"], sl["f"] = ssd_call(d, x, Bm, Cm, sl["ddt"])
                sl["ev_done"].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(sl["ev_done"])
                sl["host_y"].copy_(sl["y"], non_blocking=True)
                sl["host_f"].copy_(sl["f"], non_blocking=True)
                sl["ev_out"].record(s_out)
        for sl in slots[:min(n, NBUF)]:
            stream.wait_event(sl["ev_out"])

    with torch.cuda.stream(stream):
        e2e_run(2)
    torch.cuda.synchronize()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e2.record(stream)
        e2e_run(steps)
        e3.record(stream)
    torch.cuda.synchronize()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    _lib.read_device_status(stream.cuda_stream)

    ms_total, ms_e2e, conv_ms, ssd_ms = max_over_ranks([ms_total, ms_e2e, conv_ms, ssd_ms], device=dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    tokens = B * L * world
    ms_step = ms_total / steps
    value = tokens / (ms_step * 1e-3)
    e2e_val = tokens / (ms_e2e / steps * 1e-3)
    conv_bytes, ssd_bytes = algorithmic_bytes()
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    tensor_peak = float(peaks.get("bf16_tflops", 1590.0))
    ssd_flops = float(B * H * ((L + 127) // 128) * (2 * 128 * 128 * 128 + 3 * 2 * 128 * 64 * 128))
    ssd_gbs = ssd_bytes / (ssd_ms * 1e-3) / 1e9
    conv_gbs = conv_bytes / (conv_ms * 1e-3) / 1e9
    line = {
        "metric": "prefill_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 in / fp16+fp32 math",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": f"{NSETS} rotating input sets; per-step footprint exceeds the 126 MB L2",
                   "sharding": "independent batches per GPU, no collective on this path",
                   "e2e_pipeline": "H2D, kernels and D2H of neighbouring steps overlap (three streams, two buffer sets)"},
        "e2e": {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": int(sets[0]["host_xBC"].numel() + sets[0]["host_dt"].numel()),
                "d2h_bytes_per_step": int(host_y.numel() * 2 + host_f.numel())},
        "gpu_launches": 3 * steps,
        "roofline": {"kernel": "ssd_tc_kernel (+ ssd_prep_kernel)", "bound": "hbm", "achieved": ssd_gbs, "peak": hbm_peak, "unit": "GB/s",
                     "frac": ssd_gbs / hbm_peak, "traffic": ssd_traffic(B)[0], "traffic_source": ssd_traffic(B)[1], "peak_source": "measured" if peaks else "fallback",
                     "algorithmic_bytes": ssd_bytes, "ms": ssd_ms,
                     # the same kernel against the tensor roofline (the op is balanced between the two): dense fp16 MMA
                     # flops it issues per 128-token block (C.B^T 128x128x128 + three 128x64x128) over the measured bf16 peak
                     "tensor": {"flops": ssd_flops, "achieved_tflops": ssd_flops / (ssd_ms * 1e-3) / 1e12,
                                "peak_tflops": tensor_peak, "frac": ssd_flops / (ssd_ms * 1e-3) / 1e12 / tensor_peak},
                     "conv1d": {"achieved": conv_gbs, "frac": conv_gbs / hbm_peak, "algorithmic_bytes": conv_bytes, "ms": conv_ms}},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        tok_s, dt, sample = time_cpu(1, 1)
        line["cpu_baseline"] = {"value": tok_s, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()

