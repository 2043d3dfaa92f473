"""Head-parallel Mamba2-8B prefill behind ``bench.py --gpus N`` (N >= 2) and ``bench.py --model 8b``.

Workload (strong scaling: the same job on 1, 2, 4 or 8 GPUs): Quamba2 Mamba2-8B W4A8 geometry -- d_model 4096, 56 layers,
expand 2 (128 heads x 64), ngroups 8, d_state 128, d_conv 4, vocab 256000, random-init weights N(0, 0.02) quantized to
int4 per output channel, int8 activations with static scales calibrated on 4 random sequences -- batch 32, prefill of
4096 uniform-random token ids.  Every rank holds all token rows and 1/T of every layer's heads (in_proj column-parallel by
SSD group, conv / SSD / gated norm local, block-diagonal Hadamard, out_proj row-parallel); the only exchange is the sum of
the (tokens, 4096) fp16 layer output per layer, issued per chunk of sequences so that the transfer of one chunk overlaps
the compute of the next: by default as partial sums sent to the owners of their token rows, a block norm on those rows and
int8 rows sent to everybody, moved by copy engines into peer memory (``--exchange peer``) or by NCCL's reduce-scatter and
all-gather (``--exchange nccl``); ``--plain-allreduce`` is one NCCL all-reduce per layer with a replicated block norm.

The model is built layer by layer (float layer -> calibration taps on the running calibration batch -> quantise -> cut
this rank's shard -> drop the rest), identically on every rank from one seed.
"""
import time

import torch
import torch.distributed as dist

CFG8B = dict(d_model=4096, n_layer=56, vocab_size=256000, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=8, chunk_size=256)
BATCH, PROMPT, HAD_BLOCKS = 32, 4096, 8
COMM_SMS = 16      # multiprocessors left to NCCL while the all-reduce of one chunk overlaps the compute of the next
WORKLOAD8B = ("configs[4]: Quamba2 Mamba2-8B W4A8 (d_model 4096, 56 layers, 128 heads x 64, ngroups 8, d_state 128, vocab 256000), "
              "head-parallel, batch 32, prefill 4096 token ids")


class Stack:
    """This rank's share of the model: replicated embedding / norms / head, sharded mixers."""

    def __init__(self, cfg, rank, world, dev, seed=0, calib_len=512, calib_seqs=4):
        from quamba_b200 import calibrate as cal
        from quamba_b200.embedding import F16Embedding
        from quamba_b200.mixer import W4A8QMamba2
        from quamba_b200.modules import W4A8B16O16Linear
        from quamba_b200.norm import QRMSNorm
        from quamba_b200.parallel import shard_mixer
        self.cfg, self.rank, self.world, self.dev = cfg, rank, world, dev
        gen = torch.Generator(device=dev).manual_seed(seed)
        d, V = cfg["d_model"], cfg["vocab_size"]
        table = (torch.randn(V, d, generator=gen, device=dev) * 0.02).half()
        self.embedding = F16Embedding(V, d, device=dev)
        self.embedding.weight.data = table
        ids = torch.randint(0, V, (calib_seqs, calib_len), generator=gen, device=dev)
        h = table[ids]
        residual = torch.zeros_like(h, dtype=torch.float32)
        self.norms, self.shards = [], []
        ssm = {k: cfg[k] for k in ("d_state", "d_conv", "expand", "headdim", "ngroups", "chunk_size")}
        for i in range(cfg["n_layer"]):
            fl = cal.Mamba2Float(d, layer_idx=i, w4_group_size=-1, had_blocks=HAD_BLOCKS, generator=gen, device=dev, **ssm).half()
            norm = cal.RMSNormFloat(d).to(dev)
            taps = {}
            residual = residual + h.float()
            with torch.no_grad():
                h = fl(norm(residual).half(), taps)
            s = {k: (v / 127.0).clamp(min=1e-8).float().reshape(1) for k, v in taps.items()}
            sc = {"in_proj:input": s["in_proj:input"], "out_proj:input": s["out_proj:input"], "ssm_state_act:input": s["ssm_state_act"]}
            for name in ("x_conv_in", "B_conv_in", "C_conv_in", "x_conv_out", "B_conv_out", "C_conv_out", "dt_act", "z_act"):
                sc[name + ":input"] = sc[name + ":output"] = s[name]
            full = W4A8QMamba2.from_fp16(fl, sc)
            self.norms.append(QRMSNorm.from_fp16(norm, output_scale=sc["in_proj:input"].item()))
            self.shards.append(shard_mixer(full, rank, world))
            del fl, full
        residual = residual + h.float()
        norm_f = cal.RMSNormFloat(d).to(dev)
        head_scale = (norm_f(residual[:, -1:]).abs().amax() / 127.0).clamp(min=1e-8).float().reshape(1)
        self.norm_f = QRMSNorm.from_fp16(norm_f, output_scale=head_scale.item())
        head = torch.nn.Linear(d, V, bias=False, device=dev, dtype=torch.float16)
        head.weight.data = (torch.randn(V, d, generator=gen, device=dev) * 0.02).half()
        head.w4_group_size = -1
        self.lm_head = W4A8B16O16Linear.from_fp16(head, head_scale)
        del head, table
        torch.cuda.empty_cache()

    def runner(self):
        from quamba_b200.parallel import HeadParallelStack
        return HeadParallelStack(self.embedding, self.norms, self.shards, self.norm_f, self.lm_head, self.rank, self.world,
                                 self.cfg["d_model"])


def run(args, rank, local_rank, world, layers=None):
    """Times the head-parallel prefill; returns the result dict on rank 0 (None elsewhere)."""
    from quamba_b200 import _lib
    from quamba_b200.sharding import max_over_ranks
    dev = torch.device("cuda", local_rank)
    cfg = dict(CFG8B, n_layer=layers or CFG8B["n_layer"])
    t0 = time.time()
    stack = Stack(cfg, rank, world, dev).runner()
    stack.token_sharded_norm = not getattr(args, "plain_allreduce", False)
    stack.exchange = getattr(args, "exchange", "peer") if world > 1 and stack.token_sharded_norm else "nccl"
    chunk_seqs = getattr(args, "chunk_seqs", 0) or (8 if world > 1 else 4)
    stack.peer_lag = getattr(args, "peer_lag", 0) or None
    fallback = None
    if stack.exchange == "peer":
        # map the peers' memory now; if any rank cannot (no IPC between the processes, say), every rank takes the NCCL exchange
        try:
            stack._peer_exchange(chunk_seqs * PROMPT, BATCH // chunk_seqs)
            mine_ok, why = 1, ""
        except Exception as e:  # noqa: BLE001 - whatever the set-up raised is the reason reported
            mine_ok, why = 0, f"{type(e).__name__}: {e}"
        ok = torch.tensor([mine_ok], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            reasons = [None] * world
            dist.all_gather_object(reasons, why)
            fallback = next((r for r in reasons if r), "a peer failed")[:300]
            stack.exchange = "nccl"
    peer = stack.exchange == "peer"
    import os
    stack.early_overlap = not os.environ.get("QB_NO_EARLY_OVERLAP")
    build_s = time.time() - t0
    g = torch.Generator().manual_seed(99)
    ids = [torch.randint(0, cfg["vocab_size"], (BATCH, PROMPT), generator=g).to(dev) for _ in range(2)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(steps, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(steps):
            stack.prefill(ids[i % 2], chunk_seqs, **kw)
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / steps

    def timed_e2e(steps):
        """The same step from pinned host token ids to last-token logits in pinned host memory, both copies inside the
        timed region."""
        host_ids = [i.cpu().pin_memory() for i in ids]
        dev_ids = torch.empty_like(ids[0])
        host_logits = torch.empty((BATCH, cfg["vocab_size"]), dtype=torch.float16).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(steps):
            dev_ids.copy_(host_ids[i % 2], non_blocking=True)
            out = stack.prefill(dev_ids, chunk_seqs)
            host_logits.copy_(out, non_blocking=True)
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / steps

    # Room for the collective: the compute kernels are persistent (one CTA per SM), so with the whole GPU taken NCCL's CTAs
    # get an SM only when a kernel ends, and once they are in, the next persistent grid runs in two waves.  The library
    # sizes its grids for all but COMM_SMS multiprocessors and NCCL is capped at as many CTAs (NCCL_MAX_CTAS, set by
    # bench.py before the process group exists).
    comm_sms = getattr(args, "comm_sms", COMM_SMS) if world > 1 and not peer else 0   # copy engines need no multiprocessor
    sm_total = torch.cuda.get_device_properties(dev).multi_processor_count
    _lib.set_sm_budget(sm_total - comm_sms if comm_sms > 0 else 0)
    steps = max(1, args.steps)
    for _ in range(max(3, min(args.warmup, 3))):
        logits = stack.prefill(ids[0], chunk_seqs)
    barrier()
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
    # the two forms of the layer's collective compute the same sums: compare their last-token logits once, outside the timing
    form_diff = peer_diff = None
    if world > 1 and stack.token_sharded_norm:
        with _lib.early_overlap(stack.early_overlap), torch.no_grad():
            other = stack._prefill_allreduce(ids[0], chunk_seqs)
            via_nccl = stack._prefill_token_sharded(ids[0], chunk_seqs) if peer else None
        torch.cuda.synchronize()
        if via_nccl is not None:      # the same exchange through NCCL's reduce-scatter / all-gather
            peer_diff = {"max_abs_diff": (logits.float() - via_nccl.float()).abs().max().item(),
                         "same_argmax": bool((logits.argmax(-1) == via_nccl.argmax(-1)).all().item())}
            del via_nccl
        form_diff = {"max_abs_diff": (logits.float() - other.float()).abs().max().item(), "max_abs_logit": other.float().abs().max().item(),
                     "same_argmax": bool((logits.argmax(-1) == other.argmax(-1)).all().item())}
        del other
    barrier()
    from bench_mixer_core import ClockSampler
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    ms_step = timed(steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_compute = timed(max(1, steps // 2), collective=False)
    ms_comm = timed(max(1, steps // 2), compute=False) if world > 1 else 0.0
    ms_e2e = timed_e2e(max(1, steps // 2))
    ms_step, ms_compute, ms_comm, ms_e2e = max_over_ranks([ms_step, ms_compute, ms_comm, ms_e2e], device=dev)
    _lib.read_device_status(torch.cuda.current_stream().cuda_stream)     # a wait that gave up would have left its code here
    barrier()
    stack.close()
    if rank != 0:
        return None
    tokens = BATCH * PROMPT
    D, G, N, H = cfg["d_model"] * cfg["expand"], cfg["ngroups"], cfg["d_state"], cfg["d_model"] * cfg["expand"] // cfg["headdim"]
    flops = cfg["n_layer"] * 2 * tokens * cfg["d_model"] * (2 * D + 2 * G * N + H + D)
    reduce_bytes = cfg["n_layer"] * tokens * cfg["d_model"] * 2
    link_factor = ((world - 1) / world * 1.5 if stack.token_sharded_norm else 2 * (world - 1) / world) if world > 1 else 0.0
    return {"value": tokens / (ms_step * 1e-3), "unit": "tok/s", "ms_per_step": ms_step, "compute_only_ms": ms_compute,
            "e2e_ms_per_step": ms_e2e, "e2e_value": tokens / (ms_e2e * 1e-3),
            "allreduce_alone_ms": ms_comm, "allreduce_exposed_ms": max(0.0, ms_step - ms_compute) if world > 1 else 0.0,
            "allreduce_share_of_step": max(0.0, ms_step - ms_compute) / ms_step if world > 1 else 0.0,
            "allreduce_bytes_per_step": reduce_bytes if world > 1 else 0,
            # bytes every rank sends (= receives) per step over NVLink, and the rate when the collectives run alone:
            # all-reduce 2 (T-1)/T x 2 B per element; reduce-scatter + int8 all-gather (T-1)/T x (2 + 1) B
            "nvlink_bytes_per_rank_per_step": int(link_factor * reduce_bytes) if world > 1 else 0,
            "allreduce_bus_gbs": (link_factor * reduce_bytes / (ms_comm * 1e-3) / 1e9) if world > 1 and ms_comm > 0 else None,
            "gemm_flops_per_step": flops, "gemm_tops_per_gpu": flops / world / (ms_compute * 1e-3) / 1e12,
            "chunk_sequences": chunk_seqs, "layers": cfg["n_layer"], "build_seconds": build_s, "workload": WORKLOAD8B,
            "clocks": clocks, "compute_sms": sm_total - comm_sms, "nccl_max_ctas": comm_sms if world > 1 else None,
            "token_sharded_vs_allreduce_logits": form_diff, "peer_exchange_vs_nccl_logits": peer_diff, "exchange": stack.exchange, "exchange_fallback": fallback,
            # the same seed builds the same model on any number of GPUs: these must agree between N = 1 and N > 1
            "logits_digest": {"argmax": logits.argmax(-1).tolist(), "row0_first8": [round(v, 4) for v in logits[0, :8].float().tolist()],
                              "abs_sum": round(logits.float().abs().sum().item(), 2)},
            "collective": (("copy-engine puts into peer memory (fp16 partial sums by owner, int8 rows to all), flags, bounded waits; the "
                            "token-sharded block norm sums the received pieces itself") if peer else
                           "reduce-scatter (fp16) + all-gather (int8) around a token-sharded block norm" if stack.token_sharded_norm
                           else "all-reduce (fp16)") if world > 1 else None,
            "limiting": ("the per-layer exchange of the (tokens, 4096) layer output over NVLink: fp16 partial sums to the owners of their token rows, "
                         "int8 rows to every rank (at eight ranks the exchange alone takes longer than the compute alone)") if world > 1 else "compute"}
