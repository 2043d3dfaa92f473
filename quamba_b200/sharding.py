"""Sharding of the mixer hot path over the GPUs of one node.

The path has no exchange step: every (batch, head) unit of the conv1d -> SSD chunk scan is independent of the
others (B and C are shared by the heads of one SSD group, read-only).  So the units are dealt out to the ranks,
each rank runs the same kernels on its share, and the only communication is control-plane: a barrier around the
timed region and a MAX reduction of the device times.  Two ways of cutting are provided:

  * by sequence (batch dimension) - what ``bench.py --gpus N`` does ("weak" scaling, each rank has its own batch);
  * by head - for one batch spread over the ranks: x / dt / A_log / D / dt_bias are cut along heads, B and C
    along SSD groups when there are at least as many groups as ranks, else replicated.

Everything here is host logic on torch tensors and ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous balanced split of ``n_units``: the first ``n_units % world`` ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of size {world}")
    if n_units < 0:
        raise ValueError("n_units must be non-negative")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_sequences(tensors: Dict[str, Optional[torch.Tensor]], rank: int, world: int,
                    batched: Sequence[str]) -> Dict[str, Optional[torch.Tensor]]:
    """Cut the tensors named in ``batched`` along dim 0 (sequences); the others (weights, scales) are replicated."""
    out = dict(tensors)
    for name in batched:
        t = tensors.get(name)
        if t is not None:
            lo, hi = shard_range(t.shape[0], rank, world)
            out[name] = t[lo:hi]
    return out


def shard_ssd_heads(case: Dict[str, Optional[torch.Tensor]], rank: int, world: int) -> Dict[str, Optional[torch.Tensor]]:
    """Cut an SSD chunk-scan problem along heads.  ``case`` uses the argument names of the chunk-scan entry point:
    q_x (b, l, h, p), q_dt (b, l, h), q_A_log (h), q_D (h) or (h, p), dt_bias (h), q_z like q_x, q_B / q_C (b, l, g, n).
    Only per-tensor x / state scales are supported (grouped scale tables are indexed by absolute head and would
    have to be re-based); the heads per rank must be a multiple of the heads per SSD group, or a divisor of it."""
    if case.get("hgr") is not None or case.get("dgr") is not None:
        raise NotImplementedError("head sharding with head/dim-grouped scales is not supported")
    H = case["q_x"].shape[2]
    G = case["q_B"].shape[2]
    if H % world:
        raise ValueError(f"nheads = {H} is not divisible by the world size {world}")
    hpr, hpg = H // world, H // G
    lo, hi = rank * hpr, (rank + 1) * hpr
    out = dict(case)
    out["q_x"] = case["q_x"][:, :, lo:hi]
    out["q_dt"] = case["q_dt"][:, :, lo:hi]
    for name in ("q_A_log", "q_D", "dt_bias"):
        if case.get(name) is not None:
            out[name] = case[name][lo:hi]
    if case.get("q_z") is not None:
        out["q_z"] = case["q_z"][:, :, lo:hi]
    if hpr % hpg == 0:                                   # whole groups per rank
        g0, g1 = lo // hpg, hi // hpg
    elif hpg % hpr == 0:                                 # a rank sits inside one group
        g0, g1 = lo // hpg, lo // hpg + 1
    else:
        raise ValueError("heads per rank and heads per SSD group must divide one another")
    out["q_B"] = case["q_B"][:, :, g0:g1]
    out["q_C"] = case["q_C"][:, :, g0:g1]
    for name in ("s_B", "s_C"):
        s = case.get(name)
        if torch.is_tensor(s) and s.numel() == G and G > 1:
            out[name] = s.reshape(-1)[g0:g1]
    return out


def max_over_ranks(values: Sequence[float], device=None) -> list:
    """MAX of each value over all ranks (identity without an initialised process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return [float(v) for v in values]
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def gather_heads(y_local: torch.Tensor, world: int, dim: int = 2) -> torch.Tensor:
    """All-gather of equally sized head shards (used by tests and by callers that want the full y on every rank;
    the mixer itself feeds y into a row-parallel projection and never needs this)."""
    if world == 1:
        return y_local
    parts = [torch.empty_like(y_local) for _ in range(world)]
    dist.all_gather(parts, y_local.contiguous())
    return torch.cat(parts, dim=dim)
