#!/usr/bin/env python
"""Generate tests/golden/linear_w4a8_*.npz with the REFERENCE's own weight packer.

    python tests/golden/make_linear_golden.py /path/to/reference

quamba/marlin_utils.py is imported by file path (the package __init__ needs CUDA
extensions; this file alone does not).  For seeded weights it stores what
``w4a8_quantize`` returns (packed int32 weight, permuted s_group / s_channel, w_ref)
and what ``get_w4a8_quantize_weights`` returns before packing (the nibble matrix and
the un-permuted scales), so the checker's inverse can be pinned on both layouts.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: %s <path to the reference checkout>" % sys.argv[0])
REF = Path(sys.argv[1])
OUT = Path(__file__).resolve().parent


def load_marlin_utils():
    spec = importlib.util.spec_from_file_location("ref_marlin_utils", REF / "quamba" / "marlin_utils.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make(tag, K, N, group, seed, pad_out=0, out_scale=None):
    mu = load_marlin_utils()
    torch.manual_seed(seed)
    w = (torch.randn(K, N) * 0.02).to(torch.float16)
    w_ref0, q_w, s_group_raw, s_channel_raw = mu.get_w4a8_quantize_weights(w.clone(), 4, group)
    out_scales = None if out_scale is None else torch.full((N,), out_scale)
    w_ref, packed, s_group, s_channel = mu.w4a8_quantize(w.clone(), 4, group, out_scales=out_scales, pad_out=pad_out)
    np.savez_compressed(
        OUT / f"linear_w4a8_{tag}.npz",
        w=w.numpy(), q_w=q_w.numpy(), s_group_raw=s_group_raw.numpy(), s_channel_raw=s_channel_raw.numpy(),
        w_ref=w_ref.float().numpy(), packed=packed.numpy(), s_group=s_group.numpy(), s_channel=s_channel.numpy(),
        group=np.array(group), pad_out=np.array(pad_out),
        out_scale=np.array(0.0 if out_scale is None else out_scale))
    print("wrote", OUT / f"linear_w4a8_{tag}.npz", tuple(packed.shape), tuple(s_group.shape), tuple(s_channel.shape))


if __name__ == "__main__":
    make("g128", K=256, N=128, group=128, seed=0)
    make("g128_pad", K=384, N=112, group=128, seed=1, pad_out=16, out_scale=0.05)
    make("perchannel", K=128, N=64, group=-1, seed=2)
