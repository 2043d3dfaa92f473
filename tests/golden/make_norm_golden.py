#!/usr/bin/env python
"""Generate tests/golden/norm_*.npz and embedding_w4.npz from the REFERENCE's own code, on CPU.

    TRITON_INTERPRET=1 python tests/golden/make_norm_golden.py /path/to/reference

* The two Triton kernels ``_qlayer_norm_fwd_1pass_kernel`` (quamba/triton/quant_norm.py:68-132 and
  quamba/triton/quant_normgated.py:11-83) are launched directly (``kernel.fn[grid]`` below the autotuner /
  heuristics wrappers) in Triton interpreter mode.  They call ``tl.extra.cuda.libdevice.rint``, which the
  interpreter cannot run; it is replaced by an equivalent round-half-to-even written with tl.floor.
* The packing code of ``W4O16Embedding.from_fp16`` (quamba/qEmbedding.py:26-48) is executed as it stands in the
  file (the class itself cannot be imported: the module imports a compiled extension), and the table, scales
  and the rows dequantised as csrc/embedding/quant_embedding_kernel.cuh:140-168 does are stored.
"""
import importlib.util
import os
import re
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch
import triton
import triton.language as tl

if len(sys.argv) < 2:
    raise SystemExit("usage: make_norm_golden.py <path to the reference checkout>")
REF = Path(sys.argv[1])
OUT = Path(__file__).resolve().parent


@triton.jit
def _rint_stub(x):
    r = tl.floor(x + 0.5)
    tie = (r - x) == 0.5
    odd = (r - 2.0 * tl.floor(r * 0.5)) != 0.0
    return tl.where(tie & odd, r - 1.0, r)


tl.extra.cuda.libdevice.rint = _rint_stub


def _load(name):
    spec = importlib.util.spec_from_file_location("ref_" + name, REF / "quamba" / "triton" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _jit(k):
    while not isinstance(k, triton.runtime.jit.JITFunction) and not type(k).__name__.startswith("Interpreted"):
        k = k.fn
    return k


def norm_case(tag, M, N, residual_dtype, static_scale, seed):
    g = torch.Generator().manual_seed(seed)
    mod = _load("quant_norm")
    kern = _jit(mod._qlayer_norm_fwd_1pass_kernel)
    x = torch.randn(M, N, generator=g).to(torch.float16)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.float16)
    res = None if residual_dtype is None else torch.randn(M, N, generator=g).to(residual_dtype)
    y = torch.empty(M, N, dtype=torch.int8)
    res_out = torch.empty(M, N, dtype=residual_dtype) if res is not None else None
    dyn = torch.zeros(M, dtype=torch.float32)
    BLOCK_N = triton.next_power_of_2(N)
    kern[(M,)](x, y, w, None, res, res_out, static_scale, dyn, x.stride(0), y.stride(0),
               res.stride(0) if res is not None else 0, res_out.stride(0) if res_out is not None else 0, M, N, 1e-5,
               True, BLOCK_N, res is not None, res_out is not None, False, static_scale is not None)
    out = dict(x=x.numpy(), w=w.numpy(), y=y.numpy(), dyn=dyn.numpy(), static=np.float32(static_scale or 0.0))
    if res is not None:
        out.update(res=res.numpy(), res_out=res_out.numpy())
    np.savez_compressed(OUT / f"norm_{tag}.npz", **out)
    print("wrote", tag)


def gated_case(tag, M, N, group_size, norm_before_gate, f16_out, static_scale, seed):
    g = torch.Generator().manual_seed(seed)
    mod = _load("quant_normgated")
    kern = _jit(mod._qlayer_norm_fwd_1pass_kernel)
    x = torch.randn(M, N, generator=g).to(torch.float16)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.float16)
    zf = torch.randn(M, N, generator=g)
    z_scale = float(zf.abs().max() / 127)
    qz = torch.clamp(torch.round(zf / z_scale), -128, 127).to(torch.int8)
    G = N // group_size
    y = torch.empty(M, N, dtype=torch.float16 if f16_out else torch.int8)
    dyn = torch.zeros(G * M, dtype=torch.float32)
    BLOCK_N = triton.next_power_of_2(group_size)
    kern[(M, G)](x, y, w, None, qz, z_scale, static_scale, dyn, x.stride(0), y.stride(0), qz.stride(0), M, group_size, 1e-5,
                 BLOCK_N=BLOCK_N, HAS_BIAS=False, HAS_Z=True, NORM_BEFORE_GATE=norm_before_gate, IS_RMS_NORM=True,
                 USE_FLOAT16_OUTPUT=f16_out, IS_STATIC_SCALE=static_scale is not None)
    np.savez_compressed(OUT / f"norm_gated_{tag}.npz", x=x.numpy(), w=w.numpy(), qz=qz.numpy(), z_scale=np.float32(z_scale),
                        y=y.numpy(), dyn=dyn.numpy(), static=np.float32(static_scale or 0.0), group_size=np.int32(group_size),
                        norm_before_gate=np.int32(norm_before_gate))
    print("wrote gated", tag)


def embedding_case():
    src = (REF / "quamba" / "qEmbedding.py").read_text()
    body = re.search(r"        with torch\.no_grad\(\):\n(.*?)\n        qembed\.scales", src, re.S).group(1)
    torch.manual_seed(3)
    vocab, dim = 64, 96
    env = dict(torch=torch, np=np, embed_w=torch.randn(vocab, dim) * 0.02, vocab_size=vocab, max_val=16, zero_point=8,
               interleave=np.array([0, 2, 4, 6, 1, 3, 5, 7]),
               qembed=type("Q", (), {"pack_factor": 8, "num_bits": 4})())
    exec("if True:\n" + body, env)                      # the reference's own packing statements
    packed = env["embed_qw_packed"].astype(np.int32)
    scales = env["scales"].flatten().to(torch.float16)
    # dequantised rows as the lookup kernel forms them: half(q - 8) * scale in fp16
    q = np.zeros((vocab, dim // 8, 8), dtype=np.int32)
    for i in range(8):
        q[:, :, [0, 2, 4, 6, 1, 3, 5, 7][i]] = (packed.view(np.uint32) >> np.uint32(4 * i)) & 0xF
    rows = ((torch.from_numpy(q.reshape(vocab, dim)) - 8).to(torch.float16).float() * scales.float()[:, None]).to(torch.float16)
    np.savez_compressed(OUT / "embedding_w4.npz", embed_w=env["embed_w"].numpy(), packed=packed, scales=scales.numpy(),
                        rows=rows.numpy())
    print("wrote embedding_w4")


if __name__ == "__main__":
    norm_case("static_res32", 5, 2560, torch.float32, 0.03, 0)
    norm_case("static_res16", 4, 768, torch.float16, 0.05, 1)
    norm_case("static_nores", 3, 1024, None, 0.04, 2)
    norm_case("dynamic", 4, 2560, torch.float16, None, 3)
    gated_case("f16_g1", 4, 5120, 5120, False, True, None, 4)
    gated_case("f16_g8", 3, 1024, 128, False, True, None, 5)
    gated_case("f16_nbg", 3, 1536, 1536, True, True, None, 6)
    gated_case("s8_static", 3, 1024, 512, False, False, 0.02, 7)
    gated_case("s8_dynamic", 3, 768, 768, False, False, None, 8)
    embedding_case()
