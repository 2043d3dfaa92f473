"""CPU restatement of the quantised embedding lookups (test infrastructure only).

Follows quamba/qEmbedding.py:26-48 (W4O16 packing), :82-93 (W8O16) and
csrc/embedding/quant_embedding_kernel.cuh:47-84 (int8: ``scale * half(q)`` in fp16), :140-205 (int4:
``half(q - 8) * scale`` in fp16, nibble i of a word = element [0,2,4,6,1,3,5,7][i]).
Pinned against the reference's own packer: tests/golden/make_norm_golden.py re-runs the packing code of
``W4O16Embedding.from_fp16`` and stores table, scales and the dequantised rows.
"""
import numpy as np
import torch

INTERLEAVE = np.array([0, 2, 4, 6, 1, 3, 5, 7])


def pack_w4(embed_w: torch.Tensor):
    """qEmbedding.py:31-48: per-row scale = max / 8 (max, not absmax, as the reference writes it), value + 8 in
    [0, 15], interleave within eight, eight nibbles per int32.  Returns (int32 (V, D/8), fp16 (V))."""
    w = embed_w.float()
    scales = w.amax(dim=-1, keepdim=True) / 8.0
    q = torch.round(w / scales + 8).clamp(0, 15).to(torch.int32).numpy().astype(np.uint32)
    V = q.shape[0]
    q = q.reshape(V, -1, 8)[:, :, INTERLEAVE].reshape(V, -1)
    packed = np.zeros((V, q.shape[1] // 8), dtype=np.uint32)
    for i in range(8):
        packed |= (q[:, i::8] & 0xF) << np.uint32(4 * i)
    return torch.from_numpy(packed.view(np.int32)), scales.flatten().to(torch.float16)


def pack_w8(embed_w: torch.Tensor):
    """qEmbedding.py:87-91."""
    w = embed_w.float()
    scales = w.amax(dim=-1, keepdim=True) / 127.0
    q = torch.round(w / scales).clamp(-128, 127).to(torch.int8)
    return q, scales.flatten().to(torch.float16)


def unpack_w4(packed: torch.Tensor) -> torch.Tensor:
    """int32 (V, D/8) -> signed values (V, D) in [-8, 7] in natural element order."""
    p = packed.numpy().view(np.uint32)
    V, W = p.shape
    out = np.zeros((V, W, 8), dtype=np.int32)
    for i in range(8):
        out[:, :, INTERLEAVE[i]] = ((p >> np.uint32(4 * i)) & 0xF).astype(np.int32) - 8
    return torch.from_numpy(out.reshape(V, W * 8))


def lookup_w4(tokens, packed, scales):
    rows = unpack_w4(packed)[tokens.reshape(-1)]
    s = scales[tokens.reshape(-1)].to(torch.float16)
    out = (rows.to(torch.float16).float() * s.float()[:, None]).to(torch.float16)     # one fp16 multiply
    return out.reshape(*tokens.shape, -1)


def lookup_w8(tokens, table, scales):
    rows = table[tokens.reshape(-1)].to(torch.float16)
    s = scales[tokens.reshape(-1)].to(torch.float16)
    out = (rows.float() * s.float()[:, None]).to(torch.float16)
    return out.reshape(*tokens.shape, -1)
