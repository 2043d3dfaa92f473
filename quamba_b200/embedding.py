"""W4O16Embedding / W8O16Embedding with the reference's parameters and packing (quamba/qEmbedding.py:8-108) on
the sm_100a gather kernel.  ``from_fp16`` and the state dict work on CPU; ``forward`` needs the CUDA library."""
import numpy as np
import torch
import torch.nn as nn

from . import ops
from .modules import _dev

__all__ = ["W4O16Embedding", "W8O16Embedding", "F16Embedding"]

_INTERLEAVE = np.array([0, 2, 4, 6, 1, 3, 5, 7])


class W4O16Embedding(nn.Module):
    """Rows stored as eight 4-bit values per int32 (value + 8, interleaved [0,2,4,6,1,3,5,7]) with one fp16 scale per
    row (max / 8); lookup returns fp16 rows."""

    def __init__(self, num_embeddings, embedding_dim, device=None, **kwargs):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.num_bits = 4
        self.pack_factor = 32 // self.num_bits
        dev = _dev(device)
        # a parameter, not a buffer, because callers find the model's device through next(model.parameters())
        self.register_parameter("weight", nn.Parameter(
            torch.empty((num_embeddings, embedding_dim // self.pack_factor), dtype=torch.int32, device=dev),
            requires_grad=False))
        self.register_buffer("scales", torch.empty((num_embeddings,), dtype=torch.float16, device=dev))

    @classmethod
    def from_fp16(cls, originalLayer):
        dev = originalLayer.weight.device
        q = cls(originalLayer.num_embeddings, originalLayer.embedding_dim, device=dev)
        w = originalLayer.weight.data
        vocab = originalLayer.num_embeddings
        with torch.no_grad():
            scales = w.amax(dim=-1, keepdim=True) / 8
            qw = torch.round((w / scales) + 8).clamp(0, 15).cpu().to(torch.int32).numpy().astype(np.uint32)
            qw = qw.reshape(vocab, -1, 8)[:, :, _INTERLEAVE].reshape(vocab, -1)
            packed = np.zeros((vocab, qw.shape[1] // 8), dtype=np.uint32)
            for i in range(8):
                packed |= (qw[:, i::8] & 0xF) << np.uint32(4 * i)
        q.scales = scales.flatten().to(torch.float16).to(dev)
        q.weight.data = torch.from_numpy(packed.view(np.int32)).to(dev)
        return q

    @torch.no_grad()
    def forward(self, x):
        return ops.quant_embedding_cuda.w4a16_embedding_lookup(x, self.weight, self.scales)

    def __repr__(self):
        return f"W4O16Embedding(num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim})"


class W8O16Embedding(nn.Module):
    """Rows stored as int8 with one fp16 scale per row (max / 127); lookup returns fp16 rows."""

    def __init__(self, num_embeddings, embedding_dim, device=None, **kwargs):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        dev = _dev(device)
        self.register_parameter("weight", nn.Parameter(
            torch.empty((num_embeddings, embedding_dim), dtype=torch.int8, device=dev), requires_grad=False))
        self.register_buffer("scales", torch.empty((num_embeddings,), dtype=torch.float16, device=dev))

    @classmethod
    def from_fp16(cls, originalLayer):
        dev = originalLayer.weight.device
        q = cls(originalLayer.num_embeddings, originalLayer.embedding_dim, device=dev)
        w = originalLayer.weight.data
        with torch.no_grad():
            scales = w.amax(dim=-1, keepdim=True) / 127.0
            w8 = torch.round(w / scales).clamp(-128, 127).to(torch.int8)
        q.scales = scales.flatten().to(torch.float16).to(dev)
        q.weight.data = w8
        return q

    @torch.no_grad()
    def forward(self, x):
        return ops.quant_embedding_cuda.w8a16_embedding_lookup(x, self.weight, self.scales)

    def __repr__(self):
        return f"W8O16Embedding(num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim})"


class F16Embedding(nn.Module):
    """The unquantised table (``torch.nn.Embedding`` in the reference's model shell) on the same gather kernel."""

    def __init__(self, num_embeddings, embedding_dim, device=None, **kwargs):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.register_parameter("weight", nn.Parameter(
            torch.empty((num_embeddings, embedding_dim), dtype=torch.float16, device=_dev(device)), requires_grad=False))

    @torch.no_grad()
    def forward(self, x):
        return ops.quant_embedding_cuda.f16_embedding_lookup(x, self.weight)
