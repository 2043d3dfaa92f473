"""Float Hadamard rotation with the very matrices the quantising kernel applies (H_S (x) H_{2^k}, S in 1, 12, 20,
28, 40; quamba/hadamard_utils.py:33-47 dispatch, csrc/hadamard/code_gen.py tables).  Used offline: to calibrate the
scale of the rotated out_proj input and to fold the rotation into out_proj weights
(``HadLinear.fuse_hadamard``, quamba/qLinearLayer.py:860-868)."""
import math
import re
from functools import lru_cache
from pathlib import Path

import torch

_TABLES = Path(__file__).resolve().parent / "csrc" / "hadamard_tables.inc"


@lru_cache(maxsize=None)
def special_matrix(n: int) -> torch.Tensor:
    """+-1 matrix of order 12 / 20 / 28 / 40, read from the table file the CUDA kernels are compiled with."""
    text = _TABLES.read_text()
    m = re.search(r"kHadNeg%d\[%d\]\s*=\s*\{(.*?)\};" % (n, n), text, re.S)
    if m is None:
        raise ValueError(f"no Hadamard table of order {n}")
    masks = [int(v, 16) for v in re.findall(r"0x([0-9a-fA-F]+)ULL", m.group(1))]
    return torch.tensor([[-1.0 if (masks[i] >> j) & 1 else 1.0 for j in range(n)] for i in range(n)])


def split_dim(dim: int):
    s = 12 if dim % 12 == 0 else (40 if dim % 40 == 0 else 1)
    p2 = dim // s
    if p2 <= 0 or p2 & (p2 - 1):
        raise ValueError(f"no Hadamard transform for dim {dim}")
    return s, p2


def hadamard_transform(x: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """y = H_dim x over the last dim (fp32), element index = chunk * 2^k + j; scaled by 1 / sqrt(dim) if asked."""
    dim = x.shape[-1]
    s, p2 = split_dim(dim)
    y = x.float().reshape(-1, s, p2)
    h = 1
    while h < p2:                                   # Sylvester butterflies along the fast index
        y = y.reshape(-1, s, p2 // (2 * h), 2, h)
        a, b = y[:, :, :, 0], y[:, :, :, 1]
        y = torch.stack((a + b, a - b), dim=3)
        h *= 2
    y = y.reshape(-1, s, p2)
    if s > 1:
        y = torch.einsum("ij,bjk->bik", special_matrix(s).to(y.device), y)
    y = y.reshape(x.shape)
    return y / math.sqrt(dim) if normalize else y
