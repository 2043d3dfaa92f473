"""CPU restatement of the fused Hadamard-rotate + int8 quantise (test infrastructure only).

Parity unpinned for the kernel arithmetic (CUDA-only in the reference); the
special-order sign tables are the reference generator's own matrices (parsed
into tests/golden/hadamard_tables.json) and are verified Hadamard.

Follows
  csrc/hadamard/fast_hadamard_transform_common.h:86-124  (Sylvester butterflies, stride 1 upwards)
  csrc/hadamard/quant_hadamard_fwd.cu:189-228            (2^k part on the fast index, special
                                                          12/20/28/40 part across the chunk index)
  csrc/hadamard/fast_hadamard_transform_common.h:153     (roundf(v * scale) -> int8)
  quamba/hadamard_utils.py:33-47                          (dispatch: %12, %40, else power of two)
"""
import json
from pathlib import Path

import torch

from .quant import round_half_away

_TABLES = None


def special_matrix(n: int) -> torch.Tensor:
    """The n x n (n in 12, 20, 28, 40) +-1 matrix, fp64."""
    global _TABLES
    if _TABLES is None:
        p = Path(__file__).resolve().parent.parent / "tests" / "golden" / "hadamard_tables.json"
        _TABLES = json.loads(p.read_text())
    masks = [int(m, 16) for m in _TABLES[str(n)]]
    return torch.tensor([[-1.0 if (masks[i] >> j) & 1 else 1.0 for j in range(n)] for i in range(n)],
                        dtype=torch.float64)


def sylvester(n: int) -> torch.Tensor:
    """H[i][j] = (-1)^popcount(i & j); n a power of two."""
    assert n & (n - 1) == 0 and n > 0
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def split_dim(dim: int):
    """(special order S, power-of-two part) per quamba/hadamard_utils.py:35-46."""
    if dim % 12 == 0:
        s = 12
    elif dim % 40 == 0:
        s = 40
    else:
        s = 1
    p2 = dim // s
    assert p2 & (p2 - 1) == 0 and p2 > 0, f"dim {dim} unsupported"
    return s, p2


def hadamard_matrix(dim: int, special: int = None) -> torch.Tensor:
    """H_dim = H_special (x) H_{2^k}, element index = chunk * 2^k + j."""
    if special is None:
        special, p2 = split_dim(dim)
    else:
        p2 = dim // special
    h2 = sylvester(p2)
    if special == 1:
        return h2
    return torch.kron(special_matrix(special), h2)


def hadamard_transform(x: torch.Tensor, special: int = None) -> torch.Tensor:
    """y = x H^T over the last dim, fp64 accumulate (unscaled)."""
    dim = x.shape[-1]
    H = hadamard_matrix(dim, special)
    return x.double() @ H.t()


def quant_hadamard(x: torch.Tensor, scale: float, special: int = None, saturate: bool = True):
    """int8(roundf((H x) * scale)).  The reference casts without clamping (undefined for
    |v| > 127); this build saturates.  Returns (q int8, overflow mask bool)."""
    v = (hadamard_transform(x, special) * float(torch.tensor(scale, dtype=torch.float32))).float()
    r = round_half_away(v)
    overflow = (r > 127) | (r < -128)
    if saturate:
        r = torch.clamp(r, -128, 127)
    return r.to(torch.int8), overflow
