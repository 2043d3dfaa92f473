"""CPU oracle for the quantized Mamba mixer hot path.

TEST INFRASTRUCTURE ONLY.  Everything in this package is a CPU (torch fp32/fp64)
restatement of the reference kernels' arithmetic.  It exists to check the CUDA
library and to serve as the timed CPU baseline; it is never imported by the
product package and nothing in the product path may fall back to it.

Pinning status (what each restatement has been checked against):

* ``ssd``      -- pinned: compared with the reference's own Triton kernels
                  (chunk cumsum / chunk state / state passing / bmm chunk /
                  chunk scan) executed in Triton interpreter mode on CPU; the
                  resulting tensors are committed under ``tests/golden``.
* ``linear``   -- pinned: the packed-int4 format and the dequantised reference
                  weights come from the reference's ``quamba/marlin_utils.py``
                  imported on CPU; fixtures under ``tests/golden``.
* ``update``   -- pinned against the reference's pure-torch
                  ``selective_state_update_ref``; fixtures under ``tests/golden``.
* ``conv1d``, ``sscan``, ``hadamard`` -- the reference implements these only as
                  CUDA kernels that cannot execute without a GPU; the Hadamard
                  sign tables are parsed from the reference's generator and
                  checked for H H^T = n I, the rest is "parity unpinned" (self-
                  consistency and closed-form cases only).
"""

from . import quant, conv1d, hadamard, sscan, update, ssd, linear  # noqa: F401
