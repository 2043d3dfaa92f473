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
* ``conv1d``, ``sscan``, ``hadamard``, ``embedding`` -- pinned on the GPU: the
                  reference implements these only as CUDA kernels; its own
                  sources are compiled for sm_100a by ``oracle/build_ref.py``
                  into ``oracle/_ref`` and ``tests/test_gpu_reference_kernels.py``
                  compares the CUDA library with them on the same tensors, the
                  same tests that compare it with these restatements.  On CPU:
                  the Hadamard sign tables are parsed from the reference's
                  generator and checked for H H^T = n I, plus self-consistency
                  (forward == repeated update, scan == scan + one step).
* ``norm``     -- pinned: compared with the reference's Triton norm kernels run in
                  interpreter mode (``tests/golden/make_norm_golden.py``).
* ``model``    -- composition of the parts above following the reference's layer
                  ``forward`` / ``step`` and model loop; no reference output exists
                  for a whole model (its checkpoints are not available offline).
"""

from . import quant, conv1d, hadamard, sscan, update, ssd, linear  # noqa: F401
