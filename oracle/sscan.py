"""CPU restatement of the Mamba1 int8 selective scan forward (test infrastructure only).

Parity unpinned: the reference implements this only as a CUDA kernel; this is the
dequantise-then-fp32 sequential recurrence (the role of ``selective_scan_ref``).

Follows
  csrc/selective_scan/quant_sscan_fwd_kernel.cuh:157-173  (dequant, softplus, A = -exp(s_A q_A))
  csrc/selective_scan/quant_sscan_fwd_kernel.cuh:219-249  (h <- exp(dA) h + s_B B delta u ; y += h s_C C)
  csrc/selective_scan/quant_sscan_fwd_kernel.cuh:240-241  (chunk-end state -> int8, roundf + clamp)
  csrc/selective_scan/quant_sscan_fwd_kernel.cuh:271-272  (y * z / (1 + exp(-z)) -> fp16)
  csrc/selective_scan/quant_sscan.cpp:236-264             (2048-step chunks; output (B, L, D))
"""
import torch

from .quant import softplus_ref, to_int8_rhaz

CHUNK = 2048


def quant_sscan_fwd(q_u, s_u, q_delta, s_delta, q_A_log, s_A, q_B, s_B, q_C, s_C, s_state,
                    q_D=None, s_D=None, q_z=None, s_z=None, q_delta_bias=None, s_delta_bias=None,
                    delta_softplus=True, dtype=torch.float32):
    """q_u, q_delta, q_z: int8 (B, D, L); q_B, q_C: int8 (B, G, N, L); q_A_log int8 (D, N);
    q_D, q_delta_bias int8 (D).  Scales: python floats / 0-d tensors.
    Returns y fp16 (B, L, D), x int8 (B, D, nchunks, N), h_last fp32 (B, D, N)."""
    f = lambda v: torch.as_tensor(v, dtype=torch.float32).reshape(()).to(dtype)
    Bsz, Dm, L = q_u.shape
    G, N = q_B.shape[1], q_B.shape[2]
    u = f(s_u) * q_u.to(dtype)
    delta = f(s_delta) * q_delta.to(dtype)
    if q_delta_bias is not None:
        delta = delta + (f(s_delta_bias) * q_delta_bias.to(dtype))[None, :, None]
    if delta_softplus:
        delta = softplus_ref(delta)
    A = -torch.exp(f(s_A) * q_A_log.to(dtype))                               # (D, N)
    Bm = (f(s_B) * q_B.to(dtype)).repeat_interleave(Dm // G, dim=1)          # (B, D, N, L)
    Cm = (f(s_C) * q_C.to(dtype)).repeat_interleave(Dm // G, dim=1)
    nchunks = (L + CHUNK - 1) // CHUNK
    h = torch.zeros(Bsz, Dm, N, dtype=dtype)
    y = torch.empty(Bsz, Dm, L, dtype=dtype)
    x = torch.empty(Bsz, Dm, nchunks, N, dtype=torch.int8)
    for l in range(L):
        dA = torch.exp(delta[:, :, l, None] * A[None])
        h = dA * h + Bm[:, :, :, l] * (delta[:, :, l] * u[:, :, l])[:, :, None]
        y[:, :, l] = (h * Cm[:, :, :, l]).sum(-1)
        if (l + 1) % CHUNK == 0 or l == L - 1:
            x[:, :, l // CHUNK] = to_int8_rhaz(h.float() / f(s_state).float())
    if q_D is not None:
        y = y + (f(s_D) * q_D.to(dtype))[None, :, None] * u
    if q_z is not None:
        z = f(s_z) * q_z.to(dtype)
        y = y * z / (1.0 + torch.exp(-z))
    return y.transpose(1, 2).contiguous().to(torch.float16), x, h.float()
