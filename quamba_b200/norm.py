"""QRMSNorm and QRMSNormGated with the reference's constructor arguments, buffers and state-dict entries
(quamba/qNorm.py:15-176), running the sm_100a kernels behind ``ops._qlayer_norm_fwd`` /
``ops._qlayer_normgated_fwd``.  Construction, ``from_fp16`` and state-dict round trips work on CPU; ``forward``
needs the CUDA library."""
import torch
import torch.nn as nn

from . import ops
from .modules import _FloatStateMixin, _dev

__all__ = ["QRMSNorm", "QRMSNormGated"]


class QRMSNorm(_FloatStateMixin, nn.Module):
    """h = x + residual; y = int8(rmsnorm(h) * weight / output_scale).  ``output_scale`` None selects one dynamic
    scale per token, returned next to y."""
    _float_state = ("output_scale",)

    def __init__(self, hidden_size, eps=1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.register_buffer("weight", torch.empty(hidden_size, device=_dev(device), dtype=torch.float16))
        self.bias = None
        self.output_scale = 0.0
        self.dim = hidden_size
        self._install_float_state()

    @classmethod
    def from_fp16(cls, originalLayer, output_scale=None):
        q = cls(originalLayer.weight.shape[0], originalLayer.eps, originalLayer.weight.device)
        q.weight = originalLayer.weight.detach().clone().contiguous().to(torch.float16)
        q.output_scale = None
        if output_scale is not None:
            assert type(output_scale) is float, "Only support per-tensor static quant for output"
            q.output_scale = output_scale
        return q

    @torch.no_grad()
    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False, partials=None, out=None, **kwargs):
        """``partials`` (head-parallel exchange): (slots (n, rows, d) fp16, own_index, own or None); x is then slots[0] and
        the normalised input is the fp16-rounded sum of the slots (see ops._qlayer_norm_fwd).  ``out``: an int8 tensor of x's
        shape that receives the result instead of a new one."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        if residual is not None:
            assert residual.shape == shape
            residual = residual.reshape(-1, shape[-1])
            if residual.stride(-1) != 1:
                residual = residual.contiguous()
        residual_dtype = residual.dtype if residual is not None else (torch.float32 if residual_in_fp32 else None)
        y, residual_out, per_token = ops._qlayer_norm_fwd(x2, self.weight, self.bias, self.eps, residual,
                                                          static_out_scale=self.output_scale,
                                                          residual_dtype=residual_dtype, is_rms_norm=True, partials=partials,
                                                          out=None if out is None else out.reshape(-1, shape[-1]))
        y, residual_out = y.reshape(shape), residual_out.reshape(shape)
        if self.output_scale is not None:
            return y if not prenorm else (y, residual_out)
        per_token = per_token.reshape(shape[:-1])
        return (y, per_token) if not prenorm else (y, residual_out, per_token)

    def __repr__(self):
        return f"QRMSNorm(dim={self.dim}, eps={self.eps}, output_scale={self.output_scale})"


class QRMSNormGated(_FloatStateMixin, nn.Module):
    """Grouped RMSNorm of fp16 x gated by int8 z: norm(x) * silu(z) when ``norm_before_gate`` else
    norm(x * silu(z)); fp16, static int8 or per-token int8 output."""
    _float_state = ("z_scale", "output_scale")

    def __init__(self, hidden_size, eps=1e-5, group_size=None, norm_before_gate=True, use_float16_output=False,
                 device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.register_buffer("weight", torch.empty(hidden_size, device=_dev(device), dtype=torch.float16))
        self.bias = None
        self.group_size = group_size
        self.norm_before_gate = norm_before_gate
        self.use_float16_output = use_float16_output
        self.z_scale = 0.0
        self.output_scale = 0.0
        self._install_float_state()

    @classmethod
    def from_fp16(cls, originalLayer, z_scale=None, output_scale=None, use_float16_output=False):
        q = cls(originalLayer.weight.shape[0], originalLayer.eps, originalLayer.group_size,
                originalLayer.norm_before_gate, use_float16_output, originalLayer.weight.device)
        q.weight = originalLayer.weight.detach().clone().to(torch.float16)
        if z_scale is not None:
            assert type(z_scale) is float, "Only support per-tensor static quant for input z"
            q.z_scale = z_scale
        if output_scale is not None:
            assert type(output_scale) is float, "Only support per-tensor static quant for output"
            q.output_scale = output_scale
        else:
            q.output_scale = None
        return q

    @torch.no_grad()
    def forward(self, x, q_z=None):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        if q_z is not None:
            assert q_z.shape == shape
            q_z = q_z.reshape(-1, shape[-1])        # a strided view (a column block of in_proj's output) is fine
            if q_z.stride(-1) != 1:
                q_z = q_z.contiguous()
        y, per_token = ops._qlayer_normgated_fwd(x2, self.weight, self.bias, self.eps, q_z=q_z, z_scale=self.z_scale,
                                                 static_out_scale=self.output_scale,
                                                 use_float16_output=self.use_float16_output, group_size=self.group_size,
                                                 norm_before_gate=self.norm_before_gate, is_rms_norm=True)
        if self.use_float16_output or self.output_scale is not None:
            return y.reshape(shape)
        return y.reshape(shape), per_token.reshape(shape[:-1])

    def __repr__(self):
        return (f"QRMSNormGated(dim={self.weight.shape[0]}, eps={self.eps}, z_scale={self.z_scale}, "
                f"output_scale={self.output_scale}, use_float16_output={self.use_float16_output})")
