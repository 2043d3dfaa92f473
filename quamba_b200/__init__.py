"""quamba_b200: the quantized Mamba mixer hot path of Quamba on B200 (sm_100a).

Hand-written CUDA behind a C ABI (include/quamba_b200.h, libquamba_b200.so), wrapped with the
reference's own extension-level and module-level interfaces:

    from quamba_b200 import ops                 # quant_sscan_cuda, quamba2_conv1d_cuda, ...
    from quamba_b200 import QSScan, Quamba2ChunkScan, QCausalConv1D, Quamb2Conv1D, QHadamard, \
        W4A8B16O16Linear, W4A8B8O8Linear, W4A8B8O8LinearParallel, W8A8B8O8Linear, \
        W8A8B8O8LinearParallel, W8A8B16O16Linear, QRMSNorm, QRMSNormGated, W4O16Embedding, W8O16Embedding, \
        W4A8QMamba2, W8A8QMamba2, W4A8QMamba, W8A8QMamba, QuambaLMHeadModel

Importing the package does not touch the GPU; the shared library is loaded on first use and
its absence is an error (there is no CPU or PyTorch fallback).
"""
from . import _lib  # noqa: F401
from . import ops  # noqa: F401
from .modules import (QCausalConv1D, QHadamard, QSScan, Quamb2Conv1D, Quamba2ChunkScan,  # noqa: F401
                      W4A8B8O8Linear, W4A8B8O8LinearParallel, W4A8B16O16Linear, W8A8B8O8Linear,
                      W8A8B8O8LinearParallel, W8A8B16O16Linear)
from .packing import w4a8_quantize  # noqa: F401
from .norm import QRMSNorm, QRMSNormGated  # noqa: F401
from .embedding import W4O16Embedding, W8O16Embedding  # noqa: F401
from .mixer import W4A8QMamba2, W8A8QMamba2  # noqa: F401
from .mixer1 import QAct, W4A8QMamba, W8A8QMamba  # noqa: F401
from .model import InferenceParams, QuambaConfig, QuambaLMHeadModel, QuambaMixerModel  # noqa: F401



def check_device_status(stream=None):
    """Waits for ``stream`` (default: torch's current stream) and raises if a kernel of this library gave up on one of
    its bounded device waits, or rejected an input on the device (an embedding id out of range), since the last check.
    Outputs are valid only if this passes; call it at the natural synchronisation points of a caller (the end of a
    generation loop, after a benchmark step, before results leave the device).  ``generate_greedy`` does."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    elif hasattr(stream, "cuda_stream"):
        stream = stream.cuda_stream
    _lib.read_device_status(stream)


__version__ = "0.1.0"
