"""Minimal language-model shell around the quantized mixers: embedding -> [QRMSNorm(+residual) -> mixer] x n_layer ->
norm_f -> lm_head, with the decode step (and optionally the prefill) replayed from a CUDA graph.

Mirrors what the reference assembles from mamba_ssm's ``MixerModel`` / ``MambaLMHeadModel`` and its own
``QuambaMixerModel`` / ``QuambaLMHeadModel`` (quamba/quamba_mixer_seq.py:56-171, :263-421): module names
(``backbone.embedding``, ``backbone.layers[i].norm`` / ``.mixer``, ``backbone.norm_f``, ``lm_head``), the
``ssm_cfg["layer"]`` / ``norm_cfg`` / ``embedding_cfg`` / ``lm_head_cfg`` dispatch, ``forward(input_ids,
inference_params=..., num_last_tokens=...)`` returning an object with ``.logits``, ``allocate_inference_cache``.
Timing methods follow profile_mamba.py:190-213 (prefill) and :239-292 (decode step under one CUDA graph).
"""
import copy
from collections import namedtuple
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from . import embedding as _emb
from . import mixer as _mixer
from . import mixer1 as _mixer1
from . import modules as _modules
from . import _lib
from . import ops
from .norm import QRMSNorm

__all__ = ["QuambaConfig", "InferenceParams", "Block", "QuambaMixerModel", "QuambaLMHeadModel", "GraphRunner"]

CausalLMOutput = namedtuple("CausalLMOutput", ["logits"])
# Development switch: QB_UNFUSED_DECODE=1 keeps the decode step on the one-op-per-launch path (for A/B comparisons).
import os as _os
_UNFUSED_DECODE = bool(_os.environ.get("QB_UNFUSED_DECODE"))
# Development switch: QB_NO_EARLY_OVERLAP=1 launches the prefill kernels without early dependent starts (for A/B comparisons).
_EARLY_OVERLAP = not _os.environ.get("QB_NO_EARLY_OVERLAP")


@dataclass
class QuambaConfig:
    """The fields of the reference's QuambaConfig (MambaConfig + norm_cfg / embedding_cfg / lm_head_cfg)."""
    d_model: int = 2560
    d_intermediate: int = 0
    n_layer: int = 64
    vocab_size: int = 50277
    ssm_cfg: dict = field(default_factory=dict)
    attn_layer_idx: list = field(default_factory=list)
    attn_cfg: dict = field(default_factory=dict)
    rms_norm: bool = True
    residual_in_fp32: bool = True
    fused_add_norm: bool = True
    pad_vocab_size_multiple: int = 8
    tie_embeddings: bool = True
    norm_cfg: dict = field(default_factory=dict)
    embedding_cfg: dict = field(default_factory=dict)
    lm_head_cfg: dict = field(default_factory=dict)
    is_hybrid: bool = False


@dataclass
class InferenceParams:
    """Generation state shared by the layers (mamba_ssm.utils.generation.InferenceParams)."""
    max_seqlen: int
    max_batch_size: int
    seqlen_offset: int = 0
    batch_size_offset: int = 0
    key_value_memory_dict: dict = field(default_factory=dict)
    lengths_per_sample: Optional[torch.Tensor] = None

    def reset(self, max_seqlen, max_batch_size):
        self.max_seqlen, self.max_batch_size, self.seqlen_offset = max_seqlen, max_batch_size, 0
        if self.lengths_per_sample is not None:
            self.lengths_per_sample.zero_()


_MIXERS = {"W4A8QMamba2": _mixer.W4A8QMamba2, "W8A8QMamba2": _mixer.W8A8QMamba2,
           "W4A8QMamba": _mixer1.W4A8QMamba, "W8A8QMamba": _mixer1.W8A8QMamba}
_EMBEDDINGS = {"Embedding": _emb.F16Embedding, "W4O16Embedding": _emb.W4O16Embedding, "W8O16Embedding": _emb.W8O16Embedding}
_LM_HEADS = {"W4A8B16O16Linear": _modules.W4A8B16O16Linear, "W8A8B16O16Linear": _modules.W8A8B16O16Linear}


class Block(nn.Module):
    """Add -> norm -> mixer with the add fused into the norm kernel (mamba_ssm.modules.block.Block with
    fused_add_norm=True, the only mode the quantized models use)."""

    def __init__(self, dim, mixer_cls, norm_cls, residual_in_fp32=True):
        super().__init__()
        self.residual_in_fp32 = residual_in_fp32
        self.fused_add_norm = True
        self.norm = norm_cls(dim)
        self.mixer = mixer_cls(dim)

    def forward(self, hidden_states, residual=None, inference_params=None, **mixer_kwargs):
        hidden_states, residual = self.norm(hidden_states, residual=residual, prenorm=True,
                                            residual_in_fp32=self.residual_in_fp32)
        hidden_states = self.mixer(hidden_states, inference_params=inference_params, **mixer_kwargs)
        return hidden_states, residual

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        return self.mixer.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)


def create_quantized_block(d_model, ssm_cfg, norm_epsilon, norm_cfg, residual_in_fp32, layer_idx, device=None):
    ssm_cfg = copy.deepcopy(ssm_cfg) if ssm_cfg is not None else {}
    ssm_layer = ssm_cfg.pop("layer", "W8A8QMamba2")
    if ssm_layer not in _MIXERS:
        raise ValueError(f"Invalid ssm_layer: {ssm_layer}, only support {sorted(_MIXERS)}")
    norm_cfg = copy.deepcopy(norm_cfg) if norm_cfg is not None else {}
    block_norm = norm_cfg.pop("norm", "QRMSNorm")
    if block_norm != "QRMSNorm":
        raise ValueError(f"Invalid block_norm: {block_norm}, only support ['QRMSNorm']")
    mixer_cls = lambda dim: _MIXERS[ssm_layer](dim, layer_idx=layer_idx, device=device, **ssm_cfg)
    norm_cls = lambda dim: QRMSNorm(dim, eps=norm_epsilon, device=device)
    block = Block(d_model, mixer_cls, norm_cls, residual_in_fp32=residual_in_fp32)
    block.layer_idx = layer_idx
    return block


class QuambaMixerModel(nn.Module):
    def __init__(self, d_model, n_layer, vocab_size, embedding_cfg=None, ssm_cfg=None, norm_epsilon=1e-5, rms_norm=True,
                 norm_cfg=None, residual_in_fp32=True, device=None):
        super().__init__()
        assert rms_norm is True, "Only RMSNorm is supported in Quamba"
        self.residual_in_fp32 = residual_in_fp32
        embedding_cfg = copy.deepcopy(embedding_cfg) if embedding_cfg is not None else {}
        embed_layer = embedding_cfg.pop("layer", "Embedding")
        if embed_layer not in _EMBEDDINGS:
            raise ValueError(f"Invalid embedding layer: {embed_layer}, only support {sorted(_EMBEDDINGS)}")
        self.embedding = _EMBEDDINGS[embed_layer](vocab_size, d_model, device=device)
        self.fused_add_norm = True
        self.layers = nn.ModuleList([create_quantized_block(d_model, ssm_cfg, norm_epsilon, norm_cfg, residual_in_fp32, i,
                                                            device=device) for i in range(n_layer)])
        self.norm_f = QRMSNorm(d_model, eps=norm_epsilon, device=device)

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        return {i: layer.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)
                for i, layer in enumerate(self.layers)}

    # ---- fused decode step (1 to 4 sequences): four launches per layer instead of seven -------------------------
    def _decode_fusable(self, batch, lm_head):
        ok = self.__dict__.get("_fusable")
        if ok is None:
            from .mixer import W4A8QMamba2
            from .modules import W4A8B16O16Linear
            ok = isinstance(lm_head, W4A8B16O16Linear) and self.norm_f.output_scale and self.embedding.embedding_dim <= 8192
            for layer in self.layers:
                m = layer.mixer
                s = m.d_inner // 128 if isinstance(m, W4A8QMamba2) else 0
                ok = bool(ok and isinstance(m, W4A8QMamba2) and layer.norm.output_scale and m.conv1d.x_head_group_range is None
                          and m.d_conv == 4 and m.d_inner == m.d_ssm and m.d_inner % 128 == 0 and not m.D_has_hdim
                          and getattr(m.had, "blocks", 1) == 1
                          and (s in (12, 20, 28, 40) or (s & (s - 1)) == 0 and s <= 64)
                          and m.d_model % 32 == 0 and m.d_ssm // m.ngroups % 128 == 0 and m.ngroups <= 64
                          # the state update must land on its one-CTA-per-head kernel (the early-launch chain needs it)
                          and m.d_state == 128 and m.headdim % 64 == 0 and m.nheads <= 128 and not m.qchunk_scan.grouped)
            self.__dict__["_fusable"] = ok
        return ok and 1 <= batch <= 4 and not _UNFUSED_DECODE

    def decode_step_fused(self, input_ids, inference_params, lm_head):
        """One token per sequence through all layers and the head; returns logits fp16 (batch, vocab)."""
        h = self.embedding(input_ids[:, 0])
        residual = None
        with ops.early_dependents():
            for layer in self.layers:
                m, c, s = layer.mixer, layer.mixer.conv1d, layer.mixer.qchunk_scan
                conv_state, ssm_state = m._get_states_from_cache(inference_params, h.shape[0])
                gn = m.ngroups * m.d_state
                conv = dict(state=conv_state, weight=c.weight, bias=c.bias, col0=m.d_ssm, x_dim=m.d_ssm, gn=gn,
                            scale_in=(c.wx_scale * c.x_scale, c.wB_scale * c.B_scale, c.wC_scale * c.C_scale),
                            scale_bias=(c.bx_scale or 0.0, c.bB_scale or 0.0, c.bC_scale or 0.0),
                            out_scales=(c.x_out_scales, c.B_out_scales, c.C_out_scales))
                zxbcdt, residual = ops.decode_norm_linear(h, residual, layer.norm.weight, layer.norm.eps, layer.norm.output_scale,
                                                          m.in_proj.prepared(), m.in_proj.input_scale, True, self.residual_in_fp32, conv)
                dt = zxbcdt[:, 2 * m.d_ssm + 2 * gn:2 * m.d_ssm + 2 * gn + m.nheads]
                y = s.update(ssm_state, conv["x"], dt, conv["B"], conv["C"], z=None)
                a = ops.decode_gate_had_quant(y.flatten(-2), zxbcdt[:, :m.d_ssm], m.norm.z_scale, m.norm.weight, m.norm.eps,
                                              m.norm.group_size or m.d_ssm, m.had.had_scale / m.had.x_H_scale)
                h = ops.decode_linear(a, m.out_proj.prepared(), m.out_proj.input_scale)[:, :m.d_model]
            logits, _ = ops.decode_norm_linear(h, residual, self.norm_f.weight, self.norm_f.eps, self.norm_f.output_scale,
                                               lm_head.prepared(), lm_head.input_scale, False, self.residual_in_fp32)
        return logits[:, :lm_head.out_features]

    def forward(self, input_ids, inference_params=None, num_last_tokens=0, **mixer_kwargs):
        # the layers' kernels let their successors start early (prologue and residency overlap the tail of the kernel
        # before): the launch sequence in here consists of this library's kernels and ordinary torch launches only
        with _lib.early_overlap(_EARLY_OVERLAP):
            hidden_states = self.embedding(input_ids)
            residual = None
            for layer in self.layers:
                hidden_states, residual = layer(hidden_states, residual, inference_params=inference_params, **mixer_kwargs)
            if num_last_tokens > 0:       # the final norm works row by row: rows nobody reads are skipped
                hidden_states, residual = hidden_states[:, -num_last_tokens:], residual[:, -num_last_tokens:]
            return self.norm_f(hidden_states, residual=residual, prenorm=False, residual_in_fp32=self.residual_in_fp32)


class QuambaLMHeadModel(nn.Module):
    def __init__(self, config: QuambaConfig, device=None, **kwargs):
        super().__init__()
        self.config = config
        vocab_size = config.vocab_size
        if vocab_size % config.pad_vocab_size_multiple != 0:
            vocab_size += config.pad_vocab_size_multiple - (vocab_size % config.pad_vocab_size_multiple)
        self.vocab_size = vocab_size
        self.backbone = QuambaMixerModel(config.d_model, config.n_layer, vocab_size, embedding_cfg=config.embedding_cfg,
                                         ssm_cfg=config.ssm_cfg, rms_norm=config.rms_norm, norm_cfg=config.norm_cfg,
                                         residual_in_fp32=config.residual_in_fp32, device=device)
        lm_head_cfg = copy.deepcopy(config.lm_head_cfg) if config.lm_head_cfg is not None else {}
        lm_head_layer = lm_head_cfg.pop("layer", "W4A8B16O16Linear")
        if lm_head_layer not in _LM_HEADS:
            raise ValueError(f"Invalid lm_head layer: {lm_head_layer}, only support {sorted(_LM_HEADS)}")
        self.lm_head = _LM_HEADS[lm_head_layer](config.d_model, vocab_size, device=device)

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        return self.backbone.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)

    # ---- checkpoints in the reference's layout (quamba/quamba_mixer_seq.py:423-449) --------------------------------------
    def save_pretrained(self, save_directory):
        """Writes ``pytorch_model.bin`` (the state dict: buffers plus the float scales the modules' hooks add) and
        ``config.json`` (the config's fields)."""
        import json
        import os
        os.makedirs(save_directory, exist_ok=True)
        torch.save(self.state_dict(), os.path.join(save_directory, "pytorch_model.bin"))
        with open(os.path.join(save_directory, "config.json"), "w") as f:
            json.dump(self.config.__dict__, f, indent=4)

    @classmethod
    def from_pretrained(cls, pretrained_dir, device=None, **kwargs):
        """Builds the model from a directory holding ``config.json`` + ``pytorch_model.bin`` as ``save_pretrained`` (here
        or in the reference) writes them: constructed on the CPU, buffers resized to what the checkpoint holds (per-tensor
        or head-grouped scale tables, per-channel or group-128 weights), loaded, then moved to ``device``."""
        import json
        import os
        with open(os.path.join(pretrained_dir, "config.json")) as f:
            data = json.load(f)
        known = {k: v for k, v in data.items() if k in QuambaConfig.__dataclass_fields__}
        model = cls(QuambaConfig(**known), device="cpu", **kwargs)
        sd = torch.load(os.path.join(pretrained_dir, "pytorch_model.bin"), map_location="cpu", weights_only=True)
        _fit_buffers_to(model, sd)
        model.load_state_dict(sd)
        return model.to(device) if device is not None else model

    @torch.no_grad()
    def forward(self, input_ids, position_ids=None, inference_params=None, num_last_tokens=0, **mixer_kwargs):
        """input_ids int64 (batch, seqlen).  Prefill when ``inference_params.seqlen_offset == 0`` (the layers then also
        fill their conv / ssm caches), one decode step otherwise.  ``logits`` fp16 (batch, seqlen or num_last_tokens,
        vocab)."""
        bb = self.backbone
        if (inference_params is not None and inference_params.seqlen_offset > 0 and input_ids.shape[1] == 1
                and bb._decode_fusable(input_ids.shape[0], self.lm_head)):
            return CausalLMOutput(logits=bb.decode_step_fused(input_ids, inference_params, self.lm_head)[:, None])
        hidden_states = bb(input_ids, inference_params=inference_params, num_last_tokens=num_last_tokens, **mixer_kwargs)
        return CausalLMOutput(logits=self.lm_head(hidden_states))

    # ---- CUDA-graph runners ------------------------------------------------------------------------------------------
    def capture_prefill(self, batch_size, seqlen, stream=None):
        """A replayable prefill of a fixed (batch, seqlen): ``runner.input_ids`` in, ``runner.logits`` (last token)
        out, the layers' caches in ``runner.inference_params`` filled as a side effect."""
        return GraphRunner(self, batch_size, seqlen, decode=False, stream=stream)

    def capture_decode(self, batch_size, max_seqlen, inference_params=None, stream=None):
        """A replayable single-token step on the caches of ``inference_params`` (fresh zero caches if None).  The step
        also picks the next token greedily and writes it back into ``runner.input_ids``, so consecutive replays
        generate without the host."""
        return GraphRunner(self, batch_size, max_seqlen, decode=True, inference_params=inference_params, stream=stream)

    @torch.no_grad()
    def generate_greedy(self, input_ids, max_new_tokens, use_graph=True):
        """Prefill + greedy decode; returns int64 (batch, prompt + max_new_tokens)."""
        batch, prompt = input_ids.shape
        params = InferenceParams(max_seqlen=prompt + max_new_tokens, max_batch_size=batch)
        logits = self.forward(input_ids, inference_params=params, num_last_tokens=1).logits
        token = ops.greedy_next_token(logits[:, -1])
        out = [input_ids, token[:, None]]
        params.seqlen_offset = prompt
        runner = self.capture_decode(batch, prompt + max_new_tokens, inference_params=params) if use_graph else None
        for _ in range(max_new_tokens - 1):
            if runner is not None:
                runner.input_ids.copy_(token[:, None])
                runner.replay()
                token = runner.input_ids[:, 0].clone()
            else:
                logits = self.forward(token[:, None], inference_params=params).logits
                token = ops.greedy_next_token(logits[:, -1])
            params.seqlen_offset += 1
            out.append(token[:, None])
        from . import check_device_status
        check_device_status()          # a kernel that gave up on a bounded wait leaves garbage behind: raise, do not return it
        return torch.cat(out, dim=1)


class GraphRunner:
    """One model step captured into a CUDA graph with static buffers (the reference captures its decode step the same
    way, profile_mamba.py:265-275).  The first, eager run doubles as warm-up: it builds the linear layers' streaming
    weight copies and looks up per-device kernel attributes, none of which may happen during capture."""

    def __init__(self, model, batch_size, seqlen, decode, inference_params=None, stream=None):
        dev = next(model.parameters()).device
        self.model, self.decode = model, decode
        self.stream = stream or torch.cuda.Stream(device=dev)
        self.input_ids = torch.zeros((batch_size, 1 if decode else seqlen), dtype=torch.int64, device=dev)
        if inference_params is None:
            inference_params = InferenceParams(max_seqlen=seqlen + 1, max_batch_size=batch_size,
                                               key_value_memory_dict=model.allocate_inference_cache(batch_size, seqlen + 1))
            inference_params.seqlen_offset = seqlen if decode else 0
        self.inference_params = inference_params
        self.stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self.stream):
            saved = None
            if decode:      # the eager warm-up step must not advance the caches the caller handed in
                saved = {k: tuple(t.clone() for t in v) for k, v in inference_params.key_value_memory_dict.items()}
            self._step()
            if saved is not None:
                for k, v in saved.items():
                    for dst, src in zip(inference_params.key_value_memory_dict[k], v):
                        dst.copy_(src)
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.logits = self._step()
            if saved is not None:
                for k, v in saved.items():
                    for dst, src in zip(inference_params.key_value_memory_dict[k], v):
                        dst.copy_(src)
        torch.cuda.current_stream(dev).wait_stream(self.stream)

    def _step(self):
        if self.decode:
            logits = self.model(self.input_ids, inference_params=self.inference_params).logits[:, -1]
            ops.greedy_next_token(logits, out=self.input_ids.view(-1))
            return logits
        return self.model(self.input_ids, inference_params=self.inference_params, num_last_tokens=1).logits[:, -1]

    def replay(self):
        self.graph.replay()
        return self.logits


def _fit_buffers_to(model, state_dict):
    """Checkpoints differ in optional pieces the constructors cannot know: scale tables are per-tensor (1 element) or
    head-grouped, the range tables exist only when grouped, per-channel weights carry an empty ``s_group``.  Give every
    buffer the checkpoint's shape, drop the ones it does not hold, before ``load_state_dict``."""
    for name, mod in model.named_modules():
        prefix = name + "." if name else ""
        for bname in list(mod._buffers):
            key = prefix + bname
            buf = mod._buffers[bname]
            if key not in state_dict:
                if buf is not None and bname in ("x_head_group_range", "x_dim_group_range"):
                    del mod._buffers[bname]
                    setattr(mod, bname, None)
                continue
            t = state_dict[key]
            if buf is None or tuple(buf.shape) != tuple(t.shape) or buf.dtype != t.dtype:
                mod._buffers[bname] = torch.empty(t.shape, dtype=t.dtype)
        for pname, par in list(mod._parameters.items()):
            key = prefix + pname
            if key in state_dict and par is not None and tuple(par.shape) != tuple(state_dict[key].shape):
                par.data = torch.empty(state_dict[key].shape, dtype=state_dict[key].dtype)
