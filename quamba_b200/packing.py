"""Weight quantisation and packing into the Marlin-QQQ int4 layout the W4A8 modules store.

The on-disk / state-dict format is the reference's (quamba/marlin_utils.py:139-279), so checkpoints
are interchangeable: ``weight`` int32 (K/16, N*16/8), ``s_group`` fp16 (K/128, N) and ``s_channel``
fp32 (1, N), all in their permuted orders.  The packer here is written as index arithmetic:

  element (k, n) of the K x N matrix lives in 16 x 16 tile (k // 16, n // 16); a row of the
  tile-major matrix (all tiles of one 16-row band) is cut into blocks of 1024 elements (four tiles);
  inside a block, position j takes element ``perm[j]`` (the fragment order of the int8 tensor-core
  instruction the format was designed for, followed by an 8-element interleave that differs between
  per-group and per-channel quantisation); eight consecutive positions are packed little-end first
  into one int32, four bits each.
"""
import torch

TILE = 16
GROUP_SIZES = (-1, 128)


def _weight_perm(per_channel: bool) -> torch.Tensor:
    i = torch.arange(32)
    col = i // 4
    rows = 4 * (i % 4)[:, None] + torch.arange(4)[None, :]                       # (32, 4)
    one = torch.cat([16 * rows + col[:, None], 16 * rows + col[:, None] + 8], dim=1)  # block 0 then block 1
    full = (one[:, None, :] + 256 * torch.arange(4)[None, :, None]).reshape(-1)  # (32 * 4 * 8,)
    inter = torch.tensor([4, 0, 5, 1, 6, 2, 7, 3] if per_channel else [0, 2, 4, 6, 1, 3, 5, 7])
    return full.reshape(-1, 8)[:, inter].reshape(-1)


def _scale_perms():
    j = torch.arange(64)
    group = (j % 8) * 8 + j // 8                                                 # 8 x 8 transpose
    i = torch.arange(32)
    single = 2 * (i // 8) + torch.tensor([0, 1, 8, 9, 16, 17, 24, 25])[i % 8]
    return group, single


def pack_int4(q: torch.Tensor, per_channel: bool) -> torch.Tensor:
    """q: integer (K, N) with values 0..15 (per-group) or -8..7 (per-channel) -> int32 (K/16, N*2)."""
    K, N = q.shape
    assert K % TILE == 0 and N % 64 == 0, "K must be a multiple of 16 and N of 64"
    t = q.reshape(K // TILE, TILE, N // TILE, TILE).permute(0, 2, 1, 3).reshape(K // TILE, N * TILE)
    perm = _weight_perm(per_channel).to(q.device)
    t = t.reshape(-1, perm.numel())[:, perm].reshape(K // TILE, N * TILE).to(torch.int64) & 0xF
    t = t.reshape(K // TILE, N * TILE // 8, 8)
    shifts = 4 * torch.arange(8, dtype=torch.int64, device=q.device)
    word = (t << shifts).sum(-1)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32).contiguous()


def permute_scales(s_group: torch.Tensor, s_channel: torch.Tensor, N: int, per_channel: bool):
    gp, sp = (t.to(s_channel.device) for t in _scale_perms())
    s_channel = s_channel.reshape(-1, sp.numel())[:, sp].reshape(-1, N).contiguous()
    if not per_channel:
        s_group = s_group.reshape(-1, gp.numel())[:, gp].reshape(-1, N).contiguous()
    return s_group, s_channel


@torch.no_grad()
def quantize_w4(w: torch.Tensor, group_size: int = -1):
    """w: float (K, N).  Returns (w_ref, q, s_group, s_channel) un-permuted, following the QQQ scheme:
    per-group: 4-bit asymmetric-offset codes 0..15 with fp16 group scales, then an int8 view per channel;
    per-channel: signed 4-bit codes, channel scale pre-divided by 16 (the kernel reads the nibble in the
    high half of a byte)."""
    K, N = w.shape
    assert group_size in GROUP_SIZES or group_size == K
    if group_size == -1:
        group_size = K
    if group_size < K:
        wg = w.reshape(K // group_size, group_size, N)
        s_group = wg.abs().amax(dim=1, keepdim=True) * (2.0 / 15.0)
        q = torch.clamp(torch.round(wg / s_group).int() + 8, 0, 15)
        w_ref = (q - 8).to(torch.float16) * s_group
        q = q.reshape(K, N)
        w_ref = w_ref.reshape(K, N)
        s_channel = w_ref.abs().amax(dim=0, keepdim=True) / 127.0
        t = (w_ref / s_channel).round().clamp(-128, 127).to(torch.int8)
        w_ref = t.to(torch.float16) * s_channel
        s_channel = s_channel.reshape(1, -1).float()
        s_group = (s_group.reshape(-1, N) / s_channel).to(torch.float16)
    else:
        s_channel = w.abs().amax(dim=0, keepdim=True) / 7.0
        q = torch.clamp(torch.round(w / s_channel).int(), -7, 7)
        w_ref = q.to(torch.float16) * s_channel
        s_group = torch.tensor([], dtype=torch.float16, device=w.device)
        s_channel = (s_channel / 16.0).reshape(-1, N).float()
    return w_ref, q, s_group, s_channel


@torch.no_grad()
def w4a8_quantize(w: torch.Tensor, num_bits: int = 4, group_size: int = -1, s_group=None, s_channel=None,
                  out_scales=None, pad_out: int = 0):
    """Quantise (or, when s_group / s_channel are given, re-encode an already fake-quantised) weight
    (K, N) and pack it.  Returns [w_ref, packed int32, s_group (permuted), s_channel (permuted)] with the
    meaning of the reference's function of the same name (quamba/marlin_utils.py:220-279)."""
    assert num_bits == 4, "only 4-bit weights are packed"
    K, N = w.shape
    if group_size == -1:
        group_size = K
    per_channel = group_size == K
    if s_group is None or s_channel is None:
        w_ref, q, s_group, s_channel = quantize_w4(w, group_size)
    else:
        w_ref = w.clone()
        q = torch.clamp((w.reshape(-1, group_size, N) / s_group.unsqueeze(1) + 8).round().int(), 0, 15).reshape(K, N)
        s_channel = s_channel.float()
        s_group = torch.nan_to_num((s_group.reshape(-1, N) / s_channel).to(torch.float16), nan=0.0)
    if out_scales is not None:
        s_channel = s_channel / out_scales.to(s_channel.device).float()
    if pad_out:
        F = torch.nn.functional
        w_ref = F.pad(w_ref, (0, pad_out))
        q = F.pad(q, (0, pad_out))
        if not per_channel:
            s_group = F.pad(s_group, (0, pad_out))
        s_channel = F.pad(s_channel, (0, pad_out), value=1e-6)
        N += pad_out
    packed = pack_int4(q, per_channel)       # on the weight's device: the index arithmetic is the same on CPU and GPU
    s_group, s_channel = permute_scales(s_group, s_channel, N, per_channel)
    return [t.to(w.device) for t in (w_ref, packed, s_group, s_channel)]


def unpack_int4(packed: torch.Tensor, K: int, N: int, per_channel: bool) -> torch.Tensor:
    """Inverse of :func:`pack_int4`: int32 (K/16, N*2) -> integer codes (K, N), 0..15 (per-group) or -8..7
    (per-channel)."""
    dev = packed.device
    shifts = 4 * torch.arange(8, dtype=torch.int64, device=dev)
    t = ((packed.to(torch.int64)[..., None] >> shifts) & 0xF).reshape(K // TILE, N * TILE)
    perm = _weight_perm(per_channel).to(dev)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=dev)
    t = t.reshape(-1, perm.numel())[:, inv].reshape(K // TILE, N // TILE, TILE, TILE).permute(0, 2, 1, 3).reshape(K, N)
    if per_channel:
        t = torch.where(t >= 8, t - 16, t)
    return t.to(torch.int32)


def unpermute_scales(s_group: torch.Tensor, s_channel: torch.Tensor, N: int, per_channel: bool):
    """Inverse of :func:`permute_scales`: natural column order."""
    gp, sp = (t.to(s_channel.device) for t in _scale_perms())
    inv_sp = torch.empty_like(sp); inv_sp[sp] = torch.arange(sp.numel(), device=sp.device)
    s_channel = s_channel.reshape(-1, sp.numel())[:, inv_sp].reshape(-1, N).contiguous()
    if not per_channel:
        inv_gp = torch.empty_like(gp); inv_gp[gp] = torch.arange(gp.numel(), device=gp.device)
        s_group = s_group.reshape(-1, gp.numel())[:, inv_gp].reshape(-1, N).contiguous()
    return s_group, s_channel


def repack(q: torch.Tensor, s_group: torch.Tensor, s_channel: torch.Tensor, per_channel: bool, pad_to: int = 64):
    """Codes (K, N) + natural-order scales -> the packed buffers of a (possibly sliced) weight, N padded to a multiple
    of ``pad_to`` with zero weights and 1e-6 channel scales as the reference pads (quamba/marlin_utils.py:258-263)."""
    K, N = q.shape
    pad = (pad_to - N % pad_to) % pad_to
    if pad:
        F = torch.nn.functional
        q = F.pad(q, (0, pad), value=0 if per_channel else 8)
        s_channel = F.pad(s_channel, (0, pad), value=1e-6)
        if not per_channel:
            s_group = F.pad(s_group, (0, pad))
        N += pad
    packed = pack_int4(q, per_channel)
    s_group, s_channel = permute_scales(s_group, s_channel, N, per_channel)
    return packed, s_group, s_channel, pad
