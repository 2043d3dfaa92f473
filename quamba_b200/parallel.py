"""Head-parallel Mamba2 layers across the GPUs of one node: in_proj column-parallel by SSD group, conv / SSD / gated
norm local to a rank's heads, a block-diagonal Hadamard rotation, out_proj row-parallel, and ONE all-reduce (sum) of the
(tokens, d_model) fp16 layer output per layer over NCCL.

The reference has no tensor parallelism (its mixers assert ``process_group is None``, quamba/qMamba2.py:84-88); the cut
follows how its layer is organised: the in_proj columns are [z | x | B | C | dt] (qMamba2.py:798-800), B / C and the gated
norm are per SSD group (norm group size d_ssm / ngroups), so a rank that owns whole groups needs nothing from its peers
until out_proj's contraction over d_inner.  The out_proj input rotation becomes I_T (x) H_{d_inner / T}: a model meant to
be served this way is quantised with that block rotation (``QHadamard(blocks=T)``), and its single-GPU form computes
exactly the same function.

Shards are cut from the quantised layer: int4 codes and scales are unpacked, sliced and re-packed, so every rank multiplies
with the very integers of the unsharded layer (a per-rank re-quantisation would change the channel scales).
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib
from . import packing
from .mixer import W4A8QMamba2, _QMamba2
from .modules import QHadamard, Quamb2Conv1D, Quamba2ChunkScan, W4A8B8O8LinearParallel, W4A8B16O16Linear
from .norm import QRMSNormGated

__all__ = ["shard_w4a8_columns", "shard_w4a8_rows", "shard_mixer", "HeadParallelMixer", "HeadParallelStack", "rank_columns",
           "peer_task_order"]


def _codes(lin):
    per_channel = lin.s_group.numel() == 0
    q = packing.unpack_int4(lin.weight, lin.size_k, lin.size_n, per_channel)
    sg, sc = packing.unpermute_scales(lin.s_group, lin.s_channel, lin.size_n, per_channel)
    return q, sg, sc, per_channel


def _rebuild(cls, q, sg, sc, per_channel, in_features, out_features, input_scale, device):
    packed, sg, sc, pad = packing.repack(q, sg, sc, per_channel)
    lin = cls(in_features, out_features, group_size=128, device=device)
    assert lin.pad_out == pad and lin.size_n == out_features + pad
    lin.weight, lin.s_channel, lin.input_scale = packed, sc, input_scale.clone()
    lin.s_group = sg if not per_channel else torch.empty(0, dtype=torch.float16, device=device)
    return lin


def shard_w4a8_columns(lin, cols: torch.Tensor):
    """The linear layer that produces output columns ``cols`` (a 1-D index tensor) of ``lin``."""
    q, sg, sc, pc = _codes(lin)
    cols = cols.to(q.device)
    return _rebuild(type(lin), q[:, cols], sg if pc else sg[:, cols], sc[:, cols], pc, lin.in_features, cols.numel(),
                    lin.input_scale, q.device)


def shard_w4a8_rows(lin, k0: int, k1: int):
    """The linear layer that contracts input features [k0, k1) of ``lin`` (a partial sum of its output)."""
    q, sg, sc, pc = _codes(lin)
    assert pc or (k0 % 128 == 0 and k1 % 128 == 0), "row cuts must fall on weight-group boundaries"
    out = lin.out_features
    return _rebuild(type(lin), q[k0:k1, :out], sg if pc else sg[k0 // 128:k1 // 128, :out], sc[:, :out], pc, k1 - k0, out,
                    lin.input_scale, q.device)


def rank_columns(m, rank, world):
    """Column indices of in_proj ([z | x | B | C | dt]) that rank ``rank`` of ``world`` owns, as five index ranges."""
    G, N, D, H = m.ngroups, m.d_state, m.d_ssm, m.nheads
    assert G % world == 0, "head parallelism cuts by SSD group: ngroups must be divisible by the number of ranks"
    d, gn, h = D // world, G // world * N, H // world
    z0, x0, b0, c0, t0 = 0, D, 2 * D, 2 * D + G * N, 2 * D + 2 * G * N
    return [torch.arange(z0 + rank * d, z0 + (rank + 1) * d), torch.arange(x0 + rank * d, x0 + (rank + 1) * d),
            torch.arange(b0 + rank * gn, b0 + (rank + 1) * gn), torch.arange(c0 + rank * gn, c0 + (rank + 1) * gn),
            torch.arange(t0 + rank * h, t0 + (rank + 1) * h)]


@torch.no_grad()
def shard_mixer(m: W4A8QMamba2, rank: int, world: int):
    """Rank ``rank``'s share of a W4A8QMamba2 whose Hadamard rotation has ``world`` blocks (or a multiple)."""
    blocks = getattr(m.had, "blocks", 1)
    assert blocks % world == 0, "quantise the model with QHadamard(blocks=T) for T-way head parallelism"
    dev = m.out_proj.weight.device
    T = world
    D, H, G, N, P = m.d_ssm // T, m.nheads // T, m.ngroups // T, m.d_state, m.headdim
    parts = rank_columns(m, rank, T)
    s = _QMamba2.__new__(W4A8QMamba2)
    nn.Module.__init__(s)
    for k in ("d_model", "d_state", "d_conv", "conv_init", "expand", "headdim", "D_has_hdim", "rmsnorm", "norm_before_gate",
              "dt_limit", "activation", "chunk_size", "use_mem_eff_path", "layer_idx", "sequence_parallel"):
        setattr(s, k, getattr(m, k))
    s.process_group, s.world_size, s.local_rank = None, T, rank
    s.d_inner = s.d_ssm = D
    s.ngroups, s.nheads = G, H
    s.in_proj = shard_w4a8_columns(m.in_proj, torch.cat(parts))
    s.out_proj = shard_w4a8_rows(m.out_proj, rank * D, (rank + 1) * D)
    # conv1d: channels [x | B | C] of this rank's groups
    c = m.conv1d
    ch = (torch.cat(parts[1:4]) - m.d_ssm).to(dev)          # conv channel c is in_proj column d_ssm + c
    grouped = c.x_head_group_range is not None
    sc = Quamb2Conv1D(D, P, N, G, c.x_nhead_group if grouped else 0, c.x_ndim_group if grouped else 0, ch.numel(), ch.numel(),
                      c.kernel_size, groups=ch.numel(), padding=c.padding, bias=c.bias, device=dev)
    sc.weight, sc.bias = c.weight[ch].contiguous(), None if c.bias is None else c.bias[ch].contiguous()
    for k in sc._float_names():
        setattr(sc, k, getattr(c, k))
    gs = slice(rank * G, (rank + 1) * G)
    if grouped:
        sc.x_head_group_range, sc.x_dim_group_range = c.x_head_group_range[gs].contiguous(), c.x_dim_group_range[gs].contiguous()
        sc.x_out_scales, sc.B_out_scales, sc.C_out_scales = (t[gs].contiguous() for t in (c.x_out_scales, c.B_out_scales, c.C_out_scales))
    else:
        sc.x_out_scales, sc.B_out_scales, sc.C_out_scales = c.x_out_scales, c.B_out_scales, c.C_out_scales
    s.conv1d = sc
    # SSD: heads of this rank
    q = m.qchunk_scan
    hs = slice(rank * H, (rank + 1) * H)
    ss = Quamba2ChunkScan(D, P, N, G, q.D_has_hdim, q.chunk_size, q.nhead_groups, q.ndim_groups, q.delta_softplus, dt_limit=q.dt_limit,
                          device=dev)
    ss.dt_bias, ss.A_log, ss.A_log_scale = q.dt_bias[hs].contiguous(), q.A_log[hs].contiguous(), q.A_log_scale
    ss.D = q.D.reshape(m.nheads, -1)[hs].reshape(-1).contiguous() if q.D is not None else None
    ss.D_scale, ss.dt_scale, ss.z_scale = q.D_scale, q.dt_scale, q.z_scale
    if q.grouped:
        ss.x_scales, ss.ssm_state_scale = q.x_scales[gs].contiguous(), q.ssm_state_scale[gs].contiguous()
        ss.x_head_group_range, ss.x_dim_group_range = q.x_head_group_range[gs].contiguous(), q.x_dim_group_range[gs].contiguous()
        ss.B_scale, ss.C_scale = q.B_scale[gs].contiguous(), q.C_scale[gs].contiguous()
    else:
        ss.x_scales, ss.ssm_state_scale, ss.B_scale, ss.C_scale = q.x_scales, q.ssm_state_scale, q.B_scale, q.C_scale
    s.qchunk_scan = ss
    n = m.norm
    sn = QRMSNormGated(D, eps=n.eps, group_size=n.group_size, norm_before_gate=n.norm_before_gate, use_float16_output=True, device=dev)
    sn.weight, sn.z_scale, sn.output_scale = n.weight[rank * D:(rank + 1) * D].contiguous(), n.z_scale, n.output_scale
    s.norm = sn
    s.had = QHadamard(D, x_H_scale=m.had.x_H_scale, blocks=blocks // T)
    return s


def peer_task_order(n_layers, n_chunks, lag=None):
    """The issue order of the peer-memory prefill's tasks as a list of ("A" | "B", k), k = layer * n_chunks + chunk.

    A(k) = [sum of the partial outputs of B(k - n_chunks) ->] block norm of layer k // n_chunks on chunk k % n_chunks, then the
    put of its int8 rows (k up to n_layers * n_chunks + n_chunks - 1: the last n_chunks only sum the last layer's output);
    B(k) = the layer shard on the gathered rows of A(k), then the put of its partial output.  The order keeps A(k) before
    B(k) and B(k - n_chunks) before A(k), and skews the two so that a transfer has other chunks' compute to hide behind:
    A(k) comes ``lag`` B tasks after B(k - n_chunks) and B(k) comes n_chunks - lag - 1 B tasks after A(k)
    (``lag`` None: half the chunks; clipped to [1, n_chunks - 1])."""
    n = n_chunks
    if lag is None:
        lag = max(1, n // 2)
    lead = max(1, n - min(max(1, lag), n - 1)) if n > 1 else 1
    total_a, total_b = (n_layers + 1) * n, n_layers * n
    order = [("A", k) for k in range(min(lead, total_a))]
    next_a = len(order)
    for j in range(total_b):
        order.append(("B", j))
        if j + lead < total_a:
            order.append(("A", j + lead))
            next_a = j + lead + 1
    order.extend(("A", k) for k in range(next_a, total_a))
    return order


class HeadParallelMixer(nn.Module):
    """A rank's shard plus the layer's one collective: forward returns the all-reduced (tokens, d_model) fp16 output.
    ``async_op=True`` returns (partial output tensor, work handle) so that a caller can overlap the reduction of one
    token chunk with the compute of the next."""

    def __init__(self, shard, process_group=None):
        super().__init__()
        self.shard, self.process_group = shard, process_group

    @torch.no_grad()
    def forward(self, u, async_op=False, **kwargs):
        out = self.shard(u, **kwargs)
        if not out.is_contiguous():
            out = out.contiguous()
        work = dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.process_group, async_op=async_op)
        return (out, work) if async_op else out


class HeadParallelStack:
    """A rank's share of a whole model for head-parallel prefill: replicated embedding, block norms, final norm and head,
    sharded mixers (:func:`shard_mixer`).  ``prefill`` runs the layers on chunks of sequences so that the collective of one
    chunk overlaps the compute of the next, in one of two forms of the layer's single exchange step:

    * ``token_sharded_norm = True`` (default): reduce-scatter of the fp16 partial outputs over the token rows, residual add
      + RMSNorm + quantise on this rank's rows only, all-gather of the int8 rows for the next in_proj;
    * ``False``: one fp16 all-reduce per layer, block norm replicated on every rank.

    ``exchange`` picks who moves the bytes of the token-sharded form: ``"nccl"`` (reduce-scatter / all-gather kernels on
    NCCL's stream) or ``"peer"`` (:class:`quamba_b200.peer.LayerExchange`: copy-engine puts into the peers' memory, flags,
    time-bounded waits and a local sum, no multiprocessor spent on the transfer).

    ``collective`` / ``compute`` switch the two halves off for separate timings (the results are then meaningless)."""

    def __init__(self, embedding, norms, shards, norm_f, lm_head, rank, world, d_model):
        self.embedding, self.norms, self.shards, self.norm_f, self.lm_head = embedding, norms, shards, norm_f, lm_head
        self.rank, self.world, self.d_model = rank, world, d_model
        self.dev = lm_head.weight.device
        self.token_sharded_norm = True
        self.early_overlap = True
        self.exchange = "nccl"
        self.peer_timeout_ms = 20000
        self.peer_lag = None           # B tasks between a partial output and the norm that consumes it (None: half the chunks)
        self._peer, self._peer_key, self._peer_epoch = None, None, 0

    def prefill(self, ids, chunk_seqs, collective=True, compute=True):
        with _lib.early_overlap(self.early_overlap), torch.no_grad():
            return self._prefill(ids, chunk_seqs, collective, compute)

    def _prefill(self, ids, chunk_seqs, collective=True, compute=True):
        if self.world > 1 and self.token_sharded_norm and self.exchange == "peer":
            return self._prefill_peer(ids, chunk_seqs, collective, compute)
        if self.world > 1 and self.token_sharded_norm:
            return self._prefill_token_sharded(ids, chunk_seqs, collective, compute)
        return self._prefill_allreduce(ids, chunk_seqs, collective, compute)

    def _prefill_token_sharded(self, ids, chunk_seqs, collective=True, compute=True):
        """The layer's all-reduce split into its two halves with the block norm between them: reduce-scatter of the fp16
        partial outputs over the token rows, residual add + RMSNorm + quantise on this rank's rows only (the residual
        stream stays sharded by rows), all-gather of the INT8 rows for the next in_proj.  Same sums as the all-reduce,
        3 instead of 4 bytes per element over NVLink, and the norm is no longer replicated on every rank."""
        T, rank = self.world, self.rank
        chunks = list(ids.split(chunk_seqs))
        n = len(chunks)
        d = self.d_model
        rows = chunks[0].numel()
        assert rows % T == 0
        per = rows // T
        mine = slice(rank * per, (rank + 1) * per)
        # embedding: every rank looks up its own rows only
        hs = [self.embedding(c.reshape(-1)[mine]) if compute else torch.empty((per, d), dtype=torch.float16, device=self.dev) for c in chunks]
        res = [None] * n
        partial = [None] * n
        q_full = [torch.empty((rows, d), dtype=torch.int8, device=self.dev) for _ in range(n)]
        pend_rs, pend_ag = [None] * n, [None] * n
        L = len(self.norms)
        for li, (norm, shard) in enumerate(zip(self.norms, self.shards)):
            for c in range(n):
                if pend_rs[c] is not None:
                    pend_rs[c].wait(); pend_rs[c] = None
                if compute:
                    q, res[c] = norm(hs[c], residual=res[c], prenorm=True, residual_in_fp32=True)
                else:
                    q = q_full[c][mine]
                if collective:
                    pend_ag[c] = dist.all_gather_into_tensor(q_full[c], q.contiguous(), async_op=True)
                else:
                    q_full[c][mine].copy_(q)
            for c in range(n):
                if pend_ag[c] is not None:
                    pend_ag[c].wait(); pend_ag[c] = None
                if compute:
                    partial[c] = shard(q_full[c].view(chunks[c].shape[0], -1, d)).reshape(rows, d)
                    if not partial[c].is_contiguous():
                        partial[c] = partial[c].contiguous()
                elif partial[c] is None:
                    partial[c] = torch.zeros((rows, d), dtype=torch.float16, device=self.dev)
                if collective:
                    hs[c] = torch.empty((per, d), dtype=torch.float16, device=self.dev)
                    pend_rs[c] = dist.reduce_scatter_tensor(hs[c], partial[c], async_op=True)
                else:
                    hs[c] = partial[c][mine]
        for c in range(n):
            if pend_rs[c] is not None:
                pend_rs[c].wait()
        if not compute:
            return None
        return self._last_token_logits(chunks, hs, res, per, collective)

    def _last_token_logits(self, chunks, hs, res, per, collective):
        """Last token of every sequence: its row lives on one rank; every rank fills its own rows of a small buffer and one
        tiny all-reduce gives all of them to everybody."""
        rank, d = self.rank, self.d_model
        seqlen = chunks[0].shape[1]
        lasts = []
        for c in range(len(chunks)):
            nseq = chunks[c].shape[0]
            buf_h = torch.zeros((nseq, d), dtype=torch.float32, device=self.dev)
            buf_r = torch.zeros((nseq, d), dtype=torch.float32, device=self.dev)
            for s_ in range(nseq):
                row = (s_ + 1) * seqlen - 1
                if rank * per <= row < (rank + 1) * per:
                    buf_h[s_] = hs[c][row - rank * per].float()
                    buf_r[s_] = res[c][row - rank * per]
            if collective:
                dist.all_reduce(buf_h); dist.all_reduce(buf_r)
            lasts.append(self.norm_f(buf_h.half()[:, None], residual=buf_r[:, None], prenorm=False, residual_in_fp32=True))
        return self.lm_head(torch.cat(lasts))[:, -1]

    def _peer_exchange(self, rows, n):
        from .peer import LayerExchange
        key = (rows, n)
        if self._peer_key != key:
            if self._peer is not None:
                self._peer.close()
            self._peer = LayerExchange(self.rank, self.world, rows, self.d_model, n, self.dev, timeout_ms=self.peer_timeout_ms)
            self._peer_key, self._peer_epoch = key, 0
            dist.barrier()                       # nobody puts before every rank has mapped every region
        return self._peer

    def close(self):
        if self._peer is not None:
            self._peer.close()
            self._peer = self._peer_key = None

    def _prefill_peer(self, ids, chunk_seqs, collective=True, compute=True):
        """The token-sharded exchange of :meth:`_prefill_token_sharded` with the bytes moved by copy engines.  Two kinds of
        task per (layer, chunk) on the compute stream:

        * A: [wait for the T partial pieces of the layer before -> sum them ->] residual add + norm + quantise of this
          rank's rows, then the put of the int8 rows into every rank's buffer;
        * B: wait for everybody's int8 rows -> the layer shard -> the put of the fp16 partial output's T row pieces into
          their owners' slots.

        The puts run on side streams behind an event of their producer.  Tasks are issued skewed, so that a transfer has the
        compute of other chunks to hide behind: with n chunks and k counting (layer, chunk) pairs in order, A(k) follows
        B(k - n + lag) and so comes ``lag`` B tasks after B(k - n), whose partial output it needs; B(k) comes n - lag - 1 B
        tasks after A(k), whose rows it needs.  A buffer is reused one layer later, and every reuse is ordered behind its last
        reader by the flags themselves: a peer can only put layer l + 1's rows after it has summed layer l's pieces, and only
        put layer l + 1's pieces after it has consumed layer l + 1's rows."""
        T, rank, d = self.world, self.rank, self.d_model
        chunks = list(ids.split(chunk_seqs))
        n = len(chunks)
        rows = chunks[0].numel()
        assert rows % T == 0 and all(c.numel() == rows for c in chunks)
        per = rows // T
        mine = slice(rank * per, (rank + 1) * per)
        ex = self._peer_exchange(rows, n)
        hs = [self.embedding(c.reshape(-1)[mine]) if compute else torch.empty((per, d), dtype=torch.float16, device=self.dev) for c in chunks]
        res = [None] * n
        L = len(self.norms)
        e0 = self._peer_epoch
        if collective:
            self._peer_epoch += L
        dummy_p = None
        if not compute:
            dummy_p = torch.zeros((rows, d), dtype=torch.float16, device=self.dev)

        held = [None] * n                  # a chunk's partial output stays alive until the next layer's norm has read this rank's piece

        def task_a(k):
            li, c = divmod(k, n)
            fused = None
            if li > 0 and collective:
                ex.wait_partials(c, e0 + li)
                if compute and li == L:    # past the last layer: only the sum of its output (its own piece was copied too)
                    hs[c] = ex.reduce(c)
                elif compute:              # the norm sums the T slots itself and reads this rank's piece where shard left it
                    hs[c], fused = ex.recv[c][0], (ex.recv[c], rank, held[c][mine])
            if li == L:
                return
            q = ex.rows_int8[c][mine]      # the int8 rows are written straight into this rank's block of the gathered buffer
            if compute:
                _, res[c] = self.norms[li](hs[c], residual=res[c], prenorm=True, residual_in_fp32=True, partials=fused, out=q)
            if collective:
                ex.put_rows(c, q, e0 + li + 1, own=False)

        def task_b(k):
            li, c = divmod(k, n)
            if collective:
                ex.wait_rows(c, e0 + li + 1)
            partial = None
            if compute:
                partial = self.shards[li](ex.rows_int8[c].view(chunks[c].shape[0], -1, d)).reshape(rows, d)
                if not partial.is_contiguous():
                    partial = partial.contiguous()
            if collective:
                held[c] = partial
                ex.put_partials(c, partial if compute else dummy_p, e0 + li + 1, own=li == L - 1)
            elif compute:
                hs[c] = partial[mine]

        for kind, k in peer_task_order(L, n, self.peer_lag):
            (task_a if kind == "A" else task_b)(k)
        if not compute:
            return None
        return self._last_token_logits(chunks, hs, res, per, collective)

    def _prefill_allreduce(self, ids, chunk_seqs, collective=True, compute=True):
        """ids (batch, L) on the device -> last-token logits (batch, vocab).  ``collective`` / ``compute`` switch the two
        halves off for the separate timings."""
        chunks = list(ids.split(chunk_seqs))
        n = len(chunks)
        h = [self.embedding(c) for c in chunks]
        res = [None] * n
        pending = [None] * n
        for norm, shard in zip(self.norms, self.shards):
            for c in range(n):
                if pending[c] is not None:
                    pending[c].wait()
                    pending[c] = None
                if compute:
                    q, res[c] = norm(h[c], residual=res[c], prenorm=True, residual_in_fp32=True)
                    h[c] = shard(q)
                if collective and self.world > 1:
                    if not h[c].is_contiguous():
                        h[c] = h[c].contiguous()
                    pending[c] = dist.all_reduce(h[c], async_op=True)
        for c in range(n):
            if pending[c] is not None:
                pending[c].wait()
        if not compute:
            return None
        last = torch.cat([self.norm_f(h[c][:, -1:], residual=res[c][:, -1:], prenorm=False, residual_in_fp32=True) for c in range(n)])
        return self.lm_head(last)[:, -1]
