"""The exchange step of a head-parallel layer over peer memory (one process per GPU on one node).

Every rank allocates one region through the library (``qb_peer_alloc``), the 64-byte CUDA IPC handles travel through
``torch.distributed`` and every rank maps its peers' regions (``qb_peer_open``).  All ranks lay their regions out the same
way, so an offset names the same buffer on every rank.  Data moves with copy-engine transfers issued on a side stream
(``qb_peer_put``: no multiprocessor is used), a flag that only grows tells the receiver that a piece has landed, and the
receiver's compute stream passes a one-warp, time-bounded wait (``qb_peer_wait``) before it reads.  The reference has no
tensor parallelism (quamba/qMamba2.py:84-88); this module serves :class:`quamba_b200.parallel.HeadParallelStack`.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib

__all__ = ["PeerRegion", "LayerExchange", "sum_partials"]

MAX_PEERS = 16


class _DeviceBytes:
    """A span of device memory behind the CUDA array interface, so that torch can view it without a copy."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _bind():
    L = _lib.lib()
    if getattr(L, "_peer_bound", False):
        return L
    vp, i32, i64, u32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint32
    L.qb_peer_alloc.argtypes = [i64, ctypes.POINTER(vp), ctypes.c_char_p]
    L.qb_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.qb_peer_close.argtypes = [vp]
    L.qb_peer_free.argtypes = [vp]
    L.qb_peer_put.argtypes = [vp, vp]
    L.qb_peer_wait.argtypes = [vp, i32, u32, i32, vp]
    L.qb_sum_partials.argtypes = [vp, i32, i64, vp, i64, vp]
    L._peer_bound = True
    return L


def sum_partials(partials, out=None):
    """partials (n, ...) fp16 with contiguous trailing dims -> fp16 (...): the fp32 sum over the first dim, rounded once."""
    assert partials.is_cuda and partials.dtype == torch.float16 and partials.dim() >= 2
    assert partials[0].is_contiguous(), "every partial must be contiguous"
    n = partials[0].numel()
    if out is None:
        out = torch.empty(partials.shape[1:], dtype=torch.float16, device=partials.device)
    assert out.is_contiguous() and out.numel() == n and out.dtype == torch.float16
    with torch.cuda.device(partials.device):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_bind().qb_sum_partials(partials.data_ptr(), partials.shape[0], partials.stride(0), out.data_ptr(), n, st))
    return out


class PeerRegion:
    """``nbytes`` of this rank's device memory that every rank of ``group`` can write, plus the mappings of the peers'
    regions.  ``base[q]`` is rank q's region as an address valid in THIS process.  With ``world == 1`` nothing is
    exchanged (the region is still a library allocation, which is what a single-process test uses)."""

    def __init__(self, nbytes, rank, world, device, group=None):
        assert 1 <= world <= MAX_PEERS
        self.nbytes, self.rank, self.world, self.device, self.group = int(nbytes), rank, world, torch.device(device), group
        L = _bind()
        ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        self.base = [None] * world
        self._opened, self._bytes = [], None
        # Every rank goes through the same sequence of collectives whatever happens locally, and all ranks raise together:
        # a caller may then choose another exchange on every rank at once.
        err = None
        try:
            with torch.cuda.device(self.device):
                _lib.check(L.qb_peer_alloc(self.nbytes, ctypes.byref(ptr), handle))
            self.base[rank] = ptr.value
            self._bytes = torch.as_tensor(_DeviceBytes(ptr.value, self.nbytes))
            assert self._bytes.data_ptr() == ptr.value and self._bytes.device == self.device, (self._bytes.device, self.device)
        except Exception as e:  # noqa: BLE001
            err = f"rank {rank}: {type(e).__name__}: {e}"
        if world > 1:
            infos = [None] * world
            dist.all_gather_object(infos, (handle.raw, err), group=group)
            err = next((i[1] for i in infos if i[1]), None)
            if err is None:
                try:
                    for q in range(world):
                        if q == rank:
                            continue
                        p = ctypes.c_void_p()
                        with torch.cuda.device(self.device):
                            _lib.check(L.qb_peer_open(infos[q][0], ctypes.byref(p)))
                        self.base[q] = p.value
                        self._opened.append(p.value)
                except Exception as e:  # noqa: BLE001
                    err = f"rank {rank}: {type(e).__name__}: {e}"
                errs = [None] * world
                dist.all_gather_object(errs, err, group=group)
                err = next((e for e in errs if e), None)
        if err is not None:
            self._release()
            raise RuntimeError(f"peer memory set-up failed ({err})")

    def _release(self):
        L = _bind()
        self._bytes = None
        if self._opened or self.base[self.rank] is not None:
            with torch.cuda.device(self.device):
                for p in self._opened:
                    L.qb_peer_close(p)
                if self.base[self.rank] is not None:
                    L.qb_peer_free(self.base[self.rank])
        self.base, self._opened = None, []

    def local(self, offset, shape, dtype):
        """A view of this rank's own region."""
        n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        assert offset % 16 == 0 and offset + n <= self.nbytes
        return self._bytes[offset:offset + n].view(dtype).view(shape)

    def close(self):
        """Synchronises the device, takes the peers' mappings down, waits for every rank to have done so, frees the region."""
        if self.base is None:
            return
        L = _bind()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._opened:
                _lib.check(L.qb_peer_close(p))
            if self.world > 1:
                dist.barrier(group=self.group)
            self._bytes = None
            _lib.check(L.qb_peer_free(self.base[self.rank]))
        self.base, self._opened = None, []


def _put(args, stream):
    _lib.check(_bind().qb_peer_put(ctypes.addressof(args), stream))


class LayerExchange:
    """Buffers, flags and the two transfers of a token-sharded layer exchange, for ``n_chunks`` chunks of ``rows`` token
    rows of width ``d`` (``rows`` divisible by the number of ranks T; rank r owns rows [r * rows / T, (r + 1) * rows / T)):

    * ``put_partials``: this rank's fp16 partial layer output (rows, d) is cut by owner and piece q lands in slot
      ``recv[c][rank]`` of rank q; the owner sums its T slots (``reduce``): the reduce-scatter half;
    * ``put_rows``: this rank's normalised int8 rows land at their place in every rank's ``rows_int8[c]``: the
      all-gather half.

    Each put raises one flag per destination (a counter the caller advances once per layer); ``wait_partials`` /
    ``wait_rows`` hold the CURRENT stream until all T flags of the chunk have reached the value.  A put is issued behind
    an event of the stream that produced its source, on one high-priority stream per destination, so that the pieces of
    one put travel on several copy engines at once."""

    def __init__(self, rank, world, rows, d, n_chunks, device, group=None, timeout_ms=20000):
        assert rows % world == 0 and (rows // world * d) % 16 == 0
        self.rank, self.world, self.rows, self.d, self.n, self.timeout_ms = rank, world, rows, d, n_chunks, int(timeout_ms)
        self.per = rows // world
        self._recv_b, self._rows_b, self._flag_b = rows * d * 2, rows * d, 256
        self._chunk_b = self._recv_b + self._rows_b + self._flag_b
        self.region = PeerRegion(self._chunk_b * n_chunks, rank, world, device, group)
        T, per = world, self.per
        self.recv = [self.region.local(c * self._chunk_b, (T, per, d), torch.float16) for c in range(n_chunks)]
        self.rows_int8 = [self.region.local(c * self._chunk_b + self._recv_b, (rows, d), torch.int8) for c in range(n_chunks)]
        self._flags = [self.region.local(c * self._chunk_b + self._recv_b + self._rows_b, (64,), torch.int32) for c in range(n_chunks)]
        # flags of a chunk: words [0, T) raised by put_partials (word = source rank), words [32, 32 + T) by put_rows
        self._args_partials, self._args_rows = [], []
        for c in range(n_chunks):
            off = c * self._chunk_b
            a = _lib.make("qb_peer_put_args", n=T, self=rank, src_stride_bytes=per * d * 2, bytes=per * d * 2)
            b = _lib.make("qb_peer_put_args", n=T, self=rank, src_stride_bytes=0, bytes=per * d)
            for q in range(T):
                base = self.region.base[q]
                a.dst[q] = base + off + rank * per * d * 2
                a.flag[q] = base + off + self._recv_b + self._rows_b + 4 * rank
                b.dst[q] = base + off + self._recv_b + rank * per * d
                b.flag[q] = base + off + self._recv_b + self._rows_b + 4 * (32 + rank)
            self._args_partials.append(a)
            self._args_rows.append(b)
        with torch.cuda.device(self.region.device):
            self.streams = [torch.cuda.Stream(priority=-1) for _ in range(T)]
        for args in self._args_partials + self._args_rows:
            for q in range(T):
                args.stream_of[q] = self.streams[q].cuda_stream

    def _issue(self, args, src, value, own):
        """Behind everything queued so far on the current stream (the producer of ``src``).  ``own`` False: this rank's own
        piece is not copied (its consumer reads it where it is); the own flag is raised all the same."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.region.device))
        args.src, args.value, args.after_event = src.data_ptr(), value & 0xFFFFFFFF, ev.cuda_event
        keep = args.dst[self.rank]
        if not own:
            args.dst[self.rank] = None
        try:
            _put(args, self.streams[self.rank].cuda_stream)
        finally:
            args.dst[self.rank] = keep
        for st in self.streams:
            src.record_stream(st)

    def put_partials(self, c, partial, value, own=True):
        """partial: (rows, d) fp16 contiguous, produced on the current stream."""
        assert partial.dtype == torch.float16 and partial.is_contiguous() and partial.numel() == self.rows * self.d
        self._issue(self._args_partials[c], partial, value, own)

    def put_rows(self, c, q_rows, value, own=True):
        """q_rows: (rows / T, d) int8 contiguous, this rank's rows, produced on the current stream (``own=False`` when it
        already is this rank's row block of ``rows_int8[c]``)."""
        assert q_rows.dtype == torch.int8 and q_rows.is_contiguous() and q_rows.numel() == self.per * self.d
        self._issue(self._args_rows[c], q_rows, value, own)

    def _wait(self, c, first_word, value):
        f = self._flags[c]
        st = torch.cuda.current_stream(f.device).cuda_stream
        _lib.check(_bind().qb_peer_wait(f.data_ptr() + 4 * first_word, self.world, value & 0xFFFFFFFF, self.timeout_ms, st))

    def wait_partials(self, c, value):
        self._wait(c, 0, value)

    def wait_rows(self, c, value):
        self._wait(c, 32, value)

    def reduce(self, c, out=None):
        """The sum of the T received slots of chunk ``c``: (rows / T, d) fp16."""
        return sum_partials(self.recv[c], out)

    def close(self):
        self.recv = self.rows_int8 = self._flags = None
        self.region.close()
