"""The exchange step over peer memory (quamba_b200/peer.py; qb_peer_* and qb_sum_partials in the C ABI).

One process and one GPU cover the pieces: the reduction of the received slots (bit-exact against the same fp32 sum in
torch), puts and flags into the rank's own region, a wait that passes, and a wait whose flag nobody raises, which must
run out, leave its code in the device status word and leave the context usable.  Two processes on two GPUs (skipped with
fewer) run a small head-parallel model with the exchange moved by copy engines and by NCCL and must agree bit for bit
(two ranks: one fp16 addition per element either way).
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


@pytest.mark.parametrize("n,shape", [(1, (4, 64)), (2, (37, 4096)), (3, (5, 24)), (8, (300, 512)), (9, (3, 40)), (4, (7, 13))])
def test_sum_partials_is_the_fp32_sum_rounded_once(n, shape):
    _cuda()
    from quamba_b200.peer import sum_partials
    g = torch.Generator().manual_seed(n)
    x = (torch.randn((n,) + shape, generator=g) * 3).half().cuda()
    got = sum_partials(x)
    acc = torch.zeros(shape, dtype=torch.float32, device="cuda")
    for p in range(n):
        acc = acc + x[p].float()
    assert torch.equal(got, acc.half())


@pytest.mark.parametrize("n,rows,d,own_i", [(2, 33, 4096, 0), (4, 17, 2560, 3), (8, 9, 4096, 5), (3, 5, 200, None), (2, 4, 100, 1)])
def test_block_norm_sums_the_partial_slots_itself(n, rows, d, own_i):
    """QRMSNorm with ``partials``: the input is the fp16-rounded fp32 sum of the slots (one of them read from a tensor of
    its own) -- bit-identical to sum_partials followed by the plain norm, residual stream and int8 rows written in place."""
    _cuda()
    from quamba_b200.norm import QRMSNorm
    from quamba_b200.peer import sum_partials
    g = torch.Generator().manual_seed(n * 100 + rows)
    slots = (torch.randn(n, rows, d, generator=g) * 2).half().cuda()
    res = torch.randn(rows, d, generator=g).cuda()
    norm = QRMSNorm(d, eps=1e-5, device="cuda")
    norm.weight.data = (1 + 0.1 * torch.randn(d, generator=g)).half().cuda()
    norm.output_scale = 0.05
    own = None
    full = slots.clone()
    if own_i is not None:
        own = full[own_i].clone()
        slots[own_i].fill_(777.0)          # the slot of the own piece must not be read
    want_q, want_res = norm(sum_partials(full), residual=res, prenorm=True, residual_in_fp32=True)
    out = torch.zeros(rows + 2, d, dtype=torch.int8, device="cuda")
    got_q, got_res = norm(slots[0], residual=res, prenorm=True, residual_in_fp32=True,
                          partials=(slots, own_i if own_i is not None else 0, own), out=out[1:-1])
    assert got_q.data_ptr() == out[1:-1].data_ptr()
    assert torch.equal(got_q, want_q) and torch.equal(got_res, want_res)
    assert out[0].abs().max().item() == 0 and out[-1].abs().max().item() == 0


def test_puts_flags_and_waits_inside_one_process():
    _cuda()
    from quamba_b200 import _lib
    from quamba_b200.peer import LayerExchange
    ex = LayerExchange(0, 1, rows=64, d=256, n_chunks=2, device="cuda:0", timeout_ms=2000)
    try:
        g = torch.Generator().manual_seed(0)
        for value in (1, 2, 3):
            for c in range(2):
                q = torch.randint(-128, 128, (64, 256), generator=g, dtype=torch.int32).to(torch.int8).cuda()
                part = torch.randn(64, 256, generator=g).half().cuda()
                ex.put_rows(c, q, value)
                ex.put_partials(c, part, value)
                ex.wait_rows(c, value)
                ex.wait_partials(c, value)
                assert torch.equal(ex.rows_int8[c], q)
                assert torch.equal(ex.reduce(c), part)
        # a flag that is already past the value lets the waiter through at once (counters only grow)
        ex.wait_rows(0, 1)
        # own=False: this rank's piece is not copied, its flag is raised all the same
        before = ex.recv[0].clone()
        ex.put_partials(0, before[0] + 1, 4, own=False)
        ex.wait_partials(0, 4)
        assert torch.equal(ex.recv[0], before)
        torch.cuda.synchronize()
        _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
    finally:
        ex.close()


def test_a_wait_nobody_answers_runs_out_and_reports():
    _cuda()
    from quamba_b200 import _lib
    from quamba_b200.peer import LayerExchange, sum_partials
    ex = LayerExchange(0, 1, rows=16, d=64, n_chunks=1, device="cuda:0", timeout_ms=50)
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        ex.wait_rows(0, 7)            # nothing raises this flag
        ex.wait_partials(0, 7)        # the status word already holds an error: returns at once
        t1.record()
        with pytest.raises(RuntimeError, match="bounded device-side wait expired"):
            _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
        assert 40.0 <= t0.elapsed_time(t1) < 1000.0
        # the status word is clear again and the context still works
        _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
        x = torch.ones(2, 8, 64, dtype=torch.float16, device="cuda")
        assert torch.equal(sum_partials(x), torch.full((8, 64), 2.0, dtype=torch.float16, device="cuda"))
    finally:
        ex.close()


def _two_rank_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench_parallel as bp
    from quamba_b200 import _lib
    cfg = dict(d_model=512, n_layer=3, vocab_size=1000, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=8, chunk_size=256)
    stack = bp.Stack(cfg, rank, world, dev, calib_len=128, calib_seqs=2).runner()
    stack.peer_timeout_ms = 5000
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 1000, (4, 256), generator=g).to(dev)
    results = {}
    # the second peer pass runs on advanced flag counters, the third on four chunks (the skewed task order; the
    # exchange buffers are rebuilt for the new chunk size; chunking does not change any token's result)
    for name, chunk_seqs in (("nccl", 2), ("peer", 2), ("peer", 2), ("peer", 1)):
        stack.exchange = name
        logits = stack.prefill(ids, chunk_seqs)
        torch.cuda.synchronize()
        _lib.read_device_status(torch.cuda.current_stream().cuda_stream)
        results.setdefault(name, []).append(logits.cpu())
    dist.barrier()
    stack.close()
    torch.save(results, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_two_ranks_copy_engine_exchange_equals_the_nccl_exchange(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_two_rank_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in (0, 1))
    for r in (r0, r1):
        assert torch.isfinite(r["nccl"][0].float()).all()
        for got in r["peer"]:
            assert torch.equal(got, r["nccl"][0])
    assert torch.equal(r0["nccl"][0], r1["nccl"][0])
