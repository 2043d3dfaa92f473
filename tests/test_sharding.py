"""N > 1: the path shards by independent (batch, head) units with no data-path collective.

CPU: two gloo ranks each take their share of one seeded problem, run the oracle on it, and the gathered result
must equal the unsharded one; the control-plane reduction (max over ranks) is checked too.
GPU (one device): the ranks' shares are run one after the other through the CUDA path and must reproduce the
unsharded CUDA result bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import make_ssd_case
from oracle import ssd as ossd
from quamba_b200 import sharding as sh

BATCHED = ("q_x", "q_dt", "q_B", "q_C", "q_z")


def _oracle(c):
    return ossd.chunk_scan_faithful(c["q_x"], c["x_scales"], c["hgr"], c["dgr"], c["q_dt"], c["s_dt"], c["q_A_log"], c["s_A"],
                                    c["q_B"], c["s_B"], c["q_C"], c["s_C"], c["state_scale"], c["chunk"], c["q_D"], c["s_D"],
                                    c["q_z"], c["s_z"], c["dt_bias"], True)


def test_shard_range_is_a_balanced_partition():
    for n in (0, 1, 5, 80, 81, 320):
        for world in (1, 2, 3, 8):
            spans = [sh.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.shard_range(4, 2, 2)


def test_head_sharding_rules():
    c = make_ssd_case(1, 16, 8, 64, 2, 64, 64, seed=1)
    c["s_B"] = torch.tensor([0.1, 0.2]); c["s_C"] = torch.tensor([0.3, 0.4])
    s = sh.shard_ssd_heads(c, 1, 2)                       # 4 heads per rank = one whole group
    assert s["q_x"].shape[2] == 4 and s["q_B"].shape[2] == 1 and s["s_B"].tolist() == pytest.approx([0.2])
    s = sh.shard_ssd_heads(c, 3, 4)                       # 2 heads per rank, inside group 1
    assert s["q_x"].shape[2] == 2 and torch.equal(s["q_B"], c["q_B"][:, :, 1:2]) and torch.equal(s["q_A_log"], c["q_A_log"][6:8])
    with pytest.raises(ValueError):
        sh.shard_ssd_heads(c, 0, 3)
    g = make_ssd_case(1, 16, 8, 64, 2, 64, 64, grouped=True, seed=1)
    with pytest.raises(NotImplementedError):
        sh.shard_ssd_heads(g, 0, 2)
    assert sh.max_over_ranks([1.5, 2]) == [1.5, 2.0]       # no process group: identity


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        # by head: one batch spread over the ranks
        c = make_ssd_case(2, 96, 4, 64, 2, 64, 64, seed=7)
        y_loc, f_loc = _oracle(sh.shard_ssd_heads(c, rank, world))
        y = sh.gather_heads(y_loc, world, dim=2)
        f = sh.gather_heads(f_loc, world, dim=1)
        # by sequence, ragged: 3 sequences over 2 ranks
        c3 = make_ssd_case(3, 64, 2, 64, 1, 64, 64, seed=9)
        part = sh.shard_sequences(c3, rank, world, BATCHED)
        y3_loc, _ = _oracle(part)
        gathered = [None] * world
        dist.all_gather_object(gathered, y3_loc)
        times = sh.max_over_ranks([1.0 + rank, 5.0 - rank])
        dist.barrier()
        if rank == 0:
            y_full, f_full = _oracle(c)
            y3_full, _ = _oracle(c3)
            out.put(dict(head_y=torch.equal(y, y_full), head_f=torch.equal(f, f_full),
                         seq_sizes=[g.shape[0] for g in gathered], seq_y=torch.equal(torch.cat(gathered, 0), y3_full),
                         times=times))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    res = out.get()
    assert res["head_y"] and res["head_f"] and res["seq_y"]
    assert res["seq_sizes"] == [2, 1]
    assert res["times"] == [2.0, 5.0]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_sharded_cuda_path_equals_unsharded(world):
    from quamba_b200 import ops
    d = lambda t: None if t is None else t.to("cuda")

    def run(c):
        return ops._quant_mamba_chunk_scan_combined_fwd(
            d(c["q_x"]), d(c["x_scales"]), d(c["q_dt"]), d(c["s_dt"]), d(c["q_A_log"]), d(c["s_A"]), d(c["q_B"]), d(c["s_B"]),
            d(c["q_C"]), d(c["s_C"]), d(c["state_scale"]), c["chunk"], d(c["q_D"]), d(c["s_D"]), None, None, d(c["dt_bias"]),
            None, None, None, True)

    c = make_ssd_case(3, 300, 8, 64, 1, 128, 256, seed=13)
    y_full, f_full = run(c)
    ys, fs = zip(*(run(sh.shard_ssd_heads(c, r, world)) for r in range(world)))
    assert torch.equal(torch.cat(ys, dim=2), y_full) and torch.equal(torch.cat(fs, dim=1), f_full)
    ys, fs = zip(*(run(sh.shard_sequences(c, r, 2, BATCHED)) for r in range(2)))
    assert torch.equal(torch.cat(ys, dim=0), y_full) and torch.equal(torch.cat(fs, dim=0), f_full)
