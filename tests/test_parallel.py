"""Head-parallel sharding of the quantized Mamba2 layer: two gloo ranks on CPU cut the layer, each runs the oracle on its
shard, the partial outputs are all-reduced, and the sum must equal the oracle's output of the unsharded layer."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _layer(group, G=2, blocks=2):
    from quamba_b200 import calibrate as cal
    m = cal.Mamba2LMFloat(d_model=256, n_layer=1, vocab_size=64, ngroups=G, d_state=64, seed=7, w4_group_size=group, had_blocks=blocks)
    ids = torch.randint(0, 64, (2, 40), generator=torch.Generator().manual_seed(1))
    q = cal.quantize_model(m, cal.calibrate(m, [ids]))
    return q.backbone.layers[0].mixer


def _worker(rank, world, port, group, out_dir):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import model as omodel
    from quamba_b200.parallel import shard_mixer
    mixer = _layer(group)
    u = torch.randint(-127, 128, (2, 50, 256), generator=torch.Generator().manual_seed(3), dtype=torch.int8)
    shard = shard_mixer(mixer, rank, world)
    assert shard.nheads == mixer.nheads // world and shard.in_proj.in_features == 256
    part = omodel.mixer_forward(shard, u).float()
    dist.all_reduce(part)
    if rank == 0:
        torch.save(part, Path(out_dir) / "sum.pt")
    dist.destroy_process_group()


@pytest.mark.parametrize("group", [None, -1])
def test_two_rank_head_parallel_layer_matches_unsharded_oracle(group, tmp_path):
    from oracle import model as omodel
    port = 29650 + (0 if group is None else 1) + os.getpid() % 200
    mp.spawn(_worker, args=(2, port, group, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "sum.pt")
    mixer = _layer(group)
    u = torch.randint(-127, 128, (2, 50, 256), generator=torch.Generator().manual_seed(3), dtype=torch.int8)
    want = omodel.mixer_forward(mixer, u).float()
    # each rank rounds its partial product to fp16 before the sum; the unsharded layer rounds once
    assert (got - want).abs().max().item() <= 2e-3 * want.abs().max().item() + 1e-3


def test_shard_repacks_the_same_integers():
    from quamba_b200 import packing
    from quamba_b200.parallel import rank_columns, shard_w4a8_columns, shard_w4a8_rows
    m = _layer(None)
    q_full = packing.unpack_int4(m.in_proj.weight, m.in_proj.size_k, m.in_proj.size_n, False)
    cols = torch.cat(rank_columns(m, 1, 2))
    sh = shard_w4a8_columns(m.in_proj, cols)
    q_sh = packing.unpack_int4(sh.weight, sh.size_k, sh.size_n, False)
    assert torch.equal(q_sh[:, :cols.numel()], q_full[:, cols]) and sh.out_features == cols.numel()
    half = m.out_proj.in_features // 2
    r0, r1 = shard_w4a8_rows(m.out_proj, 0, half), shard_w4a8_rows(m.out_proj, half, 2 * half)
    q_out = packing.unpack_int4(m.out_proj.weight, m.out_proj.size_k, m.out_proj.size_n, False)
    assert torch.equal(torch.cat([packing.unpack_int4(r.weight, r.size_k, r.size_n, False) for r in (r0, r1)]), q_out)
    assert torch.equal(r0.s_channel, m.out_proj.s_channel)


def _peer_setup_worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from quamba_b200.peer import PeerRegion
    try:
        PeerRegion(4096, rank, world, "cuda:0")
        outcome = "mapped"
    except RuntimeError as e:
        outcome = str(e)
    dist.barrier()              # both ranks are still in step: the set-up ran the same collectives on each
    (Path(out_dir) / f"peer{rank}.txt").write_text(outcome)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.is_available(), reason="the failing set-up needs a machine without a GPU")
def test_peer_memory_setup_fails_on_every_rank_together(tmp_path):
    """Without a GPU the region cannot be allocated: every rank must raise the same error after the same collectives
    (a caller then moves all ranks to the NCCL exchange), never one rank ahead of the other."""
    port = 29870 + os.getpid() % 100
    mp.spawn(_peer_setup_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = ((tmp_path / f"peer{r}.txt").read_text() for r in (0, 1))
    assert a.startswith("peer memory set-up failed") and a == b


@pytest.mark.parametrize("n_layers,n_chunks,lag", [(1, 1, None), (3, 1, 2), (4, 2, None), (5, 3, 1), (5, 4, None), (5, 4, 1), (5, 4, 3),
                                                    (3, 8, None), (3, 8, 7), (2, 4, 9)])
def test_peer_task_order_respects_the_data_flow(n_layers, n_chunks, lag):
    """Every task exactly once; the norm of a (layer, chunk) before its shard; a shard before the norm that consumes its
    partial output one layer later; and the skew: ``lag`` shard tasks between a partial output and its norm."""
    from quamba_b200.parallel import peer_task_order
    order = peer_task_order(n_layers, n_chunks, lag)
    pos = {t: i for i, t in enumerate(order)}
    n = n_chunks
    assert len(order) == len(pos) == (2 * n_layers + 1) * n
    assert set(pos) == {("A", k) for k in range((n_layers + 1) * n)} | {("B", k) for k in range(n_layers * n)}
    for k in range(n_layers * n):
        assert pos[("A", k)] < pos[("B", k)]
        assert pos[("B", k)] < pos[("A", k + n)]
    if n > 1 and n_layers >= 3:
        eff = min(max(1, n // 2 if lag is None else lag), n - 1)
        k = 2 * n + 1
        between = lambda a, b: sum(1 for t in order[pos[a] + 1:pos[b]] if t[0] == "B")
        assert between(("B", k - n), ("A", k)) == eff
        assert between(("A", k), ("B", k)) == n - eff - 1
