"""Sharding over ranks: plan arithmetic, and the gather on two gloo ranks (CPU processes)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from twilight_b200.dist import gather_outputs, shard_units


def test_plans_tile_the_grid_exactly_once():
    for batch, hkv, world in [(16, 32, 8), (16, 32, 2), (128, 8, 8), (3, 8, 4), (6, 4, 8), (64, 8, 1)]:
        plan = shard_units(batch, hkv, world)
        seen = set()
        for r in range(world):
            u = plan.units(r)
            assert len(u) == batch * hkv // world
            assert not (seen & set(u))
            seen |= set(u)
        assert seen == {(b, h) for b in range(batch) for h in range(hkv)}
    # 8 KV heads on 8 GPUs with a batch that does not divide: one KV head per GPU
    plan = shard_units(3, 8, 8)
    assert all(len(plan.kv_head_ids[r]) == 1 and plan.batch_ids[r] == [0, 1, 2] for r in range(8))
    with pytest.raises(ValueError):
        shard_units(3, 5, 4)
    # both split: sequences by default, KV heads on request (config 4: B=128, 8 KV heads, 8 GPUs)
    by_batch, by_heads = shard_units(128, 8, 8), shard_units(128, 8, 8, prefer="heads")
    assert all(len(by_batch.batch_ids[r]) == 16 and len(by_batch.kv_head_ids[r]) == 8 for r in range(8))
    assert all(by_heads.kv_head_ids[r] == [r] and len(by_heads.batch_ids[r]) == 128 for r in range(8))
    assert shard_units(128, 8, 2, prefer="heads").kv_head_ids == [[0, 1, 2, 3], [4, 5, 6, 7]]
    with pytest.raises(ValueError):
        shard_units(4, 4, 2, prefer="rows")


def test_ragged_lengths_are_balanced():
    lens = [32768, 8192, 30000, 9000, 20000, 21000, 12000, 28000]
    plan = shard_units(8, 8, 4, seq_lens=lens)
    totals = [sum(lens[b] for b in plan.batch_ids[r]) for r in range(4)]
    assert max(totals) - min(totals) <= 0.2 * (sum(lens) / 4)
    assert sorted(b for r in range(4) for b in plan.batch_ids[r]) == list(range(8))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, hkv, group, lens, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = shard_units(batch, hkv, world, seq_lens=lens)
        # a stand-in for the step's output: a value that encodes (b, query head, channel)
        b_ids, h_ids = plan.batch_ids[rank], plan.q_head_ids(rank, group)
        local = torch.tensor([[[b * 1000 + h + d * 1e-3 for d in range(4)] for h in h_ids] for b in b_ids])
        full = gather_outputs(local, plan, group, rank)
        want = torch.tensor([[[b * 1000 + h + d * 1e-3 for d in range(4)] for h in range(hkv * group)]
                             for b in range(batch)])
        ret[rank] = bool(torch.equal(full, want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch,hkv,group,lens", [(4, 2, 2, [100, 50, 75, 20]), (3, 4, 1, None)])
def test_gather_on_two_gloo_ranks(batch, hkv, group, lens):
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, batch, hkv, group, lens, ret), nprocs=world, join=True)
    assert ret[0] and ret[1]
