"""Sharding of the decode step over the GPUs of one node.

Every (batch row, KV head) unit is independent through select -> estimate -> prune -> attend, so
a node is used by giving each rank a rectangular block of units (some sequences x some KV heads,
with the KV cache of exactly those units) and gathering the per-rank outputs once per layer pass.
There is no reduction and no kernel reads another GPU's memory.  The reference has no distributed
code at all (its scripts only use HF ``device_map="auto"``, benchmark/LongBench/pred.py:272-274).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass
class ShardPlan:
    """Which sequences and which KV heads each rank owns.  ``batch_ids[r]`` x ``kv_head_ids[r]`` is
    rank r's block; blocks tile the whole (batch, KV head) grid exactly once."""
    batch: int
    num_kv_heads: int
    world_size: int
    batch_ids: List[List[int]]
    kv_head_ids: List[List[int]]

    def units(self, rank: int) -> List[tuple]:
        return [(b, h) for b in self.batch_ids[rank] for h in self.kv_head_ids[rank]]

    def q_head_ids(self, rank: int, group: int) -> List[int]:
        """Query heads of the rank's KV heads (``group`` = query heads per KV head)."""
        return [h * group + g for h in self.kv_head_ids[rank] for g in range(group)]


def shard_units(batch: int, num_kv_heads: int, world_size: int,
                seq_lens: Optional[Sequence[int]] = None, prefer: str = "batch") -> ShardPlan:
    """Splits the grid into ``world_size`` equal rectangles: over sequences when the batch divides
    (balanced by context length when ``seq_lens`` is given), otherwise over KV heads, otherwise
    over both (``world = wb * wh``).  ``prefer="heads"`` tries the KV heads first (one KV head per
    GPU for an 8-KV-head model on 8 GPUs).  Raises when no rectangular tiling exists."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    if prefer not in ("batch", "heads"):
        raise ValueError("prefer must be 'batch' or 'heads'")
    wb = wh = None
    by_batch, by_heads = batch % world_size == 0, num_kv_heads % world_size == 0
    if by_heads and (prefer == "heads" or not by_batch):
        wb, wh = 1, world_size
    elif by_batch:
        wb, wh = world_size, 1
    else:
        for cand in range(world_size, 0, -1):
            if world_size % cand == 0 and batch % cand == 0 and num_kv_heads % (world_size // cand) == 0:
                wb, wh = cand, world_size // cand
                break
    if wb is None:
        raise ValueError(f"cannot tile {batch} sequences x {num_kv_heads} KV heads over {world_size} ranks")
    order = list(range(batch))
    if seq_lens is not None and wb > 1:
        # longest first, dealt in serpentine order: equal counts, near-equal token totals
        order.sort(key=lambda b: -int(seq_lens[b]))
    per_b = batch // wb
    groups: List[List[int]] = [[] for _ in range(wb)]
    for i, b in enumerate(order):
        rnd, pos = divmod(i, wb)
        groups[pos if rnd % 2 == 0 else wb - 1 - pos].append(b)
    assert all(len(g) == per_b for g in groups)
    per_h = num_kv_heads // wh
    batch_ids, head_ids = [], []
    for r in range(world_size):
        rb, rh = divmod(r, wh)
        batch_ids.append(sorted(groups[rb]))
        head_ids.append(list(range(rh * per_h, (rh + 1) * per_h)))
    return ShardPlan(batch, num_kv_heads, world_size, batch_ids, head_ids)


def gather_outputs(local_out: torch.Tensor, plan: ShardPlan, group_size: int, rank: int,
                   gathered: Optional[torch.Tensor] = None, process_group=None) -> torch.Tensor:
    """All-gathers the per-rank outputs ``[B_local, Hq_local, D]`` (one collective) and puts every
    block at its place in the full ``[B, H_q, D]`` tensor, which every rank then holds."""
    import torch.distributed as dist
    world = plan.world_size
    if gathered is None:
        gathered = torch.empty((world,) + tuple(local_out.shape), dtype=local_out.dtype,
                               device=local_out.device)
    if world == 1:
        gathered[0].copy_(local_out)
    else:
        # concatenated form ([world*B_local, ...]): accepted by both NCCL and gloo
        dist.all_gather_into_tensor(gathered.view((-1,) + tuple(local_out.shape[1:])), local_out.contiguous(),
                                    group=process_group)
    hq = plan.num_kv_heads * group_size
    full = torch.empty(plan.batch, hq, local_out.shape[-1], dtype=local_out.dtype, device=local_out.device)
    for r in range(world):
        b_idx = torch.tensor(plan.batch_ids[r], device=local_out.device)
        h_idx = torch.tensor(plan.q_head_ids(r, group_size), device=local_out.device)
        full[b_idx[:, None], h_idx[None, :]] = gathered[r]
    return full
