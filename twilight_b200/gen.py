"""Seeded synthetic decode inputs with the shapes and value distributions of the benchmark
configurations (stand-ins for real checkpoints and long-context datasets).

Per (batch row, KV head): ``q ~ N(0,1)``, ``K ~ N(0,1)``, ``V ~ N(0,1)``; a fraction ``rho`` of key
positions, chosen uniformly, is replaced by a heavy hitter ``c_h * q_hat * sqrt(D) + N(0, 0.1^2)``
and position 0 (attention sink) by ``c_s * q_hat * sqrt(D)``, with ``q_hat = q/||q||`` of the first
query head of the KV head's group.  ``recipe``:

* ``"literal"``     ``c_h = 4``, ``c_s = 8`` as the configurations state them.  Logits are then about
  45 and 90, the softmax puts all mass on the sink and the top-p budget is 1 per head.
* ``"mid"``         logits (not vector lengths) set to ``heavy_logit`` / ``sink_logit``
  (defaults 10 / 12): budgets near ``rho * L``, like the averages the reference reports.
* ``"calibrated"``  logits 4 / 8: budgets of a few thousand tokens.

Everything is generated directly in the paged layout on the target device.
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple, Union

import torch

from .cache import HEAD_DIM, PAGE, PagedKVCache


def _coeffs(recipe: str, qnorm: torch.Tensor, heavy_logit: float, sink_logit: float
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row multipliers of q_hat*sqrt(D) for heavy hitters and for the sink."""
    if recipe == "literal":
        return torch.full_like(qnorm, 4.0), torch.full_like(qnorm, 8.0)
    if recipe == "calibrated":
        heavy_logit, sink_logit = 4.0, 8.0
    elif recipe != "mid":
        raise ValueError(f"unknown recipe {recipe}")
    # logit = q.(c*q_hat*sqrt(D))/sqrt(D) = c*||q||  =>  c = logit/||q||
    return heavy_logit / qnorm, sink_logit / qnorm


def make_decode_inputs(batch: int, num_q_heads: int, num_kv_heads: int,
                       seq_lens: Union[int, Sequence[int]], *, rho: Union[float, Tuple[float, float]] = 0.01,
                       dtype: torch.dtype = torch.bfloat16, device="cuda", seed: int = 0,
                       recipe: str = "literal", heavy_logit: float = 10.0, sink_logit: float = 12.0,
                       shuffle_pages: bool = False, build_aux: bool = True
                       ) -> Tuple[torch.Tensor, PagedKVCache]:
    """Returns ``(q [B,H_q,128], cache)``.  ``rho`` is the heavy-hitter density, or a ``(lo, hi)``
    range from which a density is drawn per (row, KV head)."""
    dev = torch.device(device)
    lens: List[int] = [int(seq_lens)] * batch if isinstance(seq_lens, int) else [int(x) for x in seq_lens]
    assert len(lens) == batch and num_q_heads % num_kv_heads == 0
    g = num_q_heads // num_kv_heads
    gen = torch.Generator(device=dev).manual_seed(seed)
    indptr, indices, last, total = PagedKVCache.page_table(lens, dev, seed + 1 if shuffle_pages else None)

    q32 = torch.randn(batch, num_q_heads, HEAD_DIM, generator=gen, device=dev)
    q = q32.to(dtype)
    k_pages = torch.empty(total, num_kv_heads, PAGE, HEAD_DIM, dtype=dtype, device=dev)
    v_pages = torch.empty_like(k_pages)
    # fill in slices to keep the fp32 temporaries small
    step = max(1, (1 << 26) // (num_kv_heads * PAGE * HEAD_DIM))
    for p0 in range(0, total, step):
        p1 = min(total, p0 + step)
        k_pages[p0:p1] = torch.randn(p1 - p0, num_kv_heads, PAGE, HEAD_DIM, generator=gen, device=dev).to(dtype)
        v_pages[p0:p1] = torch.randn(p1 - p0, num_kv_heads, PAGE, HEAD_DIM, generator=gen, device=dev).to(dtype)

    qlead = q32[:, ::g]                                   # first query head of each group [B,Hkv,D]
    qnorm = qlead.norm(dim=-1, keepdim=True)
    qhat = qlead / qnorm
    c_h, c_s = _coeffs(recipe, qnorm, heavy_logit, sink_logit)
    heavy_vec = c_h * qhat * math.sqrt(HEAD_DIM)          # [B,Hkv,D]
    sink_vec = c_s * qhat * math.sqrt(HEAD_DIM)
    idx_host, ptr_host = indices.cpu().long(), indptr.cpu().long()
    for b, n in enumerate(lens):
        phys = idx_host[ptr_host[b]: ptr_host[b + 1]].to(dev)
        for h in range(num_kv_heads):
            if isinstance(rho, tuple):
                r = rho[0] + (rho[1] - rho[0]) * float(torch.rand(1, generator=gen, device=dev))
            else:
                r = rho
            n_heavy = int(math.floor(r * n))
            if n_heavy > 0:
                pos = torch.randperm(n, generator=gen, device=dev)[:n_heavy]
                noise = 0.1 * torch.randn(n_heavy, HEAD_DIM, generator=gen, device=dev)
                k_pages[phys[pos // PAGE], h, pos % PAGE] = (heavy_vec[b, h] + noise).to(dtype)
            k_pages[phys[0], h, 0] = sink_vec[b, h].to(dtype)
        if n % PAGE:  # keep the unused tail of the last page at zero
            k_pages[phys[-1], :, n % PAGE:] = 0
            v_pages[phys[-1], :, n % PAGE:] = 0
    cache = PagedKVCache(k_pages, v_pages, None, None, indptr, indices, last, lens)
    if build_aux:
        cache.build_aux()
    return q, cache


def ragged_lengths(batch: int, lo: int, hi: int, seed: int = 0) -> List[int]:
    """``batch`` context lengths uniform in ``[lo, hi]``."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (batch,), generator=g).tolist()


def make_unit_inputs(batch_ids: Sequence[int], kv_head_ids: Sequence[int], group: int,
                     seq_lens: Sequence[int], *, rho: Union[float, Tuple[float, float]] = 0.01,
                     dtype: torch.dtype = torch.bfloat16, device="cuda", seed: int = 0, recipe: str = "literal",
                     heavy_logit: float = 10.0, sink_logit: float = 12.0, shuffle_pages: bool = False
                     ) -> Tuple[torch.Tensor, PagedKVCache]:
    """The same kind of inputs for a rectangular block of (sequence, KV head) units of a larger
    problem, every unit generated from its own seed ``(seed, global sequence id, global KV head
    id)``: whichever rank owns a unit produces the same q, K and V for it, so any rank can rebuild
    a unit of another one to check a gathered result.  ``seq_lens`` holds the lengths of the
    sequences in ``batch_ids`` (in that order); ``group`` = query heads per KV head.
    Returns ``(q [B_local, H_kv_local*group, 128], cache)`` for the block."""
    dev = torch.device(device)
    lens = [int(x) for x in seq_lens]
    nb, nh = len(batch_ids), len(kv_head_ids)
    assert len(lens) == nb
    indptr, indices, last, total = PagedKVCache.page_table(lens, dev, seed + 1 if shuffle_pages else None)
    q = torch.empty(nb, nh * group, HEAD_DIM, dtype=dtype, device=dev)
    k_pages = torch.zeros(total, nh, PAGE, HEAD_DIM, dtype=dtype, device=dev)
    v_pages = torch.zeros_like(k_pages)
    idx_host, ptr_host = indices.cpu().long(), indptr.cpu().long()
    for bi, b in enumerate(batch_ids):
        n = lens[bi]
        npg = (n + PAGE - 1) // PAGE
        phys = idx_host[ptr_host[bi]: ptr_host[bi + 1]].to(dev)
        for hi, h in enumerate(kv_head_ids):
            gen = torch.Generator(device=dev).manual_seed((seed * 1000003 + int(b) * 4099 + int(h)) & 0x7FFFFFFF)
            q32 = torch.randn(group, HEAD_DIM, generator=gen, device=dev)
            k = torch.randn(npg * PAGE, HEAD_DIM, generator=gen, device=dev)
            v = torch.randn(npg * PAGE, HEAD_DIM, generator=gen, device=dev)
            qnorm = q32[0].norm()
            c_h, c_s = _coeffs(recipe, qnorm.reshape(1), heavy_logit, sink_logit)
            qhat = q32[0] / qnorm
            r = rho[0] + (rho[1] - rho[0]) * float(torch.rand(1, generator=gen, device=dev)) \
                if isinstance(rho, tuple) else rho
            n_heavy = int(math.floor(r * n))
            if n_heavy > 0:
                pos = torch.randperm(n, generator=gen, device=dev)[:n_heavy]
                noise = 0.1 * torch.randn(n_heavy, HEAD_DIM, generator=gen, device=dev)
                k[pos] = c_h * qhat * math.sqrt(HEAD_DIM) + noise
            k[0] = c_s * qhat * math.sqrt(HEAD_DIM)
            k[n:] = 0
            v[n:] = 0
            q[bi, hi * group: (hi + 1) * group] = q32.to(dtype)
            k_pages[phys, hi] = k.to(dtype).view(npg, PAGE, HEAD_DIM)
            v_pages[phys, hi] = v.to(dtype).view(npg, PAGE, HEAD_DIM)
    cache = PagedKVCache(k_pages, v_pages, None, None, indptr, indices, last, lens)
    cache.build_aux()
    return q, cache
