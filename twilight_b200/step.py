"""The fused decode step: select -> estimate -> prune -> attend, allocation-free after set-up.

Mirrors the decode branch of ``attention_forward`` (twilight/pyimpl/attention.py:188-306) on a
paged cache.  ``SparseConfig`` takes the reference's config dictionary
(attention.py:360-376, benchmark/configs/config_quest_twi.json) and keeps its names.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from . import _lib
from .cache import PAGE, HEAD_DIM, PagedKVCache, quest_max_k
from .kernel import ops


@dataclass
class SparseConfig:
    """Selector / estimator / pruner settings with the reference's key names."""
    selector: str = "none"            # "none" | "quest"                  (IndexSelectorType)
    token_budget: int = -1            # quest: tokens kept by the selector
    chunk_size: int = PAGE            # quest: must equal the page size, 16
    weight_estimator: str = "min_max_quant"   # only the INT4 estimator has a kernel
    quant_bit: int = 4
    weight_pruner: str = "top_p"      # "top_p" | "threshold" | "none"    (WeightPrunerType)
    threshold: float = 0.95
    use_estimated_weights_in_attn: bool = False
    skip_first_two_layers: bool = True

    @classmethod
    def from_dict(cls, cfg: Dict) -> "SparseConfig":
        """Parses the dictionary ``enable_sparse_attention`` takes (attention.py:379-400)."""
        def split(section: str):
            d = dict(cfg.get(section, {"type": "none"}))
            return str(d.pop("type")).lower(), d
        comp, _ = split("compressor")
        if comp != "none":
            raise _lib.TwilightError("prefill-time compressors are outside the decode path")
        sel, sel_args = split("selector")
        est, est_args = split("weight_estimator")
        prn, prn_args = split("weight_pruner")
        out = cls(selector=sel, weight_estimator=est, weight_pruner=prn,
                  use_estimated_weights_in_attn=bool(cfg.get("use_estimated_weights_in_attn", False)),
                  skip_first_two_layers=bool(cfg.get("skip_first_two_layers", True)))
        if sel == "quest":
            out.token_budget = int(sel_args.get("token_budget", -1))
            out.chunk_size = int(sel_args.get("chunk_size", PAGE))
        if est == "min_max_quant":
            out.quant_bit = int(est_args.get("quant_bit", 4))
        if prn in ("top_p", "threshold"):
            out.threshold = float(prn_args["threshold"])
        out.validate()
        return out

    def validate(self) -> None:
        if self.selector not in ("none", "quest"):
            raise _lib.TwilightError(f"selector '{self.selector}' has no kernel on this path")
        if self.selector == "quest" and (self.chunk_size != PAGE or self.token_budget <= 0):
            raise _lib.TwilightError("quest needs chunk_size == 16 (the page size) and a positive token_budget")
        if self.weight_estimator != "min_max_quant" or self.quant_bit != 4:
            raise _lib.TwilightError("the estimator kernel reads the 4-bit min/max cache only")
        if self.weight_pruner not in ("top_p", "threshold", "none"):
            raise _lib.TwilightError(f"pruner '{self.weight_pruner}' has no kernel on this path")


@dataclass
class DecodeWorkspace:
    """Every intermediate of one decode step, allocated once (so a step can be graph-captured)."""
    batch: int
    num_q_heads: int
    max_pages: int
    config: SparseConfig
    device: torch.device
    dtype: torch.dtype
    attn_chunk: int = 512
    page_scores: Optional[torch.Tensor] = None
    cand_pages: Optional[torch.Tensor] = None
    cand_npages: Optional[torch.Tensor] = None
    scores: torch.Tensor = field(init=False)
    indices: torch.Tensor = field(init=False)
    budget: torch.Tensor = field(init=False)
    threshold: torch.Tensor = field(init=False)
    out: torch.Tensor = field(init=False)
    attn_ws: torch.Tensor = field(init=False)
    weights: Optional[torch.Tensor] = None   # softmax weights of kept tokens (estimated-weights mode)
    status: torch.Tensor = field(init=False)

    def __post_init__(self) -> None:
        b, h, dev = self.batch, self.num_q_heads, self.device
        if self.config.selector == "quest":
            max_k = quest_max_k(self.config.token_budget, self.max_pages)
            self.page_scores = torch.empty(b, h, self.max_pages, dtype=torch.float32, device=dev)
            self.cand_pages = torch.empty(b, h, max_k, dtype=torch.int32, device=dev)
            self.cand_npages = torch.empty(b, h, dtype=torch.int32, device=dev)
            stride = max_k * PAGE
        else:
            stride = self.max_pages * PAGE
        self.scores = torch.empty(b, h, stride, dtype=torch.float32, device=dev)
        self.indices = torch.empty(b, h, stride, dtype=torch.int32, device=dev)
        self.budget = torch.zeros(b, h, dtype=torch.int32, device=dev)
        self.threshold = torch.zeros(b, h, 2, dtype=torch.float32, device=dev)
        self.out = torch.empty(b, h, HEAD_DIM, dtype=self.dtype, device=dev)
        self.attn_ws = torch.zeros(ops.sparse_attn_workspace_bytes(b, h, stride, self.attn_chunk),
                                   dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.config.use_estimated_weights_in_attn:
            self.weights = torch.empty(b, h, stride, dtype=torch.float32, device=dev)

    @classmethod
    def for_cache(cls, cache: PagedKVCache, num_q_heads: int, config: SparseConfig,
                  attn_chunk: int = 512) -> "DecodeWorkspace":
        return cls(cache.batch, num_q_heads, cache.max_pages, config, cache.device, cache.dtype,
                   attn_chunk)

    @property
    def kernels_per_step(self) -> int:
        return (2 if self.config.selector == "quest" else 0) + 3


def select_prune_attend_step(q: torch.Tensor, cache: PagedKVCache, ws: DecodeWorkspace,
                             variant: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step of one attention layer.  q ``[B,H_q,128]`` (or ``[B,H_q,1,128]``);
    returns ``ws.out [B,H_q,128]`` (or ``out`` when given).  ``ws.budget`` holds the per-head pruned budgets and
    ``ws.indices`` the kept tokens afterwards.  Launches 3 kernels (5 with the Quest selector)
    on the current stream and nothing else."""
    cfg = ws.config
    cand_pages = cand_npages = None
    if cfg.selector == "quest":
        cand_pages, cand_npages, _ = ops.quest_select(
            q, cache.kmeta, cache.kv_indptr, cache.kv_indices, cfg.token_budget,
            max_pages=ws.max_pages, page_scores=ws.page_scores, cand_pages=ws.cand_pages,
            cand_npages=ws.cand_npages, status=ws.status)
    ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                      max_pages=ws.max_pages, cand_pages=cand_pages, cand_npages=cand_npages,
                      scores=ws.scores, variant=variant, status=ws.status)
    # pruner "none" keeps every candidate with non-zero probability: a top-p above 1 does that
    mode = "threshold" if cfg.weight_pruner == "threshold" else "top_p"
    value = cfg.threshold if cfg.weight_pruner in ("top_p", "threshold") else 2.0
    if cfg.use_estimated_weights_in_attn:  # attention.py:295-296
        ops.prune_with_weights(ws.scores, cache.kv_indptr, cache.kv_last_page_len, value, mode=mode,
                               cand_pages=cand_pages, cand_npages=cand_npages, indices=ws.indices,
                               budget=ws.budget, weights=ws.weights, threshold=ws.threshold,
                               status=ws.status)
    elif mode == "threshold":
        ops.threshold_prune(ws.scores, cache.kv_indptr, cache.kv_last_page_len, value,
                            cand_pages=cand_pages, cand_npages=cand_npages, indices=ws.indices,
                            budget=ws.budget, cut=ws.threshold, status=ws.status)
    else:
        ops.topp_prune(ws.scores, cache.kv_indptr, cache.kv_last_page_len, value,
                       cand_pages=cand_pages, cand_npages=cand_npages, indices=ws.indices,
                       budget=ws.budget, threshold=ws.threshold, status=ws.status)
    ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                           ws.indices, ws.budget, out=ws.out if out is None else out,
                           workspace=ws.attn_ws, chunk=ws.attn_chunk, status=ws.status,
                           weights=ws.weights)
    return ws.out if out is None else out


def step_algorithmic_bytes(cache: PagedKVCache, num_q_heads: int, config: SparseConfig,
                           budgets: torch.Tensor) -> Dict[str, float]:
    """Bytes one step must move from HBM, per stage: 512 B per page and KV head of selector
    metadata, 80 B per candidate token of INT4 estimate, 512 B per kept token of K+V, plus page
    table, index lists, budgets, q and out.  Intermediate scores count as zero."""
    g = num_q_heads // cache.num_kv_heads
    esz = 2
    sel = est = meta = 0.0
    for n in cache.seq_lens:
        npg = (n + PAGE - 1) // PAGE
        if config.selector == "quest":
            k = quest_max_k(config.token_budget, npg)
            sel += npg * 2 * HEAD_DIM * esz * cache.num_kv_heads
            est += k * PAGE * 80 * num_q_heads           # per query head: each keeps its own pages
            meta += npg * 4 * cache.num_kv_heads + k * 4 * num_q_heads
        else:
            est += npg * PAGE * 80 * cache.num_kv_heads  # shared by the query-head group
            meta += npg * 4 * cache.num_kv_heads
    kept = float(budgets.sum().item())
    att = kept * 2 * HEAD_DIM * esz
    meta += kept * 4 * 2 + budgets.numel() * 4
    qo = 2 * budgets.numel() * HEAD_DIM * esz
    total = sel + est + att + meta + qo
    return dict(selector=sel, estimator=est, attention=att, metadata=meta, q_out=qo, total=total,
                group=g)
