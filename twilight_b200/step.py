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
    # not a reference key: round Quest page scores and estimated logits to the model dtype where the
    # reference's matmuls return that dtype (quest.py:76-84, attention.py:252-254); for comparisons
    round_to_dtype: bool = False

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
                  skip_first_two_layers=bool(cfg.get("skip_first_two_layers", True)),
                  round_to_dtype=bool(cfg.get("round_to_dtype", False)))
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
    """Every intermediate of one decode step in ONE device buffer, allocated (and zeroed) once, so
    that a step is a single C-ABI call and can be graph-captured.  The attributes are views of the
    buffer at the offsets ``twl_step_workspace_layout`` reports."""
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
    buffer: torch.Tensor = field(init=False)
    scores: torch.Tensor = field(init=False)
    indices: torch.Tensor = field(init=False)
    budget: torch.Tensor = field(init=False)
    threshold: torch.Tensor = field(init=False)
    out: torch.Tensor = field(init=False)
    attn_ws: torch.Tensor = field(init=False)
    weights: Optional[torch.Tensor] = None   # softmax weights of kept tokens (estimated-weights mode)
    status: torch.Tensor = field(init=False)

    def __post_init__(self) -> None:
        b, h, dev, cfg = self.batch, self.num_q_heads, self.device, self.config
        self.flags = (ops.STEP_ESTIMATED_WEIGHTS if cfg.use_estimated_weights_in_attn else 0) | \
                     (ops.STEP_ROUND_TO_DTYPE if cfg.round_to_dtype else 0)
        self.token_budget = cfg.token_budget if cfg.selector == "quest" else 0
        lay = ops.step_workspace_layout(b, h, self.max_pages, self.token_budget, self.attn_chunk, self.flags)
        self.layout = lay
        with torch.cuda.device(dev):
            self.buffer = torch.zeros(int(lay.total), dtype=torch.uint8, device=dev)
            self.out = torch.empty(b, h, HEAD_DIM, dtype=self.dtype, device=dev)
            self.status = torch.zeros(1, dtype=torch.int32, device=dev)

        def view(off: int, dtype: torch.dtype, *shape: int) -> torch.Tensor:
            n = 1
            for x in shape:
                n *= x
            nbytes = n * torch.empty(0, dtype=dtype).element_size()
            return self.buffer[off: off + nbytes].view(dtype).view(*shape)

        stride = int(lay.stride)
        if cfg.selector == "quest":
            self.page_scores = view(lay.page_scores, torch.float32, b, h, self.max_pages)
            self.cand_pages = view(lay.cand_pages, torch.int32, b, h, int(lay.max_k))
            self.cand_npages = view(lay.cand_npages, torch.int32, b, h)
        self.scores = view(lay.scores, torch.float32, b, h, stride)
        self.indices = view(lay.indices, torch.int32, b, h, stride)
        self.budget = view(lay.budget, torch.int32, b, h)
        self.threshold = view(lay.threshold, torch.float32, b, h, 2)
        self.attn_ws = self.buffer[lay.attn: lay.attn + lay.attn_bytes]
        if cfg.use_estimated_weights_in_attn:
            self.weights = view(lay.weights, torch.float32, b, h, stride)

    @classmethod
    def for_cache(cls, cache: PagedKVCache, num_q_heads: int, config: SparseConfig,
                  attn_chunk: int = 512) -> "DecodeWorkspace":
        return cls(cache.batch, num_q_heads, cache.max_pages, config, cache.device, cache.dtype,
                   attn_chunk)

    @property
    def kernels_per_step(self) -> int:
        return int(self.layout.kernels)


def select_prune_attend_step(q: torch.Tensor, cache: PagedKVCache, ws: DecodeWorkspace,
                             variant: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step of one attention layer.  q ``[B,H_q,128]`` (or ``[B,H_q,1,128]``);
    returns ``ws.out [B,H_q,128]`` (or ``out`` when given).  ``ws.budget`` holds the per-head pruned budgets and
    ``ws.indices`` the kept tokens afterwards.  One C-ABI call (``twl_select_prune_attend_step``), which
    launches 3 kernels (5 with the Quest selector) on the current stream and nothing else."""
    cfg = ws.config
    pruner = {"top_p": "top_p", "threshold": "threshold"}.get(cfg.weight_pruner, "none")
    return ops.select_prune_attend_step(
        q, cache.k_pages, cache.v_pages, cache.k4_pages, cache.kmeta, cache.kv_indptr, cache.kv_indices,
        cache.kv_last_page_len, max_pages=ws.max_pages, token_budget=ws.token_budget, pruner=pruner,
        pruner_value=cfg.threshold, out=ws.out if out is None else out, workspace=ws.buffer, flags=ws.flags,
        variant=variant, attn_chunk=ws.attn_chunk, status=ws.status)


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
