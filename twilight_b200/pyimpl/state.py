"""Enums and budget statistics with the reference's names (twilight/pyimpl/state.py)."""
from __future__ import annotations

from enum import Enum
from typing import Dict, List

import numpy as np
import torch


class _FromStr(Enum):
    @classmethod
    def from_str(cls, algo_str: str):
        return cls[algo_str.upper()]  # state.py:17-19


class CompressorType(_FromStr):
    NONE = 0
    SNAP_KV = 1


class IndexSelectorType(_FromStr):
    NONE = 0
    STREAMING = 1
    QUEST = 2
    ORACLE_TOPK = 3
    TIDAL_DECODE = 4
    SPARQ = 5
    DS = 6
    PQCACHE = 7


class WeightEstimatorType(_FromStr):
    NONE = 0
    MIN_MAX_QUANT = 1
    MAX_QUANT = 2
    THRESHOLD = 5
    H_THRESHOLD = 6


class WeightPrunerType(_FromStr):
    NONE = 0
    THRESHOLD = 1
    TOP_P = 2


class HistoryBudgetInfo:
    """Per-query, per-layer, per-head pruned budgets (state.py:136-234).  ``update`` accepts the
    reference's bool mask ``[B,H,1,L]`` or an integer budget tensor ``[B,H]`` from the kernels."""

    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        self._budget_num: List[Dict[int, torch.Tensor]] = []
        self._last_layer_id = -999

    def update(self, layer_id: int, selected: torch.Tensor) -> None:
        if selected.dtype == torch.bool:
            head_budgets = torch.sum(selected, dim=-1).flatten()  # state.py:154
        else:
            head_budgets = selected.flatten().to(torch.int64)
        if layer_id != self._last_layer_id + 1:  # new query, state.py:155-156
            self._budget_num.append({})
        self._budget_num[-1][layer_id] = head_budgets
        self._last_layer_id = layer_id

    def get_avg_budget_per_layer_single_query(self, query_index: int) -> List[float]:
        return [torch.mean(v.float()).item() for v in self._budget_num[query_index].values()]

    def get_avg_budget_cur_query(self) -> List[float]:
        return self.get_avg_budget_per_layer_single_query(-1)

    def get_avg_budget_per_query(self) -> List[float]:
        """Mean over heads and over layers >= 2 (state.py:213-222)."""
        ret = []
        for info in self._budget_num:
            per_layer = [torch.mean(v.float()).item() for lid, v in info.items() if lid > 1]
            ret.append(float(np.mean(per_layer)) if per_layer else float("nan"))
        return ret

    def get_total_avg_budget(self) -> float:
        return float(np.mean(self.get_avg_budget_per_query()))
