"""The decode branch of the reference's patched attention, on a paged cache.

``attention_forward`` (twilight/pyimpl/attention.py:60-339) projects q/k/v, applies RoPE, updates
the HF cache and then, for q_len == 1, runs Select -> Estimate -> Prune -> Attend densely
(:188-306).  ``SparseDecodeAttention`` is that last part with the same configuration dictionary,
the same "skip the first two layers" rule (:195-197) and the same budget statistics (:284-285);
projections, RoPE and the cache update stay with the caller's model code.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..cache import PAGE, PagedKVCache
from ..kernel import ops
from ..step import DecodeWorkspace, SparseConfig, select_prune_attend_step
from .state import HistoryBudgetInfo


class SparseDecodeAttention:
    """Holds what the reference keeps in its module-global ``LocalState`` (state.py:66-79)."""

    def __init__(self, sparse_config: Dict, num_q_heads: int, enable_budget_info: bool = False) -> None:
        self.config = SparseConfig.from_dict(sparse_config)
        self.num_q_heads = num_q_heads
        self.budget_info: Optional[HistoryBudgetInfo] = HistoryBudgetInfo() if enable_budget_info else None
        self._ws: Dict[Tuple, DecodeWorkspace] = {}
        self._dense: Dict[Tuple, Tuple] = {}

    def _workspace(self, cache: PagedKVCache) -> DecodeWorkspace:
        # a growing cache sizes the buffers once, for the pages it reserves per sequence
        pages = cache.capacity_pages or cache.max_pages
        key = (cache.batch, pages, cache.device, cache.dtype)
        if key not in self._ws:
            self._ws[key] = DecodeWorkspace(cache.batch, self.num_q_heads, pages, self.config, cache.device,
                                            cache.dtype)
        return self._ws[key]

    def _dense_lists(self, cache: PagedKVCache, ws: DecodeWorkspace) -> Tuple[torch.Tensor, torch.Tensor]:
        """Index lists that keep every token (layers that are not sparsified)."""
        key = (cache.batch, ws.max_pages, cache.device)
        if key not in self._dense:
            stride = ws.max_pages * PAGE
            idx = torch.arange(stride, dtype=torch.int32, device=cache.device)
            idx = idx.expand(cache.batch, self.num_q_heads, stride).contiguous()
            self._dense[key] = (idx, torch.empty(cache.batch, self.num_q_heads, dtype=torch.int32,
                                                 device=cache.device), [])
        idx, bud, lens = self._dense[key]
        if lens != list(cache.seq_lens):
            bud.copy_(torch.tensor(cache.seq_lens, dtype=torch.int32)[:, None].expand(-1, self.num_q_heads))
            lens[:] = cache.seq_lens
        return idx, bud

    def forward(self, layer_id: int, query_states: torch.Tensor, cache: PagedKVCache) -> torch.Tensor:
        """query ``[B,H_q,1,128]`` or ``[B,H_q,128]`` -> attention output ``[B,H_q,128]`` (a buffer
        that the next call overwrites)."""
        ws = self._workspace(cache)
        start_layer = 2 if self.config.skip_first_two_layers else 0
        if layer_id < start_layer:  # attention.py:195-197: full attention, nothing recorded
            idx, bud = self._dense_lists(cache, ws)
            q = query_states[:, :, 0, :] if query_states.dim() == 4 else query_states
            if not hasattr(ws, "_dense_ws"):
                ws._dense_ws = torch.zeros(ops.sparse_attn_workspace_bytes(cache.batch, self.num_q_heads,
                                                                           idx.shape[-1], ws.attn_chunk),
                                           dtype=torch.uint8, device=cache.device)
            return ops.sparse_decode_attn(q.contiguous(), cache.k_pages, cache.v_pages, cache.kv_indptr,
                                          cache.kv_indices, idx, bud, out=ws.out, workspace=ws._dense_ws,
                                          chunk=ws.attn_chunk, status=ws.status)
        out = select_prune_attend_step(query_states, cache, ws)
        if self.budget_info is not None:
            self.budget_info.update(layer_id, ws.budget)
        return out

    __call__ = forward


def enable_sparse_attention(sparse_config: Dict, num_q_heads: int, enable_budget_info: bool = False
                            ) -> Tuple[SparseDecodeAttention, Optional[HistoryBudgetInfo]]:
    """Counterpart of ``enable_sparse_attention(model, sparse_config, enable_budget_info, ...)``
    (attention.py:351-418) without the HF monkey patch: returns the decode-attention object a
    model's attention layers call, and the budget statistics object the reference returns."""
    attn = SparseDecodeAttention(sparse_config, num_q_heads, enable_budget_info)
    return attn, attn.budget_info
