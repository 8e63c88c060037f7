"""Routes the decode steps of a Hugging Face Llama-class model through the sparse decode step.

The reference's ``enable_sparse_attention(model, sparse_config, enable_budget_info, ...)``
(twilight/pyimpl/attention.py:351-418) swaps ``LlamaAttention.forward`` for its own
``attention_forward`` (:60-339).  With the attention-function registry of current transformers
releases the model's forward can stay as it is (projections, RoPE, the HF cache update): only the
function that turns ``(query, key, value)`` into the attention output is replaced.

* Prefill (more than one query token): the stock ``sdpa`` function, as the reference does for
  ``q_len > 1`` (:188-193 only sparsify ``q_len == 1``).  The keys and values it saw are kept by
  reference and turned into a paged cache (pages, INT4 slabs, page metadata) when the first decode
  step arrives.
* Decode (one query token): the new token's K/V row is appended to the layer's paged cache by the
  append kernel, then ``SparseDecodeAttention`` runs select -> estimate -> prune -> attend with
  the reference's rule that the first two layers stay dense and are not counted (:195-197), and
  records budgets like ``HistoryBudgetInfo`` (:284-285).

Limits: head_dim 128, batches without padding (every sequence has the same length), no dropout.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import _lib
from ..cache import HEAD_DIM, GrowingPagedCache
from .attention import SparseDecodeAttention
from .state import HistoryBudgetInfo

_PREFIX = "twilight_b200"


class HFSparseAttention:
    """The attention function registered for one model; keeps one paged cache per layer."""

    def __init__(self, model, sparse_config: Dict, enable_budget_info: bool = False,
                 max_len: Optional[int] = None) -> None:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
        cfg = model.config
        head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        if head_dim != HEAD_DIM:
            raise _lib.TwilightError(f"the kernels are built for head_dim {HEAD_DIM}, the model has {head_dim}")
        self.attn = SparseDecodeAttention(sparse_config, cfg.num_attention_heads, enable_budget_info)
        self.max_len = int(max_len or cfg.max_position_embeddings)
        self.dense = ALL_ATTENTION_FUNCTIONS["sdpa"]
        self.caches: Dict[int, GrowingPagedCache] = {}
        self._pending: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    @property
    def budget_info(self) -> Optional[HistoryBudgetInfo]:
        return self.attn.budget_info

    def _cache_for(self, layer: int, key: torch.Tensor, value: torch.Tensor) -> GrowingPagedCache:
        """The layer's paged cache holding every token but the newest one of ``key``/``value``."""
        if layer in self._pending:               # first decode step after a prefill
            k, v = self._pending.pop(layer)
            if k.shape[2] != key.shape[2] - 1:
                raise _lib.TwilightError("decode step does not follow the prefill this layer saw")
            c = self.caches.get(layer)
            if (c is None or c.batch != k.shape[0] or c.k_pages.shape[1] != k.shape[1]
                    or c.k_pages.dtype != k.dtype or c.k_pages.device != k.device):
                c = GrowingPagedCache(k.shape[0], k.shape[1], self.max_len, k.dtype, k.device)
                self.caches[layer] = c
            c.load(k, v)
        c = self.caches.get(layer)
        if c is None or c.length != key.shape[2] - 1:
            raise _lib.TwilightError("decode step without a matching prefill (or the HF cache was edited)")
        return c

    def __call__(self, module, query, key, value, attention_mask, dropout: float = 0.0,
                 scaling: Optional[float] = None, **kwargs):
        layer = int(module.layer_idx)
        if query.shape[2] > 1:
            self._pending[layer] = (key, value)   # all tokens so far, [B,H_kv,L,128]
            return self.dense(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                              **kwargs)
        if dropout:
            raise _lib.TwilightError("dropout is not supported on the decode path")
        if scaling is not None and abs(scaling - HEAD_DIM ** -0.5) > 1e-6:
            raise _lib.TwilightError("the decode step scales logits by 1/sqrt(head_dim)")
        if attention_mask is not None and attention_mask.dtype == torch.bool and not bool(attention_mask.all()):
            raise _lib.TwilightError("padded batches are not supported on the decode path")
        cache = self._cache_for(layer, key, value)
        cache.append(key[:, :, -1], value[:, :, -1])
        out = self.attn(layer, query.contiguous(), cache.view)     # [B,H_q,128]
        return out[:, None], None                                   # [B,1,H_q,128] as the model expects


def enable_sparse_attention(model, sparse_config: Dict, enable_budget_info: bool = False,
                            max_len: Optional[int] = None) -> Optional[HistoryBudgetInfo]:
    """Same call as the reference's (twilight/pyimpl/attention.py:351-418): patches ``model`` and
    returns the budget statistics object (or None).  The handler is left on
    ``model.twilight_attention``."""
    from transformers import AttentionInterface
    handler = HFSparseAttention(model, sparse_config, enable_budget_info, max_len)
    name = f"{_PREFIX}_{id(handler):x}"
    AttentionInterface.register(name, handler)
    model.config._attn_implementation = name
    model.twilight_attention = handler
    return handler.budget_info
