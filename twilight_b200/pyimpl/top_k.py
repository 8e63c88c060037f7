"""Oracle top-k selector with the reference's mask interface (twilight/pyimpl/top_k.py:7-30)."""
import torch

from ..cache import PAGE
from ..kernel import ops


def top_k(attn_weights: torch.Tensor, token_budget: int) -> torch.Tensor:
    """``attn_weights [B,H,1,L]`` -> bool mask ``[B,H,1,L]`` of the ``min(token_budget, L)`` largest
    entries of every row (top_k.py:7-16).  Equal values at the cut go to the lower positions
    (``torch.topk`` leaves that open).  Runs the radix-select kernel of the Quest selector with
    one "page" per token."""
    b, h, one, l = attn_weights.shape
    assert one == 1
    k = min(int(token_budget), l)
    rows = b * h
    dev = attn_weights.device
    scores = attn_weights.reshape(rows, 1, l).float().contiguous()
    indptr = torch.arange(rows + 1, dtype=torch.int32, device=dev) * l
    # a budget of 16*k tokens keeps k pages (quest.py:93-95), i.e. k entries here
    picked, n_picked, _ = ops.quest_topk(scores, indptr, PAGE * k, max_pages=l)
    return ops.indices_to_mask(picked, n_picked, l).reshape(b, h, 1, l)


def oracle_topk_selector(attn_weights: torch.Tensor, token_budget: int) -> torch.Tensor:
    """Oracle TopK index selector (top_k.py:19-30)."""
    return top_k(attn_weights, token_budget)
