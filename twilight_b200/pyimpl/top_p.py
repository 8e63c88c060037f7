"""Top-p pruner with the reference's mask interface (twilight/pyimpl/top_p.py:10-15)."""
import torch
from torch import nn

from ..kernel import top_p_fp32_return_mask


def top_p_unnormalized(attn_weights: torch.Tensor, threshold: float) -> torch.Tensor:
    """Un-normalised weights ``[B,H,1,L]`` -> bool mask of the kept tokens."""
    normalized_weights = nn.functional.softmax(attn_weights, dim=-1, dtype=torch.float32)
    return top_p_fp32_return_mask(normalized_weights, threshold)
