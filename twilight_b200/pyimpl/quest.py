"""Quest selector with the reference's mask interface (twilight/pyimpl/quest.py:17-122)."""
from typing import Optional

import torch

from .. import _lib
from ..cache import PAGE
from ..kernel import ops


def quest_selector(model, query_states: torch.Tensor, key_states: torch.Tensor, chunk_size: int,
                   token_budget: Optional[int] = -1, sparsity_rate: Optional[float] = -1,
                   attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """query ``[B,H,1,D]``, keys ``[B,H,L,D]`` (already expanded to query heads) -> bool mask
    ``[B,H,1,L]`` of the tokens in the best pages.  ``model`` is unused (the reference reads
    ``model.num_heads``).  Dense keys are re-viewed as one-head sequences of pages, their
    (min,max) metadata is built, and the paged selector kernels run on that."""
    if chunk_size != PAGE:
        raise _lib.TwilightError("chunk_size must be 16, the page size of the cache")
    b, h, l, d = key_states.shape
    if sparsity_rate != -1:
        token_budget = int(l * sparsity_rate)  # quest.py:44-45
    n_pages = (l + PAGE - 1) // PAGE
    k = key_states.contiguous()
    if l % PAGE:
        pad = torch.zeros(b, h, n_pages * PAGE - l, d, dtype=k.dtype, device=k.device)
        k = torch.cat([k, pad], dim=2).contiguous()
    rows = b * h
    k_pages = k.view(rows * n_pages, 1, PAGE, d)
    dev = k.device
    indptr = torch.arange(rows + 1, dtype=torch.int32, device=dev) * n_pages
    indices = torch.arange(rows * n_pages, dtype=torch.int32, device=dev)
    last = torch.full((rows,), (l - 1) % PAGE + 1, dtype=torch.int32, device=dev)
    kmeta = ops.build_page_meta(k_pages, indptr, indices, last, max_pages=n_pages)
    q = query_states.reshape(rows, 1, d).contiguous()
    cand_pages, cand_npages, _ = ops.quest_select(q, kmeta, indptr, indices, token_budget,
                                                  max_pages=n_pages)
    # candidate pages -> token mask
    page_mask = torch.zeros(rows, n_pages + 1, dtype=torch.bool, device=dev)
    kk = cand_pages.shape[-1]
    valid = torch.arange(kk, device=dev)[None, :] < cand_npages.reshape(rows, 1)
    idx = torch.where(valid, cand_pages.reshape(rows, kk).long(), torch.full_like(valid, n_pages, dtype=torch.long))
    page_mask.scatter_(1, idx, True)
    mask = page_mask[:, :n_pages].repeat_interleave(PAGE, dim=1)[:, :l]
    return mask.reshape(b, h, 1, l)
