"""Operator API of the Select-then-Prune decode path.

``top_p_fp32_return_mask`` / ``top_p_fp16_return_mask`` keep the names, arguments and result of
the reference's ``twilight.kernel`` (twilight/kernel/cuda/sampling.py:118-133).  The other
operators are the index-list forms the decode step is built from.  Every operator launches
hand-written sm_100a kernels through the C ABI on the current CUDA stream; none of them has a
PyTorch or CPU fallback.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch

from .. import _lib

PAGE = 16
HEAD_DIM = 128
K4_SLAB_BYTES = 1280

FLAG_ITER_CAP, FLAG_BAD_INDEX, FLAG_WAIT_LIMIT = 1, 2, 4


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise _lib.TwilightError(f"unsupported dtype {t.dtype}: the kernels take float16 or bfloat16")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _same_device(dev: torch.device, **tensors: Optional[torch.Tensor]) -> None:
    """Every tensor that crosses the C ABI in one call must live on the device the kernels run on."""
    for name, t in tensors.items():
        if t is not None and t.device != dev:
            raise _lib.TwilightError(f"{name} is on {t.device}, the call runs on {dev}")


def _on(t: torch.Tensor, **others: Optional[torch.Tensor]):
    """Context in which ``t``'s device is the current CUDA device, as the reference's operators do
    with ``with probs.device`` (twilight/kernel/cuda/sampling.py:68).  The library launches on the
    current device, so a tensor on cuda:1 while cuda:0 is current (Hugging Face ``device_map="auto"``,
    benchmark/LongBench/pred.py:272-274) needs this guard; ``others`` are checked to be on that
    device too."""
    if not t.is_cuda:
        raise _lib.TwilightError("the operators take CUDA tensors only (there is no CPU path)")
    _same_device(t.device, **others)
    return torch.cuda.device(t.device)


def _cuda_contig(t: torch.Tensor, name: str) -> None:
    # same checks as CHECK_INPUT in csrc/src/pytorch_extension_utils.h:220-233
    if not t.is_cuda:
        raise _lib.TwilightError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise _lib.TwilightError(f"{name} must be contiguous")


def _q3(q: torch.Tensor) -> torch.Tensor:
    """Accepts q as [B,H,D] or the reference's [B,H,1,D]."""
    if q.dim() == 4:
        if q.shape[2] != 1:
            raise _lib.TwilightError("decode step only: q_len must be 1")
        q = q[:, :, 0, :]
    if q.dim() != 3 or q.shape[-1] != HEAD_DIM:
        raise _lib.TwilightError(f"q must be [B,H,{HEAD_DIM}]")
    _cuda_contig(q, "q")
    return q


# ---------------------------------------------------------------------------------------------
# reference-compatible mask operators
# ---------------------------------------------------------------------------------------------
def _top_p_return_mask(probs: torch.Tensor, arr: Optional[torch.Tensor], val: float, half: bool
                       ) -> torch.Tensor:
    _cuda_contig(probs, "probs")
    if probs.dim() != 4:
        raise _lib.TwilightError("probs must be a 4D tensor")  # CHECK_DIM(4, probs)
    lib = _lib.load()
    b, h, _, d = probs.shape
    if arr is not None:
        arr = arr.to(device=probs.device, dtype=torch.float32).contiguous()
        if arr.numel() != b * h:
            raise _lib.TwilightError("top_p tensor must have batch*num_heads elements")
    with _on(probs):
        mask = torch.zeros_like(probs, dtype=torch.bool)
        if half:
            st = lib.twl_top_p_return_mask_f16(probs.data_ptr(), _dtype_code(probs), mask.data_ptr(),
                                               _p(arr), val, b * h, d, None, _stream(probs.device))
        else:
            if probs.dtype != torch.float32:
                raise _lib.TwilightError("top_p_fp32_return_mask takes float32 probabilities")
            st = lib.twl_top_p_return_mask_f32(probs.data_ptr(), mask.data_ptr(), _p(arr), val,
                                               b * h, d, None, _stream(probs.device))
    _lib.check(st, "top_p_return_mask")
    return mask


# The reference registers its two mask operators as torch custom ops without mutated arguments
# (``flashinfer::top_p_fp{16,32}_return_mask``, twilight/kernel/cuda/sampling.py:62-100), which is
# what lets them sit inside traced or compiled graphs.  Same here, under this library's namespace:
# ``torch.ops.twilight_b200.top_p_fp32_return_mask(probs, maybe_top_p_arr, top_p_val)``, with a
# fake-tensor rule.  Registered through ``torch.library.Library`` (a schema without aliased or
# mutated arguments says the same as ``mutates_args=()``): its dispatch costs about 3 us a call on
# the host against about 12 us for the ``custom_op`` decorator, which matters for small rows.
_TORCH_LIB = torch.library.Library("twilight_b200", "DEF")
_SCHEMA = "(Tensor probs, Tensor? maybe_top_p_arr, float top_p_val) -> Tensor"


def _op_top_p_fp32(probs: torch.Tensor, maybe_top_p_arr: Optional[torch.Tensor], top_p_val: float
                   ) -> torch.Tensor:
    return _top_p_return_mask(probs, maybe_top_p_arr, top_p_val, half=False)


def _op_top_p_fp16(probs: torch.Tensor, maybe_top_p_arr: Optional[torch.Tensor], top_p_val: float
                   ) -> torch.Tensor:
    return _top_p_return_mask(probs, maybe_top_p_arr, top_p_val, half=True)


def _fake_top_p_mask(probs, maybe_top_p_arr, top_p_val):
    return torch.empty_like(probs, dtype=torch.bool)


for _name, _impl in (("top_p_fp32_return_mask", _op_top_p_fp32), ("top_p_fp16_return_mask", _op_top_p_fp16)):
    _TORCH_LIB.define(_name + _SCHEMA)
    # every backend goes to the same function: it refuses anything that is not a CUDA tensor itself
    _TORCH_LIB.impl(_name, _impl, "CompositeExplicitAutograd")
    torch.library.register_fake("twilight_b200::" + _name, _fake_top_p_mask, lib=_TORCH_LIB)


def _to_tensor_scalar_tuple(x):
    # twilight/kernel/cuda/sampling.py:111-115
    return (x, 0.0) if isinstance(x, torch.Tensor) else (None, float(x))


def top_p_fp32_return_mask(probs: torch.Tensor, top_p: Union[torch.Tensor, float]) -> torch.Tensor:
    """probs ``[B,H,1,L]`` fp32 -> bool mask of the tokens the top-p search keeps
    (twilight/kernel/cuda/sampling.py:127-133, csrc/src/sampling.cu:45-63)."""
    return torch.ops.twilight_b200.top_p_fp32_return_mask(probs, *_to_tensor_scalar_tuple(top_p))


def top_p_fp16_return_mask(probs: torch.Tensor, top_p: Union[torch.Tensor, float]) -> torch.Tensor:
    """fp16/bf16 form (twilight/kernel/cuda/sampling.py:118-124, csrc/src/sampling.cu:22-43)."""
    return torch.ops.twilight_b200.top_p_fp16_return_mask(probs, *_to_tensor_scalar_tuple(top_p))


def _launch(name: str, on: torch.Tensor, *args, **same_device: Optional[torch.Tensor]) -> None:
    """Calls entry point ``twl_<name>`` with ``on``'s device current (the library launches on the
    current device); the keyword tensors are checked to live on that device.  Raises
    :class:`TwilightError` on a non-zero status."""
    lib = _lib.load()
    with _on(on, **same_device):
        st = getattr(lib, "twl_" + name)(*args)
    _lib.check(st, name)


# ---------------------------------------------------------------------------------------------
# index-list operators
# ---------------------------------------------------------------------------------------------
def quest_page_scores(q, kmeta, kv_indptr, kv_indices, *, max_pages: int, page_scores=None, status=None
                      ) -> torch.Tensor:
    """Quest's per-page upper bounds ``sum_d max(q_d*kmax_d, q_d*kmin_d)`` from the stored page
    metadata, fp32 ``[B,H,max_pages]`` (twilight/pyimpl/quest.py:37-84)."""
    q = _q3(q)
    b, hq, _ = q.shape
    if page_scores is None:
        page_scores = torch.empty(b, hq, max_pages, dtype=torch.float32, device=q.device)
    _launch("quest_page_scores", q, q.data_ptr(), _dtype_code(q), kmeta.data_ptr(), kv_indptr.data_ptr(),
            kv_indices.data_ptr(), b, hq, kmeta.shape[1], kmeta.shape[0], page_scores.data_ptr(), max_pages,
            _p(status), _stream(q.device), kmeta=kmeta, page_scores=page_scores, status=status)
    return page_scores


def quest_select(q, kmeta, kv_indptr, kv_indices, token_budget: int, *, max_pages: int,
                 page_scores=None, cand_pages=None, cand_npages=None, status=None, counters=None
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quest selector on stored page metadata (twilight/pyimpl/quest.py:17-122).

    Returns ``(cand_pages[B,H,max_k] int32 ascending, cand_npages[B,H] int32, page_scores)``.
    With ``counters`` (zeroed int32 ``[B*H_kv]``) scoring and selection run as one kernel."""
    q = _q3(q)
    b, hq, _ = q.shape
    n_total, hkv = kmeta.shape[0], kmeta.shape[1]
    max_k = max(1, token_budget // PAGE) + (1 if token_budget % PAGE else 0)
    max_k = min(max_k, max_pages)
    dev = q.device
    if page_scores is None:
        page_scores = torch.empty(b, hq, max_pages, dtype=torch.float32, device=dev)
    if cand_pages is None:
        cand_pages = torch.empty(b, hq, max_k, dtype=torch.int32, device=dev)
    if cand_npages is None:
        cand_npages = torch.empty(b, hq, dtype=torch.int32, device=dev)
    s = _stream(dev)
    if counters is not None:
        _launch("quest_select", q, q.data_ptr(), _dtype_code(q), kmeta.data_ptr(), kv_indptr.data_ptr(),
                kv_indices.data_ptr(), b, hq, hkv, n_total, token_budget, page_scores.data_ptr(), max_pages,
                cand_pages.data_ptr(), cand_npages.data_ptr(), cand_pages.shape[-1], counters.data_ptr(),
                _p(status), s, kmeta=kmeta, page_scores=page_scores, cand_pages=cand_pages, status=status)
        return cand_pages, cand_npages, page_scores
    _launch("quest_page_scores", q, q.data_ptr(), _dtype_code(q), kmeta.data_ptr(), kv_indptr.data_ptr(),
            kv_indices.data_ptr(), b, hq, hkv, n_total, page_scores.data_ptr(), max_pages, _p(status), s,
            kmeta=kmeta, page_scores=page_scores, status=status)
    _launch("quest_topk_pages", page_scores, page_scores.data_ptr(), max_pages, kv_indptr.data_ptr(), b, hq,
            token_budget, cand_pages.data_ptr(), cand_npages.data_ptr(), cand_pages.shape[-1], s,
            cand_pages=cand_pages, cand_npages=cand_npages)
    return cand_pages, cand_npages, page_scores


def quest_topk(page_scores, kv_indptr, token_budget: int, *, max_pages: int, cand_pages=None,
               cand_npages=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The selection half of :func:`quest_select` on given fp32 scores ``[B,H,max_pages]``:
    ascending positions of the ``max(1, budget//16) + (budget%16 != 0)`` best entries of each row
    (twilight/pyimpl/quest.py:93-99), ties to the lower position."""
    _cuda_contig(page_scores, "page_scores")
    b, hq, stride = page_scores.shape
    assert stride == max_pages and page_scores.dtype == torch.float32
    max_k = min(max(1, token_budget // PAGE) + (1 if token_budget % PAGE else 0), max_pages)
    dev = page_scores.device
    if cand_pages is None:
        cand_pages = torch.empty(b, hq, max_k, dtype=torch.int32, device=dev)
    if cand_npages is None:
        cand_npages = torch.empty(b, hq, dtype=torch.int32, device=dev)
    _launch("quest_topk_pages", page_scores, page_scores.data_ptr(), max_pages, kv_indptr.data_ptr(), b, hq,
            token_budget, cand_pages.data_ptr(), cand_npages.data_ptr(), cand_pages.shape[-1], _stream(dev),
            cand_pages=cand_pages, cand_npages=cand_npages)
    return cand_pages, cand_npages, page_scores


def estimate_int4(q, k4_pages, kv_indptr, kv_indices, kv_last_page_len, *, max_pages: int,
                  cand_pages=None, cand_npages=None, sm_scale: Optional[float] = None,
                  scores=None, variant: int = 0, status=None) -> torch.Tensor:
    """INT4 K-cache estimator (twilight/pyimpl/attention.py:247-255): fp32 scores
    ``[B,H,stride]``; slot s of a row is token ``cand_pages[s//16]*16+s%16`` (or token s when
    no candidate list is given)."""
    q = _q3(q)
    b, hq, _ = q.shape
    n_total, hkv = k4_pages.shape[0], k4_pages.shape[1]
    max_k = 0 if cand_pages is None else cand_pages.shape[-1]
    stride = (max_k if cand_pages is not None else max_pages) * PAGE
    if scores is None:
        scores = torch.empty(b, hq, stride, dtype=torch.float32, device=q.device)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(HEAD_DIM)
    _launch("estimate_int4", q, q.data_ptr(), _dtype_code(q), k4_pages.data_ptr(), kv_indptr.data_ptr(),
            kv_indices.data_ptr(), kv_last_page_len.data_ptr(), _p(cand_pages), _p(cand_npages), max_k, b,
            hq, hkv, n_total, sm_scale, scores.data_ptr(), scores.shape[-1], variant, _p(status),
            _stream(q.device), k4_pages=k4_pages, scores=scores, cand_pages=cand_pages, status=status)
    return scores


def topp_prune(scores, kv_indptr, kv_last_page_len, top_p: Union[torch.Tensor, float], *,
               cand_pages=None, cand_npages=None, indices=None, budget=None, threshold=None,
               status=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax + top-p search + compaction (twilight/pyimpl/top_p.py:10-15 and
    attention.py:280-285).  Returns ``(indices[B,H,stride] int32, budget[B,H] int32)``; the first
    ``budget`` entries of a row are the kept token positions in ascending order."""
    _cuda_contig(scores, "scores")
    b, hq, stride = scores.shape
    dev = scores.device
    if indices is None:
        indices = torch.empty(b, hq, stride, dtype=torch.int32, device=dev)
    if budget is None:
        budget = torch.empty(b, hq, dtype=torch.int32, device=dev)
    arr, val = (top_p, 0.0) if isinstance(top_p, torch.Tensor) else (None, float(top_p))
    if arr is not None:
        arr = arr.to(device=dev, dtype=torch.float32).contiguous()
    max_k = 0 if cand_pages is None else cand_pages.shape[-1]
    _launch("topp_prune", scores, scores.data_ptr(), stride, kv_indptr.data_ptr(),
            kv_last_page_len.data_ptr(), _p(cand_pages), _p(cand_npages), max_k, b, hq, _p(arr), val,
            indices.data_ptr(), indices.shape[-1], budget.data_ptr(), _p(threshold), _p(status),
            _stream(dev), indices=indices, budget=budget, cand_pages=cand_pages, status=status)
    return indices, budget


def threshold_prune(scores, kv_indptr, kv_last_page_len, threshold: float, *, cand_pages=None,
                    cand_npages=None, indices=None, budget=None, cut=None, status=None
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Element-wise threshold pruner (twilight/pyimpl/elementwise_threshold.py:9-18) in index-list
    form: keeps candidates whose score exceeds ``score(token 0) - threshold``."""
    _cuda_contig(scores, "scores")
    b, hq, stride = scores.shape
    dev = scores.device
    if indices is None:
        indices = torch.empty(b, hq, stride, dtype=torch.int32, device=dev)
    if budget is None:
        budget = torch.empty(b, hq, dtype=torch.int32, device=dev)
    max_k = 0 if cand_pages is None else cand_pages.shape[-1]
    _launch("threshold_prune", scores, scores.data_ptr(), stride, kv_indptr.data_ptr(),
            kv_last_page_len.data_ptr(), _p(cand_pages), _p(cand_npages), max_k, b, hq, float(threshold),
            indices.data_ptr(), indices.shape[-1], budget.data_ptr(), _p(cut), _p(status), _stream(dev),
            indices=indices, budget=budget, cand_pages=cand_pages, status=status)
    return indices, budget


def prune_with_weights(scores, kv_indptr, kv_last_page_len, value, *, mode: str = "top_p",
                       cand_pages=None, cand_npages=None, indices=None, budget=None, weights=None,
                       threshold=None, status=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Top-p (``mode="top_p"``) or element-wise threshold (``mode="threshold"``) pruner that also
    returns, for every kept token, its un-normalised softmax weight over the estimated logits
    (for attention with ``use_estimated_weights_in_attn``, twilight/pyimpl/attention.py:295-296).
    Returns ``(indices, budget, weights[B,H,stride] fp32)``."""
    _cuda_contig(scores, "scores")
    b, hq, stride = scores.shape
    dev = scores.device
    if indices is None:
        indices = torch.empty(b, hq, stride, dtype=torch.int32, device=dev)
    if budget is None:
        budget = torch.empty(b, hq, dtype=torch.int32, device=dev)
    if weights is None:
        weights = torch.empty(b, hq, indices.shape[-1], dtype=torch.float32, device=dev)
    arr, val = (value, 0.0) if isinstance(value, torch.Tensor) else (None, float(value))
    if arr is not None:
        arr = arr.to(device=dev, dtype=torch.float32).contiguous()
    max_k = 0 if cand_pages is None else cand_pages.shape[-1]
    _launch("prune_with_weights", scores, {"top_p": 0, "threshold": 1}[mode], scores.data_ptr(), stride,
            kv_indptr.data_ptr(), kv_last_page_len.data_ptr(), _p(cand_pages), _p(cand_npages), max_k, b,
            hq, _p(arr), val, indices.data_ptr(), indices.shape[-1], budget.data_ptr(), _p(threshold),
            weights.data_ptr(), _p(status), _stream(dev), indices=indices, budget=budget, weights=weights,
            status=status)
    return indices, budget, weights


def sparse_attn_workspace_bytes(batch: int, num_q_heads: int, index_stride: int, chunk: int = 256
                                ) -> int:
    return int(_lib.load().twl_sparse_attn_workspace_bytes(batch, num_q_heads, index_stride, chunk))


def sparse_decode_attn(q, k_pages, v_pages, kv_indptr, kv_indices, indices, budget, *,
                       sm_scale: Optional[float] = None, out=None, workspace=None,
                       chunk: int = 256, status=None, weights=None) -> torch.Tensor:
    """Attention of each (batch, query head) over its kept tokens
    (twilight/pyimpl/attention.py:188-190, :298-306).  Returns ``[B,H,D]`` in q's dtype.
    ``workspace``: zero-initialised uint8 tensor of ``sparse_attn_workspace_bytes`` bytes.
    ``weights`` (from :func:`prune_with_weights`): attend with these weights instead of exact
    q.k logits (attention.py:295-296); K is then not read."""
    q = _q3(q)
    b, hq, _ = q.shape
    n_total, hkv = k_pages.shape[0], k_pages.shape[1]
    stride = indices.shape[-1]
    if out is None:
        out = torch.empty(b, hq, HEAD_DIM, dtype=q.dtype, device=q.device)
    if workspace is None:
        workspace = torch.zeros(sparse_attn_workspace_bytes(b, hq, stride, chunk), dtype=torch.uint8,
                                device=q.device)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(HEAD_DIM)
    if weights is not None:
        _launch("sparse_decode_attn_weighted", q, q.data_ptr(), _dtype_code(q), k_pages.data_ptr(),
                v_pages.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(), indices.data_ptr(), stride,
                budget.data_ptr(), weights.data_ptr(), b, hq, hkv, n_total, sm_scale, out.data_ptr(),
                workspace.data_ptr(), workspace.numel(), chunk, _p(status), _stream(q.device),
                k_pages=k_pages, v_pages=v_pages, out=out, workspace=workspace, indices=indices,
                status=status)
        return out
    _launch("sparse_decode_attn", q, q.data_ptr(), _dtype_code(q), k_pages.data_ptr(), v_pages.data_ptr(),
            kv_indptr.data_ptr(), kv_indices.data_ptr(), indices.data_ptr(), stride, budget.data_ptr(), b,
            hq, hkv, n_total, sm_scale, out.data_ptr(), workspace.data_ptr(), workspace.numel(), chunk,
            _p(status), _stream(q.device), k_pages=k_pages, v_pages=v_pages, out=out, workspace=workspace,
            indices=indices, status=status)
    return out


STATIC_ATTN_MAX_ROWS = 512


def sparse_decode_attn_static(q, k_pages, v_pages, kv_indptr, kv_indices, indices, budget, *,
                              out: torch.Tensor, sm_scale: Optional[float] = None, chunk: int = 256,
                              status=None) -> torch.Tensor:
    """:func:`sparse_decode_attn` on scratch memory that is part of the library itself, for
    callers that cannot allocate device memory after start-up (a process whose own pool holds all
    of it, a plugin called where allocation is forbidden).  ``out`` must be supplied; nothing is
    allocated here or in the library.  At most ``STATIC_ATTN_MAX_ROWS`` (batch x query heads) rows.
    All calls on a device share one scratch array, so calls that could overlap on the GPU must
    not be issued; make the first call on a device outside any stream capture."""
    q = _q3(q)
    b, hq, _ = q.shape
    n_total, hkv = k_pages.shape[0], k_pages.shape[1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(HEAD_DIM)
    _launch("sparse_decode_attn_static", q, q.data_ptr(), _dtype_code(q), k_pages.data_ptr(),
            v_pages.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(), indices.data_ptr(),
            indices.shape[-1], budget.data_ptr(), b, hq, hkv, n_total, sm_scale, out.data_ptr(), chunk,
            _p(status), _stream(q.device), k_pages=k_pages, v_pages=v_pages, out=out, indices=indices,
            status=status)
    return out


def round_scores(scores: torch.Tensor, dtype: torch.dtype, post_scale: float = 1.0) -> torch.Tensor:
    """In place: ``scores <- round(round(scores) * post_scale)``, rounding to ``dtype`` (fp16/bf16), on
    an fp32 tensor.  Reproduces the model-dtype results of the reference's matmuls
    (twilight/pyimpl/quest.py:76-84, attention.py:252-254) on this library's fp32 scores."""
    _cuda_contig(scores, "scores")
    if scores.dtype != torch.float32:
        raise _lib.TwilightError("round_scores works on float32 scores")
    code = _dtype_code(torch.empty(0, dtype=dtype))
    _launch("round_scores", scores, scores.data_ptr(), scores.numel(), code, float(post_scale),
            _stream(scores.device))
    return scores


PRUNER_CODES = {"top_p": 0, "threshold": 1, "none": 2}
STEP_ESTIMATED_WEIGHTS, STEP_ROUND_TO_DTYPE = 1, 2


def step_workspace_layout(batch: int, num_q_heads: int, max_pages: int, token_budget: int,
                          attn_chunk: int = 256, flags: int = 0) -> "_lib.StepLayout":
    """Byte offsets of the parts of the one-buffer workspace of :func:`select_prune_attend_step`
    (``twl_step_workspace_layout``)."""
    lay = _lib.StepLayout()
    import ctypes
    _lib.check(_lib.load().twl_step_workspace_layout(batch, num_q_heads, max_pages, token_budget, attn_chunk,
                                                     flags, ctypes.addressof(lay)), "step_workspace_layout")
    return lay


def select_prune_attend_step(q, k_pages, v_pages, k4_pages, kmeta, kv_indptr, kv_indices, kv_last_page_len, *,
                             max_pages: int, token_budget: int, pruner: str, pruner_value: float,
                             out: torch.Tensor, workspace: torch.Tensor, top_p_arr=None,
                             sm_scale: Optional[float] = None, flags: int = 0, variant: int = 0,
                             attn_chunk: int = 256, status=None) -> torch.Tensor:
    """The decode step of one layer as ONE C-ABI call (``twl_select_prune_attend_step``): Quest
    selection when ``token_budget > 0``, INT4 estimate, pruner, sparse attention
    (twilight/pyimpl/attention.py:188-306).  ``workspace``: uint8 tensor of
    ``step_workspace_layout(...).total`` bytes, zeroed once after allocation."""
    q = _q3(q)
    b, hq, _ = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(HEAD_DIM)
    arr = None
    if top_p_arr is not None:
        arr = top_p_arr.to(device=q.device, dtype=torch.float32).contiguous()
    _launch("select_prune_attend_step", q, q.data_ptr(), _dtype_code(q), k_pages.data_ptr(), v_pages.data_ptr(),
            k4_pages.data_ptr(), _p(kmeta), kv_indptr.data_ptr(), kv_indices.data_ptr(),
            kv_last_page_len.data_ptr(), b, hq, k_pages.shape[1], k_pages.shape[0], max_pages, token_budget,
            PRUNER_CODES[pruner], float(pruner_value), _p(arr), sm_scale, flags, variant, attn_chunk,
            out.data_ptr(), workspace.data_ptr(), workspace.numel(), _p(status), _stream(q.device),
            k_pages=k_pages, v_pages=v_pages, k4_pages=k4_pages, kmeta=kmeta, out=out, workspace=workspace,
            status=status, kv_indptr=kv_indptr, kv_indices=kv_indices)
    return out


# ---------------------------------------------------------------------------------------------
# cache-append side
# ---------------------------------------------------------------------------------------------
def quantize_k_pages(k_pages: torch.Tensor, k4_pages: Optional[torch.Tensor] = None) -> torch.Tensor:
    """K pages ``[P,Hkv,16,128]`` -> INT4 slabs ``[P,Hkv,1280]`` uint8, group 32
    (twilight/pyimpl/quantize.py:4-13 per group, arithmetic in the cache dtype)."""
    _cuda_contig(k_pages, "k_pages")
    p, hkv = k_pages.shape[0], k_pages.shape[1]
    if k4_pages is None:
        k4_pages = torch.empty(p, hkv, K4_SLAB_BYTES, dtype=torch.uint8, device=k_pages.device)
    _launch("quantize_k_pages", k_pages, k_pages.data_ptr(), _dtype_code(k_pages), k4_pages.data_ptr(),
            p * hkv, _stream(k_pages.device), k4_pages=k4_pages)
    return k4_pages


def build_page_meta(k_pages, kv_indptr, kv_indices, kv_last_page_len, *, max_pages: int,
                    kmeta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Channel-wise (min,max) of every page ``[P,Hkv,2,128]`` (stored form of the chunk maxima of
    twilight/pyimpl/quest.py:39-74)."""
    _cuda_contig(k_pages, "k_pages")
    p, hkv = k_pages.shape[0], k_pages.shape[1]
    b = kv_indptr.numel() - 1
    if kmeta is None:
        kmeta = torch.zeros(p, hkv, 2, HEAD_DIM, dtype=k_pages.dtype, device=k_pages.device)
    _launch("build_page_meta", k_pages, k_pages.data_ptr(), _dtype_code(k_pages), kmeta.data_ptr(),
            kv_indptr.data_ptr(), kv_indices.data_ptr(), kv_last_page_len.data_ptr(), b, hkv, p, max_pages,
            _stream(k_pages.device), kmeta=kmeta)
    return kmeta


def append_kv(new_k, new_v, k_pages, v_pages, k4_pages, kmeta, kv_indptr, kv_indices,
              kv_last_page_len, status=None) -> None:
    """Writes one token per sequence (``new_k/new_v [B,Hkv,128]``) at the last position the page
    table describes, with its INT4 codes and the page metadata update."""
    _cuda_contig(new_k, "new_k")
    _cuda_contig(new_v, "new_v")
    b, hkv, _ = new_k.shape
    _launch("append_kv", new_k, new_k.data_ptr(), new_v.data_ptr(), _dtype_code(new_k), k_pages.data_ptr(),
            v_pages.data_ptr(), _p(k4_pages), _p(kmeta), kv_indptr.data_ptr(), kv_indices.data_ptr(),
            kv_last_page_len.data_ptr(), b, hkv, k_pages.shape[0], _p(status), _stream(new_k.device),
            k_pages=k_pages, v_pages=v_pages, k4_pages=k4_pages, kmeta=kmeta, status=status)


def indices_to_mask(indices, budget, seq_len: int) -> torch.Tensor:
    """Index lists -> the reference's mask layout ``bool[B,H,1,L]`` (attention.py:199-281)."""
    b, hq, stride = indices.shape
    mask = torch.zeros(b, hq, 1, seq_len, dtype=torch.bool, device=indices.device)
    _launch("indices_to_mask", indices, indices.data_ptr(), stride, budget.data_ptr(), b * hq,
            mask.data_ptr(), seq_len, _stream(indices.device), budget=budget, mask=mask)
    return mask


def batched_sparse_gemv_int4_k(q, o, k_cache_int4, quant_scales, quant_zeros, kv_page_indices,
                               kv_page_indptr, kv_last_page_len):
    """Same name and argument order as the absent ``ftka.cuda_ops.gemv`` op called at
    benchmark/efficiency/bench_gemv.py:445-454: raw ``q.k`` (no 1/sqrt(D)) of every token of
    every sequence written into ``o [B,H,L]``.  Differences, all forced by the group-32 cache:
    ``k_cache_int4`` is the slab tensor ``[P,Hkv,1280]`` that already carries scale and minimum,
    so ``quant_scales``/``quant_zeros`` must be ``None``; page size is 16; ``o`` is fp32 and its
    last dimension a multiple of 16."""
    if quant_scales is not None or quant_zeros is not None:
        raise _lib.TwilightError("scale/min live inside the INT4 slabs; pass None for both")
    if o.dtype != torch.float32 or o.shape[-1] % PAGE:
        raise _lib.TwilightError("o must be float32 with a last dimension that is a multiple of 16")
    estimate_int4(q, k_cache_int4, kv_page_indptr, kv_page_indices, kv_last_page_len,
                  max_pages=o.shape[-1] // PAGE, sm_scale=1.0, scores=o)
    return o
