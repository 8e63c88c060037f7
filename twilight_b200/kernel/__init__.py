"""``twilight_b200.kernel``: the operator API (same role and names as ``twilight.kernel`` of the
reference, twilight/kernel/__init__.py:1)."""
from .ops import (  # noqa: F401
    top_p_fp16_return_mask,
    top_p_fp32_return_mask,
    quest_select,
    quest_topk,
    estimate_int4,
    topp_prune,
    threshold_prune,
    prune_with_weights,
    sparse_decode_attn,
    sparse_attn_workspace_bytes,
    sparse_decode_attn_static,
    quantize_k_pages,
    build_page_meta,
    append_kv,
    indices_to_mask,
    batched_sparse_gemv_int4_k,
)
