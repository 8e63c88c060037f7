"""CPU checks of the host side: the INT4 slab format, the page table, the config dictionary,
the budget statistics, and that the C-ABI library loads and exports every declared symbol
(no kernel is launched here)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from twilight_b200 import _lib
from twilight_b200.cache import PagedKVCache, pack_k4, unpack_k4, quest_max_k
from twilight_b200.pyimpl.state import (HistoryBudgetInfo, IndexSelectorType, WeightEstimatorType,
                                        WeightPrunerType)
from twilight_b200.step import SparseConfig

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "twilight_b200.h").read_text()
    declared = set(re.findall(r"TWL_API\s+[\w\s\*]+?\b(twl_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    lib = ctypes.CDLL(str(_lib.lib_path()))
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.load().twl_version() >= 100
    assert _lib.load().twl_status_string(-6) == b"workspace missing or too small"


def test_bad_arguments_return_codes_without_a_gpu():
    lib = _lib.load()
    # null pointers / zero sizes are rejected before anything touches the device
    assert lib.twl_top_p_return_mask_f32(None, None, None, 0.9, 1, 8, None, None) == -1
    assert lib.twl_estimate_int4(None, 1, None, None, None, None, None, None, 0, 1, 1, 1, 1, 1.0,
                                 None, 16, 0, None, None) == -1
    assert lib.twl_sparse_attn_workspace_bytes(0, 1, 16, 256) == 0
    assert lib.twl_sparse_attn_workspace_bytes(2, 4, 1024, 256) >= 8 * 4 * (128 + 2) * 4
    with pytest.raises(_lib.TwilightError, match="bad argument"):
        _lib.check(-1, "x")


def test_k4_slab_nibble_order_and_roundtrip():
    codes = torch.arange(16 * 128, dtype=torch.int64).reshape(16, 128) % 16
    codes = ((codes + torch.arange(16)[:, None]) % 16).to(torch.uint8)
    scale = (torch.arange(64, dtype=torch.float32).reshape(16, 4) * 0.01 + 0.1).to(torch.float16)
    zmin = (-torch.arange(64, dtype=torch.float32).reshape(16, 4) * 0.5).to(torch.float16)
    slab = pack_k4(codes, scale, zmin)
    assert slab.shape == (1280,) and slab.dtype == torch.uint8
    # byte j of token t: channel 2j low nibble, 2j+1 high nibble
    t, j = 3, 17
    assert int(slab[t * 64 + j]) == int(codes[t, 2 * j]) | (int(codes[t, 2 * j + 1]) << 4)
    # {scale, min} of token t, group g at 1024 + t*16 + g*4
    raw = slab[1024 + 5 * 16 + 2 * 4: 1024 + 5 * 16 + 2 * 4 + 4].contiguous().view(torch.float16)
    assert raw[0] == scale[5, 2] and raw[1] == zmin[5, 2]
    c2, s2, z2 = unpack_k4(slab)
    assert torch.equal(c2, codes) and torch.equal(s2, scale) and torch.equal(z2, zmin)
    # every code value in every nibble position survives
    for v in range(16):
        full = torch.full((2, 16, 128), v, dtype=torch.uint8)
        c3, _, _ = unpack_k4(pack_k4(full, torch.ones(2, 16, 4), torch.zeros(2, 16, 4)))
        assert torch.equal(c3, full)


def test_page_table_ragged_and_shuffled():
    indptr, indices, last, total = PagedKVCache.page_table([1, 16, 17, 100], "cpu")
    assert indptr.tolist() == [0, 1, 2, 4, 11] and total == 11
    assert last.tolist() == [1, 16, 1, 4]
    assert indices.tolist() == list(range(11))
    _, shuf, _, _ = PagedKVCache.page_table([1, 16, 17, 100], "cpu", shuffle_seed=7)
    assert sorted(shuf.tolist()) == list(range(11)) and shuf.tolist() != list(range(11))


def test_quest_max_k_matches_reference_rule():
    assert quest_max_k(8192, 2048) == 512
    assert quest_max_k(16384, 4096) == 1024
    assert quest_max_k(40, 100) == 3
    assert quest_max_k(8192, 100) == 100


def test_config_dict_of_the_reference_parses():
    cfg = {  # benchmark/configs/config_quest_twi.json
        "compressor": {"type": "none"},
        "selector": {"type": "quest", "token_budget": 8192, "chunk_size": 16},
        "weight_estimator": {"type": "min_max_quant", "quant_bit": 4},
        "weight_pruner": {"type": "top_p", "threshold": 0.85},
        "skip_first_two_layers": True,
        "use_estimated_weights_in_attn": False,
    }
    c = SparseConfig.from_dict(cfg)
    assert (c.selector, c.token_budget, c.weight_pruner, c.threshold) == ("quest", 8192, "top_p", 0.85)
    cfg["selector"] = {"type": "sparq", "token_budget": 10}
    with pytest.raises(_lib.TwilightError):
        SparseConfig.from_dict(cfg)
    cfg["selector"] = {"type": "quest", "token_budget": 64, "chunk_size": 32}
    with pytest.raises(_lib.TwilightError):
        SparseConfig.from_dict(cfg)
    assert IndexSelectorType.from_str("quest") is IndexSelectorType.QUEST
    assert WeightEstimatorType.from_str("min_max_quant") is WeightEstimatorType.MIN_MAX_QUANT
    assert WeightPrunerType.from_str("top_p") is WeightPrunerType.TOP_P
    with pytest.raises(KeyError):
        IndexSelectorType.from_str("nope")


def test_history_budget_info_average_skips_first_two_layers():
    info = HistoryBudgetInfo()
    for query in range(2):
        for layer in range(4):
            mask = torch.zeros(1, 2, 1, 10, dtype=torch.bool)
            mask[..., : layer + 1 + query] = True
            info.update(layer, mask)
    # layers 2,3 only (state.py:217): query 0 -> (3+4)/2, query 1 -> (4+5)/2
    assert info.get_avg_budget_per_query() == [3.5, 4.5]
    assert info.get_total_avg_budget() == 4.0
    info2 = HistoryBudgetInfo()
    for layer in range(3):
        info2.update(layer, torch.tensor([[layer, layer + 2]], dtype=torch.int32))
    assert info2.get_avg_budget_per_query() == [3.0]


def test_operators_fail_loudly_without_cuda_tensors():
    from twilight_b200.kernel import top_p_fp32_return_mask
    with pytest.raises(_lib.TwilightError, match="CUDA tensor"):
        top_p_fp32_return_mask(torch.rand(1, 1, 1, 8), 0.9)


def test_growing_cache_page_table_follows_the_length():
    """Host side of the growing cache: every sequence owns consecutive pages from the start, the
    CSR table lists the pages in use, and its tensors are only rebuilt when a page is added."""
    from twilight_b200.cache import GrowingPagedCache, PAGE
    c = GrowingPagedCache(batch=3, num_kv_heads=2, max_len=100, dtype=torch.float16, device="cpu")
    assert c.pages_per_seq == 7 and c.k_pages.shape == (21, 2, PAGE, 128) and c.k4_pages.shape == (21, 2, 1280)
    c._set_length(16)
    v16 = c.view
    assert v16.kv_indptr.tolist() == [0, 1, 2, 3] and v16.kv_indices.tolist() == [0, 7, 14]
    assert v16.kv_last_page_len.tolist() == [16, 16, 16] and v16.seq_lens == [16, 16, 16]
    c._set_length(17)
    assert c.view.kv_indptr.tolist() == [0, 2, 4, 6] and c.view.kv_indices.tolist() == [0, 1, 7, 8, 14, 15]
    assert c.view.kv_last_page_len.tolist() == [1, 1, 1] and c.view.capacity_pages == 7 and c.view.max_pages == 2
    idx17 = c.view.kv_indices
    c._set_length(18)
    assert c.view.kv_indices is idx17 and c.view.kv_last_page_len.tolist() == [2, 2, 2]   # same page count: reused
    with pytest.raises(ValueError):
        c._set_length(101)


def test_device_guard_helpers():
    """Every C-ABI call runs with the tensors' device current and refuses tensors of other devices."""
    from twilight_b200.kernel import ops
    cpu = torch.zeros(4)
    with pytest.raises(_lib.TwilightError, match="CUDA tensors only"):
        ops._on(cpu)
    meta0 = torch.empty(1, device="meta")
    with pytest.raises(_lib.TwilightError, match="out is on meta"):
        ops._same_device(torch.device("cuda", 1), q=None, out=meta0)
    ops._same_device(torch.device("cpu"), a=cpu, b=None)      # same device, None is skipped
    with pytest.raises(_lib.TwilightError, match="CUDA tensors only"):
        ops._launch("version", cpu)


def test_mask_operators_are_registered_custom_ops_with_shape_inference():
    """The reference registers both mask operators as torch custom ops without mutated arguments
    (twilight/kernel/cuda/sampling.py:62-100); here they live under ``torch.ops.twilight_b200`` and
    carry a fake-tensor rule, so tracing needs no GPU."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from twilight_b200 import kernel
    for name in ("top_p_fp32_return_mask", "top_p_fp16_return_mask"):
        op = getattr(torch.ops.twilight_b200, name)
        schema = op.default._schema
        assert [a.name for a in schema.arguments] == ["probs", "maybe_top_p_arr", "top_p_val"]
        assert not any(a.alias_info is not None and a.alias_info.is_write for a in schema.arguments)
    with FakeTensorMode():
        probs = torch.empty(2, 3, 1, 64, device="cuda", dtype=torch.float16)
        m = kernel.top_p_fp16_return_mask(probs, 0.9)
        assert m.shape == probs.shape and m.dtype == torch.bool and m.device == probs.device
        m = kernel.top_p_fp32_return_mask(probs.float(), torch.empty(6, device="cuda"))
        assert m.shape == probs.shape and m.dtype == torch.bool


def test_step_workspace_layout_is_consistent():
    from twilight_b200.kernel import ops
    lib = _lib.load()
    for (b, h, pages, budget, flags) in [(16, 32, 2048, 8192, 0), (64, 32, 2048, 0, 0), (2, 8, 7, 1000, 3),
                                         (1, 1, 1, 16, 1)]:
        lay = ops.step_workspace_layout(b, h, pages, budget, 256, flags)
        assert lay.total == lib.twl_step_workspace_bytes(b, h, pages, budget, 256, flags)
        k = quest_max_k(budget, pages) if budget > 0 else 0
        stride = (k if budget > 0 else pages) * 16
        assert lay.max_k == k and lay.stride == stride
        assert lay.attn == 0 and lay.attn_bytes == lib.twl_sparse_attn_workspace_bytes(b, h, stride, 256)
        parts = [(lay.attn, lay.attn_bytes), (lay.page_scores, b * h * pages * 4 if budget > 0 else 0),
                 (lay.cand_pages, b * h * k * 4), (lay.cand_npages, b * h * 4 if budget > 0 else 0),
                 (lay.scores, b * h * stride * 4), (lay.indices, b * h * stride * 4), (lay.budget, b * h * 4),
                 (lay.threshold, b * h * 8), (lay.weights, b * h * stride * 4 if flags & 1 else 0)]
        end = 0
        for off, size in parts:                              # in order, 256-byte aligned, no overlap
            assert off % 256 == 0 and off >= end
            end = off + size
        assert lay.total >= end
        assert lay.kernels == (5 if budget > 0 else 3) + ((2 if budget > 0 else 1) if flags & 2 else 0)
    assert lib.twl_step_workspace_bytes(0, 1, 1, 0, 256, 0) == 0
    # null pointers are refused before anything is launched
    assert lib.twl_select_prune_attend_step(None, 1, None, None, None, None, None, None, None, 1, 1, 1, 1, 1, 0, 0,
                                            0.9, None, 0.088, 0, 0, 256, None, None, 0, None, None) == -1
    assert lib.twl_round_scores(None, 4, 1, 1.0, None) == -1
