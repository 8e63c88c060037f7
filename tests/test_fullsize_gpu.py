"""The benchmark configurations at their full sizes: size-independent properties over every row,
plus the oracle on a few sampled rows (the oracle is too slow for all of them)."""
import numpy as np
import pytest
import torch

from oracle import twilight_oracle as O
from tests import util as U
from twilight_b200.cache import PAGE, PagedKVCache, quest_max_k
from twilight_b200.gen import make_decode_inputs, ragged_lengths
from twilight_b200.kernel import ops
from twilight_b200.step import DecodeWorkspace, SparseConfig, select_prune_attend_step

pytestmark = pytest.mark.gpu
DEV = "cuda"
ATOL_MAX, ATOL_MEAN, P_TOL = 2e-2, 1e-3, 1e-4


def _properties(q, cache, ws, cfg, hq):
    """Checks that hold for every row whatever the inputs are."""
    b_n = cache.batch
    budget = ws.budget.cpu().numpy()
    stride = ws.indices.shape[-1]
    idx = ws.indices.cpu().numpy()
    lens = np.asarray(cache.seq_lens)
    pos = np.arange(stride)[None, None, :]
    valid = pos < budget[:, :, None]
    assert (budget >= 1).all() and (budget <= stride).all()
    # ascending, inside the sequence
    d = np.diff(idx, axis=-1)
    assert (d[valid[:, :, 1:]] > 0).all()
    assert (np.where(valid, idx, 0) >= 0).all()
    assert (np.where(valid, idx, 0) < lens[:, None, None]).all()
    if cfg.selector == "quest":
        # every kept token lies in a candidate page of its row
        npg = ws.cand_npages.cpu().numpy()
        cand = ws.cand_pages.cpu().numpy()
        for b in range(b_n):
            k = quest_max_k(cfg.token_budget, (lens[b] + PAGE - 1) // PAGE)
            assert (npg[b] == k).all()
            for h in range(0, hq, max(1, hq // 4)):
                pages = cand[b, h, :k]
                assert (np.diff(pages) > 0).all() and pages[-1] < (lens[b] + PAGE - 1) // PAGE
                assert np.isin(idx[b, h, : budget[b, h]] // PAGE, pages).all()
    # the mask form of the same result counts the same budgets (attention.py:280-285)
    mask = ops.indices_to_mask(ws.indices, ws.budget, int(lens.max()))
    assert torch.equal(mask.sum(-1).flatten().cpu(), torch.from_numpy(budget).flatten().long())
    assert torch.isfinite(ws.out.float()).all()
    assert int(ws.status.item()) == 0


def _oracle_rows(q, cache, ws, cfg, hq, rows):
    g = hq // cache.num_kv_heads
    errs = []
    for (b, h) in rows:
        n = cache.seq_lens[b]
        npg = (n + PAGE - 1) // PAGE
        if cfg.selector == "quest":
            k = int(ws.cand_npages[b, h])
            pages = ws.cand_pages[b, h, :k].cpu().numpy()
            want_scores = U.oracle_page_scores(q, cache, b, h, g)
            must, tie, thr = U.expected_candidates(want_scores, k)
            for pg in set(pages.tolist()) ^ (must | set(sorted(tie)[: k - len(must)])):
                assert abs(want_scores[pg] - thr) <= 1e-3 * max(1.0, abs(thr))
        else:
            pages = np.arange(npg)
        want_row, _ = U.oracle_scores_row(q, cache, b, h, g, pages)
        got_row = ws.scores[b, h, : len(pages) * PAGE].cpu().numpy()
        fin = np.isfinite(want_row)
        assert np.array_equal(np.isfinite(got_row), fin)
        assert np.abs(got_row[fin] - want_row[fin]).max() <= 2e-3 * max(1.0, float(np.abs(want_row[fin]).max()))
        probs, keep, low = U.oracle_prune_row(got_row, pages, cfg.threshold)   # identical input
        bud = int(ws.budget[b, h])
        got_idx = ws.indices[b, h, :bud].cpu().numpy()
        dd = U.check_index_parity(got_idx, probs, keep, low, pages, P_TOL)
        assert abs(bud - int(keep.sum())) <= dd
        kd, vd = cache.dense_kv(b, h // g)
        want_out = O.sparse_attention_fp32(q[b, h].float().cpu().numpy(), kd.float().cpu().numpy(),
                                           vd.float().cpu().numpy(), got_idx.astype(np.int64), U.SM_SCALE)
        errs.append(np.abs(ws.out[b, h].float().cpu().numpy() - want_out))
    errs = np.stack(errs)
    assert errs.max() <= ATOL_MAX and errs.mean() <= ATOL_MEAN


def _run_twice(q, cache, ws):
    select_prune_attend_step(q, cache, ws)
    torch.cuda.synchronize()
    b1, o1 = ws.budget.clone(), ws.out.clone()
    i1 = ws.indices.clone()
    select_prune_attend_step(q, cache, ws)
    torch.cuda.synchronize()
    assert torch.equal(ws.budget, b1)                      # budgets and index lists repeat bit for bit
    pos = torch.arange(i1.shape[-1], device=i1.device)[None, None, :]
    valid = pos < b1[:, :, None]
    assert torch.equal(torch.where(valid, ws.indices, 0), torch.where(valid, i1, 0))
    assert (ws.out.float() - o1.float()).abs().max() <= 1e-2


@pytest.mark.parametrize("recipe", ["literal", "mid"])
def test_config1_longchat7b_class(recipe):
    # B=16, 32 q = 32 kv heads, L=32768, Quest 8192, top-p 0.95, heavy-hitter density 0.5 %
    q, cache = make_decode_inputs(16, 32, 32, 32768, rho=0.005, dtype=torch.bfloat16, device=DEV, seed=1,
                                  recipe=recipe, shuffle_pages=True)
    cfg = SparseConfig(selector="quest", token_budget=8192, weight_pruner="top_p", threshold=0.95)
    ws = DecodeWorkspace.for_cache(cache, 32, cfg)
    _run_twice(q, cache, ws)
    _properties(q, cache, ws, cfg, 32)
    if recipe == "literal":
        assert (ws.budget == 1).all()
    _oracle_rows(q, cache, ws, cfg, 32, [(0, 0), (7, 13), (15, 31)])
    del ws, cache
    torch.cuda.empty_cache()


def test_config2_llama3_8b_class_ragged_gqa():
    # B=64, 32 q / 8 kv heads, ragged L in [8192, 32768], no selector, top-p 0.9, density per head 0.1-5 %
    lens = ragged_lengths(64, 8192, 32768, seed=2)
    q, cache = make_decode_inputs(64, 32, 8, lens, rho=(0.001, 0.05), dtype=torch.bfloat16, device=DEV, seed=2,
                                  recipe="mid", shuffle_pages=True)
    cfg = SparseConfig(selector="none", weight_pruner="top_p", threshold=0.9)
    ws = DecodeWorkspace.for_cache(cache, 32, cfg)
    _run_twice(q, cache, ws)
    _properties(q, cache, ws, cfg, 32)
    short = int(np.argmin(lens))
    _oracle_rows(q, cache, ws, cfg, 32, [(short, 0), (short, 31), (63, 9)])
    # budgets adapt to the per-head density: heads of one KV head see the same keys
    assert float(ws.budget.float().std()) > 0
    del ws, cache
    torch.cuda.empty_cache()


def test_config4_llama3_70b_class_one_kv_head_shard():
    # one GPU's shard of B=128, 64 q / 8 kv heads: 8 q heads on 1 kv head, L=65536, Quest 16384, top-p 0.95
    q, cache = make_decode_inputs(128, 8, 1, 65536, rho=0.005, dtype=torch.bfloat16, device=DEV, seed=4,
                                  recipe="mid", shuffle_pages=True)
    cfg = SparseConfig(selector="quest", token_budget=16384, weight_pruner="top_p", threshold=0.95)
    ws = DecodeWorkspace.for_cache(cache, 8, cfg)
    _run_twice(q, cache, ws)
    _properties(q, cache, ws, cfg, 8)
    _oracle_rows(q, cache, ws, cfg, 8, [(0, 0), (127, 7)])
    del ws, cache
    torch.cuda.empty_cache()


@pytest.mark.parametrize("batch,L", [(1, 4096), (16, 16384), (64, 65536), (16, 131072)])
def test_config3_gemv_sweep(batch, L):
    # standalone INT4 GEMV: rows = B*32, fp16 queries, group-32 fp16 scale/min, fp32 scores.
    # The slabs are filled with random codes and scales directly (the kernel only sees the format).
    hkv = 32
    n_pages = L // PAGE
    g = torch.Generator(device=DEV).manual_seed(L + batch)
    total = batch * n_pages
    k4 = torch.empty(total, hkv, 1280, dtype=torch.uint8, device=DEV)
    k4[:, :, :1024] = torch.randint(0, 256, (total, hkv, 1024), generator=g, device=DEV, dtype=torch.uint8)
    sz = torch.empty(total, hkv, 64, 2, dtype=torch.float16, device=DEV)
    sz[..., 0] = (torch.rand(total, hkv, 64, generator=g, device=DEV) * 0.4 + 0.05).half()
    sz[..., 1] = (torch.randn(total, hkv, 64, generator=g, device=DEV)).half()
    k4[:, :, 1024:] = sz.view(torch.uint8).reshape(total, hkv, 256)
    del sz
    q = torch.randn(batch, hkv, 128, generator=g, device=DEV).half()
    indptr, indices, last, _ = PagedKVCache.page_table([L] * batch, DEV, shuffle_seed=5)
    o = torch.empty(batch, hkv, L, dtype=torch.float32, device=DEV)
    ops.batched_sparse_gemv_int4_k(q, o, k4, None, None, indices, indptr, last)
    torch.cuda.synchronize()
    assert torch.isfinite(o).all()
    from twilight_b200.cache import unpack_k4
    for (b, h) in [(0, 0), (batch - 1, 31), (batch // 2, 17)]:
        lo, hi = int(indptr[b]), int(indptr[b + 1])
        phys = indices[lo:hi].long()
        codes, scale, zmin = unpack_k4(k4[phys, h].cpu())
        want = O.estimate_logits_from_codes(q[b, h].cpu(), codes.reshape(-1, 128), scale.reshape(-1, 4),
                                            zmin.reshape(-1, 4), 32, 1.0).numpy()
        got = o[b, h].cpu().numpy()
        assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max()
    # linearity in q: scores(2q) == 2*scores(q) up to the block scaling of q (a power of two: exact)
    o2 = torch.empty_like(o)
    ops.batched_sparse_gemv_int4_k((q * 2).contiguous(), o2, k4, None, None, indices, indptr, last)
    assert torch.equal(o2, o * 2)
    del k4, o, o2
    torch.cuda.empty_cache()
