"""GPU parity tests: every CUDA kernel, called through the C ABI, against the CPU oracle on the
same seeded inputs.  Integer results (codes, page lists, index lists, budgets, masks) must be
bit-exact, except kept-token sets, where tokens whose probability lies within 1e-4 of the
threshold are exempt; attention outputs must agree within 2e-2 max-abs / 1e-3 mean-abs."""
import numpy as np
import pytest
import torch

from oracle import twilight_oracle as O
from tests import util as U
from twilight_b200 import _lib
from twilight_b200.cache import PAGE, PagedKVCache, quest_max_k, unpack_k4
from twilight_b200.gen import make_decode_inputs, ragged_lengths
from twilight_b200.kernel import ops
from twilight_b200.step import DecodeWorkspace, SparseConfig, select_prune_attend_step

pytestmark = pytest.mark.gpu
DEV = "cuda"
ATOL_MAX, ATOL_MEAN, P_TOL = 2e-2, 1e-3, 1e-4


def _status_ok(ws):
    assert int(ws.status.item()) == 0, f"device status flags {int(ws.status.item())}"


# ---- cache-append side -------------------------------------------------------------------------
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_quantizer_codes_bit_exact(dt):
    g = torch.Generator().manual_seed(0)
    k = torch.randn(7, 3, PAGE, 128, generator=g) * 1.3
    k[0, 0, 0, :32] = 0.25          # constant group
    k[1, 1, 5] *= 20.0              # large-range row
    k[2, 2, 3, 64:96] = torch.linspace(-1, 1, 32)
    k = k.to(dt)
    k4 = ops.quantize_k_pages(k.to(DEV)).cpu()
    codes, scale, zmin = unpack_k4(k4)
    deq, ocodes, oscales, ozeros = O.quantize_min_max(k, 4, group=32)
    const = (k.reshape(7, 3, PAGE, 4, 32).amax(-1) == k.reshape(7, 3, PAGE, 4, 32).amin(-1))
    ok = ~const.unsqueeze(-1).expand(7, 3, PAGE, 4, 32).reshape(7, 3, PAGE, 128)
    assert torch.equal(codes[ok], ocodes[ok])
    assert (codes[~ok] == 0).all()  # constant groups: code 0 (the fp16 reference yields NaN here)
    assert torch.equal(scale[~const], oscales.to(torch.float16)[~const])
    assert torch.equal(zmin, (-ozeros).to(torch.float16))


def test_page_meta_and_append_match_bulk_build():
    lens = [1, 15, 16, 17, 33, 100]
    g = torch.Generator().manual_seed(1)
    lmax = max(lens)
    k = torch.randn(len(lens), 2, lmax, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(len(lens), 2, lmax, 128, generator=g).to(torch.bfloat16)
    full = PagedKVCache.from_dense(k.to(DEV), v.to(DEV), lens, shuffle_seed=3)
    for b, n in enumerate(lens):
        for h in range(2):
            kmin, kmax = full.dense_meta(b, h)
            kk = k[b, h, :n]
            npg = (n + PAGE - 1) // PAGE
            for pg in range(npg):
                seg = kk[pg * PAGE: min(n, pg * PAGE + PAGE)]
                assert torch.equal(kmin[pg].cpu(), seg.amin(0)) and torch.equal(kmax[pg].cpu(), seg.amax(0))
    # grow a second cache token by token with append_kv and compare everything that is defined
    grown = PagedKVCache.from_dense(k.to(DEV)[:, :, :1], v.to(DEV)[:, :, :1], [1] * len(lens), build_aux=False)
    total = full.k_pages.shape[0]
    grown.k_pages = torch.zeros_like(full.k_pages)
    grown.v_pages = torch.zeros_like(full.v_pages)
    grown.k4_pages = torch.zeros_like(full.k4_pages)
    grown.kmeta = torch.zeros_like(full.kmeta)
    grown.kv_indices = full.kv_indices
    grown.kv_indptr = full.kv_indptr.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for t in range(lmax):
        alive = [b for b, n in enumerate(lens) if t < n]
        # page table of the sequences that still grow: first t+1 tokens
        npg = [(min(t + 1, n) + PAGE - 1) // PAGE for n in lens]
        indptr_full = full.kv_indptr.cpu()
        sub_indices = torch.cat([full.kv_indices.cpu()[indptr_full[b]: indptr_full[b] + npg[b]] for b in alive])
        sub_indptr = torch.zeros(len(alive) + 1, dtype=torch.int32)
        sub_indptr[1:] = torch.tensor([npg[b] for b in alive], dtype=torch.int32).cumsum(0)
        sub_last = torch.full((len(alive),), t % PAGE + 1, dtype=torch.int32)
        ops.append_kv(k[alive, :, t].contiguous().to(DEV), v[alive, :, t].contiguous().to(DEV),
                      grown.k_pages, grown.v_pages, grown.k4_pages, grown.kmeta,
                      sub_indptr.to(DEV), sub_indices.to(DEV), sub_last.to(DEV), status=status)
    assert int(status.item()) == 0
    grown.kv_indptr, grown.seq_lens = full.kv_indptr, lens
    grown.kv_last_page_len = full.kv_last_page_len
    for b, n in enumerate(lens):
        for h in range(2):
            for a, c in zip(full.dense_kv(b, h), grown.dense_kv(b, h)):
                assert torch.equal(a, c)
            for a, c in zip(full.dense_k4(b, h), grown.dense_k4(b, h)):
                assert torch.equal(a, c)
            for a, c in zip(full.dense_meta(b, h), grown.dense_meta(b, h)):
                assert torch.equal(a, c)


# ---- selector ------------------------------------------------------------------------------------
@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 2), (8, 1)])
def test_quest_select_vs_oracle(hq, hkv):
    lens = [100, 1000, 257, 16]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV,
                                  seed=4, recipe="mid", shuffle_pages=True)
    budget = 160
    cand_pages, cand_npages, page_scores = ops.quest_select(
        q, cache.kmeta, cache.kv_indptr, cache.kv_indices, budget, max_pages=cache.max_pages)
    torch.cuda.synchronize()
    g = hq // hkv
    for b, n in enumerate(lens):
        npg = (n + PAGE - 1) // PAGE
        k = quest_max_k(budget, npg)
        for h in range(hq):
            want = U.oracle_page_scores(q, cache, b, h, g)
            got = page_scores[b, h, :npg].cpu().numpy()
            assert np.allclose(got, want, rtol=1e-5, atol=1e-4)
            assert int(cand_npages[b, h]) == k
            pages = cand_pages[b, h, :k].cpu().numpy()
            assert (np.diff(pages) > 0).all()
            # selection is exact with respect to the kernel's own scores, ties to lower pages
            must, tie, thr = U.expected_candidates(got, k)
            sel = set(pages.tolist())
            assert must <= sel <= (must | tie)
            need = k - len(must)
            assert sorted(sel - must) == sorted(tie)[:need]
            # and consistent with the oracle's scores up to rounding at the boundary
            omust, otie, othr = U.expected_candidates(want, k)
            for pg in sel ^ (omust | set(sorted(otie)[: k - len(omust)])):
                assert abs(want[pg] - othr) <= 1e-3 * max(1.0, abs(othr))


@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 2)])
def test_fused_quest_select_equals_two_step_form(hq, hkv):
    lens = [100, 1000, 257, 16, 4096]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV,
                                  seed=41, recipe="mid", shuffle_pages=True)
    counters = torch.zeros(len(lens) * hkv, dtype=torch.int32, device=DEV)
    for budget in (160, 17, 100000):
        a_pages, a_n, a_scores = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, budget,
                                                  max_pages=cache.max_pages)
        for _ in range(2):  # twice: the counters must come back to zero
            b_pages, b_n, b_scores = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, budget,
                                                      max_pages=cache.max_pages, counters=counters)
            torch.cuda.synchronize()
            assert int(counters.abs().sum()) == 0
            assert torch.equal(a_n, b_n)
            # groups of four or more query heads are scored on tensor cores in the two-step form and
            # with FMAs in the fused one: same products, another order of the fp32 additions
            same_kernel = hq // hkv < 4
            for b in range(len(lens)):
                npg = (lens[b] + PAGE - 1) // PAGE
                if same_kernel:
                    assert torch.equal(a_scores[b, :, :npg], b_scores[b, :, :npg])
                else:
                    assert torch.allclose(a_scores[b, :, :npg], b_scores[b, :, :npg], rtol=2e-6, atol=1e-4)
                for h in range(hq):
                    k = int(a_n[b, h])
                    if same_kernel:
                        assert torch.equal(a_pages[b, h, :k], b_pages[b, h, :k])
                    else:   # each selection is exact on its own scores; they differ only in near-ties
                        sc = b_scores[b, h, :npg].cpu().numpy()
                        must, tie, thr = U.expected_candidates(sc, k)
                        for pg in set(a_pages[b, h, :k].tolist()) ^ set(b_pages[b, h, :k].tolist()):
                            assert abs(sc[pg] - thr) <= 1e-4 * max(1.0, abs(thr))


def test_quest_selector_mask_interface_matches_reference_fixture(golden):
    from twilight_b200.pyimpl import quest_selector
    q = torch.from_numpy(golden["quest_q"]).to(torch.bfloat16).to(DEV)
    k = torch.from_numpy(golden["quest_k"]).to(torch.bfloat16).to(DEV)
    qf, kf = q.float().cpu(), k.float().cpu()
    scores = O.quest_page_scores(qf.reshape(2, 4, 1, 128), kf, 16)[:, :, 0].numpy()
    for budget in (32, 40, 1000):
        m = quest_selector(None, q, k, 16, token_budget=budget).cpu().numpy()
        ref = golden[f"quest_mask_bf16_{budget}"]
        assert m.shape == ref.shape
        kk = quest_max_k(budget, 7)
        for b in range(2):
            for h in range(4):
                diff_pages = set((np.nonzero(m[b, h, 0] != ref[b, h, 0])[0] // 16).tolist())
                thr = np.sort(scores[b, h])[::-1][kk - 1]
                # the reference ranks bf16-rounded scores; only pages tied with the k-th after
                # that rounding may differ
                for pg in diff_pages:
                    assert abs(scores[b, h, pg] - thr) <= 2 ** -7 * abs(thr) + 1e-3


# ---- estimator -------------------------------------------------------------------------------------
@pytest.mark.parametrize("variant,tol", [(1, 2e-4), (2, 6e-2), (3, 2e-3), (17, 2e-4), (19, 2e-3), (67, 2e-3)])
@pytest.mark.parametrize("hq,hkv,dt", [(4, 4, torch.float16), (8, 2, torch.bfloat16), (8, 1, torch.bfloat16),
                                       (4, 2, torch.float16)])
def test_estimator_full_context(variant, tol, hq, hkv, dt):
    lens = [1, 15, 16, 17, 31, 33, 700, 1025]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=5,
                                  recipe="literal", shuffle_pages=True)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices,
                               cache.kv_last_page_len, max_pages=cache.max_pages, variant=variant,
                               status=status)
    assert int(status.item()) == 0
    g = hq // hkv
    for b, n in enumerate(lens):
        npg = (n + PAGE - 1) // PAGE
        for h in range(hq):
            want, _ = U.oracle_scores_row(q, cache, b, h, g)
            got = scores[b, h, : npg * PAGE].cpu().numpy()
            assert np.array_equal(np.isinf(got), np.isinf(want))
            fin = np.isfinite(want)
            scale = max(1.0, float(np.abs(want[fin]).max()))
            assert np.abs(got[fin] - want[fin]).max() <= tol * scale, (variant, b, h)


@pytest.mark.parametrize("variant,tol", [(1, 2e-4), (3, 2e-3), (19, 2e-3), (67, 2e-3)])
def test_estimator_candidate_lists(variant, tol):
    lens = [300, 2000, 17]
    hq, hkv = 8, 2
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.01, dtype=torch.bfloat16, device=DEV,
                                  seed=6, recipe="mid", shuffle_pages=True)
    cand_pages, cand_npages, _ = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 512,
                                                  max_pages=cache.max_pages)
    scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices,
                               cache.kv_last_page_len, max_pages=cache.max_pages,
                               cand_pages=cand_pages, cand_npages=cand_npages, variant=variant)
    for b in range(len(lens)):
        for h in range(hq):
            k = int(cand_npages[b, h])
            pages = cand_pages[b, h, :k].cpu().numpy()
            want, _ = U.oracle_scores_row(q, cache, b, h, hq // hkv, pages)
            got = scores[b, h, : k * PAGE].cpu().numpy()
            assert np.array_equal(np.isinf(got), np.isinf(want))
            fin = np.isfinite(want)
            assert np.abs(got[fin] - want[fin]).max() <= tol * max(1.0, float(np.abs(want[fin]).max()))


def test_estimator_bulk_copy_rings_equal_the_default():
    """Variant +64 (warp-private rings fed by cp.async.bulk on per-warp mbarriers) moves the same
    bytes as the default's 16-byte cp.async copies and does the same integer arithmetic per
    (token, group); only the order in which the four groups' fp32 terms are added differs (a chain in
    one lane against two shuffles across four lanes): scores equal to a few ulp, with and without
    candidate lists, odd page counts included."""
    lens = [16, 17, 33, 1000, 4097, 8000]
    hq = hkv = 4
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV, seed=64,
                                  recipe="mid", shuffle_pages=True)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kw = dict(max_pages=cache.max_pages, status=status)
    a = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len, **kw)
    b_ = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                           variant=3 + 64, **kw)
    def close(x, y):
        assert torch.equal(torch.isinf(x), torch.isinf(y))
        fin = torch.isfinite(x)
        assert float((x[fin] - y[fin]).abs().max()) <= 1e-5 * max(1.0, float(x[fin].abs().max()))

    for b, n in enumerate(lens):
        npg = (n + PAGE - 1) // PAGE
        close(a[b, :, : npg * PAGE], b_[b, :, : npg * PAGE])
    cp, cn, _ = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 1000, max_pages=cache.max_pages)
    a = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                          cand_pages=cp, cand_npages=cn, **kw)
    b_ = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                           cand_pages=cp, cand_npages=cn, variant=3 + 64, **kw)
    for b in range(len(lens)):
        for h in range(hq):
            k = int(cn[b, h]) * PAGE
            close(a[b, h, :k], b_[b, h, :k])
    assert int(status.item()) == 0


def test_gemv_entry_with_the_reference_call_signature():
    lens = [64, 64]
    q, cache = make_decode_inputs(2, 4, 4, lens, dtype=torch.float16, device=DEV, seed=7)
    o = torch.empty(2, 4, 64, dtype=torch.float32, device=DEV)
    ops.batched_sparse_gemv_int4_k(q, o, cache.k4_pages, None, None, cache.kv_indices, cache.kv_indptr,
                                   cache.kv_last_page_len)
    codes, scale, zmin = (t.cpu() for t in cache.dense_k4(1, 2))
    want = O.estimate_logits_from_codes(q[1, 2].cpu(), codes, scale, zmin, 32, 1.0).numpy()
    assert np.abs(o[1, 2].cpu().numpy() - want).max() <= 2e-3 * np.abs(want).max()
    with pytest.raises(_lib.TwilightError):
        ops.batched_sparse_gemv_int4_k(q, o, cache.k4_pages, torch.ones(1), None, cache.kv_indices,
                                       cache.kv_indptr, cache.kv_last_page_len)


@pytest.mark.parametrize("hq,hkv", [(4, 2), (4, 4), (8, 1)])
def test_corrupt_page_table_is_flagged_not_followed(hq, hkv):
    """A page-table entry outside the cache must never be dereferenced: the selector scores the
    page -inf, the estimator writes -inf into its sixteen slots (so the pruner keeps none of its
    tokens), both raise FLAG_BAD_INDEX, and every other page comes out as without the corruption."""
    lens = [700, 300]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, dtype=torch.bfloat16, device=DEV, seed=41)
    good_scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                                    max_pages=cache.max_pages).clone()
    _, _, good_ps = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 64,
                                     max_pages=cache.max_pages)
    good_ps = good_ps.clone()
    bad = cache.kv_indices.clone()
    victim = 5                                       # page 5 of sequence 0
    bad[victim] = cache.k_pages.shape[0] + 123
    for entry in (bad, torch.where(torch.arange(bad.numel(), device=DEV) == victim, -7, cache.kv_indices).int()):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        scores = torch.full_like(good_scores, 777.0)
        ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, entry, cache.kv_last_page_len,
                          max_pages=cache.max_pages, scores=scores, status=status)
        assert int(status.item()) & ops.FLAG_BAD_INDEX
        lo, hi = victim * PAGE, (victim + 1) * PAGE
        assert torch.isinf(scores[0, :, lo:hi]).all() and (scores[0, :, lo:hi] < 0).all()
        idx, bud = ops.topp_prune(scores, cache.kv_indptr, cache.kv_last_page_len, 2.0)   # keep all with p > 0
        for h in range(hq):
            kept = idx[0, h, : int(bud[0, h])]
            assert not ((kept >= lo) & (kept < hi)).any()
            assert int(bud[0, h]) == lens[0] - PAGE
        keep = torch.ones(scores.shape[-1], dtype=torch.bool, device=DEV)
        keep[lo:hi] = False
        n1 = ((lens[1] + PAGE - 1) // PAGE) * PAGE     # slots past a sequence's pages are not written
        assert torch.equal(scores[0][:, keep].nan_to_num(neginf=-1e30), good_scores[0][:, keep].nan_to_num(neginf=-1e30))
        assert torch.equal(scores[1][:, :n1].nan_to_num(neginf=-1e30), good_scores[1][:, :n1].nan_to_num(neginf=-1e30))
        assert (scores[1][:, n1:] == 777.0).all()
        status.zero_()
        _, _, ps = ops.quest_select(q, cache.kmeta, cache.kv_indptr, entry, 64, max_pages=cache.max_pages,
                                    status=status)
        assert int(status.item()) & ops.FLAG_BAD_INDEX
        assert torch.isinf(ps[0, :, victim]).all() and (ps[0, :, victim] < 0).all()
        n0 = (lens[0] + PAGE - 1) // PAGE
        others = [i for i in range(n0) if i != victim]
        assert torch.equal(ps[0][:, others], good_ps[0][:, others])


# ---- pruner ------------------------------------------------------------------------------------------
def _prune_parity(q, cache, hq, top_p, cand_pages=None, cand_npages=None):
    scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices,
                               cache.kv_last_page_len, max_pages=cache.max_pages,
                               cand_pages=cand_pages, cand_npages=cand_npages)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    thr = torch.zeros(cache.batch, hq, 2, device=DEV)
    indices, budget = ops.topp_prune(scores, cache.kv_indptr, cache.kv_last_page_len, top_p,
                                     cand_pages=cand_pages, cand_npages=cand_npages, threshold=thr,
                                     status=status)
    assert int(status.item()) == 0
    exempt = 0
    for b, n in enumerate(cache.seq_lens):
        npg = (n + PAGE - 1) // PAGE
        for h in range(hq):
            if cand_pages is None:
                pages = np.arange(npg)
            else:
                pages = cand_pages[b, h, : int(cand_npages[b, h])].cpu().numpy()
            row = scores[b, h, : len(pages) * PAGE].cpu().numpy()   # identical input for both sides
            probs, keep, low = U.oracle_prune_row(row, pages, top_p)
            bud = int(budget[b, h])
            got = indices[b, h, :bud].cpu().numpy()
            assert (np.diff(got) > 0).all()
            d = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
            assert abs(bud - int(keep.sum())) <= d
            exempt += d
    return exempt, indices, budget


@pytest.mark.parametrize("recipe,top_p", [("literal", 0.95), ("mid", 0.95), ("calibrated", 0.9), ("mid", 1.0)])
def test_prune_full_context_vs_oracle(recipe, top_p):
    lens = [1, 15, 16, 17, 33, 700, 4096, 9000]
    hq, hkv = 8, 2
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.01, dtype=torch.bfloat16, device=DEV,
                                  seed=8, recipe=recipe, shuffle_pages=True)
    _prune_parity(q, cache, hq, top_p)


def test_prune_with_candidates_and_missing_sink():
    lens = [3000, 5000]
    hq, hkv = 4, 4
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.01, dtype=torch.float16, device=DEV,
                                  seed=9, recipe="mid")
    cand_pages, cand_npages, _ = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 1024,
                                                  max_pages=cache.max_pages)
    _prune_parity(q, cache, hq, 0.95, cand_pages, cand_npages)
    # drop page 0 from every list: token 0 is no longer a candidate, so nothing is pruned
    cp = cand_pages.clone()
    first_is_zero = cp[:, :, 0] == 0
    assert first_is_zero.any()
    cp[:, :, 0] = torch.where(first_is_zero, cp[:, :, 1], cp[:, :, 0])  # duplicate page 1: still ascending-ish
    scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                               max_pages=cache.max_pages, cand_pages=cp, cand_npages=cand_npages)
    _, budget = ops.topp_prune(scores, cache.kv_indptr, cache.kv_last_page_len, 0.95, cand_pages=cp,
                               cand_npages=cand_npages)
    nz = (torch.softmax(scores, -1) > 0).sum(-1)
    assert torch.equal(budget[first_is_zero].long(), nz[first_is_zero])


@pytest.mark.parametrize("n", [16, 2048, 8192, 40960, 40976, 65536])
def test_prune_synthetic_rows_all_paths(n):
    """Rows written directly (no estimator): up to 40960 slots a row is searched in shared memory
    with the working set squeezed to the search window, longer rows from global memory.  Shapes: one heavy sink,
    a flat row, a row where half the slots tie with the sink (the first round's survivors do not
    fit the list, so the search stays on the row), and a row whose kept set grows in later rounds."""
    g = torch.Generator(device=DEV).manual_seed(n)
    rows = []
    a = torch.randn(n, generator=g, device=DEV) * 2.0
    a[0] += 8.0
    rows.append(a)
    rows.append(torch.randn(n, generator=g, device=DEV) * 0.1)
    t = torch.randn(n, generator=g, device=DEV)
    t[: max(1, n // 2)] = 6.0
    rows.append(t)
    s = torch.randn(n, generator=g, device=DEV)
    s[0] = 3.0
    s[1: 1 + min(n - 1, 300)] = 5.0       # many tokens above the sink: low stays 0 in round one
    rows.append(s)
    scores = torch.stack(rows).reshape(1, 4, n).contiguous()
    indptr, _, last, _ = PagedKVCache.page_table([n], DEV)
    thr = torch.zeros(1, 4, 2, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    idx, bud, w = ops.prune_with_weights(scores, indptr, last, 0.9, mode="top_p", threshold=thr, status=status)
    idx2, bud2 = ops.topp_prune(scores, indptr, last, 0.9)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(bud, bud2)
    pages = np.arange(n // PAGE)
    for r in range(4):
        row = scores[0, r].cpu().numpy()
        probs, keep, low = U.oracle_prune_row(row, pages, 0.9)
        k = int(bud[0, r])
        got = idx[0, r, :k].cpu().numpy()
        assert np.array_equal(got, idx2[0, r, :k].cpu().numpy())
        assert (np.diff(got) > 0).all()
        d = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
        assert abs(k - int(keep.sum())) <= d
        np.testing.assert_allclose(w[0, r, :k].cpu().numpy(), probs[got], rtol=2e-3, atol=1e-9)
        assert abs(float(thr[0, r, 1]) - probs[0]) <= 2e-3 * probs[0] + 1e-9     # probability of token 0
        assert abs(float(thr[0, r, 0]) - float(low)) <= P_TOL


@pytest.mark.parametrize("n", [8192, 16384, 32768])
def test_prune_rows_that_overload_one_lane_of_the_window_search(n):
    """The block-wide search lets every lane collect the window elements among the slots it reads
    (four consecutive slots of every 128 of its warp's slice).  Rows whose large values all sit in
    the slots of the same lanes make those lanes' columns overflow, so the warps stay on the row
    and try again in later rounds; flat rows with a large or a tiny token 0 run many or few
    rounds.  All against the oracle."""
    g = torch.Generator(device=DEV).manual_seed(1000 + n)
    pos = torch.arange(n, device=DEV)
    rows = []
    a = torch.randn(n, generator=g, device=DEV) * 0.3 - 6.0
    a[(pos % 128) < 4] = torch.randn(int(((pos % 128) < 4).sum()), generator=g, device=DEV) * 0.5 + 2.0   # lane 0 only
    a[0] = 2.5
    rows.append(a)
    b = torch.randn(n, generator=g, device=DEV) * 0.3 - 6.0
    sel = ((pos % 128) >= 60) & ((pos % 128) < 68)                                                      # lanes 15 and 16
    b[sel] = torch.randn(int(sel.sum()), generator=g, device=DEV) * 1.0 + 1.0
    b[0] = 6.0
    rows.append(b)
    c = torch.randn(n, generator=g, device=DEV)            # flat, token 0 far above: high falls for many rounds
    c[0] = 9.0
    rows.append(c)
    d = torch.randn(n, generator=g, device=DEV)            # flat, token 0 far below: one or two rounds
    d[0] = -8.0
    rows.append(d)
    scores = torch.stack(rows).reshape(1, 4, n).contiguous()
    indptr, _, last, _ = PagedKVCache.page_table([n], DEV)
    pages = np.arange(n // PAGE)
    for top_p in (0.5, 0.9, 0.99):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        idx, bud = ops.topp_prune(scores, indptr, last, top_p, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for r in range(4):
            row = scores[0, r].cpu().numpy()
            probs, keep, low = U.oracle_prune_row(row, pages, top_p)
            k = int(bud[0, r])
            got = idx[0, r, :k].cpu().numpy()
            assert (np.diff(got) > 0).all()
            dd = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
            assert abs(k - int(keep.sum())) <= dd, (n, top_p, r, k, int(keep.sum()))


@pytest.mark.parametrize("n", [2048, 8192, 32768])
def test_prune_keeps_everything_when_the_mass_above_every_pivot_stays_below_p(n):
    """K1 ends with low = 0 when no pivot it tries has mass >= p above it before its window closes:
    a sink holding 93 % of the mass over flat dust with p = 0.95, or p = 0.999 on rows whose smallest
    elements together hold more than 0.1 %.  The reference's mask is then probs > 0, i.e. every
    candidate - not just the few large elements the short-list search looked at."""
    g = torch.Generator(device=DEV).manual_seed(77 + n)
    rows = []
    dust = torch.randn(n, generator=g, device=DEV) * 0.3
    a = dust.clone()
    a[0] = float(np.log(0.93 / 0.07 * n))             # sink ~ 93 % of the mass
    rows.append(a)
    b = torch.randn(n, generator=g, device=DEV) * 4.0  # wide row: the smallest elements add up to > 0.1 %
    rows.append(b)
    c = dust.clone()
    c[0] = float(np.log(0.5 * n))
    c[1: 1 + n // 64] += 3.0                           # a few hundred heavier tokens, still far below p with the sink
    rows.append(c)
    scores = torch.stack(rows).reshape(1, 3, n).contiguous()
    indptr, _, last, _ = PagedKVCache.page_table([n], DEV)
    pages = np.arange(n // PAGE)
    for top_p in (0.95, 0.999):
        idx, bud = ops.topp_prune(scores, indptr, last, top_p)
        for r in range(3):
            row = scores[0, r].cpu().numpy()
            probs, keep, low = U.oracle_prune_row(row, pages, top_p)
            k = int(bud[0, r])
            got = idx[0, r, :k].cpu().numpy()
            d = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
            assert abs(k - int(keep.sum())) <= d, (n, top_p, r, k, int(keep.sum()), float(low))
            if float(low) == 0.0:
                assert k == int((probs > 0).sum())


def test_prune_seeded_fuzz_vs_oracle():
    """Many seeded rows of 16 ... 50000 slots, seven score shapes, seven p values, every block size of
    the pruner: kept sets against the oracle, run twice (identical results)."""
    rng = np.random.default_rng(2026)
    g = torch.Generator(device=DEV).manual_seed(7)
    shapes = ("flat", "sink", "heavy", "ties", "tiny_sink", "two_level", "steps")
    differing = 0
    for case in range(16):
        nb, hq = 6, 4
        lens = [int(x) for x in rng.choice([16, 48, 700, 2048, 4096, 8192, 9000, 16384, 20000, 32768, 40960, 50000],
                                           size=nb)]
        stride = ((max(lens) + PAGE - 1) // PAGE) * PAGE
        scores = torch.full((nb, hq, stride), float("-inf"), device=DEV)
        for b, n in enumerate(lens):
            for h in range(hq):
                kind = shapes[int(rng.integers(len(shapes)))]
                row = torch.randn(n, generator=g, device=DEV) * float(rng.choice([0.1, 0.5, 1.0, 2.0, 4.0]))
                if kind == "sink":
                    row[0] += float(rng.uniform(2, 12))
                elif kind == "heavy":
                    row[0] += 12.0
                    k = max(1, int(n * rng.uniform(0.001, 0.2)))
                    at = torch.randperm(n, generator=g, device=DEV)[:k]
                    row[at] = 10.0 + 0.3 * torch.randn(k, generator=g, device=DEV)
                elif kind == "ties":
                    row[n // 3: n // 3 + max(1, n // 5)] = row[0]
                elif kind == "tiny_sink":
                    row[0] -= 10.0
                elif kind == "two_level":
                    row[: n // 2] += 5.0
                elif kind == "steps":
                    row = torch.round(row * 2) / 2
                scores[b, h, :n] = row
        indptr, _, last, _ = PagedKVCache.page_table(lens, DEV)
        top_p = torch.tensor(rng.choice([0.3, 0.5, 0.8, 0.9, 0.95, 0.99, 0.999], size=nb * hq), dtype=torch.float32,
                             device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        idx, bud = ops.topp_prune(scores, indptr, last, top_p, status=status)
        idx2, bud2 = ops.topp_prune(scores, indptr, last, top_p)
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and torch.equal(bud, bud2)
        for b, n in enumerate(lens):
            npg = (n + PAGE - 1) // PAGE
            pages = np.arange(npg)
            for h in range(hq):
                row = scores[b, h, : npg * PAGE].cpu().numpy()
                probs, keep, low = U.oracle_prune_row(row, pages, float(top_p[b * hq + h]))
                k = int(bud[b, h])
                got = idx[b, h, :k].cpu().numpy()
                assert np.array_equal(got, idx2[b, h, :k].cpu().numpy())
                assert (np.diff(got) > 0).all() and (got < n).all()
                d = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
                assert abs(k - int(keep.sum())) <= d, (case, b, h, n, k, int(keep.sum()))
                differing += d > 0
    U.record("prune_fuzz", rows=16 * 24, rows_differing=differing)
    assert differing <= 4


def test_prune_seeded_fuzz_with_candidate_lists_vs_oracle():
    """Random ascending candidate page lists (with and without page 0, short and full, the last page
    of a sequence partly past its end) and scores in candidate-slot order: kept tokens against the
    oracle, which sees token 0 only when page 0 is a candidate."""
    rng = np.random.default_rng(77)
    g = torch.Generator(device=DEV).manual_seed(77)
    for case in range(12):
        nb, hq = 3, 4
        lens = [int(x) for x in rng.choice([100, 1000, 5000, 20000, 40000, 70000], size=nb)]
        npg = [(n + PAGE - 1) // PAGE for n in lens]
        max_k = int(rng.choice([1, 4, 64, 512, 1024, 2048]))
        scores = torch.full((nb, hq, max_k * PAGE), float("-inf"), device=DEV)
        cand = torch.zeros(nb, hq, max_k, dtype=torch.int32)
        cnp = torch.zeros(nb, hq, dtype=torch.int32)
        for b, n in enumerate(lens):
            for h in range(hq):
                k = min(max_k, npg[b]) if rng.random() < 0.7 else int(rng.integers(1, min(max_k, npg[b]) + 1))
                pages = np.sort(rng.choice(npg[b], size=k, replace=False))
                if rng.random() < 0.6 and pages[0] != 0:
                    pages[0] = 0
                cand[b, h, :k] = torch.from_numpy(pages.astype(np.int32))
                cnp[b, h] = k
                row = torch.randn(k * PAGE, generator=g, device=DEV) * float(rng.choice([0.3, 1.0, 3.0]))
                if pages[0] == 0 and rng.random() < 0.7:
                    row[0] += float(rng.uniform(2, 10))
                if pages[-1] == npg[b] - 1 and n % PAGE:
                    row[(k - 1) * PAGE + n % PAGE:] = float("-inf")
                scores[b, h, : k * PAGE] = row
        cand, cnp = cand.to(DEV), cnp.to(DEV)
        indptr, _, last, _ = PagedKVCache.page_table(lens, DEV)
        top_p = torch.tensor(rng.choice([0.5, 0.9, 0.95, 0.99], size=nb * hq), dtype=torch.float32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        idx, bud = ops.topp_prune(scores, indptr, last, top_p, cand_pages=cand, cand_npages=cnp, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for b, n in enumerate(lens):
            for h in range(hq):
                k = int(cnp[b, h])
                pages = cand[b, h, :k].cpu().numpy()
                row = scores[b, h, : k * PAGE].cpu().numpy()
                probs, keep, low = U.oracle_prune_row(row, pages, float(top_p[b * hq + h]))
                kept = int(bud[b, h])
                got = idx[b, h, :kept].cpu().numpy()
                assert (np.diff(got) > 0).all() and (got < n).all()
                d = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
                assert abs(kept - int(keep.sum())) <= d, (case, b, h, kept, int(keep.sum()))


def test_prune_randomised_rows_vs_oracle():
    """Seeded random row lengths, score shapes and top-p values; every row against the oracle."""
    rng = np.random.default_rng(123)
    lens = [int(x) for x in rng.integers(1, 6000, size=14)] + [16, 17, 4096]
    hq = 4
    stride = ((max(lens) + PAGE - 1) // PAGE) * PAGE
    g = torch.Generator(device=DEV).manual_seed(5)
    scores = torch.full((len(lens), hq, stride), float("-inf"), device=DEV)
    for b, n in enumerate(lens):
        for h in range(hq):
            kind = (b + h) % 4
            row = torch.randn(n, generator=g, device=DEV) * (0.2, 1.0, 3.0, 6.0)[kind]
            if kind >= 2:
                row[0] += (2.0, 10.0)[kind - 2]
            if (b * hq + h) % 5 == 0 and n > 8:
                row[n // 2: n // 2 + n // 8 + 1] = row[0]          # a block of ties with token 0
            scores[b, h, :n] = row
    indptr, _, last, _ = PagedKVCache.page_table(lens, DEV)
    top_p = torch.tensor(rng.choice([0.5, 0.8, 0.9, 0.95, 0.99, 1.0], size=len(lens) * hq), dtype=torch.float32,
                         device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    idx, bud = ops.topp_prune(scores, indptr, last, top_p, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for b, n in enumerate(lens):
        npg = (n + PAGE - 1) // PAGE
        pages = np.arange(npg)
        for h in range(hq):
            row = scores[b, h, : npg * PAGE].cpu().numpy()
            probs, keep, low = U.oracle_prune_row(row, pages, float(top_p[b * hq + h]))
            k = int(bud[b, h])
            got = idx[b, h, :k].cpu().numpy()
            assert (np.diff(got) > 0).all() and (got < n).all()
            d = U.check_index_parity(got, probs, keep, low, pages, P_TOL)
            assert abs(k - int(keep.sum())) <= d


def test_prune_is_deterministic_and_per_row_threshold():
    lens = [2048] * 3
    hq = 4
    q, cache = make_decode_inputs(3, hq, 4, lens, rho=0.01, dtype=torch.bfloat16, device=DEV, seed=10,
                                  recipe="calibrated")
    scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                               max_pages=cache.max_pages)
    p_arr = torch.linspace(0.5, 0.99, 12, device=DEV)
    i1, b1 = ops.topp_prune(scores, cache.kv_indptr, cache.kv_last_page_len, p_arr)
    i2, b2 = ops.topp_prune(scores, cache.kv_indptr, cache.kv_last_page_len, p_arr)
    assert torch.equal(b1, b2)
    for r in range(12):
        n = int(b1.flatten()[r])
        assert torch.equal(i1.reshape(12, -1)[r, :n], i2.reshape(12, -1)[r, :n])
    assert (b1.flatten()[1:] >= b1.flatten()[:-1] - 64).any()
    for r in (0, 11):
        row = scores.reshape(12, -1)[r].cpu().numpy()
        probs, keep, low = U.oracle_prune_row(row, np.arange(128), float(p_arr[r]))
        U.check_index_parity(i1.reshape(12, -1)[r, : int(b1.flatten()[r])].cpu().numpy(), probs, keep, low,
                             np.arange(128), P_TOL)


@pytest.mark.parametrize("with_cand", [False, True])
def test_threshold_prune_is_exact(with_cand):
    """Element-wise threshold pruner: integer work on identical fp32 scores, so bit-exact."""
    lens = [17, 700, 3000]
    hq, hkv = 4, 2
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV,
                                  seed=31, recipe="calibrated", shuffle_pages=True)
    cand_pages = cand_npages = None
    if with_cand:
        cand_pages, cand_npages, _ = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 512,
                                                      max_pages=cache.max_pages)
        cand_pages[1, 0, 0] = cand_pages[1, 0, 1]   # one row without token 0 among its candidates
    scores = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                               max_pages=cache.max_pages, cand_pages=cand_pages, cand_npages=cand_npages)
    for t in (0.5, 3.0, 100.0):
        cut = torch.zeros(len(lens), hq, 2, device=DEV)
        indices, budget = ops.threshold_prune(scores, cache.kv_indptr, cache.kv_last_page_len, t,
                                              cand_pages=cand_pages, cand_npages=cand_npages, cut=cut)
        for b, n in enumerate(lens):
            npg = (n + PAGE - 1) // PAGE
            for h in range(hq):
                pages = (np.arange(npg) if cand_pages is None
                         else cand_pages[b, h, : int(cand_npages[b, h])].cpu().numpy())
                row = scores[b, h, : len(pages) * PAGE].cpu().numpy()
                # the reference's dense row: token 0's weight is row[0] iff page 0 leads the list
                w0 = row[0] if pages[0] == 0 else -np.inf
                keep = row > np.float32(w0 - np.float32(t))
                want = U.slots_to_tokens(pages, np.nonzero(keep)[0])
                got = indices[b, h, : int(budget[b, h])].cpu().numpy()
                assert np.array_equal(got, want), (t, b, h)


# ---- reference-compatible mask operators -----------------------------------------------------------------
@pytest.mark.parametrize("L", [7, 64, 1000, 4096, 32768, 60000])
def test_top_p_fp32_return_mask_vs_oracle(L):
    from twilight_b200.kernel import top_p_fp32_return_mask
    g = torch.Generator().manual_seed(L)
    logits = torch.randn(2, 3, 1, L, generator=g) * 2.5
    logits[..., 0] += 6.0
    logits[0, 1, 0, 0] = -3.0          # a row whose sink is small
    probs = torch.softmax(logits, -1)
    probs[1, 2, 0, 0] = 0.0            # a row whose sink is not a candidate
    for top_p in (0.9, torch.tensor([0.5, 0.7, 0.8, 0.9, 0.95, 0.99])):
        m = top_p_fp32_return_mask(probs.to(DEV), top_p if not torch.is_tensor(top_p) else top_p.to(DEV))
        assert m.dtype == torch.bool and m.shape == probs.shape
        want = O.top_p_return_mask(probs, top_p)
        got = m.cpu()
        rows = probs.reshape(6, L).numpy()
        for r in range(6):
            bad = np.nonzero(got.reshape(6, L)[r].numpy() != want.reshape(6, L)[r].numpy())[0]
            if bad.size:
                p = float(top_p[r]) if torch.is_tensor(top_p) else top_p
                low, _ = O.top_p_search(rows[r], p)
                assert (np.abs(rows[r][bad] - low) <= P_TOL).all()


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_top_p_fp16_return_mask_keeps_the_head_of_the_distribution(dt):
    from twilight_b200.kernel import top_p_fp16_return_mask
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(2, 2, 1, 2048, generator=g) * 3
    logits[..., 0] += 8
    probs = torch.softmax(logits, -1).to(dt)
    m = top_p_fp16_return_mask(probs.to(DEV), 0.9).cpu()
    pf = probs.float()
    kept = (pf * m).sum(-1)
    assert (kept >= 0.9 - 2e-2).all()
    assert m[..., 0].all()                                   # the sink is always kept
    thr = torch.where(m, pf, torch.full_like(pf, 9.0)).amin(-1, keepdim=True)
    assert (~(pf > thr) | m).all()                           # a threshold mask: nothing above it is dropped


def test_mask_operator_argument_errors():
    from twilight_b200.kernel import top_p_fp32_return_mask
    with pytest.raises(_lib.TwilightError, match="4D"):
        top_p_fp32_return_mask(torch.rand(4, 8, device=DEV), 0.9)
    with pytest.raises(_lib.TwilightError, match="contiguous"):
        top_p_fp32_return_mask(torch.rand(2, 3, 1, 16, device=DEV).transpose(0, 1), 0.9)
    with pytest.raises(_lib.TwilightError, match="float32"):
        top_p_fp32_return_mask(torch.rand(1, 2, 1, 16, device=DEV).half(), 0.9)


def test_oracle_topk_selector_mask_interface():
    """twilight/pyimpl/top_k.py:7-30 on the radix-select kernel: the k largest entries per row."""
    from twilight_b200.pyimpl import oracle_topk_selector
    g = torch.Generator(device=DEV).manual_seed(31)
    for (b, h, l, k) in [(2, 4, 1000, 64), (1, 3, 37, 5), (2, 2, 5000, 4096), (1, 2, 20, 50)]:
        w = torch.randn(b, h, 1, l, generator=g, device=DEV)
        got = oracle_topk_selector(w.to(torch.bfloat16).float() if l == 37 else w, k)
        ref_in = w.to(torch.bfloat16).float() if l == 37 else w
        kk = min(k, l)
        want = torch.zeros_like(ref_in, dtype=torch.bool)
        want.scatter_(-1, ref_in.topk(kk, dim=-1).indices, True)         # the reference's own lines
        assert got.dtype == torch.bool and got.shape == w.shape
        assert torch.equal(got.sum(-1), want.sum(-1))
        # equal up to ties at the cut: the kept values are the same multiset
        assert torch.equal(torch.where(got, ref_in, 0).sum(-1), torch.where(want, ref_in, 0).sum(-1)) or \
            torch.allclose(torch.where(got, ref_in, 0).sum(-1), torch.where(want, ref_in, 0).sum(-1), rtol=1e-6)
        if l != 37:
            assert torch.equal(got, want)                                # fp32 randn: no ties
    # ties go to the lower positions
    w = torch.zeros(1, 1, 1, 64, device=DEV)
    w[..., 10] = 1.0
    m = oracle_topk_selector(w, 4)
    assert m[0, 0, 0].nonzero().flatten().tolist() == [0, 1, 2, 10]


# ---- attention ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("chunk", [32, 256])
def test_sparse_attention_vs_oracle(dt, chunk):
    lens = [1, 17, 600, 3000]
    hq, hkv = 8, 2
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=12,
                                  recipe="calibrated", shuffle_pages=True)
    stride = cache.max_pages * PAGE
    g = torch.Generator().manual_seed(13)
    indices = torch.zeros(len(lens), hq, stride, dtype=torch.int32)
    budget = torch.zeros(len(lens), hq, dtype=torch.int32)
    for b, n in enumerate(lens):
        for h in range(hq):
            nb = [0, 1, min(n, 5), min(n, 33), n, min(n, 257), min(n, 1000), n // 2][h] if (b, h) != (0, 0) else 1
            budget[b, h] = nb
            indices[b, h, :nb] = torch.sort(torch.randperm(n, generator=g)[:nb])[0].int()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                 indices.to(DEV), budget.to(DEV), chunk=chunk, status=status)
    out2 = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                  indices.to(DEV), budget.to(DEV), chunk=chunk, status=status)
    assert int(status.item()) == 0
    errs = []
    for b, n in enumerate(lens):
        for h in range(hq):
            k, v = cache.dense_kv(b, h // (hq // hkv))
            nb = int(budget[b, h])
            want = O.sparse_attention_fp32(q[b, h].float().cpu().numpy(), k.float().cpu().numpy(),
                                           v.float().cpu().numpy(), indices[b, h, :nb].numpy().astype(np.int64),
                                           U.SM_SCALE)
            errs.append(np.abs(out[b, h].float().cpu().numpy() - want))
    errs = np.stack(errs)
    assert errs.max() <= ATOL_MAX and errs.mean() <= ATOL_MEAN
    # split-KV merge order may differ between runs only in the last bit of the fp32 partial sums
    assert (out.float() - out2.float()).abs().max() <= 2e-2


def test_sparse_attention_every_small_budget():
    """Budgets 1..64, one per row: the 1-4 token register path, single and multiple ring stages,
    warps with and without tokens, tails that end inside a stage or a 32-token lookup group."""
    b_n, hq, hkv, n = 8, 8, 4, 200
    q, cache = make_decode_inputs(b_n, hq, hkv, [n] * b_n, rho=0.02, dtype=torch.bfloat16, device=DEV, seed=21,
                                  recipe="calibrated", shuffle_pages=True)
    stride = cache.max_pages * PAGE
    g = torch.Generator().manual_seed(22)
    indices = torch.zeros(b_n, hq, stride, dtype=torch.int32)
    budget = torch.zeros(b_n, hq, dtype=torch.int32)
    for r in range(b_n * hq):
        nb = r + 1
        budget[r // hq, r % hq] = nb
        indices[r // hq, r % hq, :nb] = torch.sort(torch.randperm(n, generator=g)[:nb])[0].int()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for chunk in (32, 512):
        out = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                     indices.to(DEV), budget.to(DEV), chunk=chunk, status=status)
        assert int(status.item()) == 0
        for r in range(b_n * hq):
            b, h = r // hq, r % hq
            k, v = cache.dense_kv(b, h // (hq // hkv))
            want = O.sparse_attention_fp32(q[b, h].float().cpu().numpy(), k.float().cpu().numpy(),
                                           v.float().cpu().numpy(), indices[b, h, : r + 1].numpy().astype(np.int64),
                                           U.SM_SCALE)
            err = np.abs(out[b, h].float().cpu().numpy() - want)
            assert err.max() <= ATOL_MAX, (chunk, r + 1, float(err.max()))


@pytest.mark.parametrize("hq,hkv,dt", [(8, 2, torch.bfloat16), (8, 1, torch.float16), (4, 2, torch.bfloat16),
                                       (16, 2, torch.bfloat16)])
def test_group_attention_of_dense_heads(hq, hkv, dt):
    """Query-head groups whose heads keep, together, at least the sequence's length in tokens are
    served by the tensor-core group kernel (K/V pages read once per KV head); sparser groups stay
    on the per-head kernel.  Both kinds in one call, ragged lengths, partial last pages: against
    the per-head kernel on the same K/V expanded to one KV head per query head, and against the
    fp64 oracle on sampled rows."""
    lens = [16, 700, 1031, 2048, 5000, 9000]
    g = hq // hkv
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=77,
                                  recipe="calibrated", shuffle_pages=True)
    stride = cache.max_pages * PAGE
    gen = torch.Generator().manual_seed(78)
    indices = torch.zeros(len(lens), hq, stride, dtype=torch.int32)
    budget = torch.zeros(len(lens), hq, dtype=torch.int32)
    for b, n in enumerate(lens):
        for h in range(hq):
            # densities per (sequence, KV head): even KV heads dense (group kernel), odd ones sparse
            dense = ((b + h // g) % 2 == 0)
            frac = [1.0, 0.9, 0.6, 0.3][h % g % 4] if dense else [0.02, 0.1, 0.0, 0.05][h % g % 4]
            if dense and b == 3 and h % g == 1:
                frac = 0.0                        # a head without kept tokens inside a group that is served together
            nb = min(n, int(round(frac * n)))
            budget[b, h] = nb
            indices[b, h, :nb] = torch.sort(torch.randperm(n, generator=gen)[:nb])[0].int()
    indices, budget = indices.to(DEV), budget.to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices, indices,
                                 budget, chunk=256, status=status).clone()
    again = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices, indices,
                                   budget, chunk=256, status=status)
    assert int(status.item()) == 0
    assert torch.equal(out, again)                       # the workspace comes back clean, results repeat
    kx = cache.k_pages.repeat_interleave(g, dim=1).contiguous()
    vx = cache.v_pages.repeat_interleave(g, dim=1).contiguous()
    per_head = ops.sparse_decode_attn(q, kx, vx, cache.kv_indptr, cache.kv_indices, indices, budget, chunk=256)
    err = (out.float() - per_head.float()).abs()
    assert torch.isfinite(out.float()).all()
    assert float(err.max()) <= ATOL_MAX and float(err.mean()) <= ATOL_MEAN
    assert (out[budget == 0].float() == 0).all()         # rows without kept tokens give zeros
    # index lists that do not start on a 16-byte boundary: the group kernel (which reads them in 16-byte
    # pieces) must not be chosen; the per-head kernel serves every row and gives the same result as it
    # gives on the expanded cache
    flat = torch.zeros(indices.numel() + 4, dtype=torch.int32, device=DEV)
    shifted = flat[1: 1 + indices.numel()].view_as(indices)
    shifted.copy_(indices)
    assert shifted.data_ptr() % 16 != 0
    out_shifted = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices, shifted,
                                         budget, chunk=256, status=status)
    assert int(status.item()) == 0
    assert torch.equal(out_shifted, per_head)
    errs = []
    for (b, h) in [(1, 0), (3, hq - 1), (4, 1), (5, g - 1), (5, hq - 1), (2, 0)]:
        kd, vd = cache.dense_kv(b, h // g)
        idx = indices[b, h, : int(budget[b, h])].cpu().numpy().astype(np.int64)
        want = O.sparse_attention_fp32(q[b, h].float().cpu().numpy(), kd.float().cpu().numpy(),
                                       vd.float().cpu().numpy(), idx, U.SM_SCALE)
        errs.append(np.abs(out[b, h].float().cpu().numpy() - want))
    errs = np.stack(errs)
    assert errs.max() <= ATOL_MAX and errs.mean() <= ATOL_MEAN


def test_attention_seeded_fuzz_vs_fp32_reference():
    """Seeded mixes of group sizes, ragged lengths and per-head budgets (dense heads, sparse heads,
    empty heads inside served groups, single tokens): both attention kernels against an fp32
    reference on the same kept tokens."""
    rng = np.random.default_rng(11)
    worst = 0.0
    for case in range(14):
        nb = int(rng.integers(1, 5))
        hkv = int(rng.choice([1, 2, 4]))
        g = int(rng.choice([1, 2, 4, 8]))
        hq = hkv * g
        dt = [torch.bfloat16, torch.float16][case % 2]
        lens = [int(x) for x in rng.choice([1, 15, 16, 17, 100, 1000, 2049, 4096, 5000, 9000, 20000], size=nb)]
        q, cache = make_decode_inputs(nb, hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=100 + case,
                                      recipe="calibrated", shuffle_pages=True, build_aux=False)
        stride = cache.max_pages * PAGE
        gen = torch.Generator().manual_seed(case)
        indices = torch.zeros(nb, hq, stride, dtype=torch.int32)
        budget = torch.zeros(nb, hq, dtype=torch.int32)
        for b, n in enumerate(lens):
            mode = int(rng.integers(4))
            for h in range(hq):
                if mode == 0:
                    frac = rng.uniform(0.5, 1.0)
                elif mode == 1:
                    frac = rng.choice([0.0, 0.01, 0.3, 0.9, 1.0])
                elif mode == 2:
                    frac = rng.uniform(0.0, 0.05)
                else:
                    frac = 0.0 if h % g == 0 else 1.0
                kept = min(n, int(round(frac * n)))
                budget[b, h] = kept
                if kept:
                    indices[b, h, :kept] = torch.sort(torch.randperm(n, generator=gen)[:kept])[0].int()
        indices, budget = indices.to(DEV), budget.to(DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices, indices,
                                     budget, chunk=int(rng.choice([256, 512])), status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for b, n in enumerate(lens):
            for h in range(hq):
                kd, vd = cache.dense_kv(b, h // g)
                kept = int(budget[b, h])
                if kept == 0:
                    ref = torch.zeros(128, device=DEV)
                else:
                    at = indices[b, h, :kept].long()
                    pr = torch.softmax((kd[at].float() @ q[b, h].float()) * U.SM_SCALE, -1).to(dt).float()
                    ref = pr @ vd[at].float()
                e = (out[b, h].float() - ref).abs()
                assert torch.isfinite(out[b, h].float()).all()
                # mean bound plus the rounding of a 16-bit output, which a row of a few tokens shows undiluted
                assert float(e.max()) <= 2e-2 and float(e.mean()) <= 1e-3 + 2.0 ** -9 * float(ref.abs().mean()), \
                    (case, b, h, n, kept, float(e.max()), float(e.mean()))
                worst = max(worst, float(e.max()))
    U.record("attention_fuzz", worst_max_abs=worst)


def test_group_attention_flags_tokens_past_the_sequence():
    """An index past the last page of the sequence in a row served by the group kernel is skipped
    and flagged, like in the per-head kernel."""
    n, hq, hkv = 1000, 4, 1
    q, cache = make_decode_inputs(1, hq, hkv, [n], dtype=torch.bfloat16, device=DEV, seed=79, recipe="calibrated")
    stride = cache.max_pages * PAGE + 64
    indices = torch.zeros(1, hq, stride, dtype=torch.int32)
    budget = torch.full((1, hq), n, dtype=torch.int32)
    for h in range(hq):
        indices[0, h, :n] = torch.arange(n, dtype=torch.int32)
    good = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                  indices.to(DEV), budget.to(DEV), chunk=256).clone()
    indices[0, 2, n] = 5000                      # one more "kept token", far past the sequence
    budget[0, 2] = n + 1
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                 indices.to(DEV), budget.to(DEV), chunk=256, status=status)
    assert int(status.item()) & ops.FLAG_BAD_INDEX
    assert torch.equal(out, good)                # the stray index changes nothing else


def test_attention_workspace_and_bad_index_handling():
    q, cache = make_decode_inputs(1, 2, 2, [64], dtype=torch.bfloat16, device=DEV, seed=14)
    indices = torch.tensor([[[0, 5, 9999] + [0] * 61, [1, 2, 3] + [0] * 61]], dtype=torch.int32, device=DEV)
    budget = torch.tensor([[3, 3]], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                 indices, budget, status=status)
    assert int(status.item()) & ops.FLAG_BAD_INDEX            # the out-of-range token is skipped, not read
    assert torch.isfinite(out.float()).all()
    with pytest.raises(_lib.TwilightError, match="workspace"):
        ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                               indices, budget, workspace=torch.zeros(16, dtype=torch.uint8, device=DEV))


# ---- query-head groups: tensor-core kernels against the per-head kernels -----------------------------------
@pytest.mark.parametrize("hq,hkv,dt", [(8, 2, torch.bfloat16), (8, 1, torch.bfloat16), (4, 1, torch.float16),
                                       (16, 2, torch.float16), (4, 2, torch.bfloat16)])
def test_group_estimator_tensor_core_equals_integer_dot(hq, hkv, dt):
    """Default estimator for query-head groups (8-bit integer tensor-core tiles, q as 13-bit
    block-scaled integers like the single-head kernel; groups of 2 and 4 heads with both digits of q in
    one tile, which variant +512 switches off), and its 16-bit float tile form (variant +256), against
    the integer-dot group kernel (variant +32) and the fp64 oracle, ragged lengths with odd page
    counts."""
    lens = [1, 17, 33, 1000, 2049, 4000, 16 * 129]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=61,
                                  recipe="mid", shuffle_pages=True)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kw = dict(max_pages=cache.max_pages, status=status)
    b_ = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                           variant=3 + 32, **kw)
    g = hq // hkv
    # (variant, bound on the error relative to the row's largest |logit|): the float tiles multiply
    # exact values and accumulate in fp32; the integer tiles round q to 13 bits first
    for variant, bound in ((0, 2e-4), (3 + 512, 2e-4), (3 + 256, 2e-4)):
        a = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                              variant=variant, **kw)
        assert int(status.item()) == 0
        worst = 0.0
        for b, n in enumerate(lens):
            npg = (n + PAGE - 1) // PAGE
            ra, rb = a[b, :, : npg * PAGE], b_[b, :, : npg * PAGE]
            assert torch.equal(torch.isinf(ra), torch.isinf(rb))
            fin = torch.isfinite(ra)
            scale = max(1.0, float(rb[fin].abs().max()))
            assert float((ra[fin] - rb[fin]).abs().max()) <= 2e-3 * scale
            for h in (0, hq - 1):
                want, _ = U.oracle_scores_row(q, cache, b, h, g)
                got = ra[h].cpu().numpy()
                f = np.isfinite(want)
                assert np.array_equal(np.isfinite(got), f)
                worst = max(worst, float(np.abs(got[f] - want[f]).max()) / max(1.0, float(np.abs(want[f]).max())))
        U.record("group_estimator_mma", variant=variant, hq=hq, hkv=hkv, dtype=str(dt), worst_rel=worst)
        assert worst <= bound, (variant, worst)


@pytest.mark.parametrize("hq,hkv,dt", [(8, 1, torch.bfloat16), (8, 2, torch.float16), (32, 4, torch.bfloat16)])
def test_group_page_scores_tensor_core_vs_oracle(hq, hkv, dt):
    """Quest page scores of groups of 4 / 8 query heads ([min|max].[min(q,0);max(q,0)] on tensor
    cores) against the fp32 oracle: products are exact, only the order of the fp32 additions differs."""
    lens = [16, 100, 4096 + 5, 9000]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=62,
                                  recipe="mid", shuffle_pages=True)
    _, _, ps = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 256, max_pages=cache.max_pages)
    g = hq // hkv
    for b, n in enumerate(lens):
        npg = (n + PAGE - 1) // PAGE
        for h in range(hq):
            want = U.oracle_page_scores(q, cache, b, h, g)
            got = ps[b, h, :npg].cpu().numpy()
            assert np.allclose(got, want, rtol=2e-5, atol=2e-4), (b, h, np.abs(got - want).max())


def test_step_one_call_equals_the_separate_operators():
    """twl_select_prune_attend_step against the same five launches issued one by one."""
    lens = [1500, 3000, 40]
    hq, hkv = 8, 4
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV, seed=63,
                                  recipe="mid", shuffle_pages=True)
    cfg = SparseConfig(selector="quest", token_budget=1024, weight_pruner="top_p", threshold=0.9)
    ws = DecodeWorkspace.for_cache(cache, hq, cfg, attn_chunk=256)
    assert ws.buffer.numel() == _lib.load().twl_step_workspace_bytes(len(lens), hq, cache.max_pages, 1024, 256, 0)
    out = select_prune_attend_step(q, cache, ws).clone()
    _status_ok(ws)
    cp, cn, _ = ops.quest_select(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, 1024, max_pages=cache.max_pages)
    sc = ops.estimate_int4(q, cache.k4_pages, cache.kv_indptr, cache.kv_indices, cache.kv_last_page_len,
                           max_pages=cache.max_pages, cand_pages=cp, cand_npages=cn)
    idx, bud = ops.topp_prune(sc, cache.kv_indptr, cache.kv_last_page_len, 0.9, cand_pages=cp, cand_npages=cn)
    want = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices, idx, bud,
                                  chunk=256)
    assert torch.equal(ws.cand_npages, cn)
    valid_pg = torch.arange(cp.shape[-1], device=DEV)[None, None] < cn[:, :, None]
    assert torch.equal(torch.where(valid_pg, ws.cand_pages, 0), torch.where(valid_pg, cp, 0))
    assert torch.equal(ws.budget, bud)
    pos = torch.arange(idx.shape[-1], device=DEV)[None, None] < bud[:, :, None]
    assert torch.equal(torch.where(pos, ws.indices, 0), torch.where(pos, idx, 0))
    assert torch.equal(out, want)
    # a workspace that is too small or misaligned is refused before anything is launched
    with pytest.raises(_lib.TwilightError, match="workspace"):
        ops.select_prune_attend_step(q, cache.k_pages, cache.v_pages, cache.k4_pages, cache.kmeta, cache.kv_indptr,
                                     cache.kv_indices, cache.kv_last_page_len, max_pages=cache.max_pages,
                                     token_budget=1024, pruner="top_p", pruner_value=0.9, out=ws.out,
                                     workspace=ws.buffer[:4096])


def test_unit_seeded_inputs_do_not_depend_on_the_block_they_are_generated_in():
    """A (sequence, KV head) unit generated inside a rank's block equals the same unit generated
    alone: what lets one rank rebuild another rank's unit to check a gathered result."""
    from twilight_b200.gen import make_unit_inputs
    lens = {2: 300, 5: 1000, 7: 64}
    qb, cb = make_unit_inputs([2, 5, 7], [1, 3], 2, [lens[b] for b in (2, 5, 7)], rho=0.02, device=DEV, seed=9,
                              recipe="mid", shuffle_pages=True)
    q1, c1 = make_unit_inputs([5], [3], 2, [1000], rho=0.02, device=DEV, seed=9, recipe="mid", shuffle_pages=True)
    assert torch.equal(qb[1, 2:4], q1[0])
    for a, c in zip(cb.dense_kv(1, 1), c1.dense_kv(0, 0)):
        assert torch.equal(a, c)
    for a, c in zip(cb.dense_k4(1, 1), c1.dense_k4(0, 0)):
        assert torch.equal(a, c)


def test_round_scores_matches_torch_rounding():
    x = torch.randn(3, 1000, device=DEV) * 20
    x[0, :5] = float("-inf")
    for dt in (torch.float16, torch.bfloat16):
        y = ops.round_scores(x.clone(), dt)
        assert torch.equal(y, x.to(dt).float())
        z = ops.round_scores(x.clone(), dt, post_scale=U.SM_SCALE)
        assert torch.equal(z, (x.to(dt).float() * np.float32(U.SM_SCALE)).to(dt).float())


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L", [7, 64, 1000, 4096, 32768, 60000])
def test_top_p_fp16_return_mask_vs_low_precision_oracle(dt, L):
    """The fp16/bf16 mask operator against the oracle that rounds where
    csrc/include/sampling.cuh:156-217 instantiated for that dtype rounds (scalars and sums, the sums
    in the order of the reference's block reduction): equal masks, element for element.  The same
    oracle flavour is pinned against the reference's own kernel in tests/test_ref_kernel_gpu.py.
    60000 elements do not fit the kernel's shared-memory row: the global-memory path."""
    from twilight_b200.kernel import top_p_fp16_return_mask
    p = 0.95
    g = torch.Generator().manual_seed(L + (3 if dt == torch.float16 else 4))
    logits = torch.randn(1, 3, 1, L, generator=g) * 2.0
    logits[..., 0] += 7.0
    probs = torch.softmax(logits, -1).to(dt)
    m = top_p_fp16_return_mask(probs.to(DEV), p).cpu().reshape(3, L).numpy()
    for r in range(3):
        x = probs.reshape(3, L)[r]
        low, _ = O.top_p_search_lowp(x, p, "dtype")
        assert np.array_equal(m[r], x.double().numpy() > low), r


# ---- whole step ------------------------------------------------------------------------------------------------
def _step_vs_oracle(q, cache, hq, cfg, rows, dtype_faithful_report=False):
    ws = DecodeWorkspace.for_cache(cache, hq, cfg)
    out = select_prune_attend_step(q, cache, ws).clone()
    torch.cuda.synchronize()
    _status_ok(ws)
    g = hq // cache.num_kv_heads
    errs, exempt = [], 0
    for (b, h) in rows:
        n = cache.seq_lens[b]
        npg = (n + PAGE - 1) // PAGE
        if cfg.selector == "quest":
            k = int(ws.cand_npages[b, h])
            assert k == quest_max_k(cfg.token_budget, npg)
            pages = ws.cand_pages[b, h, :k].cpu().numpy()
            want_scores = U.oracle_page_scores(q, cache, b, h, g)
            must, tie, thr = U.expected_candidates(want_scores, k)
            sel = set(pages.tolist())
            for pg in (sel ^ (must | set(sorted(tie)[: k - len(must)]))):
                assert abs(want_scores[pg] - thr) <= 1e-3 * max(1.0, abs(thr))
        else:
            pages = np.arange(npg)
        want_row, _ = U.oracle_scores_row(q, cache, b, h, g, pages)
        got_row = ws.scores[b, h, : len(pages) * PAGE].cpu().numpy()
        fin = np.isfinite(want_row)
        assert np.abs(got_row[fin] - want_row[fin]).max() <= 2e-3 * max(1.0, float(np.abs(want_row[fin]).max()))
        # pruner on the oracle's own scores (end-to-end chain), tokens near the threshold exempt
        probs, keep, low = U.oracle_prune_row(want_row, pages, cfg.threshold)
        bud = int(ws.budget[b, h])
        got_idx = ws.indices[b, h, :bud].cpu().numpy()
        d = U.check_index_parity(got_idx, probs, keep, low, pages, P_TOL)
        assert abs(bud - int(keep.sum())) <= d
        exempt += d
        kd, vd = cache.dense_kv(b, h // g)
        # attention is checked on the kernel's own kept set: where that differs from the oracle's
        # (only by tokens inside the exemption window, asserted above) a single heavy token near
        # the threshold would otherwise dominate the output difference
        want_out = O.sparse_attention_fp32(q[b, h].float().cpu().numpy(), kd.float().cpu().numpy(),
                                           vd.float().cpu().numpy(), got_idx.astype(np.int64), U.SM_SCALE)
        errs.append(np.abs(out[b, h].float().cpu().numpy() - want_out))
    errs = np.stack(errs)
    assert errs.max() <= ATOL_MAX and errs.mean() <= ATOL_MEAN
    return ws, exempt


@pytest.mark.parametrize("recipe", ["literal", "mid", "calibrated"])
def test_step_config0_fp16_full_candidates(recipe):
    # B=1, 32 query heads = 32 KV heads, L=4096, fp16, 1% heavy hitters, selector none, top-p 0.95
    q, cache = make_decode_inputs(1, 32, 32, 4096, rho=0.01, dtype=torch.float16, device=DEV, seed=0, recipe=recipe)
    cfg = SparseConfig(selector="none", weight_pruner="top_p", threshold=0.95)
    ws, _ = _step_vs_oracle(q, cache, 32, cfg, [(0, h) for h in range(32)])
    if recipe == "literal":
        assert (ws.budget == 1).all()     # all softmax mass sits on the sink
    if recipe == "mid":
        assert 20 <= float(ws.budget.float().mean()) <= 80
    if recipe == "calibrated":
        assert float(ws.budget.float().mean()) > 1000


def _reference_dtype_step(q, cache, hq, **kw):
    """The reference's own dtype path (twilight/pyimpl/attention.py:188-306 restated in the model
    dtype: logits, fake-quantised K, estimate and masked attention all rounded where torch rounds)
    on the dense tensors of the cache."""
    g = hq // cache.num_kv_heads
    outs = []
    for b in range(cache.batch):
        kd = torch.stack([cache.dense_kv(b, h // g)[0] for h in range(hq)]).cpu()[None]
        vd = torch.stack([cache.dense_kv(b, h // g)[1] for h in range(hq)]).cpu()[None]
        outs.append(O.decode_step(q[b: b + 1].cpu()[:, :, None], kd, vd, quant_group=32, **kw))
    return outs


@pytest.mark.parametrize("case", ["config0", "config1_slice"])
def test_step_literal_recipe_equals_dtype_faithful_reference_exactly(case):
    """Literal recipe against the reference's dtype path: the softmax mass sits on the sink, so both
    sides must keep exactly token 0 for every head, and the outputs are V[0] on both sides."""
    if case == "config0":   # B=1, 32 = 32 heads, L=4096, fp16, selector none, top-p 0.95
        q, cache = make_decode_inputs(1, 32, 32, 4096, rho=0.01, dtype=torch.float16, device=DEV, seed=0,
                                      recipe="literal")
        cfg = SparseConfig(selector="none", weight_pruner="top_p", threshold=0.95)
        kw = dict(selector="none", threshold=0.95)
    else:                   # one sequence of config 1: 32 = 32 heads, L=32768, bf16, Quest 8192, top-p 0.95
        q, cache = make_decode_inputs(1, 32, 32, 32768, rho=0.005, dtype=torch.bfloat16, device=DEV, seed=3,
                                      recipe="literal", shuffle_pages=True)
        cfg = SparseConfig(selector="quest", token_budget=8192, weight_pruner="top_p", threshold=0.95)
        kw = dict(selector="quest", token_budget=8192, chunk_size=16, threshold=0.95)
    ws = DecodeWorkspace.for_cache(cache, 32, cfg)
    out = select_prune_attend_step(q, cache, ws).float().cpu()
    _status_ok(ws)
    ref = _reference_dtype_step(q, cache, 32, **kw)[0]
    assert (ws.budget == 1).all() and (ws.indices[:, :, 0] == 0).all()
    assert (ref["budget"] == 1).all() and ref["mask"][0, :, 0, 0].all()
    err = (out[0] - ref["out"][0, :, 0].float()).abs()
    assert float(err.max()) <= ATOL_MAX and float(err.mean()) <= ATOL_MEAN


@pytest.mark.parametrize("rounded", [False, True])
def test_step_mid_recipe_against_dtype_faithful_reference_measured(rounded):
    """Config 0 with budgets of tens of tokens against the reference's dtype path.  The reference
    rounds its logits to fp16 three times (dequantised K, the matmul, the division by sqrt(D)), the
    library keeps fp32 scores; ``round_to_dtype`` makes the library round its scores to fp16 too
    (the last two of the three).  What differs is measured and bounded: every token that one side
    keeps and the other drops has a probability within ``REL`` (relative) or 1e-4 (absolute) of the
    reference's threshold, at most ``MAX_TOKENS`` such tokens per head, and the heads whose kept
    sets agree give the same output within 2e-2 max-abs / 1e-3 mean-abs."""
    # rounded: the strict criterion (1e-4 absolute, no relative allowance); fp32 scores: measured bound
    REL, MAX_TOKENS, MIN_EQUAL_HEADS = (0.0, 1, 30) if rounded else (0.05, 4, 8)
    q, cache = make_decode_inputs(1, 32, 32, 4096, rho=0.01, dtype=torch.float16, device=DEV, seed=0, recipe="mid")
    cfg = SparseConfig(selector="none", weight_pruner="top_p", threshold=0.95, round_to_dtype=rounded)
    ws = DecodeWorkspace.for_cache(cache, 32, cfg)
    out = select_prune_attend_step(q, cache, ws).float().cpu()
    _status_ok(ws)
    ref = _reference_dtype_step(q, cache, 32, selector="none", threshold=0.95)[0]
    assert ref["out"].dtype == torch.float16
    same, errs, n_diff, worst_rel = 0, [], [], 0.0
    for h in range(32):
        probs = torch.softmax(ref["est"][0, h, 0].float(), -1).numpy()
        low, _ = O.top_p_search(probs, 0.95)
        want = set(np.nonzero(ref["mask"][0, h, 0].numpy())[0].tolist())
        got = set(ws.indices[0, h, : int(ws.budget[0, h])].cpu().numpy().tolist())
        diff = want ^ got
        n_diff.append(len(diff))
        for t in diff:
            rel = abs(probs[t] - low) / max(float(low), 1e-30)
            worst_rel = max(worst_rel, 0.0 if abs(probs[t] - low) <= P_TOL else rel)
            assert abs(probs[t] - low) <= max(P_TOL, REL * low), (h, t, probs[t], low)
        if not diff:
            same += 1
            errs.append((out[0, h] - ref["out"][0, h, 0].float()).abs().numpy())
    U.record("step_mid_vs_dtype_reference", rounded=rounded, heads_equal=same, tokens_differing=int(sum(n_diff)),
             max_tokens_per_head=int(max(n_diff)), worst_rel_distance=worst_rel,
             avg_budget=float(ws.budget.float().mean()))
    assert max(n_diff) <= MAX_TOKENS and same >= MIN_EQUAL_HEADS
    errs = np.stack(errs)
    assert errs.max() <= ATOL_MAX and errs.mean() <= ATOL_MEAN


def test_quest_pages_with_scores_rounded_to_dtype_match_reference_ranking(golden):
    """With ``round_scores`` to bf16 before the page top-k the library ranks what the reference ranks
    (its matmul returns bf16, quest.py:76-84): kept pages may differ from the reference fixture
    only in pages whose ROUNDED score equals the k-th rounded score (true ties, which torch.topk
    breaks in an unspecified order)."""
    q = torch.from_numpy(golden["quest_q"]).to(torch.bfloat16).to(DEV)[:, :, 0].contiguous()   # [2,4,128]
    k = torch.from_numpy(golden["quest_k"]).to(torch.bfloat16).to(DEV)                       # [2,4,100,128]
    bsz, h, L, _ = k.shape
    cache = PagedKVCache.from_dense(k, torch.zeros_like(k))
    for budget in (32, 40, 1000):
        ref = golden[f"quest_mask_bf16_{budget}"]
        kk = quest_max_k(budget, cache.max_pages)
        ps = ops.quest_page_scores(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, max_pages=cache.max_pages)
        ops.round_scores(ps, torch.bfloat16)
        cp, cn, _ = ops.quest_topk(ps, cache.kv_indptr, budget, max_pages=cache.max_pages)
        psn = ps.cpu().numpy()
        for b in range(bsz):
            for hh in range(h):
                ours = set(cp[b, hh, : int(cn[b, hh])].cpu().numpy().tolist())
                theirs = set((np.nonzero(ref[b, hh, 0])[0] // PAGE).tolist())
                assert len(ours) == kk == len(theirs)
                kth = np.sort(psn[b, hh])[::-1][kk - 1]
                for pg in ours ^ theirs:
                    assert psn[b, hh, pg] == kth, (budget, b, hh, pg, psn[b, hh, pg], kth)


def test_page_scores_seeded_fuzz_vs_fp64():
    """Quest page scores of every group size (FMA form for 1 and 2 heads per KV head, tensor-core form
    for 4 and 8) on ragged shuffled caches, with zero, all-negative and outlier-channel queries, and once
    at a size that takes the large block shape: against sum_d max(q_d*kmax_d, q_d*kmin_d) in fp64."""
    rng = np.random.default_rng(9)
    worst = 0.0
    for case in range(12):
        nb = int(rng.integers(1, 6))
        hkv, g = int(rng.choice([1, 2, 4, 8])), int(rng.choice([1, 2, 4, 8]))
        dt = [torch.bfloat16, torch.float16][case % 2]
        lens = [int(x) for x in rng.choice([1, 16, 17, 100, 2049, 4101, 9000, 33000], size=nb)]
        if case == 11:
            nb, hkv, g, lens = 20, 8, 8, [65536] * 20
        hq = hkv * g
        q, cache = make_decode_inputs(nb, hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=500 + case,
                                      recipe=["mid", "calibrated", "literal"][case % 3], shuffle_pages=True)
        if case % 4 == 1:
            q[:, ::2] = 0
        elif case % 4 == 2:
            q = (-q.abs()).contiguous()
        elif case % 4 == 3:
            q[:, :, ::5] *= 30
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ps = ops.quest_page_scores(q, cache.kmeta, cache.kv_indptr, cache.kv_indices, max_pages=cache.max_pages,
                                   status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for b, n in enumerate(lens):
            npg = (n + PAGE - 1) // PAGE
            for kh in range(hkv):
                kmin, kmax = (t.float() for t in cache.dense_meta(b, kh))
                for hh in range(g):
                    h = kh * g + hh
                    qq = q[b, h].float()
                    want = torch.maximum(qq[None, :] * kmax, qq[None, :] * kmin).double().sum(-1)
                    got = ps[b, h, :npg].double()
                    err = float((got - want).abs().max()) / max(1e-6, float(want.abs().max()))
                    assert torch.isfinite(got).all() and err <= 2e-5, (case, b, h, n, g, err)
                    worst = max(worst, err)
        del q, cache
    U.record("page_scores_fuzz", worst_rel=worst)


def test_topk_pages_seeded_fuzz_exact():
    """The page selection on given scores against an exact reference (descending score, ties to the
    lower page, -0 tying with +0): narrow ranges (leading key bits shared), rounded scores (many
    ties), constant rows, -inf entries, all-negative rows, one outlier; budgets from one page to all."""
    rng = np.random.default_rng(3)
    g = torch.Generator(device=DEV).manual_seed(3)
    for case in range(24):
        nb, hq = int(rng.integers(1, 5)), int(rng.choice([1, 3, 8]))
        lens = [int(x) for x in rng.choice([16, 17, 100, 1000, 4096, 5000, 20000, 32768, 65536], size=nb)]
        npg = [(n + PAGE - 1) // PAGE for n in lens]
        mp = max(npg)
        ps = torch.zeros(nb, hq, mp, device=DEV)
        for b in range(nb):
            for h in range(hq):
                kind, n = int(rng.integers(7)), npg[b]
                x = torch.randn(n, generator=g, device=DEV) * float(rng.choice([1e-3, 1.0, 50.0]))
                if kind == 1:
                    x = x + 100.0
                elif kind == 2:
                    x = torch.round(x)
                elif kind == 3:
                    x[:] = 3.25
                elif kind == 4:
                    x[torch.rand(n, generator=g, device=DEV) < 0.3] = float("-inf")
                elif kind == 5:
                    x = -x.abs() - 1.0
                elif kind == 6:
                    x[0] = 1e6
                ps[b, h, :n] = x
        indptr, _, _, _ = PagedKVCache.page_table(lens, DEV)
        budget = int(rng.choice([16, 17, 100, 1024, 8192, 16384, 1 << 20]))
        cp, cn, _ = ops.quest_topk(ps, indptr, budget, max_pages=mp)
        torch.cuda.synchronize()
        kwant = max(1, budget // PAGE) + (1 if budget % PAGE else 0)
        for b in range(nb):
            for h in range(hq):
                n = npg[b]
                k = min(kwant, n)
                x = ps[b, h, :n].cpu().numpy()
                order = np.lexsort((np.arange(n), -x))
                assert int(cn[b, h]) == k
                assert np.array_equal(cp[b, h, :k].cpu().numpy(), np.sort(order[:k])), (case, b, h, n, k)



@pytest.mark.parametrize("hq,hkv,sel", [(8, 8, "quest"), (8, 2, "quest"), (8, 2, "none")])
def test_step_ragged_gqa(hq, hkv, sel):
    lens = ragged_lengths(6, 500, 3000, seed=3) + [16, 17]
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=(0.001, 0.05), dtype=torch.bfloat16, device=DEV,
                                  seed=15, recipe="mid", shuffle_pages=True)
    cfg = SparseConfig(selector=sel, token_budget=1024, weight_pruner="top_p", threshold=0.9)
    rows = [(b, h) for b in range(len(lens)) for h in range(0, hq, 3)]
    _step_vs_oracle(q, cache, hq, cfg, rows)


def test_step_seeded_fuzz_pruner_vs_oracle_and_attention_vs_fp32():
    """Random (batch, head grouping, lengths, selector, budget, pruner, threshold, dtype, recipe) through the
    one-call step.  Each row's kept set is checked against the oracle pruner run on the scores the step itself
    wrote (so the check does not depend on the estimator's rounding), and each row's output against fp32
    attention over exactly the tokens the step kept."""
    import math
    rng = np.random.default_rng(21)
    rows = 0
    for case in range(18):
        B = int(rng.integers(1, 4))
        hkv = int(rng.choice([1, 2, 4]))
        g = int(rng.choice([1, 2, 4, 8]))
        hq = hkv * g
        dt = [torch.bfloat16, torch.float16][case % 2]
        lens = [int(x) for x in rng.choice([1, 17, 100, 1000, 2049, 4096, 9000, 20000], size=B)]
        q, cache = make_decode_inputs(B, hq, hkv, lens, rho=0.02, dtype=dt, device=DEV, seed=900 + case,
                                      recipe=["mid", "calibrated", "literal"][case % 3], shuffle_pages=True)
        sel = str(rng.choice(["none", "quest"]))
        tb = int(rng.choice([16, 100, 1024, 4096])) if sel == "quest" else -1
        pr = str(rng.choice(["top_p", "top_p", "threshold", "none"]))
        thr = float(rng.choice([0.5, 0.9, 0.95, 0.99])) if pr == "top_p" else float(rng.choice([0.5, 2.0, 6.0]))
        cfg = SparseConfig(selector=sel, token_budget=tb, weight_pruner=pr, threshold=thr)
        ws = DecodeWorkspace.for_cache(cache, hq, cfg)
        out = select_prune_attend_step(q, cache, ws).clone()
        again = select_prune_attend_step(q, cache, ws)
        _status_ok(ws)
        assert torch.equal(out, again), f"case {case}: a second step on the same workspace differs"
        for b, n in enumerate(lens):
            for h in range(hq):
                rows += 1
                tag = f"case {case} row ({b},{h}) len {n} group {g} {sel}/{tb} {pr}/{thr}"
                kept = int(ws.budget[b, h])
                idx = ws.indices[b, h, :kept].long()
                if kept:
                    assert bool((idx[1:] > idx[:-1]).all()) and int(idx.max()) < n, tag
                if sel == "quest":
                    pages = ws.cand_pages[b, h, : int(ws.cand_npages[b, h])].cpu().numpy()
                else:
                    pages = np.arange((n + PAGE - 1) // PAGE)
                row = ws.scores[b, h, : len(pages) * PAGE].cpu().numpy()
                if pr == "top_p":
                    probs, keep, low = U.oracle_prune_row(row, pages, thr)
                    d = U.check_index_parity(idx.cpu().numpy(), probs, keep, low, pages, P_TOL)
                    assert abs(kept - int(keep.sum())) <= d, tag
                elif pr == "none":
                    # every candidate whose probability is not zero in fp32: exp(s - max) is certainly positive
                    # above -87 (normal range) and certainly zero below -104.5 (under the smallest subnormal)
                    fin = row[np.isfinite(row)].astype(np.float64)
                    gap = fin - fin.max()
                    assert int((gap > -87.0).sum()) <= kept <= int((gap > -104.5).sum()), tag
                kd, vd = cache.dense_kv(b, h // g)
                if kept == 0:
                    ref = torch.zeros(128, device=DEV)
                else:
                    s = (kd[idx].float() @ q[b, h].float()) / math.sqrt(128)
                    ref = torch.softmax(s, -1).to(dt).float() @ vd[idx].float()
                err = (out[b, h].float() - ref).abs()
                assert torch.isfinite(out[b, h].float()).all(), tag
                assert float(err.max()) <= ATOL_MAX, tag
                assert float(err.mean()) <= ATOL_MEAN + 2.0 ** -9 * float(ref.abs().mean()), tag
    assert rows > 200


def test_step_repeatable_and_graph_capturable():
    q, cache = make_decode_inputs(2, 8, 8, 2048, rho=0.01, dtype=torch.bfloat16, device=DEV, seed=16, recipe="mid")
    cfg = SparseConfig(selector="quest", token_budget=512, threshold=0.95)
    ws = DecodeWorkspace.for_cache(cache, 8, cfg)
    o1 = select_prune_attend_step(q, cache, ws).clone()
    b1, i1 = ws.budget.clone(), ws.indices.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        select_prune_attend_step(q, cache, ws)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        select_prune_attend_step(q, cache, ws)
    ws.out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(ws.budget, b1)
    for r in range(16):
        n = int(b1.flatten()[r])
        assert torch.equal(ws.indices.reshape(16, -1)[r, :n], i1.reshape(16, -1)[r, :n])
    assert (ws.out.float() - o1.float()).abs().max() <= 1e-2
    _status_ok(ws)


def test_decode_attention_object_follows_the_reference_layer_rules():
    """Layers 0 and 1 run full attention and record nothing; later layers are sparsified and their
    budgets enter the average exactly as HistoryBudgetInfo does in the reference."""
    from twilight_b200.pyimpl import enable_sparse_attention
    lens = [300, 1000]
    hq, hkv = 4, 2
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV, seed=51,
                                  recipe="mid", shuffle_pages=True)
    cfg = {"compressor": {"type": "none"}, "selector": {"type": "quest", "token_budget": 256, "chunk_size": 16},
           "weight_estimator": {"type": "min_max_quant", "quant_bit": 4},
           "weight_pruner": {"type": "top_p", "threshold": 0.9}, "skip_first_two_layers": True}
    attn, info = enable_sparse_attention(cfg, hq, enable_budget_info=True)
    outs, budgets = [], []
    for layer in range(4):
        outs.append(attn(layer, q[:, :, None, :], cache).clone())
        budgets.append(attn._workspace(cache).budget.clone())
    torch.cuda.synchronize()
    # dense layers against fp64 attention over all tokens
    for b, n in enumerate(lens):
        for h in range(hq):
            k, v = cache.dense_kv(b, h // (hq // hkv))
            want = O.sparse_attention_fp32(q[b, h].float().cpu().numpy(), k.float().cpu().numpy(),
                                           v.float().cpu().numpy(), np.arange(n), U.SM_SCALE)
            assert np.abs(outs[0][b, h].float().cpu().numpy() - want).max() <= ATOL_MAX
    assert torch.equal(outs[0], outs[1]) or (outs[0].float() - outs[1].float()).abs().max() <= 1e-2
    assert (outs[2].float() - outs[0].float()).abs().max() > 0          # the sparse layers differ
    want_avg = float(torch.stack([budgets[2].float().mean(), budgets[3].float().mean()]).mean())
    assert abs(info.get_total_avg_budget() - want_avg) < 1e-4
    assert len(info._budget_num) == 1 and sorted(info._budget_num[0]) == [2, 3]


@pytest.mark.parametrize("pruner,value", [("top_p", 0.9), ("threshold", 4.0)])
def test_attention_over_estimated_weights(pruner, value):
    """use_estimated_weights_in_attn (attention.py:295-296): the final softmax runs over the
    estimator's logits of the kept tokens instead of exact q.k."""
    lens = [700, 2500, 17]
    hq, hkv = 4, 2
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV, seed=61,
                                  recipe="calibrated", shuffle_pages=True)
    cfg = SparseConfig(selector="none", weight_pruner=pruner, threshold=value, use_estimated_weights_in_attn=True)
    ws = DecodeWorkspace.for_cache(cache, hq, cfg)
    out = select_prune_attend_step(q, cache, ws).clone()
    cfg2 = SparseConfig(selector="none", weight_pruner=pruner, threshold=value)
    ws2 = DecodeWorkspace.for_cache(cache, hq, cfg2)
    out_exact = select_prune_attend_step(q, cache, ws2).clone()
    torch.cuda.synchronize()
    _status_ok(ws)
    assert torch.equal(ws.budget, ws2.budget)            # pruning itself does not change
    errs = []
    for b, n in enumerate(lens):
        for h in range(hq):
            bud = int(ws.budget[b, h])
            idx = ws.indices[b, h, :bud].cpu().numpy().astype(np.int64)
            s = ws.scores[b, h].cpu().numpy().astype(np.float64)[idx]     # no selector: slot == token
            w = np.exp(s - s.max())
            w /= w.sum()
            _, v = cache.dense_kv(b, h // (hq // hkv))
            want = w @ v.float().cpu().numpy().astype(np.float64)[idx]
            errs.append(np.abs(out[b, h].float().cpu().numpy() - want))
    errs = np.stack(errs)
    assert errs.max() <= ATOL_MAX and errs.mean() <= ATOL_MEAN
    assert (out.float() - out_exact.float()).abs().max() > 1e-4   # it really is a different attention
