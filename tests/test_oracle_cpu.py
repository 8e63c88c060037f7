"""CPU checks of the oracle: against the reference's own Python outputs (golden fixtures
produced by tests/golden/make_golden.py), against hand-derived known answers for the top-p
search of csrc/include/sampling.cuh:156-230, and internal consistency of the two forms of the
Quest score."""
import math

import numpy as np
import pytest
import torch

from oracle import twilight_oracle as O


# ---- quantiser vs twilight/pyimpl/quantize.py -----------------------------------------------
def test_quantize_repo_vector(golden):
    x = torch.from_numpy(golden["q15_in"])
    deq = O.quantize_min_max(x, 4)[0]
    assert np.array_equal(deq.numpy(), golden["q15_out"])


@pytest.mark.parametrize("name,dt", [("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_quantize_matches_reference(golden, name, dt):
    x = torch.from_numpy(golden["qx_in"]).to(dt)
    per_tok = O.quantize_min_max(x, 4)[0].float().numpy()
    g32 = O.quantize_min_max(x, 4, group=32)[0].float().numpy()
    assert np.array_equal(per_tok, golden[f"qx_tok_{name}"], equal_nan=True)
    assert np.array_equal(g32, golden[f"qx_g32_{name}"], equal_nan=True)


def test_quantize_codes_reconstruct():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 128, generator=g).to(torch.bfloat16)
    deq, codes, scales, zeros = O.quantize_min_max(x, 4, group=32)
    assert codes.max() <= 15 and codes.min() >= 0
    rec = (codes.reshape(5, 4, 32).to(torch.bfloat16) * scales.unsqueeze(-1) - zeros.unsqueeze(-1))
    assert torch.equal(rec.reshape(5, 128), deq)
    # every group uses code 0 at its minimum and 15 at its maximum
    assert (codes.reshape(5, 4, 32).amin(-1) == 0).all() and (codes.reshape(5, 4, 32).amax(-1) == 15).all()


# ---- Quest selector vs twilight/pyimpl/quest.py ------------------------------------------------
@pytest.mark.parametrize("name,dt", [("f32", torch.float32), ("bf16", torch.bfloat16)])
@pytest.mark.parametrize("budget", [32, 40, 1000])
def test_quest_matches_reference(golden, name, dt, budget):
    q = torch.from_numpy(golden["quest_q"]).to(dt)
    k = torch.from_numpy(golden["quest_k"]).to(dt)
    m = O.quest_select_mask(q, k, 16, budget)
    assert np.array_equal(m.numpy(), golden[f"quest_mask_{name}_{budget}"])


def test_elementwise_threshold_matches_reference(golden):
    w = torch.from_numpy(golden["thr_w"])
    for t in (0.5, 4.0):
        assert np.array_equal(O.elementwise_threshold(w, t).numpy(), golden[f"thr_mask_{t}"])


def test_quest_meta_form_equals_dense_form():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, 2, 1, 128, generator=g)
    q[0, 0, 0, 5] = 0.0  # q_d == 0 takes sign -1 in the reference (quest.py:37)
    k = torch.randn(1, 2, 70, 128, generator=g)
    dense = O.quest_page_scores(q, k, 16)[:, :, 0]
    n_pages = 5
    kpad_min = torch.cat([k, torch.full((1, 2, 10, 128), float("inf"))], 2).reshape(1, 2, n_pages, 16, 128)
    kpad_max = torch.cat([k, torch.full((1, 2, 10, 128), float("-inf"))], 2).reshape(1, 2, n_pages, 16, 128)
    meta = O.quest_page_scores_from_meta(q[:, :, 0], kpad_min.amin(3), kpad_max.amax(3))
    assert torch.allclose(dense, meta, rtol=1e-5, atol=1e-4)


def test_quest_chunk_budget_rule():
    assert O.quest_chunk_budget(8192, 16, 2048) == 512
    assert O.quest_chunk_budget(40, 16, 100) == 3      # 2 full + 1 for the remainder
    assert O.quest_chunk_budget(5, 16, 100) == 2       # max(1, 0) + 1
    assert O.quest_chunk_budget(0, 16, 100) == 1
    assert O.quest_chunk_budget(1000, 16, 7) == 7


# ---- top-p search: known answers ------------------------------------------------------------------
def _mask(probs, p):
    x = np.asarray(probs, dtype=np.float32)
    low, rounds = O.top_p_search(x, p)
    return x > low, low, rounds


def test_topp_paper_example():
    # the example drawn in the reference's figures/arch.png; p below 0.9 so that the fp32 sum
    # 0.5+0.25+0.15 is not compared for equality with p
    keep, _, _ = _mask([0.5, 0.03, 0.02, 0.15, 0.04, 0.25, 0.01], 0.89)
    assert keep.tolist() == [True, False, False, True, False, True, False]


def test_topp_sink_always_kept_even_if_tiny():
    keep, low, _ = _mask([0.01, 0.6, 0.3, 0.09], 0.5)
    # high starts at the sink's 0.01 (sampling.cuh:156-159): everything >= ~0.01 survives
    assert keep[0] and keep[1] and keep[2] and keep[3]
    assert low < 0.01


def test_topp_sink_absent_means_no_pruning():
    # position 0 has probability 0 (not a candidate): one round, low stays 0, all non-zeros kept
    keep, low, rounds = _mask([0.0, 0.7, 0.2, 0.1, 0.0], 0.5)
    assert low == 0.0 and rounds == 1
    assert keep.tolist() == [False, True, True, True, False]


def test_topp_uniform_row_keeps_all():
    keep, _, _ = _mask(np.full(64, 1 / 64), 0.5)
    assert keep.all()


def test_topp_p_one_keeps_every_nonzero():
    x = np.array([0.4, 0.3, 0.2, 0.1, 0.0], dtype=np.float32)
    keep, _, _ = _mask(x, 1.0)
    assert keep.tolist() == [True, True, True, True, False]


def test_topp_single_candidate():
    keep, _, _ = _mask([1.0, 0.0, 0.0], 0.95)
    assert keep.tolist() == [True, False, False]


def test_topp_superset_of_exact_and_surplus_near_threshold():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(4096, generator=g) * 2.0
    logits[0] = 9.0
    probs = torch.softmax(logits, -1).numpy()
    keep, low, rounds = _mask(probs, 0.9)
    order = np.argsort(-probs)
    csum = np.cumsum(probs[order].astype(np.float64))
    n_exact = int(np.searchsorted(csum, 0.9) + 1)
    exact = np.zeros_like(keep)
    exact[order[:n_exact]] = True
    assert (keep | ~exact).all()                         # superset of the minimal top-p set
    thr = probs[order[n_exact - 1]]
    surplus = keep & ~exact
    assert (np.abs(probs[surplus] - thr) <= 2e-5).all()  # eps = 1e-5 ties
    assert 1 <= rounds <= 40


def test_top_p_return_mask_tensor_threshold():
    g = torch.Generator().manual_seed(2)
    probs = torch.softmax(torch.randn(2, 3, 1, 50, generator=g) * 3, -1)
    p = torch.tensor([0.5, 0.6, 0.7, 0.8, 0.9, 0.95])
    m = O.top_p_return_mask(probs, p)
    for r in range(6):
        low, _ = O.top_p_search(probs.reshape(6, 50)[r].numpy(), float(p[r]))
        assert np.array_equal(m.reshape(6, 50)[r].numpy(), probs.reshape(6, 50)[r].numpy() > low)


# ---- whole step ------------------------------------------------------------------------------
def test_decode_step_dense_equivalence_without_pruning():
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 2, 1, 128, generator=g)
    k = torch.randn(1, 2, 40, 128, generator=g)
    v = torch.randn(1, 2, 40, 128, generator=g)
    r = O.decode_step(q, k, v, selector="none", estimator="none", pruner="none")
    dense = torch.softmax(q @ k.transpose(2, 3) / math.sqrt(128), -1) @ v
    assert torch.allclose(r["out"], dense, atol=1e-5)
    assert r["budget"].tolist() == [40, 40]


def test_decode_step_budget_counts_mask():
    g = torch.Generator().manual_seed(6)
    q = torch.randn(1, 2, 1, 128, generator=g)
    k = torch.randn(1, 2, 64, 128, generator=g)
    k[:, :, 0] = 1.5 * q[:, :, 0]
    v = torch.randn(1, 2, 64, 128, generator=g)
    r = O.decode_step(q, k, v, selector="quest", token_budget=32, quant_group=32, threshold=0.9)
    assert torch.equal(r["budget"], r["mask"].sum(-1).flatten())
    assert (r["budget"] <= 32).all() and (r["budget"] >= 1).all()
    # sparse fp64 attention over the kept indices agrees with the masked dense form
    idx = torch.nonzero(r["mask"][0, 0, 0]).flatten().numpy()
    o = O.sparse_attention_fp32(q[0, 0, 0].numpy(), k[0, 0].numpy(), v[0, 0].numpy(), idx, 1 / math.sqrt(128))
    assert np.allclose(o, r["out"][0, 0, 0].numpy(), atol=1e-5)


# ---- top-p search vs the reference's own CUDA kernel (masks recorded on a B200) ---------------
def test_topp_oracle_matches_recorded_reference_kernel_masks():
    """tests/golden/topp_k1.npz holds the masks TopPReturnMaskKernel (csrc/include/sampling.cuh,
    compiled unmodified) produced for seeded rows; tests/golden/make_topp_golden.py made it."""
    import importlib.util
    from pathlib import Path
    gold_dir = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_topp_golden", gold_dir / "make_topp_golden.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    data = np.load(gold_dir / "topp_k1.npz")
    assert [tuple(c) for c in data["cases"].tolist()] == [tuple(float(x) for x in c) for c in gen.CASES]
    total_diff = 0
    for i, (seed, rows, L, std, boost, p) in enumerate(gen.CASES):
        probs = gen.make_probs(seed, rows, L, std, boost).numpy()
        k1 = np.unpackbits(data[f"mask_{i}"], axis=1)[:, :L].astype(bool)
        assert (k1.sum(1) == data[f"budget_{i}"]).all()
        for r in range(rows):
            low, _ = O.top_p_search(probs[r], p)
            mine = probs[r] > low
            bad = np.nonzero(mine != k1[r])[0]
            # block-reduce summation order is the only freedom: differences sit at the threshold
            assert (np.abs(probs[r][bad] - low) <= 1e-4).all()
            total_diff += bad.size
            assert k1[r][0]                                  # the sink is always kept
    assert total_diff <= 8


# ---- the search instantiated for fp16 / bf16 rows (csrc/src/sampling.cu:22-43) ------------------
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_topp_low_precision_flavour_known_answers(dt):
    # the paper's example row is exactly representable enough: same kept set as the fp32 search
    row = torch.tensor([0.5, 0.03, 0.02, 0.15, 0.04, 0.25], dtype=dt)
    for sums in ("fp32", "dtype"):
        low, rounds = O.top_p_search_lowp(row, 0.89, sums)
        assert (row.double() > low).tolist() == [True, False, False, True, False, True]
        assert 1 <= rounds < O.SEARCH_ITER_CAP
        assert float(torch.tensor(low, dtype=torch.float64).to(dt)) == low   # low lives in the dtype
    # sink absent: high = x[0] = 0, one round, nothing pruned
    row = torch.tensor([0.0, 0.7, 0.2, 0.1], dtype=dt)
    low, rounds = O.top_p_search_lowp(row, 0.5)
    assert rounds == 1 and low == 0.0


def test_topp_low_precision_flavours_agree_up_to_sum_rounding():
    g = torch.Generator().manual_seed(5)
    for dt, tol in ((torch.float16, 5e-3), (torch.bfloat16, 4e-2)):
        logits = torch.randn(8192, generator=g) * 2.5
        logits[0] += 8
        row = torch.softmax(logits, -1).to(dt)
        la, _, margin = O.top_p_search_lowp(row, 0.9, "fp32", return_margin=True)
        lb, _ = O.top_p_search_lowp(row, 0.9, "dtype")
        x = row.double()
        ma, mb = float(x[x > la].sum()), float(x[x > lb].sum())
        assert margin >= 0 and abs(ma - mb) <= tol     # kept masses differ by the rounding of the sums only
        assert ma >= 0.9 - tol and mb >= 0.9 - tol


def test_half_block_sum_is_exact_when_nothing_rounds():
    vals = torch.arange(1024 * 8, dtype=torch.float32).remainder(2).to(torch.float16)  # 0/1 pattern: sums stay exact
    assert float(O._half_block_sum(vals, 8)) == 4096.0
