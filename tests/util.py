"""Helpers shared by the GPU parity tests: run the oracle on the rows of a paged cache."""
import json
import math
import os

import numpy as np
import torch

from oracle import twilight_oracle as O
from twilight_b200.cache import PAGE

SM_SCALE = 1.0 / math.sqrt(128)


def oracle_page_scores(q, cache, b, h, g):
    kmin, kmax = cache.dense_meta(b, h // g)
    return O.quest_page_scores_from_meta(q[b, h].cpu()[None, None], kmin.cpu()[None, None],
                                         kmax.cpu()[None, None])[0, 0].numpy()


def oracle_scores_row(q, cache, b, h, g, cand_pages=None):
    """fp32 estimator logits of one (b, query head) row in candidate-slot order (-inf padding)."""
    codes, scale, zmin = (t.cpu() for t in cache.dense_k4(b, h // g))
    est = O.estimate_logits_from_codes(q[b, h].cpu(), codes, scale, zmin, 32, SM_SCALE).numpy()
    n = cache.seq_lens[b]
    npg = (n + PAGE - 1) // PAGE
    pages = np.arange(npg) if cand_pages is None else np.asarray(cand_pages)
    out = np.full(len(pages) * PAGE, -np.inf, dtype=np.float32)
    for i, pg in enumerate(pages):
        lo, hi = pg * PAGE, min(n, pg * PAGE + PAGE)
        out[i * PAGE: i * PAGE + hi - lo] = est[lo:hi]
    return out, pages


def slots_to_tokens(pages, slots):
    pages = np.asarray(pages)
    slots = np.asarray(slots)
    return pages[slots // PAGE] * PAGE + slots % PAGE


def oracle_prune_row(scores_row, pages, top_p):
    """Oracle softmax + search on one row of scores (candidate-slot order).  The reference sees
    a dense row in token order whose entry 0 is token 0; here that is slot 0 iff page 0 leads."""
    s = np.asarray(scores_row, dtype=np.float32)
    probs = torch.softmax(torch.from_numpy(s), -1, dtype=torch.float32).numpy()
    if pages[0] != 0:
        dense = np.concatenate([[np.float32(0.0)], probs])  # token 0 is not a candidate: prob 0
        low, _ = O.top_p_search(dense, top_p)
    else:
        low, _ = O.top_p_search(probs, top_p)
    keep = probs > low
    return probs, keep, np.float32(low)


def check_index_parity(got_tokens, probs, keep, low, pages, tol=1e-4, mass_tol=2e-4):
    """Kept token sets must match except tokens whose probability is within tol of the threshold.
    For a token whose probability is itself of the order of tol that test says nothing (on a long
    flat row every probability lies within tol of any threshold), so such tokens may not carry more
    than mass_tol of the row's probability together: a pruner that dropped a row's whole tail would
    pass the first test and fails this one."""
    want_slots = np.nonzero(keep)[0]
    want = set(slots_to_tokens(pages, want_slots).tolist())
    got = set(int(t) for t in got_tokens)
    diff = want ^ got
    if not diff:
        return 0
    tok_of_slot = slots_to_tokens(pages, np.arange(len(probs)))
    p_of_tok = dict(zip(tok_of_slot.tolist(), probs.tolist()))
    mass = 0.0
    for t in diff:
        assert t in p_of_tok, f"token {t} is not a candidate"
        assert abs(p_of_tok[t] - float(low)) <= tol, (t, p_of_tok[t], float(low))
        if p_of_tok[t] <= 2 * tol:
            mass += p_of_tok[t]
    assert mass <= mass_tol, (len(diff), mass, float(low))
    return len(diff)


def expected_candidates(scores, k):
    """(must_have, may_have): pages strictly above the k-th score, and pages tied with it."""
    order = np.sort(scores)[::-1]
    thr = order[k - 1]
    return set(np.nonzero(scores > thr)[0].tolist()), set(np.nonzero(scores == thr)[0].tolist()), thr


def record(name, **stats):
    """Appends measured parity figures (counts of differing tokens, distances to thresholds) as one
    JSON line to the file named by TWL_PARITY_STATS, when that variable is set; the assertions of
    a test state the bound, this keeps the measurement behind it."""
    path = os.environ.get("TWL_PARITY_STATS")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"test": name, **stats}, default=float) + "\n")
