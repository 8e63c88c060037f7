"""The attention entry point that brings its own scratch memory (for hosts that cannot allocate
device memory after start-up) must give what the ordinary entry point gives.  Collected last on
purpose: a run that stops at the first failure has then already run everything else."""
import numpy as np
import pytest
import torch

from oracle import twilight_oracle as O
from tests import util as U
from twilight_b200 import _lib
from twilight_b200.cache import PAGE
from twilight_b200.gen import make_decode_inputs
from twilight_b200.kernel import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
ATOL_MAX, ATOL_MEAN = 2e-2, 1e-3


def _case(seed, lens, hq, hkv, budgets):
    q, cache = make_decode_inputs(len(lens), hq, hkv, lens, rho=0.02, dtype=torch.bfloat16, device=DEV,
                                  seed=seed, recipe="calibrated", shuffle_pages=True)
    stride = cache.max_pages * PAGE
    g = torch.Generator().manual_seed(seed)
    indices = torch.zeros(len(lens), hq, stride, dtype=torch.int32)
    budget = torch.zeros(len(lens), hq, dtype=torch.int32)
    for b, n in enumerate(lens):
        for h in range(hq):
            nb = min(n, budgets[(b * hq + h) % len(budgets)])
            budget[b, h] = nb
            indices[b, h, :nb] = torch.sort(torch.randperm(n, generator=g)[:nb])[0].int()
    return q, cache, indices.to(DEV), budget.to(DEV)


def test_static_scratch_attention_matches_workspace_attention_twice():
    # two different problems back to back: the second one meets whatever the first left in the
    # shared scratch array (long rows first, so stale partial results exist for every slot)
    cases = [_case(21, [3000, 700], 8, 2, [3000, 1, 600, 0, 257, 2048, 33, 1000]),
             _case(22, [900, 2500, 64], 4, 4, [5, 900, 0, 2500, 17, 64, 300])]
    for n_call, (q, cache, indices, budget) in enumerate(cases):
        b, hq, _ = q.shape
        want = ops.sparse_decode_attn(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                      indices, budget, chunk=256)
        out = torch.full((b, hq, 128), float("nan"), dtype=q.dtype, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats()["allocation.all.allocated"]   # allocations made so far
        free_before = torch.cuda.mem_get_info()[0]
        got = ops.sparse_decode_attn_static(q, cache.k_pages, cache.v_pages, cache.kv_indptr, cache.kv_indices,
                                            indices, budget, out=out, chunk=256, status=status)
        torch.cuda.synchronize()
        # nothing was allocated through torch; and on the second call, when the attention code (and
        # with it the scratch array) is certainly resident, the device's free memory did not shrink
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
        if n_call > 0:
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert int(status.item()) == 0
        err = (got.float() - want.float()).abs()
        assert torch.isfinite(got.float()).all()
        assert float(err.max()) <= ATOL_MAX and float(err.mean()) <= ATOL_MEAN
        # and against the CPU oracle on a few rows, so that both entry points drifting together shows
        g = hq // cache.num_kv_heads
        for (bb, h) in [(0, 0), (b - 1, hq - 1), (0, hq // 2)]:
            kd, vd = cache.dense_kv(bb, h // g)
            idx = indices[bb, h, : int(budget[bb, h])].cpu().numpy().astype(np.int64)
            ref = O.sparse_attention_fp32(q[bb, h].float().cpu().numpy(), kd.float().cpu().numpy(),
                                          vd.float().cpu().numpy(), idx, U.SM_SCALE)
            e = np.abs(got[bb, h].float().cpu().numpy() - ref)
            # one row alone: the mean bound plus the rounding of a bf16 output (half an ulp, 2^-9 relative),
            # which a row of a handful of tokens (outputs of order 1) shows undiluted
            assert e.max() <= ATOL_MAX and e.mean() <= ATOL_MEAN + 2.0 ** -9 * np.abs(ref).mean(), (bb, h, e.max())


def test_static_scratch_attention_rejects_more_rows_than_it_holds():
    q, cache, indices, budget = _case(23, [64], 2, 2, [8])
    rows = ops.STATIC_ATTN_MAX_ROWS + 1
    lib = _lib.load()
    out = torch.zeros(1, 2, 128, dtype=q.dtype, device=DEV)
    st = lib.twl_sparse_decode_attn_static(q.data_ptr(), 1, cache.k_pages.data_ptr(), cache.v_pages.data_ptr(),
                                           cache.kv_indptr.data_ptr(), cache.kv_indices.data_ptr(),
                                           indices.data_ptr(), indices.shape[-1], budget.data_ptr(), rows, 1, 1,
                                           cache.k_pages.shape[0], 0.088, out.data_ptr(), 256, None, None)
    assert st == -5  # TWL_ERR_TOO_LARGE, before anything is launched
    with pytest.raises(_lib.TwilightError, match="exceeds"):
        _lib.check(st, "sparse_decode_attn_static")
