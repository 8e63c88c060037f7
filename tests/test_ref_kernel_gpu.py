"""The reference's own CUDA kernel (built from its sources into oracle/_ref by oracle/build_ref.py)
against the oracle and against this library's mask operator, on the same probability rows."""
import numpy as np
import pytest
import torch

from oracle import build_ref
from oracle import twilight_oracle as O
from tests import util as U

pytestmark = pytest.mark.gpu
P_TOL = 1e-4


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/twilight_ref_sampling.so has not been built")
    return mod


def _k1(ref, probs, p):
    mask = torch.zeros_like(probs, dtype=torch.bool)
    ref.top_p_fp32_return_mask(probs, mask, None, float(p), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return mask


@pytest.mark.parametrize("L,std,boost,p", [(512, 2.0, 6.0, 0.9), (4096, 2.5, 8.0, 0.95), (8192, 1.0, 3.0, 0.5),
                                           (32768, 2.0, 9.0, 0.95), (1000, 3.0, -2.0, 0.8)])
def test_reference_kernel_vs_oracle_vs_library(ref, L, std, boost, p):
    from twilight_b200.kernel import top_p_fp32_return_mask
    g = torch.Generator().manual_seed(L)
    logits = torch.randn(2, 3, 1, L, generator=g) * std
    logits[..., 0] += boost
    probs = torch.softmax(logits, -1)
    dev = probs.cuda().contiguous()
    k1 = _k1(ref, dev, p).cpu().reshape(6, L).numpy()
    ours = top_p_fp32_return_mask(dev, p).cpu().reshape(6, L).numpy()
    rows = probs.reshape(6, L).numpy()
    for r in range(6):
        low, _ = O.top_p_search(rows[r], p)
        oracle = rows[r] > low
        for name, other in (("oracle", oracle), ("library", ours[r])):
            bad = np.nonzero(k1[r] != other)[0]
            assert (np.abs(rows[r][bad] - low) <= P_TOL).all(), (name, r, bad[:5])
        assert abs(int(k1[r].sum()) - int(ours[r].sum())) <= len(np.nonzero(k1[r] != ours[r])[0])


def test_reference_kernel_sink_quirks(ref):
    # sink absent (probability 0): the reference keeps every non-zero token
    probs = torch.tensor([0.0, 0.7, 0.2, 0.1, 0.0] + [0.0] * 3).reshape(1, 1, 1, 8).cuda()
    k1 = _k1(ref, probs, 0.5).cpu().flatten().tolist()
    low, rounds = O.top_p_search(probs.cpu().flatten().numpy(), 0.5)
    assert rounds == 1 and k1 == (probs.cpu().flatten() > float(low)).tolist()
    assert k1 == [False, True, True, True, False, False, False, False]


@pytest.mark.parametrize("L", [2048, 8192, 32768])
def test_reference_kernel_keeps_everything_when_no_pivot_reaches_p(ref, L):
    """A sink with 93 % of the mass over flat dust and p = 0.95: the mass above every pivot the search
    tries stays below p until its window closes, low stays 0 and the reference's kernel keeps every
    token with non-zero probability.  The mask operator and the fused pruner (on the logits whose
    softmax these probabilities are) must do the same - not keep just the sink."""
    from twilight_b200.cache import PAGE, PagedKVCache
    from twilight_b200.kernel import ops, top_p_fp32_return_mask
    g = torch.Generator().manual_seed(L)
    logits = torch.randn(1, 2, 1, L, generator=g) * 0.3
    logits[..., 0] = float(np.log(0.93 / 0.07 * L))
    probs = torch.softmax(logits, -1)
    dev = probs.cuda().contiguous()
    k1 = _k1(ref, dev, 0.95).cpu().reshape(2, L)
    ours = top_p_fp32_return_mask(dev, 0.95).cpu().reshape(2, L)
    assert torch.equal(k1, ours)
    scores = logits.reshape(1, 2, L).cuda().contiguous()
    indptr, _, last, _ = PagedKVCache.page_table([L], "cuda")
    idx, bud = ops.topp_prune(scores, indptr, last, 0.95)
    for r in range(2):
        low, _ = O.top_p_search(probs.reshape(2, L)[r].numpy(), 0.95)
        kept_ref = int(k1[r].sum())
        if float(low) == 0.0:
            assert kept_ref == int((probs.reshape(2, L)[r] > 0).sum())
        got = torch.zeros(L, dtype=torch.bool)
        got[idx[0, r, : int(bud[0, r])].cpu().long()] = True
        diff = (got != k1[r]).nonzero().flatten()
        # the fused pruner computes its own softmax: tokens may differ only at the threshold
        assert (probs.reshape(2, L)[r][diff] - float(low)).abs().max().item() <= P_TOL if len(diff) else True
        assert float(probs.reshape(2, L)[r][diff].sum()) <= 2e-4, (L, r, len(diff), kept_ref, int(bud[0, r]))


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L", [64, 1000, 4096, 32768])
def test_fp16_entry_reference_kernel_vs_library_vs_oracle(ref, dt, L):
    """``top_p_fp16_return_mask`` (csrc/src/sampling.cu:22-43) on fp16 and bf16 rows: the
    reference's kernel, this library's operator and the oracle's low-precision flavour (every
    scalar and every partial sum rounded to the dtype, in the order of the reference's block
    reduction) must give the same mask on every element."""
    from twilight_b200.kernel import top_p_fp16_return_mask
    p = 0.9
    g = torch.Generator().manual_seed(7 * L + (1 if dt == torch.float16 else 2))
    logits = torch.randn(2, 2, 1, L, generator=g) * 2.5
    logits[..., 0] += 8.0
    probs = torch.softmax(logits, -1).to(dt)
    dev = probs.cuda().contiguous()
    ours = top_p_fp16_return_mask(dev, p).cpu().reshape(4, L).numpy()
    k1m = torch.zeros_like(dev, dtype=torch.bool)
    ref.top_p_fp16_return_mask(dev, k1m, None, float(p), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    k1 = k1m.cpu().reshape(4, L).numpy()
    rows = probs.reshape(4, L)
    for r in range(4):
        x = rows[r]
        xf = x.double().numpy()
        low_d, rounds = O.top_p_search_lowp(x, p, "dtype")
        low_32, _ = O.top_p_search_lowp(x, p, "fp32")
        U.record("fp16_entry", dtype=str(dt), L=L, row=r, rounds=rounds, n_ours=int(ours[r].sum()),
                 n_ref=int(k1[r].sum()), n_oracle_dtype=int((xf > low_d).sum()),
                 n_oracle_fp32_sums=int((xf > low_32).sum()), diff_ours_ref=int((ours[r] != k1[r]).sum()),
                 diff_ref_oracle=int((k1[r] != (xf > low_d)).sum()))
        assert np.array_equal(k1[r], xf > low_d), (r, "oracle vs reference kernel")
        assert np.array_equal(ours[r], k1[r]), (r, "library vs reference kernel")


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_fp16_entry_per_row_threshold_tensor(ref, dt):
    """``top_p`` as a per-row fp32 tensor (sampling.cuh:125) through the fp16 entry point."""
    from twilight_b200.kernel import top_p_fp16_return_mask
    g = torch.Generator().manual_seed(99)
    logits = torch.randn(1, 6, 1, 2048, generator=g) * 2.0
    logits[..., 0] += 6.0
    probs = torch.softmax(logits, -1).to(dt).cuda().contiguous()
    arr = torch.tensor([0.5, 0.8, 0.9, 0.95, 0.99, 1.0], dtype=torch.float32, device="cuda")
    ours = top_p_fp16_return_mask(probs, arr)
    k1m = torch.zeros_like(probs, dtype=torch.bool)
    ref.top_p_fp16_return_mask(probs, k1m, arr, 0.0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(ours, k1m)
