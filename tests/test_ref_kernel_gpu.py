"""The reference's own CUDA kernel (built from its sources into oracle/_ref by oracle/build_ref.py)
against the oracle and against this library's mask operator, on the same probability rows."""
import numpy as np
import pytest
import torch

from oracle import build_ref
from oracle import twilight_oracle as O

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
