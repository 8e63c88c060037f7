"""Operators called on tensors of a GPU that is not the current CUDA device (what Hugging Face's
``device_map="auto"`` produces, the only multi-GPU mode of the reference's scripts,
benchmark/LongBench/pred.py:272-274).  Needs two GPUs; skipped on a single-GPU box."""
import pytest
import torch

from twilight_b200.gen import make_decode_inputs
from twilight_b200.step import DecodeWorkspace, SparseConfig, select_prune_attend_step

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_step_on_cuda1_while_cuda0_is_current():
    torch.cuda.set_device(0)
    lens = [700, 300]
    cfg = SparseConfig(selector="quest", token_budget=256, weight_pruner="top_p", threshold=0.9)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        q, cache = make_decode_inputs(2, 8, 2, lens, rho=0.02, dtype=torch.bfloat16, device=dev, seed=71,
                                      recipe="mid", shuffle_pages=True)
        ws = DecodeWorkspace.for_cache(cache, 8, cfg)
        assert torch.cuda.current_device() == 0
        out = select_prune_attend_step(q, cache, ws)
        torch.cuda.synchronize(dev)
        assert int(ws.status.item()) == 0 and out.device == torch.device(dev)
        outs.append((out.float().cpu(), ws.budget.cpu()))
    assert torch.cuda.current_device() == 0
    assert torch.equal(outs[0][1], outs[1][1])            # same seeds, same budgets on either GPU
    assert (outs[0][0] - outs[1][0]).abs().max() <= 1e-2
