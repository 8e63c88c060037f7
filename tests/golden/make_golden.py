"""Generates tests/golden/reference_pyimpl.npz by running the reference's own Python files.

Run once where the reference checkout is available:
    python tests/golden/make_golden.py [/path/to/Twilight]
It imports twilight/pyimpl/quantize.py and twilight/pyimpl/quest.py BY FILE PATH (the package
itself does not import with the flashinfer version installed here) and stores seeded inputs
together with the reference's outputs, so the oracle can be pinned without the checkout.
"""
import importlib.util
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

REF = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
OUT = Path(__file__).resolve().parent / "reference_pyimpl.npz"


def load(name, rel):
    spec = importlib.util.spec_from_file_location(name, REF / rel)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    quantize = load("ref_quantize", "twilight/pyimpl/quantize.py")
    quest = load("ref_quest", "twilight/pyimpl/quest.py")
    out = {}
    # the only in-repo vector that touches the INT4 formula (quantize.py:30-48)
    kv15 = torch.tensor([0.31, 0.42, -0.57, 0.23, -1.79, -2.18, 1.90, 4.32, -3.56, 0.78, 0.69,
                         1.45, 2.84, -2.09, -1.26])
    out["q15_in"] = kv15.numpy()
    out["q15_out"] = quantize.min_max_per_token_quant_kv(kv15, 4).numpy()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 3, 8, 128, generator=g) * 1.7
    x[0, 0, 0, :32] = 0.5   # a constant group
    x[0, 1, 2] *= 9.0        # a heavy-hitter-like row
    out["qx_in"] = x.numpy()
    for name, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        xd = x.to(dt)
        out[f"qx_tok_{name}"] = quantize.min_max_per_token_quant_kv(xd, 4).float().numpy()
        y = quantize.min_max_per_token_quant_kv(xd.reshape(2, 3, 8, 4, 32), 4).reshape(2, 3, 8, 128)
        out[f"qx_g32_{name}"] = y.float().numpy()
    # Quest selector: L not a multiple of the chunk, budgets below / off-multiple / above L
    q = torch.randn(2, 4, 1, 128, generator=g)
    k = torch.randn(2, 4, 100, 128, generator=g)
    k[:, :, 37] = 3.0 * q[:, :, 0] / q[:, :, 0].norm(dim=-1, keepdim=True) * 128 ** 0.5
    out["quest_q"] = q.numpy()
    out["quest_k"] = k.numpy()
    model = SimpleNamespace(num_heads=4)
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        for budget in (32, 40, 1000):
            m = quest.quest_selector(model, q.to(dt), k.to(dt), 16, token_budget=budget)
            out[f"quest_mask_{name}_{budget}"] = m.numpy()
    # element-wise threshold pruner (twilight/pyimpl/elementwise_threshold.py:9-18)
    thr = load("ref_threshold", "twilight/pyimpl/elementwise_threshold.py")
    w = torch.randn(2, 3, 1, 40, generator=g) * 3
    out["thr_w"] = w.numpy()
    for t in (0.5, 4.0):
        out[f"thr_mask_{t}"] = thr.elementwise_threshold(w, t).numpy()
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
