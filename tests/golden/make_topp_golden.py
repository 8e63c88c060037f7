"""Runs the reference's own top-p CUDA kernel (TopPReturnMaskKernel, compiled unmodified from
csrc/src/sampling.cu by oracle/build_ref.py) on seeded probability rows and stores its masks, so
that the CPU oracle can be pinned against the real kernel without a GPU:

    python tests/golden/make_topp_golden.py [out.npz]      # needs a CUDA device and oracle/_ref

The rows are regenerated from the stored seeds by tests/test_oracle_cpu.py.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402

CASES = [  # (seed, rows, L, logit std, sink boost, top_p)
    (0, 4, 512, 2.0, 6.0, 0.9),
    (1, 4, 4096, 2.5, 8.0, 0.95),
    (2, 3, 4096, 1.0, 3.0, 0.5),
    (3, 2, 32768, 2.0, 9.0, 0.95),
    (4, 3, 1000, 3.0, -2.0, 0.8),     # sink smaller than many tokens
]


def make_probs(seed, rows, L, std, boost):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(rows, L, generator=g) * std
    logits[:, 0] += boost
    return torch.softmax(logits, -1)


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden" / "topp_k1.npz"
    ref = build_ref.load()
    assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    out = {"cases": np.array(CASES, dtype=np.float64)}
    for i, (seed, rows, L, std, boost, p) in enumerate(CASES):
        probs = make_probs(seed, rows, L, std, boost).reshape(1, rows, 1, L).cuda().contiguous()
        mask = torch.zeros_like(probs, dtype=torch.bool)
        ref.top_p_fp32_return_mask(probs, mask, None, float(p), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        m = mask.reshape(rows, L).cpu().numpy()
        out[f"mask_{i}"] = np.packbits(m, axis=1)
        out[f"budget_{i}"] = m.sum(1)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
