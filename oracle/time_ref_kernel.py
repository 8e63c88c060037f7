"""Times the reference's own top-p CUDA kernel (TopPReturnMaskKernel, compiled unmodified into
oracle/_ref by oracle/build_ref.py) against this library's operators on the same inputs.

    python oracle/time_ref_kernel.py            # needs a CUDA device

Three timings per shape, CUDA events, 10 warm-ups + 50 repeats, inputs larger than L2 rotated:
  reference   softmax(fp32) by torch + TopPReturnMaskKernel          (twilight/pyimpl/top_p.py:10-15)
  mask op     softmax(fp32) by torch + twl_top_p_return_mask_f32     (same dense-mask interface)
  fused       twl_topp_prune on the raw scores (softmax + search + index list in one kernel)
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402
from twilight_b200.cache import PagedKVCache  # noqa: E402
from twilight_b200.kernel import ops, top_p_fp32_return_mask  # noqa: E402


def timeit(fn, n=50):
    for _ in range(10):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1000.0


def main():
    ref = build_ref.load()
    assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    dev = "cuda"
    for (b, h, L, recipe) in [(16, 32, 8192, "sink"), (16, 32, 32768, "sink"), (16, 32, 32768, "flat"),
                              (1, 32, 4096, "sink")]:
        g = torch.Generator(device=dev).manual_seed(0)
        logits = torch.randn(b, h, 1, L, generator=g, device=dev) * (2.0 if recipe == "sink" else 1.0)
        if recipe == "sink":
            logits[..., 0] += 8.0
        stream = torch.cuda.current_stream().cuda_stream

        def run_ref():
            probs = torch.softmax(logits, -1, dtype=torch.float32)
            mask = torch.zeros_like(probs, dtype=torch.bool)
            ref.top_p_fp32_return_mask(probs, mask, None, 0.95, stream)
            return mask

        def run_mask():
            probs = torch.softmax(logits, -1, dtype=torch.float32)
            return top_p_fp32_return_mask(probs, 0.95)

        indptr, _, last, _ = PagedKVCache.page_table([L] * b, dev)
        scores = logits.reshape(b, h, L).contiguous()
        idx = torch.empty(b, h, L, dtype=torch.int32, device=dev)
        bud = torch.empty(b, h, dtype=torch.int32, device=dev)

        def run_fused():
            return ops.topp_prune(scores, indptr, last, 0.95, indices=idx, budget=bud)

        m_ref, m_ours = run_ref(), run_mask()
        run_fused()
        torch.cuda.synchronize()
        same = float((m_ref == m_ours).float().mean())
        t_ref, t_mask, t_fused = timeit(run_ref), timeit(run_mask), timeit(run_fused)
        print(f"rows {b * h:4d} L {L:6d} {recipe:5s}: reference {t_ref:8.1f} us | mask op {t_mask:8.1f} us | "
              f"fused prune {t_fused:8.1f} us | masks equal {same:.6f} | budget ref {int(m_ref.sum()) / (b * h):.1f} "
              f"fused {float(bud.float().mean()):.1f}")


if __name__ == "__main__":
    main()
