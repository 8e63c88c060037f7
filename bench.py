#!/usr/bin/env python
"""Benchmark of the Select-then-Prune decode step (Quest selector -> INT4 estimator -> top-p
pruner -> sparse paged attention) on synthetic inputs of the Longchat-7B-class configuration:
B=16 sequences of 32768 tokens, 32 query heads = 32 KV heads, head_dim 128, page size 16,
Quest budget 8192, top-p 0.95, bf16, 32 attention layers per decoded token.

One "step" decodes one token for the whole batch: 32 layer passes of the hot path.  Only
``--resident-layers`` distinct layers' caches are held in HBM (one layer is 8 GiB of K/V plus
1.25 GiB of INT4 K and 0.5 GiB of page metadata); the 32 passes cycle through them, so every
pass streams data that is far larger than L2 and was last touched several passes ago.

Prints ONE JSON line (rank 0).  ``python bench.py --impl reference`` times the CPU restatement
of the reference's PyTorch path on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "sparse decode attn tokens/s/GPU @32k ctx; % HBM roofline; avg pruned budget"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--resident-layers", type=int, default=4)
    ap.add_argument("--token-budget", type=int, default=8192)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--rho", type=float, default=0.005)
    ap.add_argument("--recipe", default="literal", choices=["literal", "mid", "calibrated"])
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--gather-per-layer", action="store_true",
                    help="all-gather the outputs after every layer pass instead of once per decoded token")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--kernel-reps", type=int, default=5)
    ap.add_argument("--attn-chunk", type=int, default=512, help="tokens per split-KV work item of the attention kernel")
    ap.add_argument("--ablation", action="store_true",
                    help="also time the captured layer pass with each kernel left out (its marginal cost in the chain)")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's PyTorch path
# ---------------------------------------------------------------------------------------------
def cpu_reference_inputs(args, heads: int, seqs: int):
    """Seeded inputs of ``seqs`` sequences for the CPU arm (bf16, sink planted as in the recipe)."""
    L, D = args.ctx, 128
    data = []
    for i in range(seqs):
        g = torch.Generator().manual_seed(i)
        q = torch.randn(1, heads, 1, D, generator=g).to(torch.bfloat16)
        k = torch.randn(1, heads, L, D, generator=g).to(torch.bfloat16)
        v = torch.randn(1, heads, L, D, generator=g).to(torch.bfloat16)
        qh = q[:, :, 0].float()
        qh = qh / qh.norm(dim=-1, keepdim=True) * math.sqrt(D)
        k[:, :, 0] = (8.0 * qh).to(torch.bfloat16)
        data.append((q, k, v))
    return data


def cpu_reference_step(args, data):
    """One layer pass of twilight/pyimpl/attention.py:188-306 over the given sequences on the
    host cores, dtype-faithful (bf16), one sequence at a time.  Returns seconds."""
    from oracle import twilight_oracle as O
    t0 = time.perf_counter()
    for q, k, v in data:
        O.decode_step(q, k, v, selector="quest", token_budget=args.token_budget, chunk_size=16,
                      quant_group=32, threshold=args.top_p)
    return time.perf_counter() - t0


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    seqs = min(4, args.batch)
    # torchrun pins OMP_NUM_THREADS to 1 per rank; this arm runs alone on rank 0 and may use the host
    torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))
    threads = torch.get_num_threads()
    data = cpu_reference_inputs(args, args.heads, seqs)
    for _ in range(args.warmup):
        cpu_reference_step(args, data)
    times = [cpu_reference_step(args, data) for _ in range(max(1, args.steps))]
    t = statistics.mean(times)
    # `seqs` sequences of one layer measured per step; a decoded token needs `layers` passes
    value = seqs / (t * args.layers)
    sample = (f"each step = 1 of {args.layers} layer passes over {seqs} of {args.batch} sequences x {args.heads} "
              f"heads at ctx {args.ctx}; tokens/s = sequences / (step time x layers)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, n):
    return {"workload": f"Longchat-7B-class decode attention, B={args.batch}/GPU, ctx {args.ctx}, "
                        f"{args.heads}q/{args.kv_heads}kv heads, d128, page 16, Quest {args.token_budget} + top-p {args.top_p}, "
                        f"{args.layers} layers/token",
            "global_batch": args.batch * n, "seq_len": args.ctx, "parallelism": f"(batch,kv-head) shards x{n}",
            "recipe": args.recipe, "resident_layers": args.resident_layers,
            "output_gather": "none (1 GPU)" if n == 1 else ("NCCL all-gather per layer pass" if args.gather_per_layer
                                                             else "one NCCL all-gather per decoded token"),
            "l2": "inputs larger than L2: each layer pass streams >0.8 GB and layers alternate"}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
_T0 = time.time()


def log(msg):
    """Progress lines on stderr (every rank), so that a stalled multi-rank run shows where it is."""
    sys.stderr.write(f"[bench r{os.environ.get('RANK', '0')} +{time.time() - _T0:6.1f}s] {msg}\n")
    sys.stderr.flush()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    from twilight_b200 import _lib
    from twilight_b200.gen import make_decode_inputs
    from twilight_b200.step import (DecodeWorkspace, SparseConfig, select_prune_attend_step,
                                    step_algorithmic_bytes)
    _lib.load()  # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        log("process group up")

    cfg = SparseConfig(selector="quest", token_budget=args.token_budget, weight_pruner="top_p",
                       threshold=args.top_p)
    R = max(1, min(args.resident_layers, args.layers))
    layers = []
    for l in range(R):
        q, cache = make_decode_inputs(args.batch, args.heads, args.kv_heads, args.ctx, rho=args.rho,
                                      dtype=torch.bfloat16, device=dev, seed=1000 * rank + l,
                                      recipe=args.recipe, shuffle_pages=True)
        layers.append((q, cache))
    log(f"{R} resident layers generated")
    ws = DecodeWorkspace.for_cache(layers[0][1], args.heads, cfg, attn_chunk=args.attn_chunk)
    # Outputs of all layer passes of one token.  A rank's heads feed its own slice of the output
    # projection, so nothing has to cross GPUs between layers; the per-token result is gathered
    # once (NCCL all-gather), or after every layer pass with --gather-per-layer.
    outs = torch.empty(args.layers, args.batch, args.heads, 128, dtype=torch.bfloat16, device=dev)
    gathered = gathered_all = None
    if world > 1:
        gathered = torch.empty(world, args.batch, args.heads, 128, dtype=torch.bfloat16, device=dev)
        gathered_all = torch.empty(world, args.layers, args.batch, args.heads, 128, dtype=torch.bfloat16, device=dev)

    def layer_pass(i):
        q, cache = layers[i % R]
        out = select_prune_attend_step(q, cache, ws, variant=args.variant, out=outs[i % args.layers])
        if world > 1 and args.gather_per_layer:
            dist.all_gather_into_tensor(gathered.view(-1, args.heads, 128), out)

    def token_step():
        for i in range(args.layers):
            layer_pass(i)
        if world > 1 and not args.gather_per_layer:
            dist.all_gather_into_tensor(gathered_all.view(-1, args.batch, args.heads, 128), outs)

    # one eager step (also sets function attributes before any capture)
    token_step()
    torch.cuda.synchronize()
    if int(ws.status.item()) != 0:
        raise RuntimeError(f"device status flags raised: {int(ws.status.item())}")
    budgets = []
    for i in range(R):
        layer_pass(i)
        budgets.append(ws.budget.clone())
    avg_budget = float(torch.stack(budgets).float().mean().item())

    log(f"eager step done, avg budget {avg_budget:.1f}")
    graph = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                token_step()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                token_step()
        except Exception as e:  # fall back to eager launches
            sys.stderr.write(f"[bench] CUDA graph capture failed ({e}); timing eager launches\n")
            graph = None
    run_step = graph.replay if graph is not None else token_step
    log(f"graph captured: {graph is not None}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    torch.cuda.synchronize()
    elapsed_ms = e0.elapsed_time(e1)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    log("timed region done")
    ms_per_step = elapsed_ms / args.steps
    value = args.batch * world / (ms_per_step * 1e-3)

    # ---- per-kernel timings (CUDA events on the launching stream) and the roofline ----------
    q0, c0 = layers[0]
    names = ["quest_page_scores", "quest_topk_pages", "estimate_int4", "topp_prune", "sparse_decode_attn"]
    lib = _lib.load()
    launch_stream = [torch.cuda.current_stream().cuda_stream]

    def launch(kname, q, cache):
        s = launch_stream[0]
        b, hq, hkv = args.batch, args.heads, args.kv_heads
        if kname == "quest_page_scores":
            return lib.twl_quest_page_scores(q.data_ptr(), 1, cache.kmeta.data_ptr(), cache.kv_indptr.data_ptr(),
                                             cache.kv_indices.data_ptr(), b, hq, hkv, cache.kmeta.shape[0],
                                             ws.page_scores.data_ptr(), ws.max_pages, ws.status.data_ptr(), s)
        if kname == "quest_topk_pages":
            return lib.twl_quest_topk_pages(ws.page_scores.data_ptr(), ws.max_pages, cache.kv_indptr.data_ptr(), b, hq,
                                            cfg.token_budget, ws.cand_pages.data_ptr(), ws.cand_npages.data_ptr(),
                                            ws.cand_pages.shape[-1], s)
        if kname == "estimate_int4":
            return lib.twl_estimate_int4(q.data_ptr(), 1, cache.k4_pages.data_ptr(), cache.kv_indptr.data_ptr(),
                                         cache.kv_indices.data_ptr(), cache.kv_last_page_len.data_ptr(),
                                         ws.cand_pages.data_ptr(), ws.cand_npages.data_ptr(), ws.cand_pages.shape[-1],
                                         b, hq, hkv, cache.k4_pages.shape[0], 1 / math.sqrt(128),
                                         ws.scores.data_ptr(), ws.scores.shape[-1], args.variant,
                                         ws.status.data_ptr(), s)
        if kname == "topp_prune":
            return lib.twl_topp_prune(ws.scores.data_ptr(), ws.scores.shape[-1], cache.kv_indptr.data_ptr(),
                                      cache.kv_last_page_len.data_ptr(), ws.cand_pages.data_ptr(),
                                      ws.cand_npages.data_ptr(), ws.cand_pages.shape[-1], b, hq, None, cfg.threshold,
                                      ws.indices.data_ptr(), ws.indices.shape[-1], ws.budget.data_ptr(),
                                      ws.threshold.data_ptr(), ws.status.data_ptr(), s)
        return lib.twl_sparse_decode_attn(q.data_ptr(), 1, cache.k_pages.data_ptr(), cache.v_pages.data_ptr(),
                                          cache.kv_indptr.data_ptr(), cache.kv_indices.data_ptr(),
                                          ws.indices.data_ptr(), ws.indices.shape[-1], ws.budget.data_ptr(), b, hq, hkv,
                                          cache.k_pages.shape[0], 1 / math.sqrt(128), ws.out.data_ptr(),
                                          ws.attn_ws.data_ptr(), ws.attn_ws.numel(), ws.attn_chunk,
                                          ws.status.data_ptr(), s)

    ktimes = {n: [] for n in names}
    for rep in range(args.kernel_reps):
        for i in range(R):
            q, cache = layers[i]
            for n in names:
                a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                st = launch(n, q, cache)
                b_.record()
                if st != 0:
                    raise RuntimeError(f"{n} returned {st}")
                ktimes[n].append((a, b_))
    torch.cuda.synchronize()
    kavg = {n: statistics.mean(x.elapsed_time(y) for x, y in v[R:]) if len(v) > R else
            statistics.mean(x.elapsed_time(y) for x, y in v) for n, v in ktimes.items()}
    bytes_ = step_algorithmic_bytes(c0, args.heads, cfg, torch.stack(budgets).float().mean(0))
    kbytes = {"quest_page_scores": bytes_["selector"] + c0.max_pages * 4 * args.batch * args.kv_heads,
              "estimate_int4": bytes_["estimator"],
              "sparse_decode_attn": bytes_["attention"]}
    dominant = max(kavg, key=kavg.get)
    peaks = {}
    try:
        peaks = json.load(open(ROOT / "MEASURED_PEAKS.json"))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
    dom_bytes = kbytes.get(dominant, 0.0)
    # DRAM traffic per (sequence, KV head) row from the ncu capture summarised in
    # profiles/kernels_config1_small_case_ncu_full.md (256 rows; traffic is proportional to rows);
    # only valid for the configuration that capture was taken on
    ncu_bytes_per_row = {"quest_page_scores": 274.49e6 / 256, "estimate_int4": 175.33e6 / 256}
    traffic = None
    if (args.ctx, args.token_budget, args.heads, args.kv_heads) == (32768, 8192, 32, 32) and dominant in ncu_bytes_per_row:
        traffic = ncu_bytes_per_row[dominant] * args.batch * args.kv_heads
    achieved = dom_bytes / (kavg[dominant] * 1e-3) / 1e9 if dom_bytes else 0.0
    step_gbs = bytes_["total"] * args.layers / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth", "traffic": traffic,
                "algorithmic_bytes_per_launch": dom_bytes,
                "kernels_ms": {k: round(v, 5) for k, v in kavg.items()},
                "kernels_gbs": {k: round(kbytes[k] / (kavg[k] * 1e-3) / 1e9, 1) for k in kbytes},
                "step": {"algorithmic_bytes_per_layer_pass": bytes_["total"], "achieved": step_gbs,
                         "frac": step_gbs / peak, "frac_of_8000_nominal": step_gbs / 8000.0}}

    if args.ablation:
        def chain_us(skip):
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                s_ = st.cuda_stream
                launch_stream[0] = s_
                def one_pass(i):
                    q, cache = layers[i % R]
                    for n in names:
                        if n != skip and launch(n, q, cache) != 0:
                            raise RuntimeError(n)
                for i in range(R):
                    one_pass(i)
                st.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    for i in range(8 * R):
                        one_pass(i)
                for _ in range(3):
                    g.replay()
                a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(st)
                for _ in range(10):
                    g.replay()
                b_.record(st)
                st.synchronize()
                g.reset()
            return a.elapsed_time(b_) / (10 * 8 * R) * 1000.0
        full_us = chain_us(None)
        roofline["chain"] = {"layer_pass_us": round(full_us, 2),
                             "marginal_us": {n: round(full_us - chain_us(n), 2) for n in names}}
        launch_stream[0] = torch.cuda.current_stream().cuda_stream
    log("per-kernel timing done")
    # ---- end to end: q from pinned host memory in, output to pinned host memory out ------------
    e2e = None
    if not args.no_e2e:
        host_q = torch.stack([layers[i % R][0].cpu() for i in range(args.layers)]).pin_memory()
        host_out = torch.empty(args.layers, args.batch, args.heads, 128, dtype=torch.bfloat16).pin_memory()
        dq = torch.empty(args.layers, *layers[0][0].shape, dtype=layers[0][0].dtype, device=dev)
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        last = args.layers - 1

        def e2e_body():
            # per token: every layer's q from pinned host memory, the kernels, every layer's output
            # back to pinned memory.  Two copies each way on two side streams (the two copy engines):
            # the first layer's q alone, so that it can start at once, the other layers' q while it
            # runs; the outputs of all layers but the last while the last one runs, then the last.
            # The kernel chain on the main stream stays free of copy nodes.
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            s_in.wait_event(fork)
            s_out.wait_event(fork)
            first_in, rest_in = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(s_in):
                dq[:1].copy_(host_q[:1], non_blocking=True)
                first_in.record(s_in)
                if last > 0:
                    dq[1:].copy_(host_q[1:], non_blocking=True)
                rest_in.record(s_in)
            main.wait_event(first_in)
            for i in range(args.layers):
                if i == 1:
                    main.wait_event(rest_in)
                out = select_prune_attend_step(dq[i], layers[i % R][1], ws, variant=args.variant, out=outs[i])
                if world > 1 and args.gather_per_layer:
                    dist.all_gather_into_tensor(gathered.view(-1, args.heads, 128), out)
                if i == last - 1:
                    most_done = torch.cuda.Event()
                    most_done.record(main)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(most_done)
                        host_out[:last].copy_(outs[:last], non_blocking=True)
            if world > 1 and not args.gather_per_layer:
                dist.all_gather_into_tensor(gathered_all.view(-1, args.batch, args.heads, 128), outs)
            host_out[last:].copy_(outs[last:], non_blocking=True)
            join_in, join_out = torch.cuda.Event(), torch.cuda.Event()
            join_in.record(s_in)
            join_out.record(s_out)
            main.wait_event(join_in)
            main.wait_event(join_out)

        # the copies use fixed pinned buffers, so the whole token step (copies included) is one graph;
        # a caller refills the pinned q buffers before each replay
        e2e_graph = None
        e2e_body()
        torch.cuda.synchronize()
        if not args.no_graph:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    e2e_body()
                torch.cuda.current_stream().wait_stream(side)
                e2e_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_graph):
                    e2e_body()
            except Exception as e:
                sys.stderr.write(f"[bench] e2e graph capture failed ({e}); timing eager launches\n")
                e2e_graph = None

        def e2e_step():
            if e2e_graph is not None:
                e2e_graph.replay()
            else:
                e2e_body()
            torch.cuda.synchronize()   # the host holds the token's outputs from here on

        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        t1 = time.perf_counter()
        barrier()
        dt = t1 - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        nbytes = args.batch * args.heads * 128 * 2 * args.layers
        e2e = {"value": args.batch * world * args.steps / dt, "unit": "tokens/s",
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "cuda_graph": e2e_graph is not None}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        seqs = min(8, args.batch)
        data = cpu_reference_inputs(args, args.heads, seqs)
        cpu_reference_step(args, data[:1])
        times = []
        while sum(times) < 12.0 and len(times) < 20:
            times.append(cpu_reference_step(args, data))
        t = statistics.mean(times)
        cpu_baseline = {"value": seqs / (t * args.layers), "unit": "tokens/s", "cores": torch.get_num_threads(),
                        "kind": "port",
                        "sample": f"{len(times)} x (1 of {args.layers} layer passes over {seqs} of {args.batch} "
                                  f"sequences x {args.heads} heads at ctx {args.ctx}), {sum(times):.1f} s of CPU "
                                  f"work; tokens/s = sequences / (mean pass time x layers)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
            "tokens_per_s_per_gpu": value / world, "tokens_per_s_per_layer_pass": value * args.layers,
            "avg_pruned_budget": avg_budget, "cuda_graph": graph is not None,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
            "gpu_launches": ws.kernels_per_step * args.layers * args.steps,
        }
        print(json.dumps(line))
    if world > 1:
        # A captured graph that holds NCCL kernels made communicator teardown stall at exit; the
        # result is out, so synchronise, release the graph and leave without the teardown.
        sys.stdout.flush()
        torch.cuda.synchronize()
        dist.barrier()
        if graph is not None:
            graph.reset()
        if not args.no_e2e and e2e_graph is not None:
            e2e_graph.reset()
        log("done")
        os._exit(0)


if __name__ == "__main__":
    main()
