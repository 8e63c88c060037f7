#!/usr/bin/env python
"""Benchmark of the Select-then-Prune decode step (Quest selector -> INT4 estimator -> top-p
pruner -> sparse paged attention) on synthetic inputs.

Headline workload (the JSON line's ``value``): the Longchat-7B-class configuration, B=16 sequences
of 32768 tokens, 32 query heads = 32 KV heads, head_dim 128, page size 16, Quest budget 8192,
top-p 0.95, bf16, 32 attention layers per decoded token, inputs generated exactly as that
configuration states them ("literal" recipe: all softmax mass on the sink, pruned budget 1).
One "step" decodes one token for the whole batch: 32 layer passes of the hot path.  Only
``--resident-layers`` distinct layers' caches are held in HBM (one layer is 8 GiB of K/V plus
1.25 GiB of INT4 K and 0.5 GiB of page metadata); the 32 passes cycle through them, so every
pass streams data that is far larger than L2 and was last touched several passes ago.

The same line carries, under ``variants``, short timed runs of the other workloads: the same
configuration with budgets near rho*L ("mid") and in the thousands ("calibrated"), the
Llama-3-8B-class GQA configuration with ragged lengths and no selector, and one GPU's shard of
the Llama-3-70B-class configuration; under ``gemv_sweep`` the standalone INT4 estimator at
B in {1,16,64} x L in {4096..131072} (warm-up 10 / repeats 100, as
benchmark/efficiency/bench_gemv.py:458-470 of the reference times its GEMV); under
``topp_vs_reference`` the top-p operators against the reference's own CUDA kernel on the same
rows; and, on more than one GPU, under ``strong`` the same global problems partitioned over the
ranks by (sequence, KV head) units with a check of gathered rows.

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

# name -> workload.  ctx: an int, or (lo, hi) for ragged lengths drawn uniformly; token_budget 0 =
# no selector; rho: heavy-hitter density, or a (lo, hi) range drawn per (sequence, KV head).
PRESETS = {
    "config1": dict(title="Longchat-7B-class decode attention", batch=16, heads=32, kv_heads=32, ctx=32768,
                    token_budget=8192, top_p=0.95, rho=0.005, layers=32, recipe="literal"),
    "config2": dict(title="Llama-3-8B-class GQA decode attention", batch=64, heads=32, kv_heads=8,
                    ctx=(8192, 32768), token_budget=0, top_p=0.9, rho=(0.001, 0.05), layers=32, recipe="mid"),
    "config4_shard": dict(title="Llama-3-70B-class decode attention, one GPU's KV head of 8", batch=128, heads=8,
                          kv_heads=1, ctx=65536, token_budget=16384, top_p=0.95, rho=0.005, layers=80,
                          recipe="mid"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=20,
                    help="the steps-long timed loop is repeated this often; ms_per_step is the median")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="config1", choices=sorted(PRESETS))
    ap.add_argument("--batch", type=int)
    ap.add_argument("--ctx", type=int)
    ap.add_argument("--heads", type=int)
    ap.add_argument("--kv-heads", type=int)
    ap.add_argument("--layers", type=int)
    ap.add_argument("--resident-layers", type=int, default=4)
    ap.add_argument("--token-budget", type=int)
    ap.add_argument("--top-p", type=float)
    ap.add_argument("--rho", type=float)
    ap.add_argument("--recipe", choices=["literal", "mid", "calibrated"])
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--gather-per-layer", action="store_true",
                    help="all-gather the outputs after every layer pass instead of once per decoded token")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-shuffle", action="store_true",
                    help="consecutive physical pages instead of a random page table (shows what scattered pages cost)")
    ap.add_argument("--no-variants", action="store_true",
                    help="headline workload only: no variants, GEMV sweep, reference-kernel or strong-scaling legs")
    ap.add_argument("--only", default="",
                    help="comma list of extra legs to run (variants, gemv, topp, strong); default: all")
    ap.add_argument("--kernel-reps", type=int, default=5)
    ap.add_argument("--attn-chunk", type=int, default=512, help="tokens per split-KV work item of the attention kernel")
    ap.add_argument("--ablation", action="store_true",
                    help="also time the captured layer pass with each kernel left out (its marginal cost in the chain)")
    args = ap.parse_args()
    preset = dict(PRESETS[args.preset])
    for key in ("batch", "ctx", "heads", "kv_heads", "layers", "token_budget", "top_p", "rho", "recipe"):
        if getattr(args, key) is None:
            setattr(args, key, preset[key])
    args.title = preset["title"]
    return args


def workload_from_args(args):
    return dict(title=args.title, batch=args.batch, heads=args.heads, kv_heads=args.kv_heads, ctx=args.ctx,
                token_budget=args.token_budget, top_p=args.top_p, rho=args.rho, layers=args.layers,
                recipe=args.recipe)


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
    L, D = args.ctx if isinstance(args.ctx, int) else args.ctx[1], 128
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
    sel = dict(selector="quest", token_budget=args.token_budget, chunk_size=16) if args.token_budget > 0 \
        else dict(selector="none")
    t0 = time.perf_counter()
    for q, k, v in data:
        O.decode_step(q, k, v, quant_group=32, threshold=args.top_p, **sel)
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
        "config": workload_config(args, workload_from_args(args), 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, w, n):
    sel = f"Quest {w['token_budget']}" if w["token_budget"] > 0 else "no selector"
    return {"workload": f"{w['title']}, B={w['batch']}/GPU, ctx {w['ctx']}, "
                        f"{w['heads']}q/{w['kv_heads']}kv heads, d128, page 16, {sel} + top-p {w['top_p']}, "
                        f"{w['layers']} layers/token",
            "global_batch": w["batch"] * n, "seq_len": w["ctx"], "parallelism": f"(batch,kv-head) shards x{n}",
            "recipe": w["recipe"], "resident_layers": args.resident_layers,
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


def measured_peak():
    peaks = {}
    try:
        peaks = json.load(open(ROOT / "MEASURED_PEAKS.json"))
    except Exception:
        pass
    return float(peaks.get("hbm_gbs", 6650.0)), ("measured" if "hbm_gbs" in peaks else "fallback")


def ncu_traffic_per_row():
    """DRAM bytes per (sequence, KV head) row of the two streaming kernels on the headline
    configuration, from the committed ncu capture (traffic is proportional to rows)."""
    try:
        d = json.load(open(ROOT / "profiles" / "kernels_config1_small_case_traffic.json"))
        return {k: float(v["dram_bytes"]) / float(v["rows"]) for k, v in d["kernels"].items()}, d["valid_for"]
    except Exception:
        return {}, {}


class Harness:
    """One workload resident on one GPU: its layers' caches, the step workspace, the captured
    graph of a decoded token, and the timings taken on it."""
    KERNELS = ["quest_page_scores", "quest_topk_pages", "estimate_int4", "topp_prune", "sparse_decode_attn"]

    def __init__(self, w, dev, *, resident_layers, attn_chunk, variant, seed_base, units=None, dist=None,
                 world=1, gather_per_layer=False, use_graph=True, shuffle=True):
        from twilight_b200.gen import make_decode_inputs, make_unit_inputs, ragged_lengths
        from twilight_b200.step import DecodeWorkspace, SparseConfig
        self.w, self.dev, self.variant, self.dist, self.world = w, dev, variant, dist, world
        self.gather_per_layer = gather_per_layer
        self.n_layers = w["layers"]
        self.quest = w["token_budget"] > 0
        self.cfg = SparseConfig(selector="quest" if self.quest else "none", token_budget=w["token_budget"],
                                weight_pruner="top_p", threshold=w["top_p"])
        self.R = max(1, min(resident_layers, self.n_layers))
        rho = tuple(w["rho"]) if isinstance(w["rho"], (tuple, list)) else w["rho"]
        if units is None:
            lens = w["ctx"] if isinstance(w["ctx"], int) else ragged_lengths(w["batch"], w["ctx"][0], w["ctx"][1], seed=2)
            self.batch, self.heads, self.kv_heads = w["batch"], w["heads"], w["kv_heads"]
        else:  # a rank's block of a global problem: (batch ids, kv head ids, lengths of those sequences)
            self.batch, self.kv_heads = len(units[0]), len(units[1])
            self.heads = self.kv_heads * (w["heads"] // w["kv_heads"])
        self.layers = []
        for l in range(self.R):
            if units is None:
                q, cache = make_decode_inputs(self.batch, self.heads, self.kv_heads, lens, rho=rho,
                                              dtype=torch.bfloat16, device=dev, seed=seed_base + l,
                                              recipe=w["recipe"], shuffle_pages=shuffle)
            else:
                q, cache = make_unit_inputs(units[0], units[1], w["heads"] // w["kv_heads"], units[2], rho=rho,
                                            dtype=torch.bfloat16, device=dev, seed=seed_base + l,
                                            recipe=w["recipe"], shuffle_pages=True)
            self.layers.append((q, cache))
        self.ws = DecodeWorkspace.for_cache(self.layers[0][1], self.heads, self.cfg, attn_chunk=attn_chunk)
        # Outputs of all layer passes of one token.  A rank's heads feed its own slice of the output
        # projection, so nothing has to cross GPUs between layers; the per-token result is gathered
        # once (NCCL all-gather), or after every layer pass with --gather-per-layer.
        self.outs = torch.empty(self.n_layers, self.batch, self.heads, 128, dtype=torch.bfloat16, device=dev)
        self.gathered = self.gathered_all = None
        if world > 1:
            self.gathered = torch.empty(world, self.batch, self.heads, 128, dtype=torch.bfloat16, device=dev)
            self.gathered_all = torch.empty(world, self.n_layers, self.batch, self.heads, 128, dtype=torch.bfloat16,
                                            device=dev)
        self.graph = None
        self.use_graph = use_graph
        self.kernel_names = [k for k in self.KERNELS if self.quest or not k.startswith("quest_")]

    # ---- the step ------------------------------------------------------------------------------
    def layer_pass(self, i, q=None):
        from twilight_b200.step import select_prune_attend_step
        lq, cache = self.layers[i % self.R]
        out = select_prune_attend_step(lq if q is None else q, cache, self.ws, variant=self.variant,
                                       out=self.outs[i % self.n_layers])
        if self.world > 1 and self.gather_per_layer:
            self.dist.all_gather_into_tensor(self.gathered.view(-1, self.heads, 128), out)
        return out

    def token_step(self):
        for i in range(self.n_layers):
            self.layer_pass(i)
        if self.world > 1 and not self.gather_per_layer:
            self.dist.all_gather_into_tensor(self.gathered_all.view(-1, self.batch, self.heads, 128), self.outs)

    def prepare(self):
        """One eager step (sets function attributes before any capture), budgets, graph capture."""
        self.token_step()
        torch.cuda.synchronize()
        st = int(self.ws.status.item())
        budgets = []
        for i in range(self.R):
            self.layer_pass(i)
            budgets.append(self.ws.budget.clone())
        self.budgets = torch.stack(budgets).float()
        self.avg_budget = float(self.budgets.mean().item())
        self.status = st | int(self.ws.status.item())
        if self.status != 0:
            raise RuntimeError(f"device status flags raised: {self.status}")
        if self.use_graph:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.token_step()
                torch.cuda.current_stream().wait_stream(side)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    self.token_step()
            except Exception as e:  # fall back to eager launches
                sys.stderr.write(f"[bench] CUDA graph capture failed ({e}); timing eager launches\n")
                self.graph = None
        self.run_step = self.graph.replay if self.graph is not None else self.token_step

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def time_steps(self, steps, warmup, repeats):
        """``repeats`` timed loops of ``steps`` decoded tokens each (CUDA events on the launching
        stream, a barrier and a synchronize on both sides, max over ranks per loop).
        Returns ms per step of every loop."""
        for _ in range(max(warmup, 3)):
            self.run_step()
        self.barrier()
        per = []
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                self.run_step()
            e1.record()
            torch.cuda.synchronize()
            per.append(e0.elapsed_time(e1) / steps)
            self.barrier()
        if self.world > 1:
            t = torch.tensor(per, device=self.dev, dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            per = [float(x) for x in t.tolist()]
        return per

    # ---- single kernels ----------------------------------------------------------------------------
    def launch(self, kname, q, cache, stream):
        from twilight_b200 import _lib
        lib, ws, cfg = _lib.load(), self.ws, self.cfg
        b, hq, hkv = self.batch, self.heads, self.kv_heads
        cp = ws.cand_pages.data_ptr() if self.quest else None
        cn = ws.cand_npages.data_ptr() if self.quest else None
        mk = ws.cand_pages.shape[-1] if self.quest else 0
        sm = 1 / math.sqrt(128)
        if kname == "quest_page_scores":
            return lib.twl_quest_page_scores(q.data_ptr(), 1, cache.kmeta.data_ptr(), cache.kv_indptr.data_ptr(),
                                             cache.kv_indices.data_ptr(), b, hq, hkv, cache.kmeta.shape[0],
                                             ws.page_scores.data_ptr(), ws.max_pages, ws.status.data_ptr(), stream)
        if kname == "quest_topk_pages":
            return lib.twl_quest_topk_pages(ws.page_scores.data_ptr(), ws.max_pages, cache.kv_indptr.data_ptr(), b, hq,
                                            cfg.token_budget, cp, cn, mk, stream)
        if kname == "estimate_int4":
            return lib.twl_estimate_int4(q.data_ptr(), 1, cache.k4_pages.data_ptr(), cache.kv_indptr.data_ptr(),
                                         cache.kv_indices.data_ptr(), cache.kv_last_page_len.data_ptr(), cp, cn, mk,
                                         b, hq, hkv, cache.k4_pages.shape[0], sm, ws.scores.data_ptr(),
                                         ws.scores.shape[-1], self.variant, ws.status.data_ptr(), stream)
        if kname == "topp_prune":
            return lib.twl_topp_prune(ws.scores.data_ptr(), ws.scores.shape[-1], cache.kv_indptr.data_ptr(),
                                      cache.kv_last_page_len.data_ptr(), cp, cn, mk, b, hq, None, cfg.threshold,
                                      ws.indices.data_ptr(), ws.indices.shape[-1], ws.budget.data_ptr(),
                                      ws.threshold.data_ptr(), ws.status.data_ptr(), stream)
        return lib.twl_sparse_decode_attn(q.data_ptr(), 1, cache.k_pages.data_ptr(), cache.v_pages.data_ptr(),
                                          cache.kv_indptr.data_ptr(), cache.kv_indices.data_ptr(),
                                          ws.indices.data_ptr(), ws.indices.shape[-1], ws.budget.data_ptr(), b, hq, hkv,
                                          cache.k_pages.shape[0], sm, ws.out.data_ptr(), ws.attn_ws.data_ptr(),
                                          ws.attn_ws.numel(), ws.attn_chunk, ws.status.data_ptr(), stream)

    def time_kernels(self, reps):
        """Mean duration (ms) of every kernel launched alone, CUDA events on the launching stream;
        the first pass over the resident layers is warm-up."""
        stream = torch.cuda.current_stream().cuda_stream
        ev = {n: [] for n in self.kernel_names}
        for _ in range(max(2, reps)):
            for i in range(self.R):
                q, cache = self.layers[i]
                for n in self.kernel_names:
                    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    st = self.launch(n, q, cache, stream)
                    b_.record()
                    if st != 0:
                        raise RuntimeError(f"{n} returned {st}")
                    ev[n].append((a, b_))
        torch.cuda.synchronize()
        return {n: statistics.mean(x.elapsed_time(y) for x, y in v[self.R:]) for n, v in ev.items()}

    def algorithmic_bytes(self):
        """Bytes a layer pass must move from HBM, per stage (averaged over the resident layers'
        budgets).  For query-head groups the attention term counts every kept token of a KV head
        once (the union over the group's heads): the group shares the K/V rows."""
        from twilight_b200.kernel import ops
        from twilight_b200.step import step_algorithmic_bytes
        c0 = self.layers[0][1]
        by = step_algorithmic_bytes(c0, self.heads, self.cfg, self.budgets.mean(0))
        g = self.heads // self.kv_heads
        by["attention_sum_over_heads"] = by["attention"]
        if g > 1:
            union = 0.0
            for i in range(self.R):
                self.layer_pass(i)
                L = max(self.layers[i][1].seq_lens)
                for b0 in range(0, self.batch, 16):   # in slices: the dense mask is B x H x L bytes
                    b1 = min(self.batch, b0 + 16)
                    m = ops.indices_to_mask(self.ws.indices[b0:b1].contiguous(), self.ws.budget[b0:b1].contiguous(), L)
                    union += float(m.view(b1 - b0, self.kv_heads, g, L).any(2).sum().item())
                    del m
            union /= self.R
            att = union * 2 * 128 * 2
            by["total"] += att - by["attention"]
            by["attention"] = att
        by["kernel"] = {"quest_page_scores": by["selector"] + (c0.max_pages * 4 * self.batch * self.kv_heads
                                                                 if self.quest else 0),
                        "estimate_int4": by["estimator"], "sparse_decode_attn": by["attention"]}
        return by

    def chain_ablation(self):
        """The captured layer pass timed whole and with each kernel left out."""
        names = self.kernel_names

        def chain_us(skip):
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                s_ = st.cuda_stream

                def one_pass(i):
                    q, cache = self.layers[i % self.R]
                    for n in names:
                        if n != skip and self.launch(n, q, cache, s_) != 0:
                            raise RuntimeError(n)
                for i in range(self.R):
                    one_pass(i)
                st.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    for i in range(8 * self.R):
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
            return a.elapsed_time(b_) / (10 * 8 * self.R) * 1000.0
        full_us = chain_us(None)
        return {"layer_pass_us": round(full_us, 2),
                "marginal_us": {n: round(full_us - chain_us(n), 2) for n in names}}

    def release(self):
        if self.graph is not None:
            self.graph.reset()
        self.graph = None
        self.layers = []
        self.ws = None
        self.outs = self.gathered = self.gathered_all = None
        torch.cuda.empty_cache()


def roofline_block(h, ms_per_step, kavg, by, peak, peak_kind, traffic=None, dominant=None):
    kbytes = by["kernel"]
    dominant = dominant or max(kavg, key=kavg.get)
    dom_bytes = kbytes.get(dominant, 0.0)
    achieved = dom_bytes / (kavg[dominant] * 1e-3) / 1e9 if dom_bytes else 0.0
    step_gbs = by["total"] * h.n_layers / (ms_per_step * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth", "traffic": traffic,
            "algorithmic_bytes_per_launch": dom_bytes,
            "kernels_ms": {k: round(v, 5) for k, v in kavg.items()},
            "kernels_gbs": {k: round(kbytes[k] / (kavg[k] * 1e-3) / 1e9, 1) for k in kbytes if k in kavg},
            "kernels_frac": {k: round(kbytes[k] / (kavg[k] * 1e-3) / 1e9 / peak, 4) for k in kbytes if k in kavg},
            "step": {"algorithmic_bytes_per_layer_pass": by["total"], "achieved": step_gbs,
                     "frac": step_gbs / peak, "frac_of_8000_nominal": step_gbs / 8000.0}}


def run_variant(name, w, args, dev, peak, peak_kind, steps, repeats, resident=2):
    """A short timed run of one more workload, same measurements as the headline."""
    t0 = time.time()
    h = Harness(w, dev, resident_layers=resident, attn_chunk=args.attn_chunk, variant=args.variant,
                seed_base=7000, use_graph=not args.no_graph)
    try:
        h.prepare()
        per = h.time_steps(steps, 3, repeats)
        ms = statistics.median(per)
        kavg = h.time_kernels(3)
        by = h.algorithmic_bytes()
        roof = roofline_block(h, ms, kavg, by, peak, peak_kind)
        out = {"workload": workload_config(args, w, 1)["workload"], "recipe": w["recipe"], "status": h.status,
               "ms_per_step": ms, "ms_per_step_min": min(per), "ms_per_step_max": max(per), "steps": steps,
               "repeats": repeats, "resident_layers": h.R, "tokens_per_s": w["batch"] / (ms * 1e-3),
               "layer_pass_us": ms * 1e3 / h.n_layers, "avg_pruned_budget": h.avg_budget,
               "cuda_graph": h.graph is not None, "kernels_ms": roof["kernels_ms"], "kernels_gbs": roof["kernels_gbs"],
               "kernels_frac": roof["kernels_frac"], "step": roof["step"],
               "algorithmic_bytes": {k: by[k] for k in ("selector", "estimator", "attention",
                                                        "attention_sum_over_heads", "metadata", "q_out", "total")},
               "gpu_launches": h.ws.kernels_per_step * h.n_layers * steps * repeats}
        if args.ablation:
            out["chain"] = h.chain_ablation()
    finally:
        h.release()
    out["wall_s"] = round(time.time() - t0, 1)
    log(f"variant {name}: {out['ms_per_step']:.3f} ms/step, budget {out['avg_pruned_budget']:.1f}, "
        f"step frac {out['step']['frac']:.3f}")
    return out


# ---------------------------------------------------------------------------------------------
# standalone INT4 estimator sweep (the reference's bench_gemv, extended)
# ---------------------------------------------------------------------------------------------
def gemv_sweep(dev, peak):
    """Raw q.k of every token of every sequence (``batched_sparse_gemv_int4_k``, the call of
    benchmark/efficiency/bench_gemv.py:445-454): rows = B*32 KV heads, fp16 queries, group-32 fp16
    scale/min, fp32 scores.  Warm-up 10, repeats 100, CUDA events (bench_gemv.py:458-470).  Sizes
    whose slabs would fit in L2 rotate through disjoint page sets so that every launch reads HBM."""
    from twilight_b200.kernel import ops
    hkv, page = 32, 16
    bs, ls = (1, 16, 64), (4096, 16384, 65536, 131072)
    max_pages_total = max(bs) * max(ls) // page
    k4 = torch.empty(max_pages_total, hkv, 1280, dtype=torch.uint8, device=dev)
    gen = torch.Generator(device=dev).manual_seed(3)
    step = 1 << 15
    for p0 in range(0, max_pages_total, step):          # codes: random bytes; scale/min: finite fp16
        p1 = min(max_pages_total, p0 + step)
        k4[p0:p1].view(torch.int64).random_(generator=gen)
        sz = torch.empty(p1 - p0, hkv, 64, 2, dtype=torch.float16, device=dev)
        sz[..., 0] = (torch.rand(p1 - p0, hkv, 64, generator=gen, device=dev) * 0.4 + 0.05).half()
        sz[..., 1] = torch.randn(p1 - p0, hkv, 64, generator=gen, device=dev).half()
        k4[p0:p1, :, 1024:] = sz.view(torch.uint8).reshape(p1 - p0, hkv, 256)
        del sz
    out = []
    for b in bs:
        q = torch.randn(b, hkv, 128, generator=gen, device=dev).half()
        for L in ls:
            n_pages = L // page
            bytes_ = b * hkv * L * 80 + b * hkv * L * 4 + q.numel() * 2
            n_rot = max(1, min(max_pages_total // (b * n_pages), math.ceil(512e6 / bytes_)))
            tables = []
            for r in range(n_rot):
                perm = torch.randperm(b * n_pages, generator=gen, device=dev).int() + r * b * n_pages
                tables.append(perm)
            indptr = (torch.arange(b + 1, dtype=torch.int32) * n_pages).to(dev)
            last = torch.full((b,), page, dtype=torch.int32, device=dev)
            o = torch.empty(b, hkv, L, dtype=torch.float32, device=dev)
            for i in range(10):
                ops.batched_sparse_gemv_int4_k(q, o, k4, None, None, tables[i % n_rot], indptr, last)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(100):
                ops.batched_sparse_gemv_int4_k(q, o, k4, None, None, tables[i % n_rot], indptr, last)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 100 * 1e3
            gbs = bytes_ / (us * 1e-6) / 1e9
            out.append({"batch": b, "rows": b * hkv, "L": L, "us": round(us, 2), "GBps": round(gbs, 1),
                        "frac": round(gbs / peak, 4), "bytes": bytes_, "page_sets_rotated": n_rot,
                        "finite": bool(torch.isfinite(o[0, 0, :64]).all().item())})
            del o, tables
    del k4
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------
# top-p operators against the reference's own CUDA kernel
# ---------------------------------------------------------------------------------------------
def topp_vs_reference(dev):
    """``TopPReturnMaskKernel`` (csrc/include/sampling.cuh:119-231, compiled unmodified into
    oracle/_ref by oracle/build_ref.py; a baseline, never on the product path) against this
    library on the same rows: torch fp32 softmax + the reference kernel (twilight/pyimpl/top_p.py:10-15),
    torch fp32 softmax + this library's dense-mask operator, and the fused softmax + search +
    index-list kernel on the raw scores.  10 warm-ups, 50 repeats, CUDA events."""
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except Exception as e:
        return {"unavailable": f"reference kernel not loadable: {e}"}
    if ref is None:
        return {"unavailable": "oracle/_ref/twilight_ref_sampling.so has not been built"}
    from twilight_b200.cache import PagedKVCache
    from twilight_b200.kernel import ops, top_p_fp32_return_mask

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

    rows = []
    for (b, h, L, shape) in [(16, 32, 8192, "sink"), (16, 32, 32768, "sink"), (16, 32, 32768, "flat"),
                             (1, 32, 4096, "sink")]:
        g = torch.Generator(device=dev).manual_seed(0)
        logits = torch.randn(b, h, 1, L, generator=g, device=dev) * (2.0 if shape == "sink" else 1.0)
        if shape == "sink":
            logits[..., 0] += 8.0
        stream = torch.cuda.current_stream().cuda_stream

        def run_ref():
            probs = torch.softmax(logits, -1, dtype=torch.float32)
            mask = torch.zeros_like(probs, dtype=torch.bool)
            ref.top_p_fp32_return_mask(probs, mask, None, 0.95, stream)
            return mask

        def run_mask():
            return top_p_fp32_return_mask(torch.softmax(logits, -1, dtype=torch.float32), 0.95)

        indptr, _, last, _ = PagedKVCache.page_table([L] * b, dev)
        scores = logits.reshape(b, h, L).contiguous()
        idx = torch.empty(b, h, L, dtype=torch.int32, device=dev)
        bud = torch.empty(b, h, dtype=torch.int32, device=dev)

        def run_fused():
            return ops.topp_prune(scores, indptr, last, 0.95, indices=idx, budget=bud)

        m_ref, m_ours = run_ref(), run_mask()
        run_fused()
        torch.cuda.synchronize()
        rows.append({"rows": b * h, "L": L, "shape": shape,
                     "reference_us": round(timeit(run_ref), 1), "mask_op_us": round(timeit(run_mask), 1),
                     "fused_prune_us": round(timeit(run_fused), 1),
                     "masks_equal_frac": float((m_ref == m_ours).float().mean()),
                     "budget_reference": int(m_ref.sum()) / (b * h), "budget_fused": float(bud.float().mean())})
        del logits, scores, idx
    torch.cuda.empty_cache()
    return {"rows": rows, "note": "reference = torch softmax + the reference's kernel; mask_op = torch softmax + "
                                  "twl_top_p_return_mask_f32; fused_prune = twl_topp_prune on raw scores"}


# ---------------------------------------------------------------------------------------------
# strong scaling through the shard plan
# ---------------------------------------------------------------------------------------------
def strong_leg(name, w, args, dev, dist, world, rank, steps, repeats, prefer="batch"):
    """The GLOBAL problem ``w`` partitioned over the ranks by (sequence, KV head) units
    (``twilight_b200.dist.shard_units``); every rank holds only its units' caches, the outputs are
    gathered with one NCCL all-gather per decoded token.  With ``check``, rank 0 rebuilds two units
    of another rank from their seeds, runs them alone and compares budgets (bit-equal) and outputs
    (2e-2) with the gathered rows."""
    from twilight_b200.dist import gather_outputs, shard_units
    from twilight_b200.gen import ragged_lengths
    g = w["heads"] // w["kv_heads"]
    lens = [w["ctx"]] * w["batch"] if isinstance(w["ctx"], int) else ragged_lengths(w["batch"], *w["ctx"], seed=2)
    plan = shard_units(w["batch"], w["kv_heads"], world, lens, prefer=prefer)
    bids, hids = plan.batch_ids[rank], plan.kv_head_ids[rank]
    h = Harness(w, dev, resident_layers=2, attn_chunk=args.attn_chunk, variant=args.variant, seed_base=9000,
                units=(bids, hids, [lens[b] for b in bids]), dist=dist, world=world, use_graph=not args.no_graph)
    try:
        h.prepare()
        per = h.time_steps(steps, 3, repeats)
        ms = statistics.median(per)
        # check leg: layer 0 of the resident set, outputs and budgets placed by the shard plan
        out0 = h.layer_pass(0).clone()
        bud0 = h.ws.budget.clone()
        full = gather_outputs(out0, plan, g, rank)
        full_bud = gather_outputs(bud0.float().unsqueeze(-1), plan, g, rank)[..., 0]
        check = None
        if rank == 0:
            from twilight_b200.gen import make_unit_inputs
            from twilight_b200.step import DecodeWorkspace, select_prune_attend_step
            other = world - 1
            worst, bud_equal, units = 0.0, True, []
            for (b, kvh) in [(plan.batch_ids[other][0], plan.kv_head_ids[other][0]),
                             (plan.batch_ids[other][-1], plan.kv_head_ids[other][-1])]:
                # the owner generated this unit inside a block whose page table depends on the block,
                # but q, K and V of a unit depend only on (seed, sequence, KV head)
                q1, c1 = make_unit_inputs([b], [kvh], g, [lens[b]], rho=tuple(w["rho"]) if isinstance(w["rho"], (tuple, list)) else w["rho"],
                                          dtype=torch.bfloat16, device=dev, seed=9000, recipe=w["recipe"],
                                          shuffle_pages=True)
                ws1 = DecodeWorkspace.for_cache(c1, g, h.cfg, attn_chunk=args.attn_chunk)
                o1 = select_prune_attend_step(q1, c1, ws1)
                torch.cuda.synchronize()
                rows = slice(kvh * g, (kvh + 1) * g)
                worst = max(worst, float((o1[0].float() - full[b, rows].float()).abs().max()))
                bud_equal = bud_equal and bool(torch.equal(ws1.budget[0].float(), full_bud[b, rows]))
                units.append([int(b), int(kvh)])
                del ws1, c1
            check = {"units_of_rank": other, "units": units, "budgets_bit_equal": bud_equal,
                     "max_abs_output_diff": worst, "ok": bool(bud_equal and worst <= 2e-2)}
        res = {"workload": workload_config(args, w, 1)["workload"].replace(f"B={w['batch']}/GPU", f"global B={w['batch']}"),
               "recipe": w["recipe"], "plan": {"sequences_per_rank": len(bids), "kv_heads_per_rank": len(hids)},
               "ms_per_step": ms, "ms_per_step_min": min(per), "ms_per_step_max": max(per), "steps": steps,
               "repeats": repeats, "tokens_per_s": w["batch"] / (ms * 1e-3), "avg_pruned_budget": h.avg_budget,
               "layer_pass_us": ms * 1e3 / h.n_layers, "cuda_graph": h.graph is not None, "check": check}
    finally:
        h.release()
    return res


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    from twilight_b200 import _lib
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
    peak, peak_kind = measured_peak()
    legs = set(x for x in args.only.split(",") if x) or {"variants", "gemv", "topp", "strong"}
    if args.no_variants:
        legs = set()

    w = workload_from_args(args)
    h = Harness(w, dev, resident_layers=args.resident_layers, attn_chunk=args.attn_chunk, variant=args.variant,
                seed_base=1000 * rank, dist=dist, world=world, gather_per_layer=args.gather_per_layer,
                use_graph=not args.no_graph, shuffle=not args.no_shuffle)
    log(f"{h.R} resident layers generated")
    h.prepare()
    log(f"eager step done, avg budget {h.avg_budget:.1f}; graph captured: {h.graph is not None}")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    per = h.time_steps(args.steps, args.warmup, max(1, args.repeats))
    clocks = sampler.stop() if rank == 0 else None
    log("timed region done")
    ms_per_step = statistics.median(per)
    value = args.batch * world / (ms_per_step * 1e-3)

    # ---- per-kernel timings (CUDA events on the launching stream) and the roofline ----------
    kavg = h.time_kernels(args.kernel_reps)
    by = h.algorithmic_bytes()
    per_row, valid_for = ncu_traffic_per_row()
    dominant = max(kavg, key=kavg.get)
    traffic = None
    here = {"ctx": args.ctx, "token_budget": args.token_budget, "heads": args.heads, "kv_heads": args.kv_heads}
    if dominant in per_row and all(valid_for.get(k) == v for k, v in here.items()):
        traffic = per_row[dominant] * args.batch * args.kv_heads
    roofline = roofline_block(h, ms_per_step, kavg, by, peak, peak_kind, traffic, dominant)
    if args.ablation:
        roofline["chain"] = h.chain_ablation()
    log("per-kernel timing done")

    # ---- end to end: q from pinned host memory in, output to pinned host memory out ------------
    e2e = None
    e2e_graph = None
    if not args.no_e2e:
        n_layers, R = h.n_layers, h.R
        host_q = torch.stack([h.layers[i % R][0].cpu() for i in range(n_layers)]).pin_memory()
        host_out = torch.empty(n_layers, h.batch, h.heads, 128, dtype=torch.bfloat16).pin_memory()
        dq = torch.empty(n_layers, *h.layers[0][0].shape, dtype=h.layers[0][0].dtype, device=dev)
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        last = n_layers - 1

        def e2e_body():
            # per token: every layer's q from pinned host memory, the kernels, every layer's output
            # back to pinned memory.  Two copies each way on two side streams (the two copy engines):
            # the first layer's q alone, so that it can start at once, the other layers' q while it
            # runs; the outputs of all layers but the last while the last one runs, then the last.
            # The kernel chain on the main stream stays free of copy nodes.
            main_s = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main_s)
            s_in.wait_event(fork)
            s_out.wait_event(fork)
            first_in, rest_in = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(s_in):
                dq[:1].copy_(host_q[:1], non_blocking=True)
                first_in.record(s_in)
                if last > 0:
                    dq[1:].copy_(host_q[1:], non_blocking=True)
                rest_in.record(s_in)
            main_s.wait_event(first_in)
            for i in range(n_layers):
                if i == 1:
                    main_s.wait_event(rest_in)
                h.layer_pass(i, q=dq[i])
                if i == last - 1:
                    most_done = torch.cuda.Event()
                    most_done.record(main_s)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(most_done)
                        host_out[:last].copy_(h.outs[:last], non_blocking=True)
            if world > 1 and not args.gather_per_layer:
                dist.all_gather_into_tensor(h.gathered_all.view(-1, h.batch, h.heads, 128), h.outs)
            host_out[last:].copy_(h.outs[last:], non_blocking=True)
            join_in, join_out = torch.cuda.Event(), torch.cuda.Event()
            join_in.record(s_in)
            join_out.record(s_out)
            main_s.wait_event(join_in)
            main_s.wait_event(join_out)

        # the copies use fixed pinned buffers, so the whole token step (copies included) is one graph;
        # a caller refills the pinned q buffers before each replay
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
        h.barrier()
        n_e2e = args.steps * min(5, max(1, args.repeats))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        t1 = time.perf_counter()
        h.barrier()
        dt = t1 - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        nbytes = h.batch * h.heads * 128 * 2 * n_layers
        e2e = {"value": args.batch * world * n_e2e / dt, "unit": "tokens/s", "steps": n_e2e,
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "cuda_graph": e2e_graph is not None}
        log("end-to-end timing done")

    headline_launches = h.ws.kernels_per_step * h.n_layers * args.steps * max(1, args.repeats)
    cuda_graph = h.graph is not None
    avg_budget = h.avg_budget
    # release the headline's graphs and caches before the other legs (and, on several ranks, before
    # the process group goes away: see the end of main)
    if e2e_graph is not None:
        e2e_graph.reset()
        e2e_graph = None
    h.release()

    extra = {}
    if world == 1 and "variants" in legs and args.preset == "config1" and args.recipe == "literal":
        variants = {}
        todo = [("config1_mid", dict(PRESETS["config1"], recipe="mid"), 5, 5),
                ("config1_calibrated", dict(PRESETS["config1"], recipe="calibrated"), 3, 3),
                ("config2", PRESETS["config2"], 2, 3),
                ("config4_shard", PRESETS["config4_shard"], 1, 3)]
        for name, vw, vsteps, vrep in todo:
            try:
                variants[name] = run_variant(name, vw, args, dev, peak, peak_kind, vsteps, vrep)
            except Exception as e:  # a failed leg must not take the headline with it
                variants[name] = {"status": -1, "error": f"{type(e).__name__}: {e}"}
                torch.cuda.empty_cache()
        extra["variants"] = variants
    if world == 1 and "gemv" in legs:
        try:
            extra["gemv_sweep"] = gemv_sweep(dev, peak)
            log("gemv sweep done")
        except Exception as e:
            extra["gemv_sweep"] = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.empty_cache()
    if world == 1 and "topp" in legs:
        try:
            extra["topp_vs_reference"] = topp_vs_reference(dev)
            log("top-p comparison done")
        except Exception as e:
            extra["topp_vs_reference"] = {"error": f"{type(e).__name__}: {e}"}
    if world > 1 and "strong" in legs:
        strong = {}
        try:
            strong["config1"] = strong_leg("config1", dict(PRESETS["config1"]), args, dev, dist, world, rank, 10, 5)
            if 8 % world == 0:   # the 8 KV heads of config 4 over the ranks: one per GPU at N=8
                w4 = dict(PRESETS["config4_shard"], title="Llama-3-70B-class decode attention", heads=64, kv_heads=8)
                strong["config4"] = strong_leg("config4", w4, args, dev, dist, world, rank, 1, 3, prefer="heads")
        except Exception as e:
            strong["error"] = f"{type(e).__name__}: {e}"
        extra["strong"] = strong
        log("strong-scaling legs done")

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
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "ms_per_step_min": min(per),
            "ms_per_step_max": max(per), "repeats": len(per),
            "timing": f"{len(per)} timed loops of {args.steps} steps each; ms_per_step and value are the median loop",
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, w, world),
            "tokens_per_s_per_gpu": value / world, "tokens_per_s_per_layer_pass": value * args.layers,
            "avg_pruned_budget": avg_budget, "cuda_graph": cuda_graph,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
            "gpu_launches": headline_launches,
        }
        line.update(extra)
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        # Every captured graph that holds NCCL kernel nodes has been released above, before the
        # communicator goes away: a graph that still owns such nodes at teardown is what made the
        # exit stall.  Order: synchronize -> graphs released -> barrier -> destroy the group.
        # The result is out; should the teardown stall all the same, leave after 30 s.
        import threading
        guard = threading.Timer(30.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()
        guard.cancel()
        log("done")


if __name__ == "__main__":
    main()
