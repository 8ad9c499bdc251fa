"""Kernel-only sweep of one layer's decode step: ``python -m sparse_kv_reads_b200.kernel_bench``.

For each (heads, context, budget) it builds a synthetic bf16 cache of clustered keys on the GPU, fits the
clusters (256 per head, cap 64), and times the step's launches - score + pick, attention straight from the
labels, the layer step as the decoder runs it (one launch for few heads) and the insert - as CUDA-graph replays
with a 512 MB L2 flush before each, median of ``--reps``.  Default grid: contexts 8k-128k x budgets 5/10/20/40 %
x 8/64/256 heads x 2 and 4 query heads per KV head; one fit per (heads, context) serves all its points.
Bandwidth is quoted on the reference's accounting of the bytes a step reads (``accounting.step_bytes``).
Counterpart of the reference's per-layer benchmark (ssa/harness/kernel_bench.py:27-49, 74-76).
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch

from .accounting import step_bytes
from .cluster_state import SphereIndexGraph, release_workspaces
from .stamp import stamp


def synthetic_cache(heads: int, n: int, *, seed: int, device, centres: int = 64):
    """Keys = 3 x one of 64 unit directions + N(0, 0.5^2) + a shared offset of norm 2, values N(0, 1); bf16."""
    g = torch.Generator(device=device).manual_seed(seed)
    ctr = torch.nn.functional.normalize(torch.randn(centres, 128, generator=g, device=device), dim=-1)
    off = 2 * torch.nn.functional.normalize(torch.randn(128, generator=g, device=device), dim=-1)
    K = torch.empty(heads, n, 128, dtype=torch.bfloat16, device=device)
    V = torch.empty(heads, n, 128, dtype=torch.bfloat16, device=device)
    for h0 in range(0, heads, 16):
        hs = min(16, heads - h0)
        pick = torch.randint(0, centres, (hs, n), generator=g, device=device)
        K[h0:h0 + hs] = (3 * ctr[pick] + 0.5 * torch.randn(hs, n, 128, generator=g, device=device) + off).to(torch.bfloat16)
        V[h0:h0 + hs] = torch.randn(hs, n, 128, generator=g, device=device).to(torch.bfloat16)
    return K, V


def graph_time(fn, flush, reps: int, before=None) -> float:
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    out = []
    for _ in range(reps):
        flush.zero_()
        if before is not None:
            before()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) * 1e-3)
    out.sort()
    return out[len(out) // 2]


def fitted_index(heads: int, n: int, device):
    """Synthetic cache of ``heads`` heads x ``n`` tokens and its fitted cluster state (256 clusters per head,
    cap 64; 2,048 slots up to 32k tokens, 8,192 beyond)."""
    slots = 2048 if n <= 32768 else 8192
    cap = -(-(n + 80) // 16) * 16
    K, V = synthetic_cache(heads, cap, seed=heads + n, device=device)
    ix = SphereIndexGraph(budget=0.2, C=slots, C_init=256, cap_keys=64.0, window=64, capacity=cap, summary_bits=8)
    ix.observe(K, n)
    release_workspaces()
    return ix, K, V, slots


def time_case(ix, K, V, n: int, budget: float, G: int, reps: int, peak: float, flush) -> dict:
    """One (budget, group size) point on a fitted state: the selection launch, the attention launch, and the
    layer step as the decoder runs it (``SphereIndexGraph.step``: one launch where ``skv_step`` serves the
    shape, else those two)."""
    heads, device = ix.H_kv, K.device
    ix.budget = budget
    ix.need_dev.fill_(math.ceil(budget * (ix.end - 1)))
    q = torch.randn(heads * G, 128, device=device).to(torch.bfloat16)
    n_dev = torch.tensor([n], dtype=torch.int32, device=device)
    ix._select(q, n_dev, listed=False)                      # sizes the buffers of this group size outside any capture
    ix._attend_labels(q, K, V, n_dev)
    one_launch = bool(ix._step_clusters(G))
    ix.step(q, K, V, n_dev, insert=False)
    t_sel = graph_time(lambda: ix._select(q, n_dev, listed=False), flush, reps)
    t_att = graph_time(lambda: ix._attend_labels(q, K, V, n_dev), flush, reps)
    t_step = graph_time(lambda: ix.step(q, K, V, n_dev, insert=False), flush, reps)
    rows = ix.cnt.float()
    n_c = ix.n_c.float()
    nbytes = float(step_bytes(n=n, rows=rows, clusters=n_c, d=128, summary_bits=8).sum())
    att_bytes = float((rows * 512).sum()) + heads * 2.0 * n
    return {"heads": heads, "G": G, "n": n, "budget": budget, "slots": ix.C, "rows_per_head": float(rows.mean()),
            "clusters_per_head": float(n_c.mean()), "select_us": t_sel * 1e6, "attend_us": t_att * 1e6,
            "step_us": t_step * 1e6, "step_launches": 1 if one_launch else 2, "step_bytes": nbytes,
            "step_gbs": nbytes / t_step / 1e9, "step_frac_of_peak": nbytes / t_step / 1e9 / peak,
            "attend_gbs": att_bytes / t_att / 1e9, "attend_frac_of_peak": att_bytes / t_att / 1e9 / peak,
            "device_status": ix.check_status()}


def run_case(heads: int, n: int, budget: float, G: int, reps: int, peak: float, device) -> dict:
    """Build, fit and time one point (the benchmark's batch-32 leg uses this)."""
    ix, K, V, _ = fitted_index(heads, n, device)
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=device)
    return time_case(ix, K, V, n, budget, G, reps, peak, flush)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, nargs="+", default=[8, 64, 256])
    ap.add_argument("--contexts", type=int, nargs="+", default=[8192, 16384, 32768, 65536, 131072])
    ap.add_argument("--budgets", type=float, nargs="+", default=[0.05, 0.1, 0.2, 0.4])
    ap.add_argument("--groups", type=int, nargs="+", default=[2, 4], help="query heads per KV head")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    device = torch.device("cuda", 0)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peak = 6650.0
    pk = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["hbm_gbs"])
    rows = []
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=device)
    for heads in args.heads:
        for n in args.contexts:
            ix, K, V, _ = fitted_index(heads, n, device)    # one fit serves every budget and group size
            for G in args.groups:
                for b in args.budgets:
                    r = time_case(ix, K, V, n, b, G, args.reps, peak, flush)
                    rows.append(r)
                    print(json.dumps(r), flush=True)
            # the insert advances the state, so it is timed last: the length grows by one ahead of every replay, so
            # that each timed launch inserts one key per head (the cache holds 80 positions beyond n)
            n_dev = torch.tensor([n + 1], dtype=torch.int32, device=device)
            t_ins = graph_time(lambda: ix._launch_insert(K, n_dev, ix.budget), flush, 9, before=lambda: n_dev.add_(1))
            print(json.dumps({"heads": heads, "n": n, "insert_us": t_ins * 1e6}), flush=True)
            rows.append({"heads": heads, "n": n, "insert_us": t_ins * 1e6})
            del ix, K, V
            torch.cuda.empty_cache()
    if args.out:
        with open(args.out, "w") as fh:
            json.dump({"stamp": stamp(), "peak_gbs": peak, "rows": rows}, fh, indent=1)


if __name__ == "__main__":
    main()
