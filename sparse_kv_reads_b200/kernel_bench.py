"""Kernel-only sweep of one layer's decode step: ``python -m sparse_kv_reads_b200.kernel_bench``.

For each (heads, context, budget) it builds a synthetic bf16 cache of clustered keys on the GPU, fits the
clusters (256 per head, cap 64), and times the step's launches - score + pick, attention straight from the
labels, and the insert - as CUDA-graph replays with a 512 MB L2 flush before each, median of ``--reps``.
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


def graph_time(fn, flush, reps: int) -> float:
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
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) * 1e-3)
    out.sort()
    return out[len(out) // 2]


def run_case(heads: int, n: int, budget: float, G: int, reps: int, peak: float, device) -> dict:
    slots = 2048 if n <= 32768 else 8192
    cap = -(-(n + 80) // 16) * 16
    K, V = synthetic_cache(heads, cap, seed=heads + n, device=device)
    ix = SphereIndexGraph(budget=budget, C=slots, C_init=256, cap_keys=64.0, window=64, capacity=cap, summary_bits=8)
    ix.prepare(K, n, heads * G)
    release_workspaces()
    q = torch.randn(heads * G, 128, device=device).to(torch.bfloat16)
    n_dev = torch.tensor([n], dtype=torch.int32, device=device)
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=device)
    t_sel = graph_time(lambda: ix._select(q, n_dev, listed=False), flush, reps)
    t_att = graph_time(lambda: ix._attend_labels(q, K, V, n_dev), flush, reps)
    t_step = graph_time(lambda: (ix._select(q, n_dev, listed=False), ix._attend_labels(q, K, V, n_dev)), flush, reps)
    rows = ix.cnt.float()
    n_c = ix.n_c.float()
    nbytes = float(step_bytes(n=n, rows=rows, clusters=n_c, d=128, summary_bits=8).sum())
    att_bytes = float((rows * 512).sum()) + heads * 2.0 * n
    # the insert advances the state, so it is timed last, one real step
    n_dev.fill_(n + 1)
    t_ins = graph_time(lambda: ix._launch_insert(K, n_dev, budget), flush, 3)
    return {"heads": heads, "G": G, "n": n, "budget": budget, "slots": slots, "rows_per_head": float(rows.mean()),
            "clusters_per_head": float(n_c.mean()), "select_us": t_sel * 1e6, "attend_us": t_att * 1e6,
            "step_us": t_step * 1e6, "insert_us": t_ins * 1e6, "step_bytes": nbytes,
            "step_gbs": nbytes / t_step / 1e9, "step_frac_of_peak": nbytes / t_step / 1e9 / peak,
            "attend_gbs": att_bytes / t_att / 1e9, "attend_frac_of_peak": att_bytes / t_att / 1e9 / peak,
            "device_status": ix.check_status()}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, nargs="+", default=[8, 64, 256])
    ap.add_argument("--contexts", type=int, nargs="+", default=[8192, 32768])
    ap.add_argument("--budgets", type=float, nargs="+", default=[0.05, 0.2])
    ap.add_argument("--group", type=int, default=4)
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
    for heads in args.heads:
        for n in args.contexts:
            for b in args.budgets:
                r = run_case(heads, n, b, args.group, args.reps, peak, device)
                rows.append(r)
                print(json.dumps(r), flush=True)
                torch.cuda.empty_cache()
    if args.out:
        with open(args.out, "w") as fh:
            json.dump({"stamp": stamp(), "peak_gbs": peak, "rows": rows}, fh, indent=1)


if __name__ == "__main__":
    main()
