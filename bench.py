"""Benchmark of the clustered sparse decode-attention path inside a Qwen3 CUDA-graph decode loop.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one decode step of the whole model (every layer's insert / select / attend inside one CUDA
graph).  Default workload: Qwen3-0.6B architecture, random weights, bf16, batch 1, a 32,768-token random
prompt, 20 % budget, 256 clusters per KV head fitted at the prompt, cap 64.  Prints one JSON line.
With N > 1 (launched through torch.distributed.run) the KV heads, MLP columns and vocabulary are
sharded over the ranks; the attention needs no communication.  The sums after the row-parallel o_proj / down
products travel through peer memory inside the products themselves for up to 8 sequences (NCCL all-reduces
beyond that); NCCL gathers the vocabulary-parallel logits.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: (model, batch, prompt, budget, slots)
    "qwen3-0.6b_b1_32k_budget20": ("0.6b", 1, 32768, 0.20, 2048),
    "qwen3-0.6b_b8_8k_budget5": ("0.6b", 8, 8192, 0.05, 1024),
    "qwen3-4b_b1_32k_budget20": ("4b", 1, 32768, 0.20, 2048),
    "qwen3-4b_b4_8k_budget10": ("4b", 4, 8192, 0.10, 1024),
    "qwen3-0.6b_b1_4k_budget20": ("0.6b", 1, 4096, 0.20, 1024),          # quick check
    # the scaling configuration: the batch is fixed (strong scaling over the KV heads); on one GPU the cache of 32
    # sequences does not fit (155 GB of keys and values + 27 GB of cluster state + weights), so N = 1 runs 16
    "qwen3-4b_b32_32k_budget20": ("4b", 32, 32768, 0.20, 2048),
    "qwen3-4b_b32_32k_budget5": ("4b", 32, 32768, 0.05, 2048),
    # long generation: an 8,192-token prompt continued to 32,768 tokens, clusters growing with the context
    "qwen3-4b_b1_8k_to_32k_budget20": ("4b", 1, 8192, 0.20, 2048),
    "qwen3-0.6b_b1_8k_to_32k_budget20": ("0.6b", 1, 8192, 0.20, 2048),
}
FIXED_BATCH = {"qwen3-4b_b32_32k_budget20": {1: 16}, "qwen3-4b_b32_32k_budget5": {1: 16}}   # batch at N GPUs, else as named
LONG_GENERATION = {"qwen3-4b_b1_8k_to_32k_budget20": 32768, "qwen3-0.6b_b1_8k_to_32k_budget20": 32768}
DEFAULT = "qwen3-0.6b_b1_32k_budget20"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the workload's dominant kernel, from an ncu capture
# of that workload (a constant copied from the capture's summary; workloads without a capture report null)
NCU_TRAFFIC = {"qwen3-0.6b_b1_32k_budget20": 29.03e6}


def peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        if self.index is None or self.proc is not None:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def wait_first(self, seconds: float) -> None:
        """Give the sampler up to ``seconds`` to deliver its first row."""
        t0 = time.time()
        while self.proc is not None and not self.rows and time.time() - t0 < seconds:
            time.sleep(0.02)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's attention path on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_attention_path(n: int, budget: float, slots: int, layers: int, steps: int, warmup: int, h: int = 8, G: int = 2):
    """Time the CPU oracle (restatement of the reference's PyTorch path) on ONE layer of ``h`` KV heads at
    context ``n``: prompt fit once, then ``warmup + steps`` decode steps of insert + select + attention over
    the selected rows.  Returns (seconds per layer-step, fit seconds, cores)."""
    from oracle import cluster_oracle as oc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    total = warmup + steps
    K, V = oc.clustered_keys(h, n + total, 128, seed=1)
    K, V = K.to(torch.bfloat16), V.to(torch.bfloat16)
    Q = torch.randn(total + 1, h * G, 128, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    st = oc.ClusterOracle(C=slots, C_init=256, cap_keys=64.0, window=64, delta=0.03, capacity=n + total + 8)
    t0 = time.perf_counter()
    st.observe(K, n)
    fit_s = time.perf_counter() - t0
    times = []
    for t in range(1, total + 1):
        t0 = time.perf_counter()
        st.observe(K, n + t)
        labels, w = st.select(Q[t].float(), n=n + t, budget=budget)
        oc.attend_rows(Q[t], K, V, st.positions(w, n + t), dtype=torch.float32)
        times.append(time.perf_counter() - t0)
    timed = times[warmup:]
    return sum(timed) / len(timed), fit_s, cores


def reference_arm(args, wl) -> None:
    """``--impl reference``: the reference's algorithm for this path on the host CPU (its Python
    implementation cannot travel to the GPU box; the oracle is its pinned restatement)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model, B, n, budget, slots = wl
    if args.workload in FIXED_BATCH:
        B = FIXED_BATCH[args.workload].get(max(1, args.gpus), B)
    else:
        B *= max(1, args.gpus)                           # the GPU arm serves one more sequence per GPU
    layers = 28 if model == "0.6b" else 36
    G = 2 if model == "0.6b" else 4
    steps, warmup = max(1, min(args.steps, 8)), max(1, min(args.warmup, 2))
    per_layer, fit_s, cores = cpu_attention_path(min(n, 32768), budget, slots, layers, steps, warmup, h=8, G=G)
    ms = per_layer * layers * B * 1e3
    value = B / (per_layer * layers * B)
    sample = (f"oracle attention path only (insert+select+attend), 1 layer x 8 KV heads at n={min(n, 32768)}, "
              f"{steps} timed steps, scaled x{layers} layers x batch {B}; dense layers excluded; fit {fit_s:.2f}s")
    line = {"impl": "reference", "metric": "qwen3_decode_tokens_per_s", "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(args.workload, B), "batch": B, "prompt": n, "budget": budget},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def build_decoder(wl, dev, tp_group, tp_size, tp_rank, decode_steps, synthetic_cache=False):
    from sparse_kv_reads_b200 import GraphDecoder, Qwen3Config, Qwen3Model
    model_name, B, n, budget, slots = wl
    cfg = Qwen3Config.qwen3_0_6b() if model_name == "0.6b" else Qwen3Config.qwen3_4b()
    with torch.device(dev):
        model = Qwen3Model(cfg, tp_group=tp_group, tp_size=tp_size, tp_rank=tp_rank)
    model = model.to(torch.bfloat16).eval()
    model.init_random(seed=0)
    cap = -(-(n + decode_steps + 8) // 16) * 16
    cache = model.alloc_cache(cap, max_batch=B)
    ids = torch.randint(0, cfg.vocab_size, (B, n + decode_steps + 1), generator=torch.Generator().manual_seed(1))
    if synthetic_cache:
        # the prompt's keys and values are drawn directly (clustered keys of the CPU-runnable configuration, a new
        # draw per layer) instead of being computed by a prefill: the decode step costs the same, the set-up far less
        from sparse_kv_reads_b200.kernel_bench import synthetic_cache as draw
        for i in range(len(cache.k)):
            K, V = draw(B * cache.k[i].shape[1], cap, seed=1000 * tp_rank + i, device=dev)
            cache.k[i].copy_(K.view_as(cache.k[i]))
            cache.v[i].copy_(V.view_as(cache.v[i]))
            del K, V
        cache.cur_len = n
    else:
        with torch.no_grad():
            model.prefill(ids[:, :n].to(dev), cache, chunk=2048)
    dec = GraphDecoder(model, cache, mode="cluster", budget=budget, C=slots, C_init=256, cap_keys=64.0, window=64,
                       summary_bits=8)
    t0 = time.perf_counter()
    dec.prepare(n)
    torch.cuda.synchronize()
    fit_s = time.perf_counter() - t0
    dec.capture()
    return model, cache, dec, ids, fit_s


def kernel_roofline(dec, n_now, peak_gbs, which, traffic=None):
    """Per-launch duration of the layer's attention-side kernels measured with CUDA events, one launch per
    layer back to back in a CUDA graph (each layer's rows are cold: the layers' caches together are far larger
    than L2, and 512 MB are written before each replay).  The layer step is timed as the decoder runs it
    (``SphereIndexGraph.step``): ONE launch (selection + attention by thread-block clusters) for few heads,
    else the selection launch followed by the attention launch.  Bytes: for the dominant kernel what that
    kernel has to read (K and V rows, the int16 label of every cached position, and - when it also selects -
    the cluster summaries); for the layer step the full accounting formula."""
    from sparse_kv_reads_b200.accounting import step_bytes
    B, H, H_kv, d = dec.B, dec.H, dec.H_kv, dec.d
    dev = dec.tok.device
    layers = dec.attn
    q = torch.randn(B * H, d, device=dev).to(torch.bfloat16)
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)
    heads = [(dec._heads(dec.cache.k[i]), dec._heads(dec.cache.v[i])) for i in range(len(layers))]

    def graph_of(fn):
        """One launch of ``fn`` per layer, back to back in a CUDA graph (no host gaps between launches)."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for ix, kv in zip(layers, heads):
                fn(ix, kv)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for ix, kv in zip(layers, heads):
                fn(ix, kv)
        return g

    def timed(g, reps=7):
        out = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        out.sort()
        return out[len(out) // 2] * 1e-3 / len(layers)

    one_launch = bool(layers[0]._step_clusters(H // H_kv))
    sel_t = timed(graph_of(lambda ix, kv: ix._select(q, dec.n_dev, listed=False)))
    att_t = timed(graph_of(lambda ix, kv: ix._attend_labels(q, kv[0], kv[1], dec.n_dev)))
    # the step as the decoder launches it: with its own products the last merge of the one-launch step rides in the
    # output product
    defer = one_launch and dec.merge_deferred
    stp_t = timed(graph_of(lambda ix, kv: ix.step(q, kv[0], kv[1], dec.n_dev, insert=False, defer_merge=defer)))
    for ix, kv in zip(layers, heads):                                  # one untimed step that writes the rows read
        ix.step(q, kv[0], kv[1], dec.n_dev, insert=False)
    torch.cuda.synchronize()
    rows = torch.stack([ix.cnt for ix in layers]).float()              # [layers, heads]
    n_c = torch.stack([ix.n_c for ix in layers]).float()
    # attention kernel: K and V rows, the int16 label of every cached position, the selection bits
    att_bytes = float((rows * 2 * 256).sum(1).mean()) + rows.shape[1] * (2 * n_now + 4 * (layers[0].C // 32 + 1))
    # one-launch step: the same rows and labels plus every cluster's summary (128-byte direction, lengths, count)
    one_bytes = float((rows * 2 * 256 + n_c * (128 + 12)).sum(1).mean()) + rows.shape[1] * 2 * n_now
    stp_bytes = float(step_bytes(n=n_now, rows=rows, clusters=n_c, d=d, summary_bits=8).sum(1).mean())
    kernel, k_bytes, k_t = ("step_kernel", one_bytes, stp_t) if one_launch else ("attend_labels_kernel", att_bytes, att_t)
    roof = {"bound": "hbm", "kernel": kernel, "achieved": k_bytes / k_t / 1e9, "peak": peak_gbs,
            "unit": "GB/s", "frac": k_bytes / k_t / 1e9 / peak_gbs, "traffic": traffic,
            "traffic_source": "constant from the committed ncu capture of this workload, not measured in this run",
            "peak_source": which, "us_per_launch": k_t * 1e6, "bytes_per_launch": k_bytes}
    layer = {"kernels": ("select + attend in one launch" if one_launch else "select, then attend") +
                        " (insert runs once for all layers)",
             "launches": 1 if one_launch else 2, "us_per_layer": stp_t * 1e6,
             "last_merge": "in the output product, as in the decode step" if defer else "in the launch",
             "bytes_per_layer": stp_bytes, "achieved": stp_bytes / stp_t / 1e9, "unit": "GB/s",
             "frac": stp_bytes / stp_t / 1e9 / peak_gbs, "select_us": sel_t * 1e6, "attend_us": att_t * 1e6,
             "rows_per_head": float(rows.mean()),
             "clusters_per_head": float(n_c.mean())}
    del flush
    return roof, layer


def batch32_roofline(G, peak_gbs, which, dev):
    """The layer step at 256 (sequence, KV head) pairs - batch 32 - of 32,768 tokens at 20 %: one layer of
    synthetic clustered keys (4.3 GB of cache), where the step is a stream rather than a chain of latencies."""
    from sparse_kv_reads_b200.kernel_bench import run_case
    r = run_case(256, 32768, 0.2, G, 10, peak_gbs, dev)
    return {"heads": 256, "context": 32768, "budget": 0.2, "G": G, "us_select": r["select_us"],
            "us_attend": r["attend_us"], "us_step": r["step_us"], "bytes": r["step_bytes"],
            "achieved": r["step_gbs"], "unit": "GB/s", "peak": peak_gbs, "peak_source": which,
            "frac": r["step_frac_of_peak"], "attend_frac": r["attend_frac_of_peak"],
            "rows_per_head": r["rows_per_head"], "clusters_per_head": r["clusters_per_head"]}


def exact_leg(model, cache, ids_dev, pos, steps, warmup):
    """The reference publishes exact attention beside every sparse number (ssa/harness/decode_speed.py:128-137):
    the same model and cache decoded with exact attention over every cached row (the gather kernel in its dense
    mode), same graph loop, device-resident ids.  Returns (tokens/s, ms per step, next position)."""
    from sparse_kv_reads_b200 import GraphDecoder
    dec = GraphDecoder(model, cache, mode="dense")
    cache.cur_len = pos
    dec.capture()
    for _ in range(warmup):
        dec.step(ids_dev[:, pos:pos + 1], pos)
        pos += 1
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        dec.step(ids_dev[:, pos:pos + 1], pos)
        pos += 1
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    return ids_dev.shape[0] / (ms * 1e-3), ms, pos


def workload_name(name: str, batch: int) -> str:
    """The workload's name with the batch actually run (the scaling runs change it with the GPU count)."""
    import re
    return re.sub(r"_b\d+_", f"_b{batch}_", name, count=1)


def own_launches(dec) -> int:
    """Launches of this library's kernels in one decode step: the all-layer insert, then per layer the
    selection and the attention, and with the bundled model's fused layers also QK-norm/rotary/cache write and
    either the four matrix-vector products (norms and activation folded in) or the three element-wise kernels
    around cuBLAS products; one more norm ahead of the vocabulary projection."""
    counted = getattr(dec, "launches_per_step", 0)      # counted while the step was captured
    if counted:
        return counted
    per_layer = 2
    extra = 1
    if dec.fused_dense:
        per_layer += 1 + (4 if dec.own_gemv and dec.B <= 8 else 3)
        extra += 1
    return extra + per_layer * len(dec.attn)


def long_generation(args, wl) -> None:
    """An 8,192-token prompt continued to 32,768 tokens (one GPU): every step inserts a key, clusters split at the
    cap and the state recentres between replays, so the cluster count grows with the context.  Counterpart of the
    reference's long generation (docs/results.md:67-69: ms per step and clusters at the end).  Prints one JSON line:
    whole-run throughput, and per window of 2,048 steps the ms per step and the clusters per head."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    model_name, B, n, budget, slots = wl
    target = LONG_GENERATION[args.workload]
    steps = target - n
    model, cache, dec, ids, fit_s = build_decoder(wl, dev, None, 1, 0, steps + 8)
    ids_dev = ids.to(dev)
    clocks = ClockSampler(0)
    windows, pos = [], n
    start_clusters = float(torch.stack([a.n_c.float().mean() for a in dec.attn]).mean())
    t_all0 = torch.cuda.Event(enable_timing=True)
    with clocks:
        for _ in range(8):                                # warm-up steps (they advance the context too)
            dec.step(ids_dev[:, pos:pos + 1], pos)
            pos += 1
        torch.cuda.synchronize()
        t_all0.record()
        while pos < target:
            w = min(2048, target - pos)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(w):
                dec.step(ids_dev[:, pos:pos + 1], pos)
                pos += 1
            b.record()
            torch.cuda.synchronize()
            windows.append({"context": pos, "ms_per_step": a.elapsed_time(b) / w,
                            "clusters_per_head": float(torch.stack([x.n_c.float().mean() for x in dec.attn]).mean())})
        t_all1 = torch.cuda.Event(enable_timing=True)
        t_all1.record()
        torch.cuda.synchronize()
    total_ms = t_all0.elapsed_time(t_all1)
    done = target - n - 8
    status = 0
    for ix in dec.attn:
        status |= ix.check_status()
    line = {"metric": "qwen3_decode_tokens_per_s", "value": B * done / (total_ms * 1e-3), "unit": "tok/s", "n_gpus": 1,
            "steps": done, "warmup": 8, "ms_per_step": total_ms / done, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "model": f"qwen3-{model_name} architecture, random weights", "batch": B,
                       "prompt": n, "generated_to": target, "budget": budget, "slots": slots, "clusters_fitted": 256,
                       "cap_keys": 64, "window": 64, "summary_bits": 8,
                       "timing": "device time of the whole generation, host recentring between replays included"},
            "gpu_launches": done * own_launches(dec), "clocks": clocks.summary(),
            "long_generation": {"windows": windows, "clusters_per_head_start": start_clusters,
                                "clusters_per_head_end": windows[-1]["clusters_per_head"],
                                "splits": sum(ix.splits for ix in dec.attn),
                                "recentrings": sum(ix.rebuilds for ix in dec.attn),
                                "largest_cluster": float(max(float(ix.count.max()) for ix in dec.attn))},
            "prompt_fit_s": fit_s, "device_status": status}
    print(json.dumps(line), flush=True)


def gpu_arm(args, wl) -> None:
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    model_name, B, n, budget, slots = wl
    # Weak scaling over the path's independent units, the (sequence, KV head) pairs: every GPU added brings one
    # more sequence while it takes over its share of the 8 KV heads, so a GPU always serves 8 pairs per layer.
    fixed = args.workload in FIXED_BATCH
    if fixed:
        B = FIXED_BATCH[args.workload].get(world, B)     # strong scaling: the batch the workload names, split by KV head
    else:
        B = B * world
    wl = (model_name, B, n, budget, slots)
    K_steps, W = args.steps, args.warmup
    total = 3 * (K_steps + W) + 4                        # device leg, end-to-end leg, exact-attention leg
    model, cache, dec, ids, fit_s = build_decoder(wl, dev, group, world, rank, total, args.synthetic_cache)
    ids_dev = ids.to(dev)
    pinned = ids.pin_memory()
    result_host = torch.zeros(B, dtype=torch.long).pin_memory()
    pos = n

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident leg: token ids already in HBM ------------------------------------------
    # the clock sampler starts ahead of the warm-up steps (nvidia-smi needs a moment, longer on a box with many
    # GPUs) and keeps sampling through the timed steps; the warm-up runs the same kernels, so every row is
    # taken under the same load
    clocks = ClockSampler(local if rank == 0 else None)
    clocks.__enter__()
    for _ in range(W):
        dec.step(ids_dev[:, pos:pos + 1], pos)
        pos += 1
    clocks.wait_first(3.0)                               # rank 0 only; the barrier below lines the ranks up again
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clocks:
        if args.ncu_range:
            torch.cuda.profiler.start()
        start.record()
        for _ in range(K_steps):
            dec.step(ids_dev[:, pos:pos + 1], pos)
            pos += 1
        stop.record()
        barrier()
        if args.ncu_range:
            torch.cuda.profiler.stop()
    dev_ms = start.elapsed_time(stop)
    # ---- end-to-end leg: ids from pinned host memory, next-token ids read back every step ----------
    for _ in range(W):
        logits = dec.step(pinned[:, pos:pos + 1], pos)          # 8 B per sequence, pinned host -> the step's buffer
        result_host.copy_(logits[:, -1].argmax(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pos += 1
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K_steps):
        logits = dec.step(pinned[:, pos:pos + 1], pos)          # 8 B per sequence, pinned host -> the step's buffer
        result_host.copy_(logits[:, -1].argmax(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pos += 1
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    status = 0
    for ix in dec.attn:
        status |= ix.check_status()
    if getattr(dec, "_peer", None) is not None:          # a wait for another GPU's partial sums that gave up
        status |= dec._peer.status()
    if rank == 0:
        peak, which = peaks()
        roof, layer = kernel_roofline(dec, pos, peak, which, NCU_TRAFFIC.get(args.workload) if world == 1 else None)
        line = {"metric": "qwen3_decode_tokens_per_s", "value": B * K_steps / (dev_ms * 1e-3), "unit": "tok/s",
                "n_gpus": world, "steps": K_steps, "warmup": W, "ms_per_step": dev_ms / K_steps,
                "higher_is_better": True, "scaling": "strong" if fixed else "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic" + (" (keys and values of the prompt drawn directly, no prefill)" if args.synthetic_cache
                                       else ""),
                "config": {"workload": workload_name(args.workload, B), "model": f"qwen3-{model_name} architecture, random weights",
                           "batch": B, "prompt": n, "budget": budget, "slots": slots, "clusters_fitted": 256,
                           "cap_keys": 64, "window": 64, "summary_bits": 8,
                           "parallelism": (f"tp{world}: KV heads sharded, batch {B} ({B * 8 // world} sequence-head pairs "
                                           f"per GPU), sums through " +
                                           ("peer memory" if B <= 8 else "NCCL all-reduces")) if world > 1
                           else "single GPU",
                           "l2": "per-layer caches total far more than L2; the kernel leg also flushes 512 MB"},
                "e2e": {"value": B * K_steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8 * B,
                        "d2h_bytes_per_step": 8 * B, "ms_per_step": e2e_ms / K_steps},
                "gpu_launches": K_steps * own_launches(dec),
                "clocks": clocks.summary(), "roofline": roof, "layer_step": layer,
                "prompt_fit_s": fit_s, "device_status": status,
                "splits": sum(ix.splits for ix in dec.attn)}
        if world == 1 and not args.no_extra:
            xs, xw = min(K_steps, 32), min(W, 4)
            tok_s, ms, _ = exact_leg(model, cache, ids_dev, pos, xs, xw)
            line["exact"] = {"value": tok_s, "unit": "tok/s", "ms_per_step": ms, "steps": xs,
                             "what": "same model and cache, exact attention over every cached row (dense mode of "
                                     "the gather kernel), device-resident ids"}
            line["roofline_b32"] = batch32_roofline(dec.H // dec.H_kv, peak, which, dev)
        if world == 1 and not args.no_cpu:
            per_layer, cfit, cores = cpu_attention_path(min(n, 32768), budget, slots, len(dec.attn), 4, 1,
                                                        h=8, G=dec.H // dec.H_kv)
            line["cpu_baseline"] = {"value": 1.0 / (per_layer * len(dec.attn) * B), "unit": "tok/s", "cores": cores,
                                    "kind": "port",
                                    "sample": f"oracle attention path only, 1 layer x 8 KV heads at n={min(n, 32768)}, 4 "
                                              f"timed steps, scaled x{len(dec.attn)} layers x batch {B}; dense layers "
                                              f"excluded; CPU fit {cfit:.2f}s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        # Orderly teardown: the captured graph (it holds NCCL kernels) goes first, then the exchange buffers, then
        # the communicator.  Destroying the communicator while the graph object is alive blocked in earlier builds;
        # in this order it returns (2 GPUs, measured).  A watchdog leaves the process after 20 s regardless, so a
        # teardown that blocks on some other pool cannot hold a finished measurement hostage.
        import gc
        watchdog = threading.Timer(20.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        peer = getattr(dec, "_peer", None)
        dec.graph = None
        del dec
        gc.collect()
        torch.cuda.synchronize()
        if peer is not None:
            dist.barrier()
            peer.close()
        dist.destroy_process_group()
        watchdog.cancel()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--synthetic-cache", action="store_true",
                    help="draw the prompt's keys and values directly instead of running a prefill (large workloads)")
    ap.add_argument("--no-extra", action="store_true", help="skip the exact-attention and batch-32 legs (profiling runs)")
    ap.add_argument("--ncu-range", action="store_true",
                    help="bracket the timed device leg with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        reference_arm(args, wl)
    elif args.workload in LONG_GENERATION:
        long_generation(args, wl)
    else:
        gpu_arm(args, wl)


if __name__ == "__main__":
    main()
