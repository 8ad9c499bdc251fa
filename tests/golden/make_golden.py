"""Generate the golden vectors under tests/golden/ from the reference's own implementation.

Run once, in a container that holds the reference checkout (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/reference/src

The reference classes are imported unmodified and run on the CPU on seeded synthetic inputs; only
their outputs are stored (inputs are regenerated from the seeds by ``oracle.cluster_oracle.clustered_keys``
and guarded by a checksum).  Files are small ``torch.save`` dictionaries.
"""

from __future__ import annotations

import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.cluster_oracle import clustered_keys  # noqa: E402


def snapshot(ix, *, full: bool) -> dict:
    out = {"labels": ix.labels[:, :ix.n].clone(), "n_c": ix.n_c.clone(), "count": ix.count.clone(),
           "mmax": ix.mmax.clone(), "mmin": ix.mmin.clone(), "mu_ref": ix.mu_ref.clone(), "ksum": ix.ksum.clone(),
           "rbar": ix.rbar.clone(), "cap": ix.cap.clone(), "end": ix.end, "splits": ix.splits,
           "rebuilds": ix.rebuilds, "resets": ix.resets, "vthr": ix.vthr.clone(),
           "sum_dir_norm": ix.sum_dir.norm(dim=-1)}
    if full:
        out["sum_dir"] = ix.sum_dir.clone()
        out["cent"] = ix.cent.clone()
    return out


def queries(H: int, d: int, steps: int, seed: int) -> torch.Tensor:
    return torch.randn(steps, H, d, generator=torch.Generator().manual_seed(seed))


def case_kmeans(ref) -> dict:
    """ssa.attn.clusterkv.spherical_kmeans on centred clustered keys."""
    K, _ = clustered_keys(2, 500, 128, seed=11)
    X = K - K.mean(1, keepdim=True)
    assign, cent = ref["spherical_kmeans"](X, C=16, iters=10, seed=3)
    return {"input_sum": float(K.double().sum()), "assign": assign.to(torch.int16), "cent": cent}


def case_stream(ref, *, h, G, n0, steps, C, C_init, cap_keys, split_factor, window, delta, check_every, seed, budget,
                full, probe_every, **extra) -> dict:
    """SphereIndexGPU: fit at n0, then one key per step; selection and the attention spec at probes."""
    d = 128
    K, V = clustered_keys(h, n0 + steps, d, seed=seed)
    Q = queries(h * G, d, steps + 1, seed + 1000)
    opts = {"partition": "kmeans", **extra}
    ix = ref["SphereIndexGPU"](C=C, C_init=C_init, cap_keys=cap_keys, split_factor=split_factor, window=window,
                               delta=delta, capacity=n0 + steps, check_every=check_every, seed=0,
                               kmeans_iters=10, **opts)
    ix.observe(K, n0)
    gold = {"input_sum": float(K.double().sum()), "cfg": dict(h=h, G=G, n0=n0, steps=steps, C=C, C_init=C_init,
            cap_keys=cap_keys, split_factor=split_factor, window=window, delta=delta, check_every=check_every,
            seed=seed, budget=budget, **extra), "fit": snapshot(ix, full=full), "probes": {}}
    for t in range(steps + 1):
        n = n0 + t
        if t:
            ix.observe(K, n)
        if t % probe_every == 0 or t == steps:
            labels, w = ix.labels_and_weights(Q[t], n=n, budget=budget, group="sum_share")
            out = ref["label_weighted_attention"](Q[t].double(), K[:, :n].double(), V[:, :n].double(), labels, w.double())
            gold["probes"][t] = {"w": w.to(torch.uint8), "out": out.float(), "n_c": ix.n_c.clone(),
                                 "splits": ix.splits, "rebuilds": ix.rebuilds}
            lab_ph, w_ph = ix.labels_and_weights(Q[t], n=n, budget=budget, group="per_head")
            gold["probes"][t]["w_per_head"] = w_ph.to(torch.uint8)
            gold["probes"][t]["out_per_head"] = ref["label_weighted_attention"](
                Q[t].double(), K[:, :n].double(), V[:, :n].double(), lab_ph, w_ph.double()).float()
            for grp in ("max", "max_rel"):                  # the other shared ways of ranking clusters
                gold["probes"][t]["w_" + grp] = ix.labels_and_weights(Q[t], n=n, budget=budget, group=grp)[1].to(torch.uint8)
    gold["final"] = snapshot(ix, full=full)
    return gold


def case_accounting(ref) -> dict:
    """ssa.attn.accounting at the worked sizes."""
    rows = []
    for n, r, c, bits in ((32768, 6640, 1140, 8), (32768, 1700, 1140, 8), (8192, 1700, 290, 32), (4096, 900, 256, 8)):
        rows.append((n, r, c, bits, float(ref["overhead_rows"](n=n, rows=r, clusters=c, d=128, summary_bits=bits)),
                     float(ref["kv_read_fraction"](n=n, rows=r, clusters=c, d=128, summary_bits=bits))))
    return {"rows": rows}


def case_partitions(ref) -> dict:
    """_kmeans_padded and _bisect_padded on padded member sets, incl. a lopsided one (median cut)."""
    g = torch.Generator().manual_seed(5)
    U = torch.nn.functional.normalize(torch.randn(3, 40, 128, generator=g) + 0.6, dim=-1)
    lump = torch.nn.functional.normalize(torch.randn(128, generator=g), dim=0)
    U[2, :37] = torch.nn.functional.normalize(4 * lump + 0.2 * torch.randn(37, 128, generator=g), dim=-1)
    U[2, 37:] = -lump
    valid = torch.ones(3, 40, dtype=torch.bool)
    valid[1, 33:] = False
    side = ref["_bisect_padded"](U, valid)
    part = ref["_kmeans_padded"](U, valid, torch.tensor([3, 2, 4]), 10)
    return {"input_sum": float(U.double().sum()), "side": side.to(torch.uint8), "part": part.to(torch.uint8)}


def case_sampled(ref) -> dict:
    """ssa.attn.tail_sample (proposal_from_scores, tail_sample_weights) and the label-weighted attention with the
    fractional weights they give, on the state of SphereIndexGPU after a fit and 40 inserted keys.  The per-head
    score estimates are the reference's own formula (sphere_gpu.py:426-430), evaluated here on its state."""
    h, G, d, n0, steps, C = 2, 2, 128, 600, 40, 64
    K, V = clustered_keys(h, n0 + steps, d, seed=31)
    Q = queries(h * G, d, 3, 1031)
    ix = ref["SphereIndexGPU"](C=C, C_init=16, cap_keys=24.0, split_factor=0.0, window=16, delta=math.inf,
                               capacity=n0 + steps, check_every=16, seed=0, kmeans_iters=10, partition="kmeans")
    ix.observe(K, n0)
    for t in range(1, steps + 1):
        ix.observe(K, n0 + t)
    n = n0 + steps
    gold = {"input_sum": float(K.double().sum()), "cfg": dict(h=h, G=G, n0=n0, steps=steps, C=C, S=6, alpha=0.1,
                                                              budget=0.2, seed=31), "probes": []}
    for t in range(3):
        q = Q[t]
        labels, w = ix.labels_and_weights(q, n=n, budget=0.2, group="sum_share")
        cdir = ix.sum_dir / ix.sum_dir.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        p = torch.einsum("hgd,hcd->hgc", q.view(h, G, d), cdir)
        e = torch.where(p >= 0, ix.mmax.unsqueeze(1) * p, ix.mmin.unsqueeze(1) * p)
        e = e.masked_fill((ix.count == 0).unsqueeze(1), -math.inf)
        prop = ref["proposal_from_scores"](e, ix.count, scale=1.0 / math.sqrt(d))
        w2 = w.clone()
        w2[:, :C] = ref["tail_sample_weights"](prop, ix.count, w[:, :C] > 0, S=6, alpha=0.1,
                                               generator=torch.Generator().manual_seed(100 + t))
        out = ref["label_weighted_attention"](q.double(), K[:, :n].double(), V[:, :n].double(), labels, w2.double())
        gold["probes"].append({"prop": prop.clone(), "w": w.clone(), "w2": w2.clone(), "out": out.float()})
    return gold


def main() -> None:
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SKV_REFERENCE_SRC")
    if not src:
        raise SystemExit("usage: make_golden.py /path/to/reference/src  (or set SKV_REFERENCE_SRC)")
    sys.path.insert(0, src)
    from ssa.attn.accounting import kv_read_fraction, overhead_rows
    from ssa.attn.clusterkv import spherical_kmeans
    from ssa.attn.labeled import label_weighted_attention
    from ssa.attn.sphere_gpu import SphereIndexGPU, _bisect_padded, _kmeans_padded
    from ssa.attn.tail_sample import proposal_from_scores, tail_sample_weights
    ref = dict(spherical_kmeans=spherical_kmeans, SphereIndexGPU=SphereIndexGPU, _bisect_padded=_bisect_padded,
               _kmeans_padded=_kmeans_padded, label_weighted_attention=label_weighted_attention,
               overhead_rows=overhead_rows, kv_read_fraction=kv_read_fraction,
               proposal_from_scores=proposal_from_scores, tail_sample_weights=tail_sample_weights)
    torch.manual_seed(0)
    gold = {
        "torch": torch.__version__,
        "kmeans": case_kmeans(ref),
        "partitions": case_partitions(ref),
        "accounting": case_accounting(ref),
        # small, full state stored: splitting by absolute cap, no recentring
        "small_cap": case_stream(ref, h=2, G=2, n0=700, steps=160, C=128, C_init=16, cap_keys=24.0, split_factor=0.0,
                                 window=16, delta=math.inf, check_every=16, seed=21, budget=0.25, full=True,
                                 probe_every=20),
        # small, relative cap (split_factor) and recentring on
        "small_drift": case_stream(ref, h=2, G=4, n0=500, steps=200, C=64, C_init=16, cap_keys=0.0, split_factor=2.0,
                                   window=8, delta=0.003, check_every=4, seed=22, budget=0.2, full=False,
                                   probe_every=25),
        # no splitting: every slot fitted
        "small_fixed": case_stream(ref, h=3, G=2, n0=400, steps=64, C=32, C_init=None, cap_keys=0.0, split_factor=0.0,
                                   window=64, delta=math.inf, check_every=16, seed=23, budget=0.5, full=False,
                                   probe_every=16),
        # options that bound or redirect the splitting: growing cap, spread trigger, reset of a head
        "small_grow": case_stream(ref, h=2, G=2, n0=400, steps=300, C=64, C_init=16, cap_keys=0.0, split_factor=1.5,
                                  window=8, delta=math.inf, check_every=16, seed=24, budget=0.3, full=False,
                                  probe_every=100, grow_cap=True),
        "small_var": case_stream(ref, h=2, G=2, n0=400, steps=300, C=128, C_init=16, cap_keys=0.0, split_factor=0.0,
                                 window=8, delta=math.inf, check_every=16, seed=25, budget=0.3, full=False,
                                 probe_every=100, var_factor=0.9, var_min=8),
        "small_reset": case_stream(ref, h=2, G=2, n0=400, steps=300, C=64, C_init=16, cap_keys=24.0, split_factor=0.0,
                                   window=8, delta=math.inf, check_every=16, seed=26, budget=0.3, full=False,
                                   probe_every=100, reset_at=40),
        # fixed random directions instead of fitted centroids, with recentring
        "small_random": case_stream(ref, h=2, G=2, n0=400, steps=120, C=32, C_init=None, cap_keys=0.0, split_factor=0.0,
                                    window=8, delta=0.003, check_every=4, seed=27, budget=0.3, full=False,
                                    probe_every=40, partition="random"),
    }
    torch.save(gold, os.path.join(HERE, "small.pt"))
    # the CPU-runnable benchmark configuration: 8 KV heads, 16 query heads, n 4096 + 512, 256 -> cap 64
    cfg1 = case_stream(ref, h=8, G=2, n0=4096, steps=512, C=1024, C_init=256, cap_keys=64.0, split_factor=0.0,
                       window=64, delta=math.inf, check_every=16, seed=1, budget=0.2, full=False, probe_every=128)
    torch.save({"torch": torch.__version__, "config1": cfg1}, os.path.join(HERE, "config1.pt"))
    torch.save({"torch": torch.__version__, "sampled": case_sampled(ref)}, os.path.join(HERE, "sampled.pt"))
    for f in ("small.pt", "config1.pt", "sampled.pt"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
