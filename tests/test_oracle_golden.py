"""The CPU oracle against the golden vectors produced by the reference's own classes (CPU only)."""

from __future__ import annotations

import math

import pytest
import torch

from oracle import cluster_oracle as oc


def _replay(g, *, summary_bits=32):
    """Run the oracle over a stored stream case; yields (t, state, q, K, V) at every probe."""
    c = g["cfg"]
    K, V = oc.clustered_keys(c["h"], c["n0"] + c["steps"], 128, seed=c["seed"])
    assert abs(float(K.double().sum()) - g["input_sum"]) < 1e-6, "seeded inputs differ from the stored checksum"
    Q = torch.randn(c["steps"] + 1, c["h"] * c["G"], 128, generator=torch.Generator().manual_seed(c["seed"] + 1000))
    extra = {k: c[k] for k in ("grow_cap", "reset_at", "var_factor", "var_min", "partition") if k in c}
    st = oc.ClusterOracle(C=c["C"], C_init=c["C_init"], cap_keys=c["cap_keys"], split_factor=c["split_factor"],
                          window=c["window"], delta=c["delta"], capacity=c["n0"] + c["steps"],
                          check_every=c["check_every"], seed=0, summary_bits=summary_bits, **extra)
    st.observe(K, c["n0"])
    yield -1, st, None, K, V
    for t in range(c["steps"] + 1):
        if t:
            st.observe(K, c["n0"] + t)
        if t in g["probes"]:
            yield t, st, Q[t], K, V


def _same_up_to_ties(mine, ref, score):
    """Equal selections, except among clusters that share the score at the cut: the reference ranks with an
    unstable sort, so which of several exactly tied clusters it takes is not defined (``max_rel`` gives every
    query head's best cluster the score 0); here ties go to the lower slot."""
    C = score.shape[1]
    for i in range(score.shape[0]):
        diff = (mine[i, :C] != ref[i, :C]).nonzero().flatten()
        if diff.numel() == 0:
            continue
        tied = score[i, diff]
        assert bool((tied == tied[0]).all()), "selections differ beyond a tie"
        for w in (mine[i, :C], ref[i, :C]):
            assert bool(w[score[i] > tied[0]].all()) and not bool(w[score[i] < tied[0]].any())


def _same_state(st, snap):
    n = st.n
    assert torch.equal(st.labels[:, :n], snap["labels"])
    assert torch.equal(st.n_c, snap["n_c"])
    assert torch.equal(st.count, snap["count"])
    torch.testing.assert_close(st.mmax, snap["mmax"], rtol=0, atol=0)
    torch.testing.assert_close(st.mmin, snap["mmin"], rtol=0, atol=0)
    torch.testing.assert_close(st.mu_ref, snap["mu_ref"], rtol=0, atol=0)
    torch.testing.assert_close(st.ksum, snap["ksum"], rtol=0, atol=0)
    torch.testing.assert_close(st.rbar, snap["rbar"], rtol=0, atol=0)
    torch.testing.assert_close(st.cap, snap["cap"], rtol=0, atol=0)
    torch.testing.assert_close(st.sum_dir.norm(dim=-1), snap["sum_dir_norm"], rtol=0, atol=0)
    assert st.end == snap["end"] and st.splits == snap["splits"] and st.rebuilds == snap["rebuilds"]
    assert st.resets == snap["resets"]
    torch.testing.assert_close(st.vthr, snap["vthr"], rtol=0, atol=0)
    if "sum_dir" in snap:
        torch.testing.assert_close(st.sum_dir, snap["sum_dir"], rtol=0, atol=0)
        torch.testing.assert_close(st.cent, snap["cent"], rtol=0, atol=0)


@pytest.mark.parametrize("case", ["small_cap", "small_drift", "small_fixed", "small_grow", "small_var", "small_reset",
                                  "small_random"])
def test_stream_cases_reproduce_the_reference_bit_for_bit(golden_small, case):
    g = golden_small[case]
    for t, st, q, K, V in _replay(g):
        if t < 0:
            _same_state(st, g["fit"])
            continue
        p = g["probes"][t]
        n = g["cfg"]["n0"] + t
        labels, w = st.select(q, n=n, budget=g["cfg"]["budget"])
        assert torch.equal(w.to(torch.uint8), p["w"])
        lab_ph, w_ph = st.select(q, n=n, budget=g["cfg"]["budget"], group="per_head")
        assert torch.equal(w_ph.to(torch.uint8), p["w_per_head"])
        torch.testing.assert_close(oc.attend_labeled(q, K[:, :n], V[:, :n], lab_ph, w_ph).float(), p["out_per_head"],
                                   rtol=0, atol=1e-6)
        for grp in ("max", "max_rel"):
            mine = st.select(q, n=n, budget=g["cfg"]["budget"], group=grp)[1].to(torch.uint8)
            _same_up_to_ties(mine, p["w_" + grp], st.shared_score(st.scores(q), grp))
        assert torch.equal(st.n_c, p["n_c"]) and st.splits == p["splits"] and st.rebuilds == p["rebuilds"]
        out = oc.attend_labeled(q, K[:, :n], V[:, :n], labels, w)
        torch.testing.assert_close(out.float(), p["out"], rtol=0, atol=1e-6)
        rows = st.positions(w, n)
        torch.testing.assert_close(oc.attend_rows(q, K, V, rows).float(), p["out"], rtol=0, atol=1e-6)
    _same_state(st, g["final"])
    if case not in ("small_fixed", "small_random"):
        assert g["final"]["splits"] > 0
    if case == "small_reset":
        assert g["final"]["resets"] > 0
    if case in ("small_drift", "small_random"):
        assert g["final"]["rebuilds"] > 0


def test_benchmark_configuration_one_reproduces_the_reference(golden_config1):
    g = golden_config1["config1"]
    for t, st, q, K, V in _replay(g):
        if t < 0:
            _same_state(st, g["fit"])
            continue
        p = g["probes"][t]
        n = g["cfg"]["n0"] + t
        labels, w = st.select(q, n=n, budget=g["cfg"]["budget"])
        assert torch.equal(w.to(torch.uint8), p["w"])
        rows = st.positions(w, n)
        torch.testing.assert_close(oc.attend_rows(q, K, V, rows).float(), p["out"], rtol=0, atol=1e-6)
    _same_state(st, g["final"])
    assert int(st.count.max()) <= 64 and g["final"]["splits"] > 0


def test_kmeans_and_partitions(golden_small):
    g = golden_small["kmeans"]
    K, _ = oc.clustered_keys(2, 500, 128, seed=11)
    assert abs(float(K.double().sum()) - g["input_sum"]) < 1e-6
    assign, cent = oc.kmeans_cosine(K - K.mean(1, keepdim=True), 16, 10, 3)
    assert torch.equal(assign.to(torch.int16), g["assign"])
    torch.testing.assert_close(cent, g["cent"], rtol=0, atol=0)
    torch.testing.assert_close(cent.norm(dim=-1), torch.ones(2, 16), rtol=1e-6, atol=1e-6)

    g = golden_small["partitions"]
    gen = torch.Generator().manual_seed(5)
    U = torch.nn.functional.normalize(torch.randn(3, 40, 128, generator=gen) + 0.6, dim=-1)
    lump = torch.nn.functional.normalize(torch.randn(128, generator=gen), dim=0)
    U[2, :37] = torch.nn.functional.normalize(4 * lump + 0.2 * torch.randn(37, 128, generator=gen), dim=-1)
    U[2, 37:] = -lump
    assert abs(float(U.double().sum()) - g["input_sum"]) < 1e-6
    valid = torch.ones(3, 40, dtype=torch.bool)
    valid[1, 33:] = False
    side = oc.bisect_partition(U, valid)
    assert torch.equal(side.to(torch.uint8), g["side"])
    assert int(side[2].sum()) == 20                     # lopsided 2-means -> exact median cut
    part = oc.kway_partition(U, valid, torch.tensor([3, 2, 4]), 10)
    assert torch.equal(part.to(torch.uint8), g["part"])


def test_accounting(golden_small):
    for n, r, c, bits, over, frac in golden_small["accounting"]["rows"]:
        got = oc.overhead_rows(n=n, rows=r, clusters=c, d=128, summary_bits=bits)
        assert got == pytest.approx(over, rel=1e-12)
        assert (2 * r + got) / (2 * n) == pytest.approx(frac, rel=1e-12)
        assert oc.step_bytes(n=n, rows=r, clusters=c, d=128, summary_bits=bits) == pytest.approx(frac * 2 * n * 256)
    # every term of the formula: K+V rows, summaries, centroids, labels, row list, inserted key, direction sum
    b = oc.step_bytes(n=1000, rows=100, clusters=10, d=128, summary_bits=8)
    assert b == 2 * 100 * 256 + 10 * (128 + 12) + 10 * 128 + 2 * 1000 + 6 * 100 + 256 + 8 * 128


def test_selection_rule_properties():
    g = torch.Generator().manual_seed(0)
    score = torch.randn(4, 50, generator=g)
    count = torch.randint(0, 9, (4, 50), generator=g).float()
    score[count == 0] = -math.inf
    for need in (1, 17, 100, int(count.sum(1).min())):
        take = oc.ClusterOracle.take_until(score, count, need)
        got = (take * count).sum(1)
        assert torch.all(got >= need)
        # dropping the lowest-scored taken cluster falls under the need: the prefix is the shortest one
        low = torch.where(take, score, torch.full_like(score, math.inf)).argmin(1)
        assert torch.all(got - count[torch.arange(4), low] < need)
    full = oc.ClusterOracle.take_until(score, count, int(count[0].sum()))
    assert torch.equal(full[0], count[0] > 0)           # budget 1: exactly the non-empty clusters


def test_8bit_mode_keeps_invariants_and_mostly_agrees():
    K, V = oc.clustered_keys(2, 900, 128, seed=4)
    kw = dict(C=128, C_init=16, cap_keys=24.0, window=16, delta=math.inf, capacity=900)
    a, b = oc.ClusterOracle(**kw, summary_bits=32), oc.ClusterOracle(**kw, summary_bits=8)
    for n in range(700, 900):
        a.observe(K, n)
        b.observe(K, n)
    for st in (a, b):
        end = st.end
        cnt = torch.stack([torch.bincount(st.labels[i, 1:end].long(), minlength=128) for i in range(2)])
        assert torch.equal(cnt.float(), st.count) and int(st.count.max()) <= 24
    assert torch.equal(b.dir8, oc.to_int8_direction(b.sum_dir))
    assert (a.labels[:, :a.end] == b.labels[:, :b.end]).float().mean() > 0.9
    assert int(b.dir8.abs().max()) <= 127


def test_8bit_mode_fits_like_the_float_mode():
    """The prompt fit and its binning run on the float32 centroids in both modes ("the host fit does not depend
    on the copies", the reference's tests/test_quant8.py:49): only the per-step insert searches the int8 copies."""
    K, V = oc.clustered_keys(2, 900, 128, seed=6)
    kw = dict(C=128, C_init=16, cap_keys=24.0, window=16, delta=math.inf, capacity=900)
    a, b = oc.ClusterOracle(**kw, summary_bits=32), oc.ClusterOracle(**kw, summary_bits=8)
    a.observe(K, 800)
    b.observe(K, 800)
    assert torch.equal(a.labels, b.labels) and torch.equal(a.n_c, b.n_c) and torch.equal(a.sum_dir, b.sum_dir)
    assert torch.equal(b.cent8, oc.to_int8_direction(b.cent))


def test_sampled_selection_reproduces_the_reference(golden_sampled):
    """Proposal, fractional weights of the drawn clusters and the weighted attention against the reference's
    ssa.attn.tail_sample functions, same generator seeds."""
    g = golden_sampled["sampled"]
    c = g["cfg"]
    n = c["n0"] + c["steps"]
    K, V = oc.clustered_keys(c["h"], n, 128, seed=c["seed"])
    assert abs(float(K.double().sum()) - g["input_sum"]) < 1e-6
    Q = torch.randn(3, c["h"] * c["G"], 128, generator=torch.Generator().manual_seed(c["seed"] + 1000))
    st = oc.ClusterOracle(C=c["C"], C_init=16, cap_keys=24.0, window=16, delta=math.inf, capacity=n)
    for m in range(c["n0"], n + 1):
        st.observe(K, m)
    for t, p in enumerate(g["probes"]):
        prop = oc.sampling_proposal(st.scores(Q[t]), st.count, scale=1.0 / math.sqrt(128))
        torch.testing.assert_close(prop, p["prop"], rtol=0, atol=0)
        labels, w2 = st.select_sampled(Q[t], n=n, budget=c["budget"], S=c["S"], alpha=c["alpha"],
                                       generator=torch.Generator().manual_seed(100 + t))
        torch.testing.assert_close(w2, p["w2"], rtol=0, atol=0)
        drawn = (w2[:, :c["C"]] > 0) & (p["w"][:, :c["C"]] == 0)
        assert 1 <= int(drawn.sum(1).min()) and int(drawn.sum(1).max()) <= c["S"]
        out = oc.attend_labeled(Q[t], K[:, :n], V[:, :n], labels, w2)
        torch.testing.assert_close(out.float(), p["out"], rtol=0, atol=1e-6)


def test_sampled_weights_properties():
    """The reference's own checks of the sampler (tests/test_tail_sample.py:18-47): taken clusters weigh 1, empty
    ones 0, the draws add up to S, and no draw means the plain selection."""
    g = torch.Generator().manual_seed(5)
    count = torch.randint(0, 6, (3, 40), generator=g).double()
    taken = torch.rand(3, 40, generator=g) < 0.2
    prop = torch.rand(3, 40, generator=g, dtype=torch.float64) ** 3
    w = oc.sampled_weights(prop, count, taken, S=7, alpha=0.3, generator=torch.Generator().manual_seed(6))
    assert torch.all(w[taken & (count > 0)] == 1.0) and torch.all(w[count == 0] == 0.0)
    rest = ~taken & (count > 0)
    n_rest = rest.sum(1, keepdim=True)
    p = prop * rest
    pi = ((1 - 0.3) * p / p.sum(1, keepdim=True) + 0.3 / n_rest) * rest
    torch.testing.assert_close((w * pi * 7 * rest).sum(1), torch.full((3,), 7.0, dtype=torch.float64))
    none = oc.sampled_weights(prop, count, taken, S=0, alpha=0.3)
    torch.testing.assert_close(none, (taken & (count > 0)).double())
