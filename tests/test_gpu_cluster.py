"""Selection, insertion/split and prompt-fit kernels against the CPU oracle (through the C ABI)."""

from __future__ import annotations

import math

import pytest
import torch

from oracle import cluster_oracle as oc
from sparse_kv_reads_b200.cluster_state import SphereIndexGraph
from _helpers import DEV, device_index_from_oracle, isotropic_stream, row_sets

pytestmark = pytest.mark.gpu


def fitted_oracle(h=4, n=1500, *, C=256, C_init=None, cap_keys=0.0, split_factor=0.0, window=64, seed=2,
                  summary_bits=32, dtype=torch.float32, H=None, capacity=4096):
    Q, K, V = isotropic_stream(h, capacity, H or 4 * h, seed=seed, dtype=dtype)
    st = oc.ClusterOracle(C=C, C_init=C_init, cap_keys=cap_keys, split_factor=split_factor, window=window,
                          delta=math.inf, capacity=capacity, summary_bits=summary_bits)
    st.observe(K, n)
    return st, Q, K, V


# ---- selection ----------------------------------------------------------------------------------
@pytest.mark.parametrize("budget", [0.05, 0.2, 0.5, 1.0])
@pytest.mark.parametrize("bits", [32, 8])
def test_pick_is_bit_exact_given_the_oracle_scores(budget, bits):
    st, Q, K, V = fitted_oracle(summary_bits=bits)
    ix = device_index_from_oracle(st)
    n = st.n
    for t in (1400, 1450, 1499):
        q = Q[t].float()
        shared = st.shared_score(st.scores(q))
        _, w_ref = st.select(q, n=n, budget=budget)
        _, w = ix.labels_and_weights(q.to(DEV), n=n, budget=budget, shared_in=shared.to(DEV).contiguous())
        assert torch.equal(w.cpu(), w_ref)
        sets, lists = row_sets(ix)
        ref_rows = st.positions(w_ref, n)
        need = st.need(budget)
        for i in range(st.h):
            assert sets[i] == set(ref_rows[i].tolist())
            assert torch.equal(lists[i].long(), ref_rows[i])              # ascending, deterministic
            assert len(sets[i]) - (n - st.end) - 1 >= min(need, int(st.count[i].sum()))
        if budget == 1.0:
            assert torch.equal(w.cpu()[:, :st.C] > 0, st.count > 0)


@pytest.mark.parametrize("qdtype", [torch.float32, torch.bfloat16])     # bf16 queries + 8-bit summaries: tensor cores
@pytest.mark.parametrize("bits", [32, 8])
@pytest.mark.parametrize("G", [1, 2, 4, 8, 16])
def test_scores_and_full_selection_match_the_oracle(bits, G, qdtype):
    st, Q, K, V = fitted_oracle(h=4, H=4 * G, summary_bits=bits, seed=3)
    ix = device_index_from_oracle(st)
    n = st.n
    e_out = torch.full((st.h, G, st.C), float("nan"), device=DEV)
    s_out = torch.full((st.h, st.C), float("nan"), device=DEV)
    diff = 0
    for t in (1401, 1480):
        q = Q[t].to(qdtype).float()                       # the oracle sees the query as the kernel does
        e = st.scores(q)
        _, w_ref = st.select(q, n=n, budget=0.2)
        _, w = ix.labels_and_weights(Q[t].to(qdtype).to(DEV), n=n, budget=0.2, shared_out=s_out, e_out=e_out)
        live = (st.count > 0).unsqueeze(1).expand_as(e)
        got = e_out.cpu()
        assert torch.isinf(got[~live]).all() and (got[~live] < 0).all()
        scale = float(e[live].abs().max())                 # 1e-5 of the score scale: values near 0 are differences
        torch.testing.assert_close(got[live], e[live], rtol=1e-5, atol=1e-5 * max(1.0, scale))
        torch.testing.assert_close(s_out.cpu()[st.count > 0], st.shared_score(e)[st.count > 0], rtol=1e-5, atol=1e-7)
        diff = max(diff, int((w.cpu() != w_ref).sum(1).max()))
    assert diff <= 1                     # rounding of the scores may move the single boundary cluster


def test_exact_ties_go_to_the_lower_slot():
    st, Q, K, V = fitted_oracle(h=2, H=4)
    ix = device_index_from_oracle(st)
    shared = torch.zeros(st.h, st.C)
    shared[:, ::3] = 1.0                                   # many equal scores on both sides of the threshold
    shared[st.count == 0] = -math.inf
    for budget in (0.1, 0.37, 0.9):
        need = st.need(budget)
        ref = oc.ClusterOracle.take_until(shared, st.count, need)
        _, w = ix.labels_and_weights(Q[0].float().to(DEV), n=st.n, budget=budget, shared_in=shared.to(DEV))
        assert torch.equal(w.cpu()[:, :st.C] > 0, ref)


def test_budget_zero_and_short_contexts_read_only_the_always_read_rows():
    Q, K, V = isotropic_stream(2, 256, 4, seed=1, dtype=torch.float32)
    ix = SphereIndexGraph(C=16, window=64, delta=math.inf, capacity=256, summary_bits=32)
    ix.observe(K.to(DEV), 40)                              # shorter than the window: nothing clustered
    _, w = ix.labels_and_weights(Q[0].to(DEV), n=40, budget=0.5)
    sets, _ = row_sets(ix)
    assert all(s == set(range(40)) for s in sets) and float(w[:, :16].sum()) == 0


# ---- insertion and in-kernel split -------------------------------------------------------------
@pytest.mark.parametrize("bits", [32, 8])
def test_insertion_matches_the_oracle_without_splits(bits):
    st, Q, K, V = fitted_oracle(h=8, n=1000, summary_bits=bits, capacity=1408)
    ix = device_index_from_oracle(st)
    Kd = K.to(DEV)
    for n in range(1001, 1400):
        st.observe(K, n)
        ix.observe(Kd, n)
    same = (st.labels[:, :1400] == ix.labels.cpu()[:, :1400]).float().mean().item()
    assert same >= 0.999, same
    if same == 1.0:
        torch.testing.assert_close(ix.count.cpu(), st.count)
        torch.testing.assert_close(ix.mmax.cpu(), st.mmax)
        torch.testing.assert_close(ix.mmin.cpu(), st.mmin)
        torch.testing.assert_close(ix.sum_dir.cpu(), st.sum_dir, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(ix.ksum.cpu(), st.ksum, rtol=1e-5, atol=1e-3)
    if bits == 8:
        want = oc.to_int8_direction(ix.sum_dir.cpu())
        assert int((ix.dir8.cpu().int() - want.int()).abs().max()) <= 1
    assert ix.check_status() == 0


@pytest.mark.parametrize("case", ["cap_keys", "split_factor"])
def test_splitting_stream_matches_the_oracle(case):
    kw = dict(C=256, C_init=64, cap_keys=24.0) if case == "cap_keys" else dict(C=256, C_init=64, split_factor=2.0)
    st, Q, K, V = fitted_oracle(h=8, n=1000, capacity=2608, **kw)
    ix = device_index_from_oracle(st)
    Kd = K.to(DEV)
    for n in range(1001, 2600):
        st.observe(K, n)
        ix.observe(Kd, n)
    end = ix.end
    lab = ix.labels.cpu()
    assert ix.splits > 0 and int((ix.n_c.cpu() - st.n_c).abs().max()) <= 4
    same = (st.labels[:, :end] == lab[:, :end]).float().mean().item()
    assert same >= 0.999 or int((ix.n_c.cpu() - st.n_c).abs().max()) > 0, same
    # invariants of the reference's tests/test_split_kernels.py:27-41, :74-101
    assert torch.all(ix.count.cpu() <= ix.cap.cpu().unsqueeze(1))
    assert torch.all(lab[:, 1:end].long() < ix.n_c.cpu().unsqueeze(1))
    slots = torch.arange(256).unsqueeze(0)
    assert torch.all(ix.count.cpu()[slots >= ix.n_c.cpu().unsqueeze(1)] == 0)
    counts = torch.stack([torch.bincount(lab[i, 1:end].long(), minlength=256) for i in range(8)])
    torch.testing.assert_close(ix.count.cpu(), counts.float())
    Kr = K.float() - ix.mu_ref.cpu().unsqueeze(1)
    mag = Kr.norm(dim=-1)
    Kn = Kr / mag.unsqueeze(-1)
    sd = torch.zeros(8, 256, 128).scatter_add_(1, lab[:, 1:end].long().unsqueeze(-1).expand(-1, -1, 128), Kn[:, 1:end])
    torch.testing.assert_close(ix.sum_dir.cpu(), sd, rtol=1e-3, atol=1e-3)
    live = ix.count.cpu() > 0
    mx = torch.zeros(8, 256).scatter_reduce_(1, lab[:, 1:end].long(), mag[:, 1:end], reduce="amax")
    torch.testing.assert_close(ix.mmax.cpu()[live], mx[live], rtol=1e-4, atol=1e-4)
    cent = torch.nn.functional.normalize(ix.sum_dir.cpu(), dim=-1)
    split_made = torch.arange(256).unsqueeze(0) >= 64                      # slots created by splits hold unit(sum) at creation
    assert torch.isfinite(ix.cent.cpu()).all() and cent.shape == ix.cent.shape and split_made.any()
    assert ix.check_status() == 0


def test_each_split_follows_the_two_way_rule_on_the_same_members():
    """Every in-kernel split against the oracle's bisect_partition on the same members: at most
    max(1, 2 %) members on the other side; halves of 25-75 % or an exact median cut
    (the reference's tests/test_split_kernels.py:120-156)."""
    Q, K, V = isotropic_stream(4, 1800, 8, seed=3, dtype=torch.float32)
    g = torch.Generator().manual_seed(4)
    main = torch.randn(4, 1, 128, generator=g)
    K[:, 1100:] = 3 * main + 0.3 * torch.randn(4, 700, 128, generator=g)      # a tight lump: lopsided 2-means
    K[:, 1150::41] = -3 * main
    ix = SphereIndexGraph(C=256, C_init=64, split_factor=2.0, window=64, delta=math.inf, capacity=1800,
                          summary_bits=32)
    Kd = K.to(DEV)
    ix.observe(Kd, 1000)
    checked = median_cuts = 0
    for n in range(1001, 1800):
        lab0, nc0, end0 = ix.labels.cpu().clone(), ix.n_c.cpu().clone(), ix.end
        ix.observe(Kd, n)
        lab1, nc1 = ix.labels.cpu(), ix.n_c.cpu()
        for i in (nc1 > nc0).nonzero().flatten().tolist():
            new = int(nc0[i])
            assert int(nc1[i]) == new + 1 and ix.end == end0 + 1
            c = int(lab1[i, end0]) if int(lab1[i, end0]) != new else None
            moved = (lab1[i, 1:ix.end] == new).nonzero().flatten() + 1
            if c is None:
                c = int(lab0[i, moved[moved < end0][0]])
            was = lab0[i, 1:ix.end].clone()
            was[end0 - 1] = c
            pos = (was == c).nonzero().flatten() + 1
            assert set(lab1[i, pos].tolist()) == {c, new}
            U = torch.nn.functional.normalize(K[i, pos].float() - ix.mu_ref.cpu()[i], dim=-1).unsqueeze(0)
            side = oc.bisect_partition(U, torch.ones(1, len(pos), dtype=torch.bool))[0]
            got = (lab1[i, pos] == new).long()
            assert int((side != got).sum()) <= max(1, 0.02 * len(pos))
            share = got.float().mean()
            assert 0.25 <= share <= 0.75 or int(got.sum()) == len(pos) - len(pos) // 2
            median_cuts += int(got.sum()) == len(pos) - len(pos) // 2
            checked += 1
    assert checked >= 20 and median_cuts > 0


# ---- prompt fit ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["fixed", "cap_keys", "split_factor"])
def test_fit_matches_the_oracle(case, dtype):
    kw = {"fixed": dict(C=64), "cap_keys": dict(C=256, C_init=32, cap_keys=24.0),
          "split_factor": dict(C=256, C_init=32, split_factor=1.2)}[case]
    h, n = 4, 2100
    K, V = oc.clustered_keys(h, n, 128, seed=31)
    K = K.to(dtype)
    st = oc.ClusterOracle(window=64, delta=math.inf, capacity=2104, **kw)
    st.observe(K, n)
    ix = SphereIndexGraph(window=64, delta=math.inf, capacity=2104, summary_bits=32, **kw)
    ix.observe(K.to(DEV), n)
    end = st.end
    assert ix.end == end and int(ix.end_dev[0]) == end
    torch.testing.assert_close(ix.mu_ref.cpu(), st.mu_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ix.ksum.cpu(), st.ksum, rtol=1e-5, atol=1e-2)
    torch.testing.assert_close(ix.rbar.cpu(), st.rbar, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ix.cap.cpu(), st.cap)
    same = (ix.labels.cpu()[:, :n] == st.labels[:, :n]).float().mean().item()
    assert same >= 0.999, same
    assert int((ix.n_c.cpu() - st.n_c).abs().max()) <= (0 if same == 1.0 else 3)
    if same == 1.0:
        torch.testing.assert_close(ix.count.cpu(), st.count)
        torch.testing.assert_close(ix.cent.cpu(), st.cent, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(ix.sum_dir.cpu(), st.sum_dir, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(ix.mmax.cpu(), st.mmax, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(ix.mmin.cpu(), st.mmin, rtol=1e-5, atol=1e-5)
        assert ix.splits == st.splits
    lab = ix.labels.cpu()
    counts = torch.stack([torch.bincount(lab[i, 1:end].long(), minlength=ix.C) for i in range(h)])
    torch.testing.assert_close(ix.count.cpu(), counts.float())
    assert torch.all(lab[:, end:] == ix.C) and torch.all(lab[:, 0] == ix.C)
    if case != "fixed":
        assert torch.all(ix.count.cpu() <= ix.cap.cpu().unsqueeze(1)) and ix.splits > 0
    assert ix.check_status() == 0


def test_one_lloyd_step_from_the_oracle_centroids_agrees():
    """Step-wise parity: starting from the oracle's centroids after t iterations, the kernel's
    assignment agrees on >= 99.9 % of the keys, excluding keys whose two best centroids are within
    1e-6 (ten Lloyd steps amplify rounding, so the end-to-end check alone would hide errors)."""
    h, n = 4, 3000
    Q, K, V = isotropic_stream(h, n, 8, seed=7, dtype=torch.float32)
    st = oc.ClusterOracle(C=64, window=64, delta=math.inf, capacity=3000, kmeans_iters=3)
    st.observe(K, n)
    ix = device_index_from_oracle(st)
    ix.flags.fill_(1)
    ix._rebuild(K.to(DEV), torch.arange(h))                # rebin about ksum / (end-1) with the centroids kept
    Kr = K[:, 1:st.end].float() - ix.mu_ref.cpu().unsqueeze(1)
    Kn = torch.nn.functional.normalize(Kr, dim=-1)
    sims = torch.einsum("hmd,hcd->hmc", Kn, st.cent)
    top2 = sims.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 1e-6
    want = sims.argmax(-1)
    got = ix.labels.cpu()[:, 1:st.end].long()
    assert ((want == got) | ~clear).float().mean().item() >= 0.999
    assert ix.rebuilds == h


def test_recentring_follows_the_oracle():
    g = None
    h, n0 = 2, 500
    K, V = oc.clustered_keys(h, 704, 128, seed=22)
    kw = dict(C=64, C_init=16, split_factor=2.0, window=8, delta=0.003, capacity=704, check_every=4)
    st = oc.ClusterOracle(**kw)
    ix = SphereIndexGraph(**kw, summary_bits=32, async_check=False)
    Kd = K.to(DEV)
    for n in range(n0, 700):
        st.observe(K, n)
        ix.observe(Kd, n)
    assert ix.rebuilds > 0 and abs(ix.rebuilds - st.rebuilds) <= max(2, 0.05 * st.rebuilds)
    end = ix.end
    lab = ix.labels.cpu()
    counts = torch.stack([torch.bincount(lab[i, 1:end].long(), minlength=64) for i in range(h)])
    torch.testing.assert_close(ix.count.cpu(), counts.float())
    torch.testing.assert_close(ix.mu_ref.cpu(), st.mu_ref, rtol=1e-4, atol=1e-4)


def test_one_fit_for_all_layers_equals_a_fit_per_layer():
    """Three layers sharing an arena, fitted by one call over their stacked states (a table of per-layer
    caches), against the same three layers fitted one by one: identical labels, counts and caps."""
    from sparse_kv_reads_b200.cluster_state import ClusterArena, fit_layers
    h, n, layers = 2, 1500, 3
    caps = -(-(n + 8) // 8) * 8
    caches = [oc.clustered_keys(h, caps, 128, seed=60 + i)[0].to(torch.bfloat16).to(DEV) for i in range(layers)]
    kw = dict(C=256, C_init=16, cap_keys=24.0, window=16, delta=math.inf, capacity=caps, summary_bits=8)
    arena = ClusterArena(layers=layers, h=h, C=256, d=128, capacity=caps, summary_bits=8, device=DEV)
    together = [SphereIndexGraph(arena=arena, layer=i, **kw) for i in range(layers)]
    assert fit_layers(together, caches, n)
    # a workspace limit that forces one layer per group must give the same state
    arena2 = ClusterArena(layers=layers, h=h, C=256, d=128, capacity=caps, summary_bits=8, device=DEV)
    grouped = [SphereIndexGraph(arena=arena2, layer=i, **kw) for i in range(layers)]
    assert fit_layers(grouped, caches, n, max_workspace=1)
    for i in range(layers):
        alone = SphereIndexGraph(**kw)
        alone.observe(caches[i], n)
        for other in (together[i], grouped[i]):
            assert other._fitted and other.n == n and other.end == alone.end
            assert torch.equal(other.labels, alone.labels) and torch.equal(other.n_c, alone.n_c)
            assert torch.equal(other.count, alone.count) and torch.equal(other.cap, alone.cap)
            torch.testing.assert_close(other.sum_dir, alone.sum_dir, rtol=0, atol=0)
            assert torch.equal(other.dir8, alone.dir8) and other.splits == alone.splits
        assert int(alone.n_c.min()) > 16 and alone.check_status() == 0


def test_clusters_stay_under_the_cap_through_recentring():
    """Rebinning about a new mean can pile keys onto a few centroids; the clusters it leaves over the cap are
    divided at once, so that none outgrows what the in-kernel split can stage (no status bit, count <= cap)."""
    h, n0, n1 = 2, 900, 1300
    K, _ = oc.clustered_keys(h, 1304, 128, seed=31)
    K[:, 1000:] += 0.8                                    # a shift of the keys' mean: drift flags, recentring
    Kd = K.to(torch.bfloat16).to(DEV)
    ix = SphereIndexGraph(C=256, C_init=16, cap_keys=24.0, window=8, delta=0.01, capacity=1304, check_every=4,
                          summary_bits=8, async_check=False)
    for n in range(n0, n1):
        ix.observe(Kd, n)
    assert ix.rebuilds > 0
    end = ix.end
    lab = ix.labels.cpu()
    counts = torch.stack([torch.bincount(lab[i, 1:end].long(), minlength=256) for i in range(h)])
    assert torch.equal(ix.count.cpu(), counts.float())
    assert float(ix.count.max()) <= 24.0 and ix.check_status() == 0
    assert int(ix.n_c.max()) < 256


@pytest.mark.parametrize("G", [2, 4])
def test_every_query_head_ranks_for_itself(G):
    """group="per_head": from the oracle's state, each query head's selection equals the oracle's bit for bit
    and its attention reads exactly its own rows."""
    h, n = 3, 1200
    Q, K, V = isotropic_stream(h, 1208, h * G, seed=13 + G, dtype=torch.float32)
    st = oc.ClusterOracle(C=128, C_init=32, cap_keys=24.0, window=16, delta=math.inf, capacity=1208)
    st.observe(K, n)
    ix = device_index_from_oracle(st, budget=0.25)
    q = Q[0]
    _, w_want = st.select(q, n=n, budget=0.25, group="per_head")
    out, labels, w = ix.attend(q.to(DEV), K.to(DEV), V.to(DEV), n=n, budget=0.25, group="per_head")
    assert w.shape == (h * G, 129) and torch.equal(w.cpu(), w_want)
    assert not torch.equal(w_want.view(h, G, -1)[:, 0], w_want.view(h, G, -1)[:, 1])     # the heads do differ
    want = oc.attend_labeled(q, K[:, :n], V[:, :n], labels.cpu(), w_want)
    assert float((out.cpu().double() - want).abs().max()) <= 1e-5
    # the shared modes still work afterwards (their buffers were kept)
    _, w_sum = ix.labels_and_weights(q.to(DEV), n=n, budget=0.25)
    assert torch.equal(w_sum.cpu(), st.select(q, n=n, budget=0.25)[1])


def test_sampled_clusters_follow_the_reference_golden(golden_sampled):
    """attend_sampled (ssa/kernels/sphere_fused.py:503-518) against the golden made with the reference's own
    proposal_from_scores / tail_sample_weights / label_weighted_attention: same generator seed, so the same
    clusters are drawn; fractional weights to 1e-4 (the scores are the kernel's), output to 1e-2 (in fact 1e-4)."""
    g = golden_sampled["sampled"]
    c = g["cfg"]
    n = c["n0"] + c["steps"]
    K, V = oc.clustered_keys(c["h"], n, 128, seed=c["seed"])
    Q = torch.randn(3, c["h"] * c["G"], 128, generator=torch.Generator().manual_seed(c["seed"] + 1000))
    ix = SphereIndexGraph(C=c["C"], C_init=16, cap_keys=24.0, window=16, delta=math.inf, capacity=-(-n // 8) * 8,
                          summary_bits=32, async_check=False)
    Kd, Vd = K.to(DEV), V.to(DEV)
    for m in range(c["n0"], n):
        ix.observe(Kd, m)
    for t, p in enumerate(g["probes"]):
        out, labels, w2 = ix.attend_sampled(Q[t].to(DEV), Kd, Vd, n=n, budget=c["budget"], S=c["S"], alpha=c["alpha"],
                                            generator=torch.Generator().manual_seed(100 + t))
        assert torch.equal(w2.cpu() > 0, p["w2"] > 0)
        torch.testing.assert_close(w2.cpu(), p["w2"], rtol=1e-4, atol=1e-6)
        assert float((out.cpu() - p["out"]).abs().max()) <= 1e-4
        drawn = (w2[:, :c["C"]] > 0) & (ix.wbuf[:, :c["C"]] == 0)
        assert int(drawn.sum()) >= c["h"] and float(w2[:, :c["C"]][drawn].min()) > 0
    # no draws: the plain selection, and the weighted kernel equals the list-driven one
    out0, _, w0 = ix.attend_sampled(Q[0].to(DEV), Kd, Vd, n=n, budget=c["budget"], S=0, alpha=0.1)
    out0 = out0.clone()
    plain, _, w = ix.attend(Q[0].to(DEV), Kd, Vd, n=n, budget=c["budget"])
    assert torch.equal(w0, w) and float((out0 - plain).abs().max()) <= 1e-5


def test_weighted_attention_in_bf16_against_the_oracle():
    h, G, n = 4, 2, 3000
    Q, K, V = isotropic_stream(h, 3008, h * G, seed=19)
    st = oc.ClusterOracle(C=256, C_init=64, cap_keys=32.0, window=64, delta=math.inf, capacity=3008, summary_bits=8)
    st.observe(K, n)
    ix = device_index_from_oracle(st)
    labels, w2 = st.select_sampled(Q[0].float(), n=n, budget=0.1, S=12, alpha=0.2,
                                   generator=torch.Generator().manual_seed(3))
    got, _, wd = ix.attend_sampled(Q[0].to(DEV), K.to(DEV), V.to(DEV), n=n, budget=0.1, S=12, alpha=0.2,
                                   generator=torch.Generator().manual_seed(3))
    same = torch.equal(wd.cpu() > 0, w2 > 0)
    want = oc.attend_labeled(Q[0], K[:, :n], V[:, :n], labels, wd.cpu().double() if not same else w2)
    assert float((got.cpu().double() - want).abs().max()) <= 1e-2
    assert int(((wd.cpu() > 0) != (w2 > 0)).sum()) <= 4          # a boundary cluster may move a probe
