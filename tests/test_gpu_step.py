"""The one-launch decode step (``skv_step``: selection and attention by thread-block clusters) against the
two launches it replaces and against the CPU oracle."""

from __future__ import annotations

import math

import pytest
import torch

from oracle import cluster_oracle as oc
from sparse_kv_reads_b200._lib import check, lib
from sparse_kv_reads_b200.cluster_state import SphereIndexGraph
from _helpers import DEV, device_index_from_oracle, isotropic_stream

pytestmark = pytest.mark.gpu


def rows_of(bits_row: torch.Tensor, labels_row: torch.Tensor, n: int) -> torch.Tensor:
    """Positions < n whose label's bit is set."""
    lab = labels_row[:n].long()
    word = bits_row.long()[lab // 32] & 0xFFFFFFFF
    return ((word >> (lab % 32)) & 1).nonzero().squeeze(1)


@pytest.mark.parametrize("h,G,n,C,budget", [(8, 2, 6000, 512, 0.2), (8, 4, 6000, 512, 0.05), (3, 8, 2500, 256, 0.5),
                                             (16, 2, 3000, 256, 0.2), (32, 2, 1500, 128, 0.3), (8, 2, 900, 128, 1.0),
                                             (1, 1, 700, 64, 0.3)])
def test_one_launch_step_equals_the_two_launches_and_the_oracle(h, G, n, C, budget):
    cap = -(-(n + 16) // 8) * 8
    Q, K, V = isotropic_stream(h, cap, h * G, seed=h + G)
    st = oc.ClusterOracle(C=C, C_init=C // 8, cap_keys=24.0, window=64, delta=math.inf, capacity=cap, summary_bits=8)
    st.observe(K, n)
    ix = device_index_from_oracle(st, budget=budget)
    ncl = lib().skv_step_clusters(h, G, C, 8)
    if ncl == 0 and h > 16:
        pytest.skip("this device keeps fewer clusters resident than there are heads")
    assert 1 <= ncl <= 8
    Kd, Vd = K.to(DEV), V.to(DEV)
    n_dev = torch.tensor([n], dtype=torch.int32, device=DEV)
    ix.need_dev.fill_(st.need(budget))
    for t in range(3):
        q = Q[t].to(DEV)
        _, w_ref = st.select(Q[t].float(), n=n, budget=budget)
        ix._select(q, n_dev, listed=False)
        two = ix._attend_labels(q, Kd, Vd, n_dev).clone()
        w2, bits2, cnt2 = ix.wbuf.clone(), ix.selbits.clone(), ix.cnt.clone()
        ix.wbuf.fill_(7.0)
        ix.selbits.fill_(-1)
        ix.cnt.fill_(-5)
        one = ix._step_one_launch(q, Kd, Vd, n_dev, None, ncl).clone()
        w1, bits1, cnt1 = ix.wbuf.clone(), ix.selbits.clone(), ix.cnt.clone()
        assert int((w1.cpu() != w_ref).sum(1).max()) <= 1          # rounding may move the one boundary cluster
        assert int((w1 != w2).sum(1).max()) <= 1
        for i in range(h):                                         # the bit set is the weights
            on = [(int(bits1[i, c // 32]) >> (c % 32)) & 1 for c in range(C + 1)]
            assert on == [int(x > 0) for x in w1[i].cpu().tolist()]
        lab = ix.labels.cpu()
        rows = [rows_of(bits1[i].cpu(), lab[i], n) for i in range(h)]
        assert cnt1.cpu().tolist() == [len(r) for r in rows]
        ref = oc.attend_rows(Q[t], K, V, rows)
        assert float((one.cpu().double() - ref).abs().max()) <= 1e-2
        if torch.equal(w1, w2):
            assert torch.equal(cnt1, cnt2) and torch.equal(bits1, bits2)
            assert float((one.float() - two.float()).abs().max()) <= 1e-2
        # the last merge left to the output product: y = out . W^T straight from the clusters' partials
        ix.cnt.fill_(-3)
        parts = ix._step_one_launch(q, Kd, Vd, n_dev, None, ncl, defer_merge=True)
        Kin, N = h * G * 128, 192
        W = (torch.randn(N, Kin, generator=torch.Generator().manual_seed(t)) / Kin ** 0.5).to(torch.bfloat16).to(DEV)
        y = torch.empty(1, N, dtype=torch.bfloat16, device=DEV)
        check(lib().skv_gemv_attended(W.data_ptr(), N, Kin, y.data_ptr(), 1, parts.workspace.data_ptr(), parts.clusters,
                                      parts.G, parts.cnt.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream),
              "skv_gemv_attended")
        want = one.view(1, Kin).float() @ W.float().T
        torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2)
        assert torch.equal(ix.cnt, cnt1)
    assert ix.check_status() == 0


def test_one_launch_step_at_the_benchmark_shape():
    """8 heads x 32,768 tokens, 2,048 slots, 20 %: four clusters of 8 CTAs per head; rows and output against the
    oracle, the same answer on a second call (the ticket words return to zero), and nothing selected when nothing
    is clustered."""
    h, G, n = 8, 2, 32768
    K, V = oc.clustered_keys(h, n + 8, 128, seed=77)
    Kb, Vb = K.to(torch.bfloat16), V.to(torch.bfloat16)
    q = (torch.randn(h * G, 128, generator=torch.Generator().manual_seed(78)) * 2).to(torch.bfloat16)
    ix = SphereIndexGraph(C=2048, C_init=256, cap_keys=64.0, window=64, delta=0.03, capacity=n + 8, budget=0.2)
    Kd, Vd = Kb.to(DEV), Vb.to(DEV)
    ix.observe(Kd, n)
    ncl = ix._step_clusters(G)
    assert ncl >= 2
    n_dev = torch.tensor([n], dtype=torch.int32, device=DEV)
    ix.need_dev.fill_(math.ceil(0.2 * (ix.end - 1)))
    ix._select(q.to(DEV), n_dev, listed=False)
    w2 = ix.wbuf.clone()
    outs = []
    for _ in range(2):
        ix.cnt.fill_(-1)
        outs.append(ix._step_one_launch(q.to(DEV), Kd, Vd, n_dev, None, ncl).clone())
    assert torch.equal(outs[0], outs[1])
    assert int((ix.wbuf != w2).sum(1).max()) <= 1
    lab = ix.labels.cpu()
    rows = [rows_of(ix.selbits[i].cpu(), lab[i], n) for i in range(h)]
    assert ix.cnt.cpu().tolist() == [len(r) for r in rows]
    need = math.ceil(0.2 * (ix.end - 1))
    for r in rows:
        assert need <= len(r) - 65 < need + 64
    ref = oc.attend_rows(q, Kb, Vb, rows)
    assert float((outs[0].cpu().double() - ref).abs().max()) <= 1e-2
    # a context shorter than the window: nothing is clustered, every row is read
    short = SphereIndexGraph(C=64, window=64, delta=math.inf, capacity=256, budget=0.5)
    Ks, Vs = Kd[:, :256].contiguous(), Vd[:, :256].contiguous()
    short.observe(Ks, 40)                                   # all 40 positions are inside the window
    m_dev = torch.tensor([40], dtype=torch.int32, device=DEV)
    short.need_dev.fill_(0)
    got = short._step_one_launch(q.to(DEV), Ks, Vs, m_dev, None, short._step_clusters(G))
    dense = oc.attend_rows(q, Kb[:, :256], Vb[:, :256], [torch.arange(40)] * h)
    assert float((got.cpu().double() - dense).abs().max()) <= 1e-2
    assert short.cnt.cpu().tolist() == [40] * h


def test_one_launch_step_takes_exact_ties_in_slot_order():
    """Eight clusters with identical summaries (scored by one warp, so their shared scores are the same bits) and a
    budget that ends inside them: the lower slots are taken first, as the oracle's stable ranking does."""
    h, G, n, C = 4, 2, 3000, 256
    cap = -(-(n + 16) // 8) * 8
    Q, K, V = isotropic_stream(h, cap, h * G, seed=41)
    st = oc.ClusterOracle(C=C, C_init=64, cap_keys=40.0, window=64, delta=math.inf, capacity=cap, summary_bits=8)
    st.observe(K, n)
    for name in ("sum_dir", "dir8", "mmax", "mmin"):
        t = getattr(st, name)
        t[:, 8:16] = t[:, 8:9]
    st.count[:, 8:16] = torch.tensor([7.0, 3.0, 9.0, 4.0, 6.0, 5.0, 8.0, 2.0])
    ix = device_index_from_oracle(st, budget=0.3)
    ncl = lib().skv_step_clusters(h, G, C, 8)
    Kd, Vd = K.to(DEV), V.to(DEV)
    n_dev = torch.tensor([n], dtype=torch.int32, device=DEV)
    q = Q[0]
    shared = st.shared_score(st.scores(q.float()))
    assert all(len(set(shared[i, 8:16].tolist())) == 1 for i in range(h))
    for into in (1, 12, 25, 40):                            # keys of the tied clusters the budget reaches into
        # per head the need differs; the kernel takes one need per head from need_dev
        needs = []
        for i in range(h):
            ahead = float(st.count[i][shared[i] > shared[i, 8]].sum())
            needs.append(int(ahead) + into)
        ix.need_dev.copy_(torch.tensor(needs, dtype=torch.int32))
        ix._step_one_launch(q.to(DEV), Kd, Vd, n_dev, None, ncl)
        w = ix.wbuf.cpu()
        for i in range(h):
            want = oc.ClusterOracle.take_until(shared[i:i + 1], st.count[i:i + 1], needs[i])[0]
            assert torch.equal(w[i, :C] > 0, want), (into, i)
            tied = (w[i, 8:16] > 0).tolist()
            assert tied == sorted(tied, reverse=True) and any(tied) and not all(tied)
