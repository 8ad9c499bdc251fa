"""Whole decode step on the GPU: list-free attention equals the listed one, sparse at budget 1 equals
dense, graph replay equals eager, a batch equals separate runs, the engine-seam patch equals the decoder."""

from __future__ import annotations

import math

import pytest
import torch

from oracle import cluster_oracle as oc
from sparse_kv_reads_b200 import GraphDecoder, Qwen3Config, Qwen3Model, install, uninstall
from sparse_kv_reads_b200.cluster_state import SphereIndexGraph
from _helpers import DEV, isotropic_stream, row_sets

pytestmark = pytest.mark.gpu

TINY = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
            intermediate_size=512, vocab_size=1000, max_position_embeddings=2048)


def tiny_model(seed=3):
    with torch.device(DEV):
        m = Qwen3Model(Qwen3Config(**TINY))
    return m.to(torch.bfloat16).eval().init_random(seed=seed, std=0.05)


@pytest.mark.parametrize("G", [2, 4])
def test_attention_from_labels_equals_attention_over_the_list(G):
    h, n = 6, 3000
    Q, K, V = isotropic_stream(h, 3008, h * G, seed=11)
    ix = SphereIndexGraph(C=256, C_init=64, cap_keys=32.0, window=64, delta=math.inf, capacity=3008, budget=0.2)
    Kd, Vd = K.to(DEV), V.to(DEV)
    ix.observe(Kd, n)
    for t in range(5):
        ix.observe(Kd, n + t)
        q = Q[t].to(DEV)
        labels, w = ix.labels_and_weights(q, n=n + t, budget=0.2)
        want = ix._attend(q, Kd, Vd).clone()
        cnt = ix.cnt.clone()
        sets, lists = row_sets(ix)
        ix._select(q, ix._n_scalar, listed=False)
        assert int(ix.cnt.abs().sum()) == 0
        got = ix._attend_labels(q, Kd, Vd, ix._n_scalar)
        assert torch.equal(ix.cnt, cnt)
        assert float((got.float() - want.float()).abs().max()) <= 1e-2
        ref = oc.attend_rows(Q[t], K, V, [l.long() for l in lists])
        assert float((got.cpu().double() - ref).abs().max()) <= 1e-2
        bits = ix.selbits.cpu()
        for i in range(h):
            on = [(int(bits[i, c // 32]) >> (c % 32)) & 1 for c in range(257)]
            assert on == [int(x > 0) for x in w[i].cpu().tolist()]
    assert ix.check_status() == 0


def run_decoder(model, ids, P, T, capture, **kw):
    B = ids.shape[0]
    cache = model.alloc_cache(-(-(P + T + 2) // 16) * 16, max_batch=B)
    out = []
    with torch.no_grad():
        model.prefill(ids[:, :P], cache, chunk=128)
        dec = GraphDecoder(model, cache, **kw)
        dec.prepare(P)
        if capture:
            dec.capture()
        for t in range(P, P + T):
            out.append(dec.step(ids[:, t:t + 1], t)[:, -1].float().clone())
    return torch.stack(out, 1), dec


@pytest.mark.parametrize("batch", [1, 3])
def test_insert_at_the_end_of_the_step_before_gives_the_same_decode(batch):
    """The all-layer insert of a step runs at the end of the step before it, beside the vocabulary projection; ahead
    of the first layer (the reference's order) every step selects from the same state, so the logits are the same
    bits - with splits happening and at a budget where the selection matters."""
    model = tiny_model(seed=23)
    P, T = 280, 60
    ids = torch.randint(0, 1000, (batch, P + T + 1), generator=torch.Generator().manual_seed(17)).to(DEV)
    kw = dict(mode="cluster", budget=0.3, C=64, C_init=16, cap_keys=24.0, window=8, delta=float("inf"), summary_bits=8)
    ahead, d1 = run_decoder(model, ids, P, T, True, insert_ahead=True, **kw)
    first, d0 = run_decoder(model, ids, P, T, True, insert_ahead=False, **kw)
    assert d1.insert_ahead and not d0.insert_ahead and d1.insert_all is not None
    assert torch.equal(ahead, first)
    assert sum(i.splits for i in d1.attn) > 0
    for a, b in zip(d1.attn, d0.attn):
        assert [x - 1 for x in a.end_dev.cpu().tolist()] == b.end_dev.cpu().tolist()     # one key ahead between steps
        assert a.check_status() == 0 and b.check_status() == 0


def test_budget_one_equals_dense_and_graph_equals_eager():
    model = tiny_model()
    P, T = 300, 80
    ids = torch.randint(0, 1000, (1, P + T + 1), generator=torch.Generator().manual_seed(3)).to(DEV)
    kw = dict(mode="cluster", budget=1.0, C=64, C_init=16, split_factor=2.0, window=4, delta=float("inf"),
              check_every=4, summary_bits=32)
    dense, _ = run_decoder(model, ids, P, T, True, mode="dense")
    eager, d0 = run_decoder(model, ids, P, T, False, **kw)
    graph, d1 = run_decoder(model, ids, P, T, True, **kw)
    torch.testing.assert_close(eager, dense, rtol=2e-2, atol=2e-2)
    assert torch.equal(graph, eager)                                 # replay is the same arithmetic
    assert sum(i.splits for i in d1.attn) > 0 and all(int(i.n_c.max()) <= 64 for i in d1.attn)
    assert all(i.check_status() in (0, 1) for i in d1.attn)          # 1 = a head used up its 64 slots
    with torch.no_grad():                                            # the model's own dense decode agrees too
        cache = model.alloc_cache(400)
        model.prefill(ids[:, :P], cache, chunk=128)
        own = torch.stack([model(ids[:, t:t + 1], cache, start_pos=t)[:, -1].float() for t in range(P, P + 8)], 1)
    torch.testing.assert_close(own, dense[:, :8], rtol=5e-2, atol=5e-2)   # torch SDPA vs the gather kernel


def test_a_batch_equals_separate_sequences():
    model = tiny_model(seed=5)
    P, T = 260, 24
    ids = torch.randint(0, 1000, (2, P + T + 1), generator=torch.Generator().manual_seed(4)).to(DEV)
    kw = dict(mode="cluster", budget=0.3, C=64, C_init=16, cap_keys=24.0, window=16, delta=0.03, summary_bits=8)
    both, _ = run_decoder(model, ids, P, T, True, **kw)
    for b in range(2):
        one, _ = run_decoder(model, ids[b:b + 1], P, T, True, **kw)
        torch.testing.assert_close(both[b:b + 1], one, rtol=2e-2, atol=2e-2)


def test_installed_decode_op_matches_the_graph_decoder_and_tracks_reads():
    model = tiny_model(seed=7)
    P, T = 300, 12
    ids = torch.randint(0, 1000, (1, P + T + 1), generator=torch.Generator().manual_seed(5)).to(DEV)
    kw = dict(C=64, C_init=16, cap_keys=32.0, window=16, delta=float("inf"), summary_bits=32)

    def patched(budget):
        stats = install(model, "cluster_fused", capacity=512, budget=budget, **kw)
        with torch.no_grad():
            cache = model.alloc_cache(512)
            model.prefill(ids[:, :P], cache, chunk=128)
            out = torch.stack([model(ids[:, t:t + 1], cache, start_pos=t)[:, -1].float() for t in range(P, P + T)], 1)
        uninstall(model)
        return out, stats

    # at budget 1 every clustering reads every row, so the seam (fitted one token later) and the decoder agree
    want, _ = run_decoder(model, ids, P, T, False, mode="cluster", budget=1.0, **kw)
    got, stats = patched(1.0)
    torch.testing.assert_close(got, want, rtol=3e-2, atol=3e-2)
    assert stats.steps == T * 2 and stats.read_fraction > 0.99
    _, stats = patched(0.25)
    assert stats.steps == T * 2, stats.steps
    assert 0.25 < stats.read_fraction < 0.6, stats.read_fraction
    assert stats.kv_read_fraction > stats.read_fraction


def test_fused_dense_layers_match_the_module_by_module_forward():
    model = tiny_model(seed=9)
    P, T = 280, 16
    ids = torch.randint(0, 1000, (2, P + T + 1), generator=torch.Generator().manual_seed(6)).to(DEV)
    kw = dict(mode="cluster", budget=0.3, C=64, C_init=16, cap_keys=24.0, window=16, delta=float("inf"))
    plain, _ = run_decoder(model, ids, P, T, True, fused_dense=False, **kw)
    fused, dec = run_decoder(model, ids, P, T, True, **kw)
    assert dec.fused_dense
    torch.testing.assert_close(fused, plain, rtol=3e-2, atol=3e-2)


def test_recentring_between_graph_replays_keeps_budget_one_exact():
    """A small drift threshold makes heads recentre between replays (flags read without a synchronisation);
    at budget 1 every row is read whatever the clustering, so the logits must still equal dense attention."""
    model = tiny_model(seed=11)
    P, T = 200, 120
    ids = torch.randint(0, 1000, (1, P + T + 1), generator=torch.Generator().manual_seed(8)).to(DEV)
    dense, _ = run_decoder(model, ids, P, T, True, mode="dense")
    got, dec = run_decoder(model, ids, P, T, True, mode="cluster", budget=1.0, C=64, C_init=16, split_factor=2.0,
                           window=8, delta=0.002, check_every=4, summary_bits=8)
    # the two runs differ in the order of float32 sums inside the attention kernels; through the bf16 layers
    # that shows as a few units in the last place of a logit (0.03 at magnitude 4)
    torch.testing.assert_close(got, dense, rtol=2e-2, atol=5e-2)
    assert sum(i.rebuilds for i in dec.attn) > 0
    for i in dec.attn:
        end = int(i.end_dev[0])
        lab = i.labels.cpu()
        counts = torch.stack([torch.bincount(lab[k, 1:end].long(), minlength=64) for k in range(i.H_kv)])
        assert torch.equal(i.count.cpu(), counts.float())


def test_total_variation_distance_to_exact_attention_shrinks_to_zero_at_full_budget():
    from sparse_kv_reads_b200.long_gen_tvd import decode_logits, tvd
    model = tiny_model(seed=13)
    P, T = 400, 32
    ids = torch.randint(0, 1000, (1, P + T + 1), generator=torch.Generator().manual_seed(9)).to(DEV)
    exact = decode_logits(model, ids, P, T, mode="dense")
    kw = dict(mode="cluster", C=128, C_init=16, cap_keys=32.0, window=16)
    d = {b: tvd(decode_logits(model, ids, P, T, budget=b, **kw), exact) for b in (0.1, 0.5, 1.0)}
    assert d[1.0] < 0.02 and d[1.0] <= d[0.5] + 0.01 and d[0.5] <= d[0.1] + 0.01, d


def test_rotary_step_folded_into_the_selection_equals_the_separate_launch():
    """skv_select with a rope description: queries, the new K/V rows and the selection itself are bit-identical
    to skv_qk_rope_cache followed by a plain skv_select (two sequences, G = 2)."""
    from sparse_kv_reads_b200 import _lib
    from sparse_kv_reads_b200._lib import check, lib
    L = lib()
    g = torch.Generator().manual_seed(17)
    B, H, H_kv, d, n = 2, 4, 2, 128, 900
    cap = 912
    K = oc.clustered_keys(B * H_kv, cap, d, seed=5)[0].to(torch.bfloat16).to(DEV).view(B, H_kv, cap, d)
    V = torch.randn(B, H_kv, cap, d, generator=g).to(torch.bfloat16).to(DEV)
    heads = lambda t: t.view(B * H_kv, cap, d)
    ix = SphereIndexGraph(C=128, C_init=32, cap_keys=24.0, window=16, delta=math.inf, capacity=cap, budget=0.3)
    ix.prepare(heads(K), n, B * H)
    qkv = torch.randn(B, (H + 2 * H_kv) * d, generator=g).to(torch.bfloat16).to(DEV)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(DEV)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(DEV)
    ang = torch.outer(torch.arange(cap, dtype=torch.float64), 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float64) / d)))
    ang = torch.cat((ang, ang), -1)
    cos, sin = ang.cos().to(torch.bfloat16).to(DEV), ang.sin().to(torch.bfloat16).to(DEV)
    pos = torch.tensor([n], dtype=torch.long, device=DEV)
    n_dev = torch.tensor([n + 1], dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    # separate launches
    K1, V1 = K.clone(), V.clone()
    q1 = torch.empty(B * H, d, dtype=torch.bfloat16, device=DEV)
    check(L.skv_qk_rope_cache(qkv.data_ptr(), qw.data_ptr(), kw.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(),
                              0, q1.data_ptr(), K1.data_ptr(), V1.data_ptr(), B, H, H_kv, d, K1.stride(0), K1.stride(1),
                              K1.stride(2), 1e-6, st), "skv_qk_rope_cache")
    out1 = ix.step(q1, heads(K1), heads(V1), n_dev, insert=False).clone()
    w1, cnt1 = ix.wbuf.clone(), ix.cnt.clone()
    # folded
    K2, V2 = K.clone(), V.clone()
    q2 = torch.zeros(B * H, d, dtype=torch.bfloat16, device=DEV)
    rope = _lib.SkvRope(qkv.data_ptr(), qw.data_ptr(), kw.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(),
                        q2.data_ptr(), K2.data_ptr(), V2.data_ptr(), H, H_kv, K2.stride(0), K2.stride(1), K2.stride(2),
                        1e-6, 0)
    out2 = ix.step(q2, heads(K2), heads(V2), n_dev, insert=False, rope=rope).clone()
    assert torch.equal(q1, q2) and torch.equal(K1, K2) and torch.equal(V1, V2)
    assert not torch.equal(K2[:, :, n], K[:, :, n])                   # the row was written
    assert torch.equal(ix.wbuf, w1) and torch.equal(ix.cnt, cnt1) and torch.equal(out1, out2)


def test_head_reset_between_graph_replays_keeps_budget_one_exact():
    """reset_at: a head whose cluster count reaches the threshold is refitted between replays (the flag travels
    with the drift flags); at budget 1 every row is read whatever the clustering, so the logits still equal
    dense attention, and the counts still match the labels."""
    model = tiny_model(seed=12)
    P, T = 260, 100
    ids = torch.randint(0, 1000, (1, P + T + 1), generator=torch.Generator().manual_seed(9)).to(DEV)
    dense, _ = run_decoder(model, ids, P, T, True, mode="dense")
    got, dec = run_decoder(model, ids, P, T, True, mode="cluster", budget=1.0, C=64, C_init=8, cap_keys=12.0,
                           reset_at=30, window=8, delta=float("inf"), check_every=2, summary_bits=8)
    torch.testing.assert_close(got, dense, rtol=2e-2, atol=5e-2)
    assert sum(i.resets for i in dec.attn) > 0
    for i in dec.attn:
        end = int(i.end_dev[0])
        lab = i.labels.cpu()
        counts = torch.stack([torch.bincount(lab[k, 1:end].long(), minlength=64) for k in range(i.H_kv)])
        assert torch.equal(i.count.cpu(), counts.float())


@pytest.mark.parametrize("opts", [dict(C_init=8, split_factor=1.1, grow_cap=True), dict(C_init=8, var_factor=0.9, var_min=4)])
def test_growing_cap_and_spread_trigger_in_the_all_layer_insert(opts):
    """The options that bound or redirect the splitting travel through the one insert launch of all layers: the
    clusters split during decode, the counts match the labels, and at budget 1 the logits equal dense attention."""
    model = tiny_model(seed=14)
    P, T = 260, 120
    ids = torch.randint(0, 1000, (1, P + T + 1), generator=torch.Generator().manual_seed(10)).to(DEV)
    dense, _ = run_decoder(model, ids, P, T, True, mode="dense")
    got, dec = run_decoder(model, ids, P, T, True, mode="cluster", budget=1.0, C=128, window=8, delta=float("inf"),
                           summary_bits=8, **opts)
    torch.testing.assert_close(got, dense, rtol=2e-2, atol=5e-2)
    assert dec.insert_all is not None and sum(i.splits for i in dec.attn) > 0
    for i in dec.attn:
        end = int(i.end_dev[0])
        lab = i.labels.cpu()
        counts = torch.stack([torch.bincount(lab[k, 1:end].long(), minlength=128) for k in range(i.H_kv)])
        assert torch.equal(i.count.cpu(), counts.float()) and i.check_status() == 0


@pytest.mark.parametrize("mode", ["cluster", "dense"])
def test_a_batch_of_different_lengths_equals_separate_sequences(mode):
    """Three sequences with prompts of 300, 217 and 260 tokens decode in one batch - every head reads its own
    sequence's length and position from device memory - and give what three separate decoders give; the graph
    replay equals the eager step bit for bit."""
    model = tiny_model(seed=21)
    lengths, T = [300, 217, 260], 24
    g = torch.Generator().manual_seed(14)
    ids = [torch.randint(0, 1000, (n + T + 1,), generator=g).to(DEV) for n in lengths]
    kw = dict(mode=mode, budget=0.3, C=64, C_init=16, cap_keys=24.0, window=16, delta=0.03, summary_bits=8)
    cap = -(-(max(lengths) + T + 2) // 16) * 16

    def ragged(capture):
        cache = model.alloc_cache(cap, max_batch=3)
        out = []
        with torch.no_grad():
            model.prefill_ragged([x[:n] for x, n in zip(ids, lengths)], cache, chunk=128)
            dec = GraphDecoder(model, cache, **kw)
            dec.prepare(lengths)
            if capture:
                dec.capture()
            for t in range(T):
                tok = torch.stack([x[n + t] for x, n in zip(ids, lengths)]).view(3, 1)
                out.append(dec.step(tok, [n + t for n in lengths])[:, -1].float().clone())
        return torch.stack(out, 1), dec

    both, dec = ragged(True)
    eager, _ = ragged(False)
    assert torch.equal(both, eager)
    assert dec.cache.cur_len == [n + T for n in lengths]
    for b, n in enumerate(lengths):
        one, _ = run_decoder(model, ids[b].view(1, -1), n, T, True, **kw)
        # the batch and the single sequence run different products (batch 3 against batch 1), so a logit may land
        # one bf16 step apart: 0.0156 for a logit of magnitude 2-4, 0.031 for 4-8
        torch.testing.assert_close(both[b:b + 1], one, rtol=2e-2, atol=4e-2)
    if mode == "cluster":
        for a in dec.attn:
            ends = a.end_dev.cpu().tolist()
            # (between steps the state already holds the insert of the step to come: one key more)
            assert ends == [n + T + int(dec.insert_ahead) - 16 for n in lengths for _ in range(2)]
            lab = a.labels.cpu()
            for k, e in enumerate(ends):
                counts = torch.bincount(lab[k, 1:e].long(), minlength=64)
                assert torch.equal(a.count[k].cpu(), counts.float())
                assert torch.all(lab[k, e:] == 64)
            assert a.check_status() in (0, 1)
