"""Host model on the CPU: chunked prefill equals one pass, decode equals prefill, and a two-rank
tensor-parallel run (gloo) reproduces the single-rank logits."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sparse_kv_reads_b200.qwen3 import Qwen3Config, Qwen3Model

TINY = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
            intermediate_size=96, vocab_size=200, max_position_embeddings=256)


def tiny(**kw):
    return Qwen3Model(Qwen3Config(**{**TINY, **kw})).eval().init_random(seed=3, std=0.1)


def test_chunked_prefill_and_decode_agree_with_one_pass():
    m = tiny()
    ids = torch.randint(0, 200, (2, 40), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        full = m(ids, m.alloc_cache(64, 2))
        c2 = m.alloc_cache(64, 2)
        last = m.prefill(ids[:, :32], c2, chunk=8)
        torch.testing.assert_close(last[:, 0], full[:, 31], rtol=1e-4, atol=1e-4)
        for t in range(32, 40):
            step = m(ids[:, t:t + 1], c2, start_pos=t)
            torch.testing.assert_close(step[:, 0], full[:, t], rtol=1e-4, atol=1e-4)
    assert c2.cur_len == 40 and m.lm_head is None and m.cfg.num_key_value_heads == 2


def test_install_sets_and_clears_the_decode_op():
    from sparse_kv_reads_b200.patch import ReadStats, install, uninstall
    m = tiny()
    stats = install(m, "cluster_fused", budget=0.2, C=64)
    assert isinstance(stats, ReadStats) and all(l.attn.decode_attn_op is not None for l in m.layers)
    assert m.layers[0].attn.decode_attn_op.index.C == 64 and stats.read_fraction == 1.0
    uninstall(m)
    assert all(l.attn.decode_attn_op is None for l in m.layers)
    with pytest.raises(ValueError):
        install(m, "santa", budget=0.2)


def _tp_worker(rank, world, port, ids, want):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = Qwen3Model(Qwen3Config(**TINY), tp_group=dist.group.WORLD, tp_size=world, tp_rank=rank).eval()
        m.init_random(seed=3, std=0.1)
        assert m.cfg.num_key_value_heads == 1 and m.lm_head.weight.shape[0] == 100
        with torch.no_grad():
            cache = m.alloc_cache(64, 2)
            got = m(ids[:, :24], cache)
            torch.testing.assert_close(got, want[:, :24], rtol=1e-4, atol=1e-4)
            step = m(ids[:, 24:25], cache, start_pos=24)
            torch.testing.assert_close(step[:, 0], want[:, 24], rtol=1e-4, atol=1e-4)
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_matches_single_rank():
    ids = torch.randint(0, 200, (2, 25), generator=torch.Generator().manual_seed(1))
    m = Qwen3Model(Qwen3Config(**{**TINY, "tie_word_embeddings": True})).eval().init_random(seed=3, std=0.1)
    with torch.no_grad():
        want = m(ids, m.alloc_cache(64, 2))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_tp_worker, args=(2, port, ids, want), nprocs=2, join=True)
