"""Indexed-gather attention and merge kernels against the CPU oracle (through the C ABI)."""

from __future__ import annotations

import ctypes
import math

import pytest
import torch

from oracle import cluster_oracle as oc
from sparse_kv_reads_b200._lib import check, dtype_code, lib
from _helpers import DEV

pytestmark = pytest.mark.gpu


def run_attend(q, K, V, rows, *, splits=None, force_simple=False, dense_n=None, rows_limit=None):
    """Call skv_attend on host tensors; ``rows`` is a list of 1-D position tensors per head."""
    h, L, d = K.shape
    H = q.shape[0]
    G = H // h
    Lb = lib()
    qd, Kd, Vd = q.to(DEV), K.to(DEV), V.to(DEV)
    idx = torch.full((h, max(L, 8)), -7, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(h, dtype=torch.int32, device=DEV)
    if rows is not None:
        for i, r in enumerate(rows):
            idx[i, :len(r)] = r.to(torch.int32).to(DEV)
            cnt[i] = len(r)
    S = Lb.skv_attend_splits(h) if splits is None else splits
    ws = torch.zeros(Lb.skv_attend_workspace_bytes(h, G, d, S), dtype=torch.uint8, device=DEV)
    out = torch.full((H, d), float("nan"), dtype=q.dtype, device=DEV)
    status = torch.zeros(h, dtype=torch.int32, device=DEV)
    nd = None if dense_n is None else torch.tensor([dense_n], dtype=torch.int32, device=DEV)
    code = dtype_code(K.dtype) | (256 if force_simple else 0)
    for _ in range(2):            # twice: the ticket words must come back to zero
        check(Lb.skv_attend(qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), None if rows is None else idx.data_ptr(),
                            None if rows is None else cnt.data_ptr(), None if nd is None else nd.data_ptr(), 0,
                            out.data_ptr(), ws.data_ptr(), status.data_ptr(), h, G, d, code, Kd.stride(0),
                            Kd.stride(1), Vd.stride(0), Vd.stride(1), idx.stride(0),
                            L if rows_limit is None else rows_limit, S, 1.0 / math.sqrt(d),
                            torch.cuda.current_stream().cuda_stream), "skv_attend")
    torch.cuda.synchronize()
    return out.cpu(), status.cpu()


def make(h, n, G, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    K = torch.randn(h, n, 128, generator=g).to(dtype)
    V = torch.randn(h, n, 128, generator=g).to(dtype)
    q = (torch.randn(h * G, 128, generator=g) * 2).to(dtype)
    return q, K, V


def pick_rows(h, n, frac, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(h):
        k = max(1, int(round(frac * n)))
        out.append(torch.randperm(n, generator=g)[:k].sort().values)
    return out


TOL = {torch.bfloat16: 1e-2, torch.float32: 1e-5}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [1, 15, 16, 17, 63, 64, 65, 1000, 4097])
@pytest.mark.parametrize("G", [1, 2, 4])
def test_listed_rows_match_the_oracle(dtype, n, G):
    h = 3
    q, K, V = make(h, n, G, dtype, seed=n * 7 + G)
    rows = pick_rows(h, n, 0.3, seed=n)
    ref = oc.attend_rows(q, K, V, rows)
    out, status = run_attend(q, K, V, rows)
    assert int(status.abs().max()) == 0
    assert float((out.double() - ref).abs().max()) <= TOL[dtype]


@pytest.mark.parametrize("G", [8, 16])
def test_wide_groups_bf16(G):
    q, K, V = make(2, 700, G, torch.bfloat16, seed=G)
    rows = pick_rows(2, 700, 0.5, seed=3)
    out, _ = run_attend(q, K, V, rows)
    assert float((out.double() - oc.attend_rows(q, K, V, rows)).abs().max()) <= 1e-2


def test_both_bf16_paths_agree_and_every_split_count_works():
    q, K, V = make(4, 3000, 4, torch.bfloat16, seed=5)
    rows = pick_rows(4, 3000, 0.4, seed=6)
    ref = oc.attend_rows(q, K, V, rows)
    for S in (1, 2, 7, 64, 300):
        a, _ = run_attend(q, K, V, rows, splits=S)
        b, _ = run_attend(q, K, V, rows, splits=S, force_simple=True)
        assert float((a.double() - ref).abs().max()) <= 1e-2
        assert float((b.double() - ref).abs().max()) <= 1e-2


def test_unlisted_rows_are_never_read():
    """Rows that are not listed hold NaN; the output must stay finite and equal to the clean run
    (the idea of the reference's tests/test_labeled_triton.py:74-89)."""
    q, K, V = make(2, 900, 2, torch.bfloat16, seed=8)
    rows = pick_rows(2, 900, 0.2, seed=9)
    clean, _ = run_attend(q, K, V, rows)
    Kp, Vp = K.clone(), V.clone()
    for i, r in enumerate(rows):
        mask = torch.ones(900, dtype=torch.bool)
        mask[r] = False
        Kp[i, mask] = float("nan")
        Vp[i, mask] = float("nan")
    out, _ = run_attend(q, Kp, Vp, rows)
    assert torch.isfinite(out.float()).all() and torch.equal(out, clean)


def test_strided_cache_views_are_read_in_place():
    g = torch.Generator().manual_seed(10)
    big = torch.randn(2, 3, 520, 256, generator=g).to(torch.bfloat16)       # [.., head, pos, 2*d]
    K, V = big[0][:, :500, :128], big[1][:, :500, 128:]
    q = torch.randn(6, 128, generator=g).to(torch.bfloat16)
    rows = pick_rows(3, 500, 0.5, seed=11)
    h, H = 3, 6
    Lb = lib()
    bd = big.to(DEV)
    Kd, Vd = bd[0][:, :500, :128], bd[1][:, :500, 128:]
    idx = torch.zeros(h, 512, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(h, dtype=torch.int32, device=DEV)
    for i, r in enumerate(rows):
        idx[i, :len(r)] = r.to(torch.int32).to(DEV)
        cnt[i] = len(r)
    S = 5
    ws = torch.zeros(Lb.skv_attend_workspace_bytes(h, 2, 128, S), dtype=torch.uint8, device=DEV)
    out = torch.empty(H, 128, dtype=torch.bfloat16, device=DEV)
    check(Lb.skv_attend(q.to(DEV).data_ptr(), Kd.data_ptr(), Vd.data_ptr(), idx.data_ptr(), cnt.data_ptr(), None, 0,
                        out.data_ptr(), ws.data_ptr(), None, h, 2, 128, 0, Kd.stride(0), Kd.stride(1), Vd.stride(0),
                        Vd.stride(1), 512, 500, S, 1.0 / math.sqrt(128), torch.cuda.current_stream().cuda_stream),
          "skv_attend")
    ref = oc.attend_rows(q, K, V, rows)
    assert float((out.cpu().double() - ref).abs().max()) <= 1e-2


def test_dense_mode_and_bad_indices():
    q, K, V = make(2, 777, 2, torch.bfloat16, seed=12)
    full = [torch.arange(600) for _ in range(2)]
    out, _ = run_attend(q, K, V, None, dense_n=600)
    assert float((out.double() - oc.attend_rows(q, K, V, full)).abs().max()) <= 1e-2
    # a position beyond the limit is skipped and recorded, never dereferenced
    rows = [torch.tensor([0, 5, 9000, 20]), torch.tensor([1, 2, 3])]
    out, status = run_attend(q, K, V, rows)
    good = [torch.tensor([0, 5, 20]), torch.tensor([1, 2, 3])]
    assert float((out.double() - oc.attend_rows(q, K, V, good)).abs().max()) <= 1e-2
    assert status.tolist() == [4, 0]


def test_merge_matches_the_oracle_with_an_empty_split():
    g = torch.Generator().manual_seed(6)
    for S, G in ((1, 4), (18, 4), (72, 2)):
        m = torch.randn(8, S, G, generator=g) * 3
        m[:, 0, 0] = -1.0e30
        l = torch.rand(8, S, G, generator=g)
        a = torch.randn(8, S, G, 128, generator=g)
        ref = oc.merge_partials(m, l, a)
        out = torch.empty(8 * G, 128, device=DEV)
        md, ld, ad = m.to(DEV), l.to(DEV), a.to(DEV)
        check(lib().skv_merge(md.data_ptr(), ld.data_ptr(), ad.data_ptr(), out.data_ptr(), 8, S, G, 128,
                              torch.cuda.current_stream().cuda_stream), "skv_merge")
        if S > 1:
            torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)
