"""The attention entry point that owns its scratch memory (``skv_attend_static``) against the ordinary one.

Some hosts of this library cannot allocate device memory at the time they decode: a server that gave
all of HBM to its KV-cache pool at start-up, a decode loop that cannot afford the device-wide stall of
an allocation, a foreign-function caller without an allocator.  For them the library keeps the split
partials in an 8 MiB array of its own.  The test calls that entry point through the C ABI twice in a
row, with different shapes so that the second call finds the first one's leftovers in the array, and
wants the same output as ``skv_attend`` with a caller-provided workspace.  It runs last so that a run
which stops at the first failure has already been through every other test.
"""

from __future__ import annotations

import math

import pytest
import torch

from oracle import cluster_oracle as oc
from sparse_kv_reads_b200._lib import check, lib

pytestmark = pytest.mark.gpu


def both_ways(h, G, n, frac, splits, seed):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    K = torch.randn(h, n, 128, generator=g).to(torch.bfloat16)
    V = torch.randn(h, n, 128, generator=g).to(torch.bfloat16)
    q = (torch.randn(h * G, 128, generator=g) * 2).to(torch.bfloat16)
    rows = [torch.randperm(n, generator=g)[:max(1, int(frac * n))].sort().values for _ in range(h)]
    L = lib()
    Kd, Vd, qd = K.to(dev), V.to(dev), q.to(dev)
    idx = torch.zeros(h, n, dtype=torch.int32, device=dev)
    cnt = torch.zeros(h, dtype=torch.int32, device=dev)
    for i, r in enumerate(rows):
        idx[i, :len(r)] = r.to(torch.int32).to(dev)
        cnt[i] = len(r)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(128)
    common = (h, G, 128, 0, Kd.stride(0), Kd.stride(1), Vd.stride(0), Vd.stride(1), idx.stride(0), n, splits, scale,
              stream)
    ws = torch.zeros(L.skv_attend_workspace_bytes(h, G, 128, splits), dtype=torch.uint8, device=dev)
    want = torch.empty(h * G, 128, dtype=torch.bfloat16, device=dev)
    check(L.skv_attend(qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), idx.data_ptr(), cnt.data_ptr(), None, 0,
                       want.data_ptr(), ws.data_ptr(), None, *common), "skv_attend")
    got = torch.full_like(want, float("nan"))
    check(L.skv_attend_static(qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), idx.data_ptr(), cnt.data_ptr(), None, 0,
                              got.data_ptr(), None, *common), "skv_attend_static")
    torch.cuda.synchronize()
    ref = oc.attend_rows(q, K, V, rows)
    return got.cpu(), want.cpu(), ref


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    for h, G, n, frac, splits, seed in ((8, 2, 6000, 0.3, 37, 1), (3, 4, 2500, 0.5, 11, 2), (8, 2, 6000, 0.3, 37, 3)):
        got, want, ref = both_ways(h, G, n, frac, splits, seed)
        assert torch.isfinite(got.float()).all()
        assert float((got.double() - want.double()).abs().max()) <= 1e-2
        assert float((got.double() - ref).abs().max()) <= 1e-2
