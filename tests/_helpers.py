"""Helpers shared by the GPU parity tests: oracle state -> device state, seeded inputs."""

from __future__ import annotations

import torch

from oracle import cluster_oracle as oc
from sparse_kv_reads_b200.cluster_state import SphereIndexGraph

DEV = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")


def isotropic_stream(h, n, H, *, seed=0, dtype=torch.bfloat16):
    """Keys N(0, I) + 0.7, values N(0, I), queries 2 N(0, I): the stream of the reference's GPU tests
    (tests/test_sphere_fused.py:18-23), generated on the CPU so that it is the same everywhere."""
    g = torch.Generator().manual_seed(seed)
    K = (torch.randn(h, n, 128, generator=g) + 0.7).to(dtype)
    V = torch.randn(h, n, 128, generator=g).to(dtype)
    Q = (torch.randn(n, H, 128, generator=g) * 2).to(dtype)
    return Q, K, V


def device_index_from_oracle(st: oc.ClusterOracle, **kw) -> SphereIndexGraph:
    """A device index holding exactly the oracle's state."""
    ix = SphereIndexGraph(C=st.C, C_init=st.C_init, window=st.window, delta=st.delta, capacity=st.capacity,
                          check_every=st.check_every, cap_keys=st.cap_keys,
                          split_factor=st.split_factor if st.splitting and not st.cap_keys else 0.0,
                          summary_bits=st.summary_bits, **kw)
    ix._alloc(st.h, st.d, DEV)
    for name in ("sum_dir", "cent", "mmax", "mmin", "count", "cap", "vthr", "rbar", "ksum", "mu_ref", "labels"):
        getattr(ix, name).copy_(getattr(st, name))
    ix.n_c.copy_(st.n_c.to(torch.int32))
    if st.summary_bits == 8:
        ix.dir8.copy_(st.dir8)
        ix.cent8.copy_(st.cent8)
    ix.end_dev.fill_(st.end)
    ix.end, ix.n = st.end, st.n
    ix.initialized = ix._fitted = True
    return ix


def row_sets(ix: SphereIndexGraph):
    """Listed positions per head as Python sets, and the raw lists."""
    cnt = ix.cnt.cpu().tolist()
    idx = ix.idx.cpu()
    lists = [idx[i, :cnt[i]] for i in range(len(cnt))]
    return [set(l.tolist()) for l in lists], lists
