"""Device-resident cluster state of one attention layer and the per-step calls on it.

Host-side mirror of the reference's state objects for this path, collapsed into one class with the
reference's names: ``SphereIndexGPU`` (ssa/attn/sphere_gpu.py:113-442), ``SphereIndexFused``
(ssa/kernels/sphere_fused.py:316-518) and ``SphereIndexGraph`` (ssa/kernels/graph_kernels.py:192-279).
Every computation is a call into the CUDA library through its C ABI; there is no PyTorch fallback.
Built: the k-means and fixed-random-direction partitions, the shared selections (``sum_share``, ``max``, ``max_rel``) and ``per_head``, the size cap (fixed, or growing with
the context under ``grow_cap``), splits on the spread of a cluster (``var_factor``), the refit of a head
that ran out of clusters (``reset_at``) and recentring; the reference's other options raise ``ValueError``.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib
from ._lib import SkvState, check, dtype_code, lib, ptr, stream_ptr

GROUPS = {"sum_share": 0, "max": 1, "max_rel": 2}     # SKV_GROUP_* of the C ABI ("per_head" is G calls with "max")

# state arrays: name -> (trailing shape as a function of (C, d, capacity), dtype, fill value)
_FIELDS = {
    "sum_dir": (lambda C, d, cap: (C, d), torch.float32, 0.0),
    "cent": (lambda C, d, cap: (C, d), torch.float32, 0.0),
    "dir8": (lambda C, d, cap: (C, d), torch.int8, 0),
    "cent8": (lambda C, d, cap: (C, d), torch.int8, 0),
    "mmax": (lambda C, d, cap: (C,), torch.float32, 0.0),
    "mmin": (lambda C, d, cap: (C,), torch.float32, math.inf),
    "count": (lambda C, d, cap: (C,), torch.float32, 0.0),
    "n_c": (lambda C, d, cap: (), torch.int32, 0),
    "cap": (lambda C, d, cap: (), torch.float32, math.inf),
    "vthr": (lambda C, d, cap: (), torch.float32, math.inf),
    "rbar": (lambda C, d, cap: (), torch.float32, 0.0),
    "ksum": (lambda C, d, cap: (d,), torch.float32, 0.0),
    "mu_ref": (lambda C, d, cap: (d,), torch.float32, 0.0),
    "flags": (lambda C, d, cap: (), torch.int32, 0),
    "status": (lambda C, d, cap: (), torch.int32, 0),
    "nsplit": (lambda C, d, cap: (), torch.int32, 0),
    "end_dev": (lambda C, d, cap: (), torch.int32, 1),
    "need_dev": (lambda C, d, cap: (), torch.int32, 0),
    "labels": (lambda C, d, cap: (cap,), torch.int16, None),       # filled with C
}
_STRUCT_NAME = {"end_dev": "end", "need_dev": "need"}

_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Grow-only scratch buffer per device for the prompt fit (never used inside a graph)."""
    key = str(device)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        _workspaces[key] = buf = None
        buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def release_workspaces() -> None:
    """Free the fit scratch buffers (they can be several GB after a long prompt)."""
    _workspaces.clear()


class ClusterArena:
    """State arrays of ``layers`` layers x ``h`` heads stacked over layers, so that one insertion
    launch covers the whole model (the stacking ssa/kernels/graph_kernels.py:296-314 does after the
    fact is the allocation layout here)."""

    def __init__(self, *, layers: int, h: int, C: int, d: int, capacity: int, summary_bits: int, device):
        if capacity % 8:
            raise ValueError("capacity must be a multiple of 8 (labels are read in 16-byte vectors)")
        self.layers, self.h, self.C, self.d, self.capacity = layers, h, C, d, capacity
        self.summary_bits, self.device = summary_bits, device
        self.t: dict[str, torch.Tensor] = {}
        for name, (shape, dt, fill) in _FIELDS.items():
            if summary_bits == 32 and name in ("dir8", "cent8"):
                continue
            full = (layers * h, *shape(C, d, capacity))
            self.t[name] = torch.full(full, C if fill is None else fill, dtype=dt, device=device)

    def views(self, layer: int) -> dict[str, torch.Tensor]:
        return {k: v[layer * self.h:(layer + 1) * self.h] for k, v in self.t.items()}

    def struct(self, lo: int, hi: int) -> SkvState:
        """``skv_state`` over entries ``[lo, hi)`` of the stacked arrays."""
        s = SkvState()
        s.heads, s.C, s.d, s.capacity, s.summary_bits = hi - lo, self.C, self.d, self.capacity, self.summary_bits
        for name, t in self.t.items():
            setattr(s, _STRUCT_NAME.get(name, name), t[lo:hi].data_ptr())
        if self.summary_bits == 32:
            s.dir8 = s.cent8 = None
        return s


def fit_layers(layers: list["SphereIndexGraph"], caches: list[torch.Tensor], n: int,
               max_workspace: int = 6 << 30) -> bool:
    """Fit the states of several layers that share one arena with ONE ``skv_fit`` call per group of layers
    (as many layers as fit ``max_workspace`` bytes of scratch): the k-means passes and every round of the
    after-fit splits run once for the whole group, and the host waits once per round instead of once per
    round and layer.  Returns False (nothing done) when the layers cannot be batched."""
    first = layers[0]
    if len(layers) < 2 or first._arena is None or first.partition != "kmeans":
        return False
    k0 = caches[0]
    if any(k.stride() != k0.stride() or k.dtype != k0.dtype or k.shape != k0.shape for k in caches):
        return False
    for ix, K in zip(layers, caches):
        ix._init(K, n, fit=False)
    arena, h = first._arena, first.H_kv
    if any(ix._arena is not arena or ix._layer != i or ix.H_kv != h for i, ix in enumerate(layers)):
        for ix, K in zip(layers, caches):                   # not one stacked arena: layer by layer
            ix._build_all(K, n)
            ix.n = n
        return True
    m = first.end - 1
    if m < 1:
        return False
    L = lib()
    per_layer = L.skv_fit_workspace_bytes(h, m, first.C, first.d)
    group = max(1, min(len(layers), max_workspace // max(per_layer, 1)))
    g = torch.Generator(device="cpu").manual_seed(first.seed)
    init = torch.randperm(m, generator=g)[torch.arange(first.C_init) % m].to(torch.int32).to(k0.device)
    for lo in range(0, len(layers), group):
        hi = min(lo + group, len(layers))
        st = arena.struct(lo * h, hi * h)
        table = torch.tensor([k.data_ptr() for k in caches[lo:hi]], dtype=torch.int64, device=k0.device)
        nbytes = L.skv_fit_workspace_bytes((hi - lo) * h, m, first.C, first.d)
        ws = _workspace(k0.device, nbytes)
        check(L.skv_fit(ctypes.byref(st), None, dtype_code(k0.dtype), k0.stride(0), k0.stride(1), n, first.window,
                        first.C_init, first.kmeans_iters, init.data_ptr(), first.cap_keys, first.split_factor,
                        first.capk, first.var_factor, None, 0, table.data_ptr(), h, ws.data_ptr(), ws.numel(),
                        stream_ptr(k0.device)), "skv_fit")
    for ix in layers:
        ix._fitted = True
        ix._max_members = None
        ix._splits_host += int(ix.nsplit.sum())
        ix.nsplit.zero_()
        ix.n = n
    return True


def fit_layers_ragged(layers: list["SphereIndexGraph"], caches: list[torch.Tensor], lengths: list[int],
                      heads_per_seq: int) -> None:
    """Prompt fit of a batch whose sequences differ in length: one ``skv_fit`` per sequence, over the heads of that
    sequence in EVERY layer (a head list into the stacked states plus the table of per-layer caches), each with
    its own number of cached positions.  The layers must share one arena (``GraphDecoder`` allocates them so)."""
    first = layers[0]
    arena, h = first._arena, caches[0].shape[0]
    k0 = caches[0]
    if first.partition != "kmeans" or any(ix._arena is not arena or ix._layer != i for i, ix in enumerate(layers)):
        raise ValueError("a variable-length batch needs the k-means partition and layers stacked in one arena")
    if len(lengths) * heads_per_seq != h:
        raise ValueError("one length per sequence is needed")
    for ix, K in zip(layers, caches):
        ix._init(K, max(lengths), fit=False)
        ix.n_group = heads_per_seq
    L = lib()
    st = arena.struct(0, len(layers) * h)
    table = torch.tensor([k.data_ptr() for k in caches], dtype=torch.int64, device=k0.device)
    for b, n in enumerate(lengths):
        m = max(1, n - first.window) - 1
        if m < 1:
            raise ValueError(f"sequence {b}: n={n} leaves nothing to cluster behind a window of {first.window}")
        g = torch.Generator(device="cpu").manual_seed(first.seed)
        init = torch.randperm(m, generator=g)[torch.arange(first.C_init) % m].to(torch.int32).to(k0.device)
        hl = torch.tensor([layer * h + b * heads_per_seq + j for layer in range(len(layers))
                           for j in range(heads_per_seq)], dtype=torch.int32, device=k0.device)
        nbytes = L.skv_fit_workspace_bytes(int(hl.numel()), m, first.C, first.d)
        ws = _workspace(k0.device, nbytes)
        check(L.skv_fit(ctypes.byref(st), None, dtype_code(k0.dtype), k0.stride(0), k0.stride(1), n, first.window,
                        first.C_init, first.kmeans_iters, init.data_ptr(), first.cap_keys, first.split_factor,
                        first.capk, first.var_factor, hl.data_ptr(), int(hl.numel()), table.data_ptr(), h,
                        ws.data_ptr(), ws.numel(), stream_ptr(k0.device)), "skv_fit")
    for ix in layers:
        ix._fitted = True
        ix._max_members = None
        ix._splits_host += int(ix.nsplit.sum())
        ix.nsplit.zero_()
        ix.n = max(lengths)
        ix._host_end()


class AttentionPartials:
    """What ``skv_step`` leaves when the last merge is deferred: per head ``clusters`` partial outputs in
    ``workspace`` ([heads, clusters, G, 132] float32) and the buffer that is to receive the rows read."""

    def __init__(self, workspace: torch.Tensor, clusters: int, G: int, cnt: torch.Tensor):
        self.workspace, self.clusters, self.G, self.cnt = workspace, clusters, G, cnt


class SphereIndexGraph:
    """Cluster state of one layer for ``h`` (sequence, KV head) pairs, with the eager calls
    (``observe``, ``labels_and_weights``, ``attend``) and the graph-safe ones (``prepare``, ``step``,
    ``after_replay``)."""

    def __init__(self, *, budget: float = 0.2, C: int = 256, window: int = 64, delta: float = 0.03,
                 capacity: int = 65536, check_every: int = 16, seed: int = 0, kind: str = "random",
                 partition: str = "kmeans", kmeans_iters: int = 10, C_init: int | None = None,
                 split_factor: float = 0.0, grow_cap: bool = False, reset_at: int = 0, cap_keys: float = 0.0,
                 var_factor: float = 0.0, var_min: int = 8, async_check: bool = True, max_lag: int = 2,
                 split_scratch: int = 8192, summary_bits: int = 8, block_n: int = 32, compact_block: int = 1024,
                 refit_every: int = 0, arena: ClusterArena | None = None, layer: int = 0,
                 split_after_rebin: bool = True):
        if partition not in ("kmeans", "random"):
            raise ValueError(f"unknown partition {partition!r}")
        if partition == "random" and kind != "random":
            raise ValueError(f"direction kind {kind!r} is not built (only 'random')")
        if summary_bits not in (8, 32):
            raise ValueError("summary_bits must be 8 or 32")
        assert C >= 16 and C & (C - 1) == 0, "C must be a power of two >= 16"
        self.partition, self.kmeans_iters, self.kind = partition, kmeans_iters, kind
        self.C_init = C if C_init is None else C_init
        self.cap_keys = float(cap_keys)
        self.split_factor = float(split_factor) if split_factor or not cap_keys else 2.0
        self.var_factor = float(var_factor)
        self.splitting = self.split_factor > 0 or self.var_factor > 0
        # cap per clustered key when the cap follows the context (ssa/attn/sphere_gpu.py:130)
        self.capk = self.split_factor / self.C_init if grow_cap else 0.0
        if partition == "random":                           # every slot is a fixed direction: no fit, no splits
            if self.splitting and (split_factor or var_factor or cap_keys):
                raise ValueError("C_init must be <= C, and splitting needs partition='kmeans'")
            self.C_init, self.split_factor, self.var_factor, self.capk, self.splitting = C, 0.0, 0.0, 0.0, False
        if self.C_init > C:
            raise ValueError("C_init must be <= C, and splitting needs partition='kmeans'")
        self.C, self.window, self.delta, self.capacity = C, window, delta, capacity
        self.check_every, self.seed, self.budget = check_every, seed, budget
        self.async_check, self.max_lag, self.split_scratch = async_check, max_lag, split_scratch
        self.summary_bits, self.refit_every = summary_bits, refit_every
        self.split_after_rebin = split_after_rebin
        self.reset_at, self.var_min = (int(reset_at) if self.splitting else 0), int(var_min)
        self.initialized = False
        self.n = 0
        self.start, self.end = 1, 0
        self.rebuilds = self.resets = self.refits = self.head_steps = 0
        self._steps = 0
        self._splits_host = 0
        self._arena, self._layer = arena, layer
        self._pending = None
        self._waited = 0
        self._ktab = {}
        self.G = None
        # heads that share one entry of the device-side lengths: 0 = all sequences equally long (one entry); a batch
        # of sequences of different lengths passes one entry per sequence and its KV heads per sequence here
        self.n_group = 0

    # ---- allocation ------------------------------------------------------------------------------
    def _alloc(self, h: int, d: int, device) -> None:
        if d != 128:
            raise ValueError("the kernels are built for head_dim 128")
        if self._arena is None:
            self._arena = ClusterArena(layers=1, h=h, C=self.C, d=d, capacity=self.capacity,
                                       summary_bits=self.summary_bits, device=device)
            self._layer = 0
        a = self._arena
        if (a.h, a.C, a.d, a.capacity) != (h, self.C, d, self.capacity):
            raise ValueError("the shared arena was laid out for a different shape")
        for name, t in a.views(self._layer).items():
            setattr(self, name, t)
        if self.summary_bits == 32:
            self.dir8 = self.cent8 = None
        self.H_kv, self.d, self.device, self.dtype = h, d, device, torch.float32
        self._st = a.struct(self._layer * h, (self._layer + 1) * h)
        self._n_scalar = torch.zeros(1, dtype=torch.int32, device=device)
        self._flags_host = torch.zeros(h, dtype=torch.int32).pin_memory() if device.type == "cuda" else None
        self.idx = torch.empty(h, self.capacity, dtype=torch.int32, device=device)
        self.cnt = torch.zeros(h, dtype=torch.int32, device=device)
        self.wbuf = torch.zeros(h, self.C + 1, dtype=torch.float32, device=device)
        self.wbuf[:, self.C] = 1.0
        self.selbits = torch.zeros(h, self.C // 32 + 1, dtype=torch.int32, device=device)
        self._attn_ws = None
        self._attn_kept, self._sel_kept = {}, {}
        self._sel_ws = None
        self._max_members = None
        self._step_ncl, self._step_ws = {}, {}

    def _members_limit(self) -> int:
        """Largest cluster the in-kernel split has to stage: one key over the largest cap."""
        if self._max_members is None:
            lim = lib().skv_insert_max_members()
            cap = float(self.cap.max()) if self.splitting else 0.0
            cap = max(cap, self.capk * self.capacity)
            if self.split_factor > 0 and not self.cap_keys and (self.refit_every or self.reset_at):
                # a cap derived from the clustered keys (split_factor * m / C_init) is raised by every refit of a
                # longer context; a captured insert launch keeps the size given here, so size it for a full cache
                cap = max(cap, self.split_factor * self.capacity / self.C_init)
            want = int(cap) + 2 if math.isfinite(cap) else 2
            if self.var_factor > 0 and not math.isfinite(cap):
                want = lim                                  # split on spread alone: no bound on a cluster's size
            self._max_members = max(2, min(lim, want))
        return self._max_members

    def _ktable(self, K: torch.Tensor) -> torch.Tensor:
        key = K.data_ptr()
        t = self._ktab.get(key)
        if t is None:
            t = torch.tensor([key], dtype=torch.int64, device=K.device)
            self._ktab = {key: t}
        return t

    @staticmethod
    def _check_cache(K: torch.Tensor) -> None:
        if K.dim() != 3 or K.stride(2) != 1:
            raise ValueError("the cache must be [heads, positions, d] with a unit last stride")

    # ---- prompt fit ------------------------------------------------------------------------------
    def _init(self, K: torch.Tensor, n: int, fit: bool = True) -> None:
        self._check_cache(K)
        if n > self.capacity:
            raise ValueError(f"n={n} exceeds capacity {self.capacity}")
        if not self.initialized or K.shape[0] != getattr(self, "H_kv", -1):
            self._alloc(K.shape[0], K.shape[2], K.device)
        self.start, self.end = 1, max(1, n - self.window)
        self._fitted = False
        self.labels.fill_(self.C)
        self.n_c.zero_()
        self.end_dev.fill_(self.end)
        if fit:
            self._build_all(K, n)
        self.initialized = True

    def _build_all(self, K: torch.Tensor, n: int, heads: torch.Tensor | None = None) -> None:
        """Fit every head (or only ``heads``) from positions [1, end)
        (ssa/attn/sphere_gpu.py:187-230, :302-391)."""
        m = self.end - 1
        if m < 1:
            return                                          # nothing to cluster yet: fitted on a later call
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        if self.partition == "random":
            # fixed unit directions, the same for every head (ssa/attn/sphere_skip.py:54-56,:67)
            x = torch.randn(self.C, self.d, generator=g, dtype=torch.float64)
            self.cent.copy_((x / x.norm(dim=1, keepdim=True)).float().to(K.device).expand(self.H_kv, -1, -1))
            init = None
        else:
            init = torch.randperm(m, generator=g)[torch.arange(self.C_init) % m].to(torch.int32).to(K.device)
        L = lib()
        hl = None if heads is None else heads.to(torch.int32).to(K.device)
        entries = self.H_kv if hl is None else int(hl.numel())
        nbytes = L.skv_fit_workspace_bytes(entries, m, self.C, self.d)
        ws = _workspace(K.device, nbytes)
        splits_kept = self.nsplit.clone() if hl is not None else None
        check(L.skv_fit(ctypes.byref(self._st), K.data_ptr(), dtype_code(K.dtype), K.stride(0), K.stride(1), n,
                        self.window, self.C_init, self.kmeans_iters, ptr(init), self.cap_keys,
                        self.split_factor, self.capk, self.var_factor,
                        None if hl is None else hl.data_ptr(), entries, None, 0, ws.data_ptr(), ws.numel(),
                        stream_ptr(K.device)), "skv_fit")
        self._fitted = True
        self._max_members = None
        if hl is None:
            self._splits_host += int(self.nsplit.sum())
            self.nsplit.zero_()
        else:                                               # the fit restarted the listed heads' counters
            idx = hl.long()
            self._splits_host += int(splits_kept[idx].sum()) + int(self.nsplit[idx].sum())
            self.nsplit[idx] = 0

    # ---- per-step maintenance (eager: lengths known on the host) -----------------------------------
    def observe(self, K: torch.Tensor, n: int) -> None:
        """Bring the state up to ``n`` cached positions of ``K [h, >=n, d]`` (sphere_gpu.py:393-399)."""
        if not self.initialized or n < self.n or K.shape[0] != getattr(self, "H_kv", -1):
            self._init(K, n)
        elif n > self.n:                                    # the same length again: nothing arrived, no step counted
            self._advance(K, n)
        self.n = n

    def _launch_insert(self, K: torch.Tensor, n_dev: torch.Tensor, budget: float) -> None:
        check(lib().skv_insert(ctypes.byref(self._st), self._ktable(K).data_ptr(), self.H_kv, dtype_code(K.dtype),
                               K.stride(0), K.stride(1), n_dev.data_ptr(), self.n_group, self.window, float(budget),
                               float(min(self.delta, 3.0e38)), self.reset_at, self._members_limit(), self.capk,
                               self.var_min, stream_ptr(K.device)),
              "skv_insert")

    def _advance(self, K: torch.Tensor, n: int) -> None:
        self._check_cache(K)
        if n > self.capacity:
            raise ValueError(f"n={n} exceeds capacity {self.capacity}")
        new_end = max(1, n - self.window)
        if not self._fitted:
            if new_end > self.end:                          # nothing was clustered at the first build
                self.end = new_end
                self.end_dev.fill_(self.end)
                self._build_all(K, n)
        elif new_end > self.end:
            self._n_scalar.fill_(n)
            self._launch_insert(K, self._n_scalar, self.budget)
            self.end = new_end
        self.head_steps += self.H_kv
        if self.end - 1 <= 0:
            return
        self._steps += 1
        if self._steps % self.check_every == 0:
            self._check_flags(K)

    # ---- recentring (host side, between steps) ------------------------------------------------------
    def _check_flags(self, K: torch.Tensor) -> None:
        """Read the drift flags and recentre the flagged heads.  With ``async_check`` the flags travel
        to pinned memory without a synchronisation and are acted on at a later check
        (protocol of ssa/kernels/sphere_fused.py:434-451)."""
        if not self.async_check:
            self._act_on(K, self.flags.cpu())
            self.flags.zero_()
            return
        if self._pending is not None:
            self._waited += 1
            if self._waited > self.max_lag and not self._pending.query():
                self._pending.synchronize()
            if self._pending.query():
                self._pending = None
                self._act_on(K, self._flags_host.clone())
        if self._pending is None:
            self._flags_host.copy_(self.flags, non_blocking=True)
            self._pending = torch.cuda.Event()
            self._pending.record()
            self._waited = 0
            self.flags.zero_()

    def _act_on(self, K: torch.Tensor, flags_host: torch.Tensor) -> None:
        """Refit the heads whose cluster count reached ``reset_at``; recentre the others that drifted
        (ssa/kernels/sphere_fused.py:453-457)."""
        reset = (flags_host & _lib.FLAG_RESET) != 0
        if bool(reset.any()):
            self._reset_heads(K, reset.nonzero().flatten())
        heads = (((flags_host & _lib.FLAG_DRIFT) != 0) & ~reset).nonzero().flatten()
        if heads.numel():
            self._rebuild(K, heads)

    def _reset_heads(self, K: torch.Tensor, heads: torch.Tensor) -> None:
        """Fit ``heads`` again from all their clustered keys, back to ``C_init`` clusters and then the
        after-fit splits (ssa/attn/sphere_gpu.py:283-293)."""
        self._host_end()
        for end, group in self._by_end(heads):
            if end < 2:
                continue
            self.end = end
            self._build_all(K, end + self.window, group)
            self.resets += int(group.numel())
        self.end = int(self._ends[0])

    def _host_end(self) -> None:
        """Refresh the host copies of ``end`` from the device (a synchronisation; only before host work): ``end``
        is the first head's, ``_ends`` every head's (they differ in a batch of sequences of different lengths)."""
        self._ends = self.end_dev.cpu().tolist()
        self.end = int(self._ends[0])

    def _by_end(self, heads: torch.Tensor):
        """``heads`` grouped by their number of clustered positions: ``[(end, heads with that end), ...]``."""
        ends = getattr(self, "_ends", None)
        if not ends or len(set(ends)) == 1:
            return [(self.end, heads)]
        groups: dict[int, list[int]] = {}
        for hd in heads.tolist():
            groups.setdefault(int(ends[hd]), []).append(hd)
        return [(e, torch.tensor(v, dtype=heads.dtype)) for e, v in sorted(groups.items())]

    def _rebuild(self, K: torch.Tensor, heads: torch.Tensor) -> None:
        """Recentre ``heads`` about their running mean and rebin their keys, centroids kept
        (ssa/attn/sphere_gpu.py:187-219 with the mean given; ssa/kernels/sphere_fused.py:459-464)."""
        self._host_end()
        L = lib()
        # clusters the new mean pushes over their cap are divided at once (split_after_rebin): the insert's
        # in-kernel split cannot stage a cluster much larger than the cap, so it would otherwise keep growing
        sf = self.split_factor if self.split_factor > 0 and self.split_after_rebin else 0.0
        for end, group in self._by_end(heads):              # one call per sequence length
            if end < 2:
                continue
            hl = group.to(torch.int32).to(K.device)
            nbytes = L.skv_fit_workspace_bytes(int(hl.numel()), end - 1, self.C, self.d)
            ws = _workspace(K.device, nbytes)
            check(L.skv_rebin(ctypes.byref(self._st), hl.data_ptr(), int(hl.numel()), end, K.data_ptr(),
                              dtype_code(K.dtype), K.stride(0), K.stride(1), sf, self.kmeans_iters, self.capk,
                              ws.data_ptr(), ws.numel(), stream_ptr(K.device)), "skv_rebin")
            self.rebuilds += int(hl.numel())
        self._max_members = None

    # ---- selection -------------------------------------------------------------------------------
    def _select(self, q: torch.Tensor, n_dev: torch.Tensor, *, shared_in=None, shared_out=None, e_out=None,
                listed: bool = True, group: str = "sum_share", rope=None) -> None:
        """Score and pick; with ``listed`` also build the ascending row list ``idx``/``cnt`` (otherwise
        ``cnt`` is zeroed and the label-driven attention kernel fills it)."""
        H, d = q.shape
        G = H // self.H_kv
        L = lib()
        if not q.is_contiguous():
            q = q.contiguous()
        if self._sel_ws is None or self._sel_G != G:
            kept = getattr(self, "_sel_kept", None)
            if kept is None:
                kept = self._sel_kept = {}
            if self._sel_ws is not None:
                kept[self._sel_G] = self._sel_ws
            self._sel_G = G
            self._sel_ws = kept.get(G)
            if self._sel_ws is None:
                self._sel_ws = torch.zeros(L.skv_select_workspace_bytes(self.H_kv, G, self.C), dtype=torch.uint8,
                                           device=q.device)
        check(L.skv_select(ctypes.byref(self._st), q.data_ptr(), dtype_code(q.dtype), G, n_dev.data_ptr(), self.n_group,
                           self.wbuf.data_ptr(), self.selbits.data_ptr(), self.idx.data_ptr() if listed else None,
                           self.idx.stride(0), self.cnt.data_ptr(), ptr(shared_in), ptr(shared_out), ptr(e_out),
                           self._sel_ws.data_ptr(), 1.0 / math.sqrt(d), GROUPS[group],
                           None if rope is None else ctypes.byref(rope), stream_ptr(q.device)), "skv_select")

    def labels_and_weights(self, q: torch.Tensor, *, n: int, budget: float, group: str = "sum_share",
                           shared_in=None, shared_out=None, e_out=None):
        """``labels [h, n]`` int16 (label ``C`` = always read) and the 0/1 weights ``w [h, C+1]``; also
        fills ``idx``/``cnt`` with the positions to read.  Persistent buffers, overwritten by the next
        call (ssa/attn/sphere_gpu.py:412-442, ssa/kernels/sphere_fused.py:466-492)."""
        if group not in GROUPS and group != "per_head":
            raise ValueError(f"unknown group mode {group!r}")
        self.need_dev.fill_(math.ceil(budget * (self.end - 1)) if self.end > 1 else 0)
        self._n_scalar.fill_(n)
        if group == "per_head":
            return self.labels[:, :n], self._per_head(q, None, None)[0]
        self._select(q, self._n_scalar, shared_in=shared_in, shared_out=shared_out, e_out=e_out, group=group)
        return self.labels[:, :n], self.wbuf

    def _per_head(self, q: torch.Tensor, K, V):
        """``group="per_head"``: every query head ranks the clusters by its own scores and reads its own rows
        (ssa/attn/sphere_gpu.py:431-432, ssa/kernels/sphere_fused.py:466-492).  One selection (and, with ``K``,
        one attention) per query head of the group, each with a single query head per KV head, for which the
        "max" ranking is the head's own score; ``idx``/``cnt`` are left holding the last head's rows.
        Returns ``(w [H, C+1], out [H, d] or None)``."""
        H, d = q.shape
        G = H // self.H_kv
        qg = q.view(self.H_kv, G, d)
        w = torch.empty(self.H_kv, G, self.C + 1, dtype=torch.float32, device=q.device)
        out = torch.empty(self.H_kv, G, d, dtype=q.dtype, device=q.device) if K is not None else None
        for g in range(G):
            one = qg[:, g].contiguous()
            self._select(one, self._n_scalar, group="max")
            w[:, g] = self.wbuf
            if K is not None:
                out[:, g] = self._attend(one, K, V)
        return w.view(H, self.C + 1), None if out is None else out.view(H, d)

    # ---- attention -------------------------------------------------------------------------------
    def _attend_buffers(self, q: torch.Tensor) -> int:
        H, d = q.shape
        G = H // self.H_kv
        if self._attn_ws is None or self.G != G:
            L = lib()
            kept = getattr(self, "_attn_kept", None)
            if kept is None:
                kept = self._attn_kept = {}
            if self._attn_ws is not None and self.G is not None:      # another group size was in use: keep its buffers
                kept[(self.G, self.out.dtype)] = (self._attn_ws, self.out, self.num_splits)
            self.G = G
            if (G, q.dtype) in kept:
                self._attn_ws, self.out, self.num_splits = kept[(G, q.dtype)]
            else:
                self.num_splits = L.skv_attend_splits(self.H_kv)
                nbytes = L.skv_attend_workspace_bytes(self.H_kv, G, d, self.num_splits)
                self._attn_ws = torch.zeros(nbytes, dtype=torch.uint8, device=q.device)
                self.out = torch.empty(H, d, dtype=q.dtype, device=q.device)
        return G

    def _attend(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *, dense_n=None, force_simple=False):
        """Attention over the listed rows ``idx[:cnt]`` (or over ``[0, dense_n)``)."""
        H, d = q.shape
        if not q.is_contiguous():
            q = q.contiguous()
        G = self._attend_buffers(q)
        code = dtype_code(K.dtype) | (256 if force_simple else 0)
        check(lib().skv_attend(q.data_ptr(), K.data_ptr(), V.data_ptr(),
                               None if dense_n is not None else self.idx.data_ptr(),
                               None if dense_n is not None else self.cnt.data_ptr(), ptr(dense_n), self.n_group,
                               self.out.data_ptr(), self._attn_ws.data_ptr(), self.status.data_ptr(), self.H_kv, G, d,
                               code, K.stride(0), K.stride(1), V.stride(0), V.stride(1), self.idx.stride(0),
                               K.shape[1], self.num_splits, 1.0 / math.sqrt(d), stream_ptr(q.device)), "skv_attend")
        return self.out

    def _attend_labels(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, n_dev: torch.Tensor):
        """Attention over the rows whose label is selected in ``selbits``, read straight from the labels
        (no row list); adds the rows read to ``cnt``."""
        H, d = q.shape
        if not q.is_contiguous():
            q = q.contiguous()
        G = self._attend_buffers(q)
        check(lib().skv_attend_labels(q.data_ptr(), K.data_ptr(), V.data_ptr(), self.labels.data_ptr(),
                                      self.labels.stride(0), self.selbits.data_ptr(), self.C, n_dev.data_ptr(), self.n_group,
                                      self.out.data_ptr(), self._attn_ws.data_ptr(), self.cnt.data_ptr(),
                                      self.status.data_ptr(), self.H_kv, G, d, dtype_code(K.dtype), K.stride(0),
                                      K.stride(1), V.stride(0), V.stride(1), self.num_splits, 1.0 / math.sqrt(d),
                                      stream_ptr(q.device)), "skv_attend_labels")
        return self.out

    def _step_clusters(self, G: int) -> int:
        """Thread-block clusters per head for the one-launch step (``skv_step``), or 0 when the shape is served by
        the selection and attention launches instead (many heads, float32 summaries, large groups)."""
        got = self._step_ncl.get(G)
        if got is None:
            got = 0
            if self.summary_bits == 8 and os.environ.get("SKV_ONE_LAUNCH_STEP", "1") != "0":
                got = int(lib().skv_step_clusters(self.H_kv, G, self.C, self.summary_bits))
            self._step_ncl[G] = got
        return got

    def _step_one_launch(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, n_dev: torch.Tensor, rope, ncl: int,
                         defer_merge: bool = False):
        """Selection and attention in one launch (``skv_step``): fills ``wbuf``, ``selbits``, ``cnt`` and ``out``.
        ``defer_merge``: the clusters' partials stay in the workspace for the output product to merge
        (``skv_gemv_attended``); returns ``AttentionPartials`` instead of ``out``."""
        H, d = q.shape
        if not q.is_contiguous():
            q = q.contiguous()
        G = self._attend_buffers(q)
        ws = self._step_ws.get(G)
        if ws is None:
            ws = self._step_ws[G] = torch.zeros(lib().skv_step_workspace_bytes(self.H_kv, G, ncl), dtype=torch.uint8,
                                                device=q.device)
        check(lib().skv_step(ctypes.byref(self._st), q.data_ptr(), G, n_dev.data_ptr(), self.n_group, K.data_ptr(), V.data_ptr(),
                             K.stride(0), K.stride(1), V.stride(0), V.stride(1), self.wbuf.data_ptr(),
                             self.selbits.data_ptr(), self.cnt.data_ptr(), None if defer_merge else self.out.data_ptr(),
                             ws.data_ptr(), ncl, 1.0 / math.sqrt(d), None if rope is None else ctypes.byref(rope),
                             stream_ptr(q.device)),
              "skv_step")
        return AttentionPartials(ws, ncl, G, self.cnt) if defer_merge else self.out

    def _fused_rows(self, K: torch.Tensor) -> bool:
        """Whether the list-free attention applies (bf16 caches)."""
        return K.dtype == torch.bfloat16

    def attend(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *, n: int, budget: float,
               group: str = "sum_share"):
        """One eager decode step of this layer: update the clusters, select, attend over the selected
        rows.  ``K, V [h, >=n, d]`` in place.  Returns ``(out [H, d], labels, w)``
        (ssa/kernels/sphere_fused.py:494-501)."""
        self.observe(K, n)
        if group == "per_head":
            self.need_dev.fill_(math.ceil(budget * (self.end - 1)) if self.end > 1 else 0)
            self._n_scalar.fill_(n)
            w, out = self._per_head(q, K, V)
            return out, self.labels[:, :n], w
        labels, w = self.labels_and_weights(q, n=n, budget=budget, group=group)
        return self._attend(q, K, V), labels, w

    def attend_sampled(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *, n: int, budget: float, S: int,
                       alpha: float, generator: torch.Generator | None = None):
        """``attend`` plus ``S`` clusters drawn among the ones the selection left out; a drawn cluster is read in
        full and weighted ``draws / (S pi)`` (``tail_sample``), which keeps the attention sums unbiased.
        Returns ``(out [H, d], labels, w [h, C+1])`` (ssa/kernels/sphere_fused.py:503-518)."""
        from .tail_sample import proposal_from_scores, tail_sample_weights
        self.observe(K, n)
        H, d = q.shape
        G = H // self.H_kv
        if G > 8:
            raise ValueError("attend_sampled serves groups of at most 8 query heads")
        e = torch.empty(self.H_kv, G, self.C, dtype=torch.float32, device=q.device)
        labels, w = self.labels_and_weights(q, n=n, budget=budget, e_out=e)
        w2 = w.clone()
        if S > 0 and self.end > 1 and math.ceil(budget * (self.end - 1)) > 0:
            prop = proposal_from_scores(e, self.count, scale=1.0 / math.sqrt(d))
            w2[:, :self.C] = tail_sample_weights(prop, self.count, w[:, :self.C] > 0, S=S, alpha=alpha,
                                                 generator=generator)
        if not q.is_contiguous():
            q = q.contiguous()
        self._attend_buffers(q)
        self._n_scalar.fill_(n)
        check(lib().skv_attend_weighted(q.data_ptr(), K.data_ptr(), V.data_ptr(), self.labels.data_ptr(),
                                        self.labels.stride(0), w2.data_ptr(), self.C, self._n_scalar.data_ptr(), 0,
                                        self.out.data_ptr(), self._attn_ws.data_ptr(), self.status.data_ptr(),
                                        self.H_kv, G, d, dtype_code(K.dtype), K.stride(0), K.stride(1), V.stride(0),
                                        V.stride(1), self.num_splits, 1.0 / math.sqrt(d), stream_ptr(q.device)),
              "skv_attend_weighted")
        return self.out, labels, w2

    # ---- graph-safe calls --------------------------------------------------------------------------
    def prepare(self, K: torch.Tensor, n: int, H: int, fitted: bool = False, lengths: torch.Tensor | None = None) -> None:
        """Build from the prefilled cache holding ``n`` positions (eager) and allocate the step's fixed
        buffers (ssa/kernels/graph_kernels.py:204-218).  ``fitted``: ``fit_layers`` has built the state.
        ``lengths``: device int32 lengths, one per sequence, of a batch fitted by ``fit_layers_ragged``."""
        if lengths is None and not (fitted and self._fitted and self.n == n):
            self.observe(K, n)
        if not self._fitted:
            raise ValueError(f"n={n} leaves nothing to cluster behind a window of {self.window}")
        G = H // self.H_kv
        self.G = None
        q0 = torch.zeros(H, self.d, dtype=K.dtype, device=K.device)
        if lengths is not None:
            self._n_scalar = lengths.clone()                 # one entry per sequence (n_group heads each)
            self.need_dev.copy_(torch.ceil(self.budget * (self.end_dev - 1).double()).to(torch.int32))
        else:
            self._n_scalar.fill_(n)
            self.need_dev.fill_(math.ceil(self.budget * (self.end - 1)))
        self._select(q0, self._n_scalar)
        self._attend(q0, K, K)                               # sizes the workspaces and the output
        if self._fused_rows(K):
            self._select(q0, self._n_scalar, listed=False)
            self._attend_labels(q0, K, K, self._n_scalar)
            ncl = self._step_clusters(G) if q0.dtype == torch.bfloat16 else 0
            if ncl:                                          # configures the kernel ahead of any stream capture
                self._step_one_launch(q0, K, K, self._n_scalar, None, ncl)
        self._members_limit()
        self._ktable(K)
        assert self.G == G

    def step(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, n_dev: torch.Tensor, insert: bool = True,
             rope=None, defer_merge: bool = False):
        """One decode step with every length on the device; position ``n-1`` of ``K, V`` is already
        written.  ``insert=False`` when one launch inserted for all layers
        (ssa/kernels/graph_kernels.py:220-244)."""
        if insert:
            self._launch_insert(K, n_dev, self.budget)
        if self._fused_rows(K):
            # rope (an ``SkvRope``): the selection launch computes q from the raw projection, stores it to ``q``
            # and writes the token's K/V rows, in place of a separate launch ahead of it
            ncl = self._step_clusters(q.shape[0] // self.H_kv) if q.dtype == torch.bfloat16 else 0
            if ncl:                                          # few heads: selection and attention in one launch
                return self._step_one_launch(q, K, V, n_dev, rope, ncl, defer_merge)
            self._select(q, n_dev, listed=False, rope=rope)
            return self._attend_labels(q, K, V, n_dev)
        if rope is not None:
            raise ValueError("the folded rotary step needs the label-driven attention path (bf16 cache)")
        self._select(q, n_dev)
        return self._attend(q, K, V)

    def after_replay(self, K: torch.Tensor) -> None:
        """Between graph replays: every ``check_every`` steps look at the drift flags
        (ssa/kernels/graph_kernels.py:260-269)."""
        self.head_steps += self.H_kv
        self._steps += 1
        if self.refit_every and self._steps % self.refit_every == 0:
            self._refit(K)
        elif self._steps % self.check_every == 0:
            self._check_flags(K)

    def _refit(self, K: torch.Tensor) -> None:
        """Fit again on every clustered key with a fresh mean (graph_kernels.py:271-279)."""
        self._host_end()
        for end, group in self._by_end(torch.arange(self.H_kv)):
            self.end = end
            self.labels[group.to(self.labels.device), 1:end] = self.C
            self._build_all(K, end + self.window, group if len(set(self._ends)) > 1 else None)
        self.end = int(self._ends[0])
        self.flags.zero_()
        self._pending = None
        self.refits += 1

    # ---- bookkeeping ------------------------------------------------------------------------------
    @property
    def splits(self) -> int:
        """Clusters created by splitting (reads a device counter)."""
        return self._splits_host + (int(self.nsplit.sum()) if self.initialized else 0)

    @property
    def active_clusters(self) -> float:
        return float(self.n_c.float().mean()) if self.initialized else float(self.C)

    def _cap_now(self) -> torch.Tensor:
        """Each head's cap in keys; it grows with the clustered keys under ``grow_cap`` (sphere_gpu.py:270-273)."""
        return torch.clamp(self.cap, min=self.capk * (self.end - 1))

    def _spread(self) -> torch.Tensor:
        """Variance of each cluster's unit directions about their mean (sphere_gpu.py:276-279)."""
        return (1 - self.sum_dir.pow(2).sum(-1) / self.count.clamp_min(1).pow(2)).clamp_min(0) * (self.count > 0)

    # ---- checkpoint / resume --------------------------------------------------------------------------
    _HOST_FIELDS = ("n", "end", "rebuilds", "resets", "refits", "head_steps", "_steps", "_splits_host", "_fitted")

    def state_dict(self) -> dict:
        """Everything needed to resume decoding with this layer's clusters: the device arrays of the state
        (copied to the CPU) and the host counters.  The caller keeps the KV cache itself."""
        if not self.initialized:
            raise ValueError("nothing to save before the first observe()/prepare()")
        self._host_end()
        if self.end > 1:                                    # graph replays advance the device's end, not the host's n
            self.n = max(self.n, self.end + self.window)
        arrays = {name: getattr(self, name).detach().cpu().clone() for name in _FIELDS
                  if getattr(self, name, None) is not None}
        return {"arrays": arrays, "host": {k: getattr(self, k) for k in self._HOST_FIELDS},
                "shape": {"H_kv": self.H_kv, "d": self.d, "C": self.C, "capacity": self.capacity,
                          "summary_bits": self.summary_bits}}

    def load_state_dict(self, sd: dict, device) -> None:
        """Restore a state saved by ``state_dict`` onto ``device`` (the options given at construction must
        describe the same slot count, capacity and summary width)."""
        shp = sd["shape"]
        if (shp["C"], shp["capacity"], shp["summary_bits"]) != (self.C, self.capacity, self.summary_bits):
            raise ValueError("the saved state was built with a different C, capacity or summary_bits")
        self._alloc(shp["H_kv"], shp["d"], torch.device(device))
        for name, t in sd["arrays"].items():
            getattr(self, name).copy_(t)
        for k, v in sd["host"].items():
            setattr(self, k, v)
        self.initialized = True
        self._pending = None
        self._max_members = None

    def check_status(self) -> int:
        """OR of the device status words (synchronises); 0 means no device-side problem was recorded."""
        word = 0
        if self.initialized:
            for x in self.status.cpu().tolist():
                word |= int(x)
        return word


# the reference's intermediate class name
SphereIndexFused = SphereIndexGraph
