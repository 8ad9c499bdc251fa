"""CPU oracle for the clustered sparse KV-cache decode-attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch on the CPU, the algorithm of the reference project
(aaholmes/sparse-kv-reads, package ``ssa``).  It is the checker that the CUDA kernels are compared
with; nothing in the shipped package imports it.  Only the tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may call it.

Parity status: pinned.  ``tests/golden/make_golden.py`` ran the reference's own classes
(``ssa.attn.sphere_gpu.SphereIndexGPU``, ``ssa.attn.clusterkv.spherical_kmeans``,
``ssa.attn.labeled.label_weighted_attention``, ``ssa.attn.accounting``) on seeded inputs and stored
their outputs under ``tests/golden/``; ``tests/test_oracle_golden.py`` checks every function here
against those files.  The 8-bit summary mode (``summary_bits=8``) follows the reference's Triton
kernels (``ssa/kernels/sphere_fused.py``), which cannot run without a GPU: that mode is a
restatement only, "parity unpinned" beyond the float32 arithmetic it shares with the pinned path.

Layout conventions (the reference's): ``K, V [h, L, d]`` with ``h`` = sequences x KV heads, position 0
is never clustered, clustered positions are ``[1, end)`` with ``end = max(1, n - window)``, label ``C``
marks an always-read row, summaries are ``sum_dir`` (sum of unit directions), ``mmax``/``mmin`` (key
lengths about the reference mean) and ``count``.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

NEG = -1.0e30


# --------------------------------------------------------------------------------------------
# a1  cosine k-means of the prompt fit                         (ssa/attn/clusterkv.py:27-46)
# --------------------------------------------------------------------------------------------
def kmeans_init_positions(m: int, C: int, seed: int) -> torch.Tensor:
    """Positions of the starting centroids: a seeded CPU permutation of the ``m`` points, wrapped
    when ``C > m``; the same for every head (clusterkv.py:34-35)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randperm(m, generator=g)[torch.arange(C) % m]


def kmeans_cosine(X: torch.Tensor, C: int, iters: int, seed: int):
    """``X [h, m, d]`` (centred keys) -> ``assign [h, m]``, unit ``cent [h, C, d]``.
    Lloyd steps on cosine similarity; an empty cluster keeps its centroid (clusterkv.py:36-46)."""
    h, m, d = X.shape
    Xn = F.normalize(X, dim=-1)
    init = kmeans_init_positions(m, C, seed).expand(h, C)
    cent = torch.gather(Xn, 1, init.unsqueeze(-1).expand(h, C, d)).clone()
    for _ in range(iters):
        assign = torch.einsum("hmd,hcd->hmc", Xn, cent).argmax(-1)
        sums = torch.zeros(h, C, d, dtype=X.dtype).scatter_add_(1, assign.unsqueeze(-1).expand(h, m, d), Xn)
        cnt = torch.zeros(h, C, dtype=X.dtype).scatter_add_(1, assign, torch.ones_like(assign, dtype=X.dtype))
        cent = torch.where((cnt > 0).unsqueeze(-1), F.normalize(sums, dim=-1), cent)
    assign = torch.einsum("hmd,hcd->hmc", Xn, cent).argmax(-1)
    return assign, cent


# --------------------------------------------------------------------------------------------
# a3  partitions used by the splits               (ssa/attn/sphere_gpu.py:56-73 and :76-102)
# --------------------------------------------------------------------------------------------
def kway_partition(U: torch.Tensor, valid: torch.Tensor, k: torch.Tensor, iters: int) -> torch.Tensor:
    """Cosine k-means of each padded member set ``U [S, M, d]`` into ``k [S]`` parts, seeded with
    evenly spaced members (sphere_gpu.py:56-73).  Returns ``part [S, M]``."""
    S, M, d = U.shape
    N = int(k.max())
    j = torch.arange(N).unsqueeze(0)
    seeds = (j * valid.sum(1, keepdim=True) // k.unsqueeze(1)).clamp(max=M - 1)
    cent = U.gather(1, seeds.unsqueeze(-1).expand(S, N, d)).clone()
    unused = (j >= k.unsqueeze(1)).unsqueeze(1)
    wv = valid.to(U.dtype)
    for it in range(iters + 1):
        part = torch.einsum("smd,snd->smn", U, cent).masked_fill(unused, -math.inf).argmax(-1)
        if it == iters:
            return part
        sums = torch.zeros_like(cent).scatter_add_(1, part.unsqueeze(-1).expand(S, M, d), U * wv.unsqueeze(-1))
        cnt = torch.zeros(S, N, dtype=U.dtype).scatter_add_(1, part, wv)
        cent = torch.where((cnt > 0).unsqueeze(-1), F.normalize(sums, dim=-1), cent)


def bisect_partition(U: torch.Tensor, valid: torch.Tensor, min_share: float = 0.25, iters: int = 4) -> torch.Tensor:
    """Two-way split of each member set: 2-means started from the first member and the member least
    similar to it; if the smaller half would hold under ``min_share`` of the members the set is cut
    at the median projection on the line between the two centroids (sphere_gpu.py:76-102)."""
    S, M, d = U.shape
    cnt = valid.sum(1)
    far = torch.einsum("smd,sd->sm", U, U[:, 0]).masked_fill(~valid, math.inf).argmin(1)
    two = torch.stack([U[:, 0], U[torch.arange(S), far]], 1).clone()
    Uv = U * valid.to(U.dtype).unsqueeze(-1)
    for it in range(iters + 1):
        sim = torch.einsum("smd,sjd->smj", U, two)
        side = (sim[..., 1] > sim[..., 0]) & valid
        if it == iters:
            break
        s1 = (Uv * side.unsqueeze(-1)).sum(1)
        s0 = Uv.sum(1) - s1
        n1 = side.sum(1)
        two = torch.stack([torch.where((cnt - n1 > 0).unsqueeze(-1), F.normalize(s0, dim=-1), two[:, 0]),
                           torch.where((n1 > 0).unsqueeze(-1), F.normalize(s1, dim=-1), two[:, 1])], 1)
    n1 = side.sum(1)
    lopsided = (n1 < min_share * cnt) | (n1 > (1 - min_share) * cnt)
    proj = torch.einsum("smd,sd->sm", U, two[:, 1] - two[:, 0]).masked_fill(~valid, math.inf)
    order = proj.argsort(dim=1, stable=True)
    rank = torch.empty_like(order).scatter_(1, order, torch.arange(M).expand(S, M))
    upper = (rank >= (cnt // 2).unsqueeze(1)) & valid
    return torch.where(lopsided.unsqueeze(1), upper, side).long()


def fixed_directions(C: int, d: int, seed: int) -> torch.Tensor:
    """``C`` unit vectors uniform on the sphere, the same for every head: the bins of ``partition="random"``
    (ssa/attn/sphere_skip.py:54-56,:67 with ``kind="random"``)."""
    x = torch.randn(C, d, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)
    return (x / x.norm(dim=1, keepdim=True)).float()


def to_int8_direction(x: torch.Tensor) -> torch.Tensor:
    """8-bit copy of a direction: unit vector x 127, rounded half up (sphere_fused.py:394-396)."""
    return torch.floor(F.normalize(x, dim=-1) * 127 + 0.5).to(torch.int8)


# --------------------------------------------------------------------------------------------
# a2-a8, a11  cluster state                                      (ssa/attn/sphere_gpu.py:113-442)
# --------------------------------------------------------------------------------------------
class ClusterOracle:
    """Cluster state of one layer for ``h`` (sequence, KV head) pairs, k-means partition only.

    ``summary_bits=32`` is the reference's PyTorch path (sphere_gpu.py).  ``summary_bits=8`` adds the
    8-bit copies that the reference's kernels search and score with (sphere_fused.py:157-162,
    :189-205, :244-247)."""

    def __init__(self, *, C: int, C_init: int | None = None, window: int = 64, delta: float = 0.03,
                 capacity: int = 65536, check_every: int = 16, seed: int = 0, kmeans_iters: int = 10,
                 split_factor: float = 0.0, cap_keys: float = 0.0, summary_bits: int = 32, grow_cap: bool = False,
                 reset_at: int = 0, var_factor: float = 0.0, var_min: int = 8, partition: str = "kmeans"):
        if partition not in ("kmeans", "random"):
            raise ValueError(f"unknown partition {partition!r}")
        self.partition = partition
        self.C, self.C_init = C, (C if C_init is None else C_init)
        self.window, self.delta, self.capacity = window, delta, capacity
        self.check_every, self.seed, self.kmeans_iters = check_every, seed, kmeans_iters
        self.cap_keys = float(cap_keys)
        self.split_factor = float(split_factor) if split_factor or not cap_keys else 2.0   # sphere_gpu.py:123-124
        self.var_factor, self.var_min = float(var_factor), int(var_min)
        self.splitting = (self.split_factor > 0 or self.var_factor > 0) and partition == "kmeans"
        self.capk = self.split_factor / self.C_init if grow_cap else 0.0       # sphere_gpu.py:130
        self.reset_at = reset_at
        self.resets = 0
        self.summary_bits = summary_bits
        if partition == "random":                                   # every slot is a fixed direction: nothing to fit or split
            self.C_init, self.split_factor, self.var_factor, self.capk = C, 0.0, 0.0, 0.0
        if self.C_init > C:
            raise ValueError("C_init must be <= C")
        self.initialized = False
        self.n = self.end = 0
        self.splits = self.rebuilds = self.steps = 0

    # ---- state -------------------------------------------------------------------------
    def _alloc(self, h: int, d: int) -> None:
        C = self.C
        self.h, self.d = h, d
        self.cent = torch.zeros(h, C, d)
        self.sum_dir = torch.zeros(h, C, d)
        self.mmax = torch.zeros(h, C)
        self.mmin = torch.full((h, C), math.inf)
        self.count = torch.zeros(h, C)
        self.n_c = torch.full((h,), self.C_init, dtype=torch.long)
        self.cap = torch.full((h,), math.inf)
        self.vthr = torch.full((h,), math.inf)
        self.ksum = torch.zeros(h, d)
        self.mu_ref = torch.zeros(h, d)
        self.rbar = torch.zeros(h)
        self.flags = torch.zeros(h, dtype=torch.bool)
        self.fitted = torch.zeros(h, dtype=torch.bool)
        self.labels = torch.full((h, self.capacity), C, dtype=torch.int16)
        self.dir8 = self.cent8 = None
        if self.summary_bits == 8:
            self.dir8 = torch.zeros(h, C, d, dtype=torch.int8)
            self.cent8 = torch.zeros(h, C, d, dtype=torch.int8)

    def _refresh8(self) -> None:
        if self.dir8 is not None:                                   # sphere_fused.py:398-406
            self.dir8.copy_(to_int8_direction(self.sum_dir))
            self.cent8.copy_(to_int8_direction(self.cent))

    def nearest(self, Kr: torch.Tensor, heads: torch.Tensor, int8: bool = False):
        """Unit directions, lengths and nearest active centroid of centred keys ``Kr [len(heads), m, d]``
        (sphere_gpu.py:168-177).  ``int8``: the per-step insert of the 8-bit mode searches the un-normalised
        int8 centroids (sphere_fused.py:189-199, ``_dirs_arg`` :384-389); the prompt fit and the recentring
        rebuild are the float32 host path in both modes (``_build`` -> ``_bin``, sphere_fused.py:407-409), which
        the reference pins with "the host fit does not depend on the copies" (tests/test_quant8.py:49)."""
        mag = Kr.norm(dim=-1)
        Kn = Kr / mag.clamp_min(1e-12).unsqueeze(-1)
        used = int(self.n_c[heads].max())
        spare = torch.arange(used).unsqueeze(0) >= self.n_c[heads].unsqueeze(1)
        table = self.cent8.float() if int8 and self.cent8 is not None else self.cent
        m = Kr.shape[1]
        lab = torch.cat([torch.einsum("hmd,hcd->hmc", Kn[:, i:i + 4096], table[heads, :used])
                         .masked_fill(spare.unsqueeze(1), -math.inf).argmax(-1)
                         for i in range(0, m, 4096)], dim=1) if m else torch.zeros(len(heads), 0, dtype=torch.long)
        return Kn, mag, lab

    def _fold(self, Kr: torch.Tensor, heads: torch.Tensor, int8: bool = False) -> torch.Tensor:
        """Assign centred keys and add them to their clusters' summaries (sphere_gpu.py:166-185)."""
        Kn, mag, lab = self.nearest(Kr, heads, int8)
        flat = (lab + heads.unsqueeze(1) * self.C).reshape(-1)
        self.sum_dir.view(-1, self.d).index_add_(0, flat, Kn.reshape(-1, self.d))
        self.mmax.view(-1).scatter_reduce_(0, flat, mag.reshape(-1), reduce="amax")
        self.mmin.view(-1).scatter_reduce_(0, flat, mag.reshape(-1), reduce="amin")
        self.count.view(-1).index_add_(0, flat, torch.ones_like(mag).reshape(-1))
        return lab

    def _build(self, K: torch.Tensor, heads: torch.Tensor, mu: torch.Tensor | None) -> bool:
        """(Re)build ``heads`` from their clustered keys; fits centroids the first time
        (sphere_gpu.py:187-219).  Returns whether a fit happened."""
        Kb = K[heads, 1:self.end].float()
        nb = Kb.shape[1]
        if mu is None:
            mu = Kb.mean(1) if nb else torch.zeros(len(heads), self.d)
        self.sum_dir[heads] = 0
        self.mmax[heads] = 0
        self.mmin[heads] = math.inf
        self.count[heads] = 0
        self.mu_ref[heads] = mu
        self.ksum[heads] = Kb.sum(1)
        fresh = False
        if not nb:
            self.rbar[heads] = 0
            return False
        Kr = Kb - mu.unsqueeze(1)
        todo = ~self.fitted[heads]
        if todo.any():
            if self.partition == "random":                          # sphere_gpu.py:147, sphere_skip.py:54-67
                cent = fixed_directions(self.C, self.d, self.seed).expand(int(todo.sum()), -1, -1)
            else:
                _, cent = kmeans_cosine(Kr[todo], self.C_init, self.kmeans_iters, self.seed)
            self.cent[heads[todo], :self.C_init] = cent
            self.n_c[heads[todo]] = self.C_init
            self.fitted[heads[todo]] = True
            if self.split_factor > 0:
                self.cap[heads[todo]] = self.cap_keys or self.split_factor * nb / self.C_init
                fresh = True
            if self.cent8 is not None:
                self.cent8.copy_(to_int8_direction(self.cent))
        self.rbar[heads] = Kr.pow(2).sum(-1).mean(1).sqrt()
        self.labels[heads, 1:self.end] = self._fold(Kr, heads).to(torch.int16)
        if self.var_factor > 0 and bool(todo.any()):              # threshold from the fit's own clusters (:214-217)
            fit = heads[todo]
            used = (self.count[fit] > 0).float()
            self.vthr[fit] = self.var_factor * (self.spread()[fit] * used).sum(1) / used.sum(1).clamp_min(1)
        self._refresh8()
        return fresh

    def cap_now(self) -> torch.Tensor:
        """Each head's cap in keys; it grows with the clustered keys under ``grow_cap`` (sphere_gpu.py:270-273)."""
        return torch.clamp(self.cap, min=self.capk * (self.end - 1))

    def spread(self) -> torch.Tensor:
        """Variance of each cluster's unit directions about their mean (sphere_gpu.py:275-278)."""
        return (1 - self.sum_dir.pow(2).sum(-1) / self.count.clamp_min(1).pow(2)).clamp_min(0) * (self.count > 0)

    def reset_heads(self, K: torch.Tensor, heads: torch.Tensor) -> None:
        """Fit ``heads`` again from all their clustered keys, back to ``C_init`` clusters (sphere_gpu.py:283-293)."""
        if heads.numel() == 0:
            return
        self.fitted[heads] = False
        self.n_c[heads] = self.C_init
        if self._build(K, heads, None):
            self.split_overflow(K, None, kway=True)
        self.resets += int(heads.numel())

    # ---- splits ---------------------------------------------------------------------------
    def _split_group(self, K: torch.Tensor, hc: torch.Tensor, kway: bool) -> int:
        """Split up to 64 clusters ``hc [S, 2]`` (head, slot; ordered by head then slot) at once
        (sphere_gpu.py:340-391).  Spare slots are handed out in that order; a cluster whose run of
        new slots would pass ``C`` is left for a later round."""
        C, d = self.C, self.d
        hd, cl = hc[:, 0], hc[:, 1]
        S = hd.shape[0]
        member = self.labels[hd, 1:self.end] == cl.unsqueeze(1)
        cnt = member.sum(1)
        M = int(cnt.max())
        rows, cols = member.nonzero(as_tuple=True)
        rank = torch.arange(rows.shape[0]) - (cnt.cumsum(0) - cnt)[rows]
        pos = torch.zeros(S, M, dtype=torch.long)
        pos[rows, rank] = cols + 1
        valid = torch.arange(M).unsqueeze(0) < cnt.unsqueeze(1)
        Kr = K[hd.unsqueeze(1), pos].float() - self.mu_ref[hd].unsqueeze(1)
        mag = Kr.norm(dim=-1)
        U = Kr / mag.clamp_min(1e-12).unsqueeze(-1)
        if kway:
            k = torch.ceil(cnt * self.split_factor / self.cap_now()[hd]).long().clamp(min=2)
            part = kway_partition(U, valid, k, self.kmeans_iters)
        else:
            part = bisect_partition(U, valid)
        N = int(part.max()) + 1
        j = torch.arange(N).unsqueeze(0)
        sizes = torch.zeros(S, N, dtype=torch.long).scatter_add_(1, part, valid.long())
        part = ((sizes > 0).cumsum(1) - 1).gather(1, part)
        extra = (sizes > 0).sum(1) - 1
        per_head = torch.zeros(self.h, dtype=torch.long).index_add_(0, hd, extra)
        base = self.n_c[hd] + (extra.cumsum(0) - extra) - (per_head.cumsum(0) - per_head)[hd]
        keep = (extra > 0) & (base + extra <= C)
        if not bool(keep.any()):
            return 0
        slot = torch.where(j == 0, cl.unsqueeze(1), base.unsqueeze(1) + j - 1)
        tgt = (hd.unsqueeze(1) * C + slot)[keep.unsqueeze(1) & (j <= extra.unsqueeze(1))]
        sel = valid & keep.unsqueeze(1)
        hh = hd.unsqueeze(1).expand(S, M)[sel]
        new = slot.gather(1, part)[sel]
        flat = hh * C + new
        self.sum_dir.view(-1, d)[tgt] = 0
        self.mmax.view(-1)[tgt] = 0
        self.mmin.view(-1)[tgt] = math.inf
        self.count.view(-1)[tgt] = 0
        self.sum_dir.view(-1, d).index_add_(0, flat, U[sel])
        self.mmax.view(-1).scatter_reduce_(0, flat, mag[sel], reduce="amax")
        self.mmin.view(-1).scatter_reduce_(0, flat, mag[sel], reduce="amin")
        self.count.view(-1).index_add_(0, flat, torch.ones_like(mag[sel]))
        self.cent.view(-1, d)[tgt] = F.normalize(self.sum_dir.view(-1, d)[tgt], dim=-1)
        self.labels[hh, pos[sel]] = new.to(torch.int16)
        self.n_c.index_add_(0, hd[keep], extra[keep])
        self.splits += int(extra[keep].sum())
        self._touched[tgt] = True
        return int(keep.sum())

    def split_overflow(self, K: torch.Tensor, cand: torch.Tensor | None, kway: bool) -> None:
        """Split clusters over their head's cap until none is or no slot is left; ``cand [h, C]``
        limits the test to clusters that just received a key and to their pieces
        (sphere_gpu.py:307-338)."""
        if not self.splitting:
            return
        slots = torch.arange(self.C).unsqueeze(0)
        by_spread = cand is not None                  # a spread over the threshold splits once, on receiving a key
        while True:
            over = self.count > self.cap_now().unsqueeze(1)
            if by_spread:
                over |= (self.spread() > self.vthr.unsqueeze(1)) & (self.count >= self.var_min)
                by_spread = False
            over &= (slots < self.n_c.unsqueeze(1)) & (self.count >= 2)
            if cand is not None:
                over &= cand
            hc = over.nonzero()
            if hc.shape[0] == 0:
                break
            self._touched = torch.zeros(self.h * self.C, dtype=torch.bool)
            done = 0
            for i in range(0, hc.shape[0], 64):
                done += self._split_group(K, hc[i:i + 64], kway)
            if not done and not kway:
                break
            kway = False
            if cand is not None:
                cand = cand | self._touched.view(self.h, self.C)
        self._refresh8()

    # ---- per-step maintenance -----------------------------------------------------------------
    def observe(self, K: torch.Tensor, n: int) -> None:
        """Bring the state up to ``n`` cached positions of ``K [h, >=n, d]`` (sphere_gpu.py:393-399)."""
        if not self.initialized or n < self.n or K.shape[0] != getattr(self, "h", -1):
            if n > self.capacity:
                raise ValueError(f"n={n} exceeds capacity {self.capacity}")
            self._alloc(K.shape[0], K.shape[2])
            self.end = max(1, n - self.window)
            if self._build(K, torch.arange(self.h), None):
                self.split_overflow(K, None, kway=True)
            self.initialized = True
        else:
            self._advance(K, n)
        self.n = n

    def _advance(self, K: torch.Tensor, n: int) -> None:
        """Insert the keys that left the recent window, split, test the drift (sphere_gpu.py:232-263)."""
        new_end = max(1, n - self.window)
        heads = torch.arange(self.h)
        if new_end > self.end and not bool(self.fitted.all()):
            self.end = new_end
            if self._build(K, heads, None):
                self.split_overflow(K, None, kway=True)
        if new_end > self.end:
            Kn = K[:, self.end:new_end].float()
            self.ksum += Kn.sum(1)
            lab = self._fold(Kn - self.mu_ref.unsqueeze(1), heads, int8=True)
            self.labels[:, self.end:new_end] = lab.to(torch.int16)
            self.end = new_end
            if self.dir8 is not None:                               # sphere_fused.py:203-205
                self.dir8.copy_(to_int8_direction(self.sum_dir))
            if self.splitting:
                got = torch.zeros(self.h, self.C, dtype=torch.bool).scatter_(1, lab, True)
                self.split_overflow(K, got, kway=False)
                if self.reset_at:
                    self.reset_heads(K, (self.n_c >= self.reset_at).nonzero().squeeze(1))
        nb = self.end - 1
        if nb <= 0:
            return
        mu_t = self.ksum / nb
        self.flags |= (mu_t - self.mu_ref).norm(dim=1) > self.delta * self.rbar
        self.steps += 1
        if self.steps % self.check_every == 0:
            flagged = self.flags.nonzero().squeeze(1)
            if flagged.numel():
                self._build(K, flagged, mu_t[flagged])
                self.rebuilds += int(flagged.numel())
            self.flags.zero_()

    # ---- scoring and selection ----------------------------------------------------------------
    def need(self, budget: float) -> int:
        """Keys the selected clusters must hold: ceil(budget x clustered keys) (sphere_gpu.py:424)."""
        return math.ceil(budget * (self.end - 1))

    def scores(self, q: torch.Tensor) -> torch.Tensor:
        """Estimated largest logit of each cluster for each query head, ``e [h, G, C]``; empty clusters
        get -inf (sphere_gpu.py:426-430; 8-bit: sphere_fused.py:244-253)."""
        G = q.shape[0] // self.h
        src = self.sum_dir if self.dir8 is None else self.dir8.float()
        cdir = src / src.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        p = torch.einsum("hgd,hcd->hgc", q.view(self.h, G, self.d).float(), cdir)
        e = torch.where(p >= 0, self.mmax.unsqueeze(1) * p, self.mmin.unsqueeze(1) * p)
        return e.masked_fill((self.count == 0).unsqueeze(1), -math.inf)

    def shared_score(self, e: torch.Tensor, group: str = "sum_share") -> torch.Tensor:
        """One score per cluster for a group's query heads (sphere_gpu.py:431-439): the sum over the heads of
        each head's softmax over clusters (``sum_share``), the largest scaled score (``max``), or the largest
        score relative to its head's best cluster (``max_rel``)."""
        z = e * (1.0 / math.sqrt(self.d))
        if group == "max":
            return z.max(1).values
        if group == "max_rel":
            return (z - z.max(2, keepdim=True).values).max(1).values
        if group != "sum_share":
            raise ValueError(f"unknown group mode {group!r}")
        return torch.softmax(z, dim=2).sum(1).masked_fill(self.count == 0, -math.inf)

    @staticmethod
    def take_until(score: torch.Tensor, count: torch.Tensor, need: int) -> torch.Tensor:
        """Per row, clusters in decreasing score (equal scores: lower slot first) until their counts
        reach ``need``; the cluster that crosses it is included (sphere_gpu.py:402-410)."""
        R, C = score.shape
        order = torch.sort(score, dim=1, descending=True, stable=True).indices
        cum = count.gather(1, order).cumsum(1)
        n_sel = (cum < need).sum(1) + 1
        rank = torch.empty_like(order).scatter_(1, order, torch.arange(C).expand(R, C))
        return rank < n_sel.unsqueeze(1)

    def select(self, q: torch.Tensor, *, n: int, budget: float, group: str = "sum_share"):
        """``labels [h, n]`` and 0/1 weights ``w [h, C+1]`` (column ``C`` = always-read rows)
        for the shared group modes (sphere_gpu.py:412-442)."""
        need = self.need(budget)
        if group == "per_head":                                     # every query head ranks for itself (:431-432)
            G = q.shape[0] // self.h
            w = torch.zeros(q.shape[0], self.C + 1)
            w[:, self.C] = 1.0
            if self.end > 1 and need > 0:
                e = self.scores(q).reshape(q.shape[0], self.C)
                w[:, :self.C] = self.take_until(e, self.count.repeat_interleave(G, 0), need).float()
            return self.labels[:, :n], w
        w = torch.zeros(self.h, self.C + 1)
        w[:, self.C] = 1.0
        if self.end > 1 and need > 0:
            w[:, :self.C] = self.take_until(self.shared_score(self.scores(q), group), self.count, need).float()
        return self.labels[:, :n], w

    def select_sampled(self, q: torch.Tensor, *, n: int, budget: float, S: int, alpha: float,
                       generator: torch.Generator | None = None):
        """The selection plus ``S`` draws among the clusters it left out, as fractional weights
        (``attend_sampled``, ssa/kernels/sphere_fused.py:503-518).  Returns ``(labels, w [h, C+1])``."""
        labels, w = self.select(q, n=n, budget=budget)
        w = w.clone()
        if S > 0 and self.end > 1 and self.need(budget) > 0:
            prop = sampling_proposal(self.scores(q), self.count, scale=1.0 / math.sqrt(self.d))
            w[:, :self.C] = sampled_weights(prop, self.count, w[:, :self.C] > 0, S=S, alpha=alpha, generator=generator)
        return labels, w

    def positions(self, w: torch.Tensor, n: int) -> list[torch.Tensor]:
        """Ascending positions read per head: rows whose label has positive weight
        (the set that ssa/kernels/graph_kernels.py:144-155 lists, in position order)."""
        lab = self.labels[:, :n].long()
        return [(w[i][lab[i]] > 0).nonzero().squeeze(1) for i in range(self.h)]


# --------------------------------------------------------------------------------------------
# sampling the clusters that were not selected                    (ssa/attn/tail_sample.py:24-63)
# --------------------------------------------------------------------------------------------
def sampling_proposal(e: torch.Tensor, count: torch.Tensor, *, scale: float) -> torch.Tensor:
    """Probability of drawing each cluster, ``[h, C]``, rows summing to 1: per query head the estimated mass
    ``count x exp(scale x e)`` normalised over the clusters, then the mean over the group's query heads
    (``proposal_from_scores``, tail_sample.py:24-32).  ``e [h, G, C]`` with -inf for empty clusters."""
    z = e * scale
    z = z - z.amax(dim=2, keepdim=True)
    mass = torch.nan_to_num(count.unsqueeze(1) * z.exp(), nan=0.0)
    return (mass / mass.sum(dim=2, keepdim=True).clamp_min(1e-300)).mean(dim=1)


def sampled_weights(prop: torch.Tensor, count: torch.Tensor, taken: torch.Tensor, *, S: int, alpha: float,
                    generator: torch.Generator | None = None) -> torch.Tensor:
    """Cluster weights ``[h, C]`` when ``S`` of the clusters that were not taken are drawn by systematic sampling
    (``tail_sample_weights``, tail_sample.py:35-63): 1 for a taken, non-empty cluster; ``draws / (S x pi)`` for a
    drawn one, where ``pi`` mixes the proposal restricted to the rest with a uniform floor ``alpha``; 0 otherwise.
    One uniform number per head (drawn on the CPU from ``generator``) places the S equally spaced probes."""
    live = count > 0
    w_taken = (taken & live).to(prop.dtype)
    rest = live & ~taken
    if S <= 0:
        return w_taken
    n_rest = rest.sum(1, keepdim=True).clamp_min(1)
    p = prop * rest
    p = p / p.sum(1, keepdim=True).clamp_min(1e-300)
    pi = ((1 - alpha) * p + alpha / n_rest) * rest
    cdf = pi.cumsum(1)
    h, C = pi.shape
    u = torch.rand(h, 1, generator=generator, dtype=prop.dtype, device="cpu").to(prop.device) / S
    probes = (u + torch.arange(S, dtype=prop.dtype, device=prop.device) / S) * cdf[:, -1:]
    hit = torch.searchsorted(cdf.contiguous(), probes.contiguous()).clamp_(max=C - 1)
    draws = torch.zeros_like(prop).scatter_add_(1, hit, torch.ones_like(probes))
    draws = draws * rest.any(1, keepdim=True)
    w_drawn = torch.where(rest & (draws > 0), draws / (S * pi.clamp_min(1e-300)), torch.zeros_like(prop))
    return w_taken + w_drawn


# --------------------------------------------------------------------------------------------
# a9-a10  attention over the selected rows
# --------------------------------------------------------------------------------------------
def attend_labeled(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, labels: torch.Tensor, w: torch.Tensor,
                   dtype=torch.float64) -> torch.Tensor:
    """Softmax attention restricted to rows whose label weight is positive, dense masked form
    (ssa/attn/labeled.py:24-44 with shared weights).  ``q [H, d]``, ``K, V [h, n, d]`` -> ``[H, d]``."""
    H, d = q.shape
    h = K.shape[0]
    G = H // h
    if w.shape[0] == H and G > 1:                                   # one row of weights per query head
        wr = torch.gather(w.to(dtype), 1, labels.long().repeat_interleave(G, 0))
    else:
        wr = torch.gather(w.to(dtype), 1, labels.long()).repeat_interleave(G, 0)
    s = torch.einsum("hd,hnd->hn", q.to(dtype), K.to(dtype).repeat_interleave(G, 0)) / math.sqrt(d)
    logw = torch.where(wr > 0, wr.clamp_min(1e-300).log(), torch.full_like(wr, -math.inf))
    A = torch.softmax(s + logw, dim=-1)
    Vx = V.to(dtype).repeat_interleave(G, 0)
    Vx = torch.where((wr > 0).unsqueeze(-1), Vx, torch.zeros_like(Vx))
    return torch.einsum("hn,hnd->hd", A, Vx)


def attend_rows(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, rows: list[torch.Tensor],
                dtype=torch.float64) -> torch.Tensor:
    """The same attention written over explicit row lists (reads only the listed rows; used for
    long contexts where the dense masked form is too slow).  Equals ``attend_labeled`` on the
    same row set."""
    H, d = q.shape
    h = K.shape[0]
    G = H // h
    out = torch.empty(H, d, dtype=dtype)
    for i in range(h):
        Ki, Vi = K[i, rows[i]].to(dtype), V[i, rows[i]].to(dtype)
        s = (q[i * G:(i + 1) * G].to(dtype) @ Ki.T) / math.sqrt(d)
        out[i * G:(i + 1) * G] = torch.softmax(s, dim=-1) @ Vi
    return out


def merge_partials(m: torch.Tensor, l: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """Log-sum-exp merge of split partials ``m, l [h, S, G]``, ``a [h, S, G, d]`` -> ``[h*G, d]``
    (ssa/kernels/labeled_attn.py:154-160)."""
    M = m.max(dim=1, keepdim=True).values
    f = torch.exp(m - M)
    return ((f.unsqueeze(-1) * a).sum(1) / (f * l).sum(1).unsqueeze(-1)).reshape(-1, a.shape[-1])


# --------------------------------------------------------------------------------------------
# bytes read per decode step                                     (ssa/attn/accounting.py:19-32)
# --------------------------------------------------------------------------------------------
def overhead_rows(*, n, rows, clusters, d: int, summary_bits: int = 8, key_bits: int = 16):
    """Key-row equivalents read per KV head per step besides the K and V rows (fitted centroids)."""
    row = d * key_bits / 8
    vec = d * summary_bits / 8
    return (clusters * (vec + 12) + clusters * vec + 2 * n + 6 * rows + row + 8 * d) / row


def step_bytes(*, n, rows, clusters, d: int, summary_bits: int = 8, key_bits: int = 16):
    """Algorithmic bytes of one decode step of one KV head: K and V rows plus the overhead."""
    row = d * key_bits / 8
    return (2 * rows + overhead_rows(n=n, rows=rows, clusters=clusters, d=d, summary_bits=summary_bits,
                                     key_bits=key_bits)) * row


# --------------------------------------------------------------------------------------------
# synthetic inputs of the CPU-runnable configuration
# --------------------------------------------------------------------------------------------
def clustered_keys(h: int, n: int, d: int, *, seed: int, centres: int = 64):
    """Keys = 3 x one of ``centres`` unit directions + N(0, 0.5^2) + a shared offset of norm 2;
    values ~ N(0, 1).  float32 ``K, V [h, n, d]``."""
    g = torch.Generator().manual_seed(seed)
    ctr = F.normalize(torch.randn(centres, d, generator=g), dim=-1)
    off = 2 * F.normalize(torch.randn(d, generator=g), dim=-1)
    pick = torch.randint(0, centres, (h, n), generator=g)
    K = 3 * ctr[pick] + 0.5 * torch.randn(h, n, d, generator=g) + off
    V = torch.randn(h, n, d, generator=g)
    return K, V
