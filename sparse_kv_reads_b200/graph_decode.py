"""Whole decode step as one CUDA graph, with the clustered sparse attention inside it.

Mirror of the reference's ``GraphDecoder`` (ssa/models/graph_decode.py:29-157): same constructor
keywords, ``prepare(n)``, ``capture()``, ``step(token, pos)``, the attributes ``attn``, ``insert_all``,
``H, H_kv, d, B`` and ``_heads(cache)``.  The position lives in device memory, so a step is a single
graph launch; the batch is folded into the KV heads (``B`` sequences x ``H_kv`` heads are ``B*H_kv``
independent heads for every attention kernel).  Modes: ``"cluster"`` (aliases ``"sphere"``,
``"voronoi"``) and ``"dense"`` (exact attention by the same gather kernel in its dense mode).
"""

from __future__ import annotations

import os

import ctypes
import math

import torch

import torch.nn.functional as F

from . import _lib
from ._lib import check, dtype_code, lib, stream_ptr
from .cluster_state import AttentionPartials, ClusterArena, SphereIndexGraph, fit_layers, fit_layers_ragged
from .qwen3 import Qwen3Model, apply_rope


class DenseAttentionGraph:
    """Exact decode attention over ``[0, n)`` with ``n`` in device memory
    (ssa/kernels/graph_kernels.py:171-189)."""

    def __init__(self, *, H: int, H_kv: int, d: int, dtype, device):
        L = lib()
        self.H, self.H_kv, self.d, self.G = H, H_kv, d, H // H_kv
        self.n_group = 0                                   # heads per entry of the device-side lengths (0: one length)
        self.num_splits = L.skv_attend_splits(H_kv)
        self.ws = torch.zeros(L.skv_attend_workspace_bytes(H_kv, self.G, d, self.num_splits), dtype=torch.uint8,
                              device=device)
        self.out = torch.empty(H, d, dtype=dtype, device=device)

    def __call__(self, q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, n_dev: torch.Tensor) -> torch.Tensor:
        if not q.is_contiguous():
            q = q.contiguous()
        check(lib().skv_attend(q.data_ptr(), K.data_ptr(), V.data_ptr(), None, None, n_dev.data_ptr(), self.n_group,
                               self.out.data_ptr(), self.ws.data_ptr(), None, self.H_kv, self.G, self.d,
                               dtype_code(K.dtype), K.stride(0), K.stride(1), V.stride(0), V.stride(1), 0, K.shape[1],
                               self.num_splits, 1.0 / math.sqrt(self.d), stream_ptr(q.device)), "skv_attend")
        return self.out


class AllLayerInsert:
    """One insertion launch for every layer: the key that leaves the recent window at a step was written
    ``window`` steps earlier at every layer, so all layers insert (and split) together before the first
    layer runs (ssa/kernels/graph_kernels.py:286-325).  The layers' state already sits in one stacked
    arena; this object holds the table of per-layer cache addresses."""

    def __init__(self, layers: list, caches: list):
        first = layers[0]
        assert first.window >= 1, "with no recent window the key to insert is not yet written at later layers"
        assert all(i._arena is first._arena and i.end == first.end for i in layers)
        k0 = caches[0]
        assert all(k.stride() == k0.stride() and k.dtype == k0.dtype for k in caches)
        self.layers, self.L = layers, len(layers)
        self.arena = first._arena
        self.k0 = k0
        self.table = torch.tensor([k.data_ptr() for k in caches], dtype=torch.int64, device=k0.device)
        self.st = self.arena.struct(0, self.L * first.H_kv)
        self.max_members = max(i._members_limit() for i in layers)

    def __call__(self, n_dev: torch.Tensor) -> None:
        f = self.layers[0]
        check(lib().skv_insert(ctypes.byref(self.st), self.table.data_ptr(), f.H_kv, dtype_code(self.k0.dtype),
                               self.k0.stride(0), self.k0.stride(1), n_dev.data_ptr(), f.n_group, f.window, float(f.budget),
                               float(min(f.delta, 3.0e38)), f.reset_at, self.max_members, f.capk, f.var_min,
                               stream_ptr(self.k0.device)),
              "skv_insert")


class GraphDecoder:
    def __init__(self, model, cache, *, mode: str = "dense", budget: float = 0.2, C: int | None = None,
                 window: int = 64, delta: float = 0.03, check_every: int = 16, partition: str = "kmeans",
                 C_init: int | None = None, split_factor: float | None = None, refit_every: int = 0,
                 grow_cap: bool = False, reset_at: int = 0, summary_bits: int = 8, cap_keys: float = 0.0,
                 fused_insert: bool = True, var_factor: float = 0.0, var_min: int = 8, fused_dense: bool = True,
                 own_gemv: bool = True, insert_ahead: bool | None = None, **_):
        cfg = model.cfg
        # no slot count given: 1,024 slots, 256 fitted at the prompt, split over twice the mean size
        # (ssa/models/graph_decode.py:38-43)
        if C is None:
            C = 1024
            C_init = 256 if C_init is None else C_init
            split_factor = 2.0 if split_factor is None else split_factor
        split_factor = 0.0 if split_factor is None else split_factor
        mode = "cluster" if mode in ("sphere", "voronoi") else mode
        if mode not in ("dense", "cluster"):
            raise ValueError(f"unknown mode {mode!r}")
        self.model, self.cache, self.mode = model, cache, mode
        self.H, self.H_kv, self.d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.B = B = cache.k[0].shape[0]
        p = next(model.parameters())
        dev, dtype = p.device, p.dtype
        self.tok = torch.zeros(B, 1, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.n_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        cap = cache.max_seq_len
        nl = len(model.layers)
        if mode == "dense":
            self.attn = [DenseAttentionGraph(H=B * self.H, H_kv=B * self.H_kv, d=self.d, dtype=dtype, device=dev)
                         for _ in range(nl)]
        else:
            arena = ClusterArena(layers=nl, h=B * self.H_kv, C=C, d=self.d, capacity=cap, summary_bits=summary_bits,
                                 device=dev)
            self.attn = [SphereIndexGraph(budget=budget, C=C, window=window, delta=delta, capacity=cap,
                                          check_every=check_every, partition=partition, C_init=C_init,
                                          split_factor=split_factor, refit_every=refit_every, grow_cap=grow_cap,
                                          reset_at=reset_at, summary_bits=summary_bits, cap_keys=cap_keys,
                                          var_factor=var_factor, var_min=var_min, arena=arena, layer=i)
                         for i in range(nl)]
        self.graph = None
        self.logits = None
        self.ragged = False                                # True once prepare() was given one length per sequence
        # the bundled bf16 model runs its element-wise decode ops as three fused launches per layer
        self.fused_dense = fused_dense and isinstance(model, Qwen3Model) and dtype == torch.bfloat16 \
            and dev.type == "cuda"
        if self.fused_dense:
            self._fuse_weights()
        # ... and, up to 8 sequences, its projections as the library's matrix-vector products
        self.own_gemv = own_gemv and os.environ.get("SKV_OWN_GEMV", "1") != "0"
        self._peer = None
        # QK-norm + rotary in the selection launch: every scoring CTA of a KV head rotates its G query heads, so the
        # folding pays one launch with G x 16 small redundant jobs - even at G = 2 (0.6B: 583.6 against 583.0 tok/s),
        # a loss at G = 4 (4B: 253 against 257 tok/s); SKV_FOLD_ROPE=0/1 overrides
        fold = os.environ.get("SKV_FOLD_ROPE")
        self.fold_rope = (self.H // self.H_kv <= 2) if fold is None else fold != "0"
        # up to this many bytes of partial sums every CTA of the consuming product adds up for itself; beyond it one
        # reduce launch does (4 GPUs x 4 sequences, 128 KB: 2,096 tok/s with the launch, 1,955 without)
        self.fuse_sum_bytes = 65536
        # beyond 8 sequences the products are library GEMMs; their partial results go through the exchange buffers
        # (skv_comm_push + skv_comm_reduce) while every GPU receives at most this many bytes per sum, else through the
        # group's all-reduce: every rank writes to every GPU, 8 bytes per value, so the traffic grows with the group
        # (measured, 32 sequences of a 2,560-wide model: 2 GPUs, 1.3 MB: 4,417 against 4,333 tok/s with NCCL;
        # 8 GPUs, 5.2 MB: 5,661 against 6,321)
        self.push_sum_bytes = 1_500_000
        # the attention's last log-sum-exp merge rides in the output product (SKV_DEFER_MERGE=0: in the attention launch)
        self.defer_merge = os.environ.get("SKV_DEFER_MERGE", "1") != "0"
        self.fused_insert = fused_insert and mode == "cluster" and window >= 1
        self.insert_all = None
        # The all-layer insert of a step depends on nothing the step computes (the key that leaves the window was
        # written `window` steps ago), only on the step's length.  It therefore runs at the END of the step before,
        # for the length the next step will have, on a second stream beside the vocabulary projection, instead of
        # ahead of the first layer where nothing can overlap it: between steps the cluster state is one key ahead
        # of where ssa/kernels/graph_kernels.py:286-325 leaves it (prepare() inserts for the first step), and what
        # a step selects from is the same.  ``insert_ahead=False`` (or SKV_INSERT_AHEAD=0): ahead of the first layer, as
        # the reference does.
        self.insert_ahead = (os.environ.get("SKV_INSERT_AHEAD", "1") != "0") if insert_ahead is None else bool(insert_ahead)
        self.n_next = torch.zeros(1, dtype=torch.int32, device=dev)
        self._side = None
        self._warming = False

    @property
    def merge_deferred(self) -> bool:
        """Whether the one-launch step leaves the merge of its clusters' partials to the output product: the case
        when the library's own matrix-vector products serve this batch."""
        if not (self.mode == "cluster" and self.defer_merge and self.fused_dense and self.own_gemv and self.B <= 8):
            return False
        w = self.model.layers[0].attn.o.weight
        return bool(lib().skv_gemv_supported(w.shape[0], w.shape[1], self.B, 0))

    def _heads(self, c: torch.Tensor) -> torch.Tensor:
        """Cache ``[B, H_kv, L, d]`` -> ``[B*H_kv, L, d]`` (a view)."""
        return c.view(-1, c.shape[2], c.shape[3])

    def prepare(self, n) -> None:
        """Build the attention state from the first ``n`` cached positions (after the prompt).  ``n`` may be a
        list with one length per sequence: the batch then decodes sequences of different lengths (each head reads
        its own sequence's length and position from device memory), which lifts the reference's equal-length limit
        (README.md:62); ``step`` then takes one position per sequence."""
        if not isinstance(n, int):
            return self._prepare_ragged([int(x) for x in n])
        if self.mode != "cluster":
            return
        caches = [self._heads(self.cache.k[i]) for i in range(len(self.attn))]
        same = all(getattr(a, k) == getattr(self.attn[0], k) for a in self.attn
                   for k in ("C", "C_init", "window", "seed", "kmeans_iters", "cap_keys", "split_factor", "capk",
                             "var_factor", "partition"))
        fitted = same and fit_layers(self.attn, caches, n)         # one fit for all layers where they share an arena
        for idx, K in zip(self.attn, caches):
            idx.prepare(K, n, self.B * self.H, fitted=fitted)
        if self.fused_insert:
            self.insert_all = AllLayerInsert(self.attn, [self._heads(k) for k in self.cache.k[:len(self.attn)]])
            self._insert_for_first_step(n)

    def _insert_for_first_step(self, n: int | None) -> None:
        """With the insert running at the end of each step for the next one, the first step's insert happens here:
        for ``n + 1`` positions (``n`` None: one more than each sequence's length in ``n_dev``).  A second call
        for the same length inserts nothing, the kernel only moves ``end`` forward."""
        if self.insert_all is None or not self.insert_ahead:
            return
        if n is None:
            torch.add(self.n_dev, 1, out=self.n_next)
        else:
            self.n_next.fill_(n + 1)
        self.insert_all(self.n_next)

    def _finish(self, xn: torch.Tensor) -> torch.Tensor:
        """Final hidden state -> logits; the next step's all-layer insert runs beside the vocabulary projection."""
        if self.insert_all is None or not self.insert_ahead or self._warming:
            return self.model.logits(xn)
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream()
        torch.add(self.pos, 2, out=self.n_next)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            self.insert_all(self.n_next)
        out = self.model.logits(xn)
        main.wait_stream(self._side)
        return out

    def _prepare_ragged(self, lengths: list[int]) -> None:
        if len(lengths) != self.B:
            raise ValueError("one length per sequence is needed")
        if not self.fused_dense:
            raise ValueError("a variable-length batch needs the bundled bf16 model's fused layers")
        dev = self.tok.device
        self.ragged = True
        self.pos = torch.tensor(lengths, dtype=torch.long, device=dev)
        self.n_dev = torch.tensor(lengths, dtype=torch.int32, device=dev)
        self.n_next = torch.zeros_like(self.n_dev)
        for a in self.attn:
            a.n_group = self.H_kv                          # KV heads per sequence share one length
        if self.mode != "cluster":
            return
        caches = [self._heads(self.cache.k[i]) for i in range(len(self.attn))]
        fit_layers_ragged(self.attn, caches, lengths, self.H_kv)
        for idx, K in zip(self.attn, caches):
            idx.prepare(K, max(lengths), self.B * self.H, fitted=True, lengths=self.n_dev)
        if self.fused_insert:
            self.insert_all = AllLayerInsert(self.attn, caches)
            self._insert_for_first_step(None)

    # ---- checkpoint / resume -----------------------------------------------------------------------
    def state_dict(self) -> dict:
        """The cluster state of every layer (device arrays copied to the CPU, host counters) and the number of
        cached positions it describes.  Together with the KV cache itself (kept by the caller) this is all a
        later process needs to go on decoding as if it had never stopped.  Synchronises."""
        if self.ragged:
            raise ValueError("saving the state of a variable-length batch is not supported")
        if self.mode != "cluster":
            return {"n": self.cache.cur_len, "layers": []}
        return {"n": self.cache.cur_len, "layers": [a.state_dict() for a in self.attn]}

    def load_state_dict(self, sd: dict) -> None:
        """Restore what ``state_dict`` saved, in place of ``prepare``: no fit runs.  The cache this decoder was
        built on must already hold the ``sd["n"]`` positions the state describes; call ``capture`` afterwards."""
        n = int(sd["n"])
        self.cache.cur_len = n
        if self.mode != "cluster":
            return
        if len(sd["layers"]) != len(self.attn):
            raise ValueError("the saved state has a different number of layers")
        dev = self.tok.device
        for a, one in zip(self.attn, sd["layers"]):
            a.load_state_dict(one, dev)
        for i, a in enumerate(self.attn):
            # (a state saved between steps may already hold the next step's insert: its own length is one more)
            a.prepare(self._heads(self.cache.k[i]), max(n, a.n), self.B * self.H, fitted=True)
        if self.fused_insert:
            self.insert_all = AllLayerInsert(self.attn, [self._heads(k) for k in self.cache.k[:len(self.attn)]])
            self._insert_for_first_step(n)

    def _body(self) -> torch.Tensor:
        if self.fused_dense:
            return self._body_fused()
        assert not self.ragged
        m, H, H_kv, d, B = self.model, self.H, self.H_kv, self.d, self.B
        torch.add(self.pos, 1, out=self.n_dev)
        if self.insert_all is not None and not self.insert_ahead:
            self.insert_all(self.n_dev)
        h = m.embed(self.tok)
        cos = m.rope_cos.index_select(0, self.pos)
        sin = m.rope_sin.index_select(0, self.pos)
        for i, layer in enumerate(m.layers):
            a = layer.attn
            x = layer.norm1(h)
            q = a.q_norm(a.q(x).view(B, 1, H, d)).transpose(1, 2)
            k = a.k_norm(a.k(x).view(B, 1, H_kv, d)).transpose(1, 2)
            v = a.v(x).view(B, 1, H_kv, d).transpose(1, 2)
            q, k = apply_rope(q, k, cos, sin)
            kc, vc = self.cache.k[i], self.cache.v[i]
            kc.index_copy_(2, self.pos, k)
            vc.index_copy_(2, self.pos, v)
            qh = q.reshape(B * H, d)
            if self.mode == "dense":
                out = self.attn[i](qh, self._heads(kc), self._heads(vc), self.n_dev)
            else:
                out = self.attn[i].step(qh, self._heads(kc), self._heads(vc), self.n_dev,
                                        insert=self.insert_all is None)
            h = h + a.tp.all_reduce(a.o(out.view(B, 1, H * d)))
            h = h + layer.ffn(layer.norm2(h))
        return self._finish(m.final_norm(h))

    def _fuse_weights(self) -> None:
        """Lay q/k/v and gate/up weights of every layer out as one matrix each (the modules keep working:
        their weights become views of the fused tensors), so a layer needs four matrix products."""
        self._wqkv, self._wgu = [], []
        with torch.no_grad():
            for layer in self.model.layers:
                a, f = layer.attn, layer.ffn
                wqkv = torch.cat([a.q.weight, a.k.weight, a.v.weight], 0).contiguous()
                nq, nk = a.q.weight.shape[0], a.k.weight.shape[0]
                a.q.weight.data, a.k.weight.data, a.v.weight.data = wqkv[:nq], wqkv[nq:nq + nk], wqkv[nq + nk:]
                wgu = torch.cat([f.gate.weight, f.up.weight], 0).contiguous()
                ni = f.gate.weight.shape[0]
                f.gate.weight.data, f.up.weight.data = wgu[:ni], wgu[ni:]
                self._wqkv.append(wqkv)
                self._wgu.append(wgu)

    def _body_fused(self) -> torch.Tensor:
        # the cluster state is written once per step, ahead of every layer, so the selection and attention
        # launches may overlap the tails of the launches before them
        L = lib()
        L.skv_set_overlap(1 if self.insert_all is not None or self.mode == "dense" else 0)
        try:
            return self._layers_fused()
        finally:
            L.skv_set_overlap(0)

    def _layers_fused(self) -> torch.Tensor:
        if self.B <= 8 and self.own_gemv:
            return self._layers_gemv()
        m, H, H_kv, d, B = self.model, self.H, self.H_kv, self.d, self.B
        L = lib()
        st = stream_ptr(self.tok.device)
        torch.add(self.pos, 1, out=self.n_dev)
        if self.insert_all is not None and not self.insert_ahead:
            self.insert_all(self.n_dev)
        h = m.embed(self.tok).view(B, -1).contiguous()
        hidden = h.shape[1]
        eps = m.final_norm.eps
        delta = None
        xn = torch.empty_like(h)
        qh = torch.empty(B * H, d, dtype=h.dtype, device=h.device)
        world = m.layers[0].attn.tp.size
        peer = None
        if world > 1 and hidden % 8 == 0 and 2 * len(m.layers) <= 254 and world * B * hidden * 8 <= self.push_sum_bytes:
            peer = self._exchange()
        if peer is not None:
            peer.tick(st)                                  # stamps this step's exchanges

        def summed(y: torch.Tensor, tp, seq: int) -> torch.Tensor:
            """Sum of the ranks' partial results ``y [B, hidden]``: through the peer-memory exchange - every rank
            stores its values into every GPU's buffer, then adds the ranks' values up for itself, in rank order -
            or, on one GPU or with the exchange switched off, the group's all-reduce."""
            if peer is None:
                return tp.all_reduce(y)
            check(L.skv_comm_push(peer.ref(), seq, y.data_ptr(), B, hidden, st), "skv_comm_push")
            red = torch.empty_like(y)
            check(L.skv_comm_reduce(peer.ref(), seq, red.data_ptr(), B, hidden, st), "skv_comm_reduce")
            return red

        for i, layer in enumerate(m.layers):
            a, f = layer.attn, layer.ffn
            check(L.skv_add_rmsnorm(h.data_ptr(), None if delta is None else delta.data_ptr(),
                                    layer.norm1.weight.data_ptr(), xn.data_ptr(), B, hidden, eps, st), "skv_add_rmsnorm")
            qkv = F.linear(xn, self._wqkv[i])
            kc, vc = self.cache.k[i], self.cache.v[i]
            check(L.skv_qk_rope_cache(qkv.data_ptr(), a.q_norm.weight.data_ptr(), a.k_norm.weight.data_ptr(),
                                      m.rope_cos.data_ptr(), m.rope_sin.data_ptr(), self.pos.data_ptr(),
                                      int(self.ragged), qh.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, H, H_kv, d,
                                      kc.stride(0), kc.stride(1), kc.stride(2), a.q_norm.eps, st), "skv_qk_rope_cache")
            if self.mode == "dense":
                out = self.attn[i](qh, self._heads(kc), self._heads(vc), self.n_dev)
            else:
                out = self.attn[i].step(qh, self._heads(kc), self._heads(vc), self.n_dev,
                                        insert=self.insert_all is None)
            o = summed(F.linear(out.view(B, H * d), a.o.weight), a.tp, 2 * i)
            check(L.skv_add_rmsnorm(h.data_ptr(), o.data_ptr(), layer.norm2.weight.data_ptr(), xn.data_ptr(), B,
                                    hidden, eps, st), "skv_add_rmsnorm")
            gu = F.linear(xn, self._wgu[i])
            act = torch.empty(B, gu.shape[1] // 2, dtype=gu.dtype, device=gu.device)
            check(L.skv_silu_mul(gu.data_ptr(), act.data_ptr(), B, act.shape[1], st), "skv_silu_mul")
            delta = summed(F.linear(act, f.down.weight), f.tp, 2 * i + 1)
        check(L.skv_add_rmsnorm(h.data_ptr(), delta.data_ptr(), m.final_norm.weight.data_ptr(), xn.data_ptr(), B,
                                hidden, eps, st), "skv_add_rmsnorm")
        return self._finish(xn.view(B, 1, hidden))

    def _layers_gemv(self) -> torch.Tensor:
        """The layers with the library's own matrix-vector products (up to 8 sequences): a layer is seven
        launches - q/k/v product with the residual add and norm folded into its input, QK-norm + rotary +
        cache write, selection, attention, output product, gate/up product (add and norm folded in), down
        product (SiLU x up folded in) - each requesting its weights while the launch ahead of it finishes.
        In a tensor-parallel group the row-parallel products (output, down) store their partial sums into every
        GPU's exchange buffer and the product after them adds the partials up: no all-reduce launch."""
        m, H, H_kv, d, B = self.model, self.H, self.H_kv, self.d, self.B
        L = lib()
        st = stream_ptr(self.tok.device)
        torch.add(self.pos, 1, out=self.n_dev)
        if self.insert_all is not None and not self.insert_ahead:
            self.insert_all(self.n_dev)
        h = m.embed(self.tok).view(B, -1).contiguous()
        hidden = h.shape[1]
        eps = m.final_norm.eps
        h2 = torch.empty_like(h)                           # the residual stream alternates between two buffers
        buf_a, buf_b = h, h2
        dev, dt = h.device, h.dtype
        qh = torch.empty(B * H, d, dtype=dt, device=dev)
        nqkv, ngu = self._wqkv[0].shape[0], self._wgu[0].shape[0]
        qkv = torch.empty(B, nqkv, dtype=dt, device=dev)
        o = torch.empty(B, hidden, dtype=dt, device=dev)
        gu = torch.empty(B, ngu, dtype=dt, device=dev)
        xn = torch.empty_like(h)
        peer = self._exchange()
        if peer is not None:
            peer.tick(st)                                  # stamps this step's exchanges

        def ptr_of(t):
            return None if t is None else t.data_ptr()

        def product(W, y, mode, x=None, h_in=None, dl=None, g=None, h_out=None, tp=None, slot_out=None):
            """One projection.  ``dl`` is the delta to add to the residual (mode 1): a tensor, or the number of
            the exchange that holds its partial sums.  ``slot_out``: deliver the result as partial sums under
            that exchange number instead of ``y`` (returns the number), else all-reduce ``y`` over ``tp`` when
            given.  Returns (residual buffer now current, result: tensor or exchange number)."""
            N, K = W.shape
            if isinstance(x, AttentionPartials):            # the attention's last merge happens inside this product
                to_slot = slot_out is not None
                check(L.skv_gemv_attended(W.data_ptr(), N, K, None if to_slot else y.data_ptr(), B,
                                          x.workspace.data_ptr(), x.clusters, x.G, x.cnt.data_ptr(),
                                          peer.ref() if to_slot else None, slot_out if to_slot else 0, st),
                      "skv_gemv_attended")
                if to_slot:
                    return h_out, slot_out
                return h_out, (tp.all_reduce(y) if tp is not None else y)
            from_slot = isinstance(dl, int)
            own = bool(L.skv_gemv_supported(N, K, B, 3 if from_slot else mode))
            # every CTA of the product adds the ranks' partials up for itself only while that is a few KB
            if from_slot and (not own or peer.world * B * K * 8 > self.fuse_sum_bytes):
                red = torch.empty(B, K, dtype=dt, device=dev)
                check(L.skv_comm_reduce(peer.ref(), dl, red.data_ptr(), B, K, st), "skv_comm_reduce")
                dl, from_slot = red, False
                own = bool(L.skv_gemv_supported(N, K, B, mode))
            if own:
                to_slot = slot_out is not None
                if from_slot or to_slot:
                    check(L.skv_gemv_tp(W.data_ptr(), N, K, None if to_slot else y.data_ptr(), B,
                                        3 if from_slot else mode, ptr_of(x), ptr_of(h_in), ptr_of(g), ptr_of(h_out), eps,
                                        peer.ref() if from_slot else None, dl if from_slot else 0,
                                        peer.ref() if to_slot else None, slot_out if to_slot else 0, st), "skv_gemv_tp")
                else:
                    check(L.skv_gemv(W.data_ptr(), N, K, y.data_ptr(), B, mode, ptr_of(x), ptr_of(h_in), ptr_of(dl),
                                     ptr_of(g), ptr_of(h_out), eps, st), "skv_gemv")
                if to_slot:
                    return h_out, slot_out
                return h_out, (tp.all_reduce(y) if tp is not None else y)
            # shapes the library product does not serve well: the separate element-wise kernel, then cuBLAS
            if mode == 1:                                   # in place: the residual stays in h_in
                check(L.skv_add_rmsnorm(h_in.data_ptr(), ptr_of(dl), g.data_ptr(), xn.data_ptr(), B, K, eps, st),
                      "skv_add_rmsnorm")
                x = xn
            elif mode == 2:
                act = torch.empty(B, K, dtype=dt, device=dev)
                check(L.skv_silu_mul(x.data_ptr(), act.data_ptr(), B, K, st), "skv_silu_mul")
                x = act
            torch.matmul(x.view(B, K), W.t(), out=y)
            return h_in, (tp.all_reduce(y) if tp is not None else y)

        def peer_ok(W, mode):
            return peer is not None and bool(L.skv_gemv_supported(W.shape[0], W.shape[1], B, mode))

        delta = None
        for i, layer in enumerate(m.layers):
            a, f = layer.attn, layer.ffn
            res, _ = product(self._wqkv[i], qkv, 1, h_in=h, dl=delta, g=layer.norm1.weight, h_out=h2)
            h = res if res is not None else h
            h2 = buf_b if h is buf_a else buf_a
            kc, vc = self.cache.k[i], self.cache.v[i]
            # the output product merges the attention's split partials itself where it is the library's own product
            defer = self.mode == "cluster" and self.defer_merge and bool(
                L.skv_gemv_supported(a.o.weight.shape[0], a.o.weight.shape[1], B, 0))
            fold = (self.mode == "cluster" and self.fold_rope and self.attn[i]._fused_rows(self._heads(kc)))
            if fold:
                # QK-norm, rotary and the cache write ride in the selection launch: six launches per layer
                rope = _lib.SkvRope(qkv.data_ptr(), a.q_norm.weight.data_ptr(), a.k_norm.weight.data_ptr(),
                                    m.rope_cos.data_ptr(), m.rope_sin.data_ptr(), self.pos.data_ptr(), qh.data_ptr(),
                                    kc.data_ptr(), vc.data_ptr(), H, H_kv, kc.stride(0), kc.stride(1), kc.stride(2),
                                    a.q_norm.eps, int(self.ragged))
                out = self.attn[i].step(qh, self._heads(kc), self._heads(vc), self.n_dev,
                                        insert=self.insert_all is None, rope=rope, defer_merge=defer)
            else:
                check(L.skv_qk_rope_cache(qkv.data_ptr(), a.q_norm.weight.data_ptr(), a.k_norm.weight.data_ptr(),
                                          m.rope_cos.data_ptr(), m.rope_sin.data_ptr(), self.pos.data_ptr(),
                                          int(self.ragged), qh.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, H, H_kv, d,
                                          kc.stride(0), kc.stride(1), kc.stride(2), a.q_norm.eps, st),
                      "skv_qk_rope_cache")
                if self.mode == "dense":
                    out = self.attn[i](qh, self._heads(kc), self._heads(vc), self.n_dev)
                else:
                    out = self.attn[i].step(qh, self._heads(kc), self._heads(vc), self.n_dev,
                                            insert=self.insert_all is None, defer_merge=defer)
            _, o_red = product(a.o.weight, o, 0, x=out, tp=a.tp,
                               slot_out=2 * i if peer_ok(a.o.weight, 0) else None)
            res, _ = product(self._wgu[i], gu, 1, h_in=h, dl=o_red, g=layer.norm2.weight, h_out=h2)
            h = res if res is not None else h
            h2 = buf_b if h is buf_a else buf_a
            dn = torch.empty(B, hidden, dtype=dt, device=dev)
            _, delta = product(f.down.weight, dn, 2, x=gu, tp=f.tp,
                               slot_out=2 * i + 1 if peer_ok(f.down.weight, 2) else None)
        if isinstance(delta, int):
            red = torch.empty(B, hidden, dtype=dt, device=dev)
            check(L.skv_comm_reduce(peer.ref(), delta, red.data_ptr(), B, hidden, st), "skv_comm_reduce")
            delta = red
        check(L.skv_add_rmsnorm(h.data_ptr(), delta.data_ptr(), m.final_norm.weight.data_ptr(), xn.data_ptr(), B,
                                hidden, eps, st), "skv_add_rmsnorm")
        return self._finish(xn.view(B, 1, hidden))

    def _exchange(self):
        """The tensor-parallel group's exchange buffers (made on first use), or None on a single GPU."""
        tp = self.model.layers[0].attn.tp
        if tp.size <= 1 or os.environ.get("SKV_PEER_REDUCE", "1") == "0":
            return None
        if self._peer is None:
            from .peer_reduce import PeerExchange
            hidden = self.model.cfg.hidden_size
            self._peer = PeerExchange(tp.group, self.B * hidden, self.tok.device)
        return self._peer

    def capture(self) -> None:
        """Record one decode step.  Call after ``prepare`` and before the first ``step``; the warm-up
        runs write a placeholder at the current position, which the first real step overwrites."""
        if self.ragged:
            self.pos.copy_(torch.tensor(self.cache.cur_len, dtype=torch.long))
        else:
            self.pos.fill_(self.cache.cur_len)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        self._warming = True                           # (the next step's insert must not run in the warm-up steps)
        try:
            with torch.cuda.stream(s), torch.no_grad():
                for _ in range(2):
                    self._body()
        finally:
            self._warming = False
        torch.cuda.current_stream().wait_stream(s)
        if self.mode == "cluster":                     # the warm-up steps must not have advanced the clusters
            torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = _lib.launches
        with torch.no_grad(), torch.cuda.graph(g):
            self.logits = self._body()
        self.launches_per_step = _lib.launches - before     # this library's kernels in one replay
        self.graph = g

    @torch.no_grad()
    def step(self, token: torch.Tensor, pos) -> torch.Tensor:
        """Decode ``token [B, 1]`` at position ``pos`` (one position per sequence, a list or tensor ``[B]``, for a
        batch prepared with one length per sequence); returns logits ``[B, 1, vocab]`` (a buffer the next step
        overwrites)."""
        self.tok.copy_(token, non_blocking=True)           # a pinned host tensor goes straight into the step's buffer
        if self.ragged:
            if not torch.is_tensor(pos):
                pos = torch.tensor([int(x) for x in pos], dtype=torch.long)
            self.pos.copy_(pos, non_blocking=True)
        else:
            self.pos.fill_(pos)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.logits = self._body()
        if self.mode == "cluster":
            for i, idx in enumerate(self.attn):
                idx.after_replay(self._heads(self.cache.k[i]))
        self.cache.cur_len = (pos + 1).tolist() if self.ragged else pos + 1
        return self.logits
