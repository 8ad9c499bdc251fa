"""Minimal Qwen3 host model with the attribute surface the decode loop of the reference expects.

The reference drives an external engine (package ``engine`` of github.com/aaholmes/llms, absent here)
through these names: ``model.cfg``, ``model.embed``, ``model.rope_cos/rope_sin``, ``model.layers[i]
.{norm1, attn, norm2, ffn}``, ``attn.{q, k, v, o, q_norm, k_norm, decode_attn_op}``, ``model.final_norm``,
``model.lm_head``, ``apply_rope``, ``model.alloc_cache`` and ``model(ids, cache, start_pos=...)``
(call sites: ssa/models/graph_decode.py:44-50, :93-122; parameter names tests/_tiny_model.py:45-62).
This file provides them on plain PyTorch modules (the dense GEMMs around the attention are library
calls; the hot path is the attention op).  Weights are random (no checkpoint is read).

Tensor parallelism: with ``tp_size > 1`` each rank holds ``1/tp_size`` of the KV heads with their query
heads, of the MLP columns and of the vocabulary rows; ``o`` and ``down`` are followed by one
all-reduce each and the logits by an all-gather.  The attention itself needs no communication.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class Qwen3Config:
    hidden_size: int = 1024
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    vocab_size: int = 151936
    rope_theta: float = 1.0e6
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = True

    @staticmethod
    def qwen3_0_6b(**kw) -> "Qwen3Config":
        return Qwen3Config(**kw)

    @staticmethod
    def qwen3_4b(**kw) -> "Qwen3Config":
        return Qwen3Config(hidden_size=2560, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                           intermediate_size=9728, **kw)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * self.weight.float()).to(x.dtype)


def apply_rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Rotate ``q, k [B, heads, T, d]`` by the angles ``cos, sin [T, d]`` (half-split convention)."""
    def rot(x):
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat((-x2, x1), dim=-1)
    cos, sin = cos.to(q.dtype), sin.to(q.dtype)
    return q * cos + rot(q) * sin, k * cos + rot(k) * sin


class KVCache:
    """Contiguous cache: ``k[i], v[i] [B, H_kv, L, d]`` per layer."""

    def __init__(self, layers: int, batch: int, h_kv: int, max_seq_len: int, d: int, dtype, device):
        self.k = [torch.zeros(batch, h_kv, max_seq_len, d, dtype=dtype, device=device) for _ in range(layers)]
        self.v = [torch.zeros(batch, h_kv, max_seq_len, d, dtype=dtype, device=device) for _ in range(layers)]
        self.cur_len = 0
        self.max_seq_len = max_seq_len


class _TP:
    def __init__(self, group, size: int, rank: int):
        self.group, self.size, self.rank = group, size, rank

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
        return x


class Attention(nn.Module):
    def __init__(self, cfg: Qwen3Config, tp: _TP, layer_idx: int):
        super().__init__()
        self.H, self.H_kv, self.d = cfg.num_attention_heads // tp.size, cfg.num_key_value_heads // tp.size, cfg.head_dim
        self.q = nn.Linear(cfg.hidden_size, self.H * self.d, bias=False)
        self.k = nn.Linear(cfg.hidden_size, self.H_kv * self.d, bias=False)
        self.v = nn.Linear(cfg.hidden_size, self.H_kv * self.d, bias=False)
        self.o = nn.Linear(self.H * self.d, cfg.hidden_size, bias=False)
        self.q_norm = RMSNorm(self.d, cfg.rms_norm_eps)
        self.k_norm = RMSNorm(self.d, cfg.rms_norm_eps)
        self.decode_attn_op = None            # set by patch.install: op(q, full_k, full_v, *, scale, layer_idx)
        self.layer_idx, self.tp = layer_idx, tp

    def forward(self, x: torch.Tensor, cache: KVCache, start_pos: int, cos: torch.Tensor, sin: torch.Tensor):
        B, T, _ = x.shape
        q = self.q_norm(self.q(x).view(B, T, self.H, self.d)).transpose(1, 2)
        k = self.k_norm(self.k(x).view(B, T, self.H_kv, self.d)).transpose(1, 2)
        v = self.v(x).view(B, T, self.H_kv, self.d).transpose(1, 2)
        q, k = apply_rope(q, k, cos, sin)
        kc, vc = cache.k[self.layer_idx], cache.v[self.layer_idx]
        kc[:B, :, start_pos:start_pos + T] = k
        vc[:B, :, start_pos:start_pos + T] = v
        n = start_pos + T
        scale = 1.0 / math.sqrt(self.d)
        if T == 1 and self.decode_attn_op is not None:
            out = self.decode_attn_op(q, kc[:B, :, :n], vc[:B, :, :n], scale=scale, layer_idx=self.layer_idx)
        elif start_pos == 0:
            out = F.scaled_dot_product_attention(q, k, v, is_causal=T > 1, enable_gqa=True)
        else:
            mask = torch.ones(T, n, dtype=torch.bool, device=x.device).tril_(diagonal=start_pos)
            out = F.scaled_dot_product_attention(q, kc[:B, :, :n], vc[:B, :, :n], attn_mask=mask, enable_gqa=True)
        return self.tp.all_reduce(self.o(out.transpose(1, 2).reshape(B, T, self.H * self.d)))


class MLP(nn.Module):
    def __init__(self, cfg: Qwen3Config, tp: _TP):
        super().__init__()
        inter = cfg.intermediate_size // tp.size
        self.gate = nn.Linear(cfg.hidden_size, inter, bias=False)
        self.up = nn.Linear(cfg.hidden_size, inter, bias=False)
        self.down = nn.Linear(inter, cfg.hidden_size, bias=False)
        self.tp = tp

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.tp.all_reduce(self.down(F.silu(self.gate(x)) * self.up(x)))


class Block(nn.Module):
    def __init__(self, cfg: Qwen3Config, tp: _TP, layer_idx: int):
        super().__init__()
        self.norm1 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.attn = Attention(cfg, tp, layer_idx)
        self.norm2 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.ffn = MLP(cfg, tp)


class Qwen3Model(nn.Module):
    """``cfg`` seen by callers is the LOCAL view: ``num_attention_heads`` and ``num_key_value_heads``
    are this rank's shares, so the decode loop sizes its attention state for the local heads."""

    def __init__(self, cfg: Qwen3Config, *, tp_group=None, tp_size: int = 1, tp_rank: int = 0):
        super().__init__()
        if cfg.num_key_value_heads % tp_size or cfg.intermediate_size % tp_size or cfg.vocab_size % tp_size:
            raise ValueError("KV heads, MLP columns and vocabulary must divide by the tensor-parallel size")
        self.full_cfg = cfg
        self.tp = _TP(tp_group, tp_size, tp_rank)
        self.cfg = Qwen3Config(**{**cfg.__dict__, "num_attention_heads": cfg.num_attention_heads // tp_size,
                                  "num_key_value_heads": cfg.num_key_value_heads // tp_size})
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(Block(cfg, self.tp, i) for i in range(cfg.num_hidden_layers))
        self.final_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        # vocabulary-parallel output rows; None means "tied to embed" (single rank only)
        self.lm_head = None if (cfg.tie_word_embeddings and tp_size == 1) else \
            nn.Linear(cfg.hidden_size, cfg.vocab_size // tp_size, bias=False)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float64) / cfg.head_dim))
        ang = torch.outer(torch.arange(cfg.max_position_embeddings, dtype=torch.float64), inv)
        ang = torch.cat((ang, ang), dim=-1)
        self.register_buffer("rope_cos", ang.cos().float(), persistent=False)
        self.register_buffer("rope_sin", ang.sin().float(), persistent=False)

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "Qwen3Model":
        """Random weights, identical on every rank for the shared parts and sliced consistently for the
        sharded ones (each full matrix is drawn from the same seeded stream, then this rank's rows or
        columns are kept)."""
        cfg, tp = self.full_cfg, self.tp
        dev = self.embed.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)

        def draw(rows, cols):
            return torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32) * std

        def rows_of(w, parts):
            n = w.shape[0] // parts
            return w[tp.rank * n:(tp.rank + 1) * n]

        emb = draw(cfg.vocab_size, cfg.hidden_size)
        self.embed.weight.copy_(emb)
        if self.lm_head is not None:
            self.lm_head.weight.copy_(rows_of(emb if cfg.tie_word_embeddings else draw(cfg.vocab_size, cfg.hidden_size),
                                              tp.size))
        del emb
        d = cfg.head_dim
        for layer in self.layers:
            a, f = layer.attn, layer.ffn
            a.q.weight.copy_(rows_of(draw(cfg.num_attention_heads * d, cfg.hidden_size), tp.size))
            a.k.weight.copy_(rows_of(draw(cfg.num_key_value_heads * d, cfg.hidden_size), tp.size))
            a.v.weight.copy_(rows_of(draw(cfg.num_key_value_heads * d, cfg.hidden_size), tp.size))
            a.o.weight.copy_(rows_of(draw(cfg.num_attention_heads * d, cfg.hidden_size), tp.size).t())
            f.gate.weight.copy_(rows_of(draw(cfg.intermediate_size, cfg.hidden_size), tp.size))
            f.up.weight.copy_(rows_of(draw(cfg.intermediate_size, cfg.hidden_size), tp.size))
            f.down.weight.copy_(rows_of(draw(cfg.intermediate_size, cfg.hidden_size), tp.size).t())
        return self

    def alloc_cache(self, max_seq_len: int, max_batch: int = 1, dtype=None) -> KVCache:
        p = self.embed.weight
        return KVCache(len(self.layers), max_batch, self.cfg.num_key_value_heads, max_seq_len, self.cfg.head_dim,
                       dtype or p.dtype, p.device)

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        """Full-vocabulary logits of hidden states ``h [B, T, hidden]``."""
        if self.lm_head is None:
            return h @ self.embed.weight.T
        part = self.lm_head(h)
        if self.tp.size == 1:
            return part
        parts = [torch.empty_like(part) for _ in range(self.tp.size)]
        dist.all_gather(parts, part.contiguous(), group=self.tp.group)
        return torch.cat(parts, dim=-1)

    def forward(self, ids: torch.Tensor, cache: KVCache, start_pos: int = 0, last_only: bool = False) -> torch.Tensor:
        B, T = ids.shape
        h = self.embed(ids)
        cos, sin = self.rope_cos[start_pos:start_pos + T], self.rope_sin[start_pos:start_pos + T]
        for layer in self.layers:
            h = h + layer.attn(layer.norm1(h), cache, start_pos, cos, sin)
            h = h + layer.ffn(layer.norm2(h))
        cache.cur_len = start_pos + T
        h = self.final_norm(h[:, -1:] if last_only else h)
        return self.logits(h)

    @torch.no_grad()
    def prefill_ragged(self, prompts: list[torch.Tensor], cache: KVCache, chunk: int = 2048) -> list[torch.Tensor]:
        """Prompts of different lengths, one per sequence of the cache: sequence ``b`` is prefilled on its own rows
        of the cache (a view of batch 1).  Returns the last-position logits of each; ``cache.cur_len`` becomes the
        list of lengths."""
        outs = []
        for b, ids in enumerate(prompts):
            view = KVCache.__new__(KVCache)
            view.k, view.v = [k[b:b + 1] for k in cache.k], [v[b:b + 1] for v in cache.v]
            view.cur_len, view.max_seq_len = 0, cache.max_seq_len
            outs.append(self.prefill(ids.view(1, -1), view, chunk=chunk))
        cache.cur_len = [int(p.numel()) for p in prompts]
        return outs

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, cache: KVCache, chunk: int = 2048) -> torch.Tensor:
        """Run the prompt through the model in chunks; returns the logits of the last position."""
        out = None
        for s in range(0, ids.shape[1], chunk):
            out = self.forward(ids[:, s:s + chunk], cache, start_pos=s, last_only=True)
        return out
