"""Drawing some of the clusters a selection left out, so that the attention sums stay unbiased.

Host side of ``SphereIndexGraph.attend_sampled`` (the reference's ``ssa.attn.tail_sample``, tail_sample.py:24-63,
used by ``SphereIndexFused.attend_sampled``, ssa/kernels/sphere_fused.py:503-518).  The selected clusters are read
exactly (weight 1).  ``S`` of the others are drawn by systematic sampling from a proposal ``pi`` and a drawn
cluster gets the weight ``draws / (S pi)``: its expected weight is 1, so numerator and denominator of the
label-weighted attention are unbiased for the sums over the whole cache.  A few tensor operations on ``[heads, C]``
arrays that already live on the device; the attention itself is ``skv_attend_weighted``.
"""

from __future__ import annotations

import torch


def proposal_from_scores(e: torch.Tensor, count: torch.Tensor, *, scale: float) -> torch.Tensor:
    """``e [h, G, C]`` score estimates (-inf for empty clusters), ``count [h, C]`` -> ``[h, C]`` probabilities: the
    estimated softmax mass ``count * exp(scale * e)`` of each cluster, normalised per query head, averaged over
    the group."""
    z = scale * e
    z = z - z.amax(dim=2, keepdim=True)
    mass = torch.nan_to_num(count.unsqueeze(1) * torch.exp(z), nan=0.0)
    return (mass / mass.sum(dim=2, keepdim=True).clamp_min(1e-300)).mean(dim=1)


def tail_sample_weights(prop: torch.Tensor, count: torch.Tensor, head: torch.Tensor, *, S: int, alpha: float,
                        generator: torch.Generator | None = None) -> torch.Tensor:
    """Weights ``[h, C]``: 1 for the non-empty clusters in ``head`` (the selection), ``draws / (S pi)`` for the
    drawn ones among the rest, 0 elsewhere.  ``pi`` = (1 - alpha) x the proposal restricted to the rest + alpha x
    uniform over the rest.  The one random number per head comes from ``generator`` on the CPU, as in the reference,
    so equal seeds give equal draws."""
    live = count > 0
    kept = (head & live).to(prop.dtype)
    rest = live & ~head
    if S <= 0:
        return kept
    p = prop * rest
    p = p / p.sum(1, keepdim=True).clamp_min(1e-300)
    pi = ((1.0 - alpha) * p + alpha / rest.sum(1, keepdim=True).clamp_min(1)) * rest
    cdf = pi.cumsum(1)
    rows, C = pi.shape
    start = torch.rand(rows, 1, generator=generator, dtype=prop.dtype, device="cpu").to(prop.device) / S
    probes = (start + torch.arange(S, dtype=prop.dtype, device=prop.device) / S) * cdf[:, -1:]
    hit = torch.searchsorted(cdf.contiguous(), probes.contiguous()).clamp_(max=C - 1)
    draws = torch.zeros_like(prop).scatter_add_(1, hit, torch.ones_like(probes)) * rest.any(1, keepdim=True)
    drawn = torch.where(rest & (draws > 0), draws / (S * pi.clamp_min(1e-300)), torch.zeros_like(prop))
    return kept + drawn
