"""Bytes a decode step reads, per KV head: the accounting every bandwidth figure here is quoted on.

Same definition as the reference's ``ssa.attn.accounting`` (accounting.py:19-32): besides the K and V
rows attended over, a step reads the summaries of the clusters in use (mean direction at
``summary_bits`` per component, longest and shortest key and the count as float32), their centroids
(to place the inserted key), a 16-bit label per cached token, a 32-bit position and a 16-bit label per
row read, the inserted key and its cluster's float32 direction sum (read and written).  The query, the
split partials and the output are left out, as in the reference.
"""

from __future__ import annotations


def overhead_rows(*, n, rows, clusters, d: int, summary_bits: int = 8, fitted: bool = True, heads: int = 1,
                  key_bits: int = 16):
    """Key-row equivalents read per KV head per step besides the ``rows`` K and V rows themselves."""
    row = d * key_bits / 8
    vec = d * summary_bits / 8
    summaries = clusters * (vec + 12)
    centroids = clusters * vec if fitted else clusters * 4 * d / heads
    return (summaries + centroids + 2 * n + 6 * rows + row + 8 * d) / row


def kv_read_fraction(*, n, rows, clusters, d: int, **kw):
    """Fraction of the K+V cache's bytes one step reads: ``rows`` rows of each, plus the overhead."""
    return (2 * rows + overhead_rows(n=n, rows=rows, clusters=clusters, d=d, **kw)) / (2 * n)


def step_bytes(*, n, rows, clusters, d: int, summary_bits: int = 8, key_bits: int = 16):
    """Algorithmic bytes of one decode step of one KV head."""
    row = d * key_bits / 8
    return (2 * rows + overhead_rows(n=n, rows=rows, clusters=clusters, d=d, summary_bits=summary_bits,
                                     key_bits=key_bits)) * row
