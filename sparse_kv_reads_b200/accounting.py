"""Bytes a decode step reads, per KV head: the accounting every bandwidth figure here is quoted on.

The formula is the reference's (``ssa.attn.accounting``, accounting.py:19-32), so numbers are comparable:
per KV head and step ``2*rows*R + n_c*(V+12) + n_c*V + 2*n + 6*rows + R + 8*d`` bytes with ``R`` one key
row and ``V`` one cluster direction at ``summary_bits``.  In words: the K and V rows attended over; one
summary per cluster in use (direction, two key lengths and a count); the directions searched when a key is
inserted; every cached token's int16 label; position and label of each row read; the inserted key and the
float32 direction sum it is folded into.  Queries, split partials and outputs are not charged.
"""

from __future__ import annotations


def overhead_rows(*, n, rows, clusters, d: int, summary_bits: int = 8, fitted: bool = True, heads: int = 1,
                  key_bits: int = 16):
    """What a step reads for one KV head besides its ``rows`` K rows and V rows, in units of one key row.
    ``fitted=False`` charges shared float32 directions (a ``partition="random"`` state) instead of per-head
    centroids at ``summary_bits``."""
    key_row_bytes = d * key_bits / 8
    direction_bytes = d * summary_bits / 8
    per_cluster = direction_bytes + 12                                   # direction + two lengths + count
    search_bytes = clusters * direction_bytes if fitted else clusters * 4 * d / heads
    label_bytes = 2 * n                                                  # int16 per cached token
    per_row_read = 6 * rows                                              # int32 position + int16 label
    insert_bytes = key_row_bytes + 8 * d                                 # new key + its float32 sum, read and written
    total = clusters * per_cluster + search_bytes + label_bytes + per_row_read + insert_bytes
    return total / key_row_bytes


def kv_read_fraction(*, n, rows, clusters, d: int, **kw):
    """Fraction of the K+V cache's bytes one step reads: ``rows`` rows of each, plus the overhead."""
    return (2 * rows + overhead_rows(n=n, rows=rows, clusters=clusters, d=d, **kw)) / (2 * n)


def step_bytes(*, n, rows, clusters, d: int, summary_bits: int = 8, key_bits: int = 16):
    """Algorithmic bytes of one decode step of one KV head."""
    row = d * key_bits / 8
    return (2 * rows + overhead_rows(n=n, rows=rows, clusters=clusters, d=d, summary_bits=summary_bits,
                                     key_bits=key_bits)) * row
