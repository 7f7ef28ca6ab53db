"""Host-side placement for multi-GPU runs: which rank owns which sequence, and which key range.

The reference is single-GPU, single-session; this is the scheduling that the batched and long-context workloads add:
independent sequences are spread over ranks by KV bytes (no data-path collective), and one long sequence is cut
into contiguous key ranges (one exchange step: an all-gather of per-rank partial records).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

KV_BYTES_PER_KEY = 2048  # K + V rows of 4 KV heads x 128 halves
SWA_KEYS = 512           # cached keys a sliding-window layer reads at most


def kv_bytes_per_token_step(ctx_len: int, n_full_layers: int = 1, n_swa_layers: int = 0) -> int:
    """Cache bytes one decode step reads for a sequence with ctx_len cached tokens."""
    return KV_BYTES_PER_KEY * (n_full_layers * ctx_len + n_swa_layers * min(ctx_len, SWA_KEYS))


def balance_by_kv_bytes(ctx_lens: Sequence[int], n_ranks: int, n_full_layers: int = 1,
                        n_swa_layers: int = 0) -> List[List[int]]:
    """Greedy longest-processing-time placement: sequences sorted by bytes, each to the least loaded rank.
    Returns, per rank, the (sorted) global sequence indices it owns."""
    if n_ranks < 1:
        raise ValueError("n_ranks must be positive")
    cost = [kv_bytes_per_token_step(c, n_full_layers, n_swa_layers) for c in ctx_lens]
    order = sorted(range(len(ctx_lens)), key=lambda i: (-cost[i], i))
    load = [0] * n_ranks
    owned: List[List[int]] = [[] for _ in range(n_ranks)]
    for i in order:
        r = min(range(n_ranks), key=lambda k: (load[k], k))
        owned[r].append(i)
        load[r] += cost[i]
    return [sorted(o) for o in owned]


def contiguous_blocks(n_items: int, n_ranks: int) -> List[Tuple[int, int]]:
    """[begin, end) of the contiguous block of items each rank owns (sizes differ by at most one)."""
    base, extra = divmod(n_items, n_ranks)
    out, b = [], 0
    for r in range(n_ranks):
        e = b + base + (1 if r < extra else 0)
        out.append((b, e))
        b = e
    return out


def kv_shard_range(n_ctx: int, rank: int, n_ranks: int) -> Tuple[int, int]:
    """Key positions [lo, hi) a rank holds when a full layer's context is cut over ranks; the same arithmetic as
    flint_attn_open (shard = ceil(n_ctx / n_ranks))."""
    shard = (n_ctx + n_ranks - 1) // n_ranks
    lo = min(n_ctx, rank * shard)
    return lo, min(n_ctx, lo + shard)
