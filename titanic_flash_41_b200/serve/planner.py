"""Prefill chunk planner: cut a prompt into chunks from the available widths so that the summed
measured cost is minimal; full chunks widest-first, the partial chunk last, and a suspended
prefill resumes with the SAME sequence (reference: src/config.rs:833-859 plan_encoder_chunks,
:881-897).
"""
from __future__ import annotations

from functools import lru_cache
from typing import Dict, List, Optional, Sequence, Tuple


def default_cost(width: int) -> float:
    """Cost model used when no measured table is given: a fixed launch cost per chunk plus a
    per-row cost that falls slightly with width (wider chunks use the tensor cores better)."""
    return 1.0 + width * (1.0 + 64.0 / (64.0 + width)) / 1024.0


def plan_chunks(length: int, widths: Sequence[int], costs: Optional[Dict[int, float]] = None,
                max_exact: int = 4096) -> List[int]:
    """Sizes of the chunks (sum == length).  Chunks are at most max(widths) rows; a chunk
    narrower than a width runs padded in that width's profile and pays that width's cost."""
    if length <= 0:
        return []
    ws = sorted(set(int(w) for w in widths))
    cost = (lambda w: costs[w]) if costs else default_cost
    wmax = ws[-1]
    full, rem = divmod(length, wmax)
    out = [wmax] * full
    # dynamic programme over the remainder in units of the smallest width
    if rem:
        unit = ws[0]
        n_units = -(-rem // unit)
        INF = float("inf")
        best = [0.0] + [INF] * n_units
        choice = [0] * (n_units + 1)
        for u in range(1, n_units + 1):
            for w in ws:
                k = -(-w // unit)
                prev = max(0, u - k)
                c = best[prev] + cost(w)
                if c < best[u]:
                    best[u], choice[u] = c, w
        seq, u = [], n_units
        while u > 0:
            w = choice[u]
            seq.append(w)
            u = max(0, u - (-(-w // unit)))
        seq.sort(reverse=True)
        left = rem
        for w in seq:
            take = min(w, left)
            if take > 0:
                out.append(take)
                left -= take
        if left > 0:
            out.append(left)
    assert sum(out) == length
    return out
