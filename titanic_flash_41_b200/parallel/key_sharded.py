"""Key-sharded index selection: split the scoring of one long row of keys across ranks.

Every rank holds all index keys (the latent cache is replicated), so sharding is a division of
work, not of memory: rank r scores keys [r*C/W, (r+1)*C/W), keeps its local top-k, the
(score, id) pairs of all ranks are gathered, and the same exact selection kernel picks the
global top-k from the W*k candidates.  The local top-k of every shard contains every global
winner that lives in the shard, and candidates arrive in key order, so the result (ids ascending,
ties to the lower position) is identical to unsharded selection (reference:
src/key_sharded_index.rs:1-53 local top-512 -> gather -> merge; src/key_sharded_publisher.rs).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from ..ops import native

INT_MAX = 2 ** 31 - 1


def shard_range(n_keys: int, rank: int, world: int, align: int = 128) -> Tuple[int, int]:
    per = -(-n_keys // world)
    per = -(-per // align) * align
    return min(n_keys, rank * per), min(n_keys, (rank + 1) * per)


def local_candidates(q, w, region, nvalid, keys, key_region_stride: int, key_row: int, T: int, Hi: int, Di: int,
                     rows_per_group: int, scores: torch.Tensor, n_keys: int, k: int, rank: int, world: int
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Score this rank's key range and keep its top-k: (scores [T, k] with -inf padding, ids [T, k] with -1)."""
    lo, hi = shard_range(n_keys, rank, world)
    dev = scores.device
    ids = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    sc = torch.full((T, k), float("-inf"), dtype=torch.float32, device=dev)
    cnt = torch.zeros(T, dtype=torch.int32, device=dev)
    if hi > lo:
        native.call("tf_index_scores", q, w, region, nvalid, keys, key_region_stride, key_row, T, Hi, Di, rows_per_group,
                    scores, scores.stride(0), lo, hi)
        nv_local = (nvalid[:T] - lo).clamp(0, hi - lo).to(torch.int32).contiguous()
        native.call("tf_topk_select", scores[:, lo:], scores.stride(0), nv_local, k, ids, cnt, sc, lo, T)
        sc = torch.where(ids >= 0, sc, torch.full_like(sc, float("-inf")))
    return sc, ids


def merge(cand_scores: torch.Tensor, cand_ids: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cand_* [T, W*k] in rank (= key) order -> (ids [T, k] ascending with -1 padding, count [T])."""
    T, n = cand_scores.shape
    dev = cand_scores.device
    picked = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    cnt = torch.zeros(T, dtype=torch.int32, device=dev)
    nv = torch.full((T,), n, dtype=torch.int32, device=dev)
    cs = cand_scores.contiguous()
    native.call("tf_topk_select", cs, cs.stride(0), nv, k, picked, cnt, None, 0, T)
    ids = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    ci = cand_ids.to(torch.int32).contiguous()
    native.call("tf_map_ids", picked, ci, ci.stride(0), k, ids, T)
    # candidates that were only padding come back as -1: move them behind the real ids
    key = torch.where(ids >= 0, ids, torch.full_like(ids, INT_MAX))
    key, _ = torch.sort(key, dim=1)
    count = (key != INT_MAX).sum(1).to(torch.int32)
    return torch.where(key == INT_MAX, torch.full_like(key, -1), key), count


def select(q, w, region, nvalid, keys, key_region_stride: int, key_row: int, T: int, Hi: int, Di: int,
           rows_per_group: int, scores: torch.Tensor, n_keys: int, k: int, rank: int, world: int,
           gather: Callable[[torch.Tensor], torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gather(t)`` concatenates every rank's ``t`` along dim 1 in rank order (an all-gather)."""
    sc, ids = local_candidates(q, w, region, nvalid, keys, key_region_stride, key_row, T, Hi, Di, rows_per_group, scores,
                               n_keys, k, rank, world)
    return merge(gather(sc), gather(ids), k)
