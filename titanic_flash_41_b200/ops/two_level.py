"""Two-level index selection for long rows.

A *publisher* layer scores every key, and besides its own top-k keeps the ``n_blocks`` best blocks
of 8 consecutive keys (by block maximum).  *Consumer* layers score only the keys inside those
blocks (plus the newest keys, which the publisher has not seen) and select their top-k among
them.  Scoring cost of a consumer is then bounded by 8 * n_blocks keys however long the context
is (reference: src/candidates.rs:1-20 Publisher / consumers, kernels/candidate_block_scores.cuh,
kernels/sparse_index.cuh; src/sparse_index.rs candidate-only scoring).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import native

BLOCK = 8


def publish(scores: torch.Tensor, nvalid: torch.Tensor, n_blocks: int, T: int) -> torch.Tensor:
    """scores [T, lds] of the publisher -> candidate key ids [T, n_blocks * 8] ascending, -1 padded."""
    dev = scores.device
    lds = scores.stride(0)
    nblk = (int(scores.shape[1]) + BLOCK - 1) // BLOCK
    bmax = torch.empty(T, nblk, dtype=torch.float32, device=dev)
    native.call("tf_index_block_max", scores, lds, nvalid, bmax, nblk, nblk, T)
    nb_valid = ((nvalid[:T] + BLOCK - 1) // BLOCK).to(torch.int32).contiguous()
    blocks = torch.full((T, n_blocks), -1, dtype=torch.int32, device=dev)
    cnt = torch.zeros(T, dtype=torch.int32, device=dev)
    native.call("tf_topk_select", bmax, nblk, nb_valid, n_blocks, blocks, cnt, None, 0, T)
    ids = blocks[:, :, None] * BLOCK + torch.arange(BLOCK, device=dev, dtype=torch.int32)[None, None, :]
    ok = (blocks[:, :, None] >= 0) & (ids < nvalid[:T, None, None])
    return torch.where(ok, ids, torch.full_like(ids, -1)).reshape(T, n_blocks * BLOCK).contiguous()


def consume(q, w, region, cand: torch.Tensor, keys, key_region_stride: int, key_row: int, T: int, Hi: int, Di: int,
            k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Score the candidates of each row and return (ids [T, k] ascending, -1 padded; count [T])."""
    dev = cand.device
    C = cand.shape[1]
    sc = torch.empty(T, C, dtype=torch.float32, device=dev)
    native.call("tf_index_scores_sparse", q, w, region, cand, cand.stride(0), keys, key_region_stride, key_row, T, Hi, Di,
                C, sc, C)
    picked = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    cnt = torch.zeros(T, dtype=torch.int32, device=dev)
    nv = torch.full((T,), C, dtype=torch.int32, device=dev)
    native.call("tf_topk_select", sc, C, nv, k, picked, cnt, None, 0, T)
    ids = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    native.call("tf_map_ids", picked, cand, cand.stride(0), k, ids, T)
    # padding candidates (-1, score -inf) can only be picked when fewer than k real ones exist
    big = torch.iinfo(torch.int32).max
    key = torch.where(ids >= 0, ids, torch.full_like(ids, big))
    key, _ = torch.sort(key, dim=1)
    count = (key != big).sum(1).to(torch.int32)
    return torch.where(key == big, torch.full_like(key, -1), key), count
