"""Chunked prefill of one conversation.

The prompt is cut into chunks chosen by the planner (``serve/planner.py``); every chunk runs the
encoder layers [0, late_start) on all of its rows.  Layers of the late group read the long
context only through the compressed stream of the last source layer, so they replay just the
last ``window`` rows of the prompt once the encoder has finished (reference:
src/target.rs:6943-7242 prefill_wide_interruptible, :7815 execute_tail; docs/OPERATIONS.md:96-99).
A callback after every chunk lets the scheduler cancel or yield (reference :4520-4531).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.engine import Engine, StepPlan
from .planner import plan_chunks


def _patch_for(embeds, lo: int, T: int, dev):
    """The part of ``embeds`` that falls into prompt offsets [lo, lo+T), as (chunk rows, values)."""
    if embeds is None:
        return None
    offs, vals = embeds
    offs = offs.to(dev)
    m = (offs >= lo) & (offs < lo + T)
    if not bool(m.any()):
        return None
    return (offs[m] - lo).long(), vals.to(dev)[m]


def _recent(plan: StepPlan, cfg, prev, toks: np.ndarray, offset: int) -> StepPlan:
    """Models with Engram layers: give the plan the tokens right before its block (the prompt's own
    rows before ``offset``, and ``prev``, the tokens before the prompt part being prefilled)."""
    if cfg.engram is None or not cfg.engram.layers:
        return plan
    n = cfg.engram.ngram - 1
    before = (list(prev)[-n:] + toks[max(0, offset - n):offset].tolist())[-n:]
    return plan.attach_recent(cfg, [before])


def _encoder_layer_major(eng: Engine, region: int, toks: np.ndarray, sizes: List[int], start: int, late: int,
                         tail: torch.Tensor, tail_n: int, embeds=None, on_chunk=None, prev=()) -> bool:
    """Encoder layers [0, late) layer by layer over ALL chunks of the prompt.

    The residual stream of the whole prompt (n x hidden bf16: 1 GB at 129K tokens) and the current
    index source's selections stay resident between layers, so each layer's weights are touched
    once per prompt instead of once per chunk: the routed experts are re-expressed as FP8 for the
    tensor-core path once per layer, and a layer's dense weights stay in L2 across its chunks.
    Causality holds because layer l of chunk c only needs layer l's own KV of chunks < c (written
    earlier in the same sweep) and layer l-1's output of chunk c."""
    cfg = eng.cfg
    n = int(toks.shape[0])
    resid = torch.empty(n, cfg.hidden * cfg.hc_mult, dtype=torch.bfloat16, device=eng.dev)
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    plans = [_recent(StepPlan.build([(region, start + int(offs[c]), toks[offs[c]:offs[c + 1]].tolist())],
                                    logits="last"), cfg, prev, toks, int(offs[c]))
             for c in range(len(sizes))]
    shapes = [eng.plan_shape(p, cfg.compress_ratio) for p in plans]
    sel_store: dict = {}
    for li in range(late):
        Lw = eng.layers[li]
        src = Lw.index_source if Lw.kv_source >= 0 else -1
        for c, T in enumerate(sizes):
            b = eng._bufs(T)
            eng.upload_plan(plans[c], b)
            lo, hi = int(offs[c]), int(offs[c + 1])
            if src >= 0 and not Lw.is_index_source:
                b["sel"][src][:T].copy_(sel_store[src][0][lo:hi])
                b["selcnt"][src][:T].copy_(sel_store[src][1][lo:hi])
            eng.run(T, b, shapes[c][0], shapes[c][1], None, li, li + 1, x_in=None if li == 0 else resid[lo:hi],
                    x_patch=_patch_for(embeds, lo, T, eng.dev) if li == 0 else None)
            # x + pending sublayer output, rounded once to bf16
            resid[lo:hi].copy_(eng.residual_rows(b, slice(0, T)) if b.get("pending") else b["x"][:T])
            if Lw.is_index_source:
                if li not in sel_store:
                    sel_store.clear()             # followers only ever read the latest source
                    sel_store[li] = (torch.empty(n, b["sel"][li].shape[1], dtype=b["sel"][li].dtype, device=eng.dev),
                                     torch.empty(n, dtype=b["selcnt"][li].dtype, device=eng.dev))
                sel_store[li][0][lo:hi].copy_(b["sel"][li][:T])
                sel_store[li][1][lo:hi].copy_(b["selcnt"][li][:T])
            # the scheduler's hook (cancel / let decoding conversations take a step) runs between
            # units of work; rows count as done only when the last layer has seen them
            if on_chunk is not None and not on_chunk(hi if li == late - 1 else 0):
                return False
    if tail_n > 0:
        tail[:tail_n].copy_(resid[n - tail_n:])
    # leave the last chunk's residual in its buffers for a head that follows directly
    T = sizes[-1]
    b = eng._bufs(T)
    b["x"][:T].copy_(resid[n - T:])
    b["pending"] = False
    return True


def _encoder_sequence_parallel(eng: Engine, region: int, toks: np.ndarray, chunk: int, start: int, late: int,
                               tail: torch.Tensor, tail_n: int, embeds=None, on_chunk=None) -> bool:
    """Encoder layers [0, late) with every chunk's rows split over the ranks (``parallel/sp.py``),
    layer by layer over all chunks like the single-rank sweep above.  Every rank keeps the residual
    rows of ITS slices between layers; the KV state ends up identical on all ranks."""
    cfg, sp = eng.cfg, eng.sp
    n = int(toks.shape[0])
    sp._plans.clear()
    sizes = sp.chunk_sizes(n, chunk)
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    d = cfg.hidden
    resid: List[Optional[torch.Tensor]] = [None] * len(sizes)
    sel_store: dict = {}
    for li in range(late):
        Lw = sp.view.layers[li]
        src = Lw.index_source if Lw.kv_source >= 0 else -1
        for c, Tc in enumerate(sizes):
            lo, hi, _ = sp.bounds(Tc)
            sel_in = None
            if src >= 0 and not Lw.is_index_source and hi > lo:
                sel_in = (src, sel_store[src][c][0], sel_store[src][c][1])
            xp = _patch_for(embeds, int(offs[c]) + lo, hi - lo, eng.dev) if (li == 0 and hi > lo) else None
            b, lo, T = sp.run_layer(li, region, start + int(offs[c]), Tc, toks[offs[c]:offs[c + 1]],
                                    None if li == 0 else resid[c], xp, sel_in)
            if T > 0:
                # x + pending sublayer output, rounded once to bf16
                resid[c] = (sp.view.residual_rows(b, slice(0, T)) if b.get("pending") else b["x"][:T].clone())
                if Lw.is_index_source:
                    if li not in sel_store:
                        sel_store.clear()             # followers only ever read the latest source
                        sel_store[li] = {}
                    sel_store[li][c] = (b["sel"][li][:T].clone(), b["selcnt"][li][:T].clone())
            if on_chunk is not None and not on_chunk(int(offs[c + 1]) if li == late - 1 else 0):
                return False
    # the rows the late group replays (and a head that follows directly) come from the last chunk(s)
    last = len(sizes) - 1
    full_last = sp.gather_rows(resid[last], sizes[last], d, torch.bfloat16).clone()
    if tail_n > 0:
        if sizes[last] >= tail_n:
            tail[:tail_n].copy_(full_last[sizes[last] - tail_n:])
        else:
            prev = sp.gather_rows(resid[last - 1], sizes[last - 1], d, torch.bfloat16)
            tail[:tail_n].copy_(torch.cat([prev, full_last])[-tail_n:])
    T = min(sizes[-1], eng.max_chunk)              # (a head that follows needs the last row only)
    b = eng._bufs(T)
    b["x"][:T].copy_(full_last[sizes[-1] - T:])
    b["pending"] = False
    eng._sp_last_rows = T
    return True


def run_prefill(eng: Engine, region: int, tokens, chunk: int, start: int = 0, need_logits: bool = True,
                on_chunk: Optional[Callable[[int], bool]] = None,
                widths: Optional[Sequence[int]] = None, layer_major: Optional[bool] = None,
                embeds: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                prev: Sequence[int] = ()) -> Optional[torch.Tensor]:
    """Prefill ``tokens`` at positions start.. into ``region``.  Returns fp32 logits of the last
    row (or None when cancelled by ``on_chunk`` returning False).  ``embeds`` = (prompt offsets
    [m], rows [m, hidden]) replaces the token embedding at those offsets (image spans).  ``prev``:
    the tokens right before ``start`` (models with Engram layers hash n-grams across the seam)."""
    cfg = eng.cfg
    toks = np.asarray(tokens.cpu() if isinstance(tokens, torch.Tensor) else tokens, dtype=np.int32)
    n = int(toks.shape[0])
    L = len(eng.layers)
    late = cfg.late_start if 0 < cfg.late_start < L else L
    tail_n = min(n, cfg.window) if late < L else 0
    tail = torch.zeros(max(tail_n, 1), cfg.hidden * cfg.hc_mult, dtype=torch.bfloat16, device=eng.dev)
    sp = getattr(eng, "sp", None)
    if sp is not None and embeds is None and not sp.usable(start, n):
        # a prefill that begins inside a compressor group (a conversation resumed right after its
        # last committed token): the rows up to the next group boundary take the tensor-parallel
        # path through the encoder layers, the rest is split over the ranks
        k = (-start) % cfg.max_ratio
        if 0 < k and n - k >= max(cfg.window, 1) and sp.usable(start + k, n - k):
            plan = _recent(StepPlan.build([(region, start, toks[:k].tolist())], logits="last"), cfg, prev, toks, 0)
            b = eng._bufs(k)
            eng.upload_plan(plan, b)
            nmax, rpg = eng.plan_shape(plan, cfg.compress_ratio)
            eng.run(k, b, nmax, rpg, None, 0, late)
            cb = None if on_chunk is None else (lambda done: on_chunk(done + k))
            return run_prefill(eng, region, toks[k:], chunk, start + k, need_logits, cb, widths, layer_major, None,
                               (list(prev) + toks[:k].tolist())[-8:] if len(prev) else ())
    sizes = plan_chunks(n, tuple(widths) if widths else (chunk,))
    if layer_major is None:
        layer_major = len(sizes) > 1 and getattr(eng, "big_moe_full", None) is not None
    done = 0
    logits = None
    if getattr(eng, "sp", None) is not None and eng.sp.usable(start, n):
        # more than one rank: the rows of every chunk are split over the ranks
        if not _encoder_sequence_parallel(eng, region, toks, chunk, start, late, tail, tail_n, embeds, on_chunk):
            return None
        if late == L and need_logits:
            Tl = eng._sp_last_rows
            logits = eng._head(Tl, eng._bufs(Tl), torch.tensor([Tl - 1], device=eng.dev))
        sizes = []
    elif layer_major:
        if not _encoder_layer_major(eng, region, toks, sizes, start, late, tail, tail_n, embeds, on_chunk, prev):
            return None
        if late == L and need_logits:
            logits = eng._head(sizes[-1], eng._bufs(sizes[-1]), torch.tensor([sizes[-1] - 1], device=eng.dev))
        sizes = []
    for T in sizes:
        plan = _recent(StepPlan.build([(region, start + done, toks[done:done + T].tolist())], logits="last"),
                       cfg, prev, toks, done)
        b = eng._bufs(T)
        eng.upload_plan(plan, b)
        nmax, rpg = eng.plan_shape(plan, cfg.compress_ratio)
        last_chunk = done + T == n
        rows = torch.tensor([T - 1], device=eng.dev) if (late == L and last_chunk and need_logits) else None
        out = eng.run(T, b, nmax, rpg, rows, 0, late, x_patch=_patch_for(embeds, done, T, eng.dev))
        if late < L:
            # keep the encoder output of the prompt's last `window` rows for the late-group replay
            lo = max(done, n - tail_n)
            if lo < done + T:
                r = torch.arange(lo - done, T, device=eng.dev)
                tail[lo - (n - tail_n): lo - (n - tail_n) + r.numel()] = eng.residual_rows(b, r)
        else:
            logits = out
        done += T
        if on_chunk is not None and not on_chunk(done):
            return None
    if late < L and tail_n > 0:
        p0 = start + n - tail_n
        plan = _recent(StepPlan.build([(region, p0, toks[n - tail_n:].tolist())], logits="last"),
                       cfg, prev, toks, n - tail_n)
        plan.min_pos = np.full(tail_n, p0, dtype=np.int32)     # older rows never ran in the late group
        b = eng._bufs(tail_n)
        eng.upload_plan(plan, b)
        nmax, rpg = eng.plan_shape(plan, cfg.compress_ratio)
        rows = torch.tensor([tail_n - 1], device=eng.dev) if need_logits else None
        logits = eng.run(tail_n, b, nmax, rpg, rows, late, L, x_in=tail[:tail_n])
    return logits
