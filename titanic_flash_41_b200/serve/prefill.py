"""Chunked prefill of one conversation.

The prompt is cut into chunks chosen by the planner (``serve/planner.py``); every chunk runs the
encoder layers [0, late_start) on all of its rows.  Layers of the late group read the long
context only through the compressed stream of the last source layer, so they replay just the
last ``window`` rows of the prompt once the encoder has finished (reference:
src/target.rs:6943-7242 prefill_wide_interruptible, :7815 execute_tail; docs/OPERATIONS.md:96-99).
A callback after every chunk lets the scheduler cancel or yield (reference :4520-4531).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from ..models.engine import Engine, StepPlan
from .planner import plan_chunks


def run_prefill(eng: Engine, region: int, tokens, chunk: int, start: int = 0, need_logits: bool = True,
                on_chunk: Optional[Callable[[int], bool]] = None,
                widths: Optional[Sequence[int]] = None) -> Optional[torch.Tensor]:
    """Prefill ``tokens`` at positions start.. into ``region``.  Returns fp32 logits of the last
    row (or None when cancelled by ``on_chunk`` returning False)."""
    cfg = eng.cfg
    toks = np.asarray(tokens.cpu() if isinstance(tokens, torch.Tensor) else tokens, dtype=np.int32)
    n = int(toks.shape[0])
    L = len(eng.layers)
    late = cfg.late_start if 0 < cfg.late_start < L else L
    tail_n = min(n, cfg.window) if late < L else 0
    tail = torch.zeros(max(tail_n, 1), cfg.hidden, dtype=torch.bfloat16, device=eng.dev)
    sizes = plan_chunks(n, tuple(widths) if widths else (chunk,))
    done = 0
    logits = None
    for T in sizes:
        plan = StepPlan.build([(region, start + done, toks[done:done + T].tolist())], logits="last")
        b = eng._bufs(T)
        eng.upload_plan(plan, b)
        nmax, rpg = eng.plan_shape(plan, cfg.compress_ratio)
        last_chunk = done + T == n
        rows = torch.tensor([T - 1], device=eng.dev) if (late == L and last_chunk and need_logits) else None
        out = eng.run(T, b, nmax, rpg, rows, 0, late)
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
        plan = StepPlan.build([(region, p0, toks[n - tail_n:].tolist())], logits="last")
        plan.min_pos = np.full(tail_n, p0, dtype=np.int32)     # older rows never ran in the late group
        b = eng._bufs(tail_n)
        eng.upload_plan(plan, b)
        nmax, rpg = eng.plan_shape(plan, cfg.compress_ratio)
        rows = torch.tensor([tail_n - 1], device=eng.dev) if need_logits else None
        logits = eng.run(tail_n, b, nmax, rpg, rows, late, L, x_in=tail[:tail_n])
    return logits
