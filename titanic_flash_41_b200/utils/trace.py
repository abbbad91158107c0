"""Diagnostics that stay out of the serving path unless switched on.

``KernelClock``   times every exported kernel call with CUDA events on the launching stream and
                  folds them by (part, kernel) — the layer clock of the engine: ``part(name)``
                  marks forward parts (attention, moe, head...), ``report()`` gives the table a
                  request's ``timings`` carries (reference: src/layer_clock.rs:45 arm, :135 part,
                  :148 mark, :99 parts_us; globaltimer marks become event pairs here).
``GraphClock``    device timestamps (``tf_stamp``: the GPU's global timer, one tiny kernel) in front of
                  every exported kernel call while a CUDA graph is captured; every replay refreshes
                  them, so the table shows where the time goes INSIDE the graph, which CUDA events
                  cannot do (reference: the globaltimer marks of src/layer_clock.rs).
``Knockout``      skips named kernels so that their cost can be bounded by difference; results are
                  wrong on purpose while it is active (reference: src/knockout.rs:37-63).
``RouteCensus``   per-expert routing counts from the router's id tensor
                  (reference: src/route_census.rs; kernels/core.cu:161 ca_route_census).

Timing serialises nothing by itself, but reading the table synchronises the device once.
Delay / fault injection on the device is deliberately absent: failures are injected on the host.
"""
from __future__ import annotations

import contextlib
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..ops import native


class KernelClock:
    def __init__(self, shapes: bool = False):
        self.shapes = shapes      # split the weight-streaming GEMV rows of the table by matrix shape
        self.events: List[Tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = []
        self._part = "-"
        self._orig = None

    def part(self, name: str) -> None:
        self._part = name

    def __enter__(self):
        self._orig = native.call
        clock = self

        def timed(name, *args, **kw):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                return clock._orig(name, *args, **kw)
            finally:
                b.record()
                if name == "tf_smallm_gemm" and clock.shapes:
                    # kind, output features x inputs, fused second matrix
                    name = "%s[k%d %dx%d%s]" % (name, args[0], args[14], args[15], " dual" if args[2] is not None else "")
                clock.events.append((clock._part, name, a, b))
        native.call = timed
        return self

    def __exit__(self, *exc):
        native.call = self._orig
        self._orig = None
        return False

    def table(self, by_part: bool = False) -> List[Tuple[str, int, float]]:
        """[(key, calls, total_ms)] sorted by time; one device synchronisation."""
        torch.cuda.synchronize()
        tot: Dict[str, List[float]] = defaultdict(lambda: [0, 0.0])
        for part, name, a, b in self.events:
            k = f"{part}/{name}" if by_part else name
            tot[k][0] += 1
            tot[k][1] += a.elapsed_time(b)
        return sorted(((k, int(v[0]), v[1]) for k, v in tot.items()), key=lambda r: -r[2])

    def report(self, by_part: bool = False, top: int = 20) -> str:
        rows = self.table(by_part)
        total = sum(r[2] for r in rows) or 1.0
        out = [f"{'kernel':34s} {'calls':>7s} {'ms':>10s} {'share':>7s}"]
        for k, n, ms in rows[:top]:
            out.append(f"{k:34s} {n:7d} {ms:10.3f} {100 * ms / total:6.1f}%")
        out.append(f"{'total':34s} {sum(r[1] for r in rows):7d} {total:10.3f}")
        return "\n".join(out)


class GraphClock:
    """Use: ``with clock:`` around the CAPTURE of a graph (or around eager launches), replay the
    graph, synchronise, then ``table()``.  A stamp precedes and follows every exported kernel call on
    the stream the call goes to, so a call's time is the difference of its own two stamps (it
    includes one stamp, about 2 us); PyTorch's own kernels and the launch gaps between calls are what
    is left of the span.  Calls on a side stream overlap the main stream: the rows need not add up
    to the span."""

    def __init__(self, capacity: int = 8192, device="cuda"):
        self.capacity = capacity
        self.ring = torch.zeros(capacity, dtype=torch.int64, device=device)
        self.marks: List[str] = []          # kernel name per call; call i owns slots 2i (before) and 2i + 1 (after)
        self._orig = None

    def __enter__(self):
        self.marks.clear()
        self._orig = native.call
        clock = self

        def stamped(name, *args, **kw):
            i = len(clock.marks)
            if 2 * i + 1 >= clock.capacity:
                return clock._orig(name, *args, **kw)
            clock.marks.append(name)
            clock._orig("tf_stamp", clock.ring, 2 * i, clock.capacity)
            try:
                return clock._orig(name, *args, **kw)
            finally:
                clock._orig("tf_stamp", clock.ring, 2 * i + 1, clock.capacity)
        native.call = stamped
        return self

    def __exit__(self, *exc):
        native.call = self._orig
        self._orig = None
        return False

    def _times(self):
        torch.cuda.synchronize()
        return self.ring[: 2 * len(self.marks)].cpu().tolist()

    def table(self) -> List[Tuple[str, int, float]]:
        """(kernel, calls, microseconds) of the last run of the stamped launches, largest first."""
        t = self._times()
        acc: Dict[str, List[float]] = defaultdict(lambda: [0, 0.0])
        for i, name in enumerate(self.marks):
            acc[name][0] += 1
            acc[name][1] += max(0, t[2 * i + 1] - t[2 * i]) / 1e3
        return sorted(((k, int(v[0]), v[1]) for k, v in acc.items()), key=lambda r: -r[2])

    def span_us(self) -> float:
        """First stamp to last stamp of the last run."""
        t = self._times()
        return (max(t) - min(t)) / 1e3 if t else 0.0

    def report(self, top: int = 24) -> str:
        rows = self.table()
        total = sum(r[2] for r in rows) or 1.0
        span = self.span_us()
        out = ["%-32s %6s %10s %6s" % ("kernel (inside the graph)", "calls", "us", "% span")]
        for name, n, us in rows[:top]:
            out.append("%-32s %6d %10.1f %5.1f%%" % (name, n, us, 100 * us / max(span, 1e-9)))
        out.append("%-32s %6d %10.1f  (first to last stamp %.1f us; side-stream calls overlap the main stream)"
                   % ("all calls", len(self.marks), total, span))
        return "\n".join(out)


class Knockout(contextlib.AbstractContextManager):
    """``with Knockout({"tf_index_scores", "tf_topk_select"}): ...`` skips those launches."""

    def __init__(self, names: Iterable[str]):
        self.names, self._orig, self.skipped = set(names), None, 0

    def __enter__(self):
        self._orig = native.call
        ko = self

        def gated(name, *args, **kw):
            if name in ko.names:
                ko.skipped += 1
                return None
            return ko._orig(name, *args, **kw)
        native.call = gated
        return self

    def __exit__(self, *exc):
        native.call = self._orig
        return False


class RouteCensus:
    """Accumulates how often each expert was chosen."""

    def __init__(self, n_experts: int, device="cpu"):
        self.counts = torch.zeros(n_experts, dtype=torch.int64, device=device)

    def add(self, ids: torch.Tensor) -> None:
        flat = ids.reshape(-1).to(self.counts.device, torch.int64)
        self.counts += torch.bincount(flat[flat >= 0], minlength=self.counts.numel())[: self.counts.numel()]

    def summary(self) -> dict:
        c = self.counts.float()
        mean = float(c.mean()) or 1.0
        return {"total": int(c.sum()), "max_over_mean": float(c.max()) / mean, "unused": int((c == 0).sum()),
                "top": [int(i) for i in torch.topk(c, min(8, c.numel())).indices]}


class LogitExport:
    """Keeps the raw logits of chosen positions for offline divergence studies and writes them as
    one ``.npz`` (reference: src/logit_export.rs).  Off unless constructed."""

    def __init__(self, path: str, limit: int = 4096):
        self.path, self.limit = path, limit
        self.rows: Dict[int, "torch.Tensor"] = {}

    def add(self, position: int, logits: torch.Tensor) -> None:
        if len(self.rows) < self.limit:
            self.rows[int(position)] = logits.detach().float().cpu().reshape(-1).clone()

    def save(self) -> int:
        import numpy as np
        pos = sorted(self.rows)
        np.savez_compressed(self.path, positions=np.asarray(pos, dtype=np.int64),
                            logits=np.stack([self.rows[p].numpy() for p in pos]) if pos else np.zeros((0, 0), np.float32))
        return len(pos)


class DrawTrace:
    """One record per speculative step and conversation: position, proposals, uniforms used, accepted
    count and the committed token (reference: src/draw_trace.rs).  Bounded ring."""

    def __init__(self, capacity: int = 65536):
        self.capacity = capacity
        self.records: List[dict] = []

    def add(self, **rec) -> None:
        if len(self.records) >= self.capacity:
            del self.records[: self.capacity // 8]
        self.records.append(rec)

    def acceptance_histogram(self) -> Dict[int, int]:
        h: Dict[int, int] = defaultdict(int)
        for r in self.records:
            h[int(r.get("accepted", 0))] += 1
        return dict(h)

    def dump(self, path: str) -> None:
        import json
        with open(path, "w") as f:
            for r in self.records:
                f.write(json.dumps(r) + "\n")
