"""Admission and region assignment.

At most ``regions`` requests are admitted (one serving region each); the rest wait in a bounded
FIFO queue and are refused with ``QueueFull`` beyond it; background requests have their own
bound and yield to foreground ones; a priority lease lets a router hold background work for a
while.  Reference: src/http_server.rs:414 Queue, :912-923 queue_full / background_queue_full,
src/batched_admission.rs, src/router_priority.rs (``/_native/priority`` leases).
"""
from __future__ import annotations

import collections
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional


class QueueFull(Exception):
    def __init__(self, code: str):
        super().__init__(code)
        self.code = code


@dataclass
class Job:
    id: str
    tokens: List[int]
    max_new_tokens: int
    temperature: float = 1.0
    top_p: float = 1.0
    seed: int = 0
    background: bool = False
    media: str = ""
    images: list = field(default_factory=list)
    emit: Callable[[str, Any], None] = lambda kind, payload: None     # events to the HTTP side
    cancelled: threading.Event = field(default_factory=threading.Event)
    submitted: float = field(default_factory=time.monotonic)
    # filled by the worker
    region: int = -1
    generated: List[int] = field(default_factory=list)
    cache_n: int = 0
    prompt_ms: float = 0.0


class Scheduler:
    def __init__(self, regions: int = 4, queue_limit: int = 16, background_limit: int = 4):
        self.regions = regions
        self.queue_limit, self.background_limit = queue_limit, background_limit
        self.fg: Deque[Job] = collections.deque()
        self.bg: Deque[Job] = collections.deque()
        self.active: Dict[int, Job] = {}
        self.lock = threading.Condition()
        self.hold_background_until = 0.0
        self.closed = False

    # ---- HTTP side ----------------------------------------------------------------------------
    def submit(self, job: Job) -> None:
        with self.lock:
            if self.closed:
                raise QueueFull("shutting_down")
            q, limit, code = (self.bg, self.background_limit, "background_queue_full") if job.background \
                else (self.fg, self.queue_limit, "queue_full")
            if len(q) >= limit:
                raise QueueFull(code)
            q.append(job)
            self.lock.notify_all()

    def priority_lease(self, seconds: float) -> float:
        """Hold background admissions for ``seconds`` (bounded to a minute); returns the deadline."""
        with self.lock:
            self.hold_background_until = time.monotonic() + max(0.0, min(seconds, 60.0))
            return self.hold_background_until

    def waiting(self) -> int:
        with self.lock:
            return len(self.fg) + len(self.bg)

    # ---- worker side --------------------------------------------------------------------------
    def free_regions(self) -> List[int]:
        return [r for r in range(self.regions) if r not in self.active]

    def admit(self, now: Optional[float] = None) -> List[Job]:
        """Move waiting jobs into free regions: foreground first, FIFO inside a class."""
        now = time.monotonic() if now is None else now
        out = []
        with self.lock:
            for r in self.free_regions():
                job = None
                while self.fg and job is None:
                    j = self.fg.popleft()
                    job = None if self._dropped(j) else j
                if job is None and now >= self.hold_background_until:
                    while self.bg and job is None:
                        j = self.bg.popleft()
                        job = None if self._dropped(j) else j
                if job is None:
                    break
                job.region = r
                self.active[r] = job
                out.append(job)
        return out

    @staticmethod
    def _dropped(j: Job) -> bool:
        """A job cancelled while it waited never reaches a region; its HTTP handler still gets a
        terminal event, so it does not wait forever."""
        if not j.cancelled.is_set():
            return False
        try:
            j.emit("error", {"code": "cancelled", "message": "cancelled while queued"})
        except Exception:  # noqa: BLE001  (a dead client must not stop admission)
            pass
        return True

    def occupy(self, job: Job, region: int) -> None:
        """A parked conversation returns to a region (the worker resumes it there)."""
        with self.lock:
            if region in self.active:
                raise RuntimeError(f"region {region} is not free")
            job.region = region
            self.active[region] = job

    def oldest_submitted(self) -> float:
        """Submission time of the request at the head of the queue (inf when nothing waits)."""
        with self.lock:
            heads = [q[0].submitted for q in (self.fg, self.bg) if q]
            return min(heads) if heads else float("inf")

    def release(self, job: Job) -> None:
        with self.lock:
            if self.active.get(job.region) is job:
                del self.active[job.region]
            self.lock.notify_all()

    def wait_for_work(self, timeout: float) -> bool:
        with self.lock:
            if self.fg or self.bg or self.active:
                return True
            self.lock.wait(timeout)
            return bool(self.fg or self.bg or self.active)

    def close(self) -> None:
        with self.lock:
            self.closed = True
            self.lock.notify_all()
