"""Sticky health of one rank and the watchdog that keeps it current.

Everything that can make a cohort unusable ends in ONE place: the device status word of the
kernels (a bounded wait that ran out, a bad index, a non-finite probability), a poisoned control
channel (peer closed, frame out of order, diverging agreement), a process-group error raised by a
collective, an exception of the worker loop.  The first report wins and stays: a poisoned rank
never reports healthy again, it retires and the cohort is restarted from outside (reference:
src/roce.rs:442-461 health(), src/collective.rs:255 check_async; there is no elastic recovery in
the reference either).  ``/health`` serves the record; the launcher's supervisor stops the other
ranks when one leaves.

Nothing here touches the GPU: probes read host-side state (the status word arrives through a
pinned copy that the owner thread refreshes between steps).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, Optional

STATUS_CODES = {1: "bad_arg", 2: "timeout", 3: "bad_index", 4: "nonfinite"}


class Health:
    def __init__(self):
        self._lock = threading.Lock()
        self.poisoned: Optional[dict] = None
        self.beats = 0
        self.last_beat = time.monotonic()

    def report(self, source: str, why: str) -> bool:
        """Record a fatal condition; returns True when this call poisoned the rank (first report)."""
        with self._lock:
            if self.poisoned is not None:
                return False
            self.poisoned = {"source": source, "why": str(why), "at": round(time.time(), 3)}
            return True

    def beat(self) -> None:
        self.beats += 1
        self.last_beat = time.monotonic()

    @property
    def ok(self) -> bool:
        return self.poisoned is None

    def state(self) -> dict:
        with self._lock:
            out = {"poisoned": self.poisoned is not None, "beats": self.beats,
                   "idle_s": round(time.monotonic() - self.last_beat, 3)}
            if self.poisoned is not None:
                out.update(self.poisoned)
            return out


def control_probe(control) -> Callable[[], Optional[str]]:
    """Poison of the control channel (None while it is healthy or absent)."""
    return lambda: (getattr(control, "poisoned", None) if control is not None else None)


def status_probe(snapshot: Callable[[], Optional[tuple]]) -> Callable[[], Optional[str]]:
    """``snapshot`` returns the last host copy of the device status word (code, kernel, d0, d1)."""
    def probe():
        w = snapshot()
        if not w or int(w[0]) == 0:
            return None
        return f"kernel {int(w[1])} reported {STATUS_CODES.get(int(w[0]), int(w[0]))} (detail {int(w[2])}, {int(w[3])})"
    return probe


class Watchdog(threading.Thread):
    """Polls the probes every ``interval`` seconds and folds the first failure into ``health``."""

    def __init__(self, health: Health, probes: Dict[str, Callable[[], Optional[str]]], interval: float = 0.5,
                 on_poison: Optional[Callable[[dict], None]] = None):
        super().__init__(daemon=True, name="tflash-watchdog")
        self.health, self.probes, self.interval, self.on_poison = health, dict(probes), interval, on_poison
        self._stop = threading.Event()

    def poll_once(self) -> bool:
        for name, probe in self.probes.items():
            try:
                why = probe()
            except Exception as e:  # noqa: BLE001  (a probe that fails is itself a finding)
                why = f"probe failed: {e!r}"
            if why and self.health.report(name, why):
                if self.on_poison is not None:
                    try:
                        self.on_poison(self.health.state())
                    except Exception:  # noqa: BLE001
                        pass
        return self.health.ok

    def run(self) -> None:
        while not self._stop.is_set():
            if not self.poll_once():
                return
            self._stop.wait(self.interval)

    def stop(self) -> None:
        self._stop.set()


class CohortHeartbeat(threading.Thread):
    """Host-side heartbeat of the whole cohort on its OWN gloo process group.

    Every ``interval`` seconds each rank's heartbeat thread joins one small all-reduce that carries
    every rank's health flag.  Two things follow.  A rank that reported a fatal condition poisons
    the others within one interval ("rank 3 is poisoned"), instead of at their next device
    collective; and a rank whose process died or stopped on the host makes the all-reduce fail or
    time out on the others after ``timeout`` seconds, long before a device collective would give up
    (the default process-group timeout is minutes).  This is the job of the reference's async-error
    poll on its communicator (src/collective.rs:255 check_async), done on the host: nothing here
    touches the GPU or the device communicator, so it can run beside captured graphs.

    The group must be created by every rank in the same order (``CohortHeartbeat.make_group``, a
    collective call); the thread only ever issues collectives on that group.
    """

    def __init__(self, health: Health, group, rank: int, world: int, interval: float = 1.0):
        super().__init__(daemon=True, name="tflash-heartbeat")
        self.health, self.group, self.rank, self.world, self.interval = health, group, rank, world, interval
        self.failed: Optional[str] = None
        self.rounds = 0
        self._stop = threading.Event()

    @staticmethod
    def make_group(timeout: float = 10.0):
        import datetime

        import torch.distributed as dist
        return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout))

    def beat_once(self) -> Optional[str]:
        """One round; returns what is wrong with the cohort (None: every rank is alive and healthy)."""
        import torch
        import torch.distributed as dist
        flags = torch.zeros(self.world, dtype=torch.int32)
        flags[self.rank] = 1 if self.health.ok else 2
        try:
            dist.all_reduce(flags, group=self.group)
        except Exception as e:  # noqa: BLE001  (a peer that left, a timeout: both mean the cohort is gone)
            return f"cohort heartbeat failed: {e!r}"
        self.rounds += 1
        bad = [r for r in range(self.world) if int(flags[r]) != 1]
        if bad:
            return "rank(s) %s %s" % (bad, "poisoned" if all(int(flags[r]) == 2 for r in bad) else "missed the heartbeat")
        return None

    def run(self) -> None:
        while not self._stop.is_set():
            why = self.beat_once()
            if self._stop.is_set():
                return                          # stopping: a peer that already left is not a failure
            if why is not None:
                self.failed = why
                self.health.report("cohort", why)
                if not why.startswith("rank(s)"):
                    return                      # the group itself is broken: no further rounds
            if not self.health.ok and self.failed is not None and self.rounds > 0:
                # one more round has told the others; a poisoned rank retires
                return
            self._stop.wait(self.interval)

    def probe(self) -> Callable[[], Optional[str]]:
        return lambda: self.failed

    def stop(self) -> None:
        self._stop.set()
