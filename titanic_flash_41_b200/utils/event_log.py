"""Bounded in-memory event rings (general + incident) with an optional rotating disk trace,
served by ``GET /_native/diagnostics`` (reference: src/event_log.rs:172-247)."""
from __future__ import annotations

import collections
import json
import os
import threading
import time
from typing import Any, Deque, Dict, List, Optional


class EventLog:
    def __init__(self, capacity: int = 1024, incident_capacity: int = 128, trace_path: Optional[str] = None,
                 trace_bytes: int = 8 << 20):
        self.general: Deque[Dict[str, Any]] = collections.deque(maxlen=capacity)
        self.incidents: Deque[Dict[str, Any]] = collections.deque(maxlen=incident_capacity)
        self.trace_path, self.trace_bytes = trace_path, trace_bytes
        self.lock = threading.Lock()
        self.seq = 0
        self.dropped = 0

    def log(self, kind: str, incident: bool = False, **fields) -> None:
        with self.lock:
            self.seq += 1
            ev = {"seq": self.seq, "t": round(time.time(), 3), "kind": kind, **fields}
            ring = self.incidents if incident else self.general
            if len(ring) == ring.maxlen:
                self.dropped += 1
            ring.append(ev)
            if self.trace_path:
                self._trace(ev)

    def _trace(self, ev) -> None:
        try:
            if os.path.exists(self.trace_path) and os.path.getsize(self.trace_path) > self.trace_bytes:
                os.replace(self.trace_path, self.trace_path + ".1")
            with open(self.trace_path, "a") as f:
                f.write(json.dumps(ev) + "\n")
        except OSError:
            self.trace_path = None

    def snapshot(self, limit: int = 256) -> Dict[str, Any]:
        with self.lock:
            return {"seq": self.seq, "dropped": self.dropped, "events": list(self.general)[-limit:],
                    "incidents": list(self.incidents)}
