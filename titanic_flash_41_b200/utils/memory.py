"""Memory admission: every optional allocation (session images, host staging, disk-tier reads,
image inputs) is admitted against what is actually available minus a floor, and every rank must
take the same branch, so refusals are decided by an all-rank vote (``ControlChannel.all_admit``).

Host side reads MemAvailable and the cgroup limit; device side reads ``cudaMemGetInfo``.  On
B200 the two pools are separate (the reference admits everything against one unified pool):
images live in HBM while the device floor allows, then in pinned host memory, then on disk
(reference: src/memory.rs:112 floor_bytes, :167 InputCapacityError, :173 reserve_host_workspace,
:209 Available; src/cuda.rs:330-344 allocation_failure records).
"""
from __future__ import annotations

import json
import os
import sys
import threading
from dataclasses import dataclass
from typing import Callable, Optional

DEFAULT_HOST_FLOOR = 8 << 30
DEFAULT_DEVICE_FLOOR = 4 << 30


class CapacityError(MemoryError):
    """An input or cache allocation does not fit above the floor (HTTP 503 / cache refusal, not a crash)."""


def _read_int(path: str) -> Optional[int]:
    try:
        with open(path) as f:
            v = f.read().strip()
        return None if v in ("max", "") else int(v)
    except (OSError, ValueError):
        return None


def host_available(meminfo: str = "/proc/meminfo", cgroup: str = "/sys/fs/cgroup") -> int:
    """Bytes the process may still take: min(MemAvailable, cgroup limit - cgroup usage)."""
    avail = None
    try:
        with open(meminfo) as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    avail = int(line.split()[1]) * 1024
                    break
    except OSError:
        pass
    limit = _read_int(os.path.join(cgroup, "memory.max"))
    used = _read_int(os.path.join(cgroup, "memory.current"))
    if limit is not None and used is not None:
        room = max(0, limit - used)
        avail = room if avail is None else min(avail, room)
    return avail if avail is not None else 1 << 62


def device_available(device=None) -> int:
    import torch
    if not torch.cuda.is_available():
        return 0
    free, _ = torch.cuda.mem_get_info(device)
    return int(free)


@dataclass
class Reservation:
    owner: "Admission"
    nbytes: int
    released: bool = False

    def release(self) -> None:
        if not self.released:
            self.released = True
            with self.owner._lock:
                self.owner.reserved -= self.nbytes

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()
        return False


class Admission:
    """Admission against ``available() - floor - what is already reserved``."""

    def __init__(self, available: Callable[[], int], floor: int, name: str = "host",
                 log: Optional[Callable[[dict], None]] = None):
        self.available, self.floor, self.name = available, floor, name
        self.reserved = 0
        self._lock = threading.Lock()
        self.log = log or (lambda rec: sys.stderr.write(json.dumps(rec) + "\n"))

    def headroom(self) -> int:
        return self.available() - self.floor - self.reserved

    def fits(self, nbytes: int) -> bool:
        return nbytes <= self.headroom()

    def reserve(self, nbytes: int, what: str = "") -> Reservation:
        with self._lock:
            room = self.available() - self.floor - self.reserved
            if nbytes > room:
                self.log({"event": "allocation_refused", "pool": self.name, "what": what, "bytes": nbytes,
                          "headroom": room, "floor": self.floor})
                raise CapacityError(f"{what or 'allocation'} of {nbytes} bytes does not fit above the {self.name} floor")
            self.reserved += nbytes
        return Reservation(self, nbytes)


def host_admission(floor: int = DEFAULT_HOST_FLOOR, **kw) -> Admission:
    return Admission(host_available, floor, "host", **kw)


def device_admission(device=None, floor: int = DEFAULT_DEVICE_FLOOR, **kw) -> Admission:
    return Admission(lambda: device_available(device), floor, "device", **kw)


# ---------------------------------------------------------------------------------- stall counters
def pressure_snapshot(root: str = "/proc/pressure") -> dict:
    """Cumulative stall microseconds of the host (PSI 'some' totals) plus major-fault counts; the
    difference of two snapshots around a prefill says whether the host, not the GPU, held it up
    (reference: src/prefill_stall.rs)."""
    out = {}
    for res in ("memory", "io", "cpu"):
        try:
            with open(os.path.join(root, res)) as f:
                for line in f:
                    if line.startswith("some"):
                        out[res + "_us"] = int(line.split("total=")[1])
        except (OSError, IndexError, ValueError):
            out[res + "_us"] = 0
    try:
        with open("/proc/vmstat") as f:
            for line in f:
                k, _, v = line.partition(" ")
                if k in ("pgmajfault", "pswpin", "pswpout"):
                    out[k] = int(v)
    except OSError:
        pass
    return out


def pressure_delta(before: dict, after: dict) -> dict:
    return {k: after.get(k, 0) - before.get(k, 0) for k in after}
