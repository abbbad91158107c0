"""Pause and resume of an unfinished request.

A ``RequestCheckpoint`` is the complete state needed to continue a conversation later in any
region: the state image of its committed prefix, what it has emitted so far, its sampler
settings and RNG position, what is left of an interrupted prefill, and the media identity.
The scheduler parks requests this way when more conversations are admitted than regions exist
(turn taking) and when a long prefill yields (reference: src/request_checkpoint.rs;
src/parked_request.rs; src/batched_serving.rs:243 detach_active, :604 attach_peer).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from . import state_image as SI


@dataclass
class RequestCheckpoint:
    id: str
    image: SI.Image                       # state of the committed prefix
    prompt: List[int]
    committed: List[int]                  # prompt + accepted tokens the image covers
    anchor: Optional[int]                 # emitted but not yet committed token
    emitted: List[int]                    # everything sent to the client so far
    limit: int
    temperature: float
    top_p: float
    seed: int
    pending_prompt: List[int] = field(default_factory=list)     # rest of an interrupted prefill
    media: str = ""

    @property
    def charge(self) -> int:
        return self.image.nbytes

    def reach(self, region_reach) -> int:
        """Positions this conversation can still touch (for admission into a region of fixed size)."""
        return region_reach(len(self.committed) + len(self.pending_prompt), self.limit - len(self.emitted))

    def needs_prefix(self, prefix, media: str = "") -> bool:
        return media == self.media and list(prefix[:len(self.committed)]) == self.committed


def pause(worker, region: int) -> RequestCheckpoint:
    """Detach the active request of ``region`` from a worker between steps."""
    a = worker.active.pop(region)
    committed = (list(a.prompt) + list(a.job.generated))[: a.slot.length]
    img = worker.b.snapshot(region, committed, "request", a.job.media)
    return RequestCheckpoint(a.job.id, img, list(a.prompt), committed, a.slot.anchor, list(a.job.generated), a.limit,
                             a.slot.temperature, a.slot.top_p, a.slot.seed, media=a.job.media)


def resume(worker, ck: RequestCheckpoint, region: int, job) -> None:
    """Attach a paused request to ``region`` of a worker.  Sampling is addressed by position, so
    the continuation draws exactly what the uninterrupted request would have drawn."""
    import time

    from ..spec.decoder import DecodeSlot
    from .worker import Active
    worker.b.restore(region, ck.image)
    slot = DecodeSlot(region=region, length=len(ck.committed), anchor=ck.anchor, seed=ck.seed,
                      temperature=ck.temperature, top_p=ck.top_p, recent=list(ck.committed[-8:]))
    if not job.generated:                 # a placeholder job (ranks other than 0) takes over the emitted tokens
        job.generated = list(ck.emitted)
    job.region = region
    worker.active[region] = Active(job, slot, list(ck.prompt), ck.limit, time.monotonic(), time.monotonic())
    worker.jobs[job.id] = job
