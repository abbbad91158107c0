"""Start-up self-check: warm every kernel shape and prove that state is reproducible.

A fixed prompt is prefilled and decoded for a few steps in one region, then the same work is run
again in another region.  Committed tokens, final logits and the digests of both state images must
be identical: with fixed-order reductions any race or uninitialised read shows up here as a
mismatch before the server reports ready.  (The reference replays a fixture prompt at start-up and
asserts that the digest of the reset state equals the empty digest: src/resident_worker.rs:4602-4611;
state here is addressed by position, so "reset" is a no-op and reproducibility is the property to check.)
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..spec.decoder import DecodeSlot

FIXTURE_PROMPT = [3 + (i * 7919 + (i // 5) * 104729) % 997 for i in range(96)]


class SelfCheckError(RuntimeError):
    pass


def _run(backend, region: int, prompt: List[int], steps: int, seed: int):
    backend.reset(region)
    logits = backend.prefill(region, prompt, 0, None)
    first = backend.sample(logits, 0.0, 1.0, seed, len(prompt))
    slot = DecodeSlot(region=region, length=len(prompt), anchor=first, seed=seed, temperature=0.0, top_p=1.0,
                      recent=list(prompt[-8:]))
    out = [first]
    for _ in range(steps):
        out += backend.decode_step([slot])[0]
    committed = (prompt + out)[: slot.length]
    img = backend.snapshot(region, committed, "complete")
    return out, logits.detach().float().cpu(), img.digest(), img.nbytes


def self_check(backend, steps: int = 4, vocab: int = 0) -> Dict[str, object]:
    """Raises SelfCheckError on any difference between two runs of the fixture; returns a short report."""
    if backend.regions < 2:
        raise SelfCheckError("the self-check needs two regions")
    v = vocab or backend.cfg.vocab
    prompt = [t % v for t in FIXTURE_PROMPT]
    a = _run(backend, 0, prompt, steps, seed=1)
    b = _run(backend, backend.regions - 1, prompt, steps, seed=1)
    if a[0] != b[0]:
        raise SelfCheckError(f"committed tokens differ between two runs: {a[0]} vs {b[0]}")
    if not torch.equal(a[1], b[1]):
        raise SelfCheckError("prompt logits differ bitwise between two runs")
    if a[2] != b[2]:
        raise SelfCheckError("state image digests differ between two runs")
    return {"tokens": len(a[0]), "state_bytes": a[3], "digest": a[2][:16]}
