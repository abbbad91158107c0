"""Cache of state images keyed by the exact token prefix (and media identity) they restore.

Entries are ordered by insertion / restoration (a hit refreshes age).  A request restores the
entry with the longest prefix that its prompt starts with; saving an image asks the policy
which entries to evict; idle images move down the tiers (device -> host -> disk) and are
reloaded when a cost model says reading pays.  Reference: session cache of the resident worker
(src/resident_worker.rs:765-990, :1205-1370 disk tier steps) and the history book
(src/resident_history.rs).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from . import policy
from .state_image import DiskTier, Image


@dataclass(eq=False)          # identity: two images of the same prefix are still two images
class Entry:
    image: Image
    uid: int
    optional: bool = False
    hits: int = 0
    idle_requests: int = 0          # requests served since this entry was last used


class SessionCache:
    def __init__(self, slots: int = 16, budget_bytes: int = 8 << 30, long_first: bool = True,
                 short_reserve: int = 0, ladder: bool = True, disk: Optional[DiskTier] = None,
                 host_budget_bytes: int = 32 << 30, park_after: int = 4):
        self.slots, self.budget = slots, budget_bytes
        self.long_first, self.short_reserve, self.ladder = long_first, short_reserve, ladder
        self.disk, self.host_budget, self.park_after = disk, host_budget_bytes, park_after
        self.entries: List[Entry] = []
        self._uid = itertools.count(1)
        self.stats = {"hits": 0, "misses": 0, "evictions": 0, "parked": 0, "reloads": 0, "reused_tokens": 0}

    # ---- lookup -------------------------------------------------------------------------------
    def best_match(self, prompt: Sequence[int], media: str = "") -> Optional[Entry]:
        """Entry with the longest prefix that ``prompt`` starts with (same media identity)."""
        best = None
        p, pc = self._prompt_key(prompt)
        for e in self.entries:
            n = e.image.length
            if e.image.media != media or n > len(p) or (best and n <= best.image.length):
                continue
            t, tc = self._entry_key(e)
            if policy.common_prefix(p, t, pc, tc) == n:
                best = e
        return best

    def longest_shared(self, prompt: Sequence[int]) -> int:
        """Longest prefix of the prompt that any cached conversation also begins with."""
        p, pc = self._prompt_key(prompt)
        return max((policy.common_prefix(p, *self._entry_key(e)[:1], pc, self._entry_key(e)[1]) for e in self.entries),
                   default=0)

    def _prompt_key(self, prompt):
        """(token array, chained block digests) of a prompt, computed once per request."""
        last = getattr(self, "_last_prompt", None)
        if last is not None and last[0] is prompt:
            return last[1], last[2]
        arr = policy.as_array(prompt)
        chain = policy.chain_hashes(arr)
        self._last_prompt = (prompt, arr, chain)
        return arr, chain

    @staticmethod
    def _entry_key(e: "Entry"):
        k = getattr(e, "_key", None)
        if k is None:
            arr = policy.as_array(e.image.tokens)
            k = (arr, policy.chain_hashes(arr))
            e._key = k
        return k

    def touch(self, e: Entry, reused: int) -> None:
        self.entries.remove(e)
        self.entries.append(e)
        e.hits += 1
        e.idle_requests = 0
        self.stats["hits"] += 1
        self.stats["reused_tokens"] += reused

    # ---- insertion ----------------------------------------------------------------------------
    def device_bytes(self) -> int:
        return sum(e.image.nbytes for e in self.entries if e.image.tier == "device")

    def insert(self, image: Image, optional: bool = False, completed: bool = False) -> bool:
        """Store an image; returns False when the policy refuses (it would not fit or, for an
        optional image, something would have to go)."""
        # token arrays and chained block digests are computed once per image: comparing the incoming
        # image with every entry must not convert million-token sequences again and again
        ia = policy.as_array(image.tokens)
        key = (ia, policy.chain_hashes(ia))
        pairs = [(e, policy.common_prefix(ia, self._entry_key(e)[0], key[1], self._entry_key(e)[1])) for e in self.entries]
        same = [e for e, c in pairs if c == image.length == e.image.length and e.image.media == image.media]
        for e in same:
            self._drop(e)
        pairs = [(e, c) for e, c in pairs if not any(e is x for x in same)]      # in the order of self.entries
        desc = [(e.image.length, e.image.nbytes) for e in self.entries]
        incoming = (image.length, image.nbytes)
        anc = [c == e.image.length and e.image.length < image.length for e, c in pairs]
        opt = [e.optional for e in self.entries]
        if optional:
            ev = policy.prompt_cache_evictions(desc, incoming, self.budget, self.long_first, self.slots,
                                               has_media=bool(image.media))
        elif completed:
            ev = policy.completed_cache_evictions(desc, opt, anc, incoming, self.budget, self.long_first, self.slots)
        else:
            ev = policy.cache_evictions_with_optional(desc, opt, incoming, self.budget, self.long_first, self.slots,
                                                      anc if self.ladder else None)
        if ev is None:
            return False
        for e in [self.entries[i] for i in ev]:
            self._drop(e)
            self.stats["evictions"] += 1
        ent = Entry(image, next(self._uid), optional)
        ent._key = key
        self.entries.append(ent)
        return True

    def _drop(self, e: Entry) -> None:
        if e in self.entries:
            self.entries.remove(e)
        if e.image.tier == "disk" and self.disk is not None:
            self.disk.remove(f"img{e.uid}")

    # ---- tiers --------------------------------------------------------------------------------
    def idle_step(self) -> Optional[str]:
        """One unit of background work after a request: age the entries and park the oldest idle
        device image one tier down.  Returns a description of what was done (for the event log)."""
        for e in self.entries:
            e.idle_requests += 1
        for e in self.entries:
            if e.idle_requests >= self.park_after and e.image.tier == "device":
                e.image.to_host()
                self.stats["parked"] += 1
                return f"host<-img{e.uid}"
        host = [e for e in self.entries if e.image.tier == "host"]
        if self.disk is not None and sum(e.image.nbytes for e in host) > self.host_budget and host:
            e = host[0]
            self.disk.write(f"img{e.uid}", e.image)
            self.stats["parked"] += 1
            return f"disk<-img{e.uid}"
        return None

    def ensure_loaded(self, e: Entry, device, prefill_tok_s: float = 9000.0) -> bool:
        """Bring an entry's image back to the device; False when reloading would not pay."""
        img = e.image
        if img.tier == "disk":
            if not policy.reload_pays(img.nbytes, img.length, prefill_tok_s=prefill_tok_s):
                return False
            self.disk.read(f"img{e.uid}", img)
            self.stats["reloads"] += 1
        if img.tier == "host":
            img.to_device(device)
        return True
