"""Bounded, exact memoisation of tokenised plain-text regions, with optional prefix reuse.

A chat prompt is a sequence of template markers and plain regions (message bodies).  Long bodies
repeat from turn to turn, so their ids are cached by the full text of the region.  With prefix
reuse, a long region that differs from a cached one only after a long common prefix (a new
question under the same document) keeps the cached ids up to a *safe cut* before the first
differing character and tokenises only the rest.  A cut is safe where a pre-token of a byte-level
BPE tokenizer starts in any text: after a line break followed by a visible ASCII character, and
where an ASCII digit run starts or ends.  Two guards make the result exactly the whole
tokenisation or fall back to it: the cut must land on a token boundary of the cached ids, and the
tail is tokenised from an EARLIER cut whose ids must repeat the cached ids up to the splice
(reference: src/prompt_regions.rs:1-60 design and constants; cut_at :49).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, List, Optional, Sequence, Tuple

REUSE_MIN_CHARS = 16 * 1024
REUSE_MARGIN = 64
REUSE_OVERLAP = 256
REUSE_SCAN = 1 << 20
REUSE_CANDIDATES = 4


def cut_at(text: str, p: int) -> bool:
    l, r = text[p - 1], text[p]
    if ord(l) >= 0x80 or ord(r) >= 0x80:
        return False
    return ((l in "\n\r") and 0x21 <= ord(r) <= 0x7E) or ((not l.isdigit()) and r.isdigit()) or (l.isdigit() and not r.isdigit())


def _common_prefix(a: str, b: str) -> int:
    n = min(len(a), len(b))
    lo, step = 0, 4096
    while lo + step <= n and a[lo:lo + step] == b[lo:lo + step]:
        lo += step
    while lo < n and a[lo] == b[lo]:
        lo += 1
    return lo


class RegionCache:
    def __init__(self, encode: Callable[[str], List[int]], token_text: Optional[Callable[[int], str]] = None,
                 capacity_chars: int = 64 << 20, prefix_reuse: bool = True, min_chars: int = REUSE_MIN_CHARS):
        """``token_text(id)`` gives the text a token spells; needed for prefix reuse (None disables it)."""
        self.encode, self.token_text = encode, token_text
        self.capacity, self.used = capacity_chars, 0
        self.prefix_reuse = prefix_reuse and token_text is not None
        self.min_chars = min_chars
        self.items: "OrderedDict[str, List[int]]" = OrderedDict()
        self.stats = {"hits": 0, "misses": 0, "prefix_reuse": 0, "prefix_reuse_rejects": 0}

    def _put(self, text: str, ids: List[int]) -> None:
        if len(text) > self.capacity:
            return
        while self.used + len(text) > self.capacity and self.items:
            k, _ = self.items.popitem(last=False)
            self.used -= len(k)
        self.items[text] = ids
        self.used += len(text)

    def _try_prefix(self, text: str) -> Optional[List[int]]:
        for cand in list(reversed(self.items))[:REUSE_CANDIDATES]:
            same = _common_prefix(cand, text)
            if same < self.min_chars:
                continue
            ids = self.items[cand]
            # a safe cut at least REUSE_MARGIN before the first difference, and an earlier one for the overlap
            hi = same - REUSE_MARGIN
            lo = max(1, hi - REUSE_SCAN)
            cut = next((p for p in range(hi, lo, -1) if cut_at(text, p)), None)
            if cut is None:
                continue
            early = next((p for p in range(cut - REUSE_OVERLAP, lo, -1) if cut_at(text, p)), None)
            if early is None:
                continue
            # character position of every cached token boundary up to the cut
            pos, at_early, at_cut = 0, None, None
            for i, t in enumerate(ids):
                if pos == early:
                    at_early = i
                if pos == cut:
                    at_cut = i
                    break
                if pos > cut:
                    break
                pos += len(self.token_text(t))
            if at_early is None or at_cut is None:
                self.stats["prefix_reuse_rejects"] += 1
                continue
            tail = self.encode(text[early:])
            overlap = ids[at_early:at_cut]
            if tail[:len(overlap)] != overlap:
                self.stats["prefix_reuse_rejects"] += 1
                continue
            self.stats["prefix_reuse"] += 1
            return ids[:at_early] + tail
        return None

    def tokens(self, text: str) -> List[int]:
        hit = self.items.get(text)
        if hit is not None:
            self.items.move_to_end(text)
            self.stats["hits"] += 1
            return list(hit)
        self.stats["misses"] += 1
        ids = None
        if self.prefix_reuse and len(text) >= self.min_chars:
            ids = self._try_prefix(text)
        if ids is None:
            ids = self.encode(text)
        self._put(text, ids)
        return list(ids)
