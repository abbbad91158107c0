"""Exact-text copy proposals: when the committed text ends with a phrase that occurred before,
propose the tokens that followed it last time.  A proposal is a point mass (q = 1 on the proposed
token), so verification accepts it with probability p_target(token) and the output law is
unchanged.  Pure host bookkeeping on public token ids: every rank computes the same proposal.

Suffixes of several lengths are fingerprinted into small direct-mapped tables (longest match
wins); a hit is confirmed by comparing the actual tokens, so a hash collision can only lose an
opportunity, never invent a match (reference: src/history_lookup.rs:1-60 design, LENGTHS
[8,12,16,32,64], SLOTS 65,536; examples/history_lookup_*.rs screens).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

LENGTHS = (8, 12, 16, 32, 64)
SLOTS = 1 << 16
EMPTY = -1
MASK = (1 << 64) - 1


PRIME = 0x100000001B3            # odd multiplier of the polynomial hash (mod 2^64)


def _mix(v: int) -> int:
    return v ^ (v >> 32)


def fingerprint(ids: Sequence[int]) -> int:
    """Polynomial hash of a window, sum (t_k + 1) * PRIME^(L-1-k) mod 2^64, folded once.  Unlike a
    chained hash it can be ROLLED: appending a token and dropping the oldest is O(1), which is what a
    decode step does for every suffix length."""
    v = 0
    for t in ids:
        v = (v * PRIME + (t & 0xFFFFFFFF) + 1) & MASK
    return _mix(v)


@dataclass
class Proposal:
    tokens: List[int]
    matched: int            # length of the confirmed suffix match
    source_end: int         # index in the history right after the earlier occurrence


class _Text:
    """Append-only token text: an integer array for what arrived in bulk (a prompt of a million
    tokens stays one array: no Python integer per token) followed by a list of the tokens committed
    one by one.  Indexing and slicing return Python ints / lists."""

    def __init__(self):
        import numpy as np
        self.base = np.zeros(0, dtype=np.int64)
        self.tail: List[int] = []

    def __len__(self) -> int:
        return int(self.base.shape[0]) + len(self.tail)

    def __getitem__(self, i):
        nb = int(self.base.shape[0])
        if isinstance(i, slice):
            lo, hi, st = i.indices(len(self))
            assert st == 1
            out = self.base[lo:min(hi, nb)].tolist() if lo < nb else []
            if hi > nb:
                out += self.tail[max(0, lo - nb):hi - nb]
            return out
        if i < 0:
            i += len(self)
        return int(self.base[i]) if i < nb else self.tail[i - nb]

    def append(self, t: int) -> None:
        self.tail.append(t)

    def extend_array(self, arr) -> None:
        import numpy as np
        if self.tail:
            self.base = np.concatenate([self.base, np.asarray(self.tail, dtype=np.int64)])
            self.tail = []
        self.base = np.concatenate([self.base, arr]) if self.base.shape[0] else arr.copy()

    def array(self, lo: int):
        """Tokens [lo, end) as an int64 array."""
        import numpy as np
        nb = int(self.base.shape[0])
        head = self.base[min(lo, nb):]
        return np.concatenate([head, np.asarray(self.tail[max(0, lo - nb):], dtype=np.int64)]) if self.tail else head

    def truncate(self, length: int) -> None:
        nb = int(self.base.shape[0])
        if length >= nb:
            del self.tail[length - nb:]
        else:
            self.base, self.tail = self.base[:length].copy(), []


class HistoryLookup:
    BULK_SPAN = 4           # a bulk commit indexes at most this many windows per table slot

    def __init__(self, prefix: Sequence[int] = (), slots: int = SLOTS, lengths: Sequence[int] = LENGTHS,
                 minimum_match: Optional[int] = None, depth: int = 5):
        import numpy as np
        self.tokens = _Text()
        self.slots, self.lengths, self.depth = slots, tuple(lengths), depth
        self.minimum = minimum_match or self.lengths[0]
        self.tables = [np.full(slots, EMPTY, dtype=np.int64) for _ in self.lengths]
        # raw (unfolded) hash of the last min(L, length) tokens per suffix length, rolled by every commit
        self._raw = [0] * len(self.lengths)
        self._top = [pow(PRIME, L - 1, 1 << 64) for L in self.lengths]       # weight of the oldest token of a full window
        if len(prefix):
            self.commit(0, prefix)

    def commit(self, at: int, tokens: Sequence[int]) -> None:
        """Append ``tokens`` at position ``at`` (must equal the current length: history is append-only)."""
        if at != len(self.tokens):
            raise ValueError("history commits must be contiguous")
        if len(tokens) > 256:
            self._commit_bulk(tokens)
            return
        for t in tokens:
            t = int(t)
            n = len(self.tokens)                            # position of this token
            # the suffix that ENDS BEFORE this token predicts it: index it, then roll the window over the token
            for li, L in enumerate(self.lengths):
                raw = self._raw[li]
                if n >= L:
                    self.tables[li][_mix(raw) % self.slots] = n          # position of the token that followed
                    raw = (raw - ((self.tokens[n - L] & 0xFFFFFFFF) + 1) * self._top[li]) & MASK
                self._raw[li] = (raw * PRIME + (t & 0xFFFFFFFF) + 1) & MASK
            self.tokens.append(t)

    def _commit_bulk(self, tokens: Sequence[int]) -> None:
        """Index a long run (a prompt) with vectorised fingerprints: the same table contents as
        token-by-token commits (a slot keeps the LAST position that hashed to it)."""
        import numpy as np
        base = len(self.tokens)
        new = np.asarray(tokens, dtype=np.int64)
        self.tokens.extend_array(new)
        n = len(self.tokens)
        # A slot keeps the last position that hashed to it, so of a very long run only the most recent
        # windows survive: with 4 x slots windows indexed, an older one would have been overwritten
        # with probability 1 - e^-4.  Bounding the run keeps a million-token prompt at the cost of a
        # quarter-million-token one.
        first = max(0, n - self.BULK_SPAN * self.slots - self.lengths[-1])
        text = self.tokens.array(first).astype(np.uint64) & np.uint64(0xFFFFFFFF)
        for li, L in enumerate(self.lengths):
            # windows [i, i + L) predict token i + L; only windows whose predicted token is new
            lo = max(0, base - L, first)
            hi = n - L                      # predicted positions lo + L .. n - 1
            if hi <= lo:
                continue
            v = np.zeros(hi - lo, dtype=np.uint64)
            with np.errstate(over="ignore"):
                for k in range(L):
                    v = v * np.uint64(PRIME) + text[lo - first + k: hi - first + k] + np.uint64(1)
            v = v ^ (v >> np.uint64(32))
            keys = (v % np.uint64(self.slots)).astype(np.int64)
            pos = np.arange(lo + L, hi + L, dtype=np.int64)
            keep = pos >= max(base, L)
            np.maximum.at(self.tables[li], keys[keep], pos[keep])
        self._reseed()

    def _reseed(self) -> None:
        """Rolling states from the text itself (after a bulk commit or a truncation)."""
        n = len(self.tokens)
        for li, L in enumerate(self.lengths):
            raw = 0
            for t in self.tokens[max(0, n - L):n]:
                raw = (raw * PRIME + (t & 0xFFFFFFFF) + 1) & MASK
            self._raw[li] = raw

    def truncate(self, length: int) -> None:
        """Drop text past ``length`` (a cancelled or rolled-back turn); stale slots are caught by confirmation."""
        self.tokens.truncate(length)
        self._reseed()

    def propose(self, pending: Sequence[int] = ()) -> Optional[Proposal]:
        """``pending``: tokens already emitted but not yet committed (the anchor); the match runs over
        committed text followed by them."""
        pend = [int(t) for t in pending]
        nt = len(self.tokens)
        n = nt + len(pend)
        span = self.lengths[-1]
        at = lambda i: self.tokens[i] if i < nt else pend[i - nt]
        tail = None
        for li in range(len(self.lengths) - 1, -1, -1):
            L = self.lengths[li]
            if n < L or L < self.minimum:
                continue
            # hash of the last L tokens of (committed + pending): the rolling state moved over the pending tokens
            raw = self._raw[li]
            for j, t in enumerate(pend):
                if nt + j >= L:
                    raw = (raw - ((at(nt + j - L) & 0xFFFFFFFF) + 1) * self._top[li]) & MASK
                raw = (raw * PRIME + (t & 0xFFFFFFFF) + 1) & MASK
            pos = int(self.tables[li][_mix(raw) % self.slots])
            if pos == EMPTY or pos >= nt or pos < L:
                continue
            if tail is None:
                tail = self.tokens[max(0, nt - span):] + pend    # the last tokens of the text: no copy of the history
            suffix = tail[len(tail) - L:]
            if self.tokens[pos - L:pos] != suffix:
                continue                                       # collision or stale slot
            out = self.tokens[pos:pos + self.depth]
            if not out:
                continue
            m = L                                              # extend the confirmed match backwards
            while m < min(pos, n, 4096) and self.tokens[pos - m - 1] == at(n - m - 1):
                m += 1
            return Proposal(out, m, pos)
        return None
