"""Cache and checkpoint policy as pure functions over (prefix length, bytes) descriptions.

Every decision here is taken identically on every rank from agreed inputs; nothing reads the
clock, the device or the environment.  Behavioural source: the reference's policy functions
(src/resident_worker.rs:710-990): LRU replacement that protects up to two longer parents,
the checkpoint *ladder* (evict the rung whose loss costs an edit the least re-prefill), a
reserve of slots for short checkpoints, optional images that never displace conversations,
and the shared-prefix / system-prefix checkpoint placement rules.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

Entry = Tuple[int, int]          # (prefix length in tokens, image bytes)
SHORT_TOKENS = 8192              # checkpoints below this count as "short"
STALE_AFTER = 32                 # saves after which an entry no longer protects itself by cost


BLOCK = 4096


def as_array(tokens) -> "np.ndarray":
    import numpy as np
    return tokens if isinstance(tokens, np.ndarray) else np.asarray(tokens, dtype=np.int64)


def chain_hashes(tokens, block: int = BLOCK) -> List[bytes]:
    """Chained digests of the whole ``block``-token blocks of a token sequence: entry k identifies
    tokens [0, (k + 1) * block).  Two sequences share their first k blocks exactly when their first k
    entries agree, so million-token prefixes are matched by comparing a few hundred digests."""
    import hashlib
    t = as_array(tokens)
    h = hashlib.sha256()
    out = []
    for i in range(0, len(t) - len(t) % block, block):
        h.update(t[i:i + block].tobytes())
        out.append(h.digest())
    return out


def common_prefix(a, b, chain_a: Optional[List[bytes]] = None, chain_b: Optional[List[bytes]] = None) -> int:
    """Length of the common prefix of two token sequences (lists, tuples or integer arrays).  With
    the sequences' chained block digests the shared whole blocks are found without touching the
    tokens; the remainder is one vectorised comparison."""
    import numpy as np
    ta, tb = as_array(a), as_array(b)
    n = min(len(ta), len(tb))
    i = 0
    if chain_a is not None and chain_b is not None:
        k = 0
        m = min(len(chain_a), len(chain_b), n // BLOCK)
        while k < m and chain_a[k] == chain_b[k]:
            k += 1
        i = k * BLOCK
    # sequences that differ usually differ early: look at a short window before the whole remainder
    step = 1024
    while i < n:
        j = min(n, i + step)
        diff = np.flatnonzero(ta[i:j] != tb[i:j])
        if diff.size:
            return i + int(diff[0])
        i, step = j, step * 16
    return n


def cache_capacity(session_budget: int, shared_budget: int, suspended_bytes: int, suspended_count: int,
                   slot_limit: int, extra_bytes: int = 0, extra_count: int = 0) -> Tuple[int, int]:
    """(bytes, slots) left for cache entries once parked request images and a restored parent
    held outside the cache are charged."""
    room = min(session_budget, max(0, shared_budget - suspended_bytes))
    return max(0, room - extra_bytes), max(0, slot_limit - suspended_count - extra_count)


def ladder_victim(entries: Sequence[Entry], ancestors: Sequence[bool], retained: Sequence[int],
                  protected: Sequence[int]) -> Optional[int]:
    """Among the retained ancestors of the incoming prefix, the rung whose removal merges the two
    gaps with the smallest product (at - prev) * (next - at); the two latest rungs are kept."""
    rungs = sorted((i for i in retained if ancestors[i]), key=lambda i: (entries[i][0], i))
    if len(rungs) < 3:
        return None
    best, best_key = None, None
    for k in range(len(rungs) - 2):
        i = rungs[k]
        if i in protected:
            continue
        at = entries[i][0]
        prev = entries[rungs[k - 1]][0] if k else 0
        nxt = entries[rungs[k + 1]][0]
        key = ((at - prev) * (nxt - at), i)
        if best_key is None or key < best_key:
            best, best_key = i, key
    return best


def cache_evictions(entries: Sequence[Entry], incoming: Entry, budget: int, long_first: bool, slots: int,
                    ancestors: Optional[Sequence[bool]] = None, short_reserve: int = 0,
                    ladder_cap: int = 0) -> Optional[List[int]]:
    """Indices to evict (in order) so that ``incoming`` fits ``budget`` bytes and ``slots`` entries,
    or None when it cannot fit.  ``entries`` are ordered oldest first by insertion/restoration
    (a cache hit refreshes age)."""
    if incoming[1] > budget or slots == 0:
        return None
    if ancestors is not None and len(ancestors) != len(entries):
        return None
    n = len(entries)
    protected: List[int] = []
    if long_first:
        protected = sorted((i for i in range(n) if entries[i][0] > incoming[0]),
                           key=lambda i: (-entries[i][0], -i))[: min(2, max(0, slots - 2))]
    retained = list(range(n))
    removed: List[int] = []

    def first_unprotected(cands, skip=()):
        for i in cands:
            if i not in protected and i not in skip:
                return i
        return None

    while len(retained) >= slots or sum(entries[i][1] for i in retained) + incoming[1] > budget:
        if short_reserve == 0:
            oldest = first_unprotected(retained)
        else:
            shorts = [i for i in retained if entries[i][0] < SHORT_TOKENS]
            if incoming[0] >= SHORT_TOKENS:
                kept = shorts[max(0, len(shorts) - short_reserve):]
                oldest = first_unprotected(retained, kept)
            elif len(shorts) >= short_reserve:
                oldest = first_unprotected(shorts)
            else:
                oldest = first_unprotected(retained)
        if oldest is None:
            return None
        victim = oldest
        if ancestors is not None:
            own = sum(1 for i in retained if ancestors[i])
            if (ladder_cap > 0 and own >= ladder_cap) or ancestors[oldest]:
                lv = ladder_victim(entries, ancestors, retained, protected)
                if lv is not None:
                    victim = lv
        retained.remove(victim)
        removed.append(victim)
    return removed


def prompt_cache_evictions(entries, incoming, budget, long_first, slots, has_media: bool) -> Optional[List[int]]:
    """Text-only exact-logit snapshots are spare-capacity optimisations: they are stored only when
    nothing has to go.  Image prompts paid for visual prefill and use the ordinary policy."""
    ev = cache_evictions(entries, incoming, budget, long_first, slots)
    if ev is None:
        return None
    return ev if (has_media or not ev) else None


def cache_evictions_with_optional(entries, optional: Sequence[bool], incoming, budget, long_first, slots,
                                  ancestors=None) -> Optional[List[int]]:
    """Optional images (text-only final-logit snapshots) yield first, shortest first; the ordinary
    policy then runs on what is left."""
    if incoming[1] > budget or slots == 0 or len(optional) != len(entries):
        return None
    retained = list(range(len(entries)))
    removed: List[int] = []
    while len(retained) >= slots or sum(entries[i][1] for i in retained) + incoming[1] > budget:
        opts = [i for i in retained if optional[i]]
        if not opts:
            break
        v = min(opts, key=lambda i: (entries[i][0], i))
        retained.remove(v)
        removed.append(v)
    rest = [entries[i] for i in retained]
    rest_anc = [ancestors[i] for i in retained] if ancestors is not None else None
    more = cache_evictions(rest, incoming, budget, long_first, slots, rest_anc)
    if more is None:
        return None
    return removed + [retained[i] for i in more]


def completed_cache_evictions(entries, optional, ancestors, incoming, budget, long_first, slots
                              ) -> Optional[List[int]]:
    """A completed turn can be rebuilt from its saved parent, so saving it never evicts that
    parent: parents are reserved (bytes and slots) and the rest follows the optional policy."""
    if not (len(entries) == len(optional) == len(ancestors)):
        return None
    reserved = sum(entries[i][1] for i in range(len(entries)) if ancestors[i])
    count = sum(1 for a in ancestors if a)
    if reserved > budget or count > slots:
        return None
    retained = [i for i in range(len(entries)) if not ancestors[i]]
    ev = cache_evictions_with_optional([entries[i] for i in retained], [optional[i] for i in retained], incoming,
                                       budget - reserved, long_first, slots - count)
    return None if ev is None else [retained[i] for i in ev]


def eviction_cost_order(prefixes: Sequence[Sequence[int]]) -> List[int]:
    """Order (first evicted first) for prefixes given oldest first: stale entries, then a rung with
    exactly one direct extension (an older turn under its newer one), then everything else; within
    a class the cheapest loss first (tokens between the entry and the longest remaining entry it
    extends), oldest first among equals; re-chosen after every pick."""
    n = len(prefixes)
    P = [list(p) for p in prefixes]
    ext = [[a != b and len(P[b]) < len(P[a]) and P[a][: len(P[b])] == P[b] for b in range(n)] for a in range(n)]
    rung = []
    for i in range(n):
        direct = [j for j in range(n) if ext[j][i] and not any(ext[j][k] and ext[k][i] for k in range(n))]
        rung.append(len(direct) == 1)
    left = list(range(n))
    order = []
    while left:
        def key(i):
            if n - 1 - i >= STALE_AFTER:
                return (0, 0, i)
            covered = max((len(P[j]) for j in left if ext[i][j]), default=0)
            return (1 if rung[i] else 2, len(P[i]) - covered, i)
        v = min(left, key=key)
        left.remove(v)
        order.append(v)
    return order


# ---------------------------------------------------------------------------------------------
# checkpoint placement
# ---------------------------------------------------------------------------------------------
def shared_prefix_checkpoint(common: int, previous: int, otherwise: int, prompt: int, minimum: int) -> Optional[int]:
    """Save at the end of the part shared with cached conversations (rounded down to 128) when that
    serves later conversations: gain >= 1024 rows, cost <= 4096 rows, gain >= 4 * cost."""
    at = common // 128 * 128
    if at <= previous or at >= otherwise or at < minimum or prompt < at + 128:
        return None
    gain, cost = at - previous, otherwise - at
    return at if (gain >= 1024 and cost <= 4096 and gain >= 4 * cost) else None


def system_prefix_checkpoint(system: int, otherwise: int, prompt: int, minimum: int) -> Optional[int]:
    """Cold prompt, nothing shared yet: save at the end of the system part when the gain is >= 1024
    rows, at least eight times the cost, and the cost is <= 1024 rows."""
    at = system // 128 * 128
    if at >= otherwise or at < minimum or prompt < at + 128:
        return None
    gain, cost = at, otherwise - at
    return at if (gain >= 1024 and cost <= 1024 and gain >= 8 * cost) else None


def near_end_of(prompt: Sequence[int], near: Sequence[int]) -> bool:
    """``near`` is a proper non-empty prefix of ``prompt`` fewer than 128 tokens shorter."""
    return 0 < len(near) < len(prompt) and len(prompt) - len(near) < 128 and list(prompt[: len(near)]) == list(near)


def checkpoint_positions(prompt_len: int, start: int, minimum: int = SHORT_TOKENS, align: int = 8192,
                         near_end: bool = True) -> List[int]:
    """Positions at which a prefill of ``prompt_len`` tokens resuming at ``start`` saves images:
    every aligned position >= minimum, plus a near-end position (128-aligned, fewer than 128 tokens
    before the end) so that a repeated prompt restores with one short suffix."""
    out = [p for p in range((start // align + 1) * align, prompt_len - 127, align) if p >= minimum]
    if near_end:
        ne = (prompt_len - 1) // 128 * 128
        if ne > start and ne >= minimum and prompt_len - ne < 128 and ne not in out and ne < prompt_len:
            out.append(ne)
    return sorted(out)


def reload_pays(image_bytes: int, prefix_tokens: int, read_gbs: float = 2.2, prefill_tok_s: float = 9000.0,
                fixed_s: float = 0.03) -> bool:
    """Reloading a parked image from the disk tier pays when reading it is faster than prefilling
    the tokens it stands for (reference: src/disk_tier.rs:216-221)."""
    return fixed_s + image_bytes / (read_gbs * 1e9) < prefix_tokens / prefill_tok_s
