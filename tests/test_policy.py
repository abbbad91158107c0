"""Cache-eviction, ladder and checkpoint-placement policy (pure functions)."""
from titanic_flash_41_b200.serve import policy as P


def test_fits_without_eviction_and_refuses_oversize():
    assert P.cache_evictions([(100, 10), (200, 10)], (300, 10), budget=100, long_first=True, slots=4) == []
    assert P.cache_evictions([(100, 10)], (300, 200), budget=100, long_first=True, slots=4) is None
    assert P.cache_evictions([], (1, 1), 10, True, 0) is None


def test_oldest_first_and_two_longer_parents_protected():
    entries = [(9000, 10), (500, 10), (9500, 10), (400, 10)]
    # slots full: one must go; the longer parents (9000, 9500) are protected, so the oldest short one goes
    assert P.cache_evictions(entries, (600, 10), 1000, True, 4) == [1]
    assert P.cache_evictions(entries, (600, 10), 1000, False, 4) == [0]
    # byte pressure evicts several, oldest unprotected first
    assert P.cache_evictions(entries, (600, 25), 45, True, 8) == [1, 3]


def test_ladder_evicts_cheapest_rung_and_keeps_latest_two():
    entries = [(1000, 1), (1100, 1), (5000, 1), (9000, 1), (9100, 1)]
    anc = [True] * 5
    ev = P.cache_evictions(entries, (9200, 1), 100, False, 5, ancestors=anc)
    # ordinary victim would be index 0 (an ancestor) -> ladder picks the smallest (at-prev)*(next-at)
    # rung 1100: (1100-1000)*(5000-1100) = 390000 ; rung 1000: 1000*100 = 100000 -> index 0
    assert ev == [0]
    entries = [(4000, 1), (4100, 1), (8000, 1), (9000, 1), (9100, 1)]
    ev = P.cache_evictions(entries, (9200, 1), 100, False, 5, ancestors=[True] * 5)
    assert ev == [1]            # (4100-4000)*(8000-4100) is the smallest product
    assert P.ladder_victim([(1, 1), (2, 1)], [True, True], [0, 1], []) is None


def test_short_reserve():
    entries = [(100, 1), (200, 1), (9000, 1), (300, 1)]
    # a long incoming image skips the newest `reserve` short entries
    assert P.cache_evictions(entries, (10000, 1), 100, False, 4, short_reserve=2) == [0]
    assert P.cache_evictions(entries, (10000, 1), 100, False, 4, short_reserve=3) == [2]
    # a short incoming image replaces the oldest short entry once shorts hold the reserve
    assert P.cache_evictions(entries, (50, 1), 100, False, 4, short_reserve=2) == [0]


def test_optional_images_yield_first_and_never_displace():
    entries = [(100, 5), (5000, 5), (200, 5)]
    assert P.cache_evictions_with_optional(entries, [False, True, True], (300, 5), 15, False, 8) == [2]
    assert P.prompt_cache_evictions(entries, (300, 5), 15, False, 8, has_media=False) is None
    assert P.prompt_cache_evictions(entries, (300, 5), 15, False, 8, has_media=True) == [0]
    assert P.prompt_cache_evictions(entries, (300, 5), 100, False, 8, has_media=False) == []


def test_completed_turn_never_evicts_its_parent():
    entries = [(1000, 5), (300, 5), (400, 5)]
    ev = P.completed_cache_evictions(entries, [False] * 3, [True, False, False], (1100, 5), 15, False, 8)
    assert ev == [1]
    assert P.completed_cache_evictions(entries, [False] * 3, [True, False, False], (1100, 5), 4, False, 8) is None


def test_eviction_cost_order_prefers_inner_rungs():
    a = list(range(100))
    prefixes = [a[:50], a[:80], a, [7, 7, 7]]
    order = P.eviction_cost_order(prefixes)
    assert order[0] in (0, 1) and order[-1] in (2, 3)      # older turns under a newer one go first
    assert sorted(order) == [0, 1, 2, 3]


def test_checkpoint_placement_rules():
    assert P.shared_prefix_checkpoint(common=5000, previous=0, otherwise=6000, prompt=9000, minimum=1024) == 4992
    assert P.shared_prefix_checkpoint(common=5000, previous=0, otherwise=12000, prompt=20000, minimum=1024) is None
    assert P.shared_prefix_checkpoint(common=900, previous=0, otherwise=1000, prompt=9000, minimum=128) is None
    assert P.system_prefix_checkpoint(system=8200, otherwise=9000, prompt=20000, minimum=1024) == 8192
    assert P.system_prefix_checkpoint(system=2000, otherwise=9000, prompt=20000, minimum=1024) is None
    assert P.near_end_of(list(range(300)), list(range(250))) and not P.near_end_of(list(range(300)), list(range(100)))
    pos = P.checkpoint_positions(20000, 0)
    assert pos == [8192, 16384, 19968]
    assert P.checkpoint_positions(5000, 0) == []
    assert P.common_prefix(list(range(10000)), list(range(9000)) + [1]) == 9000
    assert P.cache_capacity(6, 7, 2, 1, 16, 1, 1) == (4, 14)
    assert P.reload_pays(100 << 20, 100000) and not P.reload_pays(100 << 20, 100)


def test_draw_trace_and_logit_export(tmp_path):
    import numpy as np
    import torch
    from titanic_flash_41_b200.utils.trace import DrawTrace, LogitExport, RouteCensus
    dt = DrawTrace(capacity=16)
    for i in range(40):
        dt.add(position=i, accepted=i % 4, token=i)
    assert len(dt.records) <= 16 and sum(dt.acceptance_histogram().values()) == len(dt.records)
    p = str(tmp_path / "t.jsonl")
    dt.dump(p)
    assert len(open(p).read().splitlines()) == len(dt.records)
    le = LogitExport(str(tmp_path / "l.npz"), limit=2)
    for pos in (5, 3, 9):
        le.add(pos, torch.arange(4.0) + pos)
    assert le.save() == 2
    z = np.load(str(tmp_path / "l.npz"))
    assert z["positions"].tolist() == [3, 5] and z["logits"].shape == (2, 4)
    rc = RouteCensus(8)
    rc.add(torch.tensor([[0, 1], [1, 7], [1, -1]]))
    s = rc.summary()
    assert s["total"] == 5 and s["top"][0] == 1 and s["unused"] == 5


def test_chained_block_hashes_find_million_token_prefixes_quickly():
    import time

    import numpy as np

    from titanic_flash_41_b200.serve import policy as P
    rng = np.random.default_rng(0)
    a = rng.integers(0, 129280, size=1_000_000, dtype=np.int64)
    b = a.copy()
    b[777_777] += 1
    ca, cb = P.chain_hashes(a), P.chain_hashes(b)
    assert len(ca) == 1_000_000 // P.BLOCK and ca[:189] == cb[:189] and ca[189] != cb[189]
    t0 = time.perf_counter()
    for _ in range(20):
        assert P.common_prefix(a, b, ca, cb) == 777_777
    assert (time.perf_counter() - t0) / 20 < 0.01            # digests first, one vectorised compare of a block's tail
    assert P.common_prefix(a, a[:5000], ca, P.chain_hashes(a[:5000])) == 5000
    assert P.common_prefix(list(a[:10]), tuple(a[:7])) == 7   # plain sequences still work
    assert P.common_prefix([], [1]) == 0


def test_sequence_parallel_chunk_sizes_respect_slice_and_ring_limits():
    """A sequence-parallel chunk spans every rank's slice: its size is a multiple of ranks x compression
    ratio, every slice fits the row buffers of a single-rank chunk and the whole chunk fits the window
    ring."""
    from types import SimpleNamespace as NS

    from titanic_flash_41_b200.parallel.sp import SpPrefill
    def sizes(n, chunk, world, sp_rows, max_chunk=16384, window=128, ratio=4):
        ring = max(max_chunk, sp_rows) + 2 * window
        fake = NS(W=world, eng=NS(cfg=NS(compress_ratio=ratio, max_ratio=ratio, window=window), ecfg=NS(sp_chunk_rows=sp_rows),
                                  max_chunk=max_chunk, ring=ring))
        return SpPrefill.chunk_sizes(fake, n, chunk)
    s = sizes(129553, 16384, 8, 65536)
    assert sum(s) == 129553 and len(s) == 2 and all(x % 32 == 0 for x in s[:-1]) and max(s) // 8 <= 16384
    s = sizes(129553, 16384, 2, 32768)
    assert sum(s) == 129553 and len(s) == 4 and max(s) <= 32768
    s = sizes(129553, 16384, 4, 0)                     # no larger chunks configured: the single-rank chunk
    assert sum(s) == 129553 and max(s) <= 16384
    s = sizes(40000, 16384, 8, 1 << 20, max_chunk=2048)    # slices bound the chunk: 8 x 2,048 rows
    assert sum(s) == 40000 and max(s) <= 8 * 2048
