"""Property tests (hypothesis) of host-side invariants: prefix matching by chained digests, the
array-backed history text, the causal stopping rule, checkpoint positions, sequence-parallel chunking."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from titanic_flash_41_b200.serve import policy
from titanic_flash_41_b200.spec.history_lookup import HistoryLookup, _Text
from titanic_flash_41_b200.spec.verify import causal_rows

tokens = st.lists(st.integers(0, 50), min_size=0, max_size=120)


@settings(max_examples=150, deadline=None)
@given(tokens, tokens, st.integers(1, 16))
def test_common_prefix_equals_the_naive_scan_with_and_without_digests(a, b, block):
    share = min(len(a), len(b), 17)
    b = a[:share] + b                                    # make long shared prefixes likely
    naive = 0
    while naive < min(len(a), len(b)) and a[naive] == b[naive]:
        naive += 1
    assert policy.common_prefix(a, b) == naive
    ca, cb = policy.chain_hashes(a, block), policy.chain_hashes(b, block)
    assert policy.common_prefix(np.asarray(a, dtype=np.int64), tuple(b), ca, cb) == naive
    # digests of whole blocks agree exactly as far as the sequences do
    same_blocks = sum(1 for x, y in zip(ca, cb) if x == y)
    assert same_blocks == min(naive // block, len(ca), len(cb)) or ca[:same_blocks] == cb[:same_blocks]


@settings(max_examples=100, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["append", "bulk", "truncate"]), tokens), min_size=1, max_size=12))
def test_history_text_mirrors_a_plain_list(ops):
    text, ref = _Text(), []
    for op, toks in ops:
        if op == "append":
            for t in toks:
                text.append(t)
            ref += toks
        elif op == "bulk":
            text.extend_array(np.asarray(toks, dtype=np.int64))
            ref += toks
        else:
            n = len(toks) % (len(ref) + 1)
            text.truncate(n)
            del ref[n:]
        assert len(text) == len(ref)
        if ref:
            assert text[0] == ref[0] and text[-1] == ref[-1] and text[len(ref) // 2] == ref[len(ref) // 2]
        lo, hi = len(ref) // 3, len(ref) - len(ref) // 4
        assert text[lo:hi] == ref[lo:hi] and text[:] == ref and text.array(lo).tolist() == ref[lo:]


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(3, 12), min_size=300, max_size=420), st.integers(0, 400))
def test_bulk_and_single_commits_index_the_same_positions(text, split):
    split = min(split, len(text))
    a = HistoryLookup(text[:split], depth=4)             # a bulk part (when longer than 256) ...
    for i in range(split, len(text)):
        a.commit(i, [text[i]])                           # ... then token by token
    b = HistoryLookup(depth=4)
    for i, t in enumerate(text):
        b.commit(i, [t])
    assert all((x == y).all() for x, y in zip(a.tables, b.tables)) and a._raw == b._raw
    pa, pb = a.propose(), b.propose()
    assert (pa is None) == (pb is None) and (pa is None or (pa.tokens, pa.source_end) == (pb.tokens, pb.source_end))
    if pa is not None:                                   # a proposal is what followed an earlier occurrence of the suffix
        L = 8
        assert text[pa.source_end - L: pa.source_end] == text[len(text) - L:] and pa.tokens == text[pa.source_end: pa.source_end + 4]


conf = st.lists(st.floats(0.0, 1.0, allow_nan=False), min_size=0, max_size=6)


@settings(max_examples=200, deadline=None)
@given(conf, st.lists(st.floats(0.0, 1.0, allow_nan=False), min_size=1, max_size=4), st.data())
def test_causal_rows_never_looks_past_the_stopping_confidence(c, ladder, data):
    n = causal_rows(c, ladder)
    assert (n == 0) == (len(c) == 0) and n <= len(c)
    if n >= 1:
        prod = c[0]
        for j in range(1, n):                            # every admitted proposal cleared its threshold
            prod *= c[j]
            assert prod >= ladder[min(j - 1, len(ladder) - 1)]
        for k in range(n + 1, len(c)):                   # confidences after the one that stopped do not matter
            alt = list(c)
            alt[k] = data.draw(st.floats(0.0, 1.0, allow_nan=False))
            assert causal_rows(alt, ladder) == n


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 300000), st.integers(0, 300000), st.sampled_from([128, 1024, 8192, 65536]))
def test_checkpoint_positions_are_aligned_increasing_and_inside_the_new_part(prompt, start, align):
    start = min(start, prompt - 1)
    pos = policy.checkpoint_positions(prompt, start, align, align)
    assert pos == sorted(set(pos)) and all(start < p < prompt and p >= align for p in pos)
    assert all(p % align == 0 or p % 128 == 0 for p in pos)


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 400000), st.sampled_from([2, 4, 8]), st.sampled_from([1, 2, 4]), st.sampled_from([0, 32768, 65536]))
def test_sequence_parallel_chunks_cover_the_prompt_in_rank_aligned_pieces(n, world, ratio, sp_rows):
    from types import SimpleNamespace as NS

    from titanic_flash_41_b200.parallel.sp import SpPrefill
    max_chunk, window = 16384, 128
    ring = max(max_chunk, sp_rows) + 2 * window
    fake = NS(W=world, eng=NS(cfg=NS(compress_ratio=ratio, max_ratio=ratio, window=window), ecfg=NS(sp_chunk_rows=sp_rows),
                              max_chunk=max_chunk, ring=ring))
    sizes = SpPrefill.chunk_sizes(fake, n, max_chunk)
    assert sum(sizes) == n and all(s > 0 for s in sizes)
    cap = min(max(max_chunk, sp_rows), max_chunk * world, ring - 2 * window)
    assert all(s % (world * ratio) == 0 for s in sizes[:-1]) and all(s <= max(cap, world * ratio) for s in sizes)


# ---- storage formats: decode(encode(x)) stays within the format's own error bound, and encoding what
# was decoded is a fixed point (the formats are what the kernels read and write)
import torch  # noqa: E402

from titanic_flash_41_b200.formats import codecs  # noqa: E402

rows = st.integers(1, 5)
scale = st.floats(1e-3, 1e3)
seed = st.integers(0, 10_000)


def _rand(r, n, sc, sd):
    g = torch.Generator().manual_seed(sd)
    x = torch.randn(r, n, generator=g) * sc
    x[0, : n // 8] = 0                                    # an all-zero group must survive
    return x


@settings(max_examples=60, deadline=None)
@given(rows, scale, seed)
def test_mxfp8_rows_round_trip_within_one_e4m3_step_and_requantise_exactly(r, sc, sd):
    x = _rand(r, 128, sc, sd)
    q, s = codecs.mxfp8_quant(x)
    back = codecs.mxfp8_dequant(q, s)
    amax = x.view(r, 4, 32).abs().amax(-1, keepdim=True).expand(r, 4, 32).reshape(r, 128)
    assert bool(((back - x).abs() <= amax * 2 ** -3 + 1e-30).all())       # 3 mantissa bits, scale <= 2 x amax / 448
    q2, s2 = codecs.mxfp8_quant(back)
    assert torch.equal(codecs.mxfp8_dequant(q2, s2), back)


@settings(max_examples=60, deadline=None)
@given(rows, scale, seed)
def test_mxfp4_weights_round_trip_and_requantise_exactly(r, sc, sd):
    w = _rand(r, 64, sc, sd)
    p, s = codecs.mxfp4_quant(w)
    back = codecs.mxfp4_dequant(p, s)
    amax = w.view(r, 2, 32).abs().amax(-1, keepdim=True).expand(r, 2, 32).reshape(r, 64)
    assert bool(((back - w).abs() <= amax * 0.26 + 1e-30).all())          # e2m1: the largest gap (4 -> 6) is a third of the top code
    p2, s2 = codecs.mxfp4_quant(back)
    assert torch.equal(codecs.mxfp4_dequant(p2, s2), back)
    assert torch.equal(codecs.unpack_nibbles(codecs.pack_nibbles(codecs.unpack_nibbles(p))), codecs.unpack_nibbles(p))


@settings(max_examples=40, deadline=None)
@given(rows, st.floats(1e-2, 1e2), seed)
def test_kv_row_formats_round_trip_and_are_fixed_points(r, sc, sd):
    k = _rand(r, 128, sc, sd)
    for enc, dec, tol in ((codecs.kv_v41_encode, codecs.kv_v41_decode, 2 ** -3),
                          (codecs.kv_v41fp4_encode, codecs.kv_v41fp4_decode, 0.3),
                          (codecs.index_key_encode, codecs.index_key_decode, 0.3)):
        row = enc(k)
        back = dec(row, 128)
        assert row.dtype == torch.uint8 and back.shape == k.shape
        assert bool(((back - k).abs() <= k.abs().amax(-1, keepdim=True) * tol + 1e-30).all())
        assert torch.equal(dec(enc(back), 128), back)


# ---- scheduler: random submissions, cancellations, admissions and releases
from titanic_flash_41_b200.serve.scheduler import Job, QueueFull, Scheduler  # noqa: E402

sched_ops = st.lists(st.tuples(st.sampled_from(["fg", "bg", "cancel", "admit", "release", "lease"]), st.integers(0, 7)),
                     min_size=1, max_size=60)


@settings(max_examples=150, deadline=None)
@given(sched_ops, st.integers(1, 4))
def test_scheduler_never_overfills_regions_and_serves_each_class_in_order(ops, regions):
    s = Scheduler(regions, 5, 3)
    events, jobs, admitted, n = [], [], [], 0
    now = 0.0
    for op, k in ops:
        now += 1.0
        if op in ("fg", "bg"):
            j = Job(f"j{n}", [1], 1, background=(op == "bg"), emit=lambda kind, p, _n=n: events.append((_n, kind)))
            n += 1
            try:
                s.submit(j)
                jobs.append(j)
            except QueueFull as e:
                assert str(e) in ("queue_full", "background_queue_full")
                assert len(s.bg if j.background else s.fg) >= (3 if j.background else 5)
        elif op == "cancel" and jobs:
            jobs[k % len(jobs)].cancelled.set()
        elif op == "admit":
            new = s.admit(now=now + 1e9)                       # far future: no lease holds the background back
            admitted += new
            assert not any(j.cancelled.is_set() for j in new)
            assert len({j.region for j in s.active.values()}) == len(s.active) <= regions
        elif op == "release" and s.active:
            j = list(s.active.values())[k % len(s.active)]
            s.release(j)
            assert j.region not in s.active or s.active[j.region] is not j
        elif op == "lease":
            assert s.priority_lease(float(k)) >= 0.0
        assert sorted(s.free_regions() + list(s.active)) == list(range(regions))
    # every admitted job was submitted once, in submission order within its class, and none was cancelled at admission
    order = {id(j): i for i, j in enumerate(jobs)}
    for cls in (False, True):
        seq = [order[id(j)] for j in admitted if j.background == cls]
        assert seq == sorted(seq) and len(set(seq)) == len(seq)
    # a job cancelled while it waited got a terminal event instead of a region
    dropped = {i for i, kind in events if kind == "error"}
    assert all(jobs_i.cancelled.is_set() for jobs_i in jobs if int(jobs_i.id[1:]) in dropped)
    assert not any(int(j.id[1:]) in dropped for j in admitted)


# ---- session cache: random insertions of images of related and unrelated prefixes
from titanic_flash_41_b200.serve import state_image as SI  # noqa: E402
from titanic_flash_41_b200.serve.session_cache import SessionCache  # noqa: E402

cache_ops = st.lists(st.tuples(st.integers(0, 3), st.integers(1, 40), st.sampled_from(["complete", "checkpoint", "optional"]),
                               st.integers(1, 6)), min_size=1, max_size=40)


@settings(max_examples=120, deadline=None)
@given(cache_ops, st.integers(2, 6), st.integers(8, 40))
def test_session_cache_keeps_its_bounds_and_finds_the_longest_cached_prefix(ops, slots, budget_kb):
    family = [[(7 * f + 3 * i) % 50 for i in range(64)] for f in range(4)]         # four conversations
    cache = SessionCache(slots=slots, budget_bytes=budget_kb * 1024, host_budget_bytes=1 << 30, park_after=2)
    for fam, length, kind, kb in ops:
        toks = family[fam][:length]
        img = SI.capture(np.asarray(toks, dtype=np.int64) if length % 2 else toks, [("x", torch.zeros(kb * 256))], kind)
        stored = cache.insert(img, optional=(kind == "optional"), completed=(kind == "complete"))
        assert len(cache.entries) <= slots
        assert cache.device_bytes() <= budget_kb * 1024 or not stored
        # no two entries hold the same prefix
        keys = [(e.image.length, bytes(np.asarray(e.image.tokens, dtype=np.int64).tobytes()), e.image.media) for e in cache.entries]
        assert len(set(keys)) == len(keys)
        # lookups: the longest entry that is a prefix of the prompt (and of the same conversation family)
        for f in range(4):
            prompt = family[f][:50]
            best = cache.best_match(np.asarray(prompt, dtype=np.int64))
            want = max((e.image.length for e in cache.entries
                        if e.image.length <= 50 and list(np.asarray(e.image.tokens)) == prompt[: e.image.length]), default=None)
            assert (best.image.length if best else None) == want
        assert cache.longest_shared(family[fam][:60]) >= (length if stored else 0) or not stored
