"""Host-side speculative-decoding helpers: exact-text copy proposals, request pause / resume."""
import pytest
import torch

from titanic_flash_41_b200.config import tiny_config
from titanic_flash_41_b200.models import oracle
from titanic_flash_41_b200.serve import request_checkpoint as RC
from titanic_flash_41_b200.spec.history_lookup import HistoryLookup, fingerprint


def test_history_lookup_proposes_what_followed_last_time():
    base = list(range(100, 140))
    h = HistoryLookup(base + [7, 8, 9] + base[:20])
    p = h.propose()
    assert p is not None and p.tokens == base[20:25] and p.matched >= 16 and p.source_end == 20
    # the pending anchor extends the match
    p2 = h.propose(pending=[base[20]])
    assert p2.tokens == base[21:26]
    # no earlier occurrence -> nothing
    assert HistoryLookup(list(range(50))).propose() is None
    # shorter than the minimum match -> nothing
    assert HistoryLookup([1, 2, 3, 4, 1, 2, 3]).propose() is None
    # a forged table entry (collision) is rejected by the token comparison
    h3 = HistoryLookup(list(range(30)))
    h3.tables[0][fingerprint(list(range(22, 30))) % h3.slots] = 12
    assert h3.propose() is None
    # commits must be contiguous; truncation makes stale slots harmless
    with pytest.raises(ValueError):
        h.commit(3, [1])
    h.truncate(45)
    assert h.propose() is None or h.propose().source_end <= 45
    # same text on two "ranks" gives the same proposal
    a, b = HistoryLookup(base * 3), HistoryLookup(base * 3)
    assert a.propose() == b.propose()


def test_pause_and_resume_is_token_exact():
    from titanic_flash_41_b200.serve.backend import OracleBackend
    from titanic_flash_41_b200.serve.scheduler import Job, Scheduler
    from titanic_flash_41_b200.serve.session_cache import SessionCache
    from titanic_flash_41_b200.serve.worker import Worker
    cfg = tiny_config()
    W = oracle.init_weights(cfg, 0)
    prompt = torch.randint(3, cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()

    def run(interrupt):
        b = OracleBackend(cfg, W, regions=2, max_context=256, chunk=32)
        s = Scheduler(2, 4, 2)
        w = Worker(b, s, SessionCache(slots=4, budget_bytes=1 << 30), eos_id=1, checkpoint_min=1 << 20)
        ev = []
        job = Job("r", list(prompt), 14, emit=lambda k, p: ev.append((k, p)), temperature=0.6, top_p=0.95, seed=5)
        s.submit(job)
        w.run_once(0.0)                                   # begin
        for _ in range(2):
            w.run_once(0.0)                               # two decode steps
        if interrupt:
            region = next(iter(w.active))
            ck = RC.pause(w, region)
            assert ck.charge > 0 and not w.active and ck.needs_prefix(ck.committed + [1, 2])
            b.reset(region)
            RC.resume(w, ck, 1 - region, job)
        for _ in range(100):
            if w.run_once(0.0) == "idle" and not w.active:
                break
        return [t for k, p in ev if k == "tokens" for t in p]
    plain, paused = run(False), run(True)
    assert plain == paused and len(plain) >= 1


def test_step_meta_equals_step_plans():
    """The array-built metadata of a verification round equals the StepPlan-built one."""
    import numpy as np
    from titanic_flash_41_b200.models.engine import StepPlan
    from titanic_flash_41_b200.spec.decoder import step_meta
    regions, lengths, anchors = [2, 0, 3], [130001, 7, 4095], [11, 12, 13]
    for g in (0, 3):
        mv, mds = step_meta(regions, lengths, anchors, g, 4)
        want = StepPlan.build([(r, n, [a] + [0] * g) for r, n, a in zip(regions, lengths, anchors)]).meta_host(4)
        assert mv.dtype == np.int32 and np.array_equal(mv, want)
        assert len(mds) == g
        for j in range(g):
            wd = StepPlan.build([(r, n + j, [a if j == 0 else 0]) for r, n, a in zip(regions, lengths, anchors)]).meta_host(4)
            assert np.array_equal(mds[j], wd)


def test_recent_rows_and_prefill_seams_for_engram_models():
    """Tokens before each block, newest first and padded; a prefill chunk takes them from the
    prompt's own earlier rows and, at the seam, from the tokens before the prefilled part."""
    import numpy as np
    from titanic_flash_41_b200.config import EngramConfig, tiny_config
    from titanic_flash_41_b200.models import engram as EG
    from titanic_flash_41_b200.models.engine import StepPlan
    from titanic_flash_41_b200.serve.prefill import _recent
    cfg = tiny_config(engram=EngramConfig(layers=(0,), rows_per_table=1500))
    md = EG.metadata_for(cfg)
    n = md.ngram - 1
    rows = StepPlan.recent_rows(cfg, [(2, [7, 8, 9, 10, 11]), (1, [5])])
    assert rows.shape == (3, n) and rows.dtype == np.int32
    assert rows[0].tolist() == [11, 10, 9][:n] and rows[1].tolist() == rows[0].tolist()
    assert rows[2].tolist() == ([5] + [md.pad_token] * n)[:n]
    toks = np.arange(100, 120, dtype=np.int32)
    plan = _recent(StepPlan.build([(0, 50, toks[:8].tolist())]), cfg, [1, 2, 3, 4], toks, 0)
    assert plan.engram_recent[0].tolist() == [4, 3, 2][:n]                       # seam: tokens before the part
    plan = _recent(StepPlan.build([(0, 58, toks[8:16].tolist())]), cfg, [1, 2, 3, 4], toks, 8)
    assert plan.engram_recent[0].tolist() == [107, 106, 105][:n]                 # inside the part
    plan = _recent(StepPlan.build([(0, 51, toks[1:9].tolist())]), cfg, [1, 2, 3, 4], toks, 1)
    assert plan.engram_recent[0].tolist() == [100, 4, 3][:n]                     # straddling the seam
    # the host hashes of a block agree with hashing the same rows through recent_rows' convention
    ids = EG.hash_positions(md, [4, 3, 2][::-1], toks[:4].tolist(), 50)
    assert ids.shape == (4, md.tables, md.ids_per_table)
    # models without Engram layers: the plan is left alone
    plain = tiny_config()
    assert _recent(StepPlan.build([(0, 0, [1, 2])]), plain, [], toks, 0).engram_recent is None


def test_causal_ladder_uses_only_the_confidences_before_each_admitted_proposal():
    """Proposal 1 is always verified; proposal j only while the running products c1..ci (i <= j) clear
    their thresholds; changing a confidence after the one that stopped changes nothing; NaN stops."""
    from titanic_flash_41_b200.spec.verify import causal_rows
    ladder = (0.15, 0.25, 0.20, 0.15)
    assert causal_rows([], ladder) == 0
    assert causal_rows([0.01, 0.99, 0.99], ladder) == 1            # c1 c2 = 0.0099 < 0.15
    assert causal_rows([0.9, 0.9, 0.9, 0.9, 0.9], ladder) == 5     # 0.81, 0.729, 0.656, 0.59
    assert causal_rows([0.9, 0.5, 0.5, 0.99, 0.99], ladder) == 2   # 0.45 >= 0.15; 0.225 < 0.25
    assert causal_rows([0.9, 0.5, 0.6, 0.6, 0.99], ladder) == 3    # 0.45, 0.27 >= 0.25, 0.162 < 0.20
    assert causal_rows([0.9, float("nan"), 0.9], ladder) == 1
    base = [0.9, 0.5, 0.5, 0.3, 0.3]
    n = causal_rows(base, ladder)
    for later in range(n + 1, len(base)):
        for v in (0.0, 1.0):
            alt = list(base)
            alt[later] = v
            assert causal_rows(alt, ladder) == n
    # a short ladder repeats its last threshold
    assert causal_rows([0.9, 0.9, 0.9, 0.9], (0.5,)) == 4 and causal_rows([0.9, 0.9, 0.6, 0.9], (0.5,)) == 2


def test_confidence_head_stops_blocks_early_and_greedy_text_is_unchanged():
    """Oracle backend with a confidence head: rounds verify fewer proposals when the running product
    drops under the ladder, every round records its confidences, and at temperature 0 the text is the
    plain greedy text whatever the ladder."""
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.serve.backend import OracleBackend
    from titanic_flash_41_b200.spec.decoder import DecodeSlot

    def run(ladder, temperature):
        cfg = tiny_config(draft=DraftConfig(layers=1, depth=3, confidence_head=True, markov_rank=8,
                                            confidence_ladder=ladder))
        W = oracle.init_weights(cfg, 0)
        assert W["mtp.0.confidence_head.proj.weight"].shape == (1, cfg.hidden + 8)
        b = OracleBackend(cfg, W, regions=1, max_context=256, chunk=32)
        prompt = torch.randint(3, cfg.vocab, (30,), generator=torch.Generator().manual_seed(2)).tolist()
        lg = b.prefill(0, prompt, 0, None)
        sl = DecodeSlot(region=0, length=30, anchor=b.sample(lg, temperature, 1.0, 7, 30), seed=7,
                        temperature=temperature, top_p=1.0)
        rounds = []
        while len(sl.emitted) < 24:
            toks = b.decode_step([sl])[0]
            assert 1 <= len(sl.confidence) <= 3 and all(0.0 < c < 1.0 for c in sl.confidence)
            rounds.append((len(toks), list(sl.confidence)))
        return sl.emitted[:24], rounds
    never, r_never = run((0.0,), 0.0)          # thresholds of zero: every proposal is verified
    always, r_always = run((2.0,), 0.0)        # unreachable thresholds: one proposal per round
    prod, r_prod = run((0.15, 0.25, 0.20), 0.0)
    assert never == always == prod
    assert all(len(c) == 3 for _, c in r_never) and all(len(c) == 2 and n <= 2 for n, c in r_always)
    from titanic_flash_41_b200.spec.verify import causal_rows
    for n, c in r_prod:
        # the drafter stopped exactly where the rule says (the last confidence is the one that failed)
        assert n <= len(c) + 1 and (len(c) == 3 or causal_rows(c, (0.15, 0.25, 0.20)) == len(c) - 1)
    # sampling: still runs and still commits at least the anchor every round
    sampled, r_s = run((0.15, 0.25, 0.20), 0.8)
    assert len(sampled) == 24 and all(n >= 1 for n, _ in r_s)


def test_history_text_of_bulk_and_single_commits_behaves_like_one_list():
    """The copy-proposal history keeps a bulk-committed prompt as an array and later tokens in a list:
    indexing, slicing across the seam, truncation on either side and proposals equal a plain list's."""
    import random
    rnd = random.Random(3)
    prompt = [rnd.randrange(3, 40) for _ in range(700)]           # > 256 tokens: the bulk path
    later = [rnd.randrange(3, 40) for _ in range(90)]
    a = HistoryLookup(prompt, depth=6)
    b = HistoryLookup(depth=6)
    for i, t in enumerate(prompt):
        b.commit(i, [t])
    assert all((x == y).all() for x, y in zip(a.tables, b.tables))
    for i, t in enumerate(later):
        a.commit(700 + i, [t])
        b.commit(700 + i, [t])
    ref = prompt + later
    assert len(a.tokens) == len(ref) and a.tokens[0] == ref[0] and a.tokens[-1] == ref[-1] and a.tokens[699] == ref[699]
    assert a.tokens[690:710] == ref[690:710] and a.tokens[:5] == ref[:5] and a.tokens[780:] == ref[780:]
    assert all((x == y).all() for x, y in zip(a.tables, b.tables))
    pa, pb = a.propose(pending=[ref[-1]]), b.propose(pending=[ref[-1]])
    assert (pa is None) == (pb is None) and (pa is None or (pa.tokens, pa.matched, pa.source_end) == (pb.tokens, pb.matched, pb.source_end))
    a.truncate(750)                                                # inside the list part
    assert len(a.tokens) == 750 and a.tokens[745:] == ref[745:750]
    a.truncate(650)                                                # inside the array part
    assert len(a.tokens) == 650 and a.tokens[640:] == ref[640:650]
    a.commit(650, ref[650:660])
    assert a.tokens[645:660] == ref[645:660]
    # a second bulk commit after single tokens folds the list into the array
    a.commit(660, ref[660:] + prompt)
    assert len(a.tokens) == 790 + 700 and a.tokens[785:795] == (ref + prompt)[785:795]


def test_rolling_hash_lookup_equals_a_brute_force_search():
    """The rolled suffix hashes find what a search over the text finds: for random repetitive text, every
    proposal is a true earlier occurrence of the longest indexed suffix that has one (hash collisions may only
    lose a proposal, and with 65,536 slots over 600 tokens they do not)."""
    import random
    from titanic_flash_41_b200.spec.history_lookup import LENGTHS
    rnd = random.Random(7)
    phrase = [rnd.randrange(3, 30) for _ in range(70)]
    text = []
    while len(text) < 600:
        text += phrase[: rnd.randrange(20, 70)] + [rnd.randrange(3, 30) for _ in range(rnd.randrange(1, 9))]
    h = HistoryLookup(depth=5)
    hits = 0
    for i, t in enumerate(text):
        h.commit(i, [t])
        pending = [text[i + 1]] if i + 1 < len(text) and i % 3 == 0 else []
        p = h.propose(pending=pending)
        full = text[: i + 1] + pending
        want = None
        for L in sorted(LENGTHS, reverse=True):
            if len(full) < L:
                continue
            suf = full[len(full) - L:]
            # the LAST earlier occurrence whose following token is committed text (what a slot keeps)
            cands = [e for e in range(L, i + 1) if text[e - L:e] == suf and e < len(text[: i + 1])]
            cands = [e for e in cands if e <= i]
            if cands:
                want = (L, max(cands))
                break
        if want is None:
            assert p is None
        else:
            assert p is not None and p.source_end == want[1] and p.matched >= want[0], (i, want, p)
            assert p.tokens == text[want[1]: want[1] + 5][: len(p.tokens)] and len(p.tokens) >= 1
            hits += 1
    assert hits > 100
    # a truncation re-seeds the rolling state (slots of the dropped text go stale and are caught by the
    # confirmation): committing the same continuation again ends in the state of a fresh index
    h.truncate(500)
    for i in range(500, 600):
        h.commit(i, [text[i]])
    q = HistoryLookup(text[:600], depth=5)                # bulk path over the same text
    assert h._raw == q._raw and len(h.tokens) == len(q.tokens) == 600
    pa, pb = h.propose(), q.propose()
    assert pa is None or pb is None or pa.tokens[:1] == text[pa.source_end: pa.source_end + 1]


@pytest.mark.parametrize("g,stop", [(1, None), (3, None), (3, "causal"), (2, "point")])
def test_block_verification_on_the_host_preserves_the_target_law(g, stop):
    """Monte-Carlo over the host recurrence (the oracle of the sampling kernels): the first token a round
    emits follows the (temperature / nucleus modified) target law, for full blocks, for blocks shortened by
    a rule that only looks at what precedes each proposal, and for point-mass (copy) proposals."""
    import random

    from titanic_flash_41_b200.spec import verify
    V, N = 7, 24000
    gen = torch.Generator().manual_seed(4)
    P = verify.modified_law(torch.randn(g + 1, V, generator=gen) * 1.5, 0.8, 0.9)
    Q = verify.modified_law(torch.randn(g, V, generator=gen) * 1.5, 0.8, 0.9)
    rnd = random.Random(9)
    counts = torch.zeros(V, dtype=torch.float64)
    lengths = [0] * (g + 1)
    for _ in range(N):
        if stop == "point":
            props = [int(Q[i].argmax()) for i in range(g)]           # the copy source names its tokens with certainty
            Qn = None
        else:
            props = [verify.sample_from(Q[i], rnd.random()) for i in range(g)]
            Qn = Q
        n = g
        if stop == "causal":
            # the length is decided from the tokens BEFORE each proposal only (here: a fake confidence of the previous token)
            conf = [0.9] + [0.3 + 0.1 * (props[i - 1] % 5) for i in range(1, g)]
            n = verify.causal_rows(conf, (0.3, 0.2))
        lengths[n] += 1
        Pn = P[: n + 1]
        Qb = None if Qn is None else Qn[:n]
        tau, nxt = verify.block_verify(Pn, Qb, props[:n], [rnd.random() for _ in range(n)], rnd.random())
        first = props[0] if tau >= 1 else nxt
        counts[first] += 1
    emp = counts / N
    # three standard errors of the largest cell, plus the nucleus cells that must stay empty
    assert float((emp - P[0]).abs().max()) < 3.5 * (0.25 / N) ** 0.5 + 1e-9, (emp, P[0])
    assert bool((emp[P[0] == 0] == 0).all())
    if stop == "causal":
        assert sum(1 for c in lengths if c > 0) >= 2              # blocks of different lengths really occurred
