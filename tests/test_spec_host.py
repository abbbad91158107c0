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
