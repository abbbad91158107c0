"""Serving worker on the CPU oracle backend: admission, prefix reuse, batched decode, token-exact
resume from a cached image, cancellation."""
import threading

import pytest
import torch

from titanic_flash_41_b200.config import tiny_config
from titanic_flash_41_b200.models import oracle
from titanic_flash_41_b200.serve.backend import OracleBackend
from titanic_flash_41_b200.serve.scheduler import Job, QueueFull, Scheduler
from titanic_flash_41_b200.serve.session_cache import SessionCache
from titanic_flash_41_b200.serve.worker import Worker


def _mk(regions=2, queue_limit=4, cfg=None, **kw):
    cfg = cfg or tiny_config()
    W = oracle.init_weights(cfg, 0)
    b = OracleBackend(cfg, W, regions=regions, max_context=512, chunk=32)
    s = Scheduler(regions, queue_limit, 2)
    return cfg, Worker(b, s, SessionCache(slots=8, budget_bytes=1 << 30), eos_id=1, checkpoint_min=32,
                       checkpoint_align=32, **kw), s


def _job(jid, toks, n, events, **kw):
    return Job(jid, list(toks), n, emit=lambda k, p: events.append((jid, k, p)), **kw)


def _drain(w, max_cmds=400):
    for _ in range(max_cmds):
        if w.run_once(0.0) == "idle" and not w.active and w.sched.waiting() == 0:
            return
    raise AssertionError("worker did not drain")


def test_generation_matches_plain_greedy_and_reuses_prefix():
    cfg, w, s = _mk()
    ev = []
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(3, cfg.vocab, (70,), generator=g).tolist()
    s.submit(_job("a", prompt, 12, ev, temperature=0.0))
    _drain(w)
    toks = [t for j, k, p in ev if k == "tokens" for t in p]
    ref = oracle.OracleModel(cfg, oracle.init_weights(cfg, 0))
    want, _ = oracle.greedy_generate(ref, [torch.tensor(prompt)], 12)
    # speculative decoding with a draft head must commit exactly the greedy tokens
    assert toks == want[0][: len(toks)] and len(toks) == 12
    ready = [p for j, k, p in ev if k == "ready"][0]
    assert ready["prompt_n"] == 70 and ready["cache_n"] == 0
    # the follow-up turn restores the completed image: only the new tokens are prefilled
    ev2 = []
    follow = prompt + toks + [5, 6, 7]
    s.submit(_job("b", follow, 6, ev2, temperature=0.0))
    _drain(w)
    ready2 = [p for j, k, p in ev2 if k == "ready"][0]
    assert ready2["cache_n"] >= 70 and ready2["prompt_n"] <= len(follow) - 70
    toks2 = [t for j, k, p in ev2 if k == "tokens" for t in p]
    want2, _ = oracle.greedy_generate(ref, [torch.tensor(follow)], 6)
    assert toks2 == want2[0]          # token-exact resume from the snapshot
    assert w.cache.stats["hits"] >= 1 and w.cache.stats["reused_tokens"] >= 70


def test_four_requests_two_regions_queue_and_429():
    cfg, w, s = _mk(regions=2, queue_limit=4)
    ev = []
    for i in range(4):
        s.submit(_job(f"j{i}", [10 + i] * 20, 5, ev, temperature=0.6, top_p=0.95, seed=i))
    try:
        s.submit(_job("j4", [3] * 5, 5, ev))
        assert False, "queue should be full"
    except QueueFull as e:
        assert e.code == "queue_full"
    _drain(w)
    done = sorted(j for j, k, p in ev if k == "done")
    assert done == ["j0", "j1", "j2", "j3"]
    for i in range(4):
        n = sum(len(p) for j, k, p in ev if k == "tokens" and j == f"j{i}")
        assert 1 <= n <= 5


def test_cancel_and_background_hold():
    cfg, w, s = _mk(regions=1)
    ev = []
    j = _job("c", [9] * 30, 200, ev, temperature=0.0)
    s.submit(j)
    for _ in range(3):
        w.run_once(0.0)
    j.cancelled.set()
    _drain(w)
    assert [p["finish_reason"] for jj, k, p in ev if k == "done"] == ["cancelled"]
    s.priority_lease(30.0)
    s.submit(_job("bg", [4] * 8, 2, ev, background=True))
    assert s.admit() == []            # background held by the lease
    s.priority_lease(0.0)
    _drain(w)
    assert any(jj == "bg" and k == "done" for jj, k, p in ev)


def test_long_context_stress_script_on_the_oracle():
    """The long-context serving benchmark, scaled down: every resumed conversation is served from its
    cached image (only the follow-up is prefilled)."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_long_context", os.path.join(root, "benchmarks", "bench_long_context.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = mod.main(["--backend", "oracle", "--sessions", "3", "--regions", "2", "--target", "192", "--grow", "96",
                    "--short", "4", "--short-tokens", "20", "--follow", "24", "--new-tokens", "3", "--chunk", "32",
                    "--checkpoint", "32", "--cache-slots", "16",
                    "--device-cache-gb", "0.0006", "--host-cache-gb", "0.004"])
    assert out["context"] >= 192 and len(out["resume_ttft_s"]) == 3
    # tiny cache budgets force displacement: most conversations still resume from their last image,
    # the others from an earlier checkpoint of the same conversation
    assert sum(c >= 190 for c in out["resume_cached_tokens"]) >= 2 and all(c >= 96 for c in out["resume_cached_tokens"]), out
    assert out["reused_token_share"] > 0.3 and out["cache_stats"]["parked"] > 0


def test_startup_self_check_on_the_oracle_backend():
    from titanic_flash_41_b200.serve.warmup import SelfCheckError, self_check
    cfg = tiny_config()
    W = oracle.init_weights(cfg, 0)
    b = OracleBackend(cfg, W, regions=2, max_context=256, chunk=32)
    rep = self_check(b, steps=3)
    assert rep["tokens"] >= 4 and rep["state_bytes"] > 0
    # a backend whose second run differs is caught
    orig = b.sample
    calls = {"n": 0}

    def flaky(*a, **k):
        calls["n"] += 1
        return (orig(*a, **k) + (1 if calls["n"] == 2 else 0)) % cfg.vocab
    b.sample = flaky
    try:
        self_check(b, steps=1)
        assert False, "difference not detected"
    except SelfCheckError:
        pass


def test_worker_hands_the_tokens_before_each_prefilled_part_to_backends_that_want_them():
    """Backends whose models hash n-grams (wants_prev) get the tokens right before every prefilled
    part, across the seam between a restored prefix and the new tokens; decode slots carry the
    tokens before their anchor."""
    cfg, w, s = _mk()
    seen = []

    class Wants(type(w.b)):
        wants_prev = True

        def prefill(self, region, tokens, start, on_chunk=None, prev=()):
            seen.append((start, list(tokens)[:2], list(prev)))
            return super().prefill(region, tokens, start, on_chunk)

    w.b.__class__ = Wants
    ev = []
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(3, cfg.vocab, (70,), generator=g).tolist()
    s.submit(_job("a", prompt, 6, ev, temperature=0.0))
    _drain(w)
    assert seen and seen[0][0] == 0 and seen[0][2] == []
    for start, head, prev in seen:
        assert prev == prompt[max(0, start - 8):start] and head == prompt[start:start + 2]
    toks = [t for j, k, p in ev if k == "tokens" for t in p]
    seen.clear()
    follow = prompt + toks + [5, 6, 7]
    s.submit(_job("b", follow, 4, [], temperature=0.0))
    _drain(w)
    assert seen and all(prev == follow[max(0, start - 8):start] for start, _, prev in seen)
    assert min(start for start, _, _ in seen) >= 64            # the restored prefix was not prefilled again


def test_two_ranks_follow_rank0_prefill_directives_despite_clock_skew_and_local_cancel():
    """Tensor-parallel serving: whether a prefill chunk is followed by an interleaved decode step, or
    the prefill stops because the request was cancelled, is rank 0's decision, broadcast per chunk.
    Rank 1 has a clock that never advances and no job table; it must still take exactly the same
    steps (the agreement after every command would poison the channel otherwise)."""
    import socket

    from titanic_flash_41_b200.parallel.control import ControlChannel
    from titanic_flash_41_b200.serve import worker as WK

    cfg = tiny_config()
    W = oracle.init_weights(cfg, 0)
    srv = socket.create_server(("127.0.0.1", 0))
    port = srv.getsockname()[1]
    sched = Scheduler(2, 4, 2)
    ev = []
    workers, errors = [None, None], [None, None]
    ticks = {"n": 0}
    jobs = {}

    def fast_clock():                      # rank 0: every look at the clock is a second later
        ticks["n"] += 1
        if "b" in jobs and ticks["n"] >= jobs["b_cancel_at"]:
            jobs["b"].cancelled.set()       # the client of request b goes away mid-prefill (seen by rank 0 only)
        return float(ticks["n"])

    def run(rank):
        try:
            ch = ControlChannel.connect(rank, 2, "127.0.0.1", port, b"t", 20.0, srv if rank == 0 else None)
            b = OracleBackend(cfg, W, regions=2, max_context=512, chunk=32)
            w = Worker(b, sched if rank == 0 else None, SessionCache(slots=8, budget_bytes=1 << 30), eos_id=1,
                       control=ch, rank=rank, prefill_slice_s=0.5, checkpoint_min=512, checkpoint_align=512)
            w.clock = fast_clock if rank == 0 else (lambda: 0.0)
            workers[rank] = w
            w._pending = []
            while w.running:
                w.run_once(0.0)
        except Exception as e:  # noqa: BLE001
            errors[rank] = e

    g = torch.Generator().manual_seed(4)
    sched.submit(_job("a", torch.randint(3, cfg.vocab, (40,), generator=g).tolist(), 60, ev, temperature=0.0))
    ts = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for t in ts:
        t.start()
    # wait until a decodes, then submit a long prompt b that will be cancelled on rank 0 during prefill
    import time as _t
    t0 = _t.time()
    while not any(j == "a" and k == "tokens" for j, k, p in ev) and _t.time() - t0 < 30:
        _t.sleep(0.01)
    jb = _job("b", torch.randint(3, cfg.vocab, (230,), generator=g).tolist(), 8, ev, temperature=0.0)
    jobs["b_cancel_at"] = 10 ** 9
    jobs["b"] = jb
    sched.submit(jb)
    t0 = _t.time()
    while not workers[0].directives and _t.time() - t0 < 30:
        _t.sleep(0.005)
    jobs["b_cancel_at"] = ticks["n"] + 6          # a few chunks later
    t0 = _t.time()
    while not any(j == "a" and k == "done" for j, k, p in ev) and _t.time() - t0 < 60:
        _t.sleep(0.01)
    sched.close()
    for t in ts:
        t.join(30)
    srv.close()
    assert errors == [None, None], errors
    d0, d1 = workers[0].directives, workers[1].directives
    assert d0 == d1 and len(d0) >= 3
    assert WK.D_STEP in d0                         # rank 0's clock forced interleaved steps; rank 1 followed
    assert d0[-1] == WK.D_CANCEL                   # and the cancellation seen by rank 0 only
    assert any(j == "b" and k == "error" and p["code"] == "cancelled" for j, k, p in ev)
    assert not any(j == "b" and k == "tokens" for j, k, p in ev)
    assert any(j == "a" and k == "done" for j, k, p in ev)


def test_job_cancelled_while_queued_gets_a_terminal_event():
    s = Scheduler(1, 4, 2)
    ev = []
    a, b = _job("a", [5] * 8, 4, ev), _job("b", [6] * 8, 4, ev)
    s.submit(a)
    s.submit(b)
    assert s.admit() == [a]
    b.cancelled.set()
    s.release(a)
    assert s.admit() == []
    assert ("b", "error", {"code": "cancelled", "message": "cancelled while queued"}) in ev


def test_two_conversations_take_turns_in_one_region_token_exactly():
    """More conversations than regions: the decoding conversation is parked as a request checkpoint
    after its turn, the waiting one runs, and so on; every conversation commits exactly the tokens
    it commits when it runs alone (sampling is addressed by position)."""
    cfg = tiny_config()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, cfg.vocab, (30 + 7 * i,), generator=g).tolist() for i in range(2)]

    def solo(p, seed):
        _, w, s = _mk(regions=1, turn_tokens=0)
        ev = []
        s.submit(_job("x", p, 30, ev, temperature=0.7, top_p=0.9, seed=seed))
        _drain(w)
        return [t for j, k, pl in ev if k == "tokens" for t in pl]
    want = [solo(p, 11 + i) for i, p in enumerate(prompts)]
    _, w, s = _mk(regions=1, turn_tokens=8)
    ev = []
    for i, p in enumerate(prompts):
        s.submit(_job(f"c{i}", p, 30, ev, temperature=0.7, top_p=0.9, seed=11 + i))
    _drain(w, max_cmds=2000)
    for i in range(2):
        got = [t for j, k, pl in ev if k == "tokens" and j == f"c{i}" for t in pl]
        assert got == want[i], i
    kinds = [e["kind"] for e in w.log.snapshot(4096)["events"]]
    # every Begin records what the host stalled on while the prompt was prefilled
    assert all(isinstance(e["host_stall"], dict) for e in w.log.snapshot(4096)["events"] if e["kind"] == "begin")
    assert kinds.count("pause") >= 2 and kinds.count("resume") == kinds.count("pause")
    assert sorted(j for j, k, pl in ev if k == "done") == ["c0", "c1"] and not w.parked


def test_copy_proposals_from_history_lookup_are_verified_exactly():
    """A prompt that repeats itself: the lookup proposes the continuation it saw, greedy decoding
    commits exactly what it commits without the lookup, in fewer steps."""
    cfg = tiny_config()
    g = torch.Generator().manual_seed(5)
    phrase = torch.randint(3, cfg.vocab, (40,), generator=g).tolist()
    prompt = phrase + phrase + phrase[:20]

    def run(lookup):
        _, w, s = _mk(regions=1, history_lookup=lookup)
        ev = []
        s.submit(_job("h", prompt, 16, ev, temperature=0.0))
        _drain(w)
        done = [pl for j, k, pl in ev if k == "done"][0]
        return [t for j, k, pl in ev if k == "tokens" for t in pl], done["steps"]
    plain, _ = run(False)
    with_lookup, _ = run(True)
    assert with_lookup == plain


def test_interrupted_prefill_is_resumed_from_its_last_whole_chunk():
    """A request cancelled during its prefill leaves a checkpoint of the chunks it finished; the same
    prompt sent again starts there and generates what an uninterrupted request generates."""
    cfg = tiny_config()
    W = oracle.init_weights(cfg, 0)
    sched = Scheduler(1, 4, 1)
    b = OracleBackend(cfg, W, regions=1, max_context=512, chunk=32)
    w = Worker(b, sched, SessionCache(slots=8, budget_bytes=1 << 30), eos_id=1, checkpoint_min=64, checkpoint_align=512)
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(3, cfg.vocab, (200,), generator=g).tolist()
    ev = []
    j = _job("x", prompt, 4, ev, temperature=0.0)
    looks = {"n": 0}
    decide = w._chunk_directive

    def directive(job, last_slice):            # the client goes away while the fourth chunk runs
        looks["n"] += 1
        if looks["n"] == 4:
            j.cancelled.set()
        return decide(job, last_slice)
    w._chunk_directive = directive
    sched.submit(j)
    _drain(w)
    assert any(k == "error" and p["code"] == "cancelled" for _, k, p in ev)
    saved = [e for e in w.log.snapshot(4096)["events"] if e.get("kind") == "prefill_interrupted"]
    assert saved and saved[0]["saved"] >= 64 and saved[0]["saved"] % 32 == 0 and saved[0]["saved"] < 200
    w._chunk_directive = decide
    ev2 = []
    sched.submit(_job("y", prompt, 4, ev2, temperature=0.0))
    _drain(w)
    ready = [p for _, k, p in ev2 if k == "ready"][0]
    assert ready["cache_n"] == saved[0]["saved"] and ready["prompt_n"] == 200 - saved[0]["saved"]
    # the resumed request generates what a fresh worker generates for the same prompt
    sched3 = Scheduler(1, 4, 1)
    w3 = Worker(OracleBackend(cfg, W, regions=1, max_context=512, chunk=32), sched3,
                SessionCache(slots=8, budget_bytes=1 << 30), eos_id=1, checkpoint_min=64, checkpoint_align=512)
    ev3 = []
    sched3.submit(_job("z", prompt, 4, ev3, temperature=0.0))
    _drain(w3)
    toks = lambda e: [t for _, k, p in e if k == "tokens" for t in p]
    assert toks(ev2) == toks(ev3) and len(toks(ev2)) == 4


@pytest.mark.parametrize("mixed", [False, True])
def test_relocated_conversation_continues_with_the_same_tokens(mixed):
    """A decoding conversation moved to another region between steps produces the tokens it would
    have produced in place (sampling is addressed by position; the state image travels).  ``mixed``:
    two compressed streams with their own ratios, each saved with its own entry count."""
    model = tiny_config(n_layers=3, compress_ratio=1, compress_ratios=(2, 1), kv_source_layers=(0, 1),
                        index_source_layers=(0, 1, 2), index_topk=8) if mixed else None
    def run(move):
        cfg, w, s = _mk(regions=2, cfg=model)
        ev = []
        g = torch.Generator().manual_seed(21)
        s.submit(_job("m", torch.randint(3, cfg.vocab, (40,), generator=g).tolist(), 24, ev, temperature=0.7, top_p=0.9,
                      seed=5))
        for _ in range(4):
            w.run_once(0.0)
        if move:
            assert 0 in w.active and 1 not in w.active
            w.execute({"op": "relocate", "region": 0, "to": 1})
            assert 1 in w.active and 0 not in w.active and w.active[1].job.region == 1
            assert s.free_regions() == [0]
        _drain(w)
        return [t for _, k, p in ev if k == "tokens" for t in p], [p["finish_reason"] for _, k, p in ev if k == "done"]
    a, b = run(False), run(True)
    assert a == b and len(a[0]) == 24 and a[1] == ["length"]


def test_worker_logs_the_drafters_confidences_per_round_when_asked():
    from titanic_flash_41_b200.config import DraftConfig
    cfg = tiny_config(draft=DraftConfig(layers=1, depth=3, confidence_head=True))
    _, w, s = _mk(regions=1, cfg=cfg, log_confidence=True)
    ev = []
    s.submit(_job("c", torch.randint(3, cfg.vocab, (20,), generator=torch.Generator().manual_seed(4)).tolist(), 10, ev))
    _drain(w)
    rounds = [e for e in w.log.snapshot(4096)["events"] if e["kind"] == "step_confidence"]
    assert rounds and all(1 <= e["verified"] <= 3 and e["emitted"] <= e["verified"] + 1 and
                          len(e["confidence"]) >= e["verified"] for e in rounds)
    assert not any("token" in k for e in rounds for k in e)


def test_long_context_stress_script_as_two_cpu_ranks():
    """The same script as one rank per process (gloo, oracle backend split over two ranks): rank 0 owns
    the scheduler, rank 1 follows over the control channel; the run ends by itself on both."""
    import json
    import os
    import subprocess
    import sys
    import socket
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as so:                      # a free port for the rendezvous (the control channel takes port + 13)
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(root, "benchmarks", "bench_long_context.py"), "--backend", "oracle",
           "--sessions", "2", "--regions", "2", "--target", "128", "--grow", "64", "--short", "2", "--short-tokens", "16",
           "--follow", "16", "--new-tokens", "3", "--chunk", "32", "--checkpoint", "32", "--cache-slots", "16"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0 and len(lines) == 1, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.loads(lines[0])
    assert out["n_gpus"] == 2 and out["context"] >= 128 and len(out["resume_ttft_s"]) == 2
    assert all(c >= 120 for c in out["resume_cached_tokens"]), out
