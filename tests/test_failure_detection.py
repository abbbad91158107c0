"""Failure detection on the host (no GPU is faulted, trapped or left waiting): a rank that leaves
between steps, a dropped control frame, a refused admission vote, a kernel status word, and the
launcher's cohort supervisor."""
import os
import socket
import sys
import threading
import time

import pytest

from titanic_flash_41_b200 import launcher
from titanic_flash_41_b200.config import tiny_config
from titanic_flash_41_b200.models import oracle
from titanic_flash_41_b200.parallel.control import ControlChannel, ControlError
from titanic_flash_41_b200.serve.backend import OracleBackend
from titanic_flash_41_b200.serve.scheduler import Job, Scheduler
from titanic_flash_41_b200.serve.session_cache import SessionCache
from titanic_flash_41_b200.serve.worker import Worker
from titanic_flash_41_b200.utils.health import Health, Watchdog, control_probe, status_probe


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _pair():
    srv = socket.create_server(("127.0.0.1", 0))
    port = srv.getsockname()[1]
    ch = [None, None]

    def c(rank):
        ch[rank] = ControlChannel.connect(rank, 2, "127.0.0.1", port, b"t", 10.0, srv if rank == 0 else None)
    ts = [threading.Thread(target=c, args=(r,)) for r in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(10)
    srv.close()
    return ch


def test_rank_leaving_between_steps_poisons_the_survivor_and_fails_its_requests():
    """Rank 1 serves two commands and then exits between steps (no collective in flight).  Rank 0
    learns of it on its next broadcast, the watchdog folds the poisoned channel into the sticky
    health state, the request in flight gets a terminal error event and the loop ends."""
    cfg = tiny_config()
    W = oracle.init_weights(cfg, 0)
    ch0, ch1 = _pair()
    sched = Scheduler(2, 4, 2)
    ev = []
    health = Health()
    w0 = Worker(OracleBackend(cfg, W, regions=2, max_context=256, chunk=32), sched, SessionCache(), control=ch0, rank=0,
                health=health)
    w1 = Worker(OracleBackend(cfg, W, regions=2, max_context=256, chunk=32), None, SessionCache(), control=ch1, rank=1)
    sched.submit(Job("a", [5, 6, 7, 8] * 5, 50, temperature=0.0, emit=lambda k, p: ev.append((k, p))))

    def rank1():
        w1._pending = []
        for _ in range(3):                   # begin + two steps, then leave cleanly between steps
            w1.run_once(0.0)
        ch1.close()
    t1 = threading.Thread(target=rank1)
    t1.start()
    dog = Watchdog(health, {"control": control_probe(ch0)}, interval=0.02)
    dog.start()
    t0 = threading.Thread(target=w0.run_forever)
    t0.start()
    t1.join(20)
    t0.join(20)
    assert not t0.is_alive() and not w0.running
    st = health.state()
    assert st["poisoned"] and st["source"] in ("worker", "control")
    assert any(k == "error" and p["code"] == "cohort_failed" for k, p in ev)
    assert not any(k == "done" for k, p in ev)
    # sticky: a later "healthy" probe result does not clear it
    assert not Watchdog(health, {"control": lambda: None}).poll_once()
    with pytest.raises(ControlError):
        ch0.command(b"x")


def test_dropped_frame_is_an_out_of_order_frame_and_poisons_both_sides():
    ch0, ch1 = _pair()
    got = []

    def rank1():
        got.append(ch1.command(None))
        ch1.seq += 1                          # the test drops a frame: rank 1 believes one more was exchanged
        try:
            ch1.command(None)
        except ControlError as e:
            got.append(e)
    t = threading.Thread(target=rank1)
    t.start()
    ch0.command(b"one")
    ch0.command(b"two")
    t.join(10)
    assert got[0] == b"one" and isinstance(got[1], ControlError) and ch1.poisoned
    with pytest.raises(ControlError):          # rank 0 finds out at the next exchange that needs an answer
        ch0.agree(b"s")
    assert ch0.poisoned


def test_refused_admission_vote_is_a_decision_not_a_failure():
    ch0, ch1 = _pair()
    out = [None, None]

    def vote(rank, ch, v):
        out[rank] = (ch.all_admit(v), ch.all_admit(True))
    ts = [threading.Thread(target=vote, args=(0, ch0, True)), threading.Thread(target=vote, args=(1, ch1, False))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(10)
    assert out == [(False, True), (False, True)]          # every rank takes the same branch, twice
    assert ch0.poisoned is None and ch1.poisoned is None


def test_status_word_probe_and_first_report_wins():
    word = [0, 0, 0, 0]
    h = Health()
    dog = Watchdog(h, {"device": status_probe(lambda: tuple(word)), "control": control_probe(None)})
    assert dog.poll_once() and h.state()["poisoned"] is False
    word[:] = [2, 200, 3, 7]                  # TF_TIMEOUT of the one-shot all-reduce: source rank 3, row 7
    assert not dog.poll_once()
    st = h.state()
    assert st["source"] == "device" and "timeout" in st["why"] and "200" in st["why"]
    assert not h.report("control", "later")   # first report wins
    assert h.state()["source"] == "device"


def test_health_endpoint_reports_a_poisoned_cohort():
    import asyncio

    from aiohttp.test_utils import TestClient, TestServer

    from titanic_flash_41_b200.api.server import Frontend, Server
    from titanic_flash_41_b200.api.tokenizer import ByteTokenizer
    from titanic_flash_41_b200.config import ServerConfig

    async def go():
        h = Health()
        srv = Server(ServerConfig(), Frontend(ByteTokenizer(1024), 512), Scheduler(1, 2, 1), health=h.state)
        srv.ready("x")
        async with TestClient(TestServer(srv.app)) as c:
            r = await c.get("/health")
            assert r.status == 200 and (await r.json())["cohort"]["poisoned"] is False
            h.report("control", "peer closed the control channel")
            r = await c.get("/health")
            body = await r.json()
            assert r.status == 503 and body["status"] == "poisoned" and body["cohort"]["source"] == "control"
    asyncio.run(go())


@pytest.mark.timeout(60)
def test_supervisor_stops_the_cohort_when_a_rank_leaves_cleanly():
    """Rank 1 exits 0 between steps while rank 0 keeps serving: after the grace period the
    supervisor stops rank 0 and reports the cohort incomplete."""
    code = ["-c", "import os, sys, time; time.sleep(0.2 if os.environ['RANK'] == '1' else 60); sys.exit(0)"]
    t0 = time.time()
    rc = launcher.launch(code, 2, master_port=_free_port(), pin=False, poll_s=0.02, grace_s=0.5, term_s=5.0)
    assert rc == launcher.INCOMPLETE and time.time() - t0 < 20
    # all ranks leaving together within the grace period is a normal shutdown
    ok = ["-c", "import os, time; time.sleep(0.1 * int(os.environ['RANK']))"]
    assert launcher.launch(ok, 3, master_port=_free_port(), pin=False, poll_s=0.02, grace_s=5.0) == 0


def _heartbeat_rank(rank, world, port, scenario, q):
    """One CPU rank of the heartbeat tests (gloo).  ``scenario``: "poison" = rank 1 reports a local
    fatal condition after a few rounds; "leave" = rank 2 exits between rounds without a word."""
    import torch.distributed as dist

    from titanic_flash_41_b200.utils.health import CohortHeartbeat, Health
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    group = CohortHeartbeat.make_group(timeout=3.0)
    health = Health()
    hb = CohortHeartbeat(health, group, rank, world, interval=0.1)
    hb.start()
    t0 = time.monotonic()
    while hb.rounds < 3 and time.monotonic() - t0 < 20:
        time.sleep(0.02)
    healthy_rounds = hb.rounds
    if scenario == "poison" and rank == 1:
        health.report("device", "kernel 7 reported timeout")
    if scenario == "leave" and rank == 2:
        os._exit(0)                                   # between rounds, nothing in flight on any device
    t1 = time.monotonic()
    while health.ok and time.monotonic() - t1 < 20:
        time.sleep(0.02)
    q.put((rank, healthy_rounds, health.state(), time.monotonic() - t1))
    time.sleep(0.5)                                   # let the last round reach the others
    os._exit(0)


@pytest.mark.parametrize("scenario", ["poison", "leave"])
def test_cohort_heartbeat_spreads_a_poisoned_rank_and_notices_a_rank_that_left(scenario):
    """Host-side heartbeat on its own gloo group: a rank that reports a fatal condition poisons the
    others within an interval; a rank that exits between rounds makes the others' next round fail
    (or time out after 3 s) -- no device collective has to run into its own timeout first."""
    import torch.multiprocessing as mp
    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_heartbeat_rank, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in ps:
        p.start()
    got = {}
    for _ in range(world if scenario == "poison" else world - 1):
        r, rounds, state, waited = q.get(timeout=90)
        got[r] = (rounds, state, waited)
    for p in ps:
        p.join(30)
    assert all(v[0] >= 3 for v in got.values())                       # the cohort was healthy first
    if scenario == "poison":
        assert got[1][1]["source"] == "device"
        for r in (0, 2):
            st = got[r][1]
            assert st["poisoned"] and st["source"] == "cohort" and "[1]" in st["why"] and "poisoned" in st["why"], st
            assert got[r][2] < 5.0
    else:
        for r in (0, 1):
            st = got[r][1]
            assert st["poisoned"] and st["source"] == "cohort", st
            assert got[r][2] < 10.0
