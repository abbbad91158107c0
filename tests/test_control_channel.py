"""Four ranks as threads on loopback: command broadcast, agreement, divergence -> poison,
disconnect never reads as success, all-rank admission votes."""
import socket
import threading

import pytest

from titanic_flash_41_b200.parallel.control import ControlChannel, ControlError


def _cohort(world, body):
    srv = socket.create_server(("127.0.0.1", 0))
    port = srv.getsockname()[1]
    results, errors = [None] * world, [None] * world

    def run(rank):
        try:
            ch = ControlChannel.connect(rank, world, "127.0.0.1", port, b"ticket", 10.0, srv if rank == 0 else None)
            results[rank] = body(rank, ch)
        except Exception as e:  # noqa: BLE001
            errors[rank] = e
    ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(20)
    srv.close()
    return results, errors


def test_commands_agreement_and_votes():
    def body(rank, ch):
        got = [ch.command(b"begin:%d" % i if rank == 0 else None) for i in range(3)]
        assert ch.agree(b"state-7")
        admit = ch.all_admit(rank != 2)        # rank 2 refuses (e.g. memory floor)
        nxt = ch.agree_and_next(b"tokens-1-2", b"step" if rank == 0 else None)
        return got, admit, nxt
    res, err = _cohort(4, body)
    assert err == [None] * 4
    for got, admit, nxt in res:
        assert got == [b"begin:0", b"begin:1", b"begin:2"] and admit is False and nxt == b"step"


def test_divergence_poisons_every_rank():
    def body(rank, ch):
        with pytest.raises(ControlError):
            ch.agree(b"A" if rank != 3 else b"B")
        with pytest.raises(ControlError):       # and stays poisoned
            ch.command(b"x" if rank == 0 else None)
        return True
    res, err = _cohort(4, body)
    assert err == [None] * 4 and res == [True] * 4


def test_disconnect_is_never_success():
    def body(rank, ch):
        if rank == 1:
            ch.close()                           # the rank exits between steps
            return "left"
        with pytest.raises(ControlError):
            ch.agree(b"same")
            ch.agree(b"same")
        return "poisoned"
    res, err = _cohort(3, body)
    assert err == [None] * 3 and res[0] == "poisoned"


def test_bad_ticket_is_refused():
    srv = socket.create_server(("127.0.0.1", 0))
    port = srv.getsockname()[1]
    out = {}

    def server():
        try:
            ControlChannel.connect(0, 2, "127.0.0.1", port, b"right", 5.0, srv)
        except ControlError as e:
            out["err"] = str(e)
    t = threading.Thread(target=server)
    t.start()
    try:
        ControlChannel.connect(1, 2, "127.0.0.1", port, b"wrong", 5.0)
    except (ControlError, OSError):
        pass
    t.join(10)
    srv.close()
    assert "bad control hello" in out.get("err", "")


def test_followers_that_start_before_the_leader_keep_trying():
    """Ranks start in any order: a follower whose connect is refused because rank 0 is not listening
    yet retries until the deadline (and reports a clear error when nobody ever listens)."""
    import time
    probe = socket.create_server(("127.0.0.1", 0))
    port = probe.getsockname()[1]
    probe.close()                                  # a free port nobody listens on yet
    out, err = [None, None], [None, None]

    def run(rank, delay):
        try:
            time.sleep(delay)
            ch = ControlChannel.connect(rank, 2, "127.0.0.1", port, b"late", 10.0)
            out[rank] = ch.command(b"hello" if rank == 0 else None)
        except Exception as e:  # noqa: BLE001
            err[rank] = e
    ts = [threading.Thread(target=run, args=(1, 0.0)), threading.Thread(target=run, args=(0, 0.6))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(20)
    assert err == [None, None] and out == [b"hello", b"hello"]
    t0 = time.monotonic()
    with pytest.raises(ControlError, match="no control listener"):
        ControlChannel.connect(1, 2, "127.0.0.1", port, b"late", 0.4)
    assert time.monotonic() - t0 < 5
