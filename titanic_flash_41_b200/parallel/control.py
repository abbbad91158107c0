"""CPU control plane between the ranks of one cohort.

Rank 0 turns work into binary commands; every rank executes the same command deterministically
and, after each step, all ranks check that they committed the same state.  Three primitives
(reference: src/control_channel.rs:15-24 frame kinds, :333 agree, :361 all_admit, :389
agree_and_next):

  command(bytes)        rank 0 -> all: the next command
  agree(bytes) -> bool  every rank submits its committed-state record; True iff all are equal
  all_admit(bool)       logical AND of every rank's local admission vote (memory floor etc.)

Any I/O error, short read, out-of-order frame or diverging agreement poisons the channel: every
later call raises ``ControlError`` and the rank retires (the cohort is restarted from outside;
there is no elastic recovery in the reference either).  Transport: TCP on loopback with a
ticket check, bounded timeouts.
"""
from __future__ import annotations

import hashlib
import socket
import struct
import time
import threading
from typing import List, Optional

K_COMMAND, K_AGREE, K_VERDICT, K_VOTE, K_HELLO = 1, 2, 3, 4, 5
MAX_FRAME = 1 << 20


class ControlError(RuntimeError):
    pass


def _send(sock: socket.socket, kind: int, seq: int, payload: bytes) -> None:
    sock.sendall(struct.pack("<BIQ", kind, len(payload), seq) + payload)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        part = sock.recv(n - len(buf))
        if not part:
            raise ControlError("peer closed the control channel")
        buf += part
    return bytes(buf)


def _recv(sock: socket.socket, want_kind: int, want_seq: int) -> bytes:
    kind, n, seq = struct.unpack("<BIQ", _recv_exact(sock, 13))
    if n > MAX_FRAME:
        raise ControlError("oversized control frame")
    payload = _recv_exact(sock, n)
    if kind != want_kind or seq != want_seq:
        raise ControlError(f"control frame out of order: kind {kind} seq {seq}, expected {want_kind}/{want_seq}")
    return payload


class ControlChannel:
    def __init__(self, rank: int, world: int, socks: List[socket.socket]):
        self.rank, self.world, self.socks = rank, world, socks
        self.seq = 0
        self.poisoned: Optional[str] = None
        self.lock = threading.Lock()

    # ---- construction -------------------------------------------------------------------------
    @staticmethod
    def connect(rank: int, world: int, host: str, port: int, ticket: bytes, timeout: float = 30.0,
                listener: Optional[socket.socket] = None) -> "ControlChannel":
        tag = hashlib.sha256(b"tflash-control\0" + ticket).digest()
        if world == 1:
            return ControlChannel(0, 1, [])
        if rank == 0:
            srv = listener or socket.create_server((host, port))
            srv.settimeout(timeout)
            peers: List[Optional[socket.socket]] = [None] * world
            try:
                for _ in range(world - 1):
                    c, _ = srv.accept()
                    c.settimeout(timeout)
                    hello = _recv(c, K_HELLO, 0)
                    r = struct.unpack("<I", hello[:4])[0]
                    if hello[4:] != tag or not (0 < r < world) or peers[r] is not None:
                        c.close()
                        raise ControlError("bad control hello")
                    c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                    peers[r] = c
            finally:
                if listener is None:
                    srv.close()
            return ControlChannel(0, world, [p for p in peers[1:]])
        # rank 0 may not be listening yet (the ranks start in any order): keep trying until the deadline
        deadline = time.monotonic() + timeout
        while True:
            try:
                s = socket.create_connection((host, port), timeout=timeout)
                break
            except (ConnectionRefusedError, ConnectionResetError, socket.timeout, TimeoutError) as e:
                if time.monotonic() >= deadline:
                    raise ControlError(f"rank {rank}: no control listener at {host}:{port} within {timeout:.0f} s") from e
                time.sleep(0.05)
        s.settimeout(timeout)
        s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        _send(s, K_HELLO, 0, struct.pack("<I", rank) + tag)
        return ControlChannel(rank, world, [s])

    # ---- plumbing -----------------------------------------------------------------------------
    def _guard(self):
        if self.poisoned:
            raise ControlError(f"control channel is poisoned: {self.poisoned}")

    def _poison(self, why: str):
        self.poisoned = self.poisoned or why
        for s in self.socks:
            try:
                s.close()
            except OSError:
                pass

    def _run(self, fn):
        with self.lock:
            self._guard()
            self.seq += 1
            try:
                return fn(self.seq)
            except (OSError, ControlError, struct.error) as e:
                self._poison(str(e))
                raise ControlError(str(e)) from e

    # ---- primitives ---------------------------------------------------------------------------
    def command(self, payload: Optional[bytes] = None) -> bytes:
        """Rank 0 passes the command and gets it back; other ranks pass None and receive it."""
        def go(seq):
            if self.rank == 0:
                assert payload is not None
                for s in self.socks:
                    _send(s, K_COMMAND, seq, payload)
                return payload
            return _recv(self.socks[0], K_COMMAND, seq)
        return self._run(go)

    def agree(self, record: bytes) -> bool:
        """True iff every rank submitted the same bytes.  A divergence poisons the channel on every
        rank (it is never reported as success)."""
        def go(seq):
            if self.rank == 0:
                same = True
                for s in self.socks:
                    same &= _recv(s, K_AGREE, seq) == record
                for s in self.socks:
                    _send(s, K_VERDICT, seq, b"\x01" if same else b"\x00")
            else:
                _send(self.socks[0], K_AGREE, seq, record)
                same = _recv(self.socks[0], K_VERDICT, seq) == b"\x01"
            if not same:
                raise ControlError("ranks committed different state")
            return True
        return self._run(go)

    def all_admit(self, vote: bool) -> bool:
        """AND of all ranks' votes; every rank then takes the same branch."""
        def go(seq):
            if self.rank == 0:
                ok = vote
                for s in self.socks:
                    ok &= _recv(s, K_VOTE, seq) == b"\x01"
                for s in self.socks:
                    _send(s, K_VERDICT, seq, b"\x01" if ok else b"\x00")
                return ok
            _send(self.socks[0], K_VOTE, seq, b"\x01" if vote else b"\x00")
            return _recv(self.socks[0], K_VERDICT, seq) == b"\x01"
        return self._run(go)

    def agree_and_next(self, record: bytes, next_command: Optional[bytes] = None) -> bytes:
        """One round trip for the common case: agree on the step's result, then learn the next command."""
        self.agree(record)
        return self.command(next_command)

    def close(self) -> None:
        for s in self.socks:
            try:
                s.close()
            except OSError:
                pass
