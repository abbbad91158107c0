"""Incremental context transport: a client sends only the messages appended since a base it
names by a chained SHA-256 key; the server keeps recent contexts in a bounded RAM cache and
answers 409 ``context_miss`` when it no longer has the base (reference:
docs/CONTEXT_TRANSPORT.md:9-60, src/context_transport.rs).

key chain:  root = sha256("titanic-context-v1/root")
            next = sha256("titanic-context-v1/chain\\0" || key || sha256("titanic-context-v1/message\\0" || msg))
"""
from __future__ import annotations

import collections
import hashlib
import json
import threading
from typing import Any, Dict, List, Optional, Tuple

ROOT = hashlib.sha256(b"titanic-context-v1/root").hexdigest()


def message_digest(msg_json: str) -> bytes:
    return hashlib.sha256(b"titanic-context-v1/message\0" + msg_json.encode()).digest()


def chain(key_hex: str, msg_json: str) -> str:
    return hashlib.sha256(b"titanic-context-v1/chain\0" + bytes.fromhex(key_hex) + message_digest(msg_json)).hexdigest()


def chain_all(messages_json: List[str], start: str = ROOT) -> str:
    k = start
    for m in messages_json:
        k = chain(k, m)
    return k


class ContextMiss(Exception):
    def __init__(self, code: str, message: str):
        super().__init__(message)
        self.code = code


class ContextStore:
    def __init__(self, budget_bytes: int = 64 << 20):
        self.budget = budget_bytes
        self.items: "collections.OrderedDict[Tuple[str, str, str], List[str]]" = collections.OrderedDict()
        self.bytes = 0
        self.lock = threading.Lock()

    def _size(self, msgs: List[str]) -> int:
        return sum(len(m) for m in msgs) + 64

    def resolve(self, envelope: Dict[str, Any]) -> Tuple[Dict[str, Any], Dict[str, str]]:
        """Envelope -> (chat request body with full messages, response headers)."""
        if envelope.get("version") != 1:
            raise ContextMiss("context_full_required", "unsupported context transport version")
        ns, cid = str(envelope.get("namespace", "")), str(envelope.get("id", ""))
        append = envelope.get("append") or []
        if not all(isinstance(m, str) for m in append):
            raise ContextMiss("context_full_required", "append must be an array of JSON strings")
        base = envelope.get("base")
        with self.lock:
            if base is None:
                msgs: List[str] = []
                key = ROOT
            else:
                have = self.items.get((ns, cid, base.get("key", "")))
                if have is None:
                    raise ContextMiss("context_miss", "the base context is not cached; resend it in full")
                keep = int(base.get("keep", len(have)))
                if not (0 <= keep <= len(have)):
                    raise ContextMiss("context_full_required", "keep is outside the cached context")
                msgs = have[:keep]
                key = chain_all(msgs)
            msgs = msgs + list(append)
            key = chain_all(append, key)
            if envelope.get("key") not in (None, key):
                raise ContextMiss("context_full_required", "context key does not match the messages")
            self._store((ns, cid, key), msgs)
        req = dict(envelope.get("request") or {})
        req["messages"] = [json.loads(m) for m in msgs]
        return req, {"X-Titanic-Context-Ack": "v1", "X-Titanic-Context-Key": key,
                     "X-Titanic-Context-Stored": str(len(msgs))}

    def _store(self, k, msgs: List[str]) -> None:
        if k in self.items:
            self.bytes -= self._size(self.items.pop(k))
        self.items[k] = msgs
        self.bytes += self._size(msgs)
        while self.bytes > self.budget and len(self.items) > 1:
            _, old = self.items.popitem(last=False)
            self.bytes -= self._size(old)
