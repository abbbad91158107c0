"""HTTP tier against a fake worker: a thread that consumes the queue and emits token events."""
import asyncio
import json
import threading
import time

import pytest
from aiohttp import web
from aiohttp.test_utils import TestClient, TestServer

from titanic_flash_41_b200.api import context_transport as CT
from titanic_flash_41_b200.api.server import Frontend, Server
from titanic_flash_41_b200.api.tokenizer import ByteTokenizer
from titanic_flash_41_b200.config import ServerConfig
from titanic_flash_41_b200.serve.scheduler import Scheduler

TOK = ByteTokenizer(1024)


class FakeWorker(threading.Thread):
    """Admits jobs and answers each with a fixed text, a few tokens per event."""

    def __init__(self, sched, text="plan</think>\n\nHello 😀 world", delay=0.0, hold=None):
        super().__init__(daemon=True)
        self.sched, self.text, self.delay, self.hold = sched, text, delay, hold
        self.stop = False
        self.seen = []

    def run(self):
        while not self.stop:
            if self.hold is not None and not self.hold.is_set():
                time.sleep(0.01)
                continue
            for job in self.sched.admit():
                self.seen.append(job)
                job.emit("ready", {"prompt_n": len(job.tokens), "cache_n": 0, "prompt_ms": 1.0, "scope": "request"})
                ids = TOK.encode(self.text)
                for i in range(0, len(ids), 3):
                    if job.cancelled.is_set():
                        break
                    job.emit("tokens", ids[i:i + 3])
                    time.sleep(self.delay)
                job.emit("done", {"finish_reason": "cancelled" if job.cancelled.is_set() else "stop",
                                  "completion_tokens": len(ids)})
                self.sched.release(job)
            time.sleep(0.005)


async def _client(cfg=None, **fw):
    cfg = cfg or ServerConfig(keepalive_s=0.2)
    sched = Scheduler(cfg.max_admitted, cfg.queue_limit, cfg.background_queue_limit)
    srv = Server(cfg, Frontend(TOK, 4096), sched)
    srv.ready("test")
    worker = FakeWorker(sched, **fw)
    worker.start()
    client = TestClient(TestServer(srv.app))
    await client.start_server()
    return client, srv, worker


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


BODY = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 64}


def test_non_streaming_completion_and_headers():
    async def go():
        c, srv, w = await _client()
        r = await c.post("/v1/chat/completions", json=BODY)
        assert r.status == 200 and r.headers["x-native-execution-timing"] == "v1" and "x-request-id" in r.headers
        assert r.headers["cache-control"] == "no-store"
        j = await r.json()
        m = j["choices"][0]["message"]
        assert m["content"] == "Hello 😀 world" and m["reasoning_content"] == "plan"
        assert j["timings"]["prompt_n"] > 0 and j["usage"]["completion_tokens"] > 0
        r = await c.get("/health")
        assert (await r.json())["status"] == "ready"
        r = await c.get("/v1/models")
        assert (await r.json())["data"][0]["id"] == srv.cfg.model_name
        w.stop = True
        await c.close()
    _run(go())


def test_sse_stream_framing():
    async def go():
        c, srv, w = await _client()
        r = await c.post("/v1/chat/completions", json={**BODY, "stream": True, "stream_options": {"include_usage": True}})
        raw = (await r.read()).decode()
        assert r.headers["content-type"].startswith("text/event-stream")
        assert ": native-execution waiting" in raw and ": native-execution running" in raw
        assert raw.rstrip().endswith("data: [DONE]")
        chunks = [json.loads(l[6:]) for l in raw.split("\n") if l.startswith("data: {")]
        assert "timings" in chunks[0] and chunks[0]["choices"][0]["delta"]["role"] == "assistant"
        text = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks)
        think = "".join(ch["choices"][0]["delta"].get("reasoning_content", "") for ch in chunks)
        assert text == "Hello 😀 world" and think == "plan"
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["usage"]["completion_tokens"] > 0
        w.stop = True
        await c.close()
    _run(go())


def test_rejections_auth_and_queue_full():
    async def go():
        cfg = ServerConfig(api_key="secret", max_admitted=1, queue_limit=1, keepalive_s=0.2)
        hold = threading.Event()
        c, srv, w = await _client(cfg, hold=hold)
        r = await c.post("/v1/chat/completions", json=BODY)
        assert r.status == 401
        H = {"Authorization": "Bearer secret"}
        r = await c.post("/v1/chat/completions", json={**BODY, "foo": 1}, headers=H)
        assert r.status == 400 and "unsupported native chat field" in (await r.json())["error"]["message"]
        r = await c.post("/v1/chat/completions", json={**BODY, "max_tokens": 5, "messages": [{"role": "user", "content": "x" * 5000}]}, headers=H)
        assert r.status == 400 and (await r.json())["error"]["code"] == "context_length_exceeded"
        # the worker is held: the first request waits in the queue, the second overflows it
        t1 = asyncio.ensure_future(c.post("/v1/chat/completions", json=BODY, headers=H))
        await asyncio.sleep(0.1)
        r2 = await c.post("/v1/chat/completions", json=BODY, headers=H)
        assert r2.status == 429 and (await r2.json())["error"]["code"] == "queue_full"
        tb = asyncio.ensure_future(c.post("/v1/chat/completions", json=BODY, headers={**H, "X-LocalAI-Mode": "background"}))
        await asyncio.sleep(0.05)
        hold.set()
        assert (await t1).status == 200 and (await tb).status == 200
        w.stop = True
        await c.close()
    _run(go())


def test_cancel_route_and_context_transport():
    async def go():
        c, srv, w = await _client(delay=0.01, text="a" * 300)
        t = asyncio.ensure_future(c.post("/v1/chat/completions", json={**BODY, "stream": True}))
        await asyncio.sleep(0.15)
        rid = next(iter(srv.jobs))
        r = await c.post(f"/v1/requests/{rid}/cancel")
        assert (await r.json())["cancelled"] is True
        raw = (await (await t).read()).decode()
        assert '"finish_reason": "cancelled"' in raw or "cancelled" in raw
        # context transport: full, then incremental, then a miss
        m1, m2 = json.dumps({"role": "user", "content": "one"}), json.dumps({"role": "user", "content": "two"})
        H = {"X-Titanic-Context": "v1"}
        env = {"version": 1, "namespace": "n", "id": "c", "base": None, "append": [m1], "request": {"max_tokens": 8}}
        r = await c.post("/v1/context/chat/completions", json=env, headers=H)
        assert r.status == 200 and r.headers["X-Titanic-Context-Stored"] == "1"
        k1 = r.headers["X-Titanic-Context-Key"]
        assert k1 == CT.chain(CT.ROOT, m1)
        env2 = {"version": 1, "namespace": "n", "id": "c", "base": {"key": k1, "keep": 1}, "append": [m2], "request": {"max_tokens": 8}}
        r = await c.post("/v1/context/chat/completions", json=env2, headers=H)
        assert r.status == 200 and r.headers["X-Titanic-Context-Key"] == CT.chain(k1, m2)
        env3 = {**env2, "base": {"key": "00" * 32, "keep": 1}}
        r = await c.post("/v1/context/chat/completions", json=env3, headers=H)
        assert r.status == 409 and (await r.json())["error"]["code"] == "context_miss"
        w.stop = True
        await c.close()
    _run(go())
