"""OpenAI-compatible HTTP front end (aiohttp).

Routes (reference: src/http_server.rs:1334-1341): GET /health, GET /_native/diagnostics,
GET /v1/models, POST /v1/chat/completions, POST /v1/context/chat/completions,
POST /v1/requests/{id}/cancel, POST /_native/shutdown, POST /_native/priority.

Streaming is OpenAI ``chat.completion.chunk`` server-sent events with ``reasoning_content`` /
``content`` / ``tool_calls`` deltas; the first chunk carries ``timings``; ``: native-execution
waiting|running`` comments report admission; a keep-alive comment goes out every 5 s; the stream
ends with ``data: [DONE]``; a client that disconnects cancels its request.  Errors: 401 (bearer
key compared by SHA-256 digest), 400 rejected controls, 409 context_miss, 429 queue_full /
background_queue_full.  The model behind the queue is whatever consumes ``Scheduler`` jobs: the
serving worker, or a test thread that emits token events.
"""
from __future__ import annotations

import asyncio
import hashlib
import hmac
import json
import time
import uuid
from typing import Any, Dict, List, Optional

from aiohttp import web

from ..config import ServerConfig
from ..serve.scheduler import Job, QueueFull, Scheduler
from ..utils.event_log import EventLog
from . import protocol as P
from .context_transport import ContextMiss, ContextStore
from .tokenizer import IncrementalDecoder


def _err(status: int, code: str, message: str, headers: Optional[Dict[str, str]] = None) -> web.Response:
    return web.json_response({"error": {"message": message, "type": "invalid_request_error" if status < 500
                                        else "server_error", "code": code}}, status=status, headers=headers)


class Frontend:
    """Protocol + tokenizer: request body -> token ids; token ids -> deltas."""

    def __init__(self, tokenizer, context: int, allow_sampling: bool = True, vision=None,
                 default_max_tokens: int = P.DEFAULT_MAX_NEW_TOKENS):
        """``vision``: an ``api.media.VisionFrontend`` when the deployment has a vision tower; without
        one a request that carries image parts is refused (it must never be answered as if the image
        had been seen)."""
        self.tok, self.context, self.allow_sampling, self.vision = tokenizer, context, allow_sampling, vision
        self.default_max_tokens = default_max_tokens      # new tokens of a request that names no limit
        # plain-text regions between template markers are tokenised through a bounded, exact cache:
        # long documents repeat from turn to turn (reference: src/prompt_regions.rs)
        from .prompt_regions import RegionCache
        import re
        specials = getattr(tokenizer, "special_ids", None)
        self._special_ids = dict(specials) if specials else {}
        self._split = (re.compile("(" + "|".join(re.escape(s) for s in sorted(self._special_ids, key=len, reverse=True)) + ")")
                       if self._special_ids else None)
        self.regions = RegionCache(tokenizer.encode, lambda t: tokenizer.decode([t]))

    def encode(self, text: str):
        """Token ids of a rendered prompt: template markers are single ids, the plain regions between
        them go through the region cache (a marker is a hard token boundary, so this equals encoding
        the whole text)."""
        if self._split is None:
            return self.tok.encode(text)
        out = []
        for piece in self._split.split(text):
            if not piece:
                continue
            sid = self._special_ids.get(piece)
            if sid is not None:
                out.append(sid)
            else:
                out += self.regions.tokens(piece)
        return out

    def prepare(self, body: Dict[str, Any]):
        """-> (request, prompt tokens, token limit, PromptMedia or None).  Image parts become runs of
        image-placeholder tokens (one per language-model position of the image's plan) and a media
        identity that keys prefix caches (reference: src/http_server.rs:883 chat_input)."""
        from . import media as M
        req = P.normalize_chat_request(body, self.allow_sampling)
        text = P.render_chat(req)
        tokens = self.encode(text)
        uris = P.image_parts(req.messages)
        pm = None
        if uris:
            if self.vision is None:
                raise P.ProtocolError("this deployment has no vision tower: image parts are not supported",
                                      400, "unsupported_media")
            if any(not isinstance(u, str) for u in uris):
                raise P.ProtocolError("image part without a URL", 400, "invalid_media")
            try:
                pm = self.vision.expand(tokens, uris)
            except M.MediaError as e:
                raise P.ProtocolError(str(e), 400, "invalid_media") from e
            tokens = pm.tokens
        limit = P.resolve_max_tokens(req.max_new_tokens, len(tokens), self.context, self.default_max_tokens)
        return req, tokens, limit, pm


class Server:
    def __init__(self, cfg: ServerConfig, frontend: Frontend, scheduler: Scheduler, log: Optional[EventLog] = None,
                 identity: str = "tflash", memory=None, health=None):
        """``memory``: a ``utils.memory.Admission`` for the host pool; every request reserves the bytes
        its input pins (body, token ids, image patches) against it and is refused with 503
        ``insufficient_memory`` when they do not fit above the floor (reference:
        src/http_server.rs:866, src/memory.rs:112, :209).  ``health``: a callable returning the cohort's
        sticky health record (``utils.health.Watchdog.state``); a poisoned cohort turns /health to 503."""
        self.cfg, self.front, self.sched, self.log = cfg, frontend, scheduler, log or EventLog()
        self.memory, self.health_source = memory, health
        self.state = "loading"
        self.identity = identity
        self.jobs: Dict[str, Job] = {}
        self.contexts = ContextStore(cfg.context_cache_bytes)
        self._key_digest = hashlib.sha256(cfg.api_key.encode()).digest() if cfg.api_key else None
        self.shutdown_event = asyncio.Event()
        self.app = web.Application(client_max_size=256 << 20)
        r = self.app.router
        r.add_get("/health", self.health)
        r.add_get("/_native/diagnostics", self.diagnostics)
        r.add_get("/v1/models", self.models)
        r.add_post("/v1/chat/completions", self.chat)
        r.add_post("/v1/context/chat/completions", self.context_chat)
        r.add_post("/v1/requests/{id}/cancel", self.cancel)
        r.add_post("/_native/shutdown", self.shutdown)
        r.add_post("/_native/priority", self.priority)

    def ready(self, identity: Optional[str] = None) -> None:
        self.state = "ready"
        if identity:
            self.identity = identity

    # ---- helpers ------------------------------------------------------------------------------
    def _auth(self, request: web.Request) -> Optional[web.Response]:
        if self._key_digest is None:
            return None
        h = request.headers.get("Authorization", "")
        token = h[7:] if h.startswith("Bearer ") else ""
        if not hmac.compare_digest(hashlib.sha256(token.encode()).digest(), self._key_digest):
            return _err(401, "invalid_api_key", "missing or wrong API key")
        return None

    async def _body(self, request: web.Request) -> Dict[str, Any]:
        try:
            raw = await asyncio.wait_for(request.read(), self.cfg.upload_timeout_s)
        except asyncio.TimeoutError:
            raise P.ProtocolError("request body upload timed out", 408, "upload_timeout")
        try:
            return json.loads(raw)
        except json.JSONDecodeError:
            raise P.ProtocolError("request body is not valid JSON")

    # ---- simple routes ------------------------------------------------------------------------
    async def health(self, request):
        body = {"status": self.state, "identity": self.identity}
        ok = self.state == "ready"
        if self.health_source is not None:
            h = self.health_source()
            body["cohort"] = h
            if h.get("poisoned"):
                body["status"], ok = "poisoned", False
        return web.json_response(body, status=200 if ok else 503)

    async def models(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        return web.json_response({"object": "list", "data": [{"id": self.cfg.model_name, "object": "model",
                                                               "owned_by": "tflash"}]})

    async def diagnostics(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        snap = self.log.snapshot()
        snap["queue"] = {"waiting": self.sched.waiting(), "active": len(self.sched.active)}
        return web.json_response(snap)

    async def cancel(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        job = self.jobs.get(request.match_info["id"])
        if job is None:
            return _err(404, "unknown_request", "no such request")
        job.cancelled.set()
        return web.json_response({"cancelled": True})

    async def shutdown(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        self.state = "stopping"
        self.sched.close()
        self.shutdown_event.set()
        return web.json_response({"status": "stopping"})

    async def priority(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        body = await self._body(request)
        until = self.sched.priority_lease(float(body.get("seconds", 0)))
        return web.json_response({"hold_background_for": max(0.0, until - time.monotonic())})

    # ---- chat ---------------------------------------------------------------------------------
    async def context_chat(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        if request.headers.get("X-Titanic-Context") != "v1":
            return _err(400, "context_version", "X-Titanic-Context: v1 is required")
        try:
            env = await self._body(request)
            body, headers = self.contexts.resolve(env)
        except ContextMiss as e:
            return _err(409, e.code, str(e))
        except P.ProtocolError as e:
            return _err(e.status, e.code, str(e))
        return await self._chat(request, body, headers)

    async def chat(self, request):
        bad = self._auth(request)
        if bad:
            return bad
        try:
            body = await self._body(request)
        except P.ProtocolError as e:
            return _err(e.status, e.code, str(e))
        return await self._chat(request, body, {})

    async def _chat(self, request, body, extra_headers):
        if self.state != "ready":
            return _err(503, "not_ready", f"server is {self.state}")
        try:
            req, tokens, limit, pm = self.front.prepare(body)
        except P.ProtocolError as e:
            return _err(e.status, e.code, str(e))
        # input memory admission: what this request pins on the host until it finishes
        hold = None
        if self.memory is not None:
            from ..utils.memory import CapacityError
            need = (request.content_length or 0) + 8 * len(tokens)
            if pm is not None:
                need += sum(int(p.patches.numel()) * 2 for p in pm.images)
            try:
                hold = self.memory.reserve(need, "request input")
            except CapacityError as e:
                return _err(503, "insufficient_memory", str(e), {"Retry-After": "1"})
        rid = "req-" + uuid.uuid4().hex[:16]
        loop = asyncio.get_running_loop()
        q: "asyncio.Queue" = asyncio.Queue()

        def emit(kind, payload):                       # called from the worker thread
            loop.call_soon_threadsafe(q.put_nowait, (kind, payload))
        background = request.headers.get("X-LocalAI-Mode", "").lower() == "background"
        job = Job(rid, tokens, limit, req.temperature, req.top_p, req.seed if req.seed is not None else
                  int.from_bytes(hashlib.sha256(rid.encode()).digest()[:4], "little"), background, emit=emit)
        if pm is not None:
            job.media, job.images = pm.identity, [pm]
        try:
            self.sched.submit(job)
        except QueueFull as e:
            if hold is not None:
                hold.release()
            return _err(429, e.code, "the request queue is full", {"Retry-After": "1"})
        self.jobs[rid] = job
        headers = {"x-request-id": rid, "x-native-execution-timing": "v1", "cache-control": "no-store",
                   **extra_headers}
        try:
            if req.stream:
                return await self._stream(request, req, job, q, headers, len(tokens))
            return await self._collect(req, job, q, headers, len(tokens))
        finally:
            self.jobs.pop(rid, None)
            if hold is not None:
                hold.release()

    def _chunk(self, rid, delta, finish=None, extra=None):
        c = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": self.cfg.model_name,
             "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
        if extra:
            c.update(extra)
        return c

    async def _stream(self, request, req, job, q, headers, prompt_n):
        resp = web.StreamResponse(status=200, headers={**headers, "content-type": "text/event-stream"})
        await resp.prepare(request)
        dec = IncrementalDecoder(self.front.tok)
        parser = P.StreamParser(req.thinking, bool(req.tools) and req.tool_choice != "none")
        timings, sent_role, n_tok = None, False, 0

        async def send(obj):
            await resp.write(b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n")
        try:
            await resp.write(b": native-execution waiting\n\n")
            finish = None
            while True:
                try:
                    kind, payload = await asyncio.wait_for(q.get(), self.cfg.keepalive_s)
                except asyncio.TimeoutError:
                    await resp.write(b": keep-alive\n\n")
                    continue
                if kind == "ready":
                    timings = payload
                    await resp.write(b": native-execution running\n\n")
                elif kind == "tokens":
                    n_tok += len(payload)
                    for d in parser.feed(dec.push(payload)):
                        extra = None
                        if not sent_role:
                            d = {"role": "assistant", **d}
                            extra = {"timings": timings} if timings else None
                            sent_role = True
                        await send(self._chunk(job.id, d, None, extra))
                elif kind == "error":
                    await send({"error": payload})
                    break
                elif kind == "done":
                    for d in parser.feed(dec.flush(), final=True):
                        await send(self._chunk(job.id, d))
                    finish = "tool_calls" if parser.tool_calls else payload["finish_reason"]
                    fin = self._chunk(job.id, {}, finish)
                    if req.include_usage:
                        fin["usage"] = {"prompt_tokens": prompt_n, "completion_tokens": n_tok,
                                        "total_tokens": prompt_n + n_tok}
                    if not sent_role and timings:
                        fin["timings"] = timings
                    await send(fin)
                    break
            await resp.write(b"data: [DONE]\n\n")
        except (ConnectionResetError, asyncio.CancelledError):
            job.cancelled.set()          # client went away: stop generating for it
            raise
        finally:
            if not resp.prepared or request.transport is None or request.transport.is_closing():
                job.cancelled.set()
        return resp

    async def _collect(self, req, job, q, headers, prompt_n):
        toks: List[int] = []
        timings, finish = None, "stop"
        while True:
            kind, payload = await q.get()
            if kind == "ready":
                timings = payload
            elif kind == "tokens":
                toks += payload
            elif kind == "error":
                return _err(400 if payload.get("code") == "context_length_exceeded" else 500, payload.get("code", "error"),
                            payload.get("message", ""), headers)
            elif kind == "done":
                finish = payload["finish_reason"]
                break
        out = P.parse_completion(self.front.tok.decode(toks), req.thinking, bool(req.tools) and req.tool_choice != "none",
                                 finish, prompt_n, len(toks), self.cfg.model_name)
        out["id"] = job.id
        if timings:
            out["timings"] = timings
        return web.json_response(out, headers=headers)


async def serve(server: Server) -> None:
    runner = web.AppRunner(server.app)
    await runner.setup()
    site = web.TCPSite(runner, server.cfg.host, server.cfg.port)
    await site.start()
    await server.shutdown_event.wait()
    await runner.cleanup()
