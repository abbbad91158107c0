"""The GPU-owner loop of one rank.

Rank 0 turns queued jobs into commands (Begin / Step / Finish / Idle / Shutdown); every rank
executes the same command stream deterministically and the ranks compare a digest of the
committed tokens after every step (reference: src/resident_worker.rs:342 Command codec, :4049
execute, :6115 run_http loop, :2559 agree_progress).

Begin   restore the best cached image whose prefix the prompt starts with, prefill the rest in
        chunks (saving prompt checkpoints on the way; other conversations take a batched decode
        step when a prefill slice runs long), sample the first token.  What happens after each
        chunk -- continue, interleave a decode step, or stop because the request was cancelled --
        is decided by rank 0 alone (its clock, its view of the job) and broadcast as a one-byte
        directive; the other ranks never consult their own clock or job table (reference:
        should_cancel -> PrefillDirective through the control channel, src/resident_worker.rs:4009)
Step    one batched speculative verification round for every decoding conversation
Finish  save the completed turn into the session cache and free the region
Pause   park a decoding conversation as a request checkpoint (state image + sampler position) so
        that a waiting request can take its region: with more conversations than regions they
        take turns of ``turn_tokens`` tokens (reference: 64-token turns through parked images,
        src/batched_serving.rs:1-17, src/request_checkpoint.rs)
Resume  attach a parked conversation to a free region; it continues token-exactly
Idle    one unit of background cache work (tier moves)
"""
from __future__ import annotations

import hashlib
import json
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

from ..spec.decoder import DecodeSlot
from ..utils.event_log import EventLog
from . import policy
from .scheduler import Job, Scheduler
from .session_cache import SessionCache


@dataclass
class Active:
    job: Job
    slot: DecodeSlot
    prompt: List[int]
    limit: int
    started: float
    first_token_at: float = 0.0
    steps: int = 0
    finished: Optional[str] = None
    turn: int = 0                      # tokens delivered since the conversation was last attached to a region


# per-chunk prefill directives (rank 0 decides, every rank follows)
D_CONTINUE, D_STEP, D_CANCEL = 0, 1, 2


class Worker:
    def __init__(self, backend, scheduler: Optional[Scheduler], cache: Optional[SessionCache] = None,
                 eos_id: int = 1, log: Optional[EventLog] = None, control=None, rank: int = 0,
                 prefill_slice_s: float = 0.5, checkpoint_min: int = policy.SHORT_TOKENS,
                 checkpoint_align: int = 8192, span_encoder=None, health=None, turn_tokens: int = 64,
                 history_lookup: bool = True, log_confidence: bool = False):
        """``span_encoder`` (rank 0): ``api.media.SpanEncoder`` over the vision tower; needed to serve
        requests that carry images.  ``log_confidence``: one ``step_confidence`` event per conversation
        and round with the drafter's confidences, the proposals verified and the tokens emitted (no
        token ids; reference: src/dspark_generation.rs log_step_confidence)."""
        self.log_confidence = log_confidence
        self.b, self.sched, self.cache = backend, scheduler, cache or SessionCache()
        self.eos, self.log, self.control, self.rank = eos_id, log or EventLog(), control, rank
        self.slice_s, self.ck_min, self.ck_align = prefill_slice_s, checkpoint_min, checkpoint_align
        self.active: Dict[int, Active] = {}
        self.jobs: Dict[str, Job] = {}
        self.running = True
        self.requests = 0
        self.span_encoder = span_encoder
        self.health = health                 # utils.health.Health: sticky record of what stopped this rank
        self.turn_tokens = turn_tokens       # 0: never park a decoding conversation for a waiting one
        self.history_lookup = history_lookup
        self.parked: List[Any] = []          # RequestCheckpoints waiting for a region, oldest first (every rank)
        self.parked_jobs: Dict[str, Job] = {}
        self.clock = time.monotonic          # rank 0's time source for prefill slices (tests skew it)
        self.directives: List[int] = []      # per-chunk directives this rank followed (diagnostics)

    # ---------------------------------------------------------------- command codec
    @staticmethod
    def encode(cmd: Dict[str, Any]) -> bytes:
        return json.dumps(cmd, separators=(",", ":")).encode()

    @staticmethod
    def decode(raw: bytes) -> Dict[str, Any]:
        return json.loads(raw)

    def _send_command(self, cmd: Dict[str, Any]) -> None:
        """Broadcast a command.  The prompt of a Begin does not travel as JSON text: the header frame
        names its length and the token ids follow as little-endian int32 in bounded frames, so a
        million-token prompt costs 4 MB on the wire and never exceeds the channel's frame limit."""
        import numpy as np
        toks = cmd.get("tokens")
        if toks is None:
            self.control.command(self.encode(cmd))
            return
        head = {k: v for k, v in cmd.items() if k not in ("tokens", "tokens_arr")}
        head["n_tokens"] = len(toks)
        self.control.command(self.encode(head))
        arr = cmd.get("tokens_arr")
        blob = (arr if arr is not None else np.asarray(toks)).astype("<i4").tobytes()
        for i in range(0, len(blob), self.FRAME):
            self.control.command(blob[i:i + self.FRAME])

    def _pool(self):
        """One helper thread for host work that can run beside a prefill."""
        if getattr(self, "_executor", None) is None:
            from concurrent.futures import ThreadPoolExecutor
            self._executor = ThreadPoolExecutor(max_workers=1, thread_name_prefix="tflash-host")
        return self._executor

    def _recv_command(self) -> Dict[str, Any]:
        import numpy as np
        cmd = self.decode(self.control.command(None))
        n = cmd.pop("n_tokens", None)
        if n is not None:
            blob = bytearray()
            while len(blob) < 4 * n:
                blob += self.control.command(None)
            arr = np.frombuffer(bytes(blob[:4 * n]), dtype="<i4").astype(np.int64)
            cmd["tokens"], cmd["tokens_arr"] = arr.tolist(), arr        # the array is what Begin compares and hashes
        return cmd

    def _digest(self) -> bytes:
        h = hashlib.sha256()
        for r in sorted(self.active):
            a = self.active[r]
            h.update(f"{r}:{a.slot.length}:{a.slot.anchor}:{len(a.slot.emitted)}|".encode())
        return h.digest()

    # ---------------------------------------------------------------- rank-0 driver
    def next_command(self) -> Dict[str, Any]:
        """Decide the next command from the queue and the active set (rank 0 only)."""
        for a in list(self.active.values()):
            if a.finished or a.job.cancelled.is_set():
                return {"op": "finish", "region": a.job.region, "reason": a.finished or "cancelled"}
        if self.sched is not None:
            free = self.sched.free_regions()
            waiting = self.sched.waiting()
            if self.parked and free and (not waiting or self.parked_jobs[self.parked[0].id].submitted
                                         <= self.sched.oldest_submitted()):
                # a parked conversation goes first when it has waited longer than the queue's head
                ck = self.parked[0]
                job = self.parked_jobs[ck.id]
                if job.cancelled.is_set():
                    return {"op": "drop_parked", "id": ck.id}
                self.sched.occupy(job, free[0])
                return {"op": "resume", "id": ck.id, "region": free[0]}
            if waiting and not free and self.turn_tokens > 0:
                # every region decodes and a request waits: the conversation that has had the longest turn yields
                over = [a for a in self.active.values() if not a.finished and a.turn >= self.turn_tokens]
                if over:
                    a = max(over, key=lambda x: (x.turn, -x.job.region))
                    return {"op": "pause", "region": a.job.region}
        new = self.sched.admit() if self.sched else []
        if new:
            j = new[0]
            for extra in new[1:]:            # one Begin per command; the rest stay admitted for the next rounds
                self._pending.append(extra)
            return self._begin_cmd(j)
        if getattr(self, "_pending", None):
            return self._begin_cmd(self._pending.pop(0))
        if self.active:
            return {"op": "step"}
        if self.sched is not None and self.sched.closed:
            return {"op": "shutdown"}
        return {"op": "idle"}

    _pending: List[Job] = []

    def _begin_cmd(self, j: Job) -> Dict[str, Any]:
        import numpy as np
        self.jobs[j.id] = j
        # one conversion of the prompt for the wire, the cache digests, the images and the history index
        return {"op": "begin", "id": j.id, "region": j.region, "tokens": j.tokens,
                "tokens_arr": np.asarray(j.tokens, dtype=np.int64), "limit": j.max_new_tokens,
                "temperature": j.temperature, "top_p": j.top_p, "seed": j.seed, "media": j.media,
                "images": len(j.images)}

    def run_once(self, idle_wait: float = 0.05) -> str:
        """One command: chosen by rank 0, broadcast, executed everywhere, agreed."""
        if self.rank == 0:
            cmd = self.next_command()
            if cmd["op"] == "idle" and self.sched is not None and not self.active:
                self.sched.wait_for_work(idle_wait)
            if self.control is not None:
                self._send_command(cmd)
        else:
            cmd = self._recv_command()
        self.execute(cmd)
        if self.control is not None and cmd["op"] in ("begin", "step", "finish", "pause", "resume", "relocate"):
            self.control.agree(self._digest())
        return cmd["op"]

    def run_forever(self) -> None:
        """Command loop.  Any error (a poisoned control channel, a failed collective, a kernel status
        word raised by the backend) is fatal for the rank: it is recorded in the sticky health state,
        every request in flight gets a terminal error event, and the loop ends; the launcher's
        supervisor then stops the rest of the cohort."""
        self._pending = []
        while self.running:
            try:
                self.run_once()
                if self.health is not None:
                    self.health.beat()
                    if not self.health.ok:
                        raise RuntimeError("rank poisoned: " + str(self.health.state().get("why")))
            except Exception as e:  # noqa: BLE001
                if self.health is not None:
                    self.health.report("worker", repr(e))
                self.log.log("worker_stopped", incident=True, error=repr(e))
                self.fail_all({"code": "cohort_failed", "message": "the serving cohort stopped: " + str(e)})
                self.running = False
                if self.health is None:
                    raise

    def fail_all(self, payload: Dict[str, Any]) -> None:
        """Terminal error event for every admitted or queued request (rank 0)."""
        for a in list(self.active.values()):
            self._emit(a.job, "error", payload)
            if self.sched is not None:
                self.sched.release(a.job)
        self.active.clear()
        if self.sched is not None and self.rank == 0:
            self.sched.close()
            for q in (self.sched.fg, self.sched.bg):
                while q:
                    try:
                        q.popleft().emit("error", payload)
                    except Exception:  # noqa: BLE001
                        pass

    # ---------------------------------------------------------------- execution (every rank)
    def execute(self, cmd: Dict[str, Any]) -> None:
        op = cmd["op"]
        if op == "begin":
            self._begin(cmd)
        elif op == "step":
            self._step()
        elif op == "finish":
            self._finish(cmd["region"], cmd["reason"])
        elif op == "pause":
            self._pause(cmd["region"])
        elif op == "resume":
            self._resume(cmd["id"], cmd["region"])
        elif op == "relocate":
            self._relocate(cmd["region"], cmd["to"])
        elif op == "drop_parked":
            self.parked = [c for c in self.parked if c.id != cmd["id"]]
            job = self.parked_jobs.pop(cmd["id"], None)
            self._emit(job, "done", {"finish_reason": "cancelled", "completion_tokens": len(job.generated) if job else 0,
                                     "prompt_tokens": 0, "steps": 0, "decode_tok_s": 0.0})
        elif op == "idle":
            did = self.cache.idle_step()
            if did:
                self.log.log("cache_tier", move=did)
        elif op == "shutdown":
            self.running = False

    def _chunk_directive(self, job: Optional[Job], last_slice: float) -> int:
        """What to do after a prefill chunk.  Rank 0 decides from its own clock and job state and
        broadcasts the decision; every other rank receives it, so all ranks leave the prefill, or
        interleave a decode step, at the same chunk."""
        if self.rank == 0:
            if job is not None and job.cancelled.is_set():
                d = D_CANCEL
            elif self.active and self.clock() - last_slice > self.slice_s:
                d = D_STEP
            else:
                d = D_CONTINUE
            if self.control is not None and self.control.world > 1:
                self.control.command(bytes([d]))
        else:
            raw = self.control.command(None)
            if len(raw) != 1 or raw[0] not in (D_CONTINUE, D_STEP, D_CANCEL):
                raise RuntimeError("malformed prefill directive")
            d = raw[0]
        self.directives.append(d)
        return d

    # ---------------------------------------------------------------- image spans
    FRAME = 512 << 10

    def _image_spans(self, job: Optional[Job]):
        """(prompt offsets [m], feature rows [m, hidden]) of the request's images on every rank.
        Rank 0 runs the vision tower (feature cache in front of it) and broadcasts the rows through
        the control channel in bounded frames; the other ranks receive them (reference: patches or
        spans broadcast to all ranks, src/worker_media.rs:301-470).  None on failure."""
        import numpy as np
        import torch
        multi = self.control is not None and self.control.world > 1
        if self.rank == 0:
            offs = rows = None
            try:
                if self.span_encoder is None or job is None or not job.images:
                    raise ValueError("no vision tower on this deployment")
                got = [self.span_encoder.spans(pm) for pm in job.images]
                offs = torch.cat([g[0] for g in got]).to(torch.int64).cpu()
                rows = torch.cat([g[1] for g in got]).to(torch.bfloat16).cpu().contiguous()
            except Exception as e:  # noqa: BLE001  (a bad image fails its request, not the worker)
                self.log.log("image_failed", incident=True, error=str(e))
            head = {"m": 0, "d": 0} if rows is None else {"m": int(rows.shape[0]), "d": int(rows.shape[1])}
            if multi:
                self.control.command(self.encode(head))
                if rows is not None:
                    blob = offs.numpy().tobytes() + rows.view(torch.int16).numpy().tobytes()
                    for i in range(0, len(blob), self.FRAME):
                        self.control.command(blob[i:i + self.FRAME])
            return None if rows is None else (offs, rows)
        head = self.decode(self.control.command(None))
        m, d = int(head["m"]), int(head["d"])
        if m == 0:
            return None
        total = m * 8 + m * d * 2
        blob = bytearray()
        while len(blob) < total:
            blob += self.control.command(None)
        offs = torch.from_numpy(np.frombuffer(bytes(blob[:m * 8]), dtype=np.int64).copy())
        rows = torch.from_numpy(np.frombuffer(bytes(blob[m * 8:total]), dtype=np.int16).copy()).view(torch.bfloat16).view(m, d)
        return offs, rows

    def _pause(self, region: int) -> None:
        from . import request_checkpoint as RC
        a = self.active.get(region)
        if a is None:
            return
        job = a.job
        lookup = a.slot.lookup
        ck = RC.pause(self, region)
        ck.lookup, ck.steps, ck.started, ck.first_token_at = lookup, a.steps, a.started, a.first_token_at
        self.parked.append(ck)
        self.parked_jobs[ck.id] = job
        if self.sched is not None:
            self.sched.release(job)
        self.log.log("pause", id=ck.id, region=region, committed=len(ck.committed), bytes=ck.charge)

    def _relocate(self, region: int, to: int) -> None:
        """Move a decoding conversation to another (free) region between steps: its state image is
        captured and restored there, sampling continues at the same positions, so the tokens are the
        ones it would have produced in place (reference: src/batched_serving.rs:243 detach_active /
        :604 attach_peer; the reference relocates conversations out of the region its prefills use)."""
        a = self.active.get(region)
        if a is None or to == region:
            return
        if to in self.active or not (0 <= to < self.b.regions):
            raise RuntimeError(f"relocation target {to} is not a free region")
        rid = a.job.id
        self._pause(region)
        if self.sched is not None:
            self.sched.occupy(self.parked_jobs[rid], to)
        self._resume(rid, to)
        self.log.log("relocate", id=rid, source=region, target=to)

    def _resume(self, rid: str, region: int) -> None:
        from . import request_checkpoint as RC
        ck = next((c for c in self.parked if c.id == rid), None)
        if ck is None:
            raise RuntimeError(f"resume of an unknown parked request {rid}")
        self.parked.remove(ck)
        job = self.parked_jobs.pop(rid)
        RC.resume(self, ck, region, job)
        a = self.active[region]
        a.slot.lookup = getattr(ck, "lookup", None)
        a.steps, a.started, a.first_token_at = getattr(ck, "steps", 0), getattr(ck, "started", a.started), \
            getattr(ck, "first_token_at", a.first_token_at)
        self.log.log("resume", id=rid, region=region, committed=len(ck.committed))

    def _emit(self, job: Optional[Job], kind: str, payload: Any) -> None:
        if job is not None and self.rank == 0:
            job.emit(kind, payload)

    def _begin(self, cmd: Dict[str, Any]) -> None:
        t0 = time.monotonic()
        from ..utils import memory as _mem
        stall0 = _mem.pressure_snapshot()          # host stall counters around the prefill (memory / io / cpu pressure)
        import numpy as np
        region = cmd["region"]
        prompt = cmd["tokens"] if isinstance(cmd["tokens"], list) else list(cmd["tokens"])
        # one integer array of the prompt for everything that compares, hashes or stores it (a
        # million-token list is converted once, not once per cache entry)
        parr = cmd.get("tokens_arr")
        if parr is None:
            parr = np.asarray(prompt, dtype=np.int64)
        job = self.jobs.get(cmd["id"])
        self.requests += 1
        if len(prompt) + 1 >= self.b.max_context:
            self._emit(job, "error", {"code": "context_length_exceeded", "message": "prompt does not fit"})
            if self.sched and job:
                self.sched.release(job)
            return
        embeds = None
        if cmd.get("images"):
            embeds = self._image_spans(job)
            if embeds is None:
                self._emit(job, "error", {"code": "unsupported_media", "message": "the images of this request "
                                          "could not be encoded"})
                if self.sched and job:
                    self.sched.release(job)
                return
        # ---- prefix reuse
        start, hit = 0, self.cache.best_match(parr, cmd.get("media", ""))
        if hit is not None and self.cache.ensure_loaded(hit, self.b.device):
            self.b.restore(region, hit.image)
            start = hit.image.length
            self.cache.touch(hit, start)
        else:
            self.cache.stats["misses"] += 1
            self.b.reset(region)
        if start == len(prompt):
            start -= 1                       # the last prompt token is re-run to produce its logits
        # ---- checkpoint plan for the part that is prefilled now
        cks = policy.checkpoint_positions(len(prompt), start, self.ck_min, self.ck_align)
        shared = policy.shared_prefix_checkpoint(self.cache.longest_shared(parr), start,
                                                 cks[0] if cks else len(prompt), len(prompt), 128)
        if shared is not None:
            cks = sorted(set(cks + [shared]))
        logits, pos, reached = None, start, start
        lookup_job = None
        if self.history_lookup:
            # indexing the prompt for copy proposals is host work that needs no result of the prefill:
            # it runs beside it (array arithmetic releases the interpreter lock) and is collected below
            from ..spec.history_lookup import HistoryLookup
            lookup_job = self._pool().submit(HistoryLookup, parr, depth=8)
        last_slice = self.clock()
        for stop in cks + [len(prompt)]:
            if stop <= pos:
                continue

            def on_chunk(done, _base=pos):
                nonlocal last_slice, reached
                reached = _base + done                 # the state of the region covers prompt[:reached]
                # a long prefill lets the decoding conversations take one batched step per slice
                d = self._chunk_directive(job, last_slice)
                if d == D_STEP:
                    self._step()
                    last_slice = self.clock()
                return d != D_CANCEL
            kw = {}
            if embeds is not None:
                kw["embeds"] = (embeds[0] - pos, embeds[1])       # offsets relative to this part of the prompt
            if getattr(self.b, "wants_prev", False):
                # n-gram memory layers hash across the seam between reused and new tokens
                kw["prev"] = prompt[max(0, pos - 8):pos]
            logits = self.b.prefill(region, prompt[pos:stop], pos, on_chunk, **kw)
            if logits is None:
                # an interrupted prefill keeps what it has computed: the same prompt sent again resumes
                # from the last whole chunk instead of position 0 (reference: src/resident_worker.rs
                # encoder checkpoints of an unfinished Begin)
                if reached - start >= self.ck_min and reached < len(prompt):
                    try:
                        self.cache.insert(self.b.snapshot(region, parr[:reached], "checkpoint", cmd.get("media", "")))
                        self.log.log("prefill_interrupted", id=cmd["id"], saved=reached, of=len(prompt))
                    except Exception as e:  # noqa: BLE001  (a refused save never fails the cancellation)
                        self.log.log("save_failed", incident=True, error=str(e))
                self._emit(job, "error", {"code": "cancelled", "message": "cancelled during prefill"})
                if self.sched and job:
                    self.sched.release(job)
                return
            pos = stop
            if stop != len(prompt):
                self.cache.insert(self.b.snapshot(region, parr[:stop], "checkpoint", cmd.get("media", "")))
        first = self.b.sample(logits, cmd["temperature"], cmd["top_p"], cmd["seed"], len(prompt))
        slot = DecodeSlot(region=region, length=len(prompt), anchor=first, seed=cmd["seed"],
                          temperature=cmd["temperature"], top_p=cmd["top_p"], recent=list(prompt[-8:]))
        if lookup_job is not None:
            slot.lookup = lookup_job.result()
        a = Active(job or Job(cmd["id"], prompt, cmd["limit"]), slot, prompt, cmd["limit"], t0, time.monotonic())
        a.prompt_arr = parr
        a.job.region = region
        self.active[region] = a
        ms = (time.monotonic() - t0) * 1e3
        new = len(prompt) - start
        self._emit(job, "ready", {"prompt_n": new, "cache_n": start, "prompt_ms": round(ms, 3),
                                  "prompt_per_second": round(new / max(ms / 1e3, 1e-9), 1), "scope": "request"})
        stall = {k: v for k, v in _mem.pressure_delta(stall0, _mem.pressure_snapshot()).items() if v}
        self.log.log("begin", id=cmd["id"], region=region, prompt=len(prompt), reused=start, ms=round(ms, 2),
                     host_stall=stall)
        self._deliver(a, [first], pending=True)

    def _deliver(self, a: Active, toks: Sequence[int], pending: bool = False) -> None:
        """Emit committed tokens; the anchor counts as generated as soon as it is sampled."""
        out = []
        for t in toks:
            if a.finished:
                break
            if t == self.eos:
                a.finished = "stop"
                break
            a.job.generated.append(t)
            a.turn += 1
            out.append(t)
            if len(a.job.generated) >= a.limit:
                a.finished = "length"
        if out:
            self._emit(a.job, "tokens", out)

    def _step(self) -> None:
        acts = [a for a in self.active.values() if not a.finished]
        if not acts:
            return
        acts.sort(key=lambda a: a.job.region)
        for a in acts:
            if a.slot.length + 8 >= self.b.max_context:
                a.finished = "length"
        acts = [a for a in acts if not a.finished]
        if not acts:
            return
        before = [a.slot.anchor for a in acts]
        committed = self.b.decode_step([a.slot for a in acts])
        for a, toks, old_anchor in zip(acts, committed, before):
            a.steps += 1
            # toks = [old anchor] + accepted proposals are now in the KV state; the anchor was already
            # delivered when it was sampled, so deliver the accepted proposals and the new anchor
            if self.log_confidence and getattr(a.slot, "confidence", None):
                self.log.log("step_confidence", id=a.job.id, confidence=[round(c, 4) for c in a.slot.confidence],
                             verified=a.slot.verified or len(a.slot.confidence), emitted=len(toks))
            self._deliver(a, list(toks[1:]) + [a.slot.anchor])

    def _finish(self, region: int, reason: str) -> None:
        a = self.active.pop(region, None)
        if a is None:
            return
        import numpy as np
        parr = getattr(a, "prompt_arr", None)
        if parr is None:
            parr = np.asarray(a.prompt, dtype=np.int64)
        committed = np.concatenate([parr, np.asarray(a.slot.emitted, dtype=np.int64)])
        try:
            self.cache.insert(self.b.snapshot(region, committed[: a.slot.length], "complete", a.job.media),
                              completed=True)
        except Exception as e:  # noqa: BLE001  (a refused save never fails the request)
            self.log.log("save_failed", incident=True, error=str(e))
        dt = time.monotonic() - a.first_token_at
        self._emit(a.job, "done", {"finish_reason": reason, "completion_tokens": len(a.job.generated),
                                   "prompt_tokens": len(a.prompt), "steps": a.steps,
                                   "decode_tok_s": round(max(len(a.job.generated) - 1, 0) / max(dt, 1e-9), 2)})
        self.log.log("finish", id=a.job.id, reason=reason, tokens=len(a.job.generated), steps=a.steps)
        if self.sched is not None:
            self.sched.release(a.job)
        self.jobs.pop(a.job.id, None)
