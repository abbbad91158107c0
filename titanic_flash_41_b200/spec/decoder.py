"""Speculative decoding of up to ``regions`` conversations in one batched step.

One step (reference: GreedySession::batched_step, src/dspark_generation.rs:2333; finish_phase
:2039): the draft head proposes ``depth`` tokens per conversation (sequential single-row passes,
sampled at the request's temperature / top-p), the target verifies the anchor plus the
proposals in one launch of ``S * (depth + 1)`` rows, block verification accepts a prefix and
emits one more token, and the committed length advances by ``accepted + 1``.  Rejected rows need
no rollback: all state is position-addressed.

The whole device side of a step is captured in ONE CUDA graph per (conversations, depth)
profile; per step the host uploads a small metadata block (positions, regions, uniforms, each
conversation's temperature and top-p), replays the graph and reads back (accepted, next token)
per conversation.  Conversations with different sampling settings share the launch and the graph.

Sampling and verification run on each rank's own vocabulary columns (``csrc/sample_chunks.cu``:
one launch per draft proposal and one for the verification; the ranks exchange only maxima, mass
histograms, chunk masses and the chosen token), so no logits are gathered and a step contains no
NCCL call.  Vocabularies that do not chunk fall back to gathered rows and the full-row kernels of
``csrc/sampling.cu``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.engine import Engine, StepPlan
from ..ops import native
from . import rng


@dataclass
class DecodeSlot:
    region: int
    length: int                 # committed tokens (all in the KV state)
    anchor: int                 # sampled but not yet in the KV state
    seed: int = 0
    temperature: float = 0.6
    top_p: float = 0.95
    emitted: List[int] = field(default_factory=list)
    # models with Engram layers: the committed tokens right before ``anchor`` (oldest first; the
    # last ngram-1 are used), from which the device hashes the n-gram ids of the step's rows
    recent: List[int] = field(default_factory=list)
    # spec.history_lookup.HistoryLookup over the conversation's committed text (optional): when the
    # text ends with a phrase seen before, the tokens that followed it then are proposed as point
    # masses instead of the draft head's samples (reference: src/dspark_generation.rs:1908)
    lookup: Optional[object] = None
    # models with a confidence head: the drafter's confidences of the last round and how many of
    # its proposals were verified (causal stopping)
    confidence: List[float] = field(default_factory=list)
    verified: int = 0


def step_meta(regions: Sequence[int], lengths: Sequence[int], anchors: Sequence[int], g: int, ratio: int):
    """Metadata blocks of one verification round, built with array arithmetic (this runs on the
    host every step): the verify block ``StepPlan.build([(region, length, [anchor] + [0] * g)
    ...]).meta_host(ratio)`` and, for proposal j, the block of one row per conversation at
    position length + j (token: the anchor for j = 0, else filled in on the device)."""
    S, R = len(regions), g + 1
    reg = np.asarray(regions, dtype=np.int32)
    ln = np.asarray(lengths, dtype=np.int32)
    an = np.asarray(anchors, dtype=np.int32)
    j = np.arange(R, dtype=np.int32)
    pos = (ln[:, None] + j[None, :]).reshape(-1)
    tok = np.zeros((S, R), dtype=np.int32)
    tok[:, 0] = an
    zeros = np.zeros(S * R, dtype=np.int32)
    mv = np.stack([tok.reshape(-1), pos, np.repeat(reg, R), np.repeat(np.arange(S, dtype=np.int32) * R, R),
                   np.repeat(ln + R - 1, R), (pos + 1) // ratio, zeros]).astype(np.int32)
    mds = []
    z = np.zeros(S, dtype=np.int32)
    rows = np.arange(S, dtype=np.int32)
    for jj in range(g):
        p = ln + jj
        mds.append(np.stack([an if jj == 0 else z, p, reg, rows, p, (p + 1) // ratio, z]).astype(np.int32))
    return mv, mds


class SpecDecoder:
    """``temperature`` / ``top_p`` are kept for callers that name them; the settings that count are
    the ones each ``DecodeSlot`` carries (uploaded per step)."""

    def __init__(self, engine: Engine, n_slots: int, depth: Optional[int] = None,
                 temperature: float = 0.6, top_p: float = 0.95, use_graph: bool = True):
        self.e = engine
        cfg = engine.cfg
        self.S = n_slots
        self.g = cfg.draft.depth if depth is None else depth
        if not engine.draft_layers:
            self.g = 0
        self.temperature, self.top_p = temperature, top_p
        self.use_graph = use_graph and engine.ecfg.use_cuda_graphs
        dev = engine.dev
        S, g, V = self.S, self.g, cfg.vocab
        self.R = g + 1
        self.bv = engine._bufs(S * self.R)
        self.bd = engine._bufs(S) if g > 0 else None
        sb = native.lib().tf_rowstat_bytes()
        f64 = dict(dtype=torch.float64, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        # pinned host staging + device mirrors: [meta_verify(6*S*R) | meta_draft(g*6*S)] ints, uniforms
        self.n_meta_v = StepPlan.META_ROWS * S * self.R
        self.n_meta_d = StepPlan.META_ROWS * S
        self.n_rec = (cfg.engram.ngram - 1) if engine.engram else 0
        self.n_eg = S * self.R * self.n_rec          # per verify row: the tokens before its block
        if engine.engram:
            self.bv["eg_hash"] = True
        self.n_look = S * (1 + max(g, 1))            # copy proposals: [flag per conversation | tokens S x g]
        self.h_int = torch.zeros(self.n_meta_v + g * self.n_meta_d + self.n_eg + self.n_look,
                                 dtype=torch.int32).pin_memory()
        self.lookup_hits = 0
        self.d_int = torch.zeros_like(self.h_int, device=dev)
        self.h_u = torch.zeros(S, g + 2, dtype=torch.float64).pin_memory()     # accept[g], final, spare
        self.d_u = torch.zeros_like(self.h_u, device=dev)
        self.h_ud = torch.zeros(S, max(g, 1), dtype=torch.float64).pin_memory()  # draft draws
        self.d_ud = torch.zeros_like(self.h_ud, device=dev)
        self.h_out = torch.zeros(2 + g, S, dtype=torch.int32).pin_memory()    # accepted, next, proposals
        self.d_out = torch.zeros(2 + g, S, **i32)
        self.hidden = torch.zeros(S, cfg.hidden, dtype=torch.bfloat16, device=dev)   # target hidden at length-1
        self.dhid = torch.zeros(S, cfg.hidden, dtype=torch.bfloat16, device=dev)
        from ..parallel.symm import SampleWorkspace
        self.ws = None
        if SampleWorkspace.usable(V, S * self.R, engine.world, dev) and not engine.draft_extra.get("head_mx"):
            self.ws = SampleWorkspace(V, S * self.R, dev, world=engine.world, rank=engine.rank)
        self.Vl = V // engine.world if self.ws is not None else V
        # per-conversation sampling settings: [temperature | top-p], uploaded with the step metadata
        self.h_f = torch.zeros(2, S, dtype=torch.float32).pin_memory()
        self.d_f = torch.zeros_like(self.h_f, device=dev)
        self.dlogits = torch.zeros(S, max(g, 1), self.Vl, dtype=torch.float32, device=dev)
        self.dstat = torch.zeros(S, max(g, 1), sb, dtype=torch.uint8, device=dev)
        self.tstat = torch.zeros(S, self.R, sb, dtype=torch.uint8, device=dev)
        self.props = torch.zeros(S, max(g, 1), **i32)
        # confidence head (causal stopping): confidences [S, g], running products, proposals to verify
        self.causal = bool(g > 0 and engine.draft_extra.get("confidence") is not None and self.ws is not None)
        if self.causal:
            self.conf = torch.zeros(S, g, dtype=torch.float32, device=dev)
            self.cum = torch.zeros(S, dtype=torch.float32, device=dev)
            self.nver = torch.ones(S, **i32)
            self.ladder = torch.tensor(list(cfg.draft.confidence_ladder) or [0.0], dtype=torch.float32, device=dev)
            self.h_conf = torch.zeros(S, g + 1, dtype=torch.float32).pin_memory()     # confidences | verified count
            self.d_conf = torch.zeros_like(self.h_conf, device=dev)
        self.ptok = torch.zeros(S, **i32)
        self.pacc = torch.zeros(S, **i32)
        self.u1 = torch.zeros(S, 2, **f64)
        lib = native.lib()
        self.Rm = torch.zeros(lib.tf_spec_verify_scratch_doubles(S, g, V), **f64)   # tile masses
        self.wm = torch.zeros(S, self.R, **f64)
        self.R1 = torch.zeros(lib.tf_spec_verify_scratch_doubles(S, 0, V), **f64)
        self.w1 = torch.zeros(S, 1, **f64)
        # zero-initialised scratch of the row-statistics passes (left zero by every call)
        self.rs_scratch = torch.zeros(lib.tf_rowstats_scratch_bytes(S * self.R), dtype=torch.uint8, device=dev)
        self.rows_all = torch.arange(S * self.R, device=dev)
        self.rows_d = torch.arange(S, device=dev)
        self.row_of_anchor = torch.arange(S, device=dev) * self.R
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.nmax_bucket = 0
        self.steps = 0
        # when a list: (start, end) CUDA events around the device work of every step (uploads and the
        # result download excluded), for callers that report device time of exactly the steps they ran
        self.device_events: Optional[list] = None
        # utils.trace.GraphClock (set before the first step): device timestamps in front of every kernel
        # call of the step, captured into the graph; ``clock.report()`` after a step shows the replay
        self.clock = None

    # ---------------------------------------------------------------------------------
    def _fill_host(self, slots: Sequence[DecodeSlot]) -> int:
        S, g, R = self.S, self.g, self.R
        cfg = self.e.cfg
        ratio = cfg.compress_ratio
        hi = self.h_int.numpy()
        mv, mds = step_meta([s.region for s in slots], [s.length for s in slots], [s.anchor for s in slots], g, ratio)
        hi[: self.n_meta_v] = mv.reshape(-1)
        for j in range(g):
            o = self.n_meta_v + j * self.n_meta_d
            hi[o: o + self.n_meta_d] = mds[j].reshape(-1)
        if self.n_eg:
            o = self.n_meta_v + g * self.n_meta_d
            hi[o: o + self.n_eg] = StepPlan.recent_rows(cfg, [(R, s.recent) for s in slots]).reshape(-1)
        hf = self.h_f.numpy()
        hu = self.h_u.numpy()
        o = self.n_meta_v + g * self.n_meta_d + self.n_eg
        look = hi[o: o + self.n_look]
        look[:] = 0
        gs = max(g, 1)
        for i, s in enumerate(slots):
            if g > 0 and s.lookup is not None and self.ws is not None:
                prop = s.lookup.propose(pending=[s.anchor])
                if prop is not None and len(prop.tokens) >= g:
                    look[i] = 1
                    look[S + i * gs: S + i * gs + g] = prop.tokens[:g]
                    self.lookup_hits += 1
        for i, s in enumerate(slots):
            hf[0, i] = max(float(s.temperature), 1e-3)      # temperature 0 (greedy) = a very sharp law
            hf[1, i] = min(max(float(s.top_p), 1e-6), 1.0)
            dr, ac, fin = rng.round_uniforms(s.seed, s.length, g)
            hu[i, :g] = ac
            hu[i, g] = fin
            if g:
                self.h_ud.numpy()[i, :g] = dr
        return int((max(s.length for s in slots) + g + 1) // ratio)

    def _device_step(self, nmax: int) -> None:
        """Everything between the metadata upload and the result download (graph-capturable)."""
        e, S, g, R = self.e, self.S, self.g, self.R
        cfg = e.cfg
        V = cfg.vocab
        st = e.status.t
        mv = self.d_int[: self.n_meta_v].view(StepPlan.META_ROWS, S * R)
        hid = self.hidden
        ws = self.ws
        local = ws is not None
        temp, topp = self.d_f[0], self.d_f[1]
        gs = max(g, 1)
        o = self.n_meta_v + g * self.n_meta_d + self.n_eg
        look = self.d_int[o: o + S]                              # 1: the conversation's proposals were found by lookup
        lprops = self.d_int[o + S: o + self.n_look].view(S, gs)
        for j in range(g):
            o = self.n_meta_v + j * self.n_meta_d
            md = self.d_int[o: o + self.n_meta_d].view(StepPlan.META_ROWS, S)
            self.bd["meta"].copy_(md)
            if j > 0:
                self.bd["meta"][0].copy_(self.props[:, j - 1])
            lg = e.draft_run(S, self.bd, hid, self.rows_d, local_logits=local)
            if self.causal:
                e.draft_confidence(S, self.bd, j, g, self.ladder, self.conf, self.cum, self.nver)
            self.dlogits[:, j].copy_(lg)
            hid = self.dhid
            if cfg.hc_mult > 1:
                # the next pass is conditioned on the mean of the residual copies (as the target's
                # hidden state is: Engine._head)
                hid.copy_(self.bd["x"].view(S, cfg.hc_mult, cfg.hidden).float().mean(1))
            else:
                hid.copy_(self.bd["x"])
            # sample proposal j from the modified draft law
            if local:
                # one launch: statistics of the row (kept for the verification) + the draw, on this
                # rank's columns; writes props[:, j] and dstat[:, j] in place
                ws.sample(lg, None, None, None, self.d_ud[:, j:], gs, temp, topp, S, 0, lg.stride(0),
                          self.dstat[:, j], gs, None, self.props[:, j:], gs, st, sess_point=look, forced=lprops[:, j:])
                continue
            stat = self.dstat[:, j].contiguous()
            native.call("tf_rowstats_per_session", lg, V, V, S, temp, topp, 1, stat, self.rs_scratch, st)
            self.dstat[:, j].copy_(stat)
            self.u1[:, 0].copy_(self.d_ud[:, j])
            self.u1[:, 1].copy_(self.d_ud[:, j])
            native.call("tf_spec_verify", lg, None, stat, None, None, self.u1, S, 0, V, V, 1.0, 1.0, temp, 0,
                        self.R1, self.w1, self.pacc, self.ptok, st)
            self.props[:, j].copy_(self.ptok)
        # target verification of anchor + proposals
        self.bv["meta"].copy_(mv)
        if self.n_eg:
            o = self.n_meta_v + g * self.n_meta_d
            self.bv["eg_recent"].copy_(self.d_int[o: o + self.n_eg].view(S * R, self.n_rec))
        if g > 0:
            tok = self.bv["meta"][0].view(S, R)
            tok[:, 1:].copy_(self.props[:, :g])
        logits = e.run(S * R, self.bv, nmax, R if R <= 32 else 1, self.rows_all, local_logits=local)
        if local:
            ws.sample(logits, self.dlogits if g > 0 else None, self.dstat if g > 0 else None,
                      self.props if g > 0 else None, self.d_u, g + 2, temp, topp, S, g, logits.stride(0),
                      self.tstat, 1, self.d_out[0], self.d_out[1], 1, st, sess_point=look if g > 0 else None,
                      sess_g=self.nver if self.causal else None)
            if self.causal:
                self.d_conf[:, :g].copy_(self.conf)
                self.d_conf[:, g].copy_(self.nver)
        else:
            native.call("tf_rowstats_per_session", logits, V, V, S * R, temp, topp, R, self.tstat, self.rs_scratch, st)
            native.call("tf_spec_verify", logits, self.dlogits if g > 0 else None, self.tstat,
                        self.dstat if g > 0 else None, self.props if g > 0 else None, self.d_u, S, g, V, V,
                        1.0, 1.0, temp, 0, self.Rm, self.wm, self.d_out[0], self.d_out[1], st)
        # hidden state of the last committed row feeds the next round's draft
        rows = self.row_of_anchor + self.d_out[0].long()
        self.hidden.copy_(e.last_hidden[rows])
        if g > 0:
            self.d_out[2:].copy_(self.props[:, :g].t())

    def step(self, slots: Sequence[DecodeSlot]) -> List[List[int]]:
        """Advance every conversation by one verification round; returns the committed tokens."""
        assert len(slots) == self.S
        nmax = self._fill_host(slots)
        bucket = -(-max(nmax, 1) // 4096) * 4096
        self.d_int.copy_(self.h_int, non_blocking=True)
        self.d_u.copy_(self.h_u, non_blocking=True)
        self.d_ud.copy_(self.h_ud, non_blocking=True)
        self.d_f.copy_(self.h_f, non_blocking=True)
        if self.use_graph:
            if self.graph is None or bucket != self.nmax_bucket:
                self.nmax_bucket = bucket
                torch.cuda.synchronize()
                # the step reads `hidden` first and overwrites it last, so the warm-up run must not
                # leave its result there: the replay below is the run that counts
                carried = self.hidden.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._device_step(bucket)          # warm-up outside capture
                torch.cuda.current_stream().wait_stream(s)
                torch.cuda.synchronize()
                self.hidden.copy_(carried)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    if self.clock is not None:
                        with self.clock:                # device timestamps captured with the kernels
                            self._device_step(bucket)
                    else:
                        self._device_step(bucket)
            ev = self._mark()
            self.graph.replay()
        else:
            ev = self._mark()
            if self.clock is not None:
                with self.clock:
                    self._device_step(bucket)
            else:
                self._device_step(bucket)
        if ev is not None:
            ev[1].record()
        self.h_out.copy_(self.d_out, non_blocking=True)
        if self.causal:
            self.h_conf.copy_(self.d_conf, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.steps += 1
        out = []
        acc, nxt = self.h_out[0].tolist(), self.h_out[1].tolist()
        props = self.h_out[2:].t().tolist() if self.g > 0 else None
        for i, s in enumerate(slots):
            toks = [s.anchor] + (props[i][: acc[i]] if props else [])
            if s.lookup is not None:
                s.lookup.commit(s.length, toks)
            s.length += len(toks)
            s.emitted += toks
            if self.n_rec:
                s.recent = (list(s.recent) + toks)[-self.n_rec:]
            s.anchor = nxt[i]
            if self.causal:
                s.confidence = self.h_conf[i, : self.g].tolist()
                s.verified = int(self.h_conf[i, self.g])
            out.append(toks)
        return out

    def _mark(self):
        if self.device_events is None:
            return None
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
        self.device_events.append(ev)
        return ev

    @property
    def h2d_bytes_per_step(self) -> int:
        return self.h_int.numel() * 4 + self.h_u.numel() * 8 + self.h_ud.numel() * 8 + self.h_f.numel() * 4

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.h_out.numel() * 4 + (self.h_conf.numel() * 4 if self.causal else 0)

    def count_launches(self, slots: Sequence[DecodeSlot]) -> int:
        """Kernels of this package launched by one step, counted on an eager run of the step."""
        self._fill_host(slots)
        self.d_int.copy_(self.h_int)
        self.d_u.copy_(self.h_u)
        self.d_ud.copy_(self.h_ud)
        self.d_f.copy_(self.h_f)
        n0 = native.LAUNCHES[0]
        self._device_step(max(self.nmax_bucket, 4096))
        torch.cuda.synchronize()
        return native.LAUNCHES[0] - n0
