"""Model backends behind the serving worker: the PyTorch oracle (CPU, tiny geometries; used by
the CPU test tier and the gloo plumbing runs) and the CUDA engine.

Both expose the same operations on *regions* (one admitted conversation each): prefill a token
range, run one batched speculative decode step, capture / restore a state image, reset.
Reference counterpart: the Target / GreedySession surface used by the resident worker
(src/target.rs:861, src/dspark_generation.rs:1816).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..config import ModelConfig
from ..models import oracle
from ..spec import rng, verify
from ..spec.decoder import DecodeSlot
from . import state_image as SI


class OracleBackend:
    name = "oracle"

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], regions: int = 4,
                 max_context: int = 4096, comm=None, moe_parallel: str = "ep", chunk: int = 256):
        self.cfg, self.regions, self.max_context, self.chunk = cfg, regions, max_context, chunk
        self.model = oracle.OracleModel(cfg, weights, comm, moe_parallel)
        self.sessions = [self.model.new_session(max_context) for _ in range(regions)]
        self.hidden: List[Optional[torch.Tensor]] = [None] * regions
        self.depth = cfg.draft.depth if (cfg.draft and "mtp.0.main_proj.weight" in weights) else 0
        self.device = "cpu"

    def reset(self, region: int) -> None:
        self.sessions[region] = self.model.new_session(self.max_context)
        self.hidden[region] = None

    def prefill(self, region: int, tokens: Sequence[int], start: int,
                on_chunk: Optional[Callable[[int], bool]] = None, embeds=None) -> Optional[torch.Tensor]:
        """``embeds`` = (offsets into ``tokens``, rows [m, hidden]): image spans that replace the
        embeddings of their placeholder tokens."""
        s = self.sessions[region]
        s.length = start
        toks = torch.tensor(list(tokens), dtype=torch.long)
        done, logits = 0, None
        while done < len(toks):
            n = min(self.chunk, len(toks) - done)
            xp = None
            if embeds is not None:
                m = (embeds[0] >= done) & (embeds[0] < done + n)
                if bool(m.any()):
                    xp = (embeds[0][m] - done, embeds[1][m])
            logits = self.model.forward(toks[done:done + n], s, x_patch=xp)
            self.hidden[region] = self.model.last_hidden[-1:].clone()
            done += n
            if on_chunk is not None and not on_chunk(done):
                return None
        return logits[-1] if logits is not None else None

    def sample(self, logits: torch.Tensor, temperature: float, top_p: float, seed: int, position: int) -> int:
        p = verify.modified_law(logits[None], temperature, top_p)[0]
        if temperature <= 0:
            return int(p.argmax())
        return verify.sample_from(p, rng.uniform(rng.block_round_seed(seed, position), rng.TARGET_DOMAIN, position))

    def decode_step(self, slots: Sequence[DecodeSlot]) -> List[List[int]]:
        out = []
        for sl in slots:
            s = self.sessions[sl.region]
            s.length = sl.length
            g = self.depth if sl.length + self.depth + 2 < self.max_context else 0
            draft_u, accept_u, final_u = rng.round_uniforms(sl.seed, sl.length, g)
            props, Q = [], []
            hid, tok = self.hidden[sl.region], sl.anchor
            copied = None
            if g > 0 and sl.lookup is not None:
                prop = sl.lookup.propose(pending=[sl.anchor])
                if prop is not None and len(prop.tokens) >= g:
                    copied = prop.tokens[:g]           # point-mass proposals: no draft law to sample
            conf, cum = [], 1.0
            ladder = self.cfg.draft.confidence_ladder
            for j in range(g if copied is None else 0):
                fed = tok
                lg, hid = self.model.draft_forward(torch.tensor([tok]), hid, s, sl.length + j)
                if self.cfg.draft.confidence_head:
                    # causal stopping: the confidence of proposal j + 1 is known before it is sampled;
                    # the first running product under its threshold ends the block (nothing later can
                    # change that decision, so the accepted tokens keep the target's law)
                    conf.append(float(self.model.draft_confidence(torch.tensor([fed]), hid)[0]))
                    cum *= conf[-1]
                    if j >= 1 and not (cum >= ladder[min(j - 1, len(ladder) - 1)]):
                        break
                q = verify.modified_law(lg, sl.temperature, sl.top_p)[0]
                tok = verify.sample_from(q, draft_u[j]) if sl.temperature > 0 else int(q.argmax())
                props.append(tok)
                Q.append(q)
            if copied is not None:
                props, Q = list(copied), None
            sl.confidence, sl.verified = conf, len(props)
            if len(props) < g:
                # a shorter block: its last row is the bonus row; the final draw stays the round's own
                g = len(props)
                accept_u = accept_u[:g]
            rows = torch.tensor([sl.anchor] + props)
            lg = self.model.forward(rows, s, start=sl.length, commit=False)
            P = verify.modified_law(lg, sl.temperature, sl.top_p)
            if g == 0:
                tau = 0
                nxt = int(P[0].argmax()) if sl.temperature <= 0 else verify.sample_from(P[0], final_u)
            elif sl.temperature <= 0:
                tau = 0
                while tau < g and props[tau] == int(P[tau].argmax()):
                    tau += 1
                nxt = int(P[tau].argmax())
            else:
                tau, nxt = verify.block_verify(P, torch.stack(Q) if Q is not None else None, props, accept_u, final_u)
            toks = [sl.anchor] + props[:tau]
            if sl.lookup is not None:
                sl.lookup.commit(sl.length, toks)
            sl.length += len(toks)
            s.length = sl.length
            sl.emitted += toks
            sl.anchor = nxt
            self.hidden[sl.region] = self.model.last_hidden[tau:tau + 1].clone()
            out.append(toks)
        return out

    # ---- state images ------------------------------------------------------------------------
    def _views(self, region: int, length: int) -> List[Tuple[str, torch.Tensor]]:
        s = self.sessions[region]
        ratio = lambda k: self.cfg.ratio_of_source(int(k.rsplit(".", 1)[1]))      # key: "layers.<source layer>"
        out = []
        for k, t in s.window.items():
            out.append((f"swa.{k}", t[max(0, length - self.cfg.window - 8):length]))
        for k, t in s.comp.items():
            out.append((f"compressed.{k}.kv", t[: length // ratio(k)]))
        for k, t in s.keys.items():
            out.append((f"compressed.{k}.keys", t[: length // ratio(k)]))
        for k, t in s.carry.items():
            out.append((f"compressed.{k}.carry", t[length // ratio(k) * ratio(k):length]))
        if self.hidden[region] is not None:
            out.append(("hidden", self.hidden[region]))
        return out

    def snapshot(self, region: int, tokens: Sequence[int], kind: str = "complete", media: str = "") -> SI.Image:
        return SI.capture(tokens, self._views(region, len(tokens)), kind, media, {"length": len(tokens)})

    def restore(self, region: int, img: SI.Image) -> None:
        self.reset(region)
        s = self.sessions[region]
        n = img.length
        for name, flat in img.regions:
            t = flat.view(torch.float32)
            if name == "hidden":
                self.hidden[region] = t.reshape(1, *([self.cfg.hc_mult] if self.cfg.hc_mult > 1 else []), self.cfg.hidden).clone()
                continue
            kind, key = name.split(".", 1)
            if kind == "swa":
                lo = max(0, n - self.cfg.window - 8)
                buf = s.buf(s.window, key, s.max_tokens, self.cfg.head_dim)
                buf[lo:n] = t.reshape(n - lo, -1)
            else:
                key, what = key.rsplit(".", 1)
                r = self.cfg.ratio_of_source(int(key.rsplit(".", 1)[1]))
                if what == "kv":
                    s.buf(s.comp, key, s.max_tokens // r + 1, self.cfg.head_dim)[: n // r] = t.reshape(n // r, -1)
                elif what == "keys":
                    s.buf(s.keys, key, s.max_tokens // r + 1, self.cfg.index_dim)[: n // r] = t.reshape(n // r, -1)
                else:
                    C = self.cfg.head_dim + self.cfg.index_dim
                    s.buf(s.carry, key, s.max_tokens, 2, C)[n // r * r:n] = t.reshape(n - n // r * r, 2, C)
        s.length = n


class EngineBackend:
    """The CUDA engine: tcgen05 prefill path, batched speculative decode under CUDA graphs."""
    name = "engine"

    def __init__(self, engine, chunk: int = 16384):
        from ..ops import bigpath, native
        from ..spec.decoder import SpecDecoder
        self.e, self.cfg, self.regions = engine, engine.cfg, engine.regions
        self.max_context, self.chunk = engine.ecfg.max_context, min(chunk, engine.max_chunk)
        self.device = engine.dev
        if engine.big_gemm is None:
            bigpath.attach(engine)
        self._dec: Dict[int, object] = {}
        self.max_graph_variants = 8      # decoders (one per batch size) kept with their CUDA graphs
        self._SpecDecoder, self._native = SpecDecoder, native
        self._status_host = (0, 0, 0, 0)
        self.last_hidden_rows: Dict[int, torch.Tensor] = {}

    def reset(self, region: int) -> None:
        pass     # state is position-addressed: a new conversation simply overwrites it

    def status_snapshot(self):
        """Last host copy of the kernels' status word (code, kernel, detail0, detail1), refreshed by
        the owner thread after every decode step and prefill; read by the health watchdog."""
        return self._status_host

    def _refresh_status(self) -> None:
        self._status_host = tuple(self.e.status.read())

    wants_prev = True      # prefill(..., prev=tokens right before `start`)

    def prefill(self, region, tokens, start, on_chunk=None, prev=(), embeds=None):
        from .prefill import run_prefill
        lg = run_prefill(self.e, region, torch.tensor(list(tokens), dtype=torch.int32), self.chunk, start,
                         True, on_chunk, prev=prev, embeds=embeds)
        self._refresh_status()
        if lg is None:
            return None
        self.last_hidden_rows[region] = self.e.last_hidden[-1:].clone() if self.e.last_hidden is not None else None
        return lg[-1].float()

    def sample(self, logits, temperature, top_p, seed, position) -> int:
        if temperature <= 0:
            return int(logits.argmax())
        p = verify.modified_law(logits.detach().cpu()[None], temperature, top_p)[0]
        return verify.sample_from(p, rng.uniform(rng.block_round_seed(seed, position), rng.TARGET_DOMAIN, position))

    def decode_step(self, slots):
        # one decoder (and one captured graph) per batch size: every conversation's temperature and
        # top-p travel with the step metadata, so mixed settings share the launch
        key = len(slots)
        dec = self._dec.pop(key, None)
        if dec is None:
            dec = self._SpecDecoder(self.e, len(slots))
            # bounded retention of captured graph variants (least recently used goes first)
            while len(self._dec) >= self.max_graph_variants:
                self._dec.pop(next(iter(self._dec)))
        self._dec[key] = dec                     # most recently used last
        for i, s in enumerate(slots):
            h = self.last_hidden_rows.get(s.region)
            if h is not None:
                dec.hidden[i].copy_(h.reshape(-1)[-self.cfg.hidden:])
        out = dec.step(slots)
        for i, s in enumerate(slots):
            self.last_hidden_rows[s.region] = dec.hidden[i].clone()
        self._refresh_status()
        return out

    def _views(self, region: int, length: int):
        e, cfg = self.e, self.cfg
        out = []
        keep = min(length, cfg.window + 64)
        slots = torch.arange(length - keep, length, device=e.dev) % e.ring
        out.append(("swa", e.win[:, region][:, slots]))
        for slot, src in enumerate(cfg.kv_source_layers):
            nC = length // cfg.ratio_of_source(src)
            out.append((f"compressed.kv.{slot}", e.comp[slot, region, :nC]))
            out.append((f"compressed.keys.{slot}", e.keys[slot, region, :nC]))
            out.append((f"compressed.carry.{slot}", e.carry[slot, region]))
        h = self.last_hidden_rows.get(region)
        if h is not None:
            out.append(("hidden", h))
        return out

    def snapshot(self, region, tokens, kind="complete", media=""):
        return SI.capture(tokens, self._views(region, len(tokens)), kind, media, {"length": len(tokens)})

    def restore(self, region, img):
        e, cfg = self.e, self.cfg
        n = img.length
        if img.tier != "device":
            img.to_device(e.dev)
        for name, flat in img.regions:
            if name == "swa":
                keep = min(n, cfg.window + 64)
                slots = torch.arange(n - keep, n, device=e.dev) % e.ring
                e.win[:, region][:, slots] = flat.view(e.win.shape[0], keep, e.win_row)
            elif name.startswith("compressed."):
                what, slot = name.split(".")[1], int(name.split(".")[2])
                nC = n // cfg.ratio_of_source(cfg.kv_source_layers[slot])
                if what == "kv":
                    e.comp[slot, region, :nC] = flat.view(nC, e.comp_row)
                elif what == "keys":
                    e.keys[slot, region, :nC] = flat.view(nC, e.key_row)
                else:
                    e.carry[slot, region] = flat.view(torch.float32).view(e.carry[slot, region].shape)
            elif name == "hidden":
                self.last_hidden_rows[region] = flat.view(torch.bfloat16).clone()
