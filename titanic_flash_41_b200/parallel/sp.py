"""Sequence-parallel prefill: the rows of a prefill chunk are split over the ranks.

Decode keeps the tensor-parallel layout (heads and experts split, every rank sees every row).  A
prefill chunk of thousands of rows is different: in that layout every rank would push every row
through the replicated parts (norms, KV / compressor / index projections, router, indexer) and
the two sublayer sums would each be an all-reduce of [rows, hidden].  Here rank r instead takes
rows [r * T / world, (r + 1) * T / world) of the chunk through the WHOLE dense part of a layer --
all heads of the attention, the full output projection, the full shared expert -- using the
unsharded dense matrices it keeps for the encoder layers (``LayerWeights.full``; the reference
stages such derived full matrices for its SP layers, src/staged_full.rs, and runs SP layers through
src/decoder.rs:916 gather_input / :930 reduce_attention / :991 grouped_sum_scatter).  What crosses
NVLink per layer and chunk:

  * the state rows the chunk wrote (window KV ring rows, compressed entries, index keys): an
    all-gather of ~0.6 KB per token, after which every rank holds the identical KV state, exactly
    as after a tensor-parallel prefill, so decode continues unchanged;
  * the routed experts stay expert-parallel: the normalised rows (f16), expert ids and weights of
    all ranks are all-gathered, every rank runs ITS experts over the rows routed to them, and the
    partial outputs travel back as bf16 slices that the owner of the rows sums in rank order in
    fp32 (an exchange of slices + local fixed-order sum: deterministic, unlike a ring reduction;
    reference: the quarter exchange + local fp32 sum, src/prefill_exchange.rs).  With 6 of 256
    experts per token spread over 8 ranks, an all-to-all dispatch would move about as many bytes.

Attention and the dense projections need no collective at all.  Slices end on multiples of the
compression ratio (in absolute position), so every compressor group lives on one rank.
"""
from __future__ import annotations

import types
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..models.engine import Engine, StepPlan
from ..ops import native
from .comm import LocalComm


class SpPrefill:
    """Built collectively by every rank after the tensor-core path is attached to ``eng``."""

    def __init__(self, eng: Engine):
        cfg = eng.cfg
        if eng.world < 2:
            raise ValueError("sequence-parallel prefill needs more than one rank")
        late = cfg.late_start if 0 < cfg.late_start < len(eng.layers) else len(eng.layers)
        if any(eng.layers[li].full is None for li in range(late)):
            raise ValueError("the encoder layers do not carry their unsharded dense matrices")
        if cfg.hc_mult > 1 or eng.engram:
            raise ValueError("sequence-parallel prefill covers plain residual streams without Engram layers")
        self.eng, self.late = eng, late
        self.W, self.rank = eng.world, eng.rank
        # a single-rank view of the engine for the dense sublayers: all heads, unsharded matrices, the
        # parent's KV state; its expert sublayer is the exchange below
        v = Engine.__new__(Engine)
        v.__dict__.update(eng.__dict__)
        v.comm = LocalComm()
        v.world, v.rank = 1, 0
        v.Hl = cfg.n_heads
        v.layers = [eng.layers[li].full if li < late else eng.layers[li] for li in range(len(eng.layers))]
        v.draft_layers, v.draft_extra = [], {}
        v._scratch, v._dq_cache = {}, {}
        v._side, v.symm, v.sp = None, None, None
        v.big_gemm = v.big_moe_full = None
        from ..ops import bigpath
        bigpath.attach(v)

        def _never(*a, **k):
            raise RuntimeError("the sequence-parallel view runs its experts through the exchange")
        v.big_moe_full = _never          # (kept non-null: the view's scratch then skips the per-pair expert buffers)
        v._moe = types.MethodType(lambda view, L, T, b, next_norm=None: self._moe(L, T, b), v)
        v.after_prep = self._gather_state
        self.view = v
        self._stage = {}
        self._plans: dict = {}                                      # (region, first position, rows) -> plan of a slice; cleared per prefill
        self._slice: Tuple[int, int, int, int] = (0, 0, 0, 0)      # region, first position, rows of the chunk, rows per rank

    # ------------------------------------------------------------------------------------------
    def rows_per_rank(self, T: int) -> int:
        r = self.eng.cfg.max_ratio            # slices begin on a group boundary of every stream
        per = -(-T // self.W)
        return -(-per // r) * r

    def usable(self, start: int, n: int) -> bool:
        """Chunks must begin on a compressor-group boundary and leave every rank at least the small-M
        limit of rows (shorter prompts take the tensor-parallel path)."""
        return start % self.eng.cfg.max_ratio == 0 and n >= self.W * 2 * Engine.SMALL_M

    def bounds(self, T: int) -> Tuple[int, int, int]:
        """(first row, end row, rows per rank) of this rank's slice of a chunk of T rows."""
        tq = self.rows_per_rank(T)
        lo = min(T, self.rank * tq)
        return lo, min(T, lo + tq), tq

    def _buf(self, name: str, shape, dtype) -> torch.Tensor:
        t = self._stage.get(name)
        n = int(np.prod(shape))
        if t is None or t.numel() < n or t.dtype != dtype:
            t = torch.empty(n, dtype=dtype, device=self.eng.dev)
            self._stage[name] = t
        return t[:n].view(*shape)

    def _all_gather(self, name: str, local: torch.Tensor) -> torch.Tensor:
        """[rows_per_rank, ...] -> [world, rows_per_rank, ...] (equal slices; the last ranks' slices may
        hold padding)."""
        out = self._buf(name, (self.W,) + tuple(local.shape), local.dtype)
        dist.all_gather_into_tensor(out.view(-1), local.contiguous().view(-1))
        return out

    # ---- hooks of the single-rank view ---------------------------------------------------------
    def _gather_state(self, li: int, L, T: int, b: dict) -> None:
        """After a layer's KV store: every rank receives the rows the other ranks wrote."""
        eng = self.eng
        cfg = eng.cfg
        region, p0, Tc, tq = self._slice
        dev = eng.dev
        lo, hi, _ = self.bounds(Tc)
        # window ring rows of the chunk: position p sits in slot p % ring
        # (rank r's rows are chunk rows [r * tq, ...), so the gathered [world * tq] rows are in chunk order)
        slots_all = (p0 + torch.arange(Tc, device=dev)) % eng.ring
        mine = self._buf("win_l", (tq, eng.win_row), torch.uint8)
        if hi > lo:
            mine[: hi - lo].copy_(eng.win[li, region].index_select(0, slots_all[lo:hi]))
        g = self._all_gather("win_g", mine).view(self.W * tq, eng.win_row)
        eng.win[li, region].index_copy_(0, slots_all, g[:Tc])
        if not L.is_kv_source:
            return
        # compressed entries and index keys completed inside the chunk: entry e = position // ratio
        r = cfg.ratio_of_source(li)
        slot = eng.src_slot[li]
        eq = tq // r
        e0 = p0 // r
        n_e = (p0 + Tc) // r - e0                                    # complete groups of the chunk
        elo, ehi = min(n_e, self.rank * eq), min(n_e, (self.rank + 1) * eq)
        for name, store, width in (("comp", eng.comp, eng.comp_row), ("keys", eng.keys, eng.key_row)):
            mine = self._buf(name + "_l", (eq, width), torch.uint8)
            if ehi > elo:
                mine[: ehi - elo].copy_(store[slot, region, e0 + elo:e0 + ehi])
            g = self._all_gather(name + "_g", mine).view(self.W * eq, width)
            store[slot, region, e0:e0 + n_e].copy_(g[:n_e])
        # inputs of the group left open at the end of the chunk: saved by the rank that holds the last row
        last_rank = min(self.W - 1, (Tc - 1) // tq)
        dist.broadcast(eng.carry[slot, region], src=last_rank)

    def _moe(self, L, T: int, b: Optional[dict]) -> None:
        """Expert sublayer of the view's T local rows (b holds their normalised rows in h16 / hb):
        router here, routed experts where they live, shared expert here.  T = 0 (a rank without rows in
        a short last chunk): the rank still runs its experts for the others."""
        eng, v = self.eng, self.view
        cfg = eng.cfg
        d, k = cfg.hidden, cfg.topk
        _, _, Tc, tq = self._slice
        scoring = 1 if cfg.scoring == "sqrtsoftplus" else 0
        st = eng.status.t
        if T == 0:
            pass
        elif cfg.n_experts % 128 == 0:
            native.call("tf_gemm_tc", 0, b["hb"], d, L.gate, d, b["logits_r"], cfg.n_experts, T, cfg.n_experts, d, None,
                        0, None, 0, 0, None, None, 0, st)
            native.call("tf_router_topk", b["logits_r"], L.gate_bias, L.gate_bias_vl, b["meta"][0], cfg.image_token,
                        b["ids"], b["wts"], T, cfg.n_experts, cfg.topk, scoring, 1 if cfg.renorm else 0, cfg.route_scale)
        else:
            native.call("tf_router", b["h16"], L.gate, L.gate_bias, L.gate_bias_vl, b["meta"][0], cfg.image_token,
                        b["logits_r"], b["ids"], b["wts"], T, cfg.n_experts, d, cfg.topk, scoring, 1 if cfg.renorm else 0,
                        cfg.route_scale)
        # ---- rows, ids and weights of every rank (slices padded to tq rows; padding routes nowhere)
        h_l = self._buf("h_l", (tq, d), torch.float16)
        ids_l = self._buf("ids_l", (tq, k), torch.int32)
        wts_l = self._buf("wts_l", (tq, k), torch.float32)
        if T < tq:
            h_l.zero_()
            ids_l.fill_(-1)
            wts_l.zero_()
        if T > 0:
            h_l[:T].copy_(b["h16"][:T])
            ids_l[:T].copy_(b["ids"][:T])
            wts_l[:T].copy_(b["wts"][:T])
        Tp = self.W * tq
        # rows, ids and weights of the padded chunk (all the expert path reads of its row buffers)
        pb = {"h16": self._buf("h_g", (Tp, d), torch.float16), "ids": self._buf("ids_g", (Tp, k), torch.int32),
              "wts": self._buf("wts_g", (Tp, k), torch.float32)}
        dist.all_gather_into_tensor(pb["h16"].view(-1), h_l.view(-1))
        dist.all_gather_into_tensor(pb["ids"].view(-1), ids_l.view(-1))
        dist.all_gather_into_tensor(pb["wts"].view(-1), wts_l.view(-1))
        # ---- this rank's experts over all rows (the shared expert is not part of the exchange), written
        # as bf16 slices that go back to the owners of the rows, who sum them in rank order in fp32
        send = self._buf("y_send", (self.W, tq, d), torch.bfloat16)
        eng.big_moe_full(eng, L, Tp, pb, with_shared=False, out=send.view(Tp, d))
        recv = self._buf("y_recv", (self.W, tq, d), torch.bfloat16)
        dist.all_to_all_single(recv.view(-1), send.view(-1))
        if T == 0:
            return
        shared = None
        if cfg.n_shared:
            v._linear(b["h16"], L.sw1, b["s_act"], T, w3=L.sw3)
            v._linear(b["s_act"], L.sw2, b["s_y"], T)
            shared = b["s_y"]
        native.call("tf_sum_slices", recv, self.W, (tq * d), shared, b["delta"], T * d)
        b["pending"] = True

    # ---- driver ----------------------------------------------------------------------------------
    def run_layer(self, li: int, region: int, p0: int, Tc: int, tokens: np.ndarray, x_in: Optional[torch.Tensor],
                  x_patch, sel_in, prev_recent=None) -> Tuple[dict, int, int]:
        """Layer ``li`` on this rank's slice of the chunk of Tc rows that starts at position p0.
        ``tokens``: the chunk's token ids; ``x_in``: the slice's residual rows from the previous layer
        (None at layer 0).  Returns (buffers, first row, rows) of the slice; every rank must call this
        for every layer and chunk (the exchanges are collective), also with an empty slice."""
        v = self.view
        lo, hi, tq = self.bounds(Tc)
        self._slice = (region, p0, Tc, tq)
        T = hi - lo
        if T == 0:
            # no rows of this (short, last) chunk: only the collective parts of the layer
            L = v.layers[li]
            self._gather_state(li, L, 0, None)
            self._moe(L, 0, None)
            return None, lo, 0
        key = (region, p0 + lo, T)
        hit = self._plans.get(key)
        if hit is None:                                             # one plan per slice, shared by all layers
            plan = StepPlan.build([(region, p0 + lo, tokens[lo:hi].tolist())], logits="last")
            hit = self._plans[key] = (plan,) + tuple(v.plan_shape(plan, v.cfg.compress_ratio))
        plan, nmax, rpg = hit
        b = v._bufs(T)
        v.upload_plan(plan, b)
        if sel_in is not None:
            src, ids, cnt = sel_in
            b["sel"][src][:T].copy_(ids)
            b["selcnt"][src][:T].copy_(cnt)
        v.run(T, b, nmax, rpg, None, li, li + 1, x_in=x_in, x_patch=x_patch)
        return b, lo, T

    def gather_rows(self, local: Optional[torch.Tensor], Tc: int, width: int, dtype) -> torch.Tensor:
        """The chunk's [Tc, width] rows assembled from every rank's slice."""
        lo, hi, tq = self.bounds(Tc)
        mine = self._buf("rows_l", (tq, width), dtype)
        if hi > lo:
            mine[: hi - lo].copy_(local)
        return self._all_gather("rows_g", mine).view(self.W * tq, width)[:Tc]

    def chunk_sizes(self, n: int, chunk: int) -> list:
        """Near-equal chunks whose sizes are multiples of world x compression ratio (so that every
        rank's slice of every chunk but the last is full and ends on a group boundary)."""
        unit = self.W * self.eng.cfg.max_ratio
        # a chunk may span `sp_chunk_rows` rows over all ranks as long as every rank's slice fits the
        # row buffers of a single-rank chunk and the whole chunk fits the window ring
        eng = self.eng
        cap = min(max(chunk, eng.ecfg.sp_chunk_rows), eng.max_chunk * self.W, eng.ring - 2 * eng.cfg.window)
        k = max(1, -(-n // cap))
        while True:
            per = -(-(-(-n // k)) // unit) * unit
            if per <= cap or per <= unit:
                break
            k += 1
        sizes = []
        left = n
        while left > 0:
            sizes.append(min(per, left))
            left -= sizes[-1]
        return sizes


def attach(eng: Engine) -> Optional[SpPrefill]:
    """Give ``eng`` a sequence-parallel prefill when it can have one (several ranks, the tensor-core
    path attached, unsharded dense matrices kept, plain residual stream); collective."""
    if eng.world < 2 or not eng.ecfg.sp_prefill or getattr(eng, "big_moe_full", None) is None:
        return None
    try:
        eng.sp = SpPrefill(eng)
    except ValueError:
        eng.sp = None
    return eng.sp
