"""CUDA engine: the model graph executed with the sm_100a kernels of ``csrc/``.

One ``Engine`` per rank owns the rank's quantised weight shard, the KV state of every serving
region (window rings in the V4.1 FP8 row format, compressed streams in the V4.1-FP4 format,
index keys, compressor carries) and the scratch of each row-count profile.  ``forward`` runs a
batch of rows -- a prefill chunk of one conversation or the verification blocks of up to
``regions`` conversations -- and returns fp32 logits for the requested rows.

Row state is addressed by absolute position (ring slot = pos % ring, compressed entry =
pos // ratio), so rejecting speculative rows needs no rollback copies: the next launch simply
overwrites them (the reference keeps carry snapshots for this: src/carry_state.rs).

Reference counterparts: src/target.rs (Target::execute_rows :5632, Plan :475), src/decoder.rs
(SwaLayer), src/layer_attention.rs, src/ffn.rs, src/model_io.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..config import EngineConfig, ModelConfig
from ..formats import codecs
from ..ops import native
from ..parallel.comm import Comm, LocalComm
from . import oracle

F8 = torch.float8_e4m3fn


def _pad128(n: int) -> int:
    return -(-n // 128) * 128


# ---------------------------------------------------------------------------------------------
# weight preparation
# ---------------------------------------------------------------------------------------------
@dataclass
class Fp8Weight:
    """[N, K] e4m3 + fp32 scale per 128x128 block; N padded to 128.  The scales are powers of two
    (what a UE8M0 checkpoint gives), so the same values also serve the block-scaled tensor-core GEMM:
    ``sfu`` caches their UE8M0 form in that kernel's layout (False: not expressible)."""
    q: torch.Tensor
    s: torch.Tensor
    n: int
    k: int
    sfu: object = None


@dataclass
class LayerWeights:
    proj: Fp8Weight = None
    offs: Dict[str, int] = field(default_factory=dict)
    wo: Fp8Weight = None
    attn_norm: torch.Tensor = None
    ffn_norm: torch.Tensor = None
    kv_norm: torch.Tensor = None
    comp_norm: Optional[torch.Tensor] = None
    sink: Optional[torch.Tensor] = None
    gate: torch.Tensor = None
    gate_bias: Optional[torch.Tensor] = None
    gate_bias_vl: Optional[torch.Tensor] = None    # selection bias of image-token rows
    ew1: torch.Tensor = None
    ew3: torch.Tensor = None
    ew2: torch.Tensor = None
    es1: torch.Tensor = None
    es3: torch.Tensor = None
    es2: torch.Tensor = None
    sw1: Optional[Fp8Weight] = None
    sw3: Optional[Fp8Weight] = None
    sw2: Optional[Fp8Weight] = None
    is_kv_source: bool = False
    is_index_source: bool = False
    kv_source: int = -1
    index_source: int = -1
    # geometry of the reference model proper (reference: src/layout.rs:57-144)
    q_norm: Optional[torch.Tensor] = None          # low-rank query: proj holds wq_a, then norm, then wq_b
    wq_b: Optional[Fp8Weight] = None
    wo_a: Optional[List[Fp8Weight]] = None         # grouped output projection: one [rank, per] per local group
    hc: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]] = None   # "attn"/"ffn" -> (fn, base, scale)
    # unsharded dense matrices of this layer (all heads, full shared expert) for the sequence-parallel
    # prefill, where every rank runs whole rows through the dense sublayers (reference: the derived
    # full matrices of SP layers, src/staged_full.rs)
    full: Optional["LayerWeights"] = None


POW2_SCALES = True      # block scales rounded up to powers of two (False: amax / 448 exactly; such weights stay off the block-scaled GEMM)


def quant_fp8_device(w: torch.Tensor) -> Fp8Weight:
    """Block-128 FP8 quantisation on the tensor's device; rows padded to a multiple of 128."""
    n, k = w.shape
    assert k % 128 == 0
    npad = _pad128(n)
    wf = torch.zeros(npad, k, dtype=torch.float32, device=w.device)
    wf[:n] = w.float()
    t = wf.view(npad // 128, 128, k // 128, 128)
    s = t.abs().amax(dim=(1, 3)).clamp_min(1e-12) / codecs.E4M3_MAX
    if POW2_SCALES:
        s = torch.exp2(torch.ceil(torch.log2(s)).clamp(-126, 126))     # UE8M0: the checkpoint's scale format
    q = (t / s[:, None, :, None]).clamp(-448, 448).to(F8).view(npad, k)
    return Fp8Weight(q.contiguous(), s.contiguous(), n, k)


def dequant_fp8(w: Fp8Weight) -> torch.Tensor:
    n, k = w.q.shape
    t = w.q.float().view(n // 128, 128, k // 128, 128) * w.s[:, None, :, None]
    return t.view(n, k)[: w.n]


def quant_mxfp4_device(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[..., K] -> (packed e2m1 uint8 [..., K/2], ue8m0 uint8 [..., K/32]) on the tensor's device."""
    *lead, K = w.shape
    g = w.float().reshape(*lead, K // 32, 32)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / 6.0))
    e = torch.where(torch.exp2(e) < amax / 6.0, e + 1, e)
    code = (e + 127).clamp(0, 247).to(torch.uint8)
    s = torch.exp2(code.float() - 127)
    x = g / s.unsqueeze(-1)
    a = x.abs()
    idx = torch.zeros_like(a, dtype=torch.uint8)
    for i, (mid, even_up) in enumerate(((0.25, False), (0.75, True), (1.25, False), (1.75, True),
                                        (2.5, False), (3.5, True), (5.0, False))):
        up = (a > mid) | ((a == mid) & even_up)
        idx = torch.where(up, torch.full_like(idx, i + 1), idx)
    codes = (idx | ((x < 0).to(torch.uint8) << 3)).reshape(*lead, K)
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)
    return packed.contiguous(), code.contiguous()


def quad_pack(p: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 [..., K/2] -> the decode kernels' layout: inside every 64-byte run (128 k = four
    32-wide scale groups) the sixteen 4-byte words are transposed, so that the 16 bytes one lane
    loads hold eight weights of EACH of the four groups and one FP8 tensor-core step covers exactly
    one scale group (the B200 counterpart of the reference's expert repack, src/expert_packing.rs)."""
    *lead, kb = p.shape
    assert kb % 64 == 0
    return p.reshape(*lead, kb // 64, 4, 4, 4).transpose(-3, -2).contiguous().reshape(*lead, kb)


def quad_unpack(p: torch.Tensor) -> torch.Tensor:
    return quad_pack(p)          # the word transpose is its own inverse


def dequant_mxfp4(p: torch.Tensor, code: torch.Tensor) -> torch.Tensor:
    vals = torch.tensor(codecs.E2M1_VALUES, dtype=torch.float32, device=p.device)
    lo, hi = (p & 0xF).long(), (p >> 4).long()
    c = torch.stack([lo, hi], -1).reshape(*p.shape[:-1], p.shape[-1] * 2)
    v = torch.where((c & 8) != 0, -vals[c & 7], vals[c & 7])
    *lead, K = v.shape
    s = torch.exp2(code.float() - 127).unsqueeze(-1)
    return (v.reshape(*lead, K // 32, 32) * s).reshape(*lead, K)


def _layer_prefix(cfg: ModelConfig, li: int) -> str:
    return f"mtp.{li - cfg.n_layers}" if li >= cfg.n_layers else f"layers.{li}"


def prepare_layer(cfg: ModelConfig, W: Dict[str, torch.Tensor], li: int, rank: int, world: int,
                  device, roundtrip: Optional[Dict[str, torch.Tensor]] = None, keep_full: bool = False
                  ) -> LayerWeights:
    """Quantise one layer's shard from an fp32/bf16 weight dict (full, unsharded tensors) and, when
    ``roundtrip`` is given, record the dequantised full tensors there for the oracle.  ``keep_full``
    also keeps the unsharded dense matrices (``L.full``) for the sequence-parallel prefill."""
    p = _layer_prefix(cfg, li)
    draft = li >= cfg.n_layers
    H, Dh, d = cfg.n_heads, cfg.head_dim, cfg.hidden
    Hl = H // world
    L = LayerWeights()
    L.is_kv_source = (not draft) and li in cfg.kv_source_layers
    L.is_index_source = (not draft) and li in cfg.index_source_layers
    L.kv_source = -1 if draft else cfg.kv_source_of(li)
    L.index_source = -1 if draft else cfg.index_source_of(li)

    def dev(t, dt=None):
        t = t.to(device)
        return t.to(dt) if dt is not None else t

    def rt(name, full_q: Fp8Weight):
        if roundtrip is not None:
            roundtrip[name] = dequant_fp8(full_q).cpu()

    segs: List[Tuple[str, torch.Tensor]] = []
    if cfg.q_lora_rank:
        # low-rank query: wq_a (replicated) rides in the fused projection, wq_b keeps this rank's heads
        wqa = dev(W[f"{p}.attn.wq_a.weight"])
        rt(f"{p}.attn.wq_a.weight", quant_fp8_device(wqa))
        segs.append(("qa", wqa))
        wqb = dev(W[f"{p}.attn.wq_b.weight"])
        rt(f"{p}.attn.wq_b.weight", quant_fp8_device(wqb))
        L.wq_b = quant_fp8_device(wqb[rank * Hl * Dh:(rank + 1) * Hl * Dh].contiguous())
        L.q_norm = dev(W[f"{p}.attn.q_norm.weight"], torch.bfloat16)
    else:
        wq = dev(W[f"{p}.attn.wq.weight"])
        rt(f"{p}.attn.wq.weight", quant_fp8_device(wq))
        segs.append(("q", wq[rank * Hl * Dh:(rank + 1) * Hl * Dh]))
    segs.append(("kv", dev(W[f"{p}.attn.wkv.weight"])))
    rt(f"{p}.attn.wkv.weight", quant_fp8_device(segs[-1][1]))
    if L.is_kv_source:
        for nm, key in (("cv", "wkv"), ("cg", "wgate")):
            segs.append((nm, dev(W[f"{p}.attn.compressor.{key}.weight"])))
            rt(f"{p}.attn.compressor.{key}.weight", quant_fp8_device(segs[-1][1]))
    if L.is_index_source:
        segs.append(("iq", dev(W[f"{p}.attn.indexer.wq.weight"])))
        rt(f"{p}.attn.indexer.wq.weight", quant_fp8_device(segs[-1][1]))
        segs.append(("iw", dev(W[f"{p}.attn.indexer.weights_proj.weight"])))
        rt(f"{p}.attn.indexer.weights_proj.weight", quant_fp8_device(segs[-1][1]))
    def fuse(segments):
        qs, ss, off, offs = [], [], 0, {}
        for nm, t in segments:
            fw = quant_fp8_device(t)
            offs[nm] = off
            off += fw.q.shape[0]
            qs.append(fw.q)
            ss.append(fw.s)
        return Fp8Weight(torch.cat(qs).contiguous(), torch.cat(ss).contiguous(), off, d), offs
    L.proj, L.offs = fuse(segs)
    full_ok = keep_full and world > 1 and not cfg.q_lora_rank and not cfg.o_groups and not draft
    F = LayerWeights() if full_ok else None
    if full_ok:
        F.proj, F.offs = fuse([("q", dev(W[f"{p}.attn.wq.weight"]))] + segs[1:])
        F.wo = quant_fp8_device(dev(W[f"{p}.attn.wo.weight"]))
        if cfg.attn_sink:
            F.sink = dev(W[f"{p}.attn.attn_sink"], torch.float32).contiguous()
        if cfg.n_shared:
            F.sw1, F.sw3, F.sw2 = (quant_fp8_device(dev(W[f"{p}.ffn.shared_experts.{nm}.weight"]))
                                   for nm in ("w1", "w3", "w2"))
    if cfg.o_groups:
        # grouped low-rank output projection: this rank's groups of wo_a (block-diagonal), then the
        # matching K-slice of wo_b
        G, R = cfg.o_groups // world, cfg.o_lora_rank
        woa = dev(W[f"{p}.attn.wo_a.weight"])                    # [o_groups * R, H*Dh / o_groups]
        rt(f"{p}.attn.wo_a.weight", quant_fp8_device(woa))
        L.wo_a = [quant_fp8_device(woa[(rank * G + g) * R:(rank * G + g + 1) * R].contiguous()) for g in range(G)]
        wob = dev(W[f"{p}.attn.wo_b.weight"])                    # [d, o_groups * R]
        rt(f"{p}.attn.wo_b.weight", quant_fp8_device(wob))
        L.wo = quant_fp8_device(wob[:, rank * G * R:(rank + 1) * G * R].contiguous())
    else:
        wo = dev(W[f"{p}.attn.wo.weight"])
        rt(f"{p}.attn.wo.weight", quant_fp8_device(wo))
        L.wo = quant_fp8_device(wo[:, rank * Hl * Dh:(rank + 1) * Hl * Dh].contiguous())
    if cfg.hc_mult > 1:
        L.hc = {br: (dev(W[f"{p}.hc_{br}_fn"], torch.float32).contiguous(),
                     dev(W[f"{p}.hc_{br}_base"], torch.float32).contiguous(),
                     dev(W[f"{p}.hc_{br}_scale"], torch.float32).contiguous()) for br in ("attn", "ffn")}
    L.attn_norm = dev(W[f"{p}.attn_norm.weight"], torch.bfloat16)
    L.ffn_norm = dev(W[f"{p}.ffn_norm.weight"], torch.bfloat16)
    L.kv_norm = dev(W[f"{p}.attn.kv_norm.weight"], torch.bfloat16)
    if L.is_kv_source:
        L.comp_norm = dev(W[f"{p}.attn.compressor.norm.weight"], torch.bfloat16)
    if cfg.attn_sink:
        L.sink = dev(W[f"{p}.attn.attn_sink"], torch.float32)[rank * Hl:(rank + 1) * Hl].contiguous()
    L.gate = dev(W[f"{p}.ffn.gate.weight"], torch.bfloat16).contiguous()
    if roundtrip is not None:
        roundtrip[f"{p}.ffn.gate.weight"] = L.gate.float().cpu()
    if cfg.router_bias:
        L.gate_bias = dev(W[f"{p}.ffn.gate.bias"], torch.float32)
        if cfg.router_bias_vl and f"{p}.ffn.gate.bias_vl" in W:
            L.gate_bias_vl = dev(W[f"{p}.ffn.gate.bias_vl"], torch.float32)
    El = cfg.n_experts // world
    for nm in ("w1", "w3", "w2"):
        full = dev(W[f"{p}.ffn.experts.{nm}.weight"])
        if roundtrip is not None:
            pk, sc = quant_mxfp4_device(full)
            roundtrip[f"{p}.ffn.experts.{nm}.weight"] = dequant_mxfp4(pk, sc).cpu()
        pk, sc = quant_mxfp4_device(full[rank * El:(rank + 1) * El])
        setattr(L, "e" + nm, pk)
        setattr(L, "es" + nm[1], sc)
    if cfg.n_shared:
        Is = cfg.shared_inter * cfg.n_shared
        Il = Is // world
        for nm in ("w1", "w3", "w2"):
            full = dev(W[f"{p}.ffn.shared_experts.{nm}.weight"])
            rt(f"{p}.ffn.shared_experts.{nm}.weight", quant_fp8_device(full))
            sl = full[:, rank * Il:(rank + 1) * Il] if nm == "w2" else full[rank * Il:(rank + 1) * Il]
            setattr(L, "s" + nm, quant_fp8_device(sl.contiguous()))
    if full_ok:
        for nm in ("attn_norm", "ffn_norm", "kv_norm", "comp_norm", "gate", "gate_bias", "gate_bias_vl", "ew1", "ew3",
                   "ew2", "es1", "es3", "es2", "is_kv_source", "is_index_source", "kv_source", "index_source"):
            setattr(F, nm, getattr(L, nm))
        L.full = F
    return L


def random_layer(cfg: ModelConfig, li: int, rank: int, world: int, device, seed: int,
                 keep_full: bool = False) -> LayerWeights:
    """Random-init one layer's shard directly on the device in its quantised storage formats
    (the full-size model never exists in fp32): dense weights are N(0, init_std) quantised to
    block-128 FP8; expert nibbles are uniform random e2m1 codes with a fixed 2^-7 group scale.
    Dense and replicated tensors come from a generator that does not depend on the rank: every rank
    draws the same full matrix and keeps its slice, so replicated tensors agree across ranks and a
    rank's shard is a slice of the full matrix (``keep_full`` keeps that matrix as ``L.full``)."""
    g = torch.Generator(device=device).manual_seed(seed * 1000 + li * 16)
    ge = torch.Generator(device=device).manual_seed(seed * 1000 + li * 16 + 1 + rank)     # this rank's experts
    H, Dh, d = cfg.n_heads, cfg.head_dim, cfg.hidden
    Hl, El = H // world, cfg.n_experts // world
    draft = li >= cfg.n_layers
    L = LayerWeights()
    L.is_kv_source = (not draft) and li in cfg.kv_source_layers
    L.is_index_source = (not draft) and li in cfg.index_source_layers
    L.kv_source = -1 if draft else cfg.kv_source_of(li)
    L.index_source = -1 if draft else cfg.index_source_of(li)

    def rnd(n, k, std=None):
        return torch.randn(n, k, generator=g, device=device, dtype=torch.bfloat16) * (std or cfg.init_std)

    if cfg.q_lora_rank:
        segs = [("qa", rnd(cfg.q_lora_rank, d)), ("kv", rnd(Dh, d))]
        L.wq_b = quant_fp8_device(rnd(Hl * Dh, cfg.q_lora_rank))
        L.q_norm = torch.ones(cfg.q_lora_rank, dtype=torch.bfloat16, device=device)
    else:
        wq_full = rnd(H * Dh, d)
        segs = [("q", wq_full[rank * Hl * Dh:(rank + 1) * Hl * Dh]), ("kv", rnd(Dh, d))]
    if L.is_kv_source:
        segs += [("cv", rnd(Dh + cfg.index_dim, d)), ("cg", rnd(Dh + cfg.index_dim, d))]
    if L.is_index_source:
        segs += [("iq", rnd(cfg.index_heads * cfg.index_dim, d)), ("iw", rnd(cfg.index_heads, d, 1 / math.sqrt(d)))]

    def fuse(segments):
        qs, ss, off, offs = [], [], 0, {}
        for nm, t in segments:
            fw = quant_fp8_device(t)
            offs[nm] = off
            off += fw.q.shape[0]
            qs.append(fw.q)
            ss.append(fw.s)
        return Fp8Weight(torch.cat(qs).contiguous(), torch.cat(ss).contiguous(), off, d), offs
    L.proj, L.offs = fuse(segs)
    full_ok = keep_full and world > 1 and not cfg.q_lora_rank and not cfg.o_groups and not draft
    F = LayerWeights() if full_ok else None
    if full_ok:
        F.proj, F.offs = fuse([("q", wq_full)] + segs[1:])
    if cfg.o_groups:
        G, R = cfg.o_groups // world, cfg.o_lora_rank
        L.wo_a = [quant_fp8_device(rnd(R, Hl * Dh // G)) for _ in range(G)]
        L.wo = quant_fp8_device(rnd(d, G * R))
    else:
        wo_full = rnd(d, H * Dh)
        L.wo = quant_fp8_device(wo_full[:, rank * Hl * Dh:(rank + 1) * Hl * Dh].contiguous())
        if full_ok:
            F.wo = quant_fp8_device(wo_full)
        del wo_full
    if cfg.hc_mult > 1:
        m = cfg.hc_mult
        L.hc = {br: ((torch.randn(m * (2 + m), m * d, generator=g, device=device) * cfg.init_std).contiguous(),
                     torch.zeros(m * (2 + m), device=device), torch.ones(3, device=device)) for br in ("attn", "ffn")}
    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    L.attn_norm, L.ffn_norm, L.kv_norm = ones(d), ones(d), ones(Dh)
    if L.is_kv_source:
        L.comp_norm = ones(Dh)
    if cfg.attn_sink:
        sink_full = torch.randn(H, generator=g, device=device) * 0.5
        L.sink = sink_full[rank * Hl:(rank + 1) * Hl].contiguous()
        if full_ok:
            F.sink = sink_full
    L.gate = rnd(cfg.n_experts, d, 1 / math.sqrt(d)).contiguous()
    if cfg.router_bias:
        L.gate_bias = torch.zeros(cfg.n_experts, device=device)
    I = cfg.moe_inter
    for nm, n, k in (("w1", I, d), ("w3", I, d), ("w2", d, I)):
        pk = torch.randint(0, 256, (El, n, k // 2), generator=ge, device=device, dtype=torch.uint8)
        sc = torch.full((El, n, k // 32), 120, dtype=torch.uint8, device=device)
        setattr(L, "e" + nm, pk)
        setattr(L, "es" + nm[1], sc)
    if cfg.n_shared:
        Is = cfg.shared_inter * cfg.n_shared
        Il = Is // world
        s1, s3, s2 = rnd(Is, d), rnd(Is, d), rnd(d, Is)
        L.sw1 = quant_fp8_device(s1[rank * Il:(rank + 1) * Il])
        L.sw3 = quant_fp8_device(s3[rank * Il:(rank + 1) * Il])
        L.sw2 = quant_fp8_device(s2[:, rank * Il:(rank + 1) * Il].contiguous())
        if full_ok:
            F.sw1, F.sw3, F.sw2 = quant_fp8_device(s1), quant_fp8_device(s3), quant_fp8_device(s2)
    if full_ok:
        # everything that is replicated anyway is shared with the sharded view
        for nm in ("attn_norm", "ffn_norm", "kv_norm", "comp_norm", "gate", "gate_bias", "gate_bias_vl", "ew1", "ew3",
                   "ew2", "es1", "es3", "es2", "is_kv_source", "is_index_source", "kv_source", "index_source"):
            setattr(F, nm, getattr(L, nm))
        L.full = F
    return L


# ---------------------------------------------------------------------------------------------
# step plan (host metadata of one launch; reference: Plan, src/target.rs:475-683)
# ---------------------------------------------------------------------------------------------
@dataclass
class StepPlan:
    """Rows of one launch.  Rows of a conversation are consecutive and at consecutive positions."""
    tokens: np.ndarray          # [T] int32
    pos: np.ndarray             # [T]
    region: np.ndarray          # [T]
    first_row: np.ndarray       # [T] first row index of the row's conversation in this launch
    last_pos: np.ndarray        # [T] last position of the row's conversation in this launch
    logit_rows: np.ndarray      # rows whose logits are wanted
    group_rows: int             # rows per conversation block (uniform), used to group index scoring
    min_pos: Optional[np.ndarray] = None   # [T] oldest window position a row may attend (default 0)
    engram_ids: Optional[np.ndarray] = None   # [T, tables, ids] int64 row ids of the hashed n-gram memory
    engram_recent: Optional[np.ndarray] = None  # [T, ngram-1] int32: tokens before the row's block, newest first
    blocks: Optional[list] = None          # (region, start, tokens) as given to build()

    META_ROWS = 7

    def attach_engram(self, cfg: ModelConfig, prevs: Sequence[Sequence[int]]) -> "StepPlan":
        """Hash every block's rows; ``prevs[i]`` are the (up to ngram-1) tokens right before block i."""
        from . import engram as EG
        md = EG.metadata_for(cfg)
        self.engram_ids = np.concatenate([EG.hash_positions(md, prev, list(t), start)
                                          for (region, start, t), prev in zip(self.blocks, prevs)]).astype(np.int64)
        return self

    def attach_recent(self, cfg: ModelConfig, prevs: Sequence[Sequence[int]]) -> "StepPlan":
        """Leave the hashing to the device (``tf_engram_hash`` at the start of the launch): record, for
        every row, the ngram-1 tokens right before its block (``prevs[i]``, oldest first; shorter at
        the start of a conversation), newest first and padded with the pad token."""
        return self._set_recent(self.recent_rows(cfg, [(len(t), prev) for (_, _, t), prev in zip(self.blocks, prevs)]))

    def _set_recent(self, rows: np.ndarray) -> "StepPlan":
        self.engram_recent = rows
        return self

    @staticmethod
    def recent_rows(cfg: ModelConfig, blocks: Sequence[Tuple[int, Sequence[int]]]) -> np.ndarray:
        """[(rows, previous tokens oldest first)] -> [sum rows, ngram-1] int32, newest first."""
        from . import engram as EG
        md = EG.metadata_for(cfg)
        n = md.ngram - 1
        out = []
        for rows, prev in blocks:
            rec = list(reversed(list(prev)[-n:]))
            rec += [md.pad_token] * (n - len(rec))
            out.append(np.tile(np.asarray(rec, dtype=np.int32), (rows, 1)))
        return np.concatenate(out)

    def meta_host(self, ratio: int) -> np.ndarray:
        """[META_ROWS, T] int32 block uploaded per launch: tokens, pos, region, first_row, last_pos,
        valid compressed entries, window floor."""
        mp = self.min_pos if self.min_pos is not None else np.zeros_like(self.pos)
        return np.stack([self.tokens, self.pos, self.region, self.first_row, self.last_pos,
                         (self.pos + 1) // ratio, mp]).astype(np.int32)

    @staticmethod
    def build(blocks: Sequence[Tuple[int, int, Sequence[int]]], logits: str = "all") -> "StepPlan":
        """blocks: (region, start position, tokens).  logits: "all" | "last" (last row per block)."""
        toks, pos, reg, first, last, lrows = [], [], [], [], [], []
        r0 = 0
        sizes = set()
        for region, start, t in blocks:
            n = len(t)
            sizes.add(n)
            toks += list(t)
            pos += list(range(start, start + n))
            reg += [region] * n
            first += [r0] * n
            last += [start + n - 1] * n
            lrows += list(range(r0, r0 + n)) if logits == "all" else [r0 + n - 1]
            r0 += n
        i32 = lambda a: np.asarray(a, dtype=np.int32)
        gr = sizes.pop() if len(sizes) == 1 else 1
        return StepPlan(i32(toks), i32(pos), i32(reg), i32(first), i32(last), i32(lrows), gr,
                        blocks=[(r, s, list(t)) for r, s, t in blocks])

    @property
    def T(self) -> int:
        return int(self.tokens.shape[0])


class Engine:
    SMALL_M = 32

    def __init__(self, cfg: ModelConfig, ecfg: EngineConfig, layers: List[LayerWeights],
                 embed: torch.Tensor, head: torch.Tensor, final_norm: torch.Tensor,
                 comm: Optional[Comm] = None, device="cuda", max_chunk: int = 0,
                 draft_layers: Optional[List[LayerWeights]] = None, draft_extra: Optional[dict] = None):
        self.cfg, self.ecfg = cfg, ecfg
        if ecfg.max_context > cfg.max_positions:
            raise ValueError(f"max_context {ecfg.max_context} exceeds the model's {cfg.max_positions} positions")
        self.comm = comm or LocalComm()
        self.world, self.rank = self.comm.world, self.comm.rank
        self.dev = torch.device(device)
        self.layers = layers
        self.draft_layers = draft_layers or []
        self.draft_extra = draft_extra or {}
        self.embed_w, self.head_w, self.final_norm = embed, head, final_norm
        native.lib()
        native.set_pdl(bool(getattr(ecfg, "pdl", False)))
        self.status = native.StatusWord(self.dev)
        r = cfg.rope
        self.freqs = oracle.rope_frequencies(r.dim, r.theta, r.factor, r.beta_fast, r.beta_slow,
                                             r.original_max_position).to(self.dev)
        self.cfreqs = oracle.rope_frequencies(r.dim, r.compress_theta, r.factor, r.beta_fast,
                                              r.beta_slow, r.original_max_position).to(self.dev)
        self.Hl = cfg.n_heads // self.world
        self.El = cfg.n_experts // self.world
        self.regions = ecfg.regions
        self.max_chunk = max_chunk or max(ecfg.prefill_widths)
        # the window ring holds every row of a chunk plus the window before it (a sequence-parallel
        # chunk spans all ranks' slices)
        self.ring = max(self.max_chunk, ecfg.sp_chunk_rows if self.world > 1 else 0) + 2 * cfg.window
        self.maxC = ecfg.max_context // cfg.compress_ratio + 8
        self.win_row, self.comp_row = cfg.window_kv_bytes, cfg.compressed_kv_bytes
        self.key_row = cfg.index_key_bytes
        nl = len(layers) + len(self.draft_layers)
        u8 = dict(dtype=torch.uint8, device=self.dev)
        self.win = torch.zeros(nl, self.regions, self.ring, self.win_row, **u8)
        self.src_slot = {l: i for i, l in enumerate(cfg.kv_source_layers)}
        ns = max(1, len(cfg.kv_source_layers))
        C = cfg.head_dim + cfg.index_dim
        self.comp = torch.zeros(ns, self.regions, self.maxC, self.comp_row, **u8)
        self.keys = torch.zeros(ns, self.regions, self.maxC, self.key_row, **u8)
        # position-addressed rings of open-group compressor inputs (largest ratio + 32 slots: csrc kCarrySpan)
        self.carry = torch.zeros(ns, self.regions, cfg.max_ratio + 32, 2 * C, dtype=torch.float32,
                                 device=self.dev)
        self._scratch: Dict[int, dict] = {}
        self._dq_cache: Dict[int, torch.Tensor] = {}
        self._side: Optional[torch.cuda.Stream] = None     # parallel branch for the shared expert (decode rows)
        # hashed n-gram memory, one entry per Engram layer: (table, wkv, q_weight, k_weight)
        self.engram: List[tuple] = self.draft_extra.get("engram", [])
        self.sp = None              # parallel.sp.SpPrefill: sequence-parallel prefill over the ranks
        self.after_prep = None      # hook run between the KV store and the indexer / attention of a layer
        self.big_gemm = None        # set by ops.bigpath when the tcgen05 path is attached
        self.symm = None            # SymmWorkspace: fused GEMV/combine + all-reduce over peer memory
        self.last_hidden: Optional[torch.Tensor] = None

    # -- construction helpers --------------------------------------------------------------
    @classmethod
    def from_weights(cls, cfg: ModelConfig, ecfg: EngineConfig, W: Dict[str, torch.Tensor],
                     comm: Optional[Comm] = None, device="cuda", roundtrip: Optional[dict] = None,
                     max_chunk: int = 0) -> "Engine":
        comm = comm or LocalComm()
        late = cfg.late_start if 0 < cfg.late_start < cfg.n_layers else cfg.n_layers
        layers = [prepare_layer(cfg, W, li, comm.rank, comm.world, device, roundtrip,
                                keep_full=ecfg.sp_prefill and li < late) for li in range(cfg.n_layers)]
        drafts, extra = [], {}
        if cfg.draft is not None and "mtp.0.main_proj.weight" in W:
            drafts = [prepare_layer(cfg, W, cfg.n_layers + j, comm.rank, comm.world, device, roundtrip)
                      for j in range(cfg.draft.layers)]
            mp = quant_fp8_device(W["mtp.0.main_proj.weight"].to(device))
            if roundtrip is not None:
                roundtrip["mtp.0.main_proj.weight"] = dequant_fp8(mp).cpu()
            extra = dict(main_proj=mp, enorm=W["mtp.0.enorm.weight"].to(device, torch.bfloat16),
                         hnorm=W["mtp.0.hnorm.weight"].to(device, torch.bfloat16))
            if cfg.draft.subset_rows and comm.world == 1 and cfg.hidden % 512 == 0 and cfg.draft.subset_rows % 128 == 0:
                # 4-bit vocabulary-subset head of the drafter: MXFP4 copy of the subset's head rows,
                # multiplied on the block-scaled tensor-core GEMV (one "expert" of subset_rows features)
                ids = W["mtp.head_subset.ids"].to(device, torch.int64)
                rows = W["head.weight"].to(device, torch.float32)[ids]
                pk, sc = quant_mxfp4_device(rows.unsqueeze(0))
                extra["head_mx"] = (pk.contiguous(), sc.contiguous(), ids)
                if roundtrip is not None:
                    roundtrip["mtp.head_subset.weight"] = dequant_mxfp4(pk[0], sc[0]).cpu()
            if cfg.draft.markov_rank:
                # low-rank bigram correction of the draft logits: embed replicated, head rows sharded
                Vm = cfg.vocab // comm.world
                mk = f"mtp.{cfg.draft.layers - 1}.markov_head"
                extra["markov_embed"] = W[f"{mk}.embed.weight"].to(device, torch.bfloat16).contiguous()
                extra["markov_head"] = W[f"{mk}.head.weight"][comm.rank * Vm:(comm.rank + 1) * Vm].to(
                    device, torch.bfloat16).contiguous()
            if cfg.draft.confidence_head:
                # stored bf16, widened to fp32 once (the reference does the same at load)
                extra["confidence"] = W[f"mtp.{cfg.draft.layers - 1}.confidence_head.proj.weight"].to(
                    device, torch.bfloat16).to(torch.float32).reshape(-1).contiguous()
        if cfg.hc_mult > 1:
            extra = dict(extra, hc_head=tuple(W[k].to(device, torch.float32).contiguous()
                                              for k in ("hc_head_fn", "hc_head_base", "hc_head_scale")))
        if cfg.engram is not None and cfg.engram.layers:
            # row-sharded tables in HBM (rows of other ranks read as zero and are summed in), the
            # projection replicated
            from . import engram as EG
            eg = []
            for e, l in enumerate(cfg.engram.layers):
                packed = EG.pack_rows(W[f"engram.{e}.table"].float())
                n = packed.shape[0]
                lo, hi = n * comm.rank // comm.world, n * (comm.rank + 1) // comm.world
                wkv = quant_fp8_device(W[f"layers.{l}.engram.wkv.weight"].to(device))
                if roundtrip is not None:
                    roundtrip[f"layers.{l}.engram.wkv.weight"] = dequant_fp8(wkv).cpu()
                eg.append((EG.EngramTable(packed[lo:hi], lo, device), wkv,
                           W[f"layers.{l}.engram.q_weight"].to(device, torch.bfloat16).contiguous(),
                           W[f"layers.{l}.engram.k_weight"].to(device, torch.bfloat16).contiguous()))
            extra = dict(extra, engram=eg)
        V = cfg.vocab
        Vl = V // comm.world
        embed = W["embed.weight"].to(device, torch.bfloat16).contiguous()
        head = W["head.weight"][comm.rank * Vl:(comm.rank + 1) * Vl].to(device, torch.bfloat16).contiguous()
        if roundtrip is not None:
            roundtrip["embed.weight"] = embed.float().cpu()
            roundtrip["head.weight"] = W["head.weight"].to(torch.bfloat16).float()
            for k, v in W.items():
                if k not in roundtrip:
                    roundtrip[k] = v.to(torch.bfloat16).float() if (v.dim() == 1 and v.is_floating_point()) else v
        return cls(cfg, ecfg, layers, embed, head, W["norm.weight"].to(device, torch.bfloat16), comm,
                   device, max_chunk, drafts, extra)

    @classmethod
    def random_init(cls, cfg: ModelConfig, ecfg: EngineConfig, comm: Optional[Comm] = None,
                    device="cuda", seed: int = 0, max_chunk: int = 0) -> "Engine":
        comm = comm or LocalComm()
        late = cfg.late_start if 0 < cfg.late_start < cfg.n_layers else cfg.n_layers
        layers = [random_layer(cfg, li, comm.rank, comm.world, device, seed, keep_full=ecfg.sp_prefill and li < late)
                  for li in range(cfg.n_layers)]
        drafts, extra = [], {}
        g = torch.Generator(device=device).manual_seed(seed + 7)
        d = cfg.hidden
        if cfg.draft is not None:
            drafts = [random_layer(cfg, cfg.n_layers + j, comm.rank, comm.world, device, seed)
                      for j in range(cfg.draft.layers)]
            mp = torch.randn(d, d * (1 + cfg.draft.condition_layers), generator=g, device=device,
                             dtype=torch.bfloat16) * cfg.init_std
            extra = dict(main_proj=quant_fp8_device(mp),
                         enorm=torch.ones(d, dtype=torch.bfloat16, device=device),
                         hnorm=torch.ones(d * cfg.draft.condition_layers, dtype=torch.bfloat16, device=device))
        Vl = cfg.vocab // comm.world
        embed = torch.randn(cfg.vocab, d, generator=g, device=device, dtype=torch.bfloat16) * cfg.init_std
        head = torch.randn(Vl, d, generator=g, device=device, dtype=torch.bfloat16) * cfg.init_std
        if cfg.draft is not None and Vl % 128 == 0:
            extra["head"] = quant_fp8_device(head)     # the draft reads an FP8 copy of the head
        if cfg.hc_mult > 1:
            m = cfg.hc_mult
            extra["hc_head"] = ((torch.randn(m, m * d, generator=g, device=device) * cfg.init_std).contiguous(),
                                torch.zeros(m, device=device), torch.ones(1, device=device))
        if cfg.draft is not None and cfg.draft.confidence_head:
            extra["confidence"] = (torch.randn(d + cfg.draft.markov_rank, generator=g, device=device)
                                   * (2.0 / math.sqrt(d))).contiguous()
        return cls(cfg, ecfg, layers, embed, head, torch.ones(d, dtype=torch.bfloat16, device=device),
                   comm, device, max_chunk, drafts, extra)

    # -- scratch -----------------------------------------------------------------------------
    def _bufs(self, T: int) -> dict:
        b = self._scratch.get(T)
        if b is not None:
            return b
        cfg, dev = self.cfg, self.dev
        d, Dh, Hl = cfg.hidden, cfg.head_dim, self.Hl
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        maxN = max(l.proj.q.shape[0] for l in self.layers + self.draft_layers)
        self.q_col = maxN                      # low-rank query: wq_b's output lands behind the fused projection
        if cfg.q_lora_rank:
            maxN += Hl * Dh
        npairs = T * cfg.topk
        nsplit = self._nsplit(T)
        big = T > self.SMALL_M and getattr(self, "big_moe_full", None) is not None
        Il = cfg.shared_inter * cfg.n_shared // self.world
        b = dict(
            meta=torch.zeros(StepPlan.META_ROWS, T, **i32),
            nvalid_m={r // cfg.compress_ratio: torch.zeros(T, **i32)
                      for r in set(cfg.compress_ratios) if r != cfg.compress_ratio},
            x=torch.zeros(T, d, dtype=torch.bfloat16, device=dev),
            h16=torch.zeros(T, d, dtype=torch.float16, device=dev),
            hb=torch.zeros(T, d, dtype=torch.bfloat16, device=dev),
            P=(torch.zeros(T, maxN, **f32) if not big else torch.zeros(T, maxN, dtype=torch.bfloat16, device=dev)),
            q=torch.zeros(T, Hl, Dh, dtype=torch.bfloat16, device=dev),
            iq=torch.zeros(T, cfg.index_heads, cfg.index_dim, dtype=torch.bfloat16, device=dev),
            iw=torch.zeros(T, cfg.index_heads, **f32),
            sel={s: torch.full((T, cfg.index_topk), -1, **i32) for s in cfg.index_source_layers},
            selcnt={s: torch.zeros(T, **i32) for s in cfg.index_source_layers},
            part_o=torch.zeros(T, nsplit, Hl, Dh, **f32),
            part_lse=torch.zeros(T, nsplit, Hl, **f32),
            a16=torch.zeros(T, Hl * Dh, dtype=torch.float16, device=dev),
            delta=torch.zeros(T, d, **f32),
            logits_r=torch.zeros(T, cfg.n_experts, **f32),
            ids=torch.zeros(T, cfg.topk, **i32),
            wts=torch.zeros(T, cfg.topk, **f32),
            g_expert=torch.zeros(self.El, **i32), g_start=torch.zeros(self.El, **i32),
            g_count=torch.zeros(self.El, **i32), n_groups=torch.zeros(1, **i32),
            sorted_pairs=torch.zeros(npairs, **i32), n_local=torch.zeros(1, **i32),
            act=torch.zeros(1 if big else npairs, cfg.moe_inter, dtype=torch.float16, device=dev),
            y_pair=torch.zeros(1 if big else npairs, d, **f32),
            s_act=torch.zeros(T, max(Il, 1), dtype=torch.float16, device=dev),
            s_y=torch.zeros(T, d, **f32),
        )
        if self._moe_mx_ok(T):
            # MXFP8 copies of the expert inputs for the block-scaled tensor-core GEMV
            u8 = dict(dtype=torch.uint8, device=dev)
            b.update(x8=torch.zeros(T, d, **u8), x8s=torch.zeros(T, d // 32, **u8),
                     a8=torch.zeros(npairs, cfg.moe_inter, **u8), a8s=torch.zeros(npairs, cfg.moe_inter // 32, **u8))
        m = cfg.hc_mult
        if m > 1:
            # the residual stream is m copies per row; b["x"] is their flat [T, m*d] view
            b["x"] = torch.zeros(T, m * d, dtype=torch.bfloat16, device=dev)
            b["x2"] = torch.zeros(T, m * d, dtype=torch.bfloat16, device=dev)
            b["e"] = torch.zeros(T, d, dtype=torch.bfloat16, device=dev)
            b["v"] = torch.zeros(T, d, dtype=torch.bfloat16, device=dev)
            b["coef"] = torch.zeros(T, native.lib().tf_hc_coef_bytes(), dtype=torch.uint8, device=dev)
        if cfg.q_lora_rank:
            b["qa16"] = torch.zeros(T, cfg.q_lora_rank, dtype=torch.float16, device=dev)
            b["qfull"] = torch.zeros(T, Hl * Dh, dtype=b["P"].dtype, device=dev)
        if cfg.o_groups:
            b["mid16"] = torch.zeros(T, (cfg.o_groups // self.world) * cfg.o_lora_rank, dtype=torch.float16, device=dev)
        if self.engram:
            ec = cfg.engram
            n_ids = (ec.ngram - 1) * ec.heads
            b["eg_ids"] = torch.zeros(len(ec.layers), T, n_ids, dtype=torch.int64, device=dev)
            b["eg_recent"] = torch.zeros(T, ec.ngram - 1, dtype=torch.int32, device=dev)
            b["eg_hash"] = False         # True: the launch hashes its own tokens on the device
            b["eg_rows16"] = torch.zeros(T, n_ids * ec.width, dtype=torch.float16, device=dev)
            b["eg_kv"] = torch.zeros(T, (m + 1) * d, dtype=torch.bfloat16, device=dev)
            if "x2" not in b:
                b["x2"] = torch.zeros(T, d, dtype=torch.bfloat16, device=dev)
        self._scratch[T] = b
        return b

    def _nsplit(self, T: int) -> int:
        if T > 64:
            return 1
        # decode: split the keys of a row over CTAs, at least 64 keys each, for about two CTAs per
        # SM over all rows (every CTA re-reads the row's queries, so finer splits cost more than
        # they spread: 17 splits of 128 keys beat 34 of 64 at 16 rows, measured)
        keys = self.cfg.window + self.cfg.index_topk
        sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        return max(1, min(64, -(-keys // 64), -(-2 * sms // T)))

    def scores_buffer(self, T: int, n: int, tiled: bool = False) -> torch.Tensor:
        """fp32 [T, width >= n] index scores.  ``tiled``: a view of ONE flat buffer of at most
        ``index_score_bytes`` shared by every tile shape (the tile height changes with the context
        length; a buffer per shape would pile up)."""
        width = -(-max(n, 1024) // 1024) * 1024
        if tiled:
            flat = self._scratch.get("scores_flat")
            if flat is None or flat.numel() < T * width:
                flat = torch.empty(max(T * width, self.ecfg.index_score_bytes // 4), dtype=torch.float32, device=self.dev)
                self._scratch["scores_flat"] = flat
            return flat[: T * width].view(T, width)
        key = ("scores", T)
        b = self._scratch.get(key)
        if b is None or b.shape[1] < n:
            b = torch.empty(T, width, dtype=torch.float32, device=self.dev)
            self._scratch[key] = b
        return b

    # -- linear dispatch ---------------------------------------------------------------------
    def _linear(self, x16: torch.Tensor, w: Fp8Weight, out: torch.Tensor, M: int,
                w3: Optional[Fp8Weight] = None) -> None:
        """out[:M] = x16[:M] @ W^T (f32/f16 out by dtype of ``out``); ``w3`` selects the dual
        SwiGLU form.  Rows beyond SMALL_M go through the tensor-core (tcgen05) GEMM."""
        N, K = w.q.shape
        okind = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[out.dtype]
        if M <= self.SMALL_M:
            native.call("tf_smallm_gemm", 0, w.q, w3.q if w3 else None, w.s, w3.s if w3 else None,
                        0, 0, K, K // 128, x16, x16.stride(0), out, out.stride(0), okind, N, K, M,
                        None, None, None, None, None, 1, 0, M, self.cfg.swiglu_limit)
            return
        if self.big_gemm is not None:
            self.big_gemm(self, x16, w, out, M, w3)
            return
        if not self.ecfg.reference_matmul:
            raise native.NativeError("more than %d rows need the tensor-core path: attach it with ops.bigpath.attach(engine)"
                                     % self.SMALL_M)
        # validation only (EngineConfig.reference_matmul): dequantised weights through torch.matmul
        wd = self._dequant_cached(w)
        y = x16[:M].float() @ wd.t()
        if w3 is not None:
            y = oracle.swiglu(y, x16[:M].float() @ self._dequant_cached(w3).t(), self.cfg.swiglu_limit)
        out[:M, : y.shape[1]] = y.to(out.dtype)

    def _dequant_cached(self, w: Fp8Weight) -> torch.Tensor:
        k = id(w)
        if k not in self._dq_cache:
            n, kk = w.q.shape
            self._dq_cache[k] = (w.q.float().view(n // 128, 128, kk // 128, 128)
                                 * w.s[:, None, :, None]).view(n, kk)
        return self._dq_cache[k]

    def _fused_ok(self, T: int) -> bool:
        """The fused all-reduce kernels take decode rows: every row needs its own owner CTA among the
        hidden / 32 column tiles."""
        return self.symm is not None and T <= self.SMALL_M and T <= self.cfg.hidden // 32

    def _allreduce(self, t: torch.Tensor) -> None:
        if self.world > 1:
            self.comm.all_reduce(t)

    # -- one layer ---------------------------------------------------------------------------
    def _layer(self, li: int, L: LayerWeights, T: int, b: dict, nmax: int, rpg: int, first: bool,
               next_norm: Optional[torch.Tensor] = None) -> None:
        """One decoder layer.  ``next_norm``: RMSNorm weight of the boundary that follows this layer
        (the next layer's attention norm, or the final norm); when the fused all-reduce is up it
        computes that boundary in its epilogue."""
        cfg = self.cfg
        d, Dh, Hl = cfg.hidden, cfg.head_dim, self.Hl
        pos, region, first_row, last_pos, nvalid = (b["meta"][i] for i in (1, 2, 3, 4, 5))
        # boundary: x += delta (previous sublayer); h = rmsnorm(x)
        hc = cfg.hc_mult > 1
        if first:
            b["pending"] = False
        if self.engram and li < cfg.n_layers and li in cfg.engram.layers:
            self._engram(cfg.engram.layers.index(li), L, T, b)
        self._boundary(L, "attn", T, b, want_hb=False)
        N = L.proj.q.shape[0]
        P = b["P"]
        self._linear(b["h16"], L.proj, P, T)
        o = L.offs
        q_off = o.get("q", -1)
        if cfg.q_lora_rank:
            # low-rank query: RMSNorm of the wq_a output, then this rank's heads through wq_b
            R = cfg.q_lora_rank
            qa = P[:T, o["qa"]:o["qa"] + R].float()
            qa = qa * torch.rsqrt(qa.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * L.q_norm.float()
            b["qa16"][:T].copy_(qa)
            q_off = self.q_col
            self._linear(b["qa16"], L.wq_b, P[:, q_off:q_off + Hl * Dh], T)
        slot = self.src_slot.get(li, 0)
        # the stream this layer writes (a source) or reads; the step metadata and ``nmax`` count
        # entries of the finest stream, a coarser one has 1 / mult as many
        ratio = cfg.ratio_of(li) if li < cfg.n_layers else cfg.compress_ratio
        mult = ratio // cfg.compress_ratio
        native.call("tf_attn_prep", P, 0 if P.dtype == torch.float32 else 1, P.stride(0), T, pos, region, first_row, last_pos, Hl, Dh,
                    cfg.rope.dim, self.freqs, self.cfreqs, L.kv_norm, cfg.rms_eps, b["q"], self.win[li],
                    self.win[li].stride(0), self.win_row, self.comp_row, self.key_row, self.ring,
                    q_off, o["kv"], o.get("cv", -1), o.get("cg", -1), o.get("iq", -1), o.get("iw", -1),
                    ratio, cfg.index_dim, cfg.index_heads, L.comp_norm,
                    self.carry[slot] if L.is_kv_source else None, self.carry.shape[2],
                    self.comp[slot] if L.is_kv_source else None,
                    self.keys[slot] if L.is_kv_source else None, self.maxC, b["iq"], b["iw"],
                    self.status.t)
        if self.after_prep is not None:
            self.after_prep(li, L, T, b)
        comp = None
        sel = selcnt = None
        if L.kv_source >= 0:
            sslot = self.src_slot[L.kv_source]
            comp = self.comp[sslot]
            if L.is_index_source:
                self._index(L, T, b, nmax // mult, rpg, sslot, li, b["meta"][5] if mult == 1 else b["nvalid_m"][mult])
            sel, selcnt = b["sel"][L.index_source], b["selcnt"][L.index_source]
        nsplit = b["part_o"].shape[1]
        native.call("tf_sparse_attention", b["q"], T, Hl, Dh, pos, region, b["meta"][6], self.win[li],
                    self.win[li].stride(0), self.win_row, self.ring, cfg.window, comp,
                    comp.stride(0) if comp is not None else 0, self.comp_row, sel,
                    cfg.index_topk, selcnt, self.maxC, 1.0 / math.sqrt(Dh), nsplit, b["part_o"],
                    b["part_lse"], L.sink, self.freqs, cfg.rope.dim, b["a16"], None, Hl * Dh,
                    self.status.t)
        fused = self._fused_ok(T)
        wo_in = b["a16"]
        if cfg.o_groups:
            # grouped low-rank output projection: block-diagonal wo_a per local head group, then wo_b
            G, R = cfg.o_groups // self.world, cfg.o_lora_rank
            per = Hl * Dh // G
            for g in range(G):
                self._linear(b["a16"][:, g * per:(g + 1) * per], L.wo_a[g], b["mid16"][:, g * R:(g + 1) * R], T)
            wo_in = b["mid16"]
        if hc:
            # the reduced sublayer output goes through the hc post-mix instead of a plain add
            if fused:
                self.symm.gemv_allreduce(L.wo, wo_in, T, None, b["delta"], self.status.t)
            else:
                self._linear(wo_in, L.wo, b["delta"], T)
                self._allreduce(b["delta"][:T])
            self._hc_post(T, b)
        elif fused:
            # WO projection + all-reduce + residual add in one kernel over peer memory
            # (and the FFN boundary: RMSNorm + f16 / bf16 / MXFP8 rows, in the same epilogue)
            self.symm.gemv_allreduce(L.wo, wo_in, T, b["x"], None, self.status.t,
                                     norm=self._epilogue_norm(b, L.ffn_norm))
            b["pending"] = False
            b["normed"] = True
        else:
            self._linear(wo_in, L.wo, b["delta"], T)
            self._allreduce(b["delta"][:T])
            b["pending"] = True
        # FFN boundary
        self._boundary(L, "ffn", T, b, want_hb=True)
        self._moe(L, T, b, next_norm)
        if hc:
            if not (fused and T <= self.SMALL_M):
                self._allreduce(b["delta"][:T])
            self._hc_post(T, b)
        elif not fused:
            self._allreduce(b["delta"][:T])
            b["pending"] = True

    def _engram_hash(self, T: int, b: dict) -> None:
        """Row ids of every Engram table from the tokens of this launch (the verification rows of a
        decode step carry proposals sampled inside the graph, which the host never sees)."""
        md = self._engram_md()
        ec = self.cfg.engram
        meta = b["meta"]
        native.call("tf_engram_hash", meta[0], meta[1], meta[3], b["eg_recent"], md["token_map"], self.cfg.vocab,
                    md["mult"], md["primes"], md["offsets"], b["eg_ids"], T, b["eg_ids"].stride(0), len(ec.layers),
                    ec.ngram, ec.heads, md["pad"], md["image"], self.status.t)

    def _engram_md(self) -> dict:
        md = getattr(self, "_eg_md", None)
        if md is None:
            from . import engram as EG
            h = EG.metadata_for(self.cfg)
            dev = self.dev
            as_i64 = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.uint64).view(np.int64)).to(dev)
            md = dict(token_map=as_i64(h.token_map), mult=as_i64(h.multipliers), primes=as_i64(h.primes),
                      offsets=as_i64(h.offsets), pad=h.pad_token, image=h.image_token)
            self._eg_md = md
        return md

    def _engram(self, e: int, L: LayerWeights, T: int, b: dict) -> None:
        """Hashed n-gram memory in front of an Engram layer: gather this rank's rows (others read as
        zero), sum over the ranks, project to (copies + 1) x hidden and gate into the residual copies
        (reference: src/engram_gpu.rs:40 Rows, :279 ownership reduction, :347 projection; gate
        kernels/core.cu:952)."""
        cfg = self.cfg
        d, m = cfg.hidden, cfg.hc_mult
        table, wkv, qw, kw = self.engram[e]
        if m == 1 and b.get("pending"):
            # fold the previous sublayer's output into the residual first
            native.call("tf_add_norm", b["x"], b["delta"], 0, d, L.attn_norm, b["h16"], None, None, None, T, d,
                        cfg.rms_eps)
            b["pending"] = False
        rows = table.lookup(b["eg_ids"][e, :T].reshape(-1))                  # [T * ids, 256] bf16
        if self.world > 1:
            self.comm.all_reduce(rows)                                       # disjoint ownership: exact
        b["eg_rows16"][:T].copy_(rows.view(T, -1))
        self._linear(b["eg_rows16"], wkv, b["eg_kv"], T)
        native.call("tf_engram_gate", b["x"], b["eg_kv"], qw, kw, b["x2"], T, m, d, cfg.rms_eps)
        b["x"], b["x2"] = b["x2"], b["x"]

    def _boundary(self, L: LayerWeights, br: str, T: int, b: dict, want_hb: bool) -> None:
        """Sublayer input: residual (+ pending sublayer output) -> RMSNorm, or with hc_mult > 1 the
        pre-mix collapse of the residual copies -> RMSNorm.  Fills b["h16"] (and b["hb"])."""
        cfg = self.cfg
        d = cfg.hidden
        norm_w = L.attn_norm if br == "attn" else L.ffn_norm
        if b.pop("normed", False):
            # the all-reduce that produced this residual already wrote the normalised rows
            b["x8_ready"] = "x8" in b
            return
        if cfg.hc_mult > 1:
            fn, base, scale = L.hc[br]
            native.call("tf_hc_prepare", b["x"], fn, base, scale, b["coef"], b["v"], norm_w, b["h16"],
                        b["hb"] if want_hb else None, T, cfg.hc_mult, d, cfg.sinkhorn_iters, cfg.hc_eps, cfg.rms_eps)
            return
        pc = b.pop("pending_combine", None)
        use_mx = br == "ffn" and "x8" in b
        b["x8_ready"] = use_mx
        if pc is not None or use_mx or T <= self.SMALL_M:
            # one launch: (deferred expert combine +) residual add + RMSNorm (+ the MXFP8 rows the
            # block-scaled expert GEMV reads); same arithmetic as the separate kernels
            shared, e_lo = (pc if pc is not None else (None, 0))
            native.call("tf_add_norm_fused", b["x"], b["delta"] if (pc is None and b.get("pending")) else None,
                        b["y_pair"] if pc is not None else None, b["ids"] if pc is not None else None,
                        b["wts"] if pc is not None else None, shared, cfg.topk, e_lo, e_lo + self.El, norm_w,
                        b["h16"], b["hb"] if want_hb else None, b["x8"] if use_mx else None,
                        b["x8s"] if use_mx else None, T, d, cfg.rms_eps)
            return
        native.call("tf_add_norm", b["x"], b["delta"] if b.get("pending") else None, 0, d, norm_w, b["h16"],
                    b["hb"] if want_hb else None, None, None, T, d, cfg.rms_eps)

    def _hc_post(self, T: int, b: dict) -> None:
        """New residual copies from the reduced sublayer output in b["delta"] and the coefficients of
        the boundary that fed the sublayer."""
        native.call("tf_hc_post", b["x"], b["delta"], b["coef"], b["x2"], T, self.cfg.hc_mult, self.cfg.hidden)
        b["x"], b["x2"] = b["x2"], b["x"]
        b["pending"] = False

    def _index(self, L: LayerWeights, T: int, b: dict, nmax: int, rows_per_group: int, sslot: int,
               li: int, nvalid: torch.Tensor) -> None:
        """``nmax`` / ``nvalid``: entries of THIS layer's compressed stream (largest over the rows /
        per row)."""
        cfg = self.cfg
        region = b["meta"][2]
        sel, selcnt = b["sel"][li], b["selcnt"][li]
        if nmax == 0:
            sel.fill_(-1)
            selcnt.zero_()
            return
        # two-level selection of long decode rows: the candidate source layer scores every key and
        # publishes its best blocks of 8; the index layers after it score only inside those blocks
        # (reference: src/candidates.rs:1-20, src/sparse_index.rs)
        tl_min, pub = self.ecfg.two_level_index_min, self.candidate_source
        two_level = (tl_min > 0 and pub >= 0 and T <= self.SMALL_M and nmax >= tl_min
                     and 0 < cfg.candidate_blocks * 8 < nmax)
        if two_level and li > pub and b.get("cand") is not None:
            from ..ops import two_level as TL
            ids, cnt = TL.consume(b["iq"], b["iw"], region, b["cand"], self.keys[sslot], self.keys[sslot].stride(0),
                                  self.key_row, T, cfg.index_heads, cfg.index_dim, cfg.index_topk)
            sel[:T].copy_(ids)
            selcnt[:T].copy_(cnt)
            return
        # rows scored per launch: all of them unless the fp32 score matrix would pass the limit
        # (whole scoring groups of one conversation's consecutive rows)
        rows_t = T
        width = -(-max(nmax, 1024) // 1024) * 1024
        if T > self.SMALL_M and T * width * 4 > self.ecfg.index_score_bytes:
            unit = max(rows_per_group, 32)
            rows_t = max(unit, (self.ecfg.index_score_bytes // (4 * width)) // unit * unit)
            rows_t = min(rows_t, T)
        # prefill rows with a large score matrix share the flat buffer (never captured in a graph);
        # decode rows keep a buffer per row count, whose address a captured graph may hold
        scores = self.scores_buffer(rows_t, nmax, tiled=rows_t < T or (T > self.SMALL_M and T * width * 4 > (64 << 20)))
        ks_min = self.ecfg.key_sharded_index_min
        if self.world > 1 and ks_min > 0 and T <= self.SMALL_M and nmax >= ks_min and not (two_level and li == pub):
            # every rank holds all index keys: split the scoring work by key range, gather the local
            # top-k (score, id) pairs and select the global top-k from them (identical result)
            from ..parallel import key_sharded as KS
            ids, cnt = KS.select(b["iq"], b["iw"], region, nvalid, self.keys[sslot], self.keys[sslot].stride(0),
                                 self.key_row, T, cfg.index_heads, cfg.index_dim, rows_per_group, scores, nmax,
                                 cfg.index_topk, self.rank, self.world, lambda t: self.comm.all_gather(t, dim=1))
            sel[:T].copy_(ids)
            selcnt[:T].copy_(cnt)
            return
        if rows_t < T:
            # long contexts: score and select a tile of rows at a time, so that the score matrix stays
            # within `index_score_bytes` whatever the context (a 1M-token context has 262,144 entries a row)
            Hi, Di = cfg.index_heads, cfg.index_dim
            for r0 in range(0, T, rows_t):
                n = min(rows_t, T - r0)
                native.call("tf_index_scores", b["iq"][r0:], b["iw"][r0:], region[r0:], nvalid[r0:], self.keys[sslot],
                            self.keys[sslot].stride(0), self.key_row, n, Hi, Di,
                            rows_per_group, scores, scores.stride(0), 0, nmax)
                native.call("tf_topk_select", scores, scores.stride(0), nvalid[r0:], cfg.index_topk, sel[r0:], selcnt[r0:],
                            None, 0, n)
            return
        native.call("tf_index_scores", b["iq"], b["iw"], region, nvalid, self.keys[sslot],
                    self.keys[sslot].stride(0), self.key_row, T, cfg.index_heads, cfg.index_dim,
                    rows_per_group, scores, scores.stride(0), 0, nmax)
        native.call("tf_topk_select", scores, scores.stride(0), nvalid, cfg.index_topk, sel, selcnt,
                    None, 0, T)
        if two_level and li == pub:
            from ..ops import two_level as TL
            b["cand"] = TL.publish(scores[:T, :nmax], nvalid, cfg.candidate_blocks, T)

    def memory_report(self) -> Dict[str, int]:
        """Bytes this engine holds on the device, by kind (reference: the allocation lines the
        reference logs at load, src/memory.rs / src/weights.rs): dense and expert weights, embeddings
        and heads, the KV state of all regions, and the per-row-count scratch allocated so far."""
        def nbytes(obj, seen) -> int:
            if isinstance(obj, torch.Tensor):
                key = (obj.untyped_storage().data_ptr(), obj.untyped_storage().nbytes())
                if key in seen:
                    return 0
                seen.add(key)
                return obj.untyped_storage().nbytes() if obj.is_cuda else 0
            if isinstance(obj, Fp8Weight):
                return nbytes(obj.q, seen) + nbytes(obj.s, seen) + (nbytes(obj.sfu, seen) if isinstance(obj.sfu, torch.Tensor) else 0)
            if isinstance(obj, (list, tuple)):
                return sum(nbytes(o, seen) for o in obj)
            if isinstance(obj, dict):
                return sum(nbytes(o, seen) for o in obj.values())
            if isinstance(obj, LayerWeights):
                return sum(nbytes(getattr(obj, f), seen) for f in obj.__dataclass_fields__)
            return 0
        seen: set = set()
        experts = dense = 0
        for L in list(self.layers) + list(self.draft_layers):
            for f in L.__dataclass_fields__:
                b = nbytes(getattr(L, f), seen)
                if f in ("ew1", "ew3", "ew2", "es1", "es3", "es2"):
                    experts += b
                else:
                    dense += b
        out = {"dense_weights": dense, "expert_weights": experts,
               "embeddings_and_heads": nbytes([self.embed_w, getattr(self, "head_w", None), self.draft_extra], seen),
               "kv_state": nbytes([self.win, self.comp, self.keys, self.carry], seen),
               "row_scratch": nbytes([self._scratch, getattr(self, "_buf_cache", None)], seen)}
        out["total"] = sum(out.values())
        return out

    @property
    def candidate_source(self) -> int:
        """The index source layer that publishes candidate blocks: the last one before the late
        group (the reference's layer 20), the first index source when there is no late group, -1
        when the model keeps no candidates."""
        cfg = self.cfg
        if cfg.candidate_blocks <= 0 or not cfg.index_source_layers:
            return -1
        if cfg.late_start <= 0:
            return cfg.index_source_layers[0]
        early = [l for l in cfg.index_source_layers if l < cfg.late_start]
        return early[-1] if early else -1

    def _epilogue_norm(self, b: dict, w: torch.Tensor) -> dict:
        """Boundary outputs the fused all-reduce writes from its epilogue (csrc/comm.cuh)."""
        mx = "x8" in b
        return dict(w=w, h16=b["h16"], hb=b["hb"], x8=b["x8"] if mx else None, x8s=b["x8s"] if mx else None,
                    eps=self.cfg.rms_eps)

    def _moe(self, L: LayerWeights, T: int, b: dict, next_norm: Optional[torch.Tensor] = None) -> None:
        cfg = self.cfg
        d, I = cfg.hidden, cfg.moe_inter
        scoring = 1 if cfg.scoring == "sqrtsoftplus" else 0
        side = None
        grouped = False            # True once the router launch has also grouped the pairs by expert
        if cfg.n_shared and T <= self.SMALL_M:
            # the shared expert depends only on the normalised input: run its two small GEMVs as a
            # parallel branch (second stream; a parallel branch of the step's CUDA graph) next to the
            # router and the routed experts, and join before the combine
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.dev)
            side = self._side
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._linear(b["h16"], L.sw1, b["s_act"], T, w3=L.sw3)
                self._linear(b["s_act"], L.sw2, b["s_y"], T)
        if T > self.SMALL_M and self.big_gemm is not None and cfg.n_experts % 128 == 0:
            # router logits of a prefill chunk on the tensor cores (bf16 x bf16), then top-k
            native.call("tf_gemm_tc", 0, b["hb"], d, L.gate, d, b["logits_r"], cfg.n_experts, T, cfg.n_experts,
                        d, None, 0, None, 0, 0, None, None, 0, self.status.t)
            native.call("tf_router_topk", b["logits_r"], L.gate_bias, L.gate_bias_vl, b["meta"][0], cfg.image_token,
                        b["ids"], b["wts"], T, cfg.n_experts, cfg.topk, scoring, 1 if cfg.renorm else 0, cfg.route_scale)
        elif T <= self.SMALL_M and cfg.n_experts % 32 == 0:
            # one warp per expert row over the bf16 gate matrix, then top-k
            e0 = self.rank * self.El
            native.call("tf_router_logits_small", b["hb"], d, L.gate, b["logits_r"], cfg.n_experts, T,
                        cfg.n_experts, d)
            native.call("tf_router_topk_group", b["logits_r"], L.gate_bias, L.gate_bias_vl, b["meta"][0],
                        cfg.image_token, b["ids"], b["wts"], T, cfg.n_experts,
                        cfg.topk, scoring, 1 if cfg.renorm else 0, cfg.route_scale, e0, e0 + self.El,
                        b["g_expert"], b["g_start"], b["g_count"], b["n_groups"], b["sorted_pairs"], b["n_local"])
            grouped = True
        else:
            native.call("tf_router", b["h16"], L.gate, L.gate_bias, L.gate_bias_vl, b["meta"][0], cfg.image_token,
                        b["logits_r"], b["ids"], b["wts"], T,
                        cfg.n_experts, d, cfg.topk, scoring, 1 if cfg.renorm else 0, cfg.route_scale)
        e_lo = self.rank * self.El
        npairs = T * cfg.topk
        if T <= self.SMALL_M:
            if not grouped:
                native.call("tf_route_group", b["ids"], npairs, e_lo, e_lo + self.El, b["g_expert"],
                            b["g_start"], b["g_count"], b["n_groups"], b["sorted_pairs"], b["n_local"])
            slots = min(self.El, npairs)
            if "x8" in b:
                # MXFP4 weights x MXFP8 activations on block-scaled tcgen05 MMAs: the tensor core
                # consumes nibbles and scales, the first launch hands the second its MXFP8 input
                if not b.get("x8_ready"):
                    native.call("tf_quant_rows_mx8", b["h16"], d, b["x8"], b["x8s"], T, d)
                native.call("tf_moe_gemv_mx", L.ew1, L.ew3, L.es1, L.es3, self.El, b["x8"], b["x8s"], T, None, I,
                            b["a8"], b["a8s"], I, d, cfg.topk, b["g_expert"], b["g_start"], b["g_count"],
                            b["n_groups"], b["sorted_pairs"], slots, cfg.swiglu_limit, 0, 0, T, self.status.t)
                native.call("tf_moe_gemv_mx", L.ew2, None, L.es2, None, self.El, b["a8"], b["a8s"], npairs,
                            b["y_pair"], d, None, None, d, I, 1, b["g_expert"], b["g_start"], b["g_count"],
                            b["n_groups"], b["sorted_pairs"], slots, 0.0, 0, 0, T, self.status.t)
            else:
                self._moe_small_f16(L, T, b, slots)
        elif getattr(self, "big_moe_full", None) is not None:
            self.big_moe_full(self, L, T, b)       # permute, grouped GEMMs, shared expert, combine
            return
        else:
            self._moe_large(L, T, b)
        self._moe_finish(L, T, b, side, next_norm)

    def _moe_mx_ok(self, T: int) -> bool:
        """Block-scaled tensor-core GEMV for the routed experts: up to 32 rows (16 or 32 accumulator
        columns), MXFP4 experts, widths in whole 512-input scale loads and 128-feature tiles."""
        cfg = self.cfg
        return (self.ecfg.moe_block_scaled and T <= 32 and cfg.expert_quant == "mxfp4"
                and cfg.hidden % 512 == 0 and cfg.moe_inter % 512 == 0)

    def _moe_small_f16(self, L: LayerWeights, T: int, b: dict, slots: int) -> None:
        """Register-fed form (f16 activations, nibbles unpacked on the CUDA cores): widths the
        tensor-core form does not tile."""
        cfg = self.cfg
        d, I = cfg.hidden, cfg.moe_inter
        native.call("tf_smallm_gemm", 1, L.ew1, L.ew3, L.es1, L.es3, I * (d // 2), I * (d // 32),
                    d // 2, d // 32, b["h16"], d, b["act"], I, 1, I, d, 0, b["g_expert"],
                    b["g_start"], b["g_count"], b["n_groups"], b["sorted_pairs"], cfg.topk, slots,
                    min(T, 16), cfg.swiglu_limit)
        native.call("tf_smallm_gemm", 1, L.ew2, None, L.es2, None, d * (I // 2), d * (I // 32),
                    I // 2, I // 32, b["act"], I, b["y_pair"], d, 0, d, I, 0, b["g_expert"],
                    b["g_start"], b["g_count"], b["n_groups"], b["sorted_pairs"], 1, slots,
                    min(T, 16), 0.0)

    def _moe_finish(self, L: LayerWeights, T: int, b: dict, side, next_norm: Optional[torch.Tensor] = None) -> None:
        """Join the shared-expert branch and combine (with the all-reduce when the fused kernel is up)."""
        cfg = self.cfg
        d = cfg.hidden
        e_lo = self.rank * self.El
        shared = None
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)       # join the shared-expert branch
            shared = b["s_y"]
        elif cfg.n_shared:
            self._linear(b["h16"], L.sw1, b["s_act"], T, w3=L.sw3)
            self._linear(b["s_act"], L.sw2, b["s_y"], T)
            shared = b["s_y"]
        if self._fused_ok(T):
            # expert combine + shared expert + all-reduce + residual add in one kernel
            hc = cfg.hc_mult > 1
            norm = self._epilogue_norm(b, next_norm) if (next_norm is not None and not hc) else None
            self.symm.combine_allreduce(b["y_pair"], b["ids"], b["wts"], shared, T, cfg.topk, e_lo,
                                        e_lo + self.El, None if hc else b["x"], b["delta"] if hc else None,
                                        self.status.t, norm=norm)
            b["pending"] = False
            b["normed"] = norm is not None
            return
        if b.get("defer_combine"):
            # the next layer's boundary sums the expert outputs itself (tf_add_norm_fused)
            b["pending_combine"] = (shared, e_lo)
            return
        native.call("tf_moe_combine", b["y_pair"], b["ids"], b["wts"], shared, b["delta"], T, d,
                    cfg.topk, e_lo, e_lo + self.El)

    def _moe_large(self, L: LayerWeights, T: int, b: dict) -> None:
        """Routed experts for a prefill chunk.  With the grouped tensor-core GEMM loaded this is a
        permute + two grouped launches; the staging path below loops over the active experts."""
        if getattr(self, "big_moe", None) is not None:
            self.big_moe(self, L, T, b)
            return
        if not self.ecfg.reference_matmul:
            raise native.NativeError("routed experts of more than %d rows need the tensor-core path: attach it with "
                                     "ops.bigpath.attach(engine)" % self.SMALL_M)
        cfg = self.cfg
        ids = b["ids"][:T].long()
        e_lo = self.rank * self.El
        h = b["h16"][:T].float()
        for e in range(self.El):
            m = ids == (e + e_lo)
            if not m.any():
                continue
            rows, js = m.nonzero(as_tuple=True)
            w1 = dequant_mxfp4(L.ew1[e], L.es1[e])
            w3 = dequant_mxfp4(L.ew3[e], L.es3[e])
            w2 = dequant_mxfp4(L.ew2[e], L.es2[e])
            a = oracle.swiglu(h[rows] @ w1.t(), h[rows] @ w3.t(), cfg.swiglu_limit).half().float()
            b["y_pair"][rows * cfg.topk + js] = a @ w2.t()

    # -- public ------------------------------------------------------------------------------
    def upload_plan(self, plan: StepPlan, b: dict) -> None:
        T = plan.T
        host = plan.meta_host(self.cfg.compress_ratio)
        b["meta"][:, :T].copy_(torch.from_numpy(host), non_blocking=True)
        if self.engram:
            if plan.engram_recent is not None:
                b["eg_recent"][:T].copy_(torch.from_numpy(plan.engram_recent), non_blocking=True)
                b["eg_hash"] = True
            elif plan.engram_ids is not None:
                # host-hashed ids, [tables, T, ids] on the device
                b["eg_ids"][:, :T].copy_(torch.from_numpy(np.ascontiguousarray(plan.engram_ids.transpose(1, 0, 2))),
                                         non_blocking=True)
                b["eg_hash"] = False
            else:
                raise ValueError("this model has Engram layers: the plan needs attach_recent() or attach_engram()")

    @staticmethod
    def plan_shape(plan: StepPlan, ratio: int) -> Tuple[int, int]:
        """(largest count of compressed entries any row may score, rows per scoring group): a
        scoring CTA serves consecutive rows of ONE conversation."""
        nmax = int((plan.pos.max() + 1) // ratio)
        T = plan.T
        if plan.group_rows == T:
            rpg = min(T, 32)
        else:
            rpg = plan.group_rows if plan.group_rows <= 32 else 1
        return nmax, rpg

    def forward(self, plan: StepPlan, need_logits: bool = True) -> Optional[torch.Tensor]:
        T = plan.T
        assert T <= self.max_chunk
        b = self._bufs(T)
        self.upload_plan(plan, b)
        nmax, rpg = self.plan_shape(plan, self.cfg.compress_ratio)
        rows = torch.from_numpy(plan.logit_rows).to(self.dev).long() if need_logits else None
        return self.run(T, b, nmax, rpg, rows)

    def run(self, T: int, b: dict, nmax: int, rpg: int, logit_rows: Optional[torch.Tensor],
            layer_lo: int = 0, layer_hi: Optional[int] = None, x_in: Optional[torch.Tensor] = None,
            x_patch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, local_logits: bool = False
            ) -> Optional[torch.Tensor]:
        """Launch layers [layer_lo, layer_hi) on rows whose metadata already sits in ``b['meta']``
        (no host work: this is what a CUDA graph captures).  ``x_in`` replaces the embedding as
        the input residual (late-group replay); the head runs only when the last layer does.
        ``local_logits``: return this rank's vocabulary columns [rows, vocab / world] instead of
        gathering the full rows (the chunked sampler works on the local columns)."""
        cfg = self.cfg
        layer_hi = len(self.layers) if layer_hi is None else layer_hi
        if self.engram and b.get("eg_hash"):
            self._engram_hash(T, b)
        b["cand"] = None               # candidate blocks are published and consumed within one launch
        if cfg.max_ratio != cfg.compress_ratio:
            # valid entries per row in the coarser streams (the metadata counts the finest one)
            for m, t in b["nvalid_m"].items():
                torch.div(b["meta"][5], m, rounding_mode="floor", out=t)
        if x_in is None:
            e = b["e"] if cfg.hc_mult > 1 else b["x"]
            native.call("tf_embed", b["meta"][0], self.embed_w, e, T, cfg.hidden, cfg.vocab, self.status.t)
            if x_patch is not None:
                # rows that stand for image tokens take the vision tower's features instead
                e.index_copy_(0, x_patch[0], x_patch[1].to(e.dtype))
            if cfg.hc_mult > 1:
                # every residual copy starts as the embedding (reference: kernels/core.cu:530-543)
                b["x"].view(T, cfg.hc_mult, cfg.hidden).copy_(e[:T, None, :].expand(T, cfg.hc_mult, cfg.hidden))
        else:
            b["x"][:T].copy_(x_in)
        b.pop("pending_combine", None)
        b.pop("normed", None)
        eg_layers = cfg.engram.layers if self.engram else ()
        fuse_norm = self._fused_ok(T) and cfg.hc_mult == 1
        for li in range(layer_lo, layer_hi):
            # decode rows on one GPU: leave the expert combine of this layer to the boundary kernel
            # of the next one (not before an Engram layer, which reads the folded residual first)
            b["defer_combine"] = (T <= self.SMALL_M and self.world == 1 and cfg.hc_mult == 1
                                  and li + 1 < layer_hi and (li + 1) not in eg_layers)
            nxt = None
            if fuse_norm:
                if li + 1 < layer_hi:
                    nxt = None if (li + 1) in eg_layers else self.layers[li + 1].attn_norm
                elif layer_hi == len(self.layers):
                    nxt = self.final_norm
            self._layer(li, self.layers[li], T, b, nmax, rpg, first=(li == layer_lo), next_norm=nxt)
        b["defer_combine"] = False
        if layer_hi < len(self.layers):
            return None
        return self._head(T, b, logit_rows, local=local_logits)

    def residual_rows(self, b: dict, rows: torch.Tensor) -> torch.Tensor:
        """Complete residual stream (x + pending sublayer output) of the given rows, bf16
        (with hc_mult > 1: the flat [rows, hc_mult * hidden] copies, which never carry a pending part)."""
        if self.cfg.hc_mult > 1 or not b.get("pending"):
            return b["x"][rows].clone()
        return (b["x"][rows].float() + b["delta"][rows]).to(torch.bfloat16)

    def _head(self, T: int, b: dict, rows: Optional[torch.Tensor], draft: bool = False,
              local: bool = False) -> Optional[torch.Tensor]:
        cfg = self.cfg
        d = cfg.hidden
        if cfg.hc_mult > 1:
            # final collapse of the residual copies with the head's own pre-mix weights
            # (reference: src/model_io.rs final hc combine)
            fn, base, scale = self.draft_extra["hc_head"]
            xh = b["x"][:T].view(T, cfg.hc_mult, d).float()
            flat = xh.reshape(T, -1)
            inv = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
            pre = torch.sigmoid((flat @ fn.t()) * inv * scale[0] + base) + cfg.hc_eps
            b["v"][:T].copy_((xh * pre[:, :, None]).sum(1))
            native.call("tf_add_norm", b["v"], None, 0, d, self.final_norm, b["h16"] if draft else None, b["hb"], None,
                        None, T, d, cfg.rms_eps)
            if not draft:
                self.last_hidden = xh.mean(1).to(torch.bfloat16)
        else:
            if not b.pop("normed", False):
                native.call("tf_add_norm", b["x"], b["delta"] if b.get("pending") else None, 0, d, self.final_norm,
                            b["h16"] if draft else None,
                            b["hb"], None, None, T, d, cfg.rms_eps)
            if not draft:
                self.last_hidden = b["x"]
        if rows is None:
            return None
        if draft and self.draft_extra.get("head_mx") is not None:
            return self._head_subset(b["h16"][rows].contiguous())
        if draft and self.draft_extra.get("head") is not None:
            hw = self.draft_extra["head"]
            Vl = hw.n
            h16 = b["h16"][rows].contiguous()
            logits = torch.empty(h16.shape[0], Vl, dtype=torch.float32, device=self.dev)
            self._linear(h16, hw, logits, h16.shape[0])
            return self.comm.all_gather(logits, dim=1) if (self.world > 1 and not local) else logits
        hsel = b["hb"][rows].contiguous()
        Vl = self.head_w.shape[0]
        n = hsel.shape[0]
        logits = torch.empty(n, Vl, dtype=torch.float32, device=self.dev)
        for r0 in range(0, n, self.SMALL_M):
            m = min(self.SMALL_M, n - r0)
            native.call("tf_smallm_gemm", 2, self.head_w, None, None, None, 0, 0, d * 2, 0,
                        hsel[r0:], d, logits[r0:], Vl, 0, Vl, d, m, None, None, None, None, None, 1, 0, m, 0.0)
        if self.world > 1 and not local:
            logits = self.comm.all_gather(logits, dim=1)
        return logits

    def _head_subset(self, h16: torch.Tensor) -> torch.Tensor:
        """Draft logits from the 4-bit subset head: MXFP8 rows x MXFP4 head rows on the block-scaled
        GEMV, scattered into a full-vocabulary row of -inf (the drafter proposes subset tokens only;
        reference: src/nvfp4_head.rs, a 4-bit head over 61 % of the vocabulary)."""
        pk, sc, ids = self.draft_extra["head_mx"]
        n, d, Vs = h16.shape[0], self.cfg.hidden, pk.shape[1]
        assert n <= 32
        st = self._scratch.get(("head_mx", n))
        if st is None:
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.dev)
            st = dict(x8=torch.zeros(n, d, dtype=torch.uint8, device=self.dev),
                      x8s=torch.zeros(n, d // 32, dtype=torch.uint8, device=self.dev),
                      ge=i32([0]), gs=i32([0]), gc=i32([n]), ng=i32([1]), sp=torch.arange(n, dtype=torch.int32, device=self.dev))
            self._scratch[("head_mx", n)] = st
        native.call("tf_quant_rows_mx8", h16, d, st["x8"], st["x8s"], n, d)
        y = torch.empty(n, Vs, dtype=torch.float32, device=self.dev)
        native.call("tf_moe_gemv_mx", pk, None, sc, None, 1, st["x8"], st["x8s"], n, y, Vs, None, None, Vs, d, 1,
                    st["ge"], st["gs"], st["gc"], st["ng"], st["sp"], 1, 0.0, 0, 0, n, self.status.t)
        logits = torch.full((n, self.cfg.vocab), float("-inf"), dtype=torch.float32, device=self.dev)
        logits.index_copy_(1, ids, y)
        return logits

    # -- draft head ---------------------------------------------------------------------------
    def draft_run(self, T: int, b: dict, hidden_prev: torch.Tensor, logit_rows: Optional[torch.Tensor],
                  local_logits: bool = False) -> Optional[torch.Tensor]:
        """Draft head on rows whose metadata sits in ``b['meta']``: the embedding of each row's token
        and the hidden state of the position before it are normalised, concatenated and projected
        to the model width, then run through the draft layer(s) and the FP8 copy of the vocabulary
        head (reference conditioning: src/dspark_conditioning.rs, main_proj [d, 3d])."""
        cfg = self.cfg
        d = cfg.hidden
        ex = self.draft_extra
        if "cat16" not in b:
            b["cat16"] = torch.zeros(T, 2 * d, dtype=torch.float16, device=self.dev)
            b["e16"] = torch.zeros(T, d, dtype=torch.float16, device=self.dev)
        native.call("tf_embed", b["meta"][0], self.embed_w, b["x"], T, d, cfg.vocab, self.status.t)
        native.call("tf_add_norm", b["x"], None, 0, d, ex["enorm"], b["e16"], None, None, None, T, d, cfg.rms_eps)
        native.call("tf_add_norm", hidden_prev, None, 0, d, ex["hnorm"], b["h16"], None, None, None, T, d,
                    cfg.rms_eps)
        b["cat16"][:, :d].copy_(b["e16"])
        b["cat16"][:, d:].copy_(b["h16"])
        self._linear(b["cat16"], ex["main_proj"], b["delta"], T)
        if cfg.hc_mult > 1:
            b["x"].view(T, cfg.hc_mult, d).copy_(b["delta"][:T, None, :].expand(T, cfg.hc_mult, d))
            b["pending"] = False
        else:
            b["x"].zero_()
            b["pending"] = True
        b["defer_combine"] = False
        b.pop("pending_combine", None)
        b.pop("normed", None)
        fuse_norm = self._fused_ok(T) and cfg.hc_mult == 1
        for j, L in enumerate(self.draft_layers):
            nxt = None
            if fuse_norm:
                nxt = self.draft_layers[j + 1].attn_norm if j + 1 < len(self.draft_layers) else self.final_norm
            self._layer(len(self.layers) + j, L, T, b, 0, 1, first=False, next_norm=nxt)
        if local_logits and ex.get("head_mx") is not None:
            raise ValueError("the vocabulary-subset draft head produces full rows: no local logits")
        logits = self._head(T, b, logit_rows, draft=True, local=local_logits)
        if logits is not None and "markov_head" in ex:
            logits = logits + self._markov_bias(T, b, local_logits)[logit_rows]
        return logits

    def draft_confidence(self, T: int, b: dict, j: int, g: int, ladder: torch.Tensor, conf: torch.Tensor,
                         cum: torch.Tensor, verify: torch.Tensor) -> None:
        """After ``draft_run`` of pass ``j``: the confidence of the proposal about to be sampled,
        ``conf[:, j]``, and the causal stopping rule (``verify``: proposals each conversation will have
        verified; ``csrc/confidence.cu``).  Features: the pass's residual stream before the final norm
        (the collapsed copies with hc_mult > 1) and the Markov embedding of the token it was fed."""
        cfg, ex = self.cfg, self.draft_extra
        x = b["v"] if cfg.hc_mult > 1 else b["x"]
        lat = b.get("mk_lat") if cfg.draft.markov_rank else None
        native.call("tf_draft_confidence", x, 1, x.stride(0), lat, cfg.draft.markov_rank, ex["confidence"], ladder,
                    ladder.numel(), j, g, conf, cum, verify, T, cfg.hidden)

    def _markov_bias(self, T: int, b: dict, local: bool = False) -> torch.Tensor:
        """Markov correction of the draft logits: bias[r, :] = head_m @ embed_m[token of row r], the
        token being the one the row was fed (the anchor or the previous proposal), fp32 (reference:
        src/dspark_markov.rs:886-971; kernels/core.cu:1110 ca_dspark_markov_embed, :1118
        ca_dspark_markov_local; rank-256 bf16 operands)."""
        cfg, ex = self.cfg, self.draft_extra
        r = cfg.draft.markov_rank
        hm = ex["markov_head"]
        if "mk_lat" not in b:
            b["mk_lat"] = torch.zeros(T, r, dtype=torch.bfloat16, device=self.dev)
            b["mk_bias"] = torch.zeros(T, hm.shape[0], dtype=torch.float32, device=self.dev)
        native.call("tf_embed", b["meta"][0], ex["markov_embed"], b["mk_lat"], T, r, cfg.vocab, self.status.t)
        Vl = hm.shape[0]
        for r0 in range(0, T, self.SMALL_M):
            m = min(self.SMALL_M, T - r0)
            native.call("tf_smallm_gemm", 2, hm, None, None, None, 0, 0, r * 2, 0, b["mk_lat"][r0:], r,
                        b["mk_bias"][r0:], Vl, 0, Vl, r, m, None, None, None, None, None, 1, 0, m, 0.0)
        return self.comm.all_gather(b["mk_bias"], dim=1) if (self.world > 1 and not local) else b["mk_bias"]
