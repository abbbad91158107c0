"""Streamed checkpoint loading: every tensor goes from the file straight into this rank's device
shard in its STORED format -- FP8 values with their block scales, packed FP4 nibbles with their
UE8M0 group scales, bf16 -- one layer at a time.  Nothing is dequantised to fp32 on the host and
the host never holds more than one layer (the dequantising path of ``models/loader.py`` needs the
whole model in fp32, which for the full-size experts is terabytes).

Reads are digest-checked: every tensor's bytes are hashed (SHA-256) while they pass through and the
digests are compared with the manifest when the source has one (the staged atlas,
``formats/atlas.py``) and recorded in ``report`` otherwise; routed-expert scale bytes above 247 are
refused (reference: src/weights.rs:498 load_prefixes, :541, :736 load_staged, :625-669 digests;
src/ordered_read.rs).

Dense weights stored with 32x32 UE8M0 scales (the reference's checkpoint format,
src/blockscaled.rs:21-87) are re-expressed on the device on the 128x128 grid the FP8 kernels
consume: the block's scale becomes the largest of its sixteen 32x32 scales and the other sub-blocks'
values are shifted down by their power-of-two ratio.  That is exact while the shifted value stays
representable in e4m3 and rounds to nearest below that (a sub-block more than 2^6 below its
neighbours loses low bits): NOT a bit-exact transcription.
"""
from __future__ import annotations

import hashlib
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..config import EngineConfig, ModelConfig
from ..formats import codecs
from ..formats.layout import RankPlan, confidence_name, markov_prefix, validate_checkpoint
from ..formats.safetensors import Checkpoint, CheckpointError
from . import engine as E

F8 = torch.float8_e4m3fn


class CheckpointSource:
    """Rank-local stored tensors read from safetensors shards, sliced as the rank plan says."""

    def __init__(self, ck: Checkpoint, cfg: ModelConfig, rank: int, world: int, moe_parallel: str = "ep"):
        self.ck, self.cfg, self.rank, self.world = ck, cfg, rank, world
        self.plan = RankPlan.build(ck, cfg, rank, world, moe_parallel)
        self.report: Dict[str, str] = {}          # tensor name -> sha256 of the bytes this rank loaded
        self.peak_host_bytes = 0
        self._live = 0

    def has(self, name: str) -> bool:
        return name in self.ck.tensors

    def _account(self, name: str, t: torch.Tensor) -> torch.Tensor:
        raw = t.contiguous().view(torch.uint8).reshape(-1)
        self.report[name] = hashlib.sha256(raw.numpy().tobytes()).hexdigest()
        if self.ck.tensors[name].dtype == "F8_E8M0" and ".ffn.experts." in name and raw.numel() and int(raw.max()) > 247:
            raise CheckpointError(f"{name}: expert scale byte above 247")
        self._live += raw.numel()
        self.peak_host_bytes = max(self.peak_host_bytes, self._live)
        return t

    def release(self) -> None:
        """The caller has uploaded what it read (end of a layer)."""
        self._live = 0

    def get(self, name: str) -> torch.Tensor:
        """This rank's part of ``name`` as the rank plan places it."""
        p = self.plan.entries[name]
        if p.kind == "shard":
            return self._account(name, self.ck.read_slice(name, p.start, p.length, p.axis))
        if p.kind in ("replicated", "expert_local"):
            return self._account(name, self.ck.read(name))
        raise CheckpointError(f"{name}: not placed on rank {self.rank} ({p.kind})")

    def get_full(self, name: str) -> torch.Tensor:
        return self._account(name, self.ck.read(name))


class AtlasSource:
    """Rank-local stored tensors of a staged atlas (already sliced and digest-checked by
    ``formats.atlas.load_staged``)."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.t = tensors
        self.report: Dict[str, str] = {}
        self.peak_host_bytes = 0

    def has(self, name: str) -> bool:
        return name in self.t

    def get(self, name: str) -> torch.Tensor:
        return self.t[name]

    def get_full(self, name: str) -> torch.Tensor:
        raise CheckpointError("a staged atlas holds this rank's slices only")

    def release(self) -> None:
        pass


# ---------------------------------------------------------------------------------------------
def _pad_rows(t: torch.Tensor, mult: int) -> torch.Tensor:
    n = t.shape[0]
    pad = (-n) % mult
    if not pad:
        return t.contiguous()
    return torch.cat([t, torch.zeros(pad, *t.shape[1:], dtype=t.dtype, device=t.device)]).contiguous()


def dense_weight(q: torch.Tensor, s: torch.Tensor, device) -> E.Fp8Weight:
    """Stored dense matrix (e4m3 [n, k] + block scales) -> the engine's block-128 form on ``device``."""
    n, k = q.shape
    q = q.to(device)
    s = s.to(device)
    if s.dtype == torch.float32:                      # 128x128 fp32 scales: the kernels' own format
        qp = _pad_rows(q.view(torch.uint8), 128).view(F8)
        return E.Fp8Weight(qp, _pad_rows(s, 1).contiguous(), n, k)
    # 32x32 UE8M0 scales -> 128x128 fp32 scales (see the module header)
    if k % 128:
        raise CheckpointError("dense matrices need K in multiples of 128")
    qp = _pad_rows(q.view(torch.uint8), 128).view(F8)
    npad = qp.shape[0]
    s32 = torch.exp2(_pad_rows(s, 4).float() - 127.0)                          # [npad/32, k/32]
    s32 = s32[:, : k // 32]
    blk = s32.view(npad // 128, 4, k // 128, 4)
    s128 = blk.amax(dim=(1, 3))                                                # [npad/128, k/128]
    ratio = (blk / s128[:, None, :, None]).reshape(npad // 32, k // 32)        # powers of two <= 1
    vals = qp.float().view(npad // 32, 32, k // 32, 32) * ratio[:, None, :, None]
    q128 = vals.view(npad, k).clamp(-448, 448).to(F8)
    return E.Fp8Weight(q128.contiguous(), s128.contiguous(), n, k)


class _Getter:
    def __init__(self, src, device):
        self.src, self.dev = src, device

    def dense(self, stem: str, full: bool = False) -> E.Fp8Weight:
        get = self.src.get_full if full else self.src.get
        return dense_weight(get(stem + ".weight"), get(stem + ".scale"), self.dev)

    def raw(self, name: str, dtype=None) -> torch.Tensor:
        t = self.src.get(name).to(self.dev)
        return t.to(dtype) if dtype is not None else t


def _fuse(parts: List[Tuple[str, E.Fp8Weight]], k: int) -> Tuple[E.Fp8Weight, Dict[str, int]]:
    qs, ss, off, offs = [], [], 0, {}
    for nm, fw in parts:
        offs[nm] = off
        off += fw.q.shape[0]
        qs.append(fw.q)
        ss.append(fw.s)
    return E.Fp8Weight(torch.cat(qs).contiguous(), torch.cat(ss).contiguous(), off, k), offs


def layer_from_stored(cfg: ModelConfig, src, li: int, rank: int, world: int, device, keep_full: bool = False
                      ) -> E.LayerWeights:
    """One layer's shard in the engine's formats, from stored tensors (no dequantisation)."""
    if cfg.dense_quant == "none" or cfg.expert_quant != "mxfp4":
        raise CheckpointError("streamed loading covers FP8 dense + MXFP4 expert checkpoints")
    p = E._layer_prefix(cfg, li)
    draft = li >= cfg.n_layers
    g = _Getter(src, device)
    d = cfg.hidden
    L = E.LayerWeights()
    L.is_kv_source = (not draft) and li in cfg.kv_source_layers
    L.is_index_source = (not draft) and li in cfg.index_source_layers
    L.kv_source = -1 if draft else cfg.kv_source_of(li)
    L.index_source = -1 if draft else cfg.index_source_of(li)
    parts: List[Tuple[str, E.Fp8Weight]] = []
    if cfg.q_lora_rank:
        parts.append(("qa", g.dense(f"{p}.attn.wq_a")))
        L.wq_b = g.dense(f"{p}.attn.wq_b")                       # rows of this rank's heads
        L.q_norm = g.raw(f"{p}.attn.q_norm.weight", torch.bfloat16)
    else:
        parts.append(("q", g.dense(f"{p}.attn.wq")))
    parts.append(("kv", g.dense(f"{p}.attn.wkv")))
    if L.is_kv_source:
        parts += [("cv", g.dense(f"{p}.attn.compressor.wkv")), ("cg", g.dense(f"{p}.attn.compressor.wgate"))]
    if L.is_index_source:
        parts += [("iq", g.dense(f"{p}.attn.indexer.wq")), ("iw", g.dense(f"{p}.attn.indexer.weights_proj"))]
    L.proj, L.offs = _fuse(parts, d)
    if cfg.o_groups:
        G, R = cfg.o_groups // world, cfg.o_lora_rank
        woa = g.dense(f"{p}.attn.wo_a")                          # this rank's G groups of R rows
        L.wo_a = [E.Fp8Weight(woa.q[i * R:(i + 1) * R].contiguous(), woa.s[i * R // 128:(i + 1) * R // 128].contiguous(),
                              R, woa.k) for i in range(G)]
        L.wo = g.dense(f"{p}.attn.wo_b")
    else:
        L.wo = g.dense(f"{p}.attn.wo")
    if cfg.hc_mult > 1:
        L.hc = {br: tuple(g.raw(f"{p}.hc_{br}_{k}", torch.float32).contiguous() for k in ("fn", "base", "scale"))
                for br in ("attn", "ffn")}
    L.attn_norm = g.raw(f"{p}.attn_norm.weight", torch.bfloat16)
    L.ffn_norm = g.raw(f"{p}.ffn_norm.weight", torch.bfloat16)
    L.kv_norm = g.raw(f"{p}.attn.kv_norm.weight", torch.bfloat16)
    if L.is_kv_source:
        L.comp_norm = g.raw(f"{p}.attn.compressor.norm.weight", torch.bfloat16)
    if cfg.attn_sink:
        L.sink = g.raw(f"{p}.attn.attn_sink", torch.float32).contiguous()
    L.gate = g.raw(f"{p}.ffn.gate.weight", torch.bfloat16).contiguous()
    if cfg.router_bias:
        L.gate_bias = g.raw(f"{p}.ffn.gate.bias", torch.float32)
        if cfg.router_bias_vl and src.has(f"{p}.ffn.gate.bias_vl"):
            L.gate_bias_vl = g.raw(f"{p}.ffn.gate.bias_vl", torch.float32)
    El = cfg.n_experts // world
    for nm in ("w1", "w3", "w2"):
        pk = torch.stack([src.get(f"{p}.ffn.experts.{rank * El + e}.{nm}.weight").view(torch.uint8) for e in range(El)])
        sc = torch.stack([src.get(f"{p}.ffn.experts.{rank * El + e}.{nm}.scale").view(torch.uint8) for e in range(El)])
        setattr(L, "e" + nm, pk.to(device).contiguous())
        setattr(L, "es" + nm[1], sc.to(device).contiguous())
    if cfg.n_shared:
        L.sw1, L.sw3, L.sw2 = (g.dense(f"{p}.ffn.shared_experts.{nm}") for nm in ("w1", "w3", "w2"))
    if keep_full and world > 1 and not cfg.q_lora_rank and not cfg.o_groups and not draft:
        F = E.LayerWeights()
        F.proj, F.offs = _fuse([("q", g.dense(f"{p}.attn.wq", full=True))] + parts[1:], d)
        F.wo = g.dense(f"{p}.attn.wo", full=True)
        if cfg.attn_sink:
            F.sink = src.get_full(f"{p}.attn.attn_sink").to(device, torch.float32).contiguous()
        if cfg.n_shared:
            F.sw1, F.sw3, F.sw2 = (g.dense(f"{p}.ffn.shared_experts.{nm}", full=True) for nm in ("w1", "w3", "w2"))
        for nm in ("attn_norm", "ffn_norm", "kv_norm", "comp_norm", "gate", "gate_bias", "gate_bias_vl", "ew1", "ew3",
                   "ew2", "es1", "es3", "es2", "is_kv_source", "is_index_source", "kv_source", "index_source"):
            setattr(F, nm, getattr(L, nm))
        L.full = F
    src.release()
    return L


def engine_from_stored(cfg: ModelConfig, ecfg: EngineConfig, src, comm=None, device="cuda", max_chunk: int = 0):
    """Build this rank's ``Engine`` layer by layer from a stored-format source."""
    from ..parallel.comm import LocalComm
    comm = comm or LocalComm()
    rank, world = comm.rank, comm.world
    late = cfg.late_start if 0 < cfg.late_start < cfg.n_layers else cfg.n_layers
    can_full = isinstance(src, CheckpointSource)
    layers = [layer_from_stored(cfg, src, li, rank, world, device, keep_full=ecfg.sp_prefill and can_full and li < late)
              for li in range(cfg.n_layers)]
    g = _Getter(src, device)
    drafts, extra = [], {}
    if cfg.draft is not None and src.has("mtp.0.main_proj.weight"):
        drafts = [layer_from_stored(cfg, src, cfg.n_layers + j, rank, world, device) for j in range(cfg.draft.layers)]
        extra = dict(main_proj=g.dense("mtp.0.main_proj"), enorm=g.raw("mtp.0.enorm.weight", torch.bfloat16),
                     hnorm=g.raw("mtp.0.hnorm.weight", torch.bfloat16))
        if cfg.draft.markov_rank:
            mk = markov_prefix(cfg)
            extra["markov_embed"] = g.raw(f"{mk}.embed.weight", torch.bfloat16).contiguous()
            extra["markov_head"] = g.raw(f"{mk}.head.weight", torch.bfloat16).contiguous()      # this rank's vocabulary rows
        if cfg.draft.confidence_head:
            extra["confidence"] = g.raw(confidence_name(cfg), torch.bfloat16).to(torch.float32).reshape(-1).contiguous()
    if cfg.hc_mult > 1:
        extra = dict(extra, hc_head=tuple(g.raw(k, torch.float32).contiguous()
                                          for k in ("hc_head_fn", "hc_head_base", "hc_head_scale")))
    if cfg.engram is not None and cfg.engram.layers:
        from . import engram as EG
        eg = []
        for l in cfg.engram.layers:
            vals = src.get(f"layers.{l}.engram.embed.weight").view(torch.uint8)     # this rank's rows, packed MXFP8
            scl = src.get(f"layers.{l}.engram.embed.scale").view(torch.uint8)
            lo = src.plan.entries[f"layers.{l}.engram.embed.weight"].start if hasattr(src, "plan") else 0
            if not can_full and world > 1:
                raise CheckpointError("the Engram projection is kept whole on every rank: load from the checkpoint")
            eg.append((EG.EngramTable(torch.cat([vals, scl], dim=1).contiguous(), lo, device),
                       g.dense(f"layers.{l}.engram.wkv", full=can_full),
                       g.raw(f"layers.{l}.engram.q_weight", torch.bfloat16).contiguous(),
                       g.raw(f"layers.{l}.engram.k_weight", torch.bfloat16).contiguous()))
            src.release()
        extra = dict(extra, engram=eg)
    if not can_full and world > 1:
        raise CheckpointError("the embedding is kept whole on every rank: load from the checkpoint, not from a rank's atlas")
    embed = (src.get_full("embed.weight") if can_full else src.get("embed.weight")).to(device, torch.bfloat16).contiguous()
    head = g.raw("head.weight", torch.bfloat16).contiguous()
    norm = g.raw("norm.weight", torch.bfloat16)
    src.release()
    eng = E.Engine(cfg, ecfg, layers, embed, head, norm, comm, device, max_chunk, drafts, extra)
    eng.load_report = {"tensors": len(src.report), "peak_host_bytes": src.peak_host_bytes, "sha256": src.report}
    return eng


def load_engine(ckpt_dir: str, cfg: ModelConfig, ecfg: EngineConfig, comm=None, device="cuda", max_chunk: int = 0):
    """Scan and validate a safetensors checkpoint, then stream this rank's shard onto the device."""
    from ..parallel.comm import LocalComm
    comm = comm or LocalComm()
    ck = Checkpoint.scan(ckpt_dir)
    validate_checkpoint(ck, cfg)
    return engine_from_stored(cfg, ecfg, CheckpointSource(ck, cfg, comm.rank, comm.world, ecfg.moe_parallel), comm, device,
                              max_chunk)
