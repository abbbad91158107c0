"""Rank plan: which slice of which checkpoint tensor a rank holds, and the shape contract of a
checkpoint for a given ``ModelConfig``.

Placement rules (reference: src/layout.rs:57-144 classify): embed / head rows, q heads (wq or
wq_b rows), attention sinks, wo_a rows, Engram wkv rows, w1 / w3 rows of the shared expert are
split on axis 0; wo / wo_b and shared w2 on axis 1 (K); routed experts are either split whole
("ep": expert e lives on rank e // (E / world)) or column-sliced like the shared expert ("tp",
the reference's layout); compressor / indexer tensors exist only at their source layers; the
rest is replicated.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

from ..config import ModelConfig
from .safetensors import Checkpoint, CheckpointError


@dataclass
class Placement:
    kind: str               # "replicated" | "shard" | "omitted" | "expert_local" | "expert_remote"
    axis: int = 0
    start: int = 0
    length: int = 0
    reason: str = ""


def _split(n: int, rank: int, world: int, axis: int) -> Placement:
    if n % world:
        raise CheckpointError(f"extent {n} does not divide by {world} ranks")
    return Placement("shard", axis, rank * (n // world), n // world)


_EXPERT = re.compile(r"\.ffn\.experts\.(\d+)\.")


def classify(name: str, shape: Tuple[int, ...], cfg: ModelConfig, rank: int, world: int,
             moe_parallel: str = "ep") -> Placement:
    if name in ("embed.weight", "head.weight") or re.fullmatch(r"mtp\.\d+\.markov_head\.head\.weight", name):
        # vocabulary rows; the Markov head of the last draft stage is split like the head, its
        # embedding (latents) stays whole on every rank (reference: src/layout.rs:86)
        return _split(shape[0], rank, world, 0)
    m = re.match(r"(?:layers|mtp)\.(\d+)\.", name)
    layer = int(m.group(1)) if m else None
    if layer is not None:
        if name.startswith("layers.") and layer >= cfg.n_layers:
            raise CheckpointError(f"{name}: unknown target layer")
        if name.startswith("layers.") and ".attn.compressor." in name and layer not in cfg.kv_source_layers:
            return Placement("omitted", reason="non-source compressor is not part of the graph")
        if name.startswith("layers.") and ".attn.indexer." in name and layer not in cfg.index_source_layers:
            return Placement("omitted", reason="the shared sparse source owns these tensors")
    if layer is not None:
        if ".engram.embed." in name:
            n = shape[0]
            a, b = n * rank // world, n * (rank + 1) // world       # unequal last rows are fine
            return Placement("shard", 0, a, b - a)
        if any(k in name for k in (".engram.wkv.", ".attn.wq.", ".attn.wq_b.", ".attn.wo_a.")) or name.endswith(".attn.attn_sink"):
            return _split(shape[0], rank, world, 0)
        if ".attn.wo." in name or ".attn.wo_b." in name:
            return _split(shape[1], rank, world, 1)
        e = _EXPERT.search(name)
        if e and moe_parallel == "ep":
            per = cfg.n_experts // world
            return Placement("expert_local" if int(e.group(1)) // per == rank else "expert_remote")
        if e or ".ffn.shared_experts." in name:
            if ".w1." in name or ".w3." in name:
                return _split(shape[0], rank, world, 0)
            if ".w2." in name:
                return _split(shape[1], rank, world, 1)
    return Placement("replicated")


def confidence_name(cfg: ModelConfig) -> str:
    """Tensor of the drafter's confidence head, owned by the last draft stage."""
    return f"mtp.{cfg.draft.layers - 1}.confidence_head.proj.weight"


def markov_prefix(cfg: ModelConfig) -> str:
    """Tensor-name prefix of the Markov correction head: it belongs to the last draft stage."""
    return f"mtp.{cfg.draft.layers - 1}.markov_head"


def comp_width(cfg: ModelConfig) -> int:
    """Output width of the compressor projections: the pooled latent plus the pooled index key."""
    return cfg.head_dim + cfg.index_dim


def expected_tensors(cfg: ModelConfig) -> List[Tuple[str, str, Tuple[int, ...]]]:
    """(name, dtype, shape) of every tensor a checkpoint of this geometry must contain
    (reference: src/layout.rs:220-295 validate_target_weights)."""
    d, H, Dh = cfg.hidden, cfg.n_heads, cfg.head_dim
    blk = 32 if cfg.dense_quant == "fp8_ue8m0_32" else 128
    sdt = "F8_E8M0" if cfg.dense_quant == "fp8_ue8m0_32" else "F32"
    out = [("embed.weight", "BF16", (cfg.vocab, d)), ("head.weight", "BF16", (cfg.vocab, d)),
           ("norm.weight", "BF16", (d,))]

    def dense(name, n, k):
        if cfg.dense_quant == "none":
            out.append((name + ".weight", "BF16", (n, k)))
        else:
            out.append((name + ".weight", "F8_E4M3", (n, k)))
            out.append((name + ".scale", sdt, (-(-n // blk), -(-k // blk))))

    n_draft = cfg.draft.layers if cfg.draft is not None else 0
    if cfg.hc_mult > 1:
        # final collapse of the residual copies in front of the head (reference: src/model_io.rs)
        m = cfg.hc_mult
        out += [("hc_head_fn", "F32", (m, m * d)), ("hc_head_base", "F32", (m,)), ("hc_head_scale", "F32", (1,))]
    if n_draft and cfg.draft.subset_rows:
        # token ids of the drafter's 4-bit vocabulary-subset head (the rows themselves are cut from head.weight)
        out.append(("mtp.head_subset.ids", "I64", (cfg.draft.subset_rows,)))
    if n_draft and cfg.draft.markov_rank:
        # Markov correction of the draft logits, owned by the LAST draft stage (reference:
        # mtp.2.markov_head.{embed,head}.weight, src/layout.rs:362): embedding replicated, head rows
        # split like the vocabulary head
        mk = markov_prefix(cfg)
        out.append((f"{mk}.embed.weight", "BF16", (cfg.vocab, cfg.draft.markov_rank)))
        out.append((f"{mk}.head.weight", "BF16", (cfg.vocab, cfg.draft.markov_rank)))
    if n_draft and cfg.draft.confidence_head:
        # one row over [hidden state of the draft pass ; Markov embedding of the token it was fed]
        # (reference: mtp.2.confidence_head.proj.weight [1, 5376], src/layout.rs:367)
        out.append((confidence_name(cfg), "BF16", (1, d + cfg.draft.markov_rank)))
    if cfg.engram is not None and cfg.engram.layers:
        # hashed n-gram memory (reference: src/layout.rs:277-292, src/engram_gpu.rs:174-183): the row
        # store as MXFP8 (e4m3 values + one UE8M0 per 32), the projection, the gate weights
        from ..models import engram as EG
        rows = EG.table_rows(cfg)
        ids = (cfg.engram.ngram - 1) * cfg.engram.heads
        for l in cfg.engram.layers:
            out.append((f"layers.{l}.engram.embed.weight", "F8_E4M3", (rows, cfg.engram.width)))
            out.append((f"layers.{l}.engram.embed.scale", "F8_E8M0", (rows, cfg.engram.width // 32)))
            dense(f"layers.{l}.engram.wkv", (cfg.hc_mult + 1) * d, ids * cfg.engram.width)
            out.append((f"layers.{l}.engram.q_weight", "BF16", (cfg.hc_mult, d)))
            out.append((f"layers.{l}.engram.k_weight", "BF16", (cfg.hc_mult, d)))
    for l in range(cfg.n_layers + n_draft):
        draft = l >= cfg.n_layers
        p = f"mtp.{l - cfg.n_layers}" if draft else f"layers.{l}"
        if draft and l == cfg.n_layers:
            dense(f"{p}.main_proj", d, d * (1 + cfg.draft.condition_layers))
            out.append((f"{p}.enorm.weight", "BF16", (d,)))
            out.append((f"{p}.hnorm.weight", "BF16", (d * cfg.draft.condition_layers,)))
        for br in ("attn", "ffn"):
            out.append((f"{p}.{br}_norm.weight", "BF16", (d,)))
            if cfg.hc_mult > 1:
                m = cfg.hc_mult
                out += [(f"{p}.hc_{br}_fn", "F32", (m * (2 + m), m * d)), (f"{p}.hc_{br}_base", "F32", (m * (2 + m),)),
                        (f"{p}.hc_{br}_scale", "F32", (3,))]
        if cfg.q_lora_rank:
            dense(f"{p}.attn.wq_a", cfg.q_lora_rank, d)
            out.append((f"{p}.attn.q_norm.weight", "BF16", (cfg.q_lora_rank,)))
            dense(f"{p}.attn.wq_b", H * Dh, cfg.q_lora_rank)
        else:
            dense(f"{p}.attn.wq", H * Dh, d)
        dense(f"{p}.attn.wkv", Dh, d)
        out.append((f"{p}.attn.kv_norm.weight", "BF16", (Dh,)))
        if cfg.o_groups:
            dense(f"{p}.attn.wo_a", cfg.o_groups * cfg.o_lora_rank, H * Dh // cfg.o_groups)
            dense(f"{p}.attn.wo_b", d, cfg.o_groups * cfg.o_lora_rank)
        else:
            dense(f"{p}.attn.wo", d, H * Dh)
        if cfg.attn_sink:
            out.append((f"{p}.attn.attn_sink", "F32", (H,)))
        if not draft and l in cfg.kv_source_layers:
            dense(f"{p}.attn.compressor.wkv", comp_width(cfg), d)
            dense(f"{p}.attn.compressor.wgate", comp_width(cfg), d)
            out.append((f"{p}.attn.compressor.norm.weight", "BF16", (Dh,)))
        if not draft and l in cfg.index_source_layers:
            dense(f"{p}.attn.indexer.wq", cfg.index_heads * cfg.index_dim, d)
            dense(f"{p}.attn.indexer.weights_proj", cfg.index_heads, d)
        for e in range(cfg.n_experts):
            for nm, n, k in (("w1", cfg.moe_inter, d), ("w3", cfg.moe_inter, d), ("w2", d, cfg.moe_inter)):
                if cfg.expert_quant == "mxfp4":
                    out.append((f"{p}.ffn.experts.{e}.{nm}.weight", "I8", (n, k // 2)))
                    out.append((f"{p}.ffn.experts.{e}.{nm}.scale", "F8_E8M0", (n, k // 32)))
                else:
                    out.append((f"{p}.ffn.experts.{e}.{nm}.weight", "BF16", (n, k)))
        if cfg.n_shared:
            si = cfg.shared_inter * cfg.n_shared
            for nm, n, k in (("w1", si, d), ("w3", si, d), ("w2", d, si)):
                dense(f"{p}.ffn.shared_experts.{nm}", n, k)
        out.append((f"{p}.ffn.gate.weight", "BF16", (cfg.n_experts, d)))
        out.append((f"{p}.ffn.gate.bias", "F32", (cfg.n_experts,)))
        if cfg.router_bias_vl and not draft:
            # alternative selection bias used for image-token rows (reference: src/layout.rs:275)
            out.append((f"{p}.ffn.gate.bias_vl", "F32", (cfg.n_experts,)))
    return out


def validate_checkpoint(ck: Checkpoint, cfg: ModelConfig) -> None:
    for name, dt, shape in expected_tensors(cfg):
        ck.require(name, dt, shape)


@dataclass
class RankPlan:
    rank: int
    world: int
    entries: Dict[str, Placement]

    @staticmethod
    def build(ck: Checkpoint, cfg: ModelConfig, rank: int, world: int, moe_parallel: str = "ep") -> "RankPlan":
        return RankPlan(rank, world, {n: classify(n, t.shape, cfg, rank, world, moe_parallel)
                                      for n, t in ck.tensors.items()})

    def local_bytes(self, ck: Checkpoint) -> int:
        total = 0
        for n, p in self.entries.items():
            t = ck.tensors[n]
            if p.kind in ("replicated", "expert_local"):
                total += t.nbytes
            elif p.kind == "shard":
                total += t.nbytes * p.length // max(1, t.shape[p.axis])
        return total
