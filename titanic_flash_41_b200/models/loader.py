"""Checkpoint <-> engine weights.

``export_checkpoint`` writes a weight dict (the oracle's names: stacked experts, plain fp32
matrices) as safetensors shards in the checkpoint contract (per-expert tensors, FP8 block scales,
packed FP4 + UE8M0), and ``checkpoint_weights`` reads such a checkpoint back into a dict that
``Engine.from_weights`` and ``OracleModel`` accept.  For block-128 FP8 and MXFP4 checkpoints,
re-quantising what was dequantised here is exact (the block grids line up), so the engine ends up
with the checkpoint's own bytes.  Dense weights stored with 32x32 UE8M0 scales are re-expressed on
the engine's 128x128 grid, which is NOT exact: values of sub-blocks whose scale is far below the
largest scale of their 128x128 block lose low bits.  The Engram row store travels in its packed
MXFP8 form (``layers.{l}.engram.embed.{weight,scale}``) and is exposed to the model as
``engram.{e}.table`` (reference: src/weights.rs:369-540 view selection and expert packing;
src/layout.rs:220-295).
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, Optional

import torch

from ..config import EngineConfig, ModelConfig
from ..formats import codecs
from ..formats.layout import expected_tensors, validate_checkpoint
from ..formats.safetensors import Checkpoint, write_safetensors


def export_checkpoint(W: Dict[str, torch.Tensor], cfg: ModelConfig, out_dir: str,
                      shard_bytes: int = 1 << 30) -> int:
    """Returns the number of shards written."""
    os.makedirs(out_dir, exist_ok=True)
    blk = 32 if cfg.dense_quant == "fp8_ue8m0_32" else 128
    shard, names, size, n_shards, wmap = {}, {}, 0, 0, {}

    def flush():
        nonlocal shard, names, size, n_shards
        if not shard:
            return
        n_shards += 1
        fn = f"model-{n_shards:05d}.safetensors"
        write_safetensors(os.path.join(out_dir, fn), shard, names)
        for k in shard:
            wmap[k] = fn
        shard, names, size = {}, {}, 0

    def put(name, t, dn=None):
        nonlocal size
        shard[name] = t.contiguous()
        if dn:
            names[name] = dn
        size += t.numel() * t.element_size()
        if size >= shard_bytes:
            flush()

    for name, dt, shape in expected_tensors(cfg):
        if name.endswith(".scale"):
            continue                                        # written with its weight
        stem = name[:-len(".weight")] if name.endswith(".weight") else name
        if name.endswith(".engram.embed.weight"):
            # the row store in its packed form: e4m3 values + one UE8M0 scale per 32
            from . import engram as EG
            e = cfg.engram.layers.index(int(name.split(".")[1]))
            packed = EG.pack_rows(W[f"engram.{e}.table"].float())
            put(name, packed[:, :cfg.engram.width].contiguous().view(torch.float8_e4m3fn))
            put(stem + ".scale", packed[:, cfg.engram.width:].contiguous(), "F8_E8M0")
            continue
        if ".ffn.experts." in name:
            pre, rest = name.split(".ffn.experts.")
            e, nm, _ = rest.split(".")
            w = W[f"{pre}.ffn.experts.{nm}.weight"][int(e)].float()
            if dt == "I8":
                pk, sc = codecs.mxfp4_quant(w)
                put(name, pk, "I8")
                put(stem + ".scale", sc, "F8_E8M0")
            else:
                put(name, w.bfloat16())
            continue
        w = W[name]
        if dt == "F8_E4M3":
            q, s = codecs.fp8_block_quant(w.float(), blk, cfg.dense_quant == "fp8_ue8m0_32")
            put(name, q)
            put(stem + ".scale", s, "F8_E8M0" if cfg.dense_quant == "fp8_ue8m0_32" else None)
        elif dt == "BF16":
            put(name, w.bfloat16())
        else:
            put(name, w.float())
    flush()
    import json
    json.dump({"weight_map": wmap}, open(os.path.join(out_dir, "model.safetensors.index.json"), "w"))
    return n_shards


def checkpoint_weights(ck: Checkpoint, cfg: ModelConfig, validate: bool = True) -> Dict[str, torch.Tensor]:
    """Dequantised fp32 weight dict with stacked experts."""
    if validate:
        validate_checkpoint(ck, cfg)
    blk = 32 if cfg.dense_quant == "fp8_ue8m0_32" else 128
    W: Dict[str, torch.Tensor] = {}
    experts: Dict[str, Dict[int, torch.Tensor]] = {}
    for name, dt, _ in expected_tensors(cfg):
        if name.endswith(".scale"):
            continue
        stem = name[:-len(".weight")] if name.endswith(".weight") else name
        if name.endswith(".engram.embed.weight"):
            from . import engram as EG
            e = cfg.engram.layers.index(int(name.split(".")[1]))
            packed = torch.cat([ck.read(name).view(torch.uint8), ck.read(stem + ".scale").view(torch.uint8)], dim=1)
            W[f"engram.{e}.table"] = EG.unpack_rows(packed)
            continue
        if ".ffn.experts." in name:
            pre, rest = name.split(".ffn.experts.")
            e, nm, _ = rest.split(".")
            if dt == "I8":
                w = codecs.mxfp4_dequant(ck.read(name), ck.read(stem + ".scale"))
            else:
                w = ck.read(name).float()
            experts.setdefault(f"{pre}.ffn.experts.{nm}.weight", {})[int(e)] = w
        elif dt == "F8_E4M3":
            W[name] = codecs.fp8_block_dequant(ck.read(name), ck.read(stem + ".scale"), blk)
        else:
            W[name] = ck.read(name).float()
    for k, d in experts.items():
        W[k] = torch.stack([d[i] for i in range(len(d))])
    return W


def load_engine(ckpt_dir: str, cfg: ModelConfig, ecfg: EngineConfig, comm=None, device="cuda", max_chunk: int = 0):
    """Scan, validate and build an ``Engine`` shard for ``comm.rank``."""
    from .engine import Engine
    ck = Checkpoint.scan(ckpt_dir)
    return Engine.from_weights(cfg, ecfg, checkpoint_weights(ck, cfg), comm, device, max_chunk=max_chunk)
