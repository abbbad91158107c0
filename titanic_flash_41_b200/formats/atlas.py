"""Per-rank staged weight atlas: one ``atlas.bin`` of 256-byte-aligned tensor views and an
``atlas.json`` index with a SHA-256 per tensor and of the whole file, written once by
``stage`` and read back (digest-checked, optionally straight to a device) by ``load_staged``.
Tensors that the kernels want contiguous are grouped by allocation key (fused projection
inputs, shared w1/w3, routed experts) so one upload serves them (reference: src/weights.rs:369
select_views, :279 allocation_key, :672 stage, :736 load_staged, :625-669 device digest).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..config import ModelConfig
from .layout import RankPlan
from .safetensors import DTYPES, Checkpoint, CheckpointError

ALIGN = 256
CHUNK = 16 << 20


def allocation_key(name: str) -> Tuple[int, str]:
    """Sort key that keeps tensors used together adjacent in the atlas."""
    parts = name.split(".")
    layer = int(parts[1]) if parts[0] in ("layers", "mtp") and parts[1].isdigit() else -1
    base = (10_000 if parts[0] == "mtp" else 0) + layer
    if ".ffn.experts." in name:
        group = "2experts"
    elif ".ffn.shared_experts." in name:
        group = "1shared"
    elif ".attn." in name:
        group = "0attn"
    else:
        group = "3misc"
    return base, group + ":" + name


def stage(ck: Checkpoint, cfg: ModelConfig, plan: RankPlan, out_dir: str) -> Dict:
    """Write this rank's atlas.  Expert scale bytes above 247 are refused (the MXFP4 kernels keep
    headroom in the exponent; reference src/weights.rs:541)."""
    os.makedirs(out_dir, exist_ok=True)
    names = sorted((n for n, p in plan.entries.items() if p.kind in ("replicated", "shard", "expert_local")),
                   key=allocation_key)
    index, off = [], 0
    whole = hashlib.sha256()
    with open(os.path.join(out_dir, "atlas.bin.tmp"), "wb") as f:
        for n in names:
            p, t = plan.entries[n], ck.tensors[n]
            if p.kind == "shard":
                data = ck.read_slice(n, p.start, p.length, p.axis)
            else:
                data = ck.read(n)
            raw = data.contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
            if t.dtype == "F8_E8M0" and ".ffn.experts." in n and raw and max(raw) > 247:
                raise CheckpointError(f"{n}: expert scale byte above 247")
            pad = (-off) % ALIGN
            f.write(b"\0" * pad)
            whole.update(b"\0" * pad)
            off += pad
            f.write(raw)
            whole.update(raw)
            index.append({"name": n, "dtype": t.dtype, "shape": list(data.shape), "offset": off, "bytes": len(raw),
                          "sha256": hashlib.sha256(raw).hexdigest()})
            off += len(raw)
    os.replace(os.path.join(out_dir, "atlas.bin.tmp"), os.path.join(out_dir, "atlas.bin"))
    meta = {"version": 1, "rank": plan.rank, "world": plan.world, "model": cfg.digest(), "bytes": off,
            "sha256": whole.hexdigest(), "tensors": index}
    with open(os.path.join(out_dir, "atlas.json"), "w") as f:
        json.dump(meta, f)
    return meta


def load_staged(out_dir: str, cfg: Optional[ModelConfig] = None, device=None, verify: bool = True
                ) -> Dict[str, torch.Tensor]:
    meta = json.load(open(os.path.join(out_dir, "atlas.json")))
    if cfg is not None and meta["model"] != cfg.digest():
        raise CheckpointError("atlas was staged for a different model configuration")
    path = os.path.join(out_dir, "atlas.bin")
    if os.path.getsize(path) != meta["bytes"]:
        raise CheckpointError("atlas.bin has the wrong size")
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        for e in meta["tensors"]:
            f.seek(e["offset"])
            raw = f.read(e["bytes"])
            if verify and hashlib.sha256(raw).hexdigest() != e["sha256"]:
                raise CheckpointError(f"{e['name']}: digest mismatch in the staged atlas")
            t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(DTYPES[e["dtype"]][1]).reshape(e["shape"])
            out[e["name"]] = t.to(device) if device is not None else t
    return out


def device_digest(tensors: Dict[str, torch.Tensor]) -> str:
    """Digest of what actually sits on the device (downloaded in name order)."""
    h = hashlib.sha256()
    for n in sorted(tensors):
        h.update(n.encode())
        h.update(tensors[n].detach().cpu().contiguous().view(torch.uint8).reshape(-1).numpy().tobytes())
    return h.hexdigest()
