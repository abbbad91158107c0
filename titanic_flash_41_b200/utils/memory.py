"""Memory admission: every optional allocation (session images, host staging, disk-tier reads,
image inputs) is admitted against what is actually available minus a floor, and every rank must
take the same branch, so refusals are decided by an all-rank vote (``ControlChannel.all_admit``).

Host side reads MemAvailable and the cgroup limit; device side reads ``cudaMemGetInfo``.  On
B200 the two pools are separate (the reference admits everything against one unified pool):
images live in HBM while the device floor allows, then in pinned host memory, then on disk
(reference: src/memory.rs:112 floor_bytes, :167 InputCapacityError, :173 reserve_host_workspace,
:209 Available; src/cuda.rs:330-344 allocation_failure records).
"""
from __future__ import annotations

import json
import os
import sys
import threading
from dataclasses import dataclass
from typing import Callable, Optional

DEFAULT_HOST_FLOOR = 8 << 30
DEFAULT_DEVICE_FLOOR = 4 << 30


class CapacityError(MemoryError):
    """An input or cache allocation does not fit above the floor (HTTP 503 / cache refusal, not a crash)."""


def _read_int(path: str) -> Optional[int]:
    try:
        with open(path) as f:
            v = f.read().strip()
        return None if v in ("max", "") else int(v)
    except (OSError, ValueError):
        return None


def host_available(meminfo: str = "/proc/meminfo", cgroup: str = "/sys/fs/cgroup") -> int:
    """Bytes the process may still take: min(MemAvailable, cgroup limit - cgroup usage)."""
    avail = None
    try:
        with open(meminfo) as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    avail = int(line.split()[1]) * 1024
                    break
    except OSError:
        pass
    limit = _read_int(os.path.join(cgroup, "memory.max"))
    used = _read_int(os.path.join(cgroup, "memory.current"))
    if limit is not None and used is not None:
        room = max(0, limit - used)
        avail = room if avail is None else min(avail, room)
    return avail if avail is not None else 1 << 62


def device_available(device=None) -> int:
    import torch
    if not torch.cuda.is_available():
        return 0
    free, _ = torch.cuda.mem_get_info(device)
    return int(free)


@dataclass
class Reservation:
    owner: "Admission"
    nbytes: int
    released: bool = False

    def release(self) -> None:
        if not self.released:
            self.released = True
            with self.owner._lock:
                self.owner.reserved -= self.nbytes

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()
        return False


class Admission:
    """Admission against ``available() - floor - what is already reserved``."""

    def __init__(self, available: Callable[[], int], floor: int, name: str = "host",
                 log: Optional[Callable[[dict], None]] = None):
        self.available, self.floor, self.name = available, floor, name
        self.reserved = 0
        self._lock = threading.Lock()
        self.log = log or (lambda rec: sys.stderr.write(json.dumps(rec) + "\n"))

    def headroom(self) -> int:
        return self.available() - self.floor - self.reserved

    def fits(self, nbytes: int) -> bool:
        return nbytes <= self.headroom()

    def reserve(self, nbytes: int, what: str = "") -> Reservation:
        with self._lock:
            room = self.available() - self.floor - self.reserved
            if nbytes > room:
                self.log({"event": "allocation_refused", "pool": self.name, "what": what, "bytes": nbytes,
                          "headroom": room, "floor": self.floor})
                raise CapacityError(f"{what or 'allocation'} of {nbytes} bytes does not fit above the {self.name} floor")
            self.reserved += nbytes
        return Reservation(self, nbytes)


def host_admission(floor: int = DEFAULT_HOST_FLOOR, **kw) -> Admission:
    return Admission(host_available, floor, "host", **kw)


def device_admission(device=None, floor: int = DEFAULT_DEVICE_FLOOR, **kw) -> Admission:
    return Admission(lambda: device_available(device), floor, "device", **kw)


# ---------------------------------------------------------------------------------- stall counters
def pressure_snapshot(root: str = "/proc/pressure") -> dict:
    """Cumulative stall microseconds of the host (PSI 'some' totals) plus major-fault counts; the
    difference of two snapshots around a prefill says whether the host, not the GPU, held it up
    (reference: src/prefill_stall.rs)."""
    out = {}
    for res in ("memory", "io", "cpu"):
        try:
            with open(os.path.join(root, res)) as f:
                for line in f:
                    if line.startswith("some"):
                        out[res + "_us"] = int(line.split("total=")[1])
        except (OSError, IndexError, ValueError):
            out[res + "_us"] = 0
    try:
        with open("/proc/vmstat") as f:
            for line in f:
                k, _, v = line.partition(" ")
                if k in ("pgmajfault", "pswpin", "pswpout"):
                    out[k] = int(v)
    except OSError:
        pass
    return out


def pressure_delta(before: dict, after: dict) -> dict:
    return {k: after.get(k, 0) - before.get(k, 0) for k in after}


# ---------------------------------------------------------------------------------------------
# device memory plan: what one rank will hold, from the configuration alone
# ---------------------------------------------------------------------------------------------
def plan_device_memory(cfg, ecfg, world: int = 1, sp_prefill: Optional[bool] = None, chunk: Optional[int] = None) -> dict:
    """Bytes one rank holds on its GPU, by kind, computed from the model and engine configuration
    (no device needed): expert and dense weights in their stored formats, the unsharded dense
    matrices a sequence-parallel prefill keeps, embeddings and heads, the KV state of all regions, the
    scratch of the largest prefill chunk and of the decode rows, and the index-score buffer.  Mirrors
    the shapes ``models/engine.py`` allocates; meant to answer "does this fit in 180 GB at this rank
    count and context" before anything is loaded (the reference sizes its shards against a memory
    floor at start-up, src/memory.rs)."""
    d, H, Dh = cfg.hidden, cfg.n_heads, cfg.head_dim
    Hl, El = H // world, cfg.n_experts // world
    fp8 = lambda n, k: n * k + -(-n // 128) * -(-k // 128) * 4          # values + one fp32 scale per 128 x 128 block
    n_draft = cfg.draft.layers if cfg.draft is not None else 0
    sp = (world > 1 and ecfg.sp_prefill) if sp_prefill is None else sp_prefill
    late = cfg.late_start if 0 < cfg.late_start < cfg.n_layers else cfg.n_layers
    dense = full = experts = 0
    for li in range(cfg.n_layers + n_draft):
        draft = li >= cfg.n_layers
        kv_src = (not draft) and li in cfg.kv_source_layers
        ix_src = (not draft) and li in cfg.index_source_layers
        other = fp8(Dh, d)                                                   # kv projection
        if kv_src:
            other += 2 * fp8(Dh + cfg.index_dim, d)                          # compressor value / gate
        if ix_src:
            other += fp8(cfg.index_heads * cfg.index_dim, d) + fp8(cfg.index_heads, d)
        if cfg.q_lora_rank:
            qb = fp8(cfg.q_lora_rank, d) + fp8(Hl * Dh, cfg.q_lora_rank)
        else:
            qb = fp8(Hl * Dh, d)
        if cfg.o_groups:
            G, R = cfg.o_groups // world, cfg.o_lora_rank
            wo = G * fp8(R, Hl * Dh // max(G, 1)) + fp8(d, G * R)
        else:
            wo = fp8(d, Hl * Dh)
        Is = cfg.shared_inter * cfg.n_shared
        shared = (2 * fp8(Is // world, d) + fp8(d, Is // world)) if cfg.n_shared else 0
        gate = cfg.n_experts * d * 2 + (cfg.n_experts * 4 if cfg.router_bias else 0)
        hc = 2 * (cfg.hc_mult * (2 + cfg.hc_mult) * cfg.hc_mult * d * 4) if cfg.hc_mult > 1 else 0
        dense += other + qb + wo + shared + gate + hc + (3 * d + 2 * Dh) * 2
        if cfg.expert_quant == "mxfp4":
            I = cfg.moe_inter
            experts += El * 3 * (I * d // 2 + I * d // 32)
        else:
            experts += El * 3 * cfg.moe_inter * d * 2
        if sp and not draft and li < late and not cfg.q_lora_rank and not cfg.o_groups:
            # the unsharded dense matrices of the encoder layers (every rank runs whole layers on its rows)
            full += other + fp8(H * Dh, d) + fp8(d, H * Dh) + ((2 * fp8(Is, d) + fp8(d, Is)) if cfg.n_shared else 0)
    Vl = cfg.vocab // world
    heads = cfg.vocab * d * 2 + Vl * d * 2                                   # embedding (replicated) + this rank's head rows
    if n_draft:
        heads += fp8(Vl, d) + fp8(d, d * (1 + cfg.draft.condition_layers))   # FP8 copy of the head for the drafter, conditioning
        if cfg.draft.markov_rank:
            heads += (cfg.vocab + Vl) * cfg.draft.markov_rank * 2
    # ---- KV state of all regions
    chunk = chunk or max(ecfg.prefill_widths)
    ring = max(chunk, ecfg.sp_chunk_rows if world > 1 else 0) + 2 * cfg.window
    nl = cfg.n_layers + n_draft
    ns = max(1, len(cfg.kv_source_layers))
    maxC = ecfg.max_context // cfg.compress_ratio + 8
    C = Dh + cfg.index_dim
    kv = (nl * ecfg.regions * ring * cfg.window_kv_bytes
          + ns * ecfg.regions * maxC * (cfg.compressed_kv_bytes + cfg.index_key_bytes)
          + ns * ecfg.regions * (cfg.max_ratio + 32) * 2 * C * 4)
    # ---- scratch: the row buffers of one prefill chunk (this rank's rows) and of a decode block
    def rows(T: int, big: bool) -> int:
        maxN = Hl * Dh + Dh + 2 * C + cfg.index_heads * (cfg.index_dim + 1)
        per = (d * (2 + 2 + 2 + 4 + 4) + maxN * (2 if big else 4) + Hl * Dh * (2 + 2 + 4) + cfg.n_experts * 4
               + len(cfg.index_source_layers) * (cfg.index_topk + 1) * 4 + (cfg.shared_inter * cfg.n_shared // world) * 2)
        if not big:
            per += cfg.topk * (cfg.moe_inter * 2 + d * 4)
        else:
            # grouped expert GEMMs of a chunk: permuted rows, both activations and the pair outputs
            per += cfg.topk * (d * 2 + d + cfg.moe_inter * (2 + 1) + d * 2)
        return T * per * cfg.hc_mult if cfg.hc_mult > 1 else T * per
    t_prefill = -(-max(chunk, ecfg.sp_chunk_rows if (sp and world > 1) else 0) // (world if sp else 1))
    scratch = rows(min(t_prefill, chunk), True) + rows(32, False)
    nmax = ecfg.max_context // cfg.compress_ratio
    scores = min(ecfg.index_score_bytes, t_prefill * nmax * 4) if cfg.index_source_layers else 0
    out = {"expert_weights": experts, "dense_weights": dense, "dense_unsharded_for_sp": full, "embedding_and_heads": heads,
           "kv_state": kv, "scratch": scratch, "index_scores": scores}
    out["total"] = sum(out.values())
    return out
