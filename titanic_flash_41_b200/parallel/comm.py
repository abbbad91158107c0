"""Collective interface used by the model code, with a single-process and a
``torch.distributed`` implementation.

The reference's communicator (src/collective.rs:137-486) exposes all-reduce, reduce-scatter,
all-gather, grouped all-to-all and broadcast; the same surface is offered here over
``torch.distributed`` (NCCL on GPUs, gloo for the CPU plumbing runs).  On GPUs these library
collectives are the *baseline*: the hot paths use the fused kernels of
``parallel/symm.py`` + ``ops/fused_comm.py`` instead.
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class Comm:
    world: int = 1
    rank: int = 0

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor: ...
    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor: ...
    def reduce_scatter(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor: ...
    def all_to_all(self, chunks: Sequence[torch.Tensor]) -> List[torch.Tensor]: ...
    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor: ...
    def barrier(self) -> None: ...


class LocalComm(Comm):
    """world size 1: every collective is the identity."""

    def all_reduce(self, t):
        return t

    def all_gather(self, t, dim=0):
        return t

    def reduce_scatter(self, t, dim=0):
        return t

    def all_to_all(self, chunks):
        return list(chunks)

    def broadcast(self, t, src=0):
        return t

    def barrier(self):
        pass


class DistComm(Comm):
    """``torch.distributed`` process-group collectives (sum in the tensor's own dtype, fixed
    by the library; fp32 inputs give the deterministic plumbing check)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def all_reduce(self, t):
        t = t.contiguous()
        dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t, dim=0):
        t = t.contiguous()
        outs = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(outs, t, group=self.group)
        return torch.cat(outs, dim)

    def reduce_scatter(self, t, dim=0):
        # gloo has no reduce_scatter: all-reduce then slice (baseline path only)
        full = self.all_reduce(t.clone())
        n = full.shape[dim] // self.world
        return full.narrow(dim, self.rank * n, n).contiguous()

    def all_to_all(self, chunks):
        chunks = [c.contiguous() for c in chunks]
        # sizes may differ per peer: exchange shapes first
        shapes = [None] * self.world
        dist.all_gather_object(shapes, [tuple(c.shape) for c in chunks], group=self.group)
        outs = [torch.empty(shapes[src][self.rank], dtype=chunks[0].dtype, device=chunks[0].device)
                for src in range(self.world)]
        if dist.get_backend(self.group) == "gloo":
            reqs = []
            for peer in range(self.world):
                if peer == self.rank:
                    outs[peer].copy_(chunks[peer])
                    continue
                reqs.append(dist.isend(chunks[peer], peer, group=self.group))
                reqs.append(dist.irecv(outs[peer], peer, group=self.group))
            for r in reqs:
                r.wait()
        else:
            dist.all_to_all(outs, chunks, group=self.group)
        return outs

    def broadcast(self, t, src=0):
        dist.broadcast(t, src, group=self.group)
        return t

    def barrier(self):
        dist.barrier(group=self.group)


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> Comm:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun's
    contract).  Replaces the reference's TCP rendezvous (src/rendezvous.rs:10-172): rank 0's
    store distributes the NCCL id; a bounded timeout covers peers that never join."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and not dist.is_initialized():
        return LocalComm()
    if not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return DistComm()
