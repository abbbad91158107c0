"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

Every rank allocates one workspace of the same size, the ranks exchange handles, and each rank
ends up with the base address of every peer's workspace mapped into its own address space
(NVLink peer-to-peer through NVSwitch).  The kernels of ``csrc/comm.cuh`` store partial tiles
and flags straight into those addresses.  Allocation and handle exchange go through
``torch.distributed._symmetric_memory`` (plumbing only: no library kernel ever receives a peer
pointer).  Replaces the reference's pinned-host RoCE region + CPU proxy (src/roce.rs:179-243).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native


class SymmWorkspace:
    """Workspace of the one-shot all-reduce epilogue for matrices [rows <= max_rows, N] (layout:
    ``csrc/comm.cuh``).  ``norm`` arguments name the boundary computed in the epilogue: a dict with
    ``w`` (RMSNorm weight) and any of ``h16``, ``hb``, ``x8``, ``x8s`` output tensors, plus ``eps``."""

    def __init__(self, N: int, max_rows: int = 32, device=None, group: Optional[dist.ProcessGroup] = None,
                 spin_limit: int = 2_000_000):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.N, self.max_rows, self.spin_limit = N, max_rows, spin_limit
        lib = native.lib()
        nbytes = int(lib.tf_comm_workspace_bytes(self.world, N, max_rows))
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(ptrs) == self.world
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=dev)
        self.epoch = torch.zeros(N // 32, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)

    @staticmethod
    def _norm_args(norm: Optional[dict]):
        if not norm:
            return (None, None, None, None, None, 0.0)
        return (norm["w"], norm.get("h16"), norm.get("hb"), norm.get("x8"), norm.get("x8s"), float(norm["eps"]))

    # ---- fused ops ---------------------------------------------------------------------------
    def gemv_allreduce(self, w, x16: torch.Tensor, M: int, resid: Optional[torch.Tensor],
                       out: Optional[torch.Tensor], status: torch.Tensor, norm: Optional[dict] = None) -> None:
        """resid[:M] += all-reduce(x16[:M] @ W^T), then the boundary ``norm``, in ONE kernel (FP8
        block-128 weights)."""
        N, K = w.q.shape
        assert N == self.N
        native.call("tf_smallm_gemm_allreduce", w.q, w.s, K, K // 128, x16, x16.stride(0), N, K, M, self.peers,
                    self.world, self.rank, self.max_rows, self.epoch, resid, out, *self._norm_args(norm),
                    self.spin_limit, status)

    def combine_allreduce(self, y_pair, ids, wts, shared_y, rows: int, topk: int, e_lo: int, e_hi: int,
                          resid: Optional[torch.Tensor], out: Optional[torch.Tensor], status: torch.Tensor,
                          norm: Optional[dict] = None) -> None:
        native.call("tf_moe_combine_allreduce", y_pair, ids, wts, shared_y, rows, self.N, topk, e_lo, e_hi,
                    self.peers, self.world, self.rank, self.max_rows, self.epoch, resid, out,
                    *self._norm_args(norm), self.spin_limit, status)

    def allreduce(self, x: torch.Tensor, rows: int, out: torch.Tensor, status: torch.Tensor) -> None:
        """out[:rows] = sum over ranks of x[:rows] (fp32 on the wire, rows <= max_rows, width N)."""
        native.call("tf_moe_combine_allreduce", None, None, None, x, rows, self.N, 0, 0, 0, self.peers,
                    self.world, self.rank, self.max_rows, self.epoch, None, out, *self._norm_args(None),
                    self.spin_limit, status)


class EmulatedRanks:
    """``world`` ranks of the one-shot all-reduce emulated on ONE GPU by a single cooperative launch
    (every emulated rank gets its own workspace area in the same device memory).  Exercises the
    push / poll / rank-ordered sum / boundary epilogue without a second device."""

    def __init__(self, world: int, N: int, max_rows: int = 32, device="cuda", spin_limit: int = 2_000_000):
        lib = native.lib()
        self.world, self.N, self.max_rows, self.spin_limit = world, N, max_rows, spin_limit
        nbytes = int(lib.tf_comm_workspace_bytes(world, N, max_rows))
        dev = torch.device(device)
        self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
        self.peers = torch.tensor([b.data_ptr() for b in self.bufs], dtype=torch.int64, device=dev)
        self.epoch = torch.zeros(world * (N // 32), dtype=torch.int32, device=dev)

    def allreduce(self, partial: torch.Tensor, rows: int, status: torch.Tensor, resid=None, out=None,
                  norm: Optional[dict] = None) -> None:
        """partial [world, rows_alloc, N] fp32; resid / out / norm outputs [world, rows_alloc, N]
        (x8s [world, rows_alloc, N / 32]): every emulated rank updates its own slice."""
        assert partial.shape[0] == self.world and partial.shape[2] == self.N and partial.is_contiguous()
        native.call("tf_comm_allreduce_emulated", partial, rows, partial.shape[1], self.N, self.peers, self.world,
                    self.max_rows, self.epoch, resid, out, *SymmWorkspace._norm_args(norm), self.spin_limit, status)


class SampleWorkspace:
    """Exchange area and call counters of the chunked sampler (``csrc/sample_chunks.cu``): one
    launch computes the row statistics and the block verification (or a plain draw) of up to
    ``max_rows`` rows from this rank's columns of the logits.  With ``world > 1`` the area is
    symmetric memory and construction is collective; ``emulate > 1`` places that many ranks on this
    GPU (tests on one device)."""

    def __init__(self, V: int, max_rows: int, device, world: int = 1, rank: int = 0,
                 group: Optional[dist.ProcessGroup] = None, emulate: int = 1, spin_limit: int = 4_000_000):
        lib = native.lib()
        self.V, self.max_rows, self.spin_limit = V, max_rows, spin_limit
        self.P = int(lib.tf_sample_chunks_count(V))
        if self.P == 0:
            raise ValueError(f"a vocabulary of {V} cannot be chunked for rank-local sampling")
        self.emulate = emulate
        self.world = emulate if emulate > 1 else world
        self.rank = 0 if emulate > 1 else rank
        if self.P % self.world:
            raise ValueError(f"{self.P} chunks do not split over {self.world} ranks")
        self.csplit = self.P // self.world
        self.Vl = V // self.world
        nbytes = int(lib.tf_sample_chunks_workspace_bytes(V, max_rows))
        dev = torch.device(device)
        if emulate > 1:
            self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(emulate)]
            ptrs = [b.data_ptr() for b in self.bufs]
        elif world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.group = group or dist.group.WORLD
            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            ptrs = [self.buf.data_ptr()]
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=dev)
        self.ctr = torch.zeros(max(emulate, 1) * max_rows * self.csplit, dtype=torch.int32, device=dev)
        if world > 1 and emulate <= 1:
            torch.cuda.synchronize(dev)
            dist.barrier(self.group)

    @staticmethod
    def usable(V: int, rows: int, world: int, device) -> bool:
        """Whether ``rows`` rows of a ``V``-token vocabulary can be sampled by the chunked kernel on
        ``world`` ranks: V must chunk, and the (row, local chunk) CTAs of a GPU must all be resident."""
        P = int(native.lib().tf_sample_chunks_count(V))
        if P == 0 or P % world:
            return False
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        return rows * (P // world) <= sms

    def sample(self, tlogits, dlogits, dstat, proposals, uniforms, u_stride: int, sess_temp, sess_top_p, S: int,
               g: int, ldl: int, tstat, stat_stride: int, n_accept, next_token, tok_stride: int, status,
               point_mass: bool = False, emu_strides=(0, 0, 0, 0, 0), sess_point=None, forced=None,
               sess_g=None) -> None:
        """``sess_g`` [S] int32 (g > 0): proposals each conversation verifies (causal stopping)."""
        native.call("tf_sample_chunks", tlogits, dlogits, dstat, proposals, uniforms, u_stride, sess_temp, sess_top_p,
                    S, g, self.V, ldl, 1 if point_mass else 0, sess_point, forced, sess_g, tstat, stat_stride, n_accept,
                    next_token, tok_stride,
                    self.peers, self.world, self.rank, self.max_rows, self.ctr, self.spin_limit, status,
                    self.emulate, *emu_strides)


class RsWorkspace:
    """Workspace of the GEMM -> reduce-scatter kernel for partial products [M, N] (bf16 transport)."""

    def __init__(self, M: int, N: int, device=None, group: Optional[dist.ProcessGroup] = None,
                 spin_limit: int = 4_000_000):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.M, self.N, self.spin_limit = M, N, spin_limit
        nbytes = int(native.lib().tf_gemm_rs_workspace_bytes(M, N, self.world))
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.peers = torch.tensor([int(p) for p in self.handle.buffer_ptrs], dtype=torch.int64, device=dev)
        self.epoch = 0
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)

    def gemm_reduce_scatter(self, kind: int, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor,
                            status: torch.Tensor, sa: Optional[torch.Tensor] = None,
                            sb: Optional[torch.Tensor] = None) -> None:
        """out[M/world, N] (bf16) = rows of this rank of sum_r a_r[M, K] @ b_r[N, K]^T."""
        M, K = a.shape
        N = b.shape[0]
        assert (M, N) == (self.M, self.N)
        self.epoch += 1
        native.call("tf_gemm_rs", kind, a, a.stride(0), b, b.stride(0), M, N, K, sa, sa.stride(0) if sa is not None else 0,
                    sb, sb.stride(0) if sb is not None else 0, self.peers, self.world, self.rank, self.epoch, out,
                    out.stride(0), self.spin_limit, status)


class AgWorkspace:
    """Workspace of the all-gather -> GEMM kernel for row-sharded activations [M/world, K] per rank.

    ``shard(kind)`` returns views of this call's slot for the rank's rows (and, for FP8, their
    1x128 scales); fill them, then call ``allgather_gemm``: the kernel's copy CTAs pull every
    rank's slot over NVLink with bulk copies while its GEMM CTAs multiply the blocks that have
    already arrived."""

    def __init__(self, kind: int, M: int, K: int, device=None, group: Optional[dist.ProcessGroup] = None,
                 spin_limit: int = 4_000_000, copy_ctas: int = 16):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.kind, self.M, self.K, self.spin_limit, self.copy_ctas = kind, M, K, spin_limit, copy_ctas
        nbytes = int(native.lib().tf_gemm_ag_workspace_bytes(kind, M, K, self.world))
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.peers = torch.tensor([int(p) for p in self.handle.buffer_ptrs], dtype=torch.int64, device=dev)
        self.epoch = 0
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)

    def shard(self):
        """(rows view, scales view or None) of the slot the NEXT allgather_gemm call will publish."""
        rows = self.M // self.world
        off = int(native.lib().tf_gemm_ag_shard_offset(self.kind, self.M, self.K, self.world, self.epoch + 1))
        es = 2 if self.kind == 0 else 1
        a = self.buf[off:off + rows * self.K * es].view(torch.bfloat16 if self.kind == 0 else torch.float8_e4m3fn)
        a = a.view(rows, self.K)
        s = None
        if self.kind == 2:
            so = off + rows * self.K
            s = self.buf[so:so + rows * (self.K // 128) * 4].view(torch.float32).view(rows, self.K // 128)
        return a, s

    def allgather_gemm(self, b: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                       sb: Optional[torch.Tensor] = None) -> None:
        """out[M, N] = allgather(shards)[M, K] @ b[N, K]^T (out bf16 or fp32)."""
        self.epoch += 1
        N = b.shape[0]
        native.call("tf_gemm_ag", self.kind, b, b.stride(0), out, out.stride(0), self.M, N, self.K, sb,
                    sb.stride(0) if sb is not None else 0, 2 if out.dtype == torch.bfloat16 else 0, self.peers,
                    self.buf, self.world, self.rank, self.epoch, self.copy_ctas, self.spin_limit, status)
