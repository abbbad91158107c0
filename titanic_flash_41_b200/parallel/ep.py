"""Expert-parallel MoE layer over NVLink peer memory (token-sharded ranks).

``EpMoE.forward`` = dispatch kernel (FP8 quantise + peer stores) -> receive plan + gather ->
grouped tcgen05 GEMMs (FC1, SwiGLU + requantise, FC2) -> return kernel (peer stores) -> combine
kernel.  Five of our kernels touch NVLink or its flags; no NCCL call and no host synchronisation
sit inside.  ``EpMoE.forward_nccl`` is the baseline with the same expert math but
``all_to_all_single`` for both exchanges.  Kernels: csrc/ep_moe.cu.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native


class EpMoE:
    def __init__(self, d: int, inter: int, n_experts: int, topk: int, tl_max: int, ew1, es1, ew3, es3, ew2, es2,
                 device=None, group: Optional[dist.ProcessGroup] = None, swiglu_limit: float = 10.0,
                 spin_limit: int = 4_000_000, symmetric: bool = True):
        """ew*/es*: this rank's experts in MXFP4 ([El, N, K/2] packed nibbles, [El, N, K/32] UE8M0)."""
        self.group = group or (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.d, self.I, self.E, self.k, self.tl_max = d, inter, n_experts, topk, tl_max
        self.El = n_experts // self.world
        self.cap = tl_max * topk
        self.limit, self.spin_limit = swiglu_limit, spin_limit
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        L = native.lib()
        nbytes = int(L.tf_ep_workspace_bytes(self.world, self.cap, d, tl_max, topk))
        if self.world > 1 and symmetric:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            ptrs = [self.buf.data_ptr()]
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=dev)
        El, I = self.El, inter
        self.w13 = torch.empty(El, 2 * I, d, dtype=torch.uint8, device=dev)
        self.s13 = torch.empty(El * 2 * I // 128, d // 128, dtype=torch.float32, device=dev)
        self.w2 = torch.empty(El, d, I, dtype=torch.uint8, device=dev)
        self.s2 = torch.empty(El * d // 128, I // 128, dtype=torch.float32, device=dev)
        native.call("tf_mxfp4_to_fp8_block", ew1, es1, self.w13, self.s13, El, I, d, 0, 2 * I)
        native.call("tf_mxfp4_to_fp8_block", ew3, es3, self.w13, self.s13, El, I, d, I, 2 * I)
        native.call("tf_mxfp4_to_fp8_block", ew2, es2, self.w2, self.s2, El, d, I, 0, d)
        n_in = self.world * self.cap
        rows = -(-(n_in + El * 127) // 128) * 128
        self.rows, self.max_tiles = rows, rows // 128
        i32 = dict(dtype=torch.int32, device=dev)
        self.ids_recv = torch.empty(n_in, **i32)
        self.counts = torch.zeros(El, **i32)
        self.offsets = torch.empty(El + 1, **i32)
        self.cursor = torch.empty(El, **i32)
        self.tile_e = torch.empty(self.max_tiles, **i32)
        self.ntile = torch.zeros(2, **i32)
        self.pair_dst = torch.empty(n_in, **i32)
        self.xp = torch.zeros(rows, d, dtype=torch.uint8, device=dev)
        self.xps = torch.zeros(rows, d // 128, dtype=torch.float32, device=dev)
        self.y1 = torch.empty(rows, 2 * I, dtype=torch.bfloat16, device=dev)
        self.aq = torch.empty(rows, I, dtype=torch.uint8, device=dev)
        self.aqs = torch.empty(rows, I // 128, dtype=torch.float32, device=dev)
        self.y2 = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)
        self.epoch = 0
        torch.cuda.synchronize(dev)
        if self.group is not None and self.world > 1:
            dist.barrier(self.group)

    # ---- expert math on rows that are already in the padded, expert-sorted layout
    def _experts(self, status: torch.Tensor) -> None:
        d, I, El = self.d, self.I, self.El
        native.call("tf_gemm_tc", 2, self.xp, d, self.w13, d, self.y1, 2 * I, self.rows, 2 * I, d, self.xps, d // 128,
                    self.s13, d // 128, 2, self.tile_e, self.ntile[0:1], El, status)
        native.call("tf_swiglu_rows", self.y1, 2, 2 * I, None, 0, self.aq, self.aqs, self.rows, I, self.limit,
                    self.ntile[1:2])
        native.call("tf_gemm_tc", 2, self.aq, I, self.w2, I, self.y2, d, self.rows, d, I, self.aqs, I // 128, self.s2,
                    I // 128, 2, self.tile_e, self.ntile[0:1], El, status)

    def forward(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor,
                status: torch.Tensor, shared: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [Tl, d] bf16, ids [Tl, k] int32 (global expert ids), wts [Tl, k] fp32 -> out [Tl, d] bf16."""
        Tl = x.shape[0]
        assert Tl <= self.tl_max and x.dtype == torch.bfloat16 and ids.dtype == torch.int32
        self.epoch += 1
        a = (self.peers, self.world, self.rank, self.cap, self.d, self.k, self.El, self.tl_max)
        native.call("tf_ep_dispatch", *a, self.epoch, x, x.stride(0) if Tl else self.d, ids, Tl, status)
        native.call("tf_ep_recv_ids", *a, self.epoch, self.ids_recv, self.spin_limit, status)
        native.call("tf_moe_plan", self.ids_recv, self.world * self.cap, self.rank * self.El, self.El, self.counts,
                    self.offsets, self.cursor, self.tile_e, self.max_tiles, self.ntile[0:1], self.ntile[1:2],
                    self.pair_dst)
        native.call("tf_ep_gather", *a, self.pair_dst, self.xp, self.xps)
        self._experts(status)
        native.call("tf_ep_return", *a, self.epoch, self.pair_dst, self.y2, self.d, status)
        native.call("tf_ep_combine", *a, self.epoch, ids, wts, shared, out, out.stride(0) if Tl else self.d, Tl,
                    self.spin_limit, status)
        return out

    # ---- baseline: NCCL all-to-all both ways around the same expert math
    def forward_nccl(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, status: torch.Tensor
                     ) -> torch.Tensor:
        Tl, k, W, El, d = x.shape[0], self.k, self.world, self.El, self.d
        flat = ids.reshape(-1).long()
        dst_rank = flat // El
        order = torch.argsort(dst_rank, stable=True)
        send_counts = torch.bincount(dst_rank, minlength=W)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        rows_out = x[order // k].contiguous()
        ids_out = flat[order].int().contiguous()
        n_in = sum(rc)
        rows_in = torch.empty(n_in, d, dtype=x.dtype, device=x.device)
        ids_in = torch.empty(n_in, dtype=torch.int32, device=x.device)
        dist.all_to_all_single(rows_in, rows_out, rc, sc, group=self.group)
        dist.all_to_all_single(ids_in, ids_out, rc, sc, group=self.group)
        pair_dst = self.pair_dst[:max(n_in, 1)]
        native.call("tf_moe_plan", ids_in, n_in, self.rank * El, El, self.counts, self.offsets, self.cursor, self.tile_e,
                    self.max_tiles, self.ntile[0:1], self.ntile[1:2], pair_dst)
        native.call("tf_quant_rows", rows_in, 2, d, None, 1, pair_dst, self.xp, self.xps, n_in, d)
        self._experts(status)
        back = self.y2[pair_dst[:n_in].long()].contiguous()
        ret = torch.empty(Tl * k, d, dtype=torch.bfloat16, device=x.device)
        dist.all_to_all_single(ret, back, sc, rc, group=self.group)
        y = torch.empty(Tl * k, d, dtype=torch.bfloat16, device=x.device)
        y[order] = ret
        return (y.view(Tl, k, d).float() * wts[:, :, None]).sum(1).to(torch.bfloat16)
