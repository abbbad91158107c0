"""Fused tensor-parallel collective GEMMs against NCCL + cuBLAS on the same GPUs.

    torchrun --nproc-per-node N benchmarks/bench_tp_collective.py

GEMM -> all-reduce (M <= 32: one kernel, FP8 weight stream, one-shot exchange over peer memory)
and GEMM -> reduce-scatter (M >= 512: tcgen05 GEMM whose epilogue stores tiles into the owner's
memory, then the owner-side sum) for A [M, K/tp] x W [N, K/tp], K = N = 4096.  Times are CUDA
events, max over ranks, L2 flushed between iterations.  Roofline of each fused op: the slower
of FLOPs / measured GEMM peak and bytes that must cross NVLink / 770 GB/s.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import flush_l2, peaks  # noqa: E402
from titanic_flash_41_b200.models import engine as E  # noqa: E402
from titanic_flash_41_b200.ops import native  # noqa: E402
from titanic_flash_41_b200.parallel.symm import AgWorkspace, RsWorkspace, SymmWorkspace  # noqa: E402

NVLINK_GBS = 770.0


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush_l2()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(float(t))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    pk = peaks()
    st = native.StatusWord(dev)
    K = N = 4096
    Kl = K // world
    g = torch.Generator(device=dev).manual_seed(rank)
    w = torch.randn(N, Kl, device=dev, generator=g) * 0.02
    w8 = E.quant_fp8_device(w)
    wb = w.bfloat16()
    rows = []
    ws = SymmWorkspace(N, 32, device=dev)
    # decode-sized op.  One call is ~10 us, far below what a barrier + event pair resolves, and in a
    # decode step the calls come back to back inside a CUDA graph: time a CHAIN of calls over
    # distinct weight matrices (more bytes than L2 holds, so every call streams its weights from HBM)
    # replayed as one graph, and report time per call.  `nccl` is the same chain as cuBLAS GEMV +
    # NCCL all-reduce + the separate boundary kernel.
    chain = 48
    ws8 = [E.quant_fp8_device(torch.randn(N, Kl, device=dev, generator=g) * 0.02) for _ in range(chain)]
    wbs = [dq.bfloat16() for dq in (E.dequant_fp8(w_) for w_ in ws8)]
    nw = torch.ones(N, device=dev, dtype=torch.bfloat16)
    for M in (1, 4, 16, 32):
        x = torch.randn(M, Kl, device=dev, generator=g)
        x16, xb = x.half(), x.bfloat16()
        resid = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
        h16 = torch.zeros(M, N, device=dev, dtype=torch.float16)
        hb = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
        x8 = torch.zeros(M, N, device=dev, dtype=torch.uint8)
        x8s = torch.zeros(M, N // 32, device=dev, dtype=torch.uint8)
        norm = dict(w=nw, h16=h16, hb=hb, x8=x8, x8s=x8s, eps=1e-6)
        ref = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        delta = torch.zeros(M, N, device=dev)

        def fused_chain():
            for w_ in ws8:
                ws.gemv_allreduce(w_, x16, M, resid, None, st.t, norm=norm)

        def nccl_chain():
            for wb_ in wbs:
                torch.matmul(xb, wb_.t(), out=ref)
                dist.all_reduce(ref)
                delta.copy_(ref)
                native.call("tf_add_norm_fused", resid, delta, None, None, None, None, 0, 0, 0, nw, h16, hb, x8, x8s,
                            M, N, 1e-6)

        def graphed(fn):
            fn()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            return gr.replay
        fused = timed(graphed(fused_chain)) / chain
        try:
            nccl = timed(graphed(nccl_chain)) / chain
        except Exception:                                   # noqa: BLE001  (NCCL under capture is optional)
            torch.cuda.synchronize()
            nccl = timed(nccl_chain) / chain
        out = torch.zeros(M, N, device=dev)
        ws.gemv_allreduce(w8, x16, M, None, out, st.t)
        want = x16.float() @ E.dequant_fp8(w8).t()
        dist.all_reduce(want)
        err = float((out - want).abs().max() / want.abs().max())
        # roofline of the decode-sized op: weight bytes from HBM, one NVLink one-way flight (~1.5 us
        # measured for a flag round trip / 2) and the bf16 partials of M rows to 7 peers
        hbm_us = (N * Kl) / (pk["hbm_gbs"] * 1e3)
        link_us = 1.5 + M * N * 4 * (world - 1) / (NVLINK_GBS * 1e3)
        roof = hbm_us + link_us
        rows.append(dict(op="gemv+allreduce+residual+norm (chain of 48 in one graph)", M=M, fused_us=round(fused * 1e3, 2),
                         nccl_cublas_us=round(nccl * 1e3, 2), speedup=round(nccl / fused, 2), rel_err=round(err, 5),
                         roofline_us=round(roof, 2), frac_of_roofline=round(roof / (fused * 1e3), 3)))
    for M in (512, 4096, 16384):
        if M % (world * 128):
            continue
        rsw = RsWorkspace(M, N, device=dev)
        x = torch.randn(M, Kl, device=dev, generator=g)
        xb = x.bfloat16()
        out = torch.zeros(M // world, N, device=dev, dtype=torch.bfloat16)
        flops = 2.0 * M * N * Kl
        link_bytes = M * N * 2 * (world - 1) / world
        roof_ms = max(flops / (pk["bf16_tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        fused = timed(lambda: rsw.gemm_reduce_scatter(0, xb, wb, out, st.t))
        full = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        rs_out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)

        def base():
            torch.matmul(xb, wb.t(), out=full)
            dist.reduce_scatter_tensor(rs_out, full)
        nccl = timed(base)
        base()
        rsw.gemm_reduce_scatter(0, xb, wb, out, st.t)
        torch.cuda.synchronize()
        err = float((out.float() - rs_out.float()).abs().max() / rs_out.float().abs().max())
        row = dict(op="gemm+reduce_scatter bf16", M=M, fused_ms=round(fused, 4), nccl_cublas_ms=round(nccl, 4),
                   speedup=round(nccl / fused, 2), roofline_ms=round(roof_ms, 4), frac_of_roofline=round(roof_ms / fused, 3),
                   rel_err=round(err, 5))
        # FP8 block-scaled operands
        xg = x.view(M, Kl // 128, 128)
        sa = (xg.abs().amax(-1).clamp_min(1e-12) / 448.0).contiguous()
        xq = (xg / sa[:, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(M, Kl)
        f8 = timed(lambda: rsw.gemm_reduce_scatter(2, xq, w8.q, out, st.t, sa, w8.s))
        row.update(fp8_fused_ms=round(f8, 4), fp8_speedup_vs_bf16_baseline=round(nccl / f8, 2))
        rows.append(row)
        del rsw
    # ---- all-gather -> GEMM: activations row-sharded [M/tp, K], weight column shard [N/tp, K]
    Nl = N // world
    wn = torch.randn(Nl, K, device=dev, generator=g) * 0.02
    wnb, wn8 = wn.bfloat16(), E.quant_fp8_device(wn)
    for M in (512, 4096, 16384):
        if M % (world * 128):
            continue
        xs = torch.randn(M // world, K, device=dev, generator=g)
        xsb = xs.bfloat16()
        agw = AgWorkspace(0, M, K, device=dev)
        out = torch.zeros(M, Nl, device=dev, dtype=torch.bfloat16)

        def fused():
            a, _ = agw.shard()
            a.copy_(xsb)
            agw.allgather_gemm(wnb, out, st.t)
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        ref = torch.empty(M, Nl, device=dev, dtype=torch.bfloat16)

        def base():
            dist.all_gather_into_tensor(full, xsb)
            torch.matmul(full, wnb.t(), out=ref)
        tf_, tn = timed(fused), timed(base)
        base()
        fused()
        torch.cuda.synchronize()
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        flops = 2.0 * M * Nl * K
        link_bytes = M * K * 2 * (world - 1) / world
        roof_ms = max(flops / (pk["bf16_tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        row = dict(op="allgather+gemm bf16", M=M, fused_ms=round(tf_, 4), nccl_cublas_ms=round(tn, 4),
                   speedup=round(tn / tf_, 2), roofline_ms=round(roof_ms, 4), frac_of_roofline=round(roof_ms / tf_, 3),
                   rel_err=round(err, 5))
        del agw
        ag8 = AgWorkspace(2, M, K, device=dev)
        xg = xs.view(M // world, K // 128, 128)
        sa = (xg.abs().amax(-1).clamp_min(1e-12) / 448.0).contiguous()
        xq = (xg / sa[:, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(M // world, K)

        def fused8():
            a, s_ = ag8.shard()
            a.copy_(xq)
            s_.copy_(sa)
            ag8.allgather_gemm(wn8.q, out, st.t, wn8.s)
        t8 = timed(fused8)
        fused8()
        torch.cuda.synchronize()
        err8 = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        row.update(fp8_fused_ms=round(t8, 4), fp8_speedup_vs_bf16_baseline=round(tn / t8, 2), fp8_rel_err=round(err8, 4))
        rows.append(row)
        del ag8
    st.check()
    if rank == 0:
        print(json.dumps({"world": world, "K": K, "N": N, "peaks": pk, "rows": rows}, indent=1), flush=True)
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
