"""Multi-GPU checks, launched by torchrun (one rank per GPU):  fused all-reduce kernels against
torch references, and the tensor/expert-parallel engine against the single-GPU engine."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from titanic_flash_41_b200.config import DraftConfig, EngineConfig  # noqa: E402
from titanic_flash_41_b200.models import engine as E  # noqa: E402
from titanic_flash_41_b200.models import oracle  # noqa: E402
from titanic_flash_41_b200.ops import native  # noqa: E402
from titanic_flash_41_b200.parallel.comm import DistComm, LocalComm  # noqa: E402
from titanic_flash_41_b200.parallel.symm import SymmWorkspace  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    comm = DistComm()
    st = native.StatusWord(dev)

    def say(msg):
        if rank == 0:
            print("[mgpu]", msg, flush=True)
    say("process group up")
    # ---- 1. one-shot all-reduce of a small fp32 matrix, many epochs back to back
    N = 1024
    ws = SymmWorkspace(N, max_rows=32, device=dev, spin_limit=2_000_000)
    say("workspace ready")
    for it, rows in enumerate([1, 5, 16, 32, 7, 7, 7, 32]):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(rows, N, device=dev, generator=g)
        out = torch.zeros(rows, N, device=dev)
        ws.allreduce(x, rows, out, st.t)
        ref = x.clone()
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        st.check()
        assert torch.allclose(out, ref, atol=1e-5), (it, float((out - ref).abs().max()))
        # every rank holds the bit-identical sum
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(gathered[0], t) for t in gathered)
    say("all-reduce ok")
    # ---- 2. FP8 GEMV fused with all-reduce and residual update
    K, M = 1024, 9
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    w = E.quant_fp8_device(torch.randn(N, K, device=dev, generator=g) * 0.05)
    x16 = torch.randn(M, K, device=dev, generator=g).half()
    resid = torch.randn(M, N, device=dev, generator=torch.Generator(device=dev).manual_seed(1)).bfloat16()
    r0 = resid.clone()
    nw = (1 + 0.1 * torch.randn(N, device=dev, generator=torch.Generator(device=dev).manual_seed(2))).bfloat16()
    h16 = torch.zeros(M, N, device=dev, dtype=torch.float16)
    hb = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    x8 = torch.zeros(M, N, device=dev, dtype=torch.uint8)
    x8s = torch.zeros(M, N // 32, device=dev, dtype=torch.uint8)
    ws.gemv_allreduce(w, x16, M, resid, None, st.t, norm=dict(w=nw, h16=h16, hb=hb, x8=x8, x8s=x8s, eps=1e-6))
    part = x16.float() @ E.dequant_fp8(w).t()
    dist.all_reduce(part)
    torch.cuda.synchronize()
    st.check()
    want = (r0.float() + part).bfloat16()
    assert (resid.float() - want.float()).abs().max() < 0.08, float((resid.float() - want.float()).abs().max())
    # the boundary computed in the epilogue: RMSNorm of the NEW residual, and its MXFP8 form
    xf = resid.float()
    hn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).bfloat16().float()
    assert (hb.float() - hn).abs().max() <= 0.02 * hn.abs().max()
    assert (h16.float() - hn).abs().max() <= 0.02 * hn.abs().max()
    deq = x8.view(torch.float8_e4m3fn).float().view(M, N // 32, 32) * torch.exp2(x8s.float() - 127)[..., None]
    assert (deq.view(M, N) - hn).abs().max() <= 0.08 * hn.abs().max()
    for t in (resid, h16, x8):                              # bit-identical on every rank
        gathered = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        assert all(torch.equal(gathered[0].view(torch.uint8), g_.view(torch.uint8)) for g_ in gathered)
    say("fused gemv + boundary ok")
    # ---- 3. engine: TP/EP over `world` GPUs (fused kernels) == single GPU
    from tests.test_engine_gpu import small_config
    # keep every per-rank slice at least one 128-wide block: heads and shared-expert width grow with the world
    # (moe_inter 512: the routed experts of decode rows run on the block-scaled tensor-core GEMV)
    cfg = small_config(n_heads=4 * world if world > 4 else 4, shared_inter=max(256, 128 * world),
                       moe_inter=512, draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    chunk = max(128, 64 * world)       # sequence-parallel slices of 64 rows: every rank stays on the tensor-core path
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=4096, prefill_widths=(chunk,))
    # the TP engine also splits index scoring by key range from 8 keys on (decode rows)
    # (a sequence-parallel chunk spans two single-rank chunks: the window ring holds all of it)
    ecfg_tp = EngineConfig(reference_matmul=True, regions=2, max_context=4096, prefill_widths=(chunk,), key_sharded_index_min=8,
                           sp_chunk_rows=2 * chunk)
    eng = E.Engine.from_weights(cfg, ecfg_tp, W, comm=comm, device=dev)
    eng.symm = SymmWorkspace(cfg.hidden, 32, device=dev, spin_limit=2_000_000)
    ref = E.Engine.from_weights(cfg, ecfg, W, comm=LocalComm(), device=dev)
    gen = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (90,), generator=gen).tolist()
    a = eng.forward(E.StepPlan.build([(0, 0, prompt)], logits="last"))
    b = ref.forward(E.StepPlan.build([(0, 0, prompt)], logits="last"))
    errs = [float((a - b).abs().max() / b.abs().max())]
    pos = 90
    for step in range(5):
        toks = torch.randint(0, cfg.vocab, (4,), generator=gen).tolist()
        a = eng.forward(E.StepPlan.build([(0, pos, toks)]))
        b = ref.forward(E.StepPlan.build([(0, pos, toks)]))
        errs.append(float((a - b).abs().max() / b.abs().max()))
        pos += 4
    torch.cuda.synchronize()
    eng.status.check()
    srt = sorted(errs)
    assert srt[(len(srt) - 1) // 2] < 0.11, errs
    say("engine ok %s" % errs)
    # ---- 3b. sequence-parallel prefill (rows of every chunk split over the ranks) == single GPU,
    #          and the KV state it leaves on every rank serves the tensor-parallel decode rows
    from titanic_flash_41_b200.ops import bigpath
    from titanic_flash_41_b200.parallel import sp as SP
    from titanic_flash_41_b200.serve.prefill import run_prefill
    bigpath.attach(eng)
    bigpath.attach(ref)
    assert SP.attach(eng) is not None
    long_prompt = torch.randint(0, cfg.vocab, (chunk * 3 + 37,), generator=gen, dtype=torch.int32)
    a = run_prefill(eng, 1, long_prompt, chunk)
    b = run_prefill(ref, 1, long_prompt, chunk)
    errs_sp = [float((a - b).abs().max() / b.abs().max())]
    p1 = int(long_prompt.numel())
    for step in range(3):
        toks = torch.randint(0, cfg.vocab, (4,), generator=gen).tolist()
        a = eng.forward(E.StepPlan.build([(1, p1, toks)]))
        b = ref.forward(E.StepPlan.build([(1, p1, toks)]))
        errs_sp.append(float((a - b).abs().max() / b.abs().max()))
        p1 += 4
    torch.cuda.synchronize()
    eng.status.check()
    # The prefill logits must agree; a decode step after it can move by several tenths when one
    # router near-tie flips an expert in this small random model (seen at 4 and 8 ranks), so the
    # decode steps are only required to agree closely at least once and never wildly.
    assert errs_sp[0] < 0.2 and min(errs_sp[1:]) < 0.25 and max(errs_sp) < 0.9, errs_sp
    # every rank holds the same KV state after the gathers
    for t in (eng.win, eng.comp, eng.keys):
        got = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        assert all(torch.equal(got[0], g_) for g_ in got)
    say("sequence-parallel prefill ok %s" % errs_sp)
    # ---- 4. speculative decode under a CUDA graph with the fused collectives
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    dec = SpecDecoder(eng, 1, temperature=0.6, top_p=0.95, use_graph=True)
    slots = [DecodeSlot(region=0, length=pos, anchor=5, seed=11)]
    outs = [dec.step(slots) for _ in range(6)]
    eng.status.check()
    flat = [t for o in outs for t in o[0]]
    toks_all = [None] * world
    dist.all_gather_object(toks_all, flat)
    assert all(t == toks_all[0] for t in toks_all), "ranks committed different tokens"
    # ---- 5. tensor-core GEMMs fused with reduce-scatter / all-gather, and the expert-parallel layer
    from titanic_flash_41_b200.parallel.ep import EpMoE
    from titanic_flash_41_b200.parallel.symm import AgWorkspace, RsWorkspace
    M, Nn, Kl = 256 * world, 256, 512
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    xa = torch.randn(M, Kl, device=dev, generator=g).bfloat16()
    wb = (torch.randn(Nn, Kl, device=dev, generator=g) * 0.05).bfloat16()
    rsw = RsWorkspace(M, Nn, device=dev)
    for _ in range(3):
        out = torch.zeros(M // world, Nn, device=dev, dtype=torch.bfloat16)
        rsw.gemm_reduce_scatter(0, xa, wb, out, st.t)
        full = (xa.float() @ wb.float().t()).bfloat16()
        want = torch.empty(M // world, Nn, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(want, full)
        torch.cuda.synchronize()
        st.check()
        assert (out.float() - want.float()).abs().max() <= 0.02 * want.float().abs().max()
    agw = AgWorkspace(0, M, Kl, device=dev, copy_ctas=4)
    for _ in range(3):
        shard = torch.randn(M // world, Kl, device=dev, generator=g).bfloat16()
        a_view, _ = agw.shard()
        a_view.copy_(shard)
        out = torch.zeros(M, Nn, device=dev, dtype=torch.bfloat16)
        agw.allgather_gemm(wb, out, st.t)
        full = torch.empty(M, Kl, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, shard)
        torch.cuda.synchronize()
        st.check()
        want = full.float() @ wb.float().t()
        assert (out.float() - want).abs().max() <= 0.02 * want.abs().max()
    say("gemm + reduce-scatter / all-gather ok")
    d, I, Eg, k, Tl = 512, 256, 8 * world, 2, 40 + rank
    El = Eg // world
    q = [E.quant_mxfp4_device(torch.randn(El, n, kk, device=dev, generator=g) * 0.06)
         for n, kk in ((I, d), (I, d), (d, I))]
    moe = EpMoE(d, I, Eg, k, 64, q[0][0], q[0][1], q[1][0], q[1][1], q[2][0], q[2][1], device=dev)
    for _ in range(2):
        x = torch.randn(Tl, d, device=dev, generator=g).bfloat16()
        ids = torch.stack([torch.randperm(Eg, device=dev, generator=g)[:k] for _ in range(Tl)]).int().contiguous()
        wts = torch.rand(Tl, k, device=dev, generator=g).contiguous()
        out = torch.zeros(Tl, d, device=dev, dtype=torch.bfloat16)
        moe.forward(x, ids, wts, out, st.t)
        want = moe.forward_nccl(x, ids, wts, st.t)
        torch.cuda.synchronize()
        st.check()
        assert float((out.float() - want.float()).norm() / want.float().norm()) < 1e-2
    say("expert-parallel dispatch / combine ok")
    dist.barrier()
    if rank == 0:
        print("MGPU_OK", world, errs, flush=True)
    # tearing down the process group while symmetric-memory mappings are alive can block: the
    # checks are done, leave without the collective teardown
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    try:
        main()
    except BaseException:            # noqa: BLE001  (the launcher only shows its own error: print ours first)
        import traceback
        print("[mgpu] FAILED on rank", os.environ.get("RANK"), flush=True)
        traceback.print_exc(file=sys.stdout)
        sys.stdout.flush()
        os._exit(1)
