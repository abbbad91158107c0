"""Headline benchmark: speculative decode throughput of 4 concurrent conversations at 131,072
tokens of context, and the cold prefill of a 129,553-token prompt, on the full-size random-init
model (43 layers, hidden 4096, 64 heads x 128, 256 MXFP4 experts top-6 + 1 shared, FP8 dense,
vocab 129280, 1-layer draft head depth 3; T = 0.6, top-p = 0.95).

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched with torchrun)

Prints ONE JSON line on rank 0.  Both numbers come from the SAME loop of ``SpecDecoder.step`` calls:
``e2e`` is tokens over the wall time of the loop on the device clock (pinned-memory upload of each
step's metadata, the captured step, the download of its result, host bookkeeping); ``value`` is
the same tokens over the summed device time of the steps alone (CUDA events around every graph
replay).  The decode starts from the KV state that the timed prefill wrote: the prompt is extended
to the decode start and the conversation is copied into the other regions.  Strong scaling: the
model and workload are fixed, N GPUs share them (tensor-parallel attention and expert-parallel
MoE for decode rows, sequence-parallel prefill).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_DECODE_TOK_S = 90.0        # reference: pooled decode at ~131K context (README.md:11)
BASELINE_PREFILL_S = 13.65          # reference: cold 129,553-token prefill (README.md:11)
CONTEXT = 131072
PREFILL_TOKENS = 129553
SESSIONS = 4
DECODE_TOKENS = 512


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, path):
        self.path, self.p = path, None

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self, gpu_index=0):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(5)
        except Exception:
            self.p.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9 or not c[0].isdigit() or int(c[0]) != gpu_index:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            busy = [v for v in sm if v > 0.5 * max(mx)] or sm
            out = {"sm_mhz": busy[len(busy) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Rust crate with prebuilt aarch64/sm_121 kernel bundles and no "
                      "setup.py/pyproject.toml: pip reports 'Directory is not installable'; it refuses any GPU "
                      "that is not CC 12.1 with 48 SMs (src/cuda.rs:774-781)"}))


def synth_state(eng, gen):
    """Fill every region's caches with valid random rows so that decode at CONTEXT reads real bytes."""
    import torch
    dev = eng.dev
    cfg = eng.cfg
    Dh, Di = cfg.head_dim, cfg.index_dim

    def rnd(shape, hi):
        return torch.randint(0, hi, shape, generator=gen, device=dev, dtype=torch.uint8)

    for li in range(eng.win.shape[0]):
        w = eng.win[li]
        w[..., :Dh] = rnd(w[..., :Dh].shape, 0x70) | (rnd(w[..., :Dh].shape, 2) << 7)
        w[..., Dh:Dh + Dh // 32] = 124
    for s in range(eng.comp.shape[0]):
        c = eng.comp[s]
        c[..., :Dh // 2] = rnd(c[..., :Dh // 2].shape, 256)
        c[..., Dh // 2:Dh // 2 + Dh // 16] = 0x30
        k = eng.keys[s]
        k[..., :Di // 2] = rnd(k[..., :Di // 2].shape, 256)
        k[..., Di // 2:Di // 2 + Di // 32] = 124


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--index-heads", type=int, default=0, help="indexer heads (flagship: 8; the reference's geometry has 32)")
    ap.add_argument("--impl", default="own")
    ap.add_argument("--model", default="flash-b200")
    ap.add_argument("--layers", type=int, default=0, help="debug: override the layer count (result is then not a headline number)")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--knockout", default="", help="diagnostic: comma-separated exported kernel names whose launches are "
                    "left out of the captured decode graph (the printed number is then NOT a benchmark value)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--pdl", type=int, default=-1, help="1 / 0: launch kernels with programmatic dependent launch "
                    "(default: the engine configuration's setting)")
    ap.add_argument("--nvtx-step", action="store_true", help="run one extra eager decode step inside the NVTX range "
                    "'tf_decode_step' (a profiler can then list exactly the kernels of a step)")
    ap.add_argument("--graph-clock", action="store_true", help="after the timed steps: capture the decode step once more with a "
                    "device timestamp in front of every kernel call and print where the time goes inside the replayed graph")
    ap.add_argument("--trace", action="store_true", help="print per-kernel time tables of one extra prefill pass and one eager decode step")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    import torch
    import torch.distributed as dist
    from titanic_flash_41_b200.config import NAMED_MODELS, EngineConfig
    from titanic_flash_41_b200.models.engine import Engine
    from titanic_flash_41_b200.parallel.comm import init_distributed
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    from titanic_flash_41_b200.serve.prefill import run_prefill
    from titanic_flash_41_b200.ops import native as native_mod
    import __graft_entry__
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if rank == 0:
        __graft_entry__.build()
    comm = init_distributed("nccl") if world > 1 else init_distributed()
    if world > 1:
        comm.barrier()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    over = {}
    if args.layers:
        over = dict(n_layers=args.layers, kv_source_layers=(0,), index_source_layers=(0,), late_start=-1)
    if args.index_heads:
        over["index_heads"] = args.index_heads
    cfg = NAMED_MODELS[args.model](**over)
    chunk = 16384
    # several ranks: a sequence-parallel prefill chunk spans every rank's slice (up to 65,536 rows), so the
    # slices keep the single-rank kernel shapes and the host launches a quarter as many kernels
    ecfg = EngineConfig(tp=world, regions=SESSIONS, max_context=CONTEXT + 4096, prefill_widths=(chunk,),
                        use_cuda_graphs=not args.no_graph, sp_chunk_rows=min(chunk * world, 65536) if world > 1 else 0)
    if args.pdl >= 0:
        ecfg.pdl = bool(args.pdl)
    t0 = time.time()
    eng = Engine.random_init(cfg, ecfg, comm, device=dev, seed=0, max_chunk=chunk)
    from titanic_flash_41_b200.ops import bigpath
    bigpath.attach(eng)
    if world > 1:
        from titanic_flash_41_b200.parallel import sp
        from titanic_flash_41_b200.parallel.symm import SymmWorkspace
        eng.symm = SymmWorkspace(cfg.hidden, 32, device=dev)
        sp.attach(eng)
    gen = torch.Generator(device=dev).manual_seed(1234)
    synth_state(eng, gen)
    torch.cuda.synchronize()
    init_s = time.time() - t0

    def barrier():
        if world > 1:
            comm.barrier()
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ cold prefill
    prefill_s = None
    if not args.no_prefill:
        cpu_gen = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, cfg.vocab, (args.prefill_tokens,), generator=cpu_gen, dtype=torch.int32)
        if world > 1:
            pt = prompt.to(dev)
            dist.broadcast(pt, 0)
            prompt = pt.cpu()
        run_prefill(eng, 0, prompt[: chunk + 2048], chunk)         # warm-up of every kernel shape and buffer
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run_prefill(eng, 0, prompt, chunk)
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b) / 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_s = float(t)
        if args.trace:
            # a second, untimed pass under the kernel clock: where the prefill time goes
            from titanic_flash_41_b200.utils.trace import KernelClock
            with KernelClock() as kc:
                run_prefill(eng, 0, prompt, chunk)
            if rank == 0:
                print(kc.report(), file=sys.stderr, flush=True)

    # ------------------------------------------------------------------ decode
    start_len = CONTEXT - DECODE_TOKENS
    state_from = "synthetic KV state at 131072 tokens"
    last_hidden = None
    if prefill_s is not None and args.prefill_tokens <= start_len:
        # decode from what the prefill wrote: extend the conversation to the decode start (untimed) and
        # copy it into the other regions
        ext = torch.randint(0, cfg.vocab, (start_len - args.prefill_tokens,), generator=cpu_gen, dtype=torch.int32)
        if world > 1:
            et = ext.to(dev)
            dist.broadcast(et, 0)
            ext = et.cpu()
        if ext.numel():
            run_prefill(eng, 0, ext, chunk, start=args.prefill_tokens)
        torch.cuda.synchronize()
        if eng.status.read()[0] == 0:
            for r in range(1, SESSIONS):
                for t in (eng.win, eng.comp, eng.keys, eng.carry):
                    t[:, r].copy_(t[:, 0])
            if eng.last_hidden is not None:
                last_hidden = eng.last_hidden[-1:].clone()
            state_from = "KV state written by the timed prefill (extended to the decode start, copied to 4 regions)"
        else:
            eng.status.t.zero_()
            synth_state(eng, gen)
    slots = [DecodeSlot(region=r, length=start_len, anchor=100 + r, seed=r + 1) for r in range(SESSIONS)]
    dec = SpecDecoder(eng, SESSIONS, temperature=0.6, top_p=0.95, use_graph=not args.no_graph)
    if last_hidden is not None:
        dec.hidden.copy_(last_hidden.reshape(1, -1)[:, -cfg.hidden:].expand(SESSIONS, cfg.hidden))
    if args.knockout:
        # capture the graph without the named families: the difference to a plain run is what they
        # cost inside the graph, dependent-launch gaps included
        from titanic_flash_41_b200.utils.trace import Knockout
        with Knockout(set(args.knockout.split(","))):
            dec.step(slots)
    launches = dec.count_launches(slots)
    if args.trace:
        # one eager decode step under the kernel clock: where the step time goes
        from titanic_flash_41_b200.utils.trace import KernelClock
        with KernelClock(shapes=True) as kc:
            dec.count_launches(slots)
        if rank == 0:
            print("decode step (eager, per-kernel CUDA events)\n" + kc.report(top=30), file=sys.stderr, flush=True)
    for _ in range(args.warmup):
        dec.step(slots)
    barrier()
    if args.nvtx_step:
        torch.cuda.nvtx.range_push("tf_decode_step")
        dec.count_launches(slots)
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
    if eng.status.read()[0] != 0 and state_from.startswith("KV"):
        # the prefilled state of this random-init model produced non-finite logits: fall back to the
        # synthetic state rather than time a step that reports errors
        eng.status.t.zero_()
        synth_state(eng, gen)
        state_from = "synthetic KV state at 131072 tokens (the prefilled state gave non-finite logits)"
        slots = [DecodeSlot(region=r, length=start_len, anchor=100 + r, seed=r + 1) for r in range(SESSIONS)]
        for _ in range(args.warmup):
            dec.step(slots)
        barrier()
    sampler = ClockSampler(f"/tmp/clocks_{rank}.csv")
    if rank == 0:
        sampler.start()
    # e2e: the public API, upload + graph + download every step
    tok0 = sum(len(s.emitted) for s in slots)
    # exactly `steps` steps, timed in three consecutive segments (their spread is reported)
    nseg = 3 if args.steps >= 30 else 1
    seg_steps = [args.steps // nseg + (1 if i < args.steps % nseg else 0) for i in range(nseg)]
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(nseg + 1)]
    dec.device_events = []
    barrier()
    marks[0].record()
    for i, k in enumerate(seg_steps):
        for _ in range(k):
            dec.step(slots)
        marks[i + 1].record()
    barrier()
    seg_ms = [marks[i].elapsed_time(marks[i + 1]) for i in range(nseg)]
    e2e_ms = marks[0].elapsed_time(marks[nseg])
    tokens = sum(len(s.emitted) for s in slots) - tok0
    # device time of the very same steps: CUDA events around every step's captured graph
    dev_ms = sum(x.elapsed_time(y) for x, y in dec.device_events)
    dec.device_events = None
    clocks = sampler.stop(local) if rank == 0 else {}
    eng.status.check()
    if args.graph_clock and not args.no_graph:
        # a second decoder (the timed one stays as it was): its graph carries a timestamp kernel in front
        # of every kernel call; the table is read after a replay
        from titanic_flash_41_b200.utils.trace import GraphClock
        dec2 = SpecDecoder(eng, SESSIONS, temperature=0.6, top_p=0.95, use_graph=True)
        dec2.hidden.copy_(dec.hidden)
        dec2.clock = GraphClock(device=dev)
        probe = [DecodeSlot(region=s.region, length=s.length, anchor=s.anchor, seed=s.seed) for s in slots]
        for _ in range(3):
            dec2.step(probe)
        if rank == 0:
            print("decode step inside the replayed graph (device timestamps before and after every call; a call's time includes one ~2 us stamp)\n"
                  + dec2.clock.report(top=30), file=sys.stderr, flush=True)
    t = torch.tensor([e2e_ms, dev_ms] + [m / k for m, k in zip(seg_ms, seg_steps)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms, dev_ms = float(t[0]), float(t[1])
    seg_per_step = [round(float(v), 4) for v in t[2:]]
    if rank == 0:
        tok_per_step = tokens / args.steps
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (e2e_ms / 1e3)
        par = f"tp{world}+ep{world}" if world > 1 else "single"
        mem_gb = torch.cuda.max_memory_allocated() / 2 ** 30
        out = {
            "metric": "decode tok/s at 131K ctx; cold 129.5K-token prefill s (max over ranks)",
            "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 4),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / BASELINE_DECODE_TOK_S, 3), "dtype": "bf16",
            "data": "synthetic token ids, random-init weights; decode from: " + state_from,
            "config": {"model": cfg.name, "layers": cfg.n_layers, "global_batch": SESSIONS,
                       "seq_len": CONTEXT, "parallelism": par, "draft_depth": dec.g,
                       "temperature": 0.6, "top_p": 0.95,
                       "tokens_per_step": round(tok_per_step, 3),
                       "index_heads": cfg.index_heads, "index_topk": cfg.index_topk, "late_start": cfg.late_start,
                       "kv_source_layers": list(cfg.kv_source_layers),
                       "index_source_layers": list(cfg.index_source_layers),
                       "prefill": ("sequence-parallel rows" if getattr(eng, "sp", None) is not None else "single rank"),
                       "prefill_chunk_rows": (ecfg.sp_chunk_rows if getattr(eng, "sp", None) is not None else chunk),
                       "prefill_gemm": ("block-scaled by the tensor core (MXFP8 activations x FP8 / MXFP4 weights)"
                                        if ecfg.prefill_mx else "FP8 with fp32 scales per 128, promoted in software"),
                       "sampling": ("rank-local chunks" if dec.ws is not None else "gathered rows"),
                       "programmatic_dependent_launch": native_mod.pdl_enabled(),
                       "l2": "inputs larger than L2 (>= 5 GB of weights touched per step)",
                       "weights": "FP8 dense with power-of-two scales per 128 x 128 block, MXFP4 experts, bf16 head (FP8 draft head)"},
            "prefill_s": None if prefill_s is None else round(prefill_s, 3),
            "prefill_tokens": args.prefill_tokens if prefill_s is not None else None,
            "prefill_vs_baseline": None if prefill_s is None else round(BASELINE_PREFILL_S / prefill_s, 3),
            "e2e": {"value": round(e2e, 2), "unit": "tok/s", "ms_per_step": round(e2e_ms / args.steps, 4),
                    "ms_per_step_segments": seg_per_step,
                    "h2d_bytes_per_step": dec.h2d_bytes_per_step, "d2h_bytes_per_step": dec.d2h_bytes_per_step},
            "gpu_launches": launches * args.steps,
            "gpu_launches_per_step": launches,
            "clocks": clocks, "init_s": round(init_s, 1), "peak_mem_gb": round(mem_gb, 1), "impl": "own",
        }
        if args.knockout:
            out["diagnostic"] = "decode graph captured WITHOUT " + args.knockout + ": not a benchmark value"
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)        # skip the collective teardown (it can block on live peer mappings)


if __name__ == "__main__":
    main()
