"""Long-context serving stress: several conversations grown in large appended chunks, short
requests interleaved, then every conversation resumed with a small follow-up.

    python benchmarks/bench_long_context.py [--sessions 4] [--target 131072] [--grow 65536]
                                            [--short 17] [--follow 2048] [--backend engine|oracle]

Runs the real serving stack (scheduler, worker, session cache with host and disk tiers, state
images, engine): in one process, or as one rank per GPU under torchrun

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        benchmarks/bench_long_context.py --target 1000000 --grow 65536

where rank 0 owns the scheduler and the clients and every rank runs a worker that follows rank 0's
commands over the control channel (tensor-parallel decode through the fused all-reduce kernels,
sequence-parallel prefill).  Reports, as one JSON line: time to first token of the resumed
turns, the share of prompt tokens served from cached state, and where the restored images came
from (device / host / disk).  The oracle backend with ``--preset tiny`` runs the same script on
the CPU in seconds (used by the tests).
"""
import argparse
import json
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from titanic_flash_41_b200.config import EngineConfig, flash_b200_config, tiny_config  # noqa: E402
from titanic_flash_41_b200.serve.scheduler import Job, Scheduler  # noqa: E402
from titanic_flash_41_b200.serve.session_cache import SessionCache  # noqa: E402
from titanic_flash_41_b200.serve.state_image import DiskTier  # noqa: E402
from titanic_flash_41_b200.serve.worker import Worker  # noqa: E402


def small_gpu_config(world: int = 1):
    """A model the CUDA engine runs in seconds (the geometry of the GPU tests), for trials of this script."""
    from titanic_flash_41_b200.config import DraftConfig, ModelConfig, RopeConfig
    return ModelConfig(name="small", n_layers=3, hidden=512, vocab=2048, n_heads=4 * world if world > 4 else 4, head_dim=128,
                       window=32, compress_ratio=4, kv_source_layers=(0,), index_source_layers=(0, 2), index_heads=4,
                       index_dim=128, index_topk=16, n_experts=8, topk=2, moe_inter=512, n_shared=1,
                       shared_inter=max(256, 128 * world), scoring="sqrtsoftplus", router_bias=True, route_scale=1.5,
                       swiglu_limit=10.0, rope=RopeConfig(theta=10000.0, compress_theta=160000.0, dim=64),
                       dense_quant="fp8_block128", expert_quant="mxfp4", kv_quant="v41", init_std=0.05,
                       draft=DraftConfig(layers=1, depth=3))


def build_backend(a, comm=None):
    if a.backend == "oracle":
        from titanic_flash_41_b200.models import oracle
        from titanic_flash_41_b200.serve.backend import OracleBackend
        cfg = tiny_config()
        kw = {"comm": comm} if comm is not None else {}
        return cfg, OracleBackend(cfg, oracle.init_weights(cfg, 0), regions=a.regions, max_context=a.target + a.follow + 512,
                                  chunk=a.chunk, **kw)
    from titanic_flash_41_b200.models.engine import Engine
    from titanic_flash_41_b200.serve.backend import EngineBackend
    world = comm.world if comm is not None else 1
    cfg = {"flash-b200": flash_b200_config, "tiny": tiny_config, "small": lambda: small_gpu_config(world)}[a.preset]()
    ecfg = EngineConfig(tp=world, regions=a.regions, max_context=a.target + a.follow + 4096, prefill_widths=(a.chunk,),
                        sp_chunk_rows=min(a.chunk * world, 65536) if world > 1 else 0)
    if a.preset == "small":
        ecfg.reference_matmul = True          # the trial model's prompt tails are shorter than a tensor-core tile
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    eng = Engine.random_init(cfg, ecfg, comm, device=dev, seed=0, max_chunk=a.chunk)
    if world > 1:
        from titanic_flash_41_b200.parallel.symm import SymmWorkspace
        eng.symm = SymmWorkspace(cfg.hidden, 32, device=dev)
    backend = EngineBackend(eng, chunk=a.chunk)
    if world > 1:
        from titanic_flash_41_b200.parallel import sp
        sp.attach(eng)
    return cfg, backend


def drain(w, limit=100000):
    for _ in range(limit):
        if w.run_once(0.0) == "idle" and not w.active and w.sched.waiting() == 0:
            return
    raise RuntimeError("worker did not drain")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="engine", choices=["engine", "oracle"])
    ap.add_argument("--preset", default="flash-b200")
    ap.add_argument("--sessions", type=int, default=4)
    ap.add_argument("--regions", type=int, default=4)
    ap.add_argument("--target", type=int, default=131072, help="context each conversation is grown to")
    ap.add_argument("--grow", type=int, default=65536, help="tokens appended per turn")
    ap.add_argument("--short", type=int, default=17, help="short requests interleaved between the long turns")
    ap.add_argument("--short-tokens", type=int, default=200)
    ap.add_argument("--follow", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=8)
    ap.add_argument("--chunk", type=int, default=16384)
    ap.add_argument("--cache-slots", type=int, default=64)
    ap.add_argument("--checkpoint", type=int, default=65536, help="prompt checkpoint spacing (tokens)")
    ap.add_argument("--device-cache-gb", type=float, default=2.0)
    ap.add_argument("--host-cache-gb", type=float, default=16.0)
    ap.add_argument("--progress", action="store_true", help="one line per turn on stderr (elapsed time, context)")
    a = ap.parse_args(argv)
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    comm = control = None
    if world > 1:
        import torch.distributed as dist
        from titanic_flash_41_b200.parallel.comm import DistComm
        from titanic_flash_41_b200.parallel.control import ControlChannel
        if a.backend == "oracle":
            dist.init_process_group("gloo")          # the CPU plumbing run of the same driver
        else:
            torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
            dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
        comm = DistComm()
        control = ControlChannel.connect(rank, world, "127.0.0.1", int(os.environ["MASTER_PORT"]) + 13, b"long-context", 600.0)
    t_load = time.monotonic()
    cfg, backend = build_backend(a, comm)
    if a.progress and rank == 0:
        print(f"[long-context] model ready in {time.monotonic() - t_load:.1f} s", file=sys.stderr, flush=True)
    tmp = tempfile.mkdtemp(prefix="tflash_tier_")
    disk = DiskTier(tmp)
    cache = SessionCache(slots=a.cache_slots, budget_bytes=int(a.device_cache_gb * 2 ** 30), disk=disk,
                         host_budget_bytes=int(a.host_cache_gb * 2 ** 30), park_after=2)
    sched = Scheduler(a.regions, 64, 8) if rank == 0 else None
    w = Worker(backend, sched, cache, eos_id=-1, checkpoint_min=a.checkpoint, checkpoint_align=a.checkpoint,
               control=control, rank=rank)
    if rank != 0:
        # follow rank 0's commands until it says stop; the numbers are rank 0's
        w._pending = []
        while w.running:
            w.run_once(0.05)
        _leave(world, disk, tmp)
        return None
    g = torch.Generator().manual_seed(0)
    rand = lambda n: torch.randint(3, cfg.vocab, (n,), generator=g).tolist()
    events = {}

    def submit(jid, toks, n):
        events[jid] = []
        sched.submit(Job(jid, list(toks), n, emit=lambda k, p, _j=jid: events[_j].append((k, p, time.monotonic())),
                         temperature=0.6, top_p=0.95, seed=len(events)))

    def ready(jid):
        return [p for k, p, _ in events[jid] if k == "ready"][0]

    def tokens_of(jid):
        return [t for k, p, _ in events[jid] if k == "tokens" for t in p]

    convs = [[] for _ in range(a.sessions)]
    turns = max(1, a.target // a.grow)
    shorts_left = a.short
    t_start = time.monotonic()
    prompt_total = reused_total = 0
    for turn in range(turns):
        for s in range(a.sessions):
            convs[s] = convs[s] + rand(a.grow)
            jid = f"s{s}t{turn}"
            submit(jid, convs[s], a.new_tokens)
            # interleave short requests so that regions are recycled and images get displaced
            if shorts_left > 0 and (turn * a.sessions + s) % max(1, (turns * a.sessions) // max(1, a.short)) == 0:
                submit(f"short{shorts_left}", rand(a.short_tokens), a.new_tokens)
                shorts_left -= 1
        while shorts_left > 0 and turn == turns - 1:
            submit(f"short{shorts_left}", rand(a.short_tokens), a.new_tokens)
            shorts_left -= 1
        drain(w)
        if a.progress:
            print(f"[long-context] turn {turn + 1}/{turns}: context {len(convs[0])}, {time.monotonic() - t_start:.1f} s",
                  file=sys.stderr, flush=True)
        for s in range(a.sessions):
            jid = f"s{s}t{turn}"
            r = ready(jid)
            prompt_total += r["prompt_n"] + r["cache_n"]
            reused_total += r["cache_n"]
            convs[s] = convs[s] + tokens_of(jid)
    grow_s = time.monotonic() - t_start
    # let idle steps write images behind to the lower tiers (on every rank: idle commands travel too)
    for _ in range(64):
        w.run_once(0.0)
    tiers_before = {t: sum(1 for e in cache.entries if e.image.tier == t) for t in ("device", "host", "disk")}
    # ---- resume every conversation with a short follow-up
    ttft, resumed = [], []
    for s in range(a.sessions):
        jid = f"s{s}resume"
        t0 = time.monotonic()
        submit(jid, convs[s] + rand(a.follow), a.new_tokens)
        drain(w)
        first = [t for k, p, t in events[jid] if k == "tokens"][0]
        ttft.append(first - t0)
        r = ready(jid)
        resumed.append(r)
        prompt_total += r["prompt_n"] + r["cache_n"]
        reused_total += r["cache_n"]
    out = {"metric": "resume TTFT (s) and cached-prefix share, long-context serving stress", "backend": a.backend,
           "sessions": a.sessions, "context": len(convs[0]), "grow": a.grow, "short_requests": a.short,
           "grow_phase_s": round(grow_s, 3), "resume_ttft_s": [round(t, 4) for t in ttft],
           "resume_ttft_mean_s": round(sum(ttft) / len(ttft), 4),
           "resume_cached_tokens": [r["cache_n"] for r in resumed], "resume_prefilled_tokens": [r["prompt_n"] for r in resumed],
           "reused_token_share": round(reused_total / max(1, prompt_total), 4), "cache_stats": dict(cache.stats),
           "image_tiers_before_resume": tiers_before, "n_gpus": world, "model": a.preset,
           "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if a.backend == "engine" else None,
           "data": "synthetic token ids, random-init weights"}
    print(json.dumps(out), flush=True)
    if world > 1:
        sched.close()
        w._pending = []
        while w.running:                      # the stop command reaches the other ranks through the worker
            w.run_once(0.05)
    _leave(world, disk, tmp)
    return out


def _leave(world, disk, tmp):
    disk.reset_dir()
    os.rmdir(tmp)
    if world > 1:
        import torch.distributed as dist
        if torch.cuda.is_available() and dist.get_backend() == "nccl":
            torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)          # no collective teardown while symmetric-memory mappings are alive


if __name__ == "__main__":
    main()
