"""Command line: ``python -m titanic_flash_41_b200 {serve,bench,stage-weights,probe,launch}``.

``serve`` runs the OpenAI-compatible server on rank 0 and a worker loop on every rank;
``bench`` times prefill and speculative decode; ``stage-weights`` writes this rank's weight atlas,
``verify-staged`` re-reads one and checks its digests, ``pack-engram`` packs an n-gram table;
``probe`` prints the device / peer-access / build facts the engine depends on (reference:
src/main.rs Cli and its subcommands).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import sys
import threading
from typing import Dict, Optional

from .config import EngineConfig, ModelConfig, ServerConfig, flash_b200_config, reference_1017_config, tiny_config

PRESETS = {"tiny": tiny_config, "flash-b200": flash_b200_config, "v41-1017": reference_1017_config}


def model_config(args) -> ModelConfig:
    if args.model_config:
        return ModelConfig.from_json(open(args.model_config).read())
    return PRESETS[args.preset]()


def _common(p: argparse.ArgumentParser) -> None:
    p.add_argument("--preset", choices=sorted(PRESETS), default="tiny")
    p.add_argument("--model-config", help="JSON file written by ModelConfig.to_json")
    p.add_argument("--checkpoint", help="directory of safetensors shards; random weights when absent")
    p.add_argument("--backend", choices=["engine", "oracle"], default="engine")
    p.add_argument("--regions", type=int, default=4)
    p.add_argument("--max-context", type=int, default=131072)
    p.add_argument("--seed", type=int, default=0)


def _cache_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--disk-cache", help="directory for the disk tier of the session cache (every rank uses its own "
                   "sub-directory)")
    p.add_argument("--cache-slots", type=int, default=16, help="entries of the session cache")
    p.add_argument("--device-cache-gib", type=float, default=8.0, help="device memory for cached state images")
    p.add_argument("--host-cache-gib", type=float, default=32.0, help="pinned host memory for parked state images")
    p.add_argument("--checkpoint-tokens", type=int, default=8192, help="spacing of prompt checkpoints; shorter prompts "
                   "leave none")
    p.add_argument("--prefill-slice-ms", type=int, default=500, help="a long prefill yields to a decode step of the "
                   "other conversations this often")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="titanic_flash_41_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="OpenAI-compatible HTTP server")
    _common(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--api-key", default=os.environ.get("TFLASH_API_KEY", ""))
    s.add_argument("--queue-limit", type=int, default=16)
    s.add_argument("--tokenizer", help="tokenizer.json (byte-level BPE); byte tokenizer when absent")
    _cache_flags(s)
    s.add_argument("--event-log", help="JSONL event log path")
    s.add_argument("--no-self-check", action="store_true", help="skip the start-up reproducibility check")
    s.add_argument("--log-confidence", action="store_true", help="event per decode round with the drafter's confidences "
                   "and the proposals verified (models with a confidence head)")
    s.add_argument("--vision", action="store_true", help="accept image parts (the model config must describe a vision "
                   "tower; random tower weights when the checkpoint has none)")
    s.add_argument("--memory-floor-gib", type=float, default=4.0, help="host memory that must stay available; "
                   "requests are refused with 429 below it")
    b = sub.add_parser("bench", help="prefill + decode timing (bench.py of the source tree)")
    b.add_argument("rest", nargs=argparse.REMAINDER)
    w = sub.add_parser("stage-weights", help="write this rank's staged weight atlas")
    _common(w)
    w.add_argument("--out", required=True)
    w.add_argument("--rank", type=int, default=int(os.environ.get("RANK", 0)))
    w.add_argument("--world", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    w.add_argument("--moe-parallel", choices=["ep", "tp"], default="ep")
    sub.add_parser("probe", help="device, peer access and build facts as JSON")
    # ---- protocol / checkpoint utilities (no GPU)
    e = sub.add_parser("encode-chat", help="chat request JSON (file or -) -> rendered prompt and token ids")
    e.add_argument("request")
    e.add_argument("--tokenizer")
    e.add_argument("--vocab", type=int, default=129280)
    dt = sub.add_parser("decode-tokens", help="token ids (JSON list, file or -) -> text")
    dt.add_argument("tokens")
    dt.add_argument("--tokenizer")
    dt.add_argument("--vocab", type=int, default=129280)
    pc = sub.add_parser("parse-completion", help="raw completion text (file or -) -> OpenAI message JSON")
    pc.add_argument("text")
    pc.add_argument("--no-thinking", action="store_true")
    pc.add_argument("--tools", action="store_true")
    cv = sub.add_parser("config-validate", help="validate a model configuration JSON and print its digest")
    cv.add_argument("config")
    sc = sub.add_parser("scan", help="scan a safetensors checkpoint and check it against a model configuration")
    sc.add_argument("checkpoint")
    sc.add_argument("--preset", choices=sorted(PRESETS))
    sc.add_argument("--model-config")
    pl = sub.add_parser("plan", help="per-rank placement of a checkpoint's tensors (replicated / sharded / local experts) "
                        "and the bytes every rank would hold")
    pl.add_argument("checkpoint")
    pl.add_argument("--preset")
    pl.add_argument("--model-config")
    pl.add_argument("--world", type=int, default=8)
    pl.add_argument("--moe-parallel", choices=["ep", "tp"], default="ep")
    pm = sub.add_parser("plan-memory", help="bytes one rank will hold on its GPU (weights, KV state of all regions, scratch, "
                        "score buffer), from the configuration alone")
    pm.add_argument("--preset", choices=sorted(PRESETS), default="flash-b200")
    pm.add_argument("--model-config")
    pm.add_argument("--gpus", type=int, default=1)
    pm.add_argument("--regions", type=int, default=4)
    pm.add_argument("--max-context", type=int, default=131072)
    pm.add_argument("--chunk", type=int, default=16384, help="rows of a prefill chunk on one rank")
    pm.add_argument("--device-cache-gib", type=float, default=8.0, help="device budget of the session cache")
    pm.add_argument("--device-gib", type=float, default=180.0, help="memory of one GPU")
    bf = sub.add_parser("bench-frontend", help="protocol front end alone: normalise + render + tokenise a growing conversation, "
                        "cold and with the region cache warm (requests / s, prompt tokens / s)")
    bf.add_argument("--tokenizer")
    bf.add_argument("--vocab", type=int, default=129280)
    bf.add_argument("--turns", type=int, default=16)
    bf.add_argument("--chars", type=int, default=20000, help="characters of document text added per turn")
    pf = sub.add_parser("preflight", help="checks before a cohort is launched: GPUs and peer access, the native library and "
                        "its provenance, the memory plan, the ports, the checkpoint (reference: deploy/fleet.py preflight)")
    pf.add_argument("--preset", choices=sorted(PRESETS), default="flash-b200")
    pf.add_argument("--model-config")
    pf.add_argument("--checkpoint")
    pf.add_argument("--gpus", type=int, default=1)
    pf.add_argument("--regions", type=int, default=4)
    pf.add_argument("--max-context", type=int, default=131072)
    pf.add_argument("--port", type=int, default=8000)
    pf.add_argument("--master-port", type=int, default=29511)
    pf.add_argument("--device-cache-gib", type=float, default=8.0)
    rf = sub.add_parser("run-file", help="file-driven finite run: requests from a JSONL file through the serving stack "
                        "(scheduler, worker, cache), results to a JSONL file; no HTTP")
    _common(rf)
    rf.add_argument("--requests", required=True, help='JSONL: {"id", "tokens" | "messages", "max_tokens", "temperature", '
                    '"top_p", "seed"} per line')
    rf.add_argument("--out", required=True)
    rf.add_argument("--tokenizer")
    _cache_flags(rf)
    vs = sub.add_parser("verify-staged", help="re-read a staged weight atlas and check every tensor's digest "
                        "(and, with a preset / model config, that it was staged for that model)")
    vs.add_argument("dir")
    vs.add_argument("--preset")
    vs.add_argument("--model-config")
    pe = sub.add_parser("pack-engram", help="pack an n-gram memory table ([rows, 256] values: .npy, or a tensor of a "
                        "safetensors checkpoint) into the 264-byte MXFP8 row file the row store reads")
    pe.add_argument("source", help=".npy file, or a checkpoint directory / .safetensors file with --tensor")
    pe.add_argument("--tensor", help="tensor name inside the checkpoint")
    pe.add_argument("--out", required=True)
    pe.add_argument("--row-start", type=int, default=0, help="first row of this shard in the whole table")
    sm = sub.add_parser("smoke", help="live endpoint check: health, models, one completion, one stream")
    sm.add_argument("--url", default="http://127.0.0.1:8000")
    sm.add_argument("--api-key", default=os.environ.get("TFLASH_API_KEY", ""))
    l = sub.add_parser("launch", help="start one process per GPU running a sub-command")
    l.add_argument("--gpus", type=int, required=True)
    l.add_argument("--master-port", type=int, default=29511)
    l.add_argument("rest", nargs=argparse.REMAINDER)
    return ap


def probe() -> dict:
    import torch
    from .utils import build
    out = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(),
           "library": str(build.OUT / "libtflash_cuda.so"), "devices": []}
    out["library_built"] = os.path.exists(out["library"])
    out["build"] = build.provenance()          # sources changed since the libraries were built show up here
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            out["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                   "memory_gib": round(p.total_memory / 2 ** 30, 1),
                                   "peers": [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)]})
        out["sm_100"] = all(d["sm"] == "10.0" for d in out["devices"])
    return out


def stage_weights(args) -> dict:
    from .formats import atlas, layout
    from .formats.safetensors import Checkpoint
    cfg = model_config(args)
    if not args.checkpoint:
        raise SystemExit("stage-weights needs --checkpoint")
    ck = Checkpoint.scan(args.checkpoint)
    layout.validate_checkpoint(ck, cfg)
    plan = layout.RankPlan.build(ck, cfg, args.rank, args.world, args.moe_parallel)
    meta = atlas.stage(ck, cfg, plan, os.path.join(args.out, f"rank{args.rank}"))
    return {"rank": args.rank, "world": args.world, "bytes": meta["bytes"], "tensors": len(meta["tensors"]),
            "sha256": meta["sha256"]}


def engine_config(args, world: int) -> EngineConfig:
    """Runtime policy from the command line (what the serving stack reads: regions, context, cache
    tiers, checkpoint spacing, prefill slices)."""
    g = lambda name, default: getattr(args, name, default)
    return EngineConfig(tp=world, regions=args.regions, max_context=args.max_context,
                        session_slots=g("cache_slots", 16), session_budget_bytes=int(g("device_cache_gib", 8.0) * 2 ** 30),
                        host_tier_bytes=int(g("host_cache_gib", 32.0) * 2 ** 30), disk_tier_dir=g("disk_cache", None) or "",
                        checkpoint_min_tokens=g("checkpoint_tokens", 8192), prefill_slice_ms=g("prefill_slice_ms", 500))


def make_session_cache(ecfg: EngineConfig, rank: int):
    """The session cache with its three tiers as the policy describes them."""
    from .serve.session_cache import SessionCache
    disk = None
    if ecfg.disk_tier_dir:
        from .serve.state_image import DiskTier
        disk = DiskTier(os.path.join(ecfg.disk_tier_dir, f"rank{rank}"))
    return SessionCache(slots=ecfg.session_slots, budget_bytes=ecfg.session_budget_bytes, disk=disk,
                        host_budget_bytes=ecfg.host_tier_bytes)


def make_backend(args, cfg: ModelConfig, comm):
    import torch
    from .serve.backend import EngineBackend, OracleBackend
    if args.backend == "oracle":
        from .models import loader, oracle
        from .formats.safetensors import Checkpoint
        W = (loader.checkpoint_weights(Checkpoint.scan(args.checkpoint), cfg) if args.checkpoint
             else oracle.init_weights(cfg, seed=args.seed))
        return OracleBackend(cfg, W, regions=args.regions, max_context=args.max_context, comm=comm)
    from .models.engine import Engine
    world = getattr(comm, "world", 1)
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    ecfg = engine_config(args, world)
    if world > 1:
        ecfg.sp_chunk_rows = min(max(ecfg.prefill_widths) * world, 65536)      # sequence-parallel chunks span the ranks' slices
    import time as _time
    t_load = _time.monotonic()
    if args.checkpoint:
        # streamed, digest-checked, in the stored formats: never more than one layer on the host
        from .models import stream_loader
        eng = stream_loader.load_engine(args.checkpoint, cfg, ecfg, comm, device=dev)
    else:
        eng = Engine.random_init(cfg, ecfg, comm, device=dev, seed=args.seed)
    # one structured line per rank: what was loaded, how long it took, what it occupies
    import json as _json
    import sys as _sys
    print(_json.dumps({"event": "engine_loaded", "rank": getattr(comm, "rank", 0), "world": world,
                       "source": args.checkpoint or "random-init", "load_s": round(_time.monotonic() - t_load, 3),
                       "bytes": eng.memory_report()}), file=_sys.stderr, flush=True)
    if world > 1:
        # the product runs what the benchmark measures: decode rows go through the fused
        # GEMV / combine + all-reduce kernels over peer memory, not NCCL all-reduces per sublayer
        from .parallel.symm import SymmWorkspace
        eng.symm = SymmWorkspace(cfg.hidden, 32, device=dev)
    backend = EngineBackend(eng)          # attaches the tensor-core prefill path
    if world > 1:
        from .parallel import sp
        sp.attach(eng)                    # prefill chunks split by rows over the ranks
    return backend


def policy_digest(cfg: ModelConfig, args, world: int) -> str:
    """Digest of everything the ranks must agree on before they load: the model geometry and the
    serving policy values that decide regions, context, backend and sampling determinism."""
    import hashlib
    from .config import agree_digest
    h = hashlib.sha256(agree_digest([cfg]).encode())
    for k in ("backend", "regions", "max_context", "seed", "checkpoint", "vision", "cache_slots", "device_cache_gib",
              "host_cache_gib", "checkpoint_tokens", "prefill_slice_ms"):
        h.update(f"{k}={getattr(args, k, None)!r};".encode())
    h.update(f"world={world}".encode())
    return h.hexdigest()


def serve_main(args) -> int:
    from .api.server import Frontend, Server, serve
    from .api.tokenizer import load_tokenizer
    from .parallel.comm import LocalComm, init_distributed
    from .parallel.control import ControlChannel
    from .serve.scheduler import Scheduler
    from .serve.session_cache import SessionCache
    from .serve.worker import Worker
    from .utils.event_log import EventLog
    cfg = model_config(args)
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    comm = init_distributed() if world > 1 else LocalComm()
    control = None
    scfg = ServerConfig(host=args.host, port=args.port, api_key=args.api_key, queue_limit=args.queue_limit,
                        max_admitted=args.regions)
    if world > 1:
        control = ControlChannel.connect(rank, world, "127.0.0.1", int(os.environ.get("TFLASH_CONTROL_PORT", 29512)),
                                         os.environ.get("TFLASH_CONTROL_TICKET", "").encode())
        # every value that shapes the deterministic command stream must be the same on all ranks
        # before anything is loaded (reference: src/resident_worker.rs:5935-5977)
        control.agree(policy_digest(cfg, args, world).encode())
    backend = make_backend(args, cfg, comm)
    log = EventLog(args.event_log) if args.event_log else EventLog()
    tok = load_tokenizer(args.tokenizer, cfg.vocab)
    sched = Scheduler(scfg.max_admitted, scfg.queue_limit, scfg.background_queue_limit) if rank == 0 else None
    vision_front = span_encoder = None
    if args.vision:
        if cfg.vision is None:
            raise SystemExit("--vision needs a model configuration with a vision tower")
        from .api.media import SpanEncoder, VisionFrontend
        vision_front = VisionFrontend(tok.image_id, cfg.vision.image_token_id, cfg.vision.max_image_tokens)
        if rank == 0:
            from .models import vision as V
            VW = V.init_vision_weights(cfg.vision, cfg.hidden, args.seed)
            tower = (V.VisionTower(cfg.vision, cfg.hidden, VW, device=backend.device) if args.backend == "engine"
                     else V.VisionOracle(cfg.vision, cfg.hidden, VW))
            span_encoder = SpanEncoder(tower)
    from .utils.health import Health, Watchdog, control_probe, status_probe
    health = Health()
    policy_cfg = engine_config(args, world)
    worker = Worker(backend, sched, make_session_cache(policy_cfg, rank), eos_id=getattr(tok, "eos_id", 1), log=log,
                    control=control, rank=rank, span_encoder=span_encoder, health=health,
                    log_confidence=getattr(args, "log_confidence", False),
                    prefill_slice_s=policy_cfg.prefill_slice_ms / 1e3, checkpoint_min=policy_cfg.checkpoint_min_tokens,
                    checkpoint_align=policy_cfg.checkpoint_min_tokens)
    probes = {"control": control_probe(control)}
    if hasattr(backend, "status_snapshot"):
        probes["device"] = status_probe(backend.status_snapshot)
    if world > 1:
        # host-side heartbeat of the cohort on its own gloo group: a poisoned rank poisons the others
        # within a second, a rank that died is noticed without waiting for a device collective to time out
        from .utils.health import CohortHeartbeat
        heartbeat = CohortHeartbeat(health, CohortHeartbeat.make_group(timeout=20.0), rank, world, interval=1.0)
        heartbeat.start()
        probes["cohort"] = heartbeat.probe()
    Watchdog(health, probes, on_poison=lambda rec: log.log("poisoned", incident=True, **rec)).start()
    if not args.no_self_check and backend.regions >= 2:
        # every rank runs the same fixture (its collectives line up); raises before the server reports ready
        from .serve.warmup import self_check
        log.log("self_check", **self_check(backend))
    if rank != 0:
        worker.run_forever()
        if world > 1:
            heartbeat.stop()
        return 0
    from .utils.memory import host_admission
    server = Server(scfg, Frontend(tok, args.max_context, vision=vision_front, default_max_tokens=scfg.default_max_tokens), sched, log,
                    memory=host_admission(int(args.memory_floor_gib * 2 ** 30),
                                          log=lambda rec: log.log(rec.get("event", "memory"), incident=True,
                                                                  **{k: v for k, v in rec.items() if k != "event"})),
                    health=health.state)
    t = threading.Thread(target=worker.run_forever, daemon=True)
    t.start()
    server.ready(f"{cfg.digest()[:12]}/{backend.name}/tp{world}")
    asyncio.run(serve(server))
    sched.close()
    t.join(timeout=30)
    if world > 1:
        heartbeat.stop()
    return 0


def preflight(args) -> dict:
    """Everything that can be checked before ``launch``: each check is (ok, detail); ``ok`` is their AND."""
    import socket

    from .utils import build
    from .utils.memory import plan_device_memory
    checks: Dict[str, dict] = {}
    info = probe()
    n = len(info["devices"])
    checks["gpus"] = {"ok": n >= args.gpus, "detail": f"{n} visible, {args.gpus} wanted"}
    if n >= args.gpus and args.gpus > 1:
        missing = [(d["index"], j) for d in info["devices"][: args.gpus] for j in range(args.gpus)
                   if j != d["index"] and j not in d["peers"]]
        checks["peer_access"] = {"ok": not missing, "detail": f"{len(missing)} device pairs without peer access"}
    if n:
        checks["sm_100"] = {"ok": bool(info.get("sm_100")), "detail": sorted({d["sm"] for d in info["devices"]})}
    prov = build.provenance()
    checks["library"] = {"ok": info["library_built"] and prov["recorded"] and not prov["stale_sources"] and prov["libraries_match"],
                         "detail": {"built": info["library_built"], "stale_sources": prov["stale_sources"],
                                    "libraries_match": prov["libraries_match"]}}
    cfg = model_config(args)
    w = args.gpus
    ecfg = EngineConfig(tp=w, regions=args.regions, max_context=args.max_context,
                        sp_chunk_rows=min(max(EngineConfig().prefill_widths) * w, 65536) if w > 1 else 0)
    need = plan_device_memory(cfg, ecfg, w)["total"] / 2 ** 30 + args.device_cache_gib + (7.0 if w == 1 else 21.0)
    have = min((d["memory_gib"] for d in info["devices"][: args.gpus]), default=180.0)
    checks["memory"] = {"ok": need <= have, "detail": f"{need:.1f} GiB needed per GPU, {have:.1f} GiB there"}
    checks["context"] = {"ok": args.max_context <= cfg.max_positions, "detail": f"{args.max_context} of {cfg.max_positions} positions"}
    busy = []
    for port in (args.port, args.master_port, args.master_port + 1):
        with socket.socket() as so:
            try:
                so.bind(("127.0.0.1", port))
            except OSError:
                busy.append(port)
    checks["ports"] = {"ok": not busy, "detail": {"busy": busy}}
    if args.checkpoint:
        try:
            from .formats import layout
            from .formats.safetensors import Checkpoint
            ck = Checkpoint.scan(args.checkpoint)
            layout.validate_checkpoint(ck, cfg)
            checks["checkpoint"] = {"ok": True, "detail": f"{len(ck.tensors)} tensors match the configuration"}
        except Exception as e:  # noqa: BLE001  (a preflight reports, it does not raise)
            checks["checkpoint"] = {"ok": False, "detail": str(e)}
    return {"ok": all(c["ok"] for c in checks.values()), "checks": checks}


def run_file(args) -> int:
    """Requests from a JSONL file through the serving stack of ONE process (the reference's
    file-driven finite run, src/main.rs resident-token-peer): every request is admitted by the
    scheduler, served by the worker (prefix reuse, batching, speculative decode) and written with its
    tokens, finish reason and timings."""
    from .api import protocol as P
    from .api.tokenizer import load_tokenizer
    from .parallel.comm import LocalComm
    from .serve.scheduler import Job, Scheduler
    from .serve.worker import Worker
    cfg = model_config(args)
    backend = make_backend(args, cfg, LocalComm())
    tok = load_tokenizer(args.tokenizer, cfg.vocab)
    sched = Scheduler(args.regions, 1 << 16, 1 << 16)
    ecfg = engine_config(args, 1)
    worker = Worker(backend, sched, make_session_cache(ecfg, 0), eos_id=getattr(tok, "eos_id", 1),
                    checkpoint_min=ecfg.checkpoint_min_tokens, checkpoint_align=ecfg.checkpoint_min_tokens)
    results: Dict[str, dict] = {}
    order = []
    for n, line in enumerate(l for l in open(args.requests).read().splitlines() if l.strip()):
        req = json.loads(line)
        jid = str(req.get("id", n))
        if "tokens" in req:
            toks = [int(t) for t in req["tokens"]]
        else:
            toks = tok.encode(P.render_chat(P.normalize_chat_request({"messages": req["messages"], "model": "x"})))
        limit = P.resolve_max_tokens(req.get("max_tokens"), len(toks), args.max_context, 256)
        results[jid] = {"id": jid, "prompt_tokens": len(toks), "tokens": []}
        order.append(jid)

        def emit(kind, payload, _r=results[jid]):
            if kind == "tokens":
                _r["tokens"] += list(payload)
            elif kind == "ready":
                _r["cache_n"], _r["prompt_ms"] = payload["cache_n"], payload["prompt_ms"]
            elif kind == "done":
                _r.update(finish_reason=payload["finish_reason"], decode_tok_s=payload.get("decode_tok_s"))
            elif kind == "error":
                _r.update(finish_reason="error", error=payload)
        sched.submit(Job(jid, toks, limit, temperature=float(req.get("temperature", 0.0)), top_p=float(req.get("top_p", 1.0)),
                         seed=int(req.get("seed", 0)), emit=emit))
    sched.close()
    worker._pending = []
    while worker.running:
        worker.run_once(0.0)
    with open(args.out, "w") as f:
        for jid in order:
            r = results[jid]
            r["text"] = tok.decode(r["tokens"])
            f.write(json.dumps(r) + "\n")
    done = sum(1 for r in results.values() if r.get("finish_reason") not in (None, "error"))
    print(json.dumps({"requests": len(order), "completed": done, "out": args.out}))
    return 0 if done == len(order) else 1


def _read(arg: str) -> str:
    return sys.stdin.read() if arg == "-" else open(arg).read()


def utility(args) -> Optional[int]:
    """Protocol / checkpoint sub-commands; returns None when ``args.cmd`` is not one of them."""
    from .api import protocol as P
    from .api.tokenizer import load_tokenizer
    if args.cmd == "encode-chat":
        req = P.normalize_chat_request(json.loads(_read(args.request)))
        text = P.render_chat(req)
        tok = load_tokenizer(args.tokenizer, args.vocab)
        ids = tok.encode(text)
        print(json.dumps({"prompt": text, "tokens": ids, "n": len(ids), "images": len(P.image_parts(req.messages))}))
        return 0
    if args.cmd == "decode-tokens":
        tok = load_tokenizer(args.tokenizer, args.vocab)
        print(json.dumps({"text": tok.decode(json.loads(_read(args.tokens)))}))
        return 0
    if args.cmd == "parse-completion":
        out = P.parse_completion(_read(args.text), not args.no_thinking, args.tools, "stop", 0, 0, "cli")
        print(json.dumps(out))
        return 0
    if args.cmd == "config-validate":
        cfg = ModelConfig.from_json(_read(args.config))
        print(json.dumps({"ok": True, "name": cfg.name, "digest": cfg.digest(), "layers": cfg.n_layers,
                          "experts": cfg.n_experts, "kv_bytes_per_token": cfg.window_kv_bytes}))
        return 0
    if args.cmd == "scan":
        from .formats import layout
        from .formats.safetensors import Checkpoint
        ck = Checkpoint.scan(args.checkpoint)
        out = {"tensors": len(ck.tensors), "bytes": sum(t.nbytes for t in ck.tensors.values()),
               "dtypes": sorted({t.dtype for t in ck.tensors.values()})}
        if args.preset or args.model_config:
            layout.validate_checkpoint(ck, model_config(args))
            out["matches_config"] = True
        print(json.dumps(out))
        return 0
    if args.cmd == "plan":
        from .formats import layout
        from .formats.safetensors import Checkpoint
        ck = Checkpoint.scan(args.checkpoint)
        cfg = model_config(args) if (args.preset or args.model_config) else None
        if cfg is None:
            raise SystemExit("plan needs --preset or --model-config")
        layout.validate_checkpoint(ck, cfg)
        ranks = []
        for r in range(args.world):
            plan = layout.RankPlan.build(ck, cfg, r, args.world, args.moe_parallel)
            kinds: dict = {}
            for p_ in plan.entries.values():
                kinds[p_.kind] = kinds.get(p_.kind, 0) + 1
            ranks.append({"rank": r, "bytes": plan.local_bytes(ck), "tensors_by_kind": kinds})
        print(json.dumps({"world": args.world, "moe_parallel": args.moe_parallel, "checkpoint_bytes":
                          sum(t.nbytes for t in ck.tensors.values()), "ranks": ranks}))
        return 0
    if args.cmd == "run-file":
        return run_file(args)
    if args.cmd == "bench-frontend":
        import random
        import time as _t

        from .api.server import Frontend
        from .api.tokenizer import load_tokenizer
        tok = load_tokenizer(args.tokenizer, args.vocab)
        rnd = random.Random(0)
        words = ["".join(rnd.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rnd.randrange(2, 10))) for _ in range(4000)]
        doc = lambda: " ".join(rnd.choice(words) for _ in range(args.chars // 6))
        msgs = [{"role": "system", "content": "You are terse."}]
        out = {}
        for name in ("cold", "warm"):
            front = Frontend(tok, 1 << 22)
            rnd.seed(1)
            conv = list(msgs)
            t0, ntok, nreq = _t.perf_counter(), 0, 0
            for turn in range(args.turns):
                conv = conv + [{"role": "user", "content": doc()}]
                if name == "cold":
                    front = Frontend(tok, 1 << 22)           # nothing remembered between requests
                _, tokens, _, _ = front.prepare({"model": "x", "messages": conv, "max_tokens": 8})
                ntok += len(tokens)
                nreq += 1
                conv = conv + [{"role": "assistant", "content": "ok"}]
            dt = _t.perf_counter() - t0
            out[name] = {"requests_per_s": round(nreq / dt, 2), "prompt_tokens_per_s": round(ntok / dt), "last_prompt_tokens": len(tokens)}
        print(json.dumps(out))
        return 0
    if args.cmd == "preflight":
        report = preflight(args)
        print(json.dumps(report))
        return 0 if report["ok"] else 1
    if args.cmd == "plan-memory":
        from .utils.memory import plan_device_memory
        cfg = model_config(args)
        w = args.gpus
        ecfg = EngineConfig(tp=w, regions=args.regions, max_context=args.max_context, prefill_widths=(args.chunk,),
                            sp_chunk_rows=min(args.chunk * w, 65536) if w > 1 else 0)
        plan = plan_device_memory(cfg, ecfg, w, chunk=args.chunk)
        gib = {k: round(v / 2 ** 30, 2) for k, v in plan.items()}
        gib["session_cache_budget"] = args.device_cache_gib
        # measured on the runs recorded with the benchmarks: the row buffers of every other launch shape,
        # the staging of the sequence-parallel exchanges and allocator slack add 7 GiB (one GPU) to 21 GiB (four)
        gib["allowance_other_shapes_and_allocator"] = 7.0 if w == 1 else 21.0
        need = gib["total"] + gib["session_cache_budget"] + gib["allowance_other_shapes_and_allocator"]
        print(json.dumps({"model": cfg.name, "gpus": w, "regions": args.regions, "max_context": args.max_context,
                          "gib_per_gpu": gib, "needed_gib": round(need, 1), "device_gib": args.device_gib,
                          "fits": need <= args.device_gib}))
        return 0
    if args.cmd == "verify-staged":
        from .formats import atlas
        cfg = model_config(args) if (args.preset or args.model_config) else None
        tensors = atlas.load_staged(args.dir, cfg, verify=True)          # raises on a size, digest or model mismatch
        print(json.dumps({"ok": True, "tensors": len(tensors), "bytes": sum(t.numel() * t.element_size() for t in tensors.values()),
                          "digest": atlas.device_digest(tensors), "model_checked": cfg is not None}))
        return 0
    if args.cmd == "pack-engram":
        import numpy as np
        import torch
        from .models import engram as EG
        if args.tensor:
            from .formats.safetensors import Checkpoint
            vals = Checkpoint.scan(args.source).read(args.tensor).float()
        else:
            vals = torch.from_numpy(np.load(args.source)).float()
        if vals.dim() != 2 or vals.shape[1] != 256:
            raise SystemExit(f"pack-engram: expected [rows, 256] values, got {tuple(vals.shape)}")
        packed = EG.pack_rows(vals)
        EG.write_table(args.out, packed, args.row_start)
        err = float((EG.unpack_rows(packed) - vals).abs().max())
        print(json.dumps({"rows": int(vals.shape[0]), "row_start": args.row_start, "bytes": int(packed.numel()),
                          "max_abs_error": err}))
        return 0
    if args.cmd == "smoke":
        from .api.smoke import run as smoke_run
        return smoke_run(args.url, args.api_key)
    return None


def main(argv: Optional[list] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.cmd in ("encode-chat", "decode-tokens", "parse-completion", "config-validate", "scan", "smoke", "verify-staged",
                    "pack-engram", "plan", "run-file", "plan-memory", "preflight", "bench-frontend"):
        return utility(args)
    if args.cmd == "probe":
        print(json.dumps(probe()))
        return 0
    if args.cmd == "stage-weights":
        print(json.dumps(stage_weights(args)))
        return 0
    if args.cmd == "bench":
        import runpy
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        sys.argv = [os.path.join(root, "bench.py")] + [a for a in args.rest if a != "--"]
        runpy.run_path(sys.argv[0], run_name="__main__")
        return 0
    if args.cmd == "launch":
        from .launcher import launch
        rest = [a for a in args.rest if a != "--"]
        return launch(["-m", "titanic_flash_41_b200", *rest], args.gpus, args.master_port)
    return serve_main(args)
