"""Tensor-parallel SERVING on real GPUs, launched by torchrun (one rank per GPU): the stack that
``launch --gpus N -- serve`` builds -- control channel, a worker per rank following rank 0's commands,
the engine backend with the fused all-reduce workspace and the sequence-parallel prefill -- driven by
a scheduler on rank 0.  Checks: requests complete; a repeated prompt is served from its cached image
and yields exactly the tokens of the first run; an appended turn reuses its prefix; every rank took
the same commands and holds the same KV state; no kernel reported a problem."""
import os
import sys
import threading
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from titanic_flash_41_b200.config import DraftConfig, EngineConfig  # noqa: E402
from titanic_flash_41_b200.models import engine as E  # noqa: E402
from titanic_flash_41_b200.models import oracle  # noqa: E402
from titanic_flash_41_b200.parallel import sp as SP  # noqa: E402
from titanic_flash_41_b200.parallel.comm import DistComm  # noqa: E402
from titanic_flash_41_b200.parallel.control import ControlChannel  # noqa: E402
from titanic_flash_41_b200.parallel.symm import SymmWorkspace  # noqa: E402
from titanic_flash_41_b200.serve.backend import EngineBackend  # noqa: E402
from titanic_flash_41_b200.serve.scheduler import Job, Scheduler  # noqa: E402
from titanic_flash_41_b200.serve.session_cache import SessionCache  # noqa: E402
from titanic_flash_41_b200.serve.worker import Worker  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    comm = DistComm()
    control = ControlChannel.connect(rank, world, "127.0.0.1", int(os.environ["MASTER_PORT"]) + 11, b"mgpu-serve", 60.0)
    from tests.test_engine_gpu import small_config
    cfg = small_config(n_heads=4 * world if world > 4 else 4, shared_inter=max(256, 128 * world), moe_inter=512,
                       draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    chunk = max(128, 64 * world)
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=4096, prefill_widths=(chunk,),
                        key_sharded_index_min=8, sp_chunk_rows=2 * chunk)
    eng = E.Engine.from_weights(cfg, ecfg, W, comm=comm, device=dev)
    eng.symm = SymmWorkspace(cfg.hidden, 32, device=dev, spin_limit=2_000_000)
    backend = EngineBackend(eng, chunk=chunk)
    assert SP.attach(eng) is not None
    sched = Scheduler(2, 8, 2) if rank == 0 else None
    # the host-side heartbeat of the cohort runs beside the serving loop, on its own gloo group
    from titanic_flash_41_b200.utils.health import CohortHeartbeat, Health
    health = Health()
    heartbeat = CohortHeartbeat(health, CohortHeartbeat.make_group(timeout=30.0), rank, world, interval=0.2)
    heartbeat.start()
    worker = Worker(backend, sched, SessionCache(slots=8, budget_bytes=1 << 30), eos_id=-1, control=control, rank=rank,
                    checkpoint_min=chunk, checkpoint_align=chunk, health=health)
    events, failure, shared = {}, [], {}

    def submit(jid, toks, n, **kw):
        events[jid] = []
        sched.submit(Job(jid, list(toks), n, emit=lambda k, p, _j=jid: events[_j].append((k, p)), **kw))

    def wait(jid, limit=120.0):
        t0 = time.time()
        while time.time() - t0 < limit:
            if any(k in ("done", "error") for k, _ in events[jid]):
                return
            time.sleep(0.005)
        raise TimeoutError(jid)

    toks_of = lambda jid: [t for k, p in events[jid] if k == "tokens" for t in p]
    ready_of = lambda jid: [p for k, p in events[jid] if k == "ready"][0]

    def client():
        """Rank 0: the requests of two clients, in an order that exercises batching, reuse and resume."""
        try:
            g = torch.Generator().manual_seed(5)
            rand = lambda n: torch.randint(3, cfg.vocab, (n,), generator=g).tolist()
            long_prompt, short_prompt = rand(3 * chunk + 37), rand(50)
            submit("long", long_prompt, 13, temperature=0.0, top_p=1.0, seed=1)
            submit("short", short_prompt, 10, temperature=0.7, top_p=0.9, seed=2)          # decodes beside the long prefill
            wait("long")
            wait("short")
            submit("again", long_prompt, 13, temperature=0.0, top_p=1.0, seed=1)           # served from the cached image
            wait("again")
            # appended turn: the cached prefix ends inside a compressor group (421 + 12 committed tokens), so the
            # new part starts on the tensor-parallel path and continues split over the ranks
            follow = long_prompt + toks_of("long") + rand(3 * chunk)
            shared["follow"] = follow
            submit("follow", follow, 6, temperature=0.6, top_p=0.95, seed=3)
            wait("follow")
        except BaseException as e:  # noqa: BLE001
            failure.append(e)
        finally:
            sched.close()

    if rank == 0:
        th = threading.Thread(target=client)
        th.start()
    worker._pending = []
    while worker.running:
        worker.run_once(0.05)
    if rank == 0:
        th.join(30)
        assert not failure, failure
        for jid in ("long", "short", "again", "follow"):
            assert any(k == "done" for k, _ in events[jid]), (jid, events[jid][-2:])
        assert len(toks_of("long")) == 13 and len(toks_of("short")) == 10 and len(toks_of("follow")) == 6
        assert toks_of("again") == toks_of("long"), (toks_of("again"), toks_of("long"))
        assert ready_of("long")["cache_n"] == 0
        assert ready_of("again")["cache_n"] >= 3 * chunk and ready_of("again")["prompt_n"] <= chunk
        assert ready_of("follow")["cache_n"] == 3 * chunk + 37 + 12
    torch.cuda.synchronize()
    eng.status.check()
    assert health.ok and heartbeat.rounds > 0 and heartbeat.failed is None, (health.state(), heartbeat.rounds)
    # every rank took the same commands ...
    kinds = [(e["kind"], e.get("id")) for e in worker.log.snapshot(4096)["events"] if e["kind"] in ("begin", "finish")]
    all_kinds = [None] * world
    dist.all_gather_object(all_kinds, kinds)
    assert all(k == all_kinds[0] for k in all_kinds) and len(kinds) >= 8, all_kinds
    # the appended turn ran sequence-parallel after its unaligned head, and left the state that a
    # prefill of the whole conversation from position 0 leaves
    assert len(eng.sp._plans) > 0
    box = [shared.get("follow"), next((e["region"] for e in worker.log.snapshot(4096)["events"]
                                       if e["kind"] == "begin" and e.get("id") == "follow"), None)]
    dist.broadcast_object_list(box, src=0)
    follow, region = box
    from titanic_flash_41_b200.serve.prefill import run_prefill
    run_prefill(eng, 1 - region, torch.tensor(follow, dtype=torch.int32), chunk)
    torch.cuda.synchronize()
    eng.status.check()
    nC = len(follow) // cfg.compress_ratio
    for t in (eng.comp, eng.keys):
        same = (t[:, region, :nC] == t[:, 1 - region, :nC]).float().mean()
        assert same > 0.95, float(same)
    # ... and every rank holds the same KV state
    for t in (eng.win, eng.comp, eng.keys):
        got = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(got, t)
        assert all(torch.equal(got[0], g_) for g_ in got)
    heartbeat.stop()
    dist.barrier()
    if rank == 0:
        print("MGPU_SERVE_OK", world, ready_of("again"), ready_of("follow"), flush=True)
    sys.stdout.flush()
    os._exit(0)          # no collective teardown while symmetric-memory mappings are alive


if __name__ == "__main__":
    try:
        main()
    except BaseException:            # noqa: BLE001  (the launcher only shows its own error: print ours first)
        import traceback
        print("[mgpu-serve] FAILED on rank", os.environ.get("RANK"), flush=True)
        traceback.print_exc(file=sys.stdout)
        sys.stdout.flush()
        os._exit(1)
