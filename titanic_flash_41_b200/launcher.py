"""One process per GPU on one node.

``launch`` starts ``world`` copies of a module with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* and a
shared control ticket in the environment, pins each to the cores nearest its GPU when the
topology is known, forwards SIGTERM / SIGINT to the exact PIDs it started, and supervises the
cohort: a rank that fails stops the others at once; a rank that leaves cleanly while the others
keep running gives them ``grace_s`` to follow (a coordinated shutdown), after which they are
stopped too and the launch reports an incomplete cohort -- a tensor-parallel job cannot serve
with a rank missing (reference: cohort health loop and coordinated stop, deploy/fleet.py:255,
:437-458; per-rank environment of run-ds41-demo.sh).
"""
from __future__ import annotations

import os
import secrets
import signal
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence


def rank_env(rank: int, world: int, master_port: int, ticket: str, base: Optional[Dict[str, str]] = None
             ) -> Dict[str, str]:
    env = dict(base if base is not None else os.environ)
    env.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world),
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(master_port), TFLASH_CONTROL_TICKET=ticket,
               TFLASH_CONTROL_PORT=str(master_port + 1))
    env.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")
    env.setdefault("OMP_NUM_THREADS", "4")
    return env


def cores_for(rank: int, world: int, n_cores: Optional[int] = None) -> List[int]:
    """An even split of the visible cores; rank r gets the r-th contiguous block."""
    try:
        cores = sorted(os.sched_getaffinity(0))
    except AttributeError:
        cores = list(range(n_cores or os.cpu_count() or 1))
    if n_cores is not None:
        cores = list(range(n_cores))
    per = max(1, len(cores) // world)
    block = cores[rank * per:(rank + 1) * per]
    return block or cores


INCOMPLETE = 70          # exit code: a rank left and the rest had to be stopped


def launch(argv: Sequence[str], world: int, master_port: int = 29511, pin: bool = True,
           poll_s: float = 0.2, grace_s: float = 15.0, term_s: float = 10.0) -> int:
    ticket = secrets.token_hex(16)
    procs: List[subprocess.Popen] = []
    for r in range(world):
        env = rank_env(r, world, master_port, ticket)

        def pre(r=r):
            if pin:
                try:
                    os.sched_setaffinity(0, cores_for(r, world))
                except (AttributeError, OSError):
                    pass
        procs.append(subprocess.Popen([sys.executable, *argv], env=env, preexec_fn=pre))

    def forward(sig, _frm):
        for p in procs:
            if p.poll() is None:
                p.send_signal(sig)
    old = {s: signal.signal(s, forward) for s in (signal.SIGTERM, signal.SIGINT)}
    code = 0
    try:
        live = set(range(world))
        first_exit: Optional[float] = None
        stopping: Optional[float] = None
        while live:
            for r in list(live):
                rc = procs[r].poll()
                if rc is None:
                    continue
                live.discard(r)
                if first_exit is None:
                    first_exit = time.monotonic()
                if rc != 0 and code == 0:
                    code = rc
                    stopping = stopping or time.monotonic()
                    for q in live:                       # a rank failed: the job cannot continue
                        procs[q].terminate()
            now = time.monotonic()
            if live and stopping is None and first_exit is not None and now - first_exit > grace_s:
                # a rank left cleanly and the others did not follow: stop them, report the cohort incomplete
                code = code or INCOMPLETE
                stopping = now
                for q in live:
                    procs[q].terminate()
            if live and stopping is not None and now - stopping > term_s:
                for q in live:                           # SIGTERM was not enough
                    procs[q].kill()
            time.sleep(poll_s)
    finally:
        for s, h in old.items():
            signal.signal(s, h)
        for p in procs:
            if p.poll() is None:
                p.kill()
    return code
