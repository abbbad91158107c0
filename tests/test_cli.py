"""Command line, launcher and an end-to-end HTTP request against the oracle backend (CPU)."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest
import requests

from titanic_flash_41_b200 import cli, launcher
from titanic_flash_41_b200.config import tiny_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_probe_and_parser():
    info = cli.probe()
    assert "torch" in info and isinstance(info["devices"], list)
    a = cli.build_parser().parse_args(["serve", "--preset", "tiny", "--backend", "oracle", "--port", "1234"])
    assert a.cmd == "serve" and a.port == 1234 and cli.model_config(a).digest() == tiny_config().digest()


def test_build_provenance_notices_changed_sources(tmp_path, monkeypatch):
    """The build writes what it was built from; a source that changed afterwards is reported (a stale
    library would otherwise be loaded without a word)."""
    import shutil

    from titanic_flash_41_b200.utils import build
    src, out = tmp_path / "csrc", tmp_path / "lib"
    src.mkdir()
    out.mkdir()
    (src / "a.cu").write_text("// a\n")
    (src / "b.cuh").write_text("// b\n")
    (out / "libx.so").write_bytes(b"\x7fELF fake")
    monkeypatch.setattr(build, "CSRC", src)
    monkeypatch.setattr(build, "OUT", out)
    monkeypatch.setattr(build, "_run", lambda cmd: "nvcc: fake\nBuild fake_1.0")
    assert build.provenance() == {"recorded": False, "stale_sources": [], "libraries_match": False}
    build._write_provenance("nvcc")
    ok = build.provenance()
    assert ok["recorded"] and ok["stale_sources"] == [] and ok["libraries_match"] and ok["nvcc"] == "Build fake_1.0"
    (src / "a.cu").write_text("// a changed\n")
    (src / "c.cu").write_text("// new\n")
    assert build.provenance()["stale_sources"] == ["a.cu", "c.cu"]
    (out / "libx.so").write_bytes(b"other")
    assert build.provenance()["libraries_match"] is False
    shutil.rmtree(src)


def test_stage_weights_command(tmp_path, capsys):
    from titanic_flash_41_b200.models import loader, oracle
    cfg = tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4")
    cfgp = os.path.join(str(tmp_path), "cfg.json")
    open(cfgp, "w").write(cfg.to_json())
    ck = os.path.join(str(tmp_path), "ck")
    loader.export_checkpoint(oracle.init_weights(cfg, seed=1), cfg, ck)
    rc = cli.main(["stage-weights", "--model-config", cfgp, "--checkpoint", ck, "--out", os.path.join(str(tmp_path), "st"),
                   "--rank", "1", "--world", "2"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["rank"] == 1 and out["bytes"] > 0
    assert os.path.exists(os.path.join(str(tmp_path), "st", "rank1", "atlas.bin"))


def test_launcher_env_and_failure_propagation(tmp_path):
    env = launcher.rank_env(3, 8, 29000, "t", base={})
    assert env["RANK"] == "3" and env["WORLD_SIZE"] == "8" and env["MASTER_ADDR"] == "127.0.0.1"
    assert len(launcher.cores_for(1, 4, n_cores=16)) == 4 and launcher.cores_for(1, 4, n_cores=16)[0] == 4
    out = os.path.join(str(tmp_path), "r")
    ok = ["-c", f"import os; open(r'{out}' + os.environ['RANK'], 'w').write(os.environ['TFLASH_CONTROL_TICKET'])"]
    assert launcher.launch(ok, 2, master_port=_free_port(), pin=False, poll_s=0.02) == 0
    assert open(out + "0").read() == open(out + "1").read() != ""
    bad = ["-c", "import os, sys, time; time.sleep(0 if os.environ['RANK'] == '1' else 30); sys.exit(7)"]
    t0 = time.time()
    assert launcher.launch(bad, 2, master_port=_free_port(), pin=False, poll_s=0.02) == 7
    assert time.time() - t0 < 20            # rank 0 was stopped, not waited for


@pytest.mark.timeout(180)
def test_serve_end_to_end_oracle_backend():
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.Popen([sys.executable, "-m", "titanic_flash_41_b200", "serve", "--preset", "tiny", "--backend", "oracle",
                          "--port", str(port), "--max-context", "512", "--regions", "2", "--api-key", "k"],
                         env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        base = f"http://127.0.0.1:{port}"
        for _ in range(600):
            try:
                if requests.get(base + "/health", timeout=1).status_code == 200:
                    break
            except requests.RequestException:
                pass
            assert p.poll() is None, p.stdout.read().decode()[-2000:]
            time.sleep(0.1)
        h = {"Authorization": "Bearer k"}
        assert requests.post(base + "/v1/chat/completions", json={}, timeout=5).status_code == 401
        body = {"model": "x", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0}
        r = requests.post(base + "/v1/chat/completions", json=body, headers=h, timeout=120)
        assert r.status_code == 200, r.text
        j = r.json()
        assert j["usage"]["completion_tokens"] >= 1 and j["choices"][0]["finish_reason"] in ("stop", "length")
        r2 = requests.post(base + "/v1/chat/completions", json=body, headers=h, timeout=120).json()
        assert r2["choices"][0]["message"] == j["choices"][0]["message"]          # greedy is deterministic
        # the smoke client: health, models, a completion, a stream, two turns of the context transport
        from titanic_flash_41_b200.api import smoke
        assert smoke.run(base, "k") == 0
        assert requests.post(base + "/_native/shutdown", headers=h, timeout=5).status_code == 200
        assert p.wait(timeout=60) == 0
    finally:
        if p.poll() is None:
            p.kill()


def test_protocol_and_checkpoint_utilities(tmp_path, capsys):
    req = os.path.join(str(tmp_path), "req.json")
    open(req, "w").write(json.dumps({"model": "m", "messages": [{"role": "user", "content": "hello"}]}))
    assert cli.main(["encode-chat", req, "--vocab", "1024"]) == 0
    enc = json.loads(capsys.readouterr().out)
    assert enc["n"] == len(enc["tokens"]) > 0 and "hello" in enc["prompt"]
    toks = os.path.join(str(tmp_path), "t.json")
    open(toks, "w").write(json.dumps(enc["tokens"]))
    assert cli.main(["decode-tokens", toks, "--vocab", "1024"]) == 0
    assert "hello" in json.loads(capsys.readouterr().out)["text"]
    txt = os.path.join(str(tmp_path), "c.txt")
    open(txt, "w").write("thinking...</think>\\n\\nThe answer.")
    assert cli.main(["parse-completion", txt]) == 0
    msg = json.loads(capsys.readouterr().out)
    assert "The answer." in json.dumps(msg)
    cfgp = os.path.join(str(tmp_path), "cfg.json")
    open(cfgp, "w").write(tiny_config().to_json())
    assert cli.main(["config-validate", cfgp]) == 0
    assert json.loads(capsys.readouterr().out)["digest"] == tiny_config().digest()
    from titanic_flash_41_b200.models import loader, oracle
    cfg = tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4")
    open(cfgp, "w").write(cfg.to_json())
    ck = os.path.join(str(tmp_path), "ck")
    loader.export_checkpoint(oracle.init_weights(cfg, seed=1), cfg, ck)
    assert cli.main(["scan", ck, "--model-config", cfgp]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["matches_config"] and "F8_E4M3" in out["dtypes"]


def test_serve_policy_flags_reach_the_session_cache(tmp_path):
    """--disk-cache / --cache-slots / --device-cache-gib / --host-cache-gib / --checkpoint-tokens shape the
    cache and the worker the server builds (every rank its own disk directory)."""
    from titanic_flash_41_b200 import cli
    args = cli.build_parser().parse_args(["serve", "--preset", "tiny", "--disk-cache", str(tmp_path), "--cache-slots", "5",
                                          "--device-cache-gib", "0.5", "--host-cache-gib", "2", "--checkpoint-tokens", "1024",
                                          "--prefill-slice-ms", "250"])
    ecfg = cli.engine_config(args, world=2)
    assert (ecfg.session_slots, ecfg.session_budget_bytes, ecfg.host_tier_bytes) == (5, 1 << 29, 2 << 30)
    assert ecfg.checkpoint_min_tokens == 1024 and ecfg.prefill_slice_ms == 250 and ecfg.tp == 2
    cache = cli.make_session_cache(ecfg, rank=1)
    assert cache.slots == 5 and cache.budget == 1 << 29 and cache.host_budget == 2 << 30
    assert cache.disk is not None and cache.disk.dir.endswith("rank1") and (tmp_path / "rank1").is_dir()
    none = cli.make_session_cache(cli.engine_config(cli.build_parser().parse_args(["serve", "--preset", "tiny"]), 1), 0)
    assert none.disk is None and none.slots == 16
    # ranks that were started with different cache policies must not form a cohort
    other = cli.build_parser().parse_args(["serve", "--preset", "tiny", "--cache-slots", "6"])
    cfg = cli.model_config(args)
    assert cli.policy_digest(cfg, args, 2) != cli.policy_digest(cfg, other, 2)


@pytest.mark.timeout(300)
def test_launch_two_cpu_ranks_serve_end_to_end():
    """``launch --gpus 2 -- serve`` on CPU (gloo, oracle backend split over two ranks): the ranks agree
    on the policy, connect the control channel in whatever order they start, run the start-up check and
    the cohort heartbeat, rank 0 answers over HTTP, and a shutdown request ends both ranks with code 0."""
    port, mport = _free_port(), _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.Popen([sys.executable, "-m", "titanic_flash_41_b200", "launch", "--gpus", "2", "--master-port", str(mport),
                          "--", "serve", "--preset", "tiny", "--backend", "oracle", "--port", str(port),
                          "--max-context", "512", "--regions", "2", "--api-key", "k"],
                         env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        base = f"http://127.0.0.1:{port}"
        for _ in range(1200):
            try:
                if requests.get(base + "/health", timeout=1).status_code == 200:
                    break
            except requests.RequestException:
                pass
            assert p.poll() is None, p.stdout.read().decode()[-3000:]
            time.sleep(0.1)
        h = {"Authorization": "Bearer k"}
        body = {"model": "x", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 5, "temperature": 0}
        r = requests.post(base + "/v1/chat/completions", json=body, headers=h, timeout=120)
        assert r.status_code == 200, r.text
        again = requests.post(base + "/v1/chat/completions", json=body, headers=h, timeout=120).json()
        assert again["choices"][0]["message"] == r.json()["choices"][0]["message"]
        health = requests.get(base + "/health", timeout=5).json()
        assert health["status"] == "ready" and health["cohort"]["poisoned"] is False, health
        assert requests.post(base + "/_native/shutdown", headers=h, timeout=5).status_code == 200
        assert p.wait(timeout=90) == 0, p.stdout.read().decode()[-3000:]
    finally:
        if p.poll() is None:
            p.kill()


def test_verify_staged_and_pack_engram_commands(tmp_path, capsys):
    """Weight tools: a staged atlas is re-read and its digests checked (a flipped byte or another model is
    refused); an n-gram table is packed into the row file the row store reads."""
    import numpy as np
    import torch

    from titanic_flash_41_b200.formats.safetensors import CheckpointError
    from titanic_flash_41_b200.models import engram as EG
    from titanic_flash_41_b200.models import loader, oracle
    cfg = tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4")
    cfgp = os.path.join(str(tmp_path), "cfg.json")
    open(cfgp, "w").write(cfg.to_json())
    ck, st = os.path.join(str(tmp_path), "ck"), os.path.join(str(tmp_path), "st")
    loader.export_checkpoint(oracle.init_weights(cfg, seed=1), cfg, ck)
    assert cli.main(["stage-weights", "--model-config", cfgp, "--checkpoint", ck, "--out", st, "--rank", "0", "--world", "1"]) == 0
    capsys.readouterr()
    d = os.path.join(st, "rank0")
    assert cli.main(["verify-staged", d, "--model-config", cfgp]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["ok"] and out["tensors"] > 10 and out["model_checked"] and len(out["digest"]) == 64
    other = os.path.join(str(tmp_path), "other.json")
    open(other, "w").write(tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4", n_layers=3).to_json())
    with pytest.raises(CheckpointError):
        cli.main(["verify-staged", d, "--model-config", other])
    with open(os.path.join(d, "atlas.bin"), "r+b") as f:
        f.seek(100)
        b = f.read(1)
        f.seek(100)
        f.write(bytes([b[0] ^ 0x40]))
    with pytest.raises(CheckpointError):
        cli.main(["verify-staged", d])
    # ---- n-gram table
    vals = torch.randn(37, 256) * 3
    np.save(os.path.join(str(tmp_path), "t.npy"), vals.numpy())
    tab = os.path.join(str(tmp_path), "t.engram")
    assert cli.main(["pack-engram", os.path.join(str(tmp_path), "t.npy"), "--out", tab, "--row-start", "100"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["rows"] == 37 and out["row_start"] == 100 and out["bytes"] == 37 * 264 and out["max_abs_error"] < 0.5
    packed, start = EG.read_table(tab)
    assert start == 100 and torch.equal(packed, EG.pack_rows(vals))
    with pytest.raises(SystemExit):
        np.save(os.path.join(str(tmp_path), "bad.npy"), np.zeros((4, 100), dtype=np.float32))
        cli.main(["pack-engram", os.path.join(str(tmp_path), "bad.npy"), "--out", tab])


def test_plan_and_run_file_commands(tmp_path, capsys):
    """`plan`: bytes and tensor kinds per rank of a checkpoint; `run-file`: a JSONL of requests through the
    serving stack without HTTP (a repeated prompt is served from the cache, greedy results repeat)."""
    from titanic_flash_41_b200.models import loader, oracle
    cfg = tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4")
    cfgp = os.path.join(str(tmp_path), "cfg.json")
    open(cfgp, "w").write(cfg.to_json())
    ck = os.path.join(str(tmp_path), "ck")
    loader.export_checkpoint(oracle.init_weights(cfg, seed=1), cfg, ck)
    assert cli.main(["plan", ck, "--model-config", cfgp, "--world", "2"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["world"] == 2 and len(out["ranks"]) == 2
    assert all(0 < r["bytes"] < out["checkpoint_bytes"] for r in out["ranks"])
    assert sum(r["bytes"] for r in out["ranks"]) >= out["checkpoint_bytes"]          # replicated tensors count twice
    assert "expert_local" in out["ranks"][0]["tensors_by_kind"] and "shard" in out["ranks"][0]["tensors_by_kind"]
    # ---- file-driven run on the CPU oracle
    reqs = os.path.join(str(tmp_path), "reqs.jsonl")
    prompt = [5 + (i * 37) % 900 for i in range(200)]
    with open(reqs, "w") as f:
        f.write(json.dumps({"id": "a", "tokens": prompt, "max_tokens": 6}) + "\n")
        f.write(json.dumps({"id": "b", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0.8,
                            "seed": 3}) + "\n")
        f.write(json.dumps({"id": "c", "tokens": prompt, "max_tokens": 6}) + "\n")
    res = os.path.join(str(tmp_path), "res.jsonl")
    assert cli.main(["run-file", "--preset", "tiny", "--backend", "oracle", "--regions", "1", "--max-context", "256",
                     "--requests", reqs, "--out", res, "--checkpoint-tokens", "16"]) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary == {"requests": 3, "completed": 3, "out": res}
    rows = {r["id"]: r for r in map(json.loads, open(res).read().splitlines())}
    assert rows["a"]["tokens"] == rows["c"]["tokens"] and len(rows["a"]["tokens"]) == 6
    assert rows["a"]["cache_n"] == 0 and rows["c"]["cache_n"] >= 64              # the repeat came from the cache
    assert rows["b"]["finish_reason"] in ("stop", "length") and isinstance(rows["b"]["text"], str)


def test_preflight_reports_every_check(tmp_path, capsys, monkeypatch):
    """`preflight`: the checks a launch depends on, each with its finding; on a box without GPUs the GPU
    check fails and the command exits 1; with a fake probe of eight peered B200s everything passes; a busy
    port, an oversized context and a checkpoint of another model are each reported."""
    import socket

    from titanic_flash_41_b200.models import loader, oracle
    assert cli.main(["preflight", "--gpus", "2", "--port", str(_free_port()), "--master-port", str(_free_port())]) == 1
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["ok"] is False and out["checks"]["gpus"]["ok"] is False and out["checks"]["library"]["ok"] is True
    devices = [{"index": i, "name": "B200", "sm": "10.0", "sms": 148, "memory_gib": 178.4,
                "peers": [j for j in range(8) if j != i]} for i in range(8)]
    monkeypatch.setattr(cli, "probe", lambda: {"devices": devices, "sm_100": True, "library_built": True})
    p1, p2 = _free_port(), _free_port()
    assert cli.main(["preflight", "--gpus", "8", "--max-context", "1000000", "--port", str(p1), "--master-port", str(p2)]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["ok"] and set(out["checks"]) >= {"gpus", "peer_access", "sm_100", "library", "memory", "context", "ports"}
    # one GPU cannot hold the model plus a large session cache; a taken port; more context than the model has positions
    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        taken = so.getsockname()[1]
        assert cli.main(["preflight", "--gpus", "1", "--device-cache-gib", "40", "--port", str(taken), "--master-port", str(p2),
                         "--max-context", "2000000"]) == 1
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["checks"]
    assert not out["memory"]["ok"] and not out["ports"]["ok"] and taken in out["ports"]["detail"]["busy"] and not out["context"]["ok"]
    # a checkpoint that does not match the configuration
    cfg = tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4")
    ck = os.path.join(str(tmp_path), "ck")
    loader.export_checkpoint(oracle.init_weights(cfg, seed=1), cfg, ck)
    assert cli.main(["preflight", "--gpus", "1", "--preset", "flash-b200", "--checkpoint", ck, "--port", str(p1),
                     "--master-port", str(p2)]) == 1
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["checks"]
    assert out["checkpoint"]["ok"] is False and out["gpus"]["ok"] is True


def test_bench_frontend_command(capsys):
    assert cli.main(["bench-frontend", "--turns", "4", "--chars", "3000", "--vocab", "1024"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["cold"]["last_prompt_tokens"] == out["warm"]["last_prompt_tokens"] > 1000
    assert out["warm"]["prompt_tokens_per_s"] > out["cold"]["prompt_tokens_per_s"] > 0      # the region cache pays
