"""Memory admission against fake pools, and the stall-counter reader."""
import json
import os

import pytest

from titanic_flash_41_b200.utils import memory as M


def test_admission_floor_reservations_and_refusal_record():
    pool = {"free": 100}
    recs = []
    adm = M.Admission(lambda: pool["free"], floor=30, name="fake", log=recs.append)
    assert adm.headroom() == 70 and adm.fits(70) and not adm.fits(71)
    with adm.reserve(50, "image") as r:
        assert adm.headroom() == 20
        with pytest.raises(M.CapacityError):
            adm.reserve(21, "input")
        assert recs[-1]["event"] == "allocation_refused" and recs[-1]["what"] == "input" and recs[-1]["headroom"] == 20
        r2 = adm.reserve(20)
        r2.release()
        r2.release()                      # idempotent
    assert adm.headroom() == 70
    pool["free"] = 25                     # the pool shrank below the floor: nothing fits
    assert not adm.fits(1)


def test_host_available_honours_cgroup(tmp_path):
    mi = os.path.join(str(tmp_path), "meminfo")
    open(mi, "w").write("MemTotal: 100 kB\nMemAvailable:    2048 kB\n")
    cg = os.path.join(str(tmp_path), "cg")
    os.makedirs(cg)
    assert M.host_available(mi, cg) == 2048 * 1024
    open(os.path.join(cg, "memory.max"), "w").write("1000000\n")
    open(os.path.join(cg, "memory.current"), "w").write("400000\n")
    assert M.host_available(mi, cg) == 600000
    open(os.path.join(cg, "memory.max"), "w").write("max\n")
    assert M.host_available(mi, cg) == 2048 * 1024


def test_pressure_snapshot_and_delta(tmp_path):
    root = str(tmp_path)
    for res, tot in (("memory", 100), ("io", 5), ("cpu", 7)):
        open(os.path.join(root, res), "w").write(f"some avg10=0.00 avg60=0.00 avg300=0.00 total={tot}\nfull avg10=0 total=1\n")
    a = M.pressure_snapshot(root)
    assert a["memory_us"] == 100 and a["io_us"] == 5
    open(os.path.join(root, "memory"), "w").write("some avg10=0.00 total=350\n")
    d = M.pressure_delta(a, M.pressure_snapshot(root))
    assert d["memory_us"] == 250 and d["io_us"] == 0
    assert isinstance(M.pressure_snapshot("/nonexistent"), dict)


def test_device_memory_plan_scales_as_the_engine_allocates():
    """The planner's arithmetic: experts split over the ranks, a sequence-parallel prefill adds the
    unsharded dense matrices of the encoder layers, compressed KV grows with the context, and the
    flagship on one GPU lands under its measured peak (161.5 GiB) with the experts at 140 GiB."""
    from titanic_flash_41_b200.config import EngineConfig, flash_b200_config
    from titanic_flash_41_b200.utils.memory import plan_device_memory
    cfg = flash_b200_config()
    mk = lambda w, ctx: EngineConfig(tp=w, regions=4, max_context=ctx, prefill_widths=(16384,),
                                     sp_chunk_rows=min(16384 * w, 65536) if w > 1 else 0)
    one, eight = plan_device_memory(cfg, mk(1, 135168), 1), plan_device_memory(cfg, mk(8, 135168), 8)
    layers = cfg.n_layers + cfg.draft.layers
    per_expert = 3 * (cfg.moe_inter * cfg.hidden // 2 + cfg.moe_inter * cfg.hidden // 32)
    assert one["expert_weights"] == layers * cfg.n_experts * per_expert and eight["expert_weights"] * 8 == one["expert_weights"]
    assert abs(one["expert_weights"] / 2 ** 30 - 140.25) < 0.01
    assert one["dense_unsharded_for_sp"] == 0 and 1.5 * 2 ** 30 < eight["dense_unsharded_for_sp"] < 2.5 * 2 ** 30
    assert 140 * 2 ** 30 < one["total"] < 161.5 * 2 ** 30 and one["total"] == sum(v for k, v in one.items() if k != "total")
    long = plan_device_memory(cfg, mk(8, 1_006_144), 8)
    grow = long["kv_state"] - eight["kv_state"]
    per_entry = len(cfg.kv_source_layers) * 4 * (cfg.compressed_kv_bytes + cfg.index_key_bytes)
    assert grow == per_entry * (1_006_144 // 4 - 135168 // 4)
    assert long["total"] < 40 * 2 ** 30                       # a million-token context on eight GPUs is far from 180 GB


def test_plan_memory_command(capsys):
    from titanic_flash_41_b200 import cli
    assert cli.main(["plan-memory", "--gpus", "1"]) == 0
    one = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert one["fits"] and 160 < one["needed_gib"] < 180 and one["gib_per_gpu"]["expert_weights"] > 140
    assert cli.main(["plan-memory", "--gpus", "1", "--device-gib", "80"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["fits"] is False
    assert cli.main(["plan-memory", "--gpus", "8", "--max-context", "1006144"]) == 0
    eight = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert eight["fits"] and eight["needed_gib"] < 70
