"""Memory admission against fake pools, and the stall-counter reader."""
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
