import os

import pytest
import torch

from titanic_flash_41_b200.serve import state_image as SI


def _img():
    a = torch.arange(5_000_000, dtype=torch.int32)
    b = torch.randn(333)
    return a, b, SI.capture([1, 2, 3], [("win", a), ("carry", b)], meta={"length": 3})


def test_capture_restore_and_digest():
    a, b, img = _img()
    d0 = img.digest()
    a2, b2 = torch.zeros_like(a), torch.zeros_like(b)
    SI.restore_into(img, {"win": a2, "carry": b2})
    assert torch.equal(a, a2) and torch.equal(b, b2)
    img.to_host(pin=False)
    assert img.tier == "host" and img.digest() == d0
    with pytest.raises(SI.ImageError):
        SI.restore_into(img, {"win": a2})


def test_disk_tier_round_trip_and_corruption(tmp_path):
    a, b, img = _img()
    d0, n = img.digest(), img.nbytes
    tier = SI.DiskTier(str(tmp_path))
    assert tier.write("c1", img) == n and img.tier == "disk" and img.nbytes == n
    back = tier.read("c1", img)
    assert back.tier == "host" and back.digest() == d0 and back.tokens == (1, 2, 3)
    # corrupt one byte in the second chunk: the digest check names the chunk
    tier.write("c2", back)
    path = os.path.join(str(tmp_path), "c2.img")
    raw = bytearray(open(path, "rb").read())
    raw[-(6 << 20)] ^= 0xFF
    open(path, "wb").write(bytes(raw))
    with pytest.raises(SI.ImageError, match="fails its digest"):
        tier.read("c2")
    open(path, "wb").write(bytes(raw[:-100]))
    with pytest.raises(SI.ImageError, match="truncated"):
        tier.read("c2")


def test_fault_hook_fires_at_named_points(tmp_path):
    seen = []

    def hook(point):
        seen.append(point)
        if point == "write_chunk" and seen.count("write_chunk") == 2:
            raise OSError("injected")
    _, _, img = _img()
    tier = SI.DiskTier(str(tmp_path), hook)
    with pytest.raises(OSError):
        tier.write("x", img)
    assert img.tier == "device" and not os.path.exists(os.path.join(str(tmp_path), "x.img"))
