"""C++ host runtime against hashlib / zlib / plain file I/O (and its pure-Python fallbacks)."""
import hashlib
import os

import pytest

from titanic_flash_41_b200.ops import native
from titanic_flash_41_b200.utils import hostio


@pytest.fixture(params=["native", "fallback"])
def mode(request, monkeypatch):
    if request.param == "fallback":
        monkeypatch.setattr(native, "host_lib", lambda: None)
    elif native.host_lib() is None:
        pytest.skip("host library not built")
    return request.param


def test_chunk_digests(mode):
    data = os.urandom(3 * 65536 + 1234)
    got = hostio.sha256_chunks(data, 65536, threads=4)
    want = [hashlib.sha256(data[i:i + 65536]).digest() for i in range(0, len(data), 65536)]
    assert got == want and len(got) == 4
    assert hostio.sha256_chunks(b"", 4096) == []
    assert hostio.sha256_chunks(bytearray(b"abc"), 4096) == [hashlib.sha256(b"abc").digest()]


def test_direct_file_round_trip(mode, tmp_path):
    p = os.path.join(str(tmp_path), "x.bin")
    for n in (0, 1, 4096, 4097, (9 << 20) + 77):
        data = os.urandom(n)
        assert hostio.write_file(p, data) == n
        assert os.path.getsize(p) == n
        assert bytes(hostio.read_file(p, n)) == data
        if n > 5000:
            assert bytes(hostio.read_file(p, 1000, offset=4096)) == data[4096:5096]
            assert bytes(hostio.read_file(p, 10, offset=3)) == data[3:13]
    with pytest.raises(OSError):
        hostio.read_file(p, n + 10)
    with pytest.raises(OSError):
        hostio.read_file(os.path.join(str(tmp_path), "missing"), 1)


def test_frames(mode):
    f = hostio.frame_encode(3, 1 << 40, b"hello")
    assert hostio.frame_decode(f) == (3, 1 << 40, b"hello")
    assert hostio.frame_decode(hostio.frame_encode(0, 0, b"")) == (0, 0, b"")
    bad = bytearray(f)
    bad[21] ^= 1
    with pytest.raises(ValueError, match="checksum"):
        hostio.frame_decode(bytes(bad))
    with pytest.raises(ValueError, match="truncated"):
        hostio.frame_decode(f[:-3])
    with pytest.raises(ValueError, match="magic"):
        hostio.frame_decode(b"\\0" * 24)


def test_native_and_fallback_frames_are_identical():
    if native.host_lib() is None:
        pytest.skip("host library not built")
    a = hostio.frame_encode(7, 99, b"payload")
    import struct, zlib
    head = struct.pack("<IIQI", hostio.FRAME_MAGIC, 7, 99, 7) + b"payload"
    assert a == head + struct.pack("<I", zlib.crc32(head) & 0xFFFFFFFF)
