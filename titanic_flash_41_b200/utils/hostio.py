"""Python face of the C++ host runtime (``csrc/host_runtime.cc``) with pure-Python fallbacks, so
callers never branch on whether the library was built."""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
import zlib
from typing import List, Optional, Tuple

from ..ops import native

FRAME_MAGIC = 0x31465454


def _buf(data) -> Tuple[ctypes.c_void_p, int, object]:
    mv = memoryview(data).cast("B")
    if mv.readonly:
        keep = ctypes.create_string_buffer(bytes(mv), len(mv))
        return ctypes.cast(keep, ctypes.c_void_p), len(mv), keep
    keep = (ctypes.c_char * len(mv)).from_buffer(mv)
    return ctypes.cast(keep, ctypes.c_void_p), len(mv), keep


def sha256_chunks(data, chunk: int, threads: int = 8) -> List[bytes]:
    """One SHA-256 per ``chunk`` bytes, in order."""
    h = native.host_lib()
    n = len(memoryview(data).cast("B"))
    count = -(-n // chunk) if n else 0
    if h is None or count == 0:
        mv = memoryview(data).cast("B")
        return [hashlib.sha256(mv[i:i + chunk]).digest() for i in range(0, n, chunk)]
    ptr, n, keep = _buf(data)
    out = ctypes.create_string_buffer(32 * count)
    if h.tf_host_sha256_chunks(ptr, n, chunk, ctypes.cast(out, ctypes.c_void_p), threads) != 0:
        raise RuntimeError("tf_host_sha256_chunks failed")
    return [out.raw[32 * i:32 * i + 32] for i in range(count)]


def write_file(path: str, data, direct: bool = True) -> int:
    """Durable write (fsync) that bypasses the page cache where the filesystem allows."""
    h = native.host_lib()
    if h is None:
        with open(path, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        return len(memoryview(data).cast("B"))
    ptr, n, keep = _buf(data)
    r = h.tf_host_write_direct(path.encode(), ptr, n, 1 if direct else 0)
    if r < 0:
        raise OSError(-r, os.strerror(-r), path)
    return int(r)


def read_file(path: str, n: int, offset: int = 0, direct: bool = True) -> bytearray:
    h = native.host_lib()
    out = bytearray(n)
    if h is None:
        with open(path, "rb") as f:
            f.seek(offset)
            got = f.readinto(out)
        if got != n:
            raise OSError(5, "short read", path)
        return out
    keep = (ctypes.c_char * n).from_buffer(out)
    r = h.tf_host_read_direct(path.encode(), ctypes.cast(keep, ctypes.c_void_p), n, offset, 1 if direct else 0)
    if r < 0:
        raise OSError(-r, os.strerror(-r), path)
    if r != n:
        raise OSError(5, "short read", path)
    return out


def frame_encode(kind: int, seq: int, payload: bytes) -> bytes:
    h = native.host_lib()
    if h is None:
        head = struct.pack("<IIQI", FRAME_MAGIC, kind, seq, len(payload)) + payload
        return head + struct.pack("<I", zlib.crc32(head) & 0xFFFFFFFF)
    out = ctypes.create_string_buffer(24 + len(payload))
    src = ctypes.create_string_buffer(payload, len(payload)) if payload else None
    n = h.tf_host_frame_encode(kind, seq, ctypes.cast(src, ctypes.c_void_p) if src else None, len(payload),
                               ctypes.cast(out, ctypes.c_void_p))
    return out.raw[:n]


def frame_decode(frame: bytes) -> Tuple[int, int, bytes]:
    """(kind, seq, payload); ValueError on bad magic, truncation or checksum."""
    h = native.host_lib()
    if h is None:
        if len(frame) < 24:
            raise ValueError("truncated frame")
        magic, kind, seq, n = struct.unpack("<IIQI", frame[:20])
        if magic != FRAME_MAGIC:
            raise ValueError("bad frame magic")
        if 24 + n > len(frame):
            raise ValueError("truncated frame")
        if struct.unpack("<I", frame[20 + n:24 + n])[0] != zlib.crc32(frame[:20 + n]) & 0xFFFFFFFF:
            raise ValueError("frame checksum")
        return kind, seq, frame[20:20 + n]
    kind, seq = ctypes.c_int(0), ctypes.c_long(0)
    cap = max(1, len(frame))
    out = ctypes.create_string_buffer(cap)
    src = ctypes.create_string_buffer(frame, len(frame))
    n = h.tf_host_frame_decode(ctypes.cast(src, ctypes.c_void_p), len(frame), ctypes.cast(ctypes.byref(kind), ctypes.c_void_p),
                               ctypes.cast(ctypes.byref(seq), ctypes.c_void_p), ctypes.cast(out, ctypes.c_void_p), cap)
    if n < 0:
        raise ValueError({-1: "bad frame magic", -2: "truncated frame", -3: "frame checksum"}[int(n)])
    return kind.value, seq.value, out.raw[:n]
