"""Lossless snapshots of a conversation's device state, and the tiers they live in.

An image is an ordered list of named byte regions (window rings, compressed streams, index
keys, compressor carries, draft state, logits) cut at the conversation's frontier, plus the
token prefix it stands for.  Tiers: device (as captured), pinned host memory, and a directory
of chunked files with a SHA-256 per 4 MiB chunk that is verified on reload.  Reference:
src/state_image.rs:218-525 (Image, try_allocate, save, drop_device, reload, digest),
src/disk_tier.rs:20-221 (CHUNK 4 MiB, batches of 32 chunks, digest check on read).
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..utils import hostio

CHUNK = 4 << 20
BATCH_CHUNKS = 32


class ImageError(RuntimeError):
    pass


@dataclass(eq=False)          # identity: two images of the same prefix are still two images
class Image:
    tokens: Tuple[int, ...]                    # the prefix this image restores (tuple of ints, or a read-only int64 array)
    regions: List[Tuple[str, torch.Tensor]]    # (name, flat uint8 tensor)
    kind: str = "complete"                     # complete | checkpoint | encoder | request | optional
    media: str = ""                            # identity of images inside the prefix
    meta: Dict[str, int] = field(default_factory=dict)
    tier: str = "device"                       # device | host | disk
    path: Optional[str] = None
    _bytes: int = 0

    @property
    def length(self) -> int:
        return len(self.tokens)

    @property
    def nbytes(self) -> int:
        if self.regions:
            self._bytes = sum(int(t.numel()) for _, t in self.regions)
        return self._bytes

    def digest(self) -> str:
        h = hashlib.sha256()
        for name, t in self.regions:
            h.update(name.encode())
            h.update(struct.pack("<Q", t.numel()))
            h.update(t.detach().cpu().contiguous().numpy().tobytes())
        return h.hexdigest()

    # ---- tier moves ---------------------------------------------------------------------------
    def to_host(self, pin: bool = True) -> None:
        if self.tier != "device":
            return
        moved = []
        for name, t in self.regions:
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=pin and torch.cuda.is_available())
            h.copy_(t)
            moved.append((name, h))
        self.regions, self.tier = moved, "host"
        self.release_pool()

    def release_pool(self) -> None:
        """Give a pooled image's chunks back (after its device copies are no longer needed)."""
        rng = getattr(self, "_range", None)
        if rng is not None:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            rng.free()
            self._range = None

    def to_device(self, device) -> None:
        if self.tier == "disk":
            raise ImageError("reload from the disk tier first")
        self.regions = [(n, t.to(device, non_blocking=True)) for n, t in self.regions]
        self.tier = "device"


def _token_tuple(tokens):
    """The prefix an image restores, immutable: a tuple of plain ints, or, when the caller hands an
    integer array (the worker does: a million-token prefix must not become a million Python ints
    for every image), a read-only int64 copy of it."""
    import numpy as np
    if isinstance(tokens, tuple):
        return tokens
    if isinstance(tokens, np.ndarray):
        arr = np.array(tokens, dtype=np.int64)
        arr.flags.writeable = False
        return arr
    return tuple(np.asarray(tokens, dtype=np.int64).tolist())


def capture(tokens: Sequence[int], named: Sequence[Tuple[str, torch.Tensor]], kind: str = "complete",
            media: str = "", meta: Optional[Dict[str, int]] = None, pool=None) -> Image:
    """Copy the given tensor views (any dtype/shape) into a new image on their own device.

    With ``pool`` (a ``utils.vmm.ChunkPool``) the image's regions are carved from ONE pooled range
    (256-byte aligned slices), so saving and dropping images never touches the device heap; the
    range goes back to the pool when the image leaves the device tier.  ``PoolExhausted``
    propagates: the caller treats it like any other refused optional allocation."""
    if pool is None:
        regs = [(n, t.contiguous().view(torch.uint8).reshape(-1).clone()) for n, t in named]
        return Image(_token_tuple(tokens), regs, kind, media, dict(meta or {}))
    flats = [(n, t.contiguous().view(torch.uint8).reshape(-1)) for n, t in named]
    offs, total = [], 0
    for _, f in flats:
        offs.append(total)
        total += -(-int(f.numel()) // 256) * 256
    rng = pool.alloc(max(total, 1))
    whole = rng.tensor()
    regs = []
    for (n, f), o in zip(flats, offs):
        dst = whole[o:o + f.numel()]
        dst.copy_(f)
        regs.append((n, dst))
    img = Image(_token_tuple(tokens), regs, kind, media, dict(meta or {}))
    img._range = rng
    return img


def restore_into(img: Image, targets: Dict[str, torch.Tensor]) -> None:
    """Copy every region back into the view of the same name (sizes must match exactly)."""
    if img.tier == "disk":
        raise ImageError("image is parked on disk")
    for name, src in img.regions:
        dst = targets.get(name)
        if dst is None:
            raise ImageError(f"no target for region {name}")
        flat = dst.view(torch.uint8).reshape(-1) if dst.is_contiguous() else None
        if flat is None or flat.numel() != src.numel():
            # non-contiguous view: go through a contiguous staging copy
            tmp = src.to(dst.device).view(dst.dtype).reshape(dst.shape)
            dst.copy_(tmp)
        else:
            flat.copy_(src, non_blocking=True)


# ---------------------------------------------------------------------------------------------
# disk tier
# ---------------------------------------------------------------------------------------------
class DiskTier:
    """Write-behind snapshot files.  Layout of ``<id>.img``: JSON header line, then the regions'
    bytes back to back; ``<id>.idx`` holds one SHA-256 per 4 MiB chunk of the payload.  A hook can
    inject faults at named points (reference feature ``storage-fault-injection``; never enabled in
    serving)."""

    def __init__(self, directory: str, fault_hook: Optional[Callable[[str], None]] = None):
        self.dir = directory
        self.fault = fault_hook or (lambda point: None)
        os.makedirs(directory, exist_ok=True)

    def reset_dir(self) -> None:
        for f in os.listdir(self.dir):
            if f.endswith((".img", ".idx")):
                os.remove(os.path.join(self.dir, f))

    def write(self, image_id: str, img: Image) -> int:
        if img.tier == "disk":
            return img.nbytes
        path = os.path.join(self.dir, image_id + ".img")
        header = {"tokens": [int(t) for t in img.tokens] if isinstance(img.tokens, tuple) else img.tokens.tolist(), "kind": img.kind, "media": img.media, "meta": img.meta,
                  "regions": [[n, int(t.numel())] for n, t in img.regions]}
        self.fault("write_open")
        hb = json.dumps(header).encode() + b"\n"
        blob = bytearray(struct.pack("<Q", len(hb)) + hb)
        head_len = len(blob)
        for _, t in img.regions:
            blob += t.detach().cpu().contiguous().numpy().tobytes()
        total = len(blob) - head_len
        # digests of every 4 MiB chunk by the host runtime's thread pool, then one durable write
        # that bypasses the page cache
        digests = [d.hex() for d in hostio.sha256_chunks(memoryview(blob)[head_len:], CHUNK)]
        for _ in digests:
            self.fault("write_chunk")
        hostio.write_file(path + ".tmp", blob)
        with open(os.path.join(self.dir, image_id + ".idx"), "w") as f:
            json.dump({"chunk": CHUNK, "digests": digests, "bytes": total}, f)
        os.replace(path + ".tmp", path)
        img._bytes = total
        img.regions, img.tier, img.path = [], "disk", path
        return total

    def read(self, image_id: str, img: Optional[Image] = None, pin: bool = False) -> Image:
        path = os.path.join(self.dir, image_id + ".img")
        with open(os.path.join(self.dir, image_id + ".idx")) as f:
            idx = json.load(f)
        self.fault("read_open")
        size = os.path.getsize(path)
        raw = hostio.read_file(path, size)
        (hl,) = struct.unpack("<Q", raw[:8])
        header = json.loads(bytes(raw[8:8 + hl]))
        payload = memoryview(raw)[8 + hl:]
        if len(payload) != idx["bytes"]:
            raise ImageError(f"{image_id}: truncated image ({len(payload)} of {idx['bytes']} bytes)")
        for i, (got, want) in enumerate(zip(hostio.sha256_chunks(payload, idx["chunk"]), idx["digests"])):
            if got.hex() != want:
                raise ImageError(f"{image_id}: chunk {i} fails its digest")
        regs, off = [], 0
        for name, n in header["regions"]:
            t = torch.frombuffer(bytearray(payload[off:off + n]), dtype=torch.uint8) if n else torch.empty(0, dtype=torch.uint8)
            regs.append((name, t.pin_memory() if (pin and torch.cuda.is_available()) else t))
            off += n
        out = img or Image(tuple(header["tokens"]), [], header["kind"], header["media"], header["meta"])
        out.regions, out.tier, out.path = regs, "host", path
        return out

    def remove(self, image_id: str) -> None:
        for ext in (".img", ".idx"):
            p = os.path.join(self.dir, image_id + ext)
            if os.path.exists(p):
                os.remove(p)
