"""Header-only safetensors scanner/writer and the checkpoint tensor contract.

``scan`` reads just the JSON header of every shard, validates that the data region has no
overlaps or holes, refuses path traversal in shard names, and answers ``require(name, dtype,
shape)`` / ``read_slice``.  Dtypes follow the reference's packing: F32, BF16, F8_E4M3, F8_E8M0
(UE8M0 scale bytes) and I8 = packed FP4 nibbles (reference: src/checkpoint.rs:15-26 Dtype,
:110-177 scan, :178 validate, :217 read_slice, :244 require, :91 traversal guard).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

DTYPES = {"F32": (4, torch.float32), "BF16": (2, torch.bfloat16), "F16": (2, torch.float16),
          "F8_E4M3": (1, torch.float8_e4m3fn), "F8_E8M0": (1, torch.uint8), "I8": (1, torch.uint8),
          "U8": (1, torch.uint8), "I32": (4, torch.int32), "I64": (8, torch.int64)}
_REV = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.float8_e4m3fn: "F8_E4M3",
        torch.uint8: "U8", torch.int32: "I32", torch.int64: "I64"}


class CheckpointError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    file: str
    begin: int          # absolute byte offsets in the file
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


def _read_header(path: str) -> Tuple[Dict, int]:
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise CheckpointError(f"{path}: truncated header")
        (n,) = struct.unpack("<Q", raw)
        if n > (100 << 20):
            raise CheckpointError(f"{path}: implausible header length {n}")
        head = f.read(n)
        if len(head) != n:
            raise CheckpointError(f"{path}: truncated header")
    return json.loads(head), 8 + n


class Checkpoint:
    def __init__(self, root: str, tensors: Dict[str, TensorInfo]):
        self.root, self.tensors = root, tensors

    @staticmethod
    def scan(root: str) -> "Checkpoint":
        index = os.path.join(root, "model.safetensors.index.json")
        if os.path.exists(index):
            files = sorted(set(json.load(open(index))["weight_map"].values()))
        else:
            files = sorted(f for f in os.listdir(root) if f.endswith(".safetensors"))
        if not files:
            raise CheckpointError(f"{root}: no safetensors shards")
        tensors: Dict[str, TensorInfo] = {}
        for fn in files:
            if os.path.isabs(fn) or ".." in fn.replace("\\", "/").split("/"):
                raise CheckpointError(f"shard name escapes the checkpoint directory: {fn}")
            path = os.path.join(root, fn)
            header, base = _read_header(path)
            size = os.path.getsize(path)
            spans: List[Tuple[int, int, str]] = []
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                dt, shape = meta["dtype"], tuple(int(x) for x in meta["shape"])
                if dt not in DTYPES:
                    raise CheckpointError(f"{name}: unsupported dtype {dt}")
                b, e = meta["data_offsets"]
                want = DTYPES[dt][0] * int(np.prod(shape, dtype=np.int64)) if shape else DTYPES[dt][0]
                if e - b != want:
                    raise CheckpointError(f"{name}: {e - b} bytes for shape {shape} of {dt}")
                if name in tensors:
                    raise CheckpointError(f"{name}: defined twice")
                tensors[name] = TensorInfo(name, dt, shape, path, base + b, base + e)
                spans.append((b, e, name))
            spans.sort()
            pos = 0
            for b, e, name in spans:
                if b != pos:
                    raise CheckpointError(f"{fn}: {'overlap' if b < pos else 'hole'} before {name}")
                pos = e
            if base + pos != size:
                raise CheckpointError(f"{fn}: data region is {size - base} bytes, tensors cover {pos}")
        return Checkpoint(root, tensors)

    def require(self, name: str, dtype: str, shape: Sequence[int]) -> TensorInfo:
        t = self.tensors.get(name)
        if t is None:
            raise CheckpointError(f"missing tensor {name}")
        if t.dtype != dtype or tuple(t.shape) != tuple(shape):
            raise CheckpointError(f"{name}: have {t.dtype}{list(t.shape)}, need {dtype}{list(shape)}")
        return t

    def read(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        return self.read_slice(name, 0, t.shape[0] if t.shape else 1)

    def read_slice(self, name: str, row0: int, rows: int, axis: int = 0) -> torch.Tensor:
        """Rows [row0, row0+rows) along ``axis`` (axis 0 is one contiguous read)."""
        t = self.tensors[name]
        esize, tdt = DTYPES[t.dtype]
        if not t.shape:
            shape = ()
        else:
            shape = t.shape
        if axis == 0 or not shape:
            inner = int(np.prod(shape[1:], dtype=np.int64)) if len(shape) > 1 else 1
            if row0 < 0 or (shape and row0 + rows > shape[0]):
                raise CheckpointError(f"{name}: slice outside the tensor")
            with open(t.file, "rb") as f:
                f.seek(t.begin + row0 * inner * esize)
                raw = f.read(rows * inner * esize)
            out = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(tdt)
            return out.reshape((rows,) + tuple(shape[1:])) if shape else out.reshape(())
        full = self.read(name)
        return full.narrow(axis, row0, rows).contiguous()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], dtype_names: Optional[Dict[str, str]] = None
                      ) -> None:
    """Write one shard.  ``dtype_names`` overrides the header dtype of uint8 tensors that hold
    packed formats (``F8_E8M0`` scales, ``I8`` packed FP4)."""
    header, off, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.contiguous()
        dn = (dtype_names or {}).get(name) or _REV[t.dtype]
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.dtype != torch.uint8 else t.reshape(-1).numpy().tobytes()
        header[name] = {"dtype": dn, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b)
