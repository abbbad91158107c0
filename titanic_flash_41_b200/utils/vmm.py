"""Python face of the device chunk pool (``csrc/vmm_pool.cu``): pooled allocations for state
images and elastic ranges whose mapped size follows the occupancy of a serving region."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from ..ops import native


class PoolExhausted(MemoryError):
    pass


class _Raw:
    """Zero-copy view of device memory for ``torch.as_tensor``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _err(code: int, what: str):
    if code == -2:
        raise PoolExhausted(f"{what}: the chunk pool has no free chunks left")
    if code != 0:
        raise RuntimeError(f"{what}: chunk pool error {code}")


class Range:
    """A virtual range whose first ``mapped`` bytes are backed by pool chunks."""

    def __init__(self, pool: "ChunkPool", base: int, reserved: int, mapped: int):
        self.pool, self.base, self.reserved, self.mapped = pool, base, reserved, mapped

    def tensor(self, nbytes: Optional[int] = None, dtype=torch.uint8) -> torch.Tensor:
        n = self.mapped if nbytes is None else nbytes
        if n > self.mapped:
            raise ValueError("view beyond the mapped part of the range")
        t = torch.as_tensor(_Raw(self.base, n), device=torch.device("cuda", self.pool.device))
        return t.view(dtype)

    def resize(self, mapped: int) -> None:
        """Map or unmap chunks at the tail; what stays mapped keeps its contents and address."""
        _err(native.lib().tf_vmm_resize(self.pool.handle, self.base, mapped), "resize")
        self.mapped = -(-mapped // self.pool.chunk) * self.pool.chunk if mapped else 0

    def free(self) -> None:
        if self.base:
            _err(native.lib().tf_vmm_free(self.pool.handle, self.base), "free")
            self.base = 0


class ChunkPool:
    def __init__(self, n_chunks: int, chunk_bytes: int = 16 << 20, device: int = 0):
        L = native.lib()
        out = ctypes.c_long(0)
        self.handle = L.tf_vmm_pool_create(device, chunk_bytes, n_chunks, ctypes.cast(ctypes.byref(out), ctypes.c_void_p))
        if not self.handle:
            raise RuntimeError("could not create the device chunk pool")
        self.chunk, self.device = int(out.value), device

    def counts(self) -> Tuple[int, int]:
        """(total chunks, free chunks)"""
        a, b = ctypes.c_int(0), ctypes.c_int(0)
        native.lib().tf_vmm_pool_chunks(self.handle, ctypes.cast(ctypes.byref(a), ctypes.c_void_p),
                                        ctypes.cast(ctypes.byref(b), ctypes.c_void_p))
        return a.value, b.value

    def reserve(self, max_bytes: int, mapped_bytes: int = 0) -> Range:
        err = ctypes.c_int(0)
        base = native.lib().tf_vmm_reserve(self.handle, max_bytes, mapped_bytes, ctypes.cast(ctypes.byref(err), ctypes.c_void_p))
        _err(err.value, "reserve")
        reserved = -(-max_bytes // self.chunk) * self.chunk
        return Range(self, int(base), reserved, -(-mapped_bytes // self.chunk) * self.chunk)

    def alloc(self, nbytes: int) -> Range:
        return self.reserve(nbytes, nbytes)

    def destroy(self) -> None:
        if self.handle:
            torch.cuda.synchronize(self.device)
            native.lib().tf_vmm_pool_destroy(self.handle)
            self.handle = 0
