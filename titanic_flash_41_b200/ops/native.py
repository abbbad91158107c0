"""ctypes binding of the in-tree CUDA library (``lib/libtflash_cuda.so``).

The kernels export a C ABI that takes raw device pointers and a ``cudaStream_t``; this module
turns ``torch.Tensor`` arguments into pointers, passes the current stream, and raises on a
non-zero return code.  On a machine with a GPU the library MUST load: a missing or stale
``.so`` is an error, never a silent fall back to PyTorch ops.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path
from typing import Optional

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lib: Optional[ctypes.CDLL] = None
_host: Optional[ctypes.CDLL] = None

# signature letters: p pointer, i int32, l int64, f float, d double, s stream
_CSRC = Path(__file__).resolve().parent.parent / "csrc"
_DECL = re.compile(r"TF_API\s+(\w+)\s+(\w+)\s*\(([^)]*)\)", re.S)


def _parse_signatures(pattern: str = "*.cu"):
    """Read the exported declarations out of csrc/*.cu (device library) or csrc/*.cc (host
    library) so the argument types used by ctypes can never drift from the C side."""
    sigs, rets = {}, {}
    for src in sorted(_CSRC.glob(pattern)):
        for ret, name, args in _DECL.findall(src.read_text()):
            sig = ""
            for a in [x.strip() for x in args.split(",") if x.strip()]:
                if a == "void":
                    continue
                if "char*" in a.replace(" *", "*") and "const" in a:
                    sig += "c"
                elif "*" in a:
                    sig += "p"
                elif a.startswith("cudaStream_t"):
                    sig += "s"
                elif a.startswith(("long", "int64_t", "size_t", "unsigned long")):
                    sig += "l"
                elif a.startswith("float"):
                    sig += "f"
                elif a.startswith("double"):
                    sig += "d"
                else:
                    sig += "i"
            sigs[name], rets[name] = sig, ret
    return sigs, rets


_SIGS, _RETS = _parse_signatures("*.cu")
_HSIGS, _HRETS = _parse_signatures("*.cc")
_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_long, "f": ctypes.c_float,
       "d": ctypes.c_double, "s": ctypes.c_void_p, "c": ctypes.c_char_p}


class NativeError(RuntimeError):
    pass


def available() -> bool:
    return (_LIB_DIR / "libtflash_cuda.so").exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _LIB_DIR / "libtflash_cuda.so"
        if not path.exists():
            raise NativeError(f"{path} is missing: run `python -m titanic_flash_41_b200.utils.build` "
                              "(or __graft_entry__.build())")
        _lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        for name, sig in _SIGS.items():
            fn = getattr(_lib, name, None)
            if fn is None:
                raise NativeError(f"{path} does not export {name}: rebuild the library")
            fn.argtypes = [_CT[c] for c in sig]
            fn.restype = ctypes.c_long if _RETS[name] == "long" else ctypes.c_int
    return _lib


def host_lib() -> Optional[ctypes.CDLL]:
    """The C++ host runtime (digests, direct I/O, frame codec); None when it has not been built."""
    global _host
    if _host is None:
        path = _LIB_DIR / "libtflash_host.so"
        if path.exists():
            _host = ctypes.CDLL(str(path))
            for name, sig in _HSIGS.items():
                fn = getattr(_host, name, None)
                if fn is None:
                    raise NativeError(f"{path} does not export {name}: rebuild the library")
                fn.argtypes = [_CT[c] for c in sig]
                fn.restype = ctypes.c_long if _HRETS[name] == "long" else ctypes.c_int
    return _host


def _conv(a, kind: str):
    if kind in "ps":
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            return a.data_ptr()
        return int(a)
    if kind in "il":
        return int(a)
    return float(a)


# kernels launched per exported call (for launch accounting); default 1
_KERNELS_PER_CALL = {"tf_sparse_attention": 2, "tf_router": 2, "tf_spec_verify": 2, "tf_rowstats": 7, "tf_rowstats_per_session": 7,
                     "tf_moe_plan": 3}
LAUNCHES = [0]


def call(name: str, *args, stream: Optional[int] = None) -> None:
    """Invoke an exported kernel launcher; a trailing stream argument is filled in here."""
    l = lib()
    sig = _SIGS[name]
    takes_stream = sig.endswith("s")
    want = len(sig) - (1 if takes_stream else 0)
    if len(args) != want:
        raise NativeError(f"{name}: expected {want} arguments, got {len(args)}")
    cargs = [_conv(a, k) for a, k in zip(args, sig)]
    if takes_stream:
        cargs.append(torch.cuda.current_stream().cuda_stream if stream is None else stream)
    rc = getattr(l, name)(*cargs)
    LAUNCHES[0] += _KERNELS_PER_CALL.get(name, 1)
    if rc != 0:
        raise NativeError(f"{name} failed with code {rc}" + (" (bad argument)" if rc == -1 else " (CUDA error)"))


def set_pdl(on: bool) -> bool:
    """Launch every kernel of the library with the programmatic-dependent-launch attribute (the next
    kernel of a stream is made resident while the current one runs; each kernel still waits for its
    predecessor's completion before it touches memory).  Applies to launches made from now on,
    including those captured into CUDA graphs.  Returns the previous setting."""
    return bool(lib().tf_set_pdl(1 if on else 0))


def pdl_enabled() -> bool:
    return bool(lib().tf_get_pdl())


STATUS_CODES = {0: "ok", 1: "bad_arg", 2: "timeout", 3: "bad_index", 4: "nonfinite"}


class StatusWord:
    """Device status word shared by the kernels of one engine: {code, kernel, detail0, detail1}.
    ``check()`` reads it back (a synchronising copy) and raises if a kernel reported a problem."""

    def __init__(self, device):
        self.t = torch.zeros(4, dtype=torch.int32, device=device)

    def ptr(self):
        return self.t

    def read(self):
        return [int(v) for v in self.t.tolist()]

    def check(self, reset: bool = True) -> None:
        code, kern, d0, d1 = self.read()
        if code != 0:
            if reset:
                self.t.zero_()
            raise NativeError(f"kernel {kern} reported {STATUS_CODES.get(code, code)} "
                              f"(detail {d0}, {d1})")
