"""Build the native libraries in-tree with nvcc / g++ (no JIT cache, no torch headers).

``libtflash_cuda.so``  every ``csrc/*.cu`` compiled for sm_100a and linked into one shared
                       object with a C ABI (loaded through ctypes by ``ops/native.py``)
``libtflash_host.so``  every ``csrc/*.cc``: host-side runtime pieces (digests, O_DIRECT tier
                       I/O, control-frame codec)

Objects are rebuilt only when their source (or a header) is newer.  The reference's equivalent
is tools/build.sh (nvcc --cubin -arch=sm_121 + cargo); here the arch is compute_100a/sm_100a.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
OUT = PKG / "lib"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
# exact transcendental and division semantics are wanted in the sampling / norm kernels
NO_FAST_MATH = {"sampling.cu", "sample_chunks.cu", "elementwise.cu", "indexer.cu", "fused_norm.cu"}


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _stale(target: Path, deps: List[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: List[str]) -> str:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build(verbose: bool = False, ptxas_info: bool = False) -> None:
    OUT.mkdir(exist_ok=True)
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    cus = sorted(CSRC.glob("*.cu"))
    ccs = sorted(CSRC.glob("*.cc"))
    nvcc = _nvcc()
    jobs = []
    for src in cus:
        obj = objdir / (src.stem + ".o")
        if _stale(obj, [src] + headers):
            flags = [f for f in NVCC_FLAGS if not (f == "--use_fast_math" and src.name in NO_FAST_MATH)]
            if ptxas_info:
                flags += ["-Xptxas", "-v"]
            jobs.append([nvcc, *flags, "-c", str(src), "-o", str(obj)])
    for src in ccs:
        obj = objdir / (src.stem + ".host.o")
        if _stale(obj, [src] + headers):
            jobs.append(["g++", "-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-c",
                         str(src), "-o", str(obj)])
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for out in ex.map(_run, jobs):
            if verbose or ptxas_info:
                sys.stderr.write(out)
    cuda_objs = [objdir / (s.stem + ".o") for s in cus]
    lib = OUT / "libtflash_cuda.so"
    if cus and _stale(lib, cuda_objs):
        _run([nvcc, "-shared", "-o", str(lib), *map(str, cuda_objs)])
    host_objs = [objdir / (s.stem + ".host.o") for s in ccs]
    hlib = OUT / "libtflash_host.so"
    if ccs and _stale(hlib, host_objs):
        _run(["g++", "-shared", "-pthread", "-o", str(hlib), *map(str, host_objs)])
    _write_provenance(nvcc)


def _sha256(path: Path) -> str:
    import hashlib
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _sources() -> List[Path]:
    return sorted(p for pat in ("*.cu", "*.cuh", "*.h", "*.cc") for p in CSRC.glob(pat))


def _write_provenance(nvcc: str) -> None:
    """``lib/build.json``: what the libraries were built from (reference: the build-provenance record
    of src/main.rs and tools/verify_runtime.py, which check bundles by SHA-256)."""
    import json
    ver = _run([nvcc, "--version"]).strip().splitlines()[-1]
    rec = {"nvcc": ver, "flags": NVCC_FLAGS, "no_fast_math": sorted(NO_FAST_MATH),
           "sources": {p.name: _sha256(p) for p in _sources()},
           "libraries": {p.name: _sha256(p) for p in sorted(OUT.glob("*.so"))}}
    (OUT / "build.json").write_text(json.dumps(rec, indent=1, sort_keys=True))


def provenance() -> dict:
    """Compare the tree with the record of the last build: sources changed, added or removed since then
    (the loaded library would be stale) and libraries that are not the ones the build wrote."""
    import json
    path = OUT / "build.json"
    if not path.exists():
        return {"recorded": False, "stale_sources": [], "libraries_match": False}
    rec = json.loads(path.read_text())
    now = {p.name: _sha256(p) for p in _sources()}
    stale = sorted(n for n in set(now) | set(rec["sources"]) if now.get(n) != rec["sources"].get(n))
    libs = {p.name: _sha256(p) for p in sorted(OUT.glob("*.so"))}
    return {"recorded": True, "nvcc": rec["nvcc"], "arch": "sm_100a", "stale_sources": stale,
            "libraries_match": libs == rec["libraries"] and bool(libs), "libraries": sorted(libs)}


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
    print("built", *(p.name for p in OUT.glob("*.so")))
