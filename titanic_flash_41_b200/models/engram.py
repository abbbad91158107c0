"""Engram: an n-gram hashed embedding memory read at a few layers.

Host side: ``HashMetadata`` (compressed-vocabulary map, multipliers, primes, offsets),
``HashHistory`` (transactional n-gram hashing that follows speculative acceptance:
``prepare`` hashes a batch against the committed history, ``commit(batch, accepted)`` advances it
by the accepted prefix only), the packed row format (4096-byte header + rows of 256 e4m3 values
and 8 UE8M0 scales) with a writer and a row store, and fp32 references of the device ops.
Device side: ``EngramTable`` keeps this rank's row interval in HBM and looks rows up with
``tf_engram_dequant``; ``gate`` mixes the projected memory into the residual copies
(reference: src/hash_history.rs:6-15 metadata, :87 prepare, :122-133 hash, :175 commit;
src/engram.rs:15 ROW_BYTES; tools/pack_engram.py; src/engram_gpu.rs; kernels/core.cu:952, :967).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..formats import codecs

ROW_BYTES = 264
HEADER_BYTES = 4096
MAGIC = b"TFENGRAM1\0"
CONTEXT_LIMIT = 1 << 20


@dataclass
class HashMetadata:
    token_map: np.ndarray            # [vocab] -> compressed vocabulary id
    multipliers: np.ndarray          # [tables, ngram] uint64
    primes: np.ndarray               # [tables, (ngram-1) * heads] uint64
    offsets: np.ndarray              # [tables, (ngram-1) * heads] uint64
    pad_token: int = 2
    image_token: int = -1
    heads: int = 8
    ngram: int = 4

    @property
    def tables(self) -> int:
        return int(self.multipliers.shape[0])

    @property
    def ids_per_table(self) -> int:
        return (self.ngram - 1) * self.heads

    @property
    def table_rows(self) -> int:
        return int(self.offsets[:, -1].max() + self.primes[:, -1].max())

    @staticmethod
    def synthetic(vocab: int, rows_per_head: int = 1000, tables: int = 2, heads: int = 8, ngram: int = 4,
                  seed: int = 0, image_token: int = -1) -> "HashMetadata":
        rng = np.random.default_rng(seed)
        n = (ngram - 1) * heads

        def primes_from(start, count):
            out, p = [], start
            while len(out) < count:
                p += 1
                if all(p % q for q in range(2, int(p ** 0.5) + 1)):
                    out.append(p)
            return out
        primes = np.array([primes_from(rows_per_head + 97 * t, n) for t in range(tables)], dtype=np.uint64)
        offsets = np.zeros_like(primes)
        for t in range(tables):
            offsets[t] = np.concatenate([[0], np.cumsum(primes[t][:-1])])
        return HashMetadata(token_map=rng.permutation(vocab).astype(np.uint64),
                            multipliers=rng.integers(1, 1 << 31, size=(tables, ngram), dtype=np.uint64) * 2 + 1,
                            primes=primes, offsets=offsets, image_token=image_token, heads=heads, ngram=ngram)


@dataclass
class HashBatch:
    parent: Tuple[int, int, int, Tuple[int, ...]]
    tokens: List[int]
    rows: np.ndarray                 # [len, tables, ids_per_table] uint64


class HashHistory:
    """Causal n-gram history of one conversation."""

    def __init__(self, lineage: int, pad_token: int = 2, ngram: int = 4):
        if lineage == 0:
            raise ValueError("history needs an owned sequence lineage")
        self.lineage, self.generation, self.position = lineage, 0, 0
        self.recent = [pad_token] * (ngram - 1)

    def _key(self):
        return (self.lineage, self.generation, self.position, tuple(self.recent))

    def prepare(self, tokens: Sequence[int], md: HashMetadata) -> HashBatch:
        n = len(tokens)
        if self.position + n > CONTEXT_LIMIT:
            raise ValueError("Engram context limit")
        if any(t < 0 or t >= len(md.token_map) for t in tokens):
            raise ValueError("token outside canonical vocabulary")
        pad = int(md.token_map[md.pad_token])
        rows = np.zeros((n, md.tables, md.ids_per_table), dtype=np.uint64)
        mask = (1 << 64) - 1
        for i in range(n):
            comp, blocked = [pad] * md.ngram, False
            for back in range(md.ngram):
                if self.position + i < back:
                    blocked = True
                tok = tokens[i - back] if back <= i else self.recent[back - i - 1]
                if tok == md.image_token:
                    blocked = True
                if not blocked:
                    comp[back] = int(md.token_map[tok])
            for t in range(md.tables):
                rolling = (comp[0] * int(md.multipliers[t][0])) & mask
                for back in range(1, md.ngram):
                    rolling ^= (comp[back] * int(md.multipliers[t][back])) & mask
                    for head in range(md.heads):
                        h = (back - 1) * md.heads + head
                        rows[i, t, h] = rolling % int(md.primes[t][h]) + int(md.offsets[t][h])
        return HashBatch(self._key(), list(tokens), rows)

    def prepare_padded(self, tokens: Sequence[int], live: int, md: HashMetadata) -> HashBatch:
        """Fixed-width launch: rows beyond ``live`` are padding and can never be committed."""
        if not (0 < live <= len(tokens)) or any(t != md.pad_token for t in tokens[live:]):
            raise ValueError("invalid Engram live/padding extent")
        in_range = min(len(tokens), max(0, CONTEXT_LIMIT - self.position))
        if live > in_range:
            raise ValueError("Engram context limit")
        b = self.prepare(tokens[:in_range], md)
        if in_range < len(tokens):
            b.rows = np.concatenate([b.rows, np.repeat(b.rows[-1:], len(tokens) - in_range, 0)])
        b.tokens = b.tokens[:live]
        return b

    def commit(self, batch: HashBatch, accepted: int) -> None:
        if batch.parent != self._key():
            raise ValueError("stale or foreign Engram history commit")
        if accepted > len(batch.tokens):
            raise ValueError("accepted prefix exceeds prepared batch")
        if accepted == 0:
            return
        for t in batch.tokens[:accepted]:
            self.recent = [t] + self.recent[:-1]
        self.position += accepted
        self.generation += 1


# ---------------------------------------------------------------------------------- row format
def pack_rows(values: torch.Tensor) -> torch.Tensor:
    """[rows, 256] fp32 -> [rows, 264] uint8 (MXFP8: e4m3 + one UE8M0 per 32)."""
    q, s = codecs.mxfp8_quant(values.float())
    return torch.cat([q.view(torch.uint8), s], dim=1).contiguous()


def unpack_rows(packed: torch.Tensor) -> torch.Tensor:
    q = packed[:, :256].contiguous().view(torch.float8_e4m3fn)
    return codecs.mxfp8_dequant(q, packed[:, 256:])


def write_table(path: str, packed: torch.Tensor, row_start: int = 0) -> None:
    head = MAGIC + struct.pack("<QQI", packed.shape[0], row_start, ROW_BYTES)
    with open(path, "wb") as f:
        f.write(head + b"\0" * (HEADER_BYTES - len(head)))
        f.write(packed.cpu().numpy().tobytes())


def read_table(path: str) -> Tuple[torch.Tensor, int]:
    with open(path, "rb") as f:
        head = f.read(HEADER_BYTES)
        if head[:len(MAGIC)] != MAGIC:
            raise ValueError(f"{path}: not an Engram table")
        rows, row_start, rb = struct.unpack("<QQI", head[len(MAGIC):len(MAGIC) + 20])
        if rb != ROW_BYTES:
            raise ValueError(f"{path}: row size {rb}")
        raw = np.frombuffer(f.read(rows * ROW_BYTES), dtype=np.uint8)
    if raw.size != rows * ROW_BYTES:
        raise ValueError(f"{path}: truncated table")
    return torch.from_numpy(raw.copy()).view(rows, ROW_BYTES), row_start


# ---------------------------------------------------------------------------------- references
def gate_reference(x: torch.Tensor, kv: torch.Tensor, qw: torch.Tensor, kw: torch.Tensor, eps: float) -> torch.Tensor:
    """x [r, m, d], kv [r, m+1, d], qw / kw [m, d] (fp32 math on bf16-valued inputs)."""
    r, m, d = x.shape
    keys, val = kv[:, :m], kv[:, m:]
    dot = ((x * (qw * kw)[None]) * keys).sum(-1)
    dot = dot * torch.rsqrt((x * x).mean(-1) + eps) * torch.rsqrt((keys * keys).mean(-1) + eps) / d ** 0.5
    g = torch.sigmoid(torch.sign(dot) * torch.sqrt(dot.abs().clamp_min(1e-6)))
    return x + g[..., None] * val


class EngramTable:
    """This rank's interval of one packed table, resident on the device."""

    def __init__(self, packed: torch.Tensor, row_start: int, device):
        self.row_start, self.row_end = row_start, row_start + packed.shape[0]
        self.data = packed.to(device).contiguous()
        self.device = device

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [n] int64 -> [n, 256] bf16; rows owned by other ranks come back zero."""
        from ..ops import native
        ids = ids.to(self.device, torch.int64).contiguous()
        out = torch.empty(ids.numel(), 256, dtype=torch.bfloat16, device=self.device)
        native.call("tf_engram_dequant", self.data, ids, out, ids.numel(), self.row_start, self.row_end)
        return out


class EngramRowStore:
    """The packed row store of one Engram table on disk with a set-associative cache in host memory.

    The full-size tables (hundreds of millions of 264-byte rows per layer) do not belong in HBM: the
    file written by ``write_table`` stays on NVMe, a lookup reads the rows it misses with one batched
    call into the host runtime (a pool of positional reads), and recently used rows stay in a
    ``ways``-way set-associative cache of pinned host memory, replaced least-recently-used within a
    set (reference: set-associative RAM cache + SSD reads, src/engram.rs, src/engram_io.rs:209-329).
    Rows outside [row_start, row_end) -- other ranks' intervals -- come back as zeros."""

    def __init__(self, path: str, cache_rows: int = 1 << 20, ways: int = 4, threads: int = 8):
        with open(path, "rb") as f:
            head = f.read(len(MAGIC) + 20)
        if head[:len(MAGIC)] != MAGIC:
            raise ValueError("not an Engram table file")
        rows, row_start, rb = struct.unpack("<QQI", head[len(MAGIC):])
        if rb != ROW_BYTES:
            raise ValueError("unexpected Engram row size")
        self.path, self.header = path, HEADER_BYTES
        self.rows, self.row_start, self.row_end = int(rows), int(row_start), int(row_start + rows)
        self.ways, self.threads = ways, threads
        self.sets = max(1, cache_rows // ways)
        self.tags = np.full((self.sets, ways), -1, dtype=np.int64)
        self.stamp = np.zeros((self.sets, ways), dtype=np.int64)
        self.data = np.zeros((self.sets, ways, ROW_BYTES), dtype=np.uint8)
        self.clock = 0
        self.stats = {"hits": 0, "misses": 0, "reads": 0, "foreign": 0}

    def _read(self, ids: np.ndarray) -> np.ndarray:
        """Rows ``ids`` (local row numbers) from the file."""
        from ..ops import native
        out = np.empty((len(ids), ROW_BYTES), dtype=np.uint8)
        if len(ids) == 0:
            return out
        h = native.host_lib()
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        if h is not None:
            r = h.tf_host_read_rows(self.path.encode(), self.header, ROW_BYTES, self.rows, ids.ctypes.data, len(ids),
                                    out.ctypes.data, self.threads)
            if r < 0:
                raise OSError(-r, "Engram row read failed", self.path)
        else:
            with open(self.path, "rb") as f:
                for i, r in enumerate(ids):
                    f.seek(self.header + int(r) * ROW_BYTES)
                    out[i] = np.frombuffer(f.read(ROW_BYTES), dtype=np.uint8)
        self.stats["reads"] += len(ids)
        return out

    def lookup(self, ids) -> np.ndarray:
        """Global row ids [n] -> packed rows [n, 264] (zeros for rows this store does not own)."""
        ids = np.asarray(ids, dtype=np.int64).reshape(-1)
        out = np.zeros((len(ids), ROW_BYTES), dtype=np.uint8)
        own = (ids >= self.row_start) & (ids < self.row_end)
        self.stats["foreign"] += int((~own).sum())
        loc = ids - self.row_start
        sets = loc % self.sets
        self.clock += 1
        miss_pos = []
        for i in np.flatnonzero(own):
            st = int(sets[i])
            w = np.flatnonzero(self.tags[st] == loc[i])
            if w.size:
                out[i] = self.data[st, w[0]]
                self.stamp[st, w[0]] = self.clock
                self.stats["hits"] += 1
            else:
                miss_pos.append(i)
        if miss_pos:
            mp = np.asarray(miss_pos)
            uniq, inv = np.unique(loc[mp], return_inverse=True)
            rows = self._read(uniq)
            self.stats["misses"] += len(mp)
            out[mp] = rows[inv]
            for k, r in enumerate(uniq):                # insert: evict the least recently used way of the set
                st = int(r % self.sets)
                w = int(np.argmin(self.stamp[st])) if (self.tags[st] >= 0).all() else int(np.flatnonzero(self.tags[st] < 0)[0])
                self.tags[st, w], self.stamp[st, w] = r, self.clock
                self.data[st, w] = rows[k]
        return out


class EngramHostTable:
    """An Engram table whose rows live in an ``EngramRowStore`` (disk + host cache): same ``lookup``
    as ``EngramTable``.  The ids must come to the host, so a step that uses it runs eagerly (the
    reference splits its graphs around these reads: engram_graphs, src/target.rs)."""

    def __init__(self, store: EngramRowStore, device):
        self.store, self.device = store, device
        self.row_start, self.row_end = store.row_start, store.row_end

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        from ..ops import native
        host_ids = ids.detach().to("cpu", torch.int64).numpy()
        packed = torch.from_numpy(self.store.lookup(host_ids)).to(self.device)
        n = packed.shape[0]
        out = torch.empty(n, 256, dtype=torch.bfloat16, device=self.device)
        # rows this store does not own are already zero rows: a zero scale byte decodes them to ~0
        own = torch.from_numpy(((host_ids >= self.row_start) & (host_ids < self.row_end))).to(self.device)
        seq = torch.arange(n, dtype=torch.int64, device=self.device)
        native.call("tf_engram_dequant", packed.contiguous(), torch.where(own, seq, torch.full_like(seq, -1)), out, n, 0, n)
        return out


def gate(x: torch.Tensor, kv: torch.Tensor, qw: torch.Tensor, kw: torch.Tensor, eps: float) -> torch.Tensor:
    from ..ops import native
    r, m, d = x.shape
    out = torch.empty_like(x)
    native.call("tf_engram_gate", x.contiguous(), kv.contiguous(), qw.contiguous(), kw.contiguous(), out, r, m, d, eps)
    return out


# ---------------------------------------------------------------------------------- model glue
_MD_CACHE: dict = {}


def metadata_for(cfg) -> HashMetadata:
    """The hash metadata that belongs to a model configuration (deterministic; one table per
    Engram layer, ``rows_per_table`` split over the (ngram-1) * heads id slots)."""
    ec = cfg.engram
    key = (cfg.vocab, ec.rows_per_table, len(ec.layers), ec.heads, ec.ngram)
    if key not in _MD_CACHE:
        per_head = max(16, ec.rows_per_table // ((ec.ngram - 1) * ec.heads) - 8)
        _MD_CACHE[key] = HashMetadata.synthetic(cfg.vocab, rows_per_head=per_head, tables=len(ec.layers), heads=ec.heads,
                                                ngram=ec.ngram, seed=20240917)
    return _MD_CACHE[key]


def table_rows(cfg) -> int:
    return metadata_for(cfg).table_rows


def hash_positions(md: HashMetadata, prev: Sequence[int], tokens: Sequence[int], start: int) -> np.ndarray:
    """Row ids [T, tables, ids] of ``tokens`` placed at positions start.. after the ``prev`` tokens
    (the up to ngram-1 tokens right before ``start``, oldest first)."""
    h = HashHistory(lineage=1, pad_token=md.pad_token, ngram=md.ngram)
    h.position = start
    rec = list(reversed(list(prev)[-(md.ngram - 1):]))
    h.recent = rec + [md.pad_token] * (md.ngram - 1 - len(rec))
    return h.prepare(list(tokens), md).rows


def apply_reference(x: torch.Tensor, rows: torch.Tensor, wkv: torch.Tensor, qw: torch.Tensor, kw: torch.Tensor,
                    eps: float) -> torch.Tensor:
    """x [T, m, d] residual copies, rows [T, ids*256] looked-up memory -> gated update (fp32)."""
    T, m, d = x.shape
    kv = (rows @ wkv.t()).reshape(T, m + 1, d)
    return gate_reference(x, kv, qw, kw, eps)
