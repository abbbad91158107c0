"""Counter-addressed random stream for sampling.

The complete random state is (seed, domain, absolute token position): draws are addressed, not
consumed, so discarding speculative rows never shifts another position's draw.  The PRF and
its constants follow the reference contract (src/categorical.rs:11-40): the first 8 bytes of
SHA-256("canada-sampling-v1\\0" || seed || domain || position), shifted to 53 bits.
"""
from __future__ import annotations

import hashlib
import struct

TARGET_DOMAIN = 0x43415F5441524745
DRAFT_DOMAIN = 0x43415F4452414654
ACCEPT_DOMAIN = 0x43415F4143434550
RESIDUAL_DOMAIN = 0x43415F5245534944
_M64 = (1 << 64) - 1


def uniform(seed: int, domain: int, position: int) -> float:
    h = hashlib.sha256()
    h.update(b"canada-sampling-v1\0")
    h.update(struct.pack("<QQQ", seed & _M64, domain & _M64, position & _M64))
    bits = struct.unpack("<Q", h.digest()[:8])[0] >> 11
    return bits * (1.0 / 9007199254740992.0)


def block_round_seed(seed: int, frontier: int) -> int:
    """Re-key every verification round: block verification inspects later draws even when it
    commits a shorter prefix, so the next round must not reuse them."""
    h = hashlib.sha256()
    h.update(b"canada-block-round-v1\0")
    h.update(struct.pack("<QQ", seed & _M64, frontier & _M64))
    return struct.unpack("<Q", h.digest()[:8])[0]


def round_uniforms(seed: int, frontier: int, depth: int):
    """Draws of one verification round at committed length `frontier`:
    (draft draws [depth], acceptance draws [depth], final draw)."""
    rs = block_round_seed(seed, frontier)
    draft = [uniform(rs, DRAFT_DOMAIN, frontier + i) for i in range(depth)]
    accept = [uniform(rs, ACCEPT_DOMAIN, frontier + i) for i in range(depth)]
    final = uniform(rs, RESIDUAL_DOMAIN, frontier)
    return draft, accept, final
