"""Number-format codecs in plain PyTorch: the CPU oracles for every quantised layout.

* UE8M0 power-of-two scales (reference decode rule: kernels/core.cu:973)
* MXFP8 activations: e4m3 values + one UE8M0 per 32 along K
  (reference: kernels/moe_frontend.cuh:22-26 ``scale = 2^ceil(log2(amax/448))``)
* block-scaled FP8 weights: 128x128 fp32 scales or 32x32 UE8M0 scales
  (reference: src/layout.rs:220-295, src/blockscaled.rs)
* MXFP4 experts: packed e2m1 nibbles [n, k/2] + UE8M0 [n, k/32] (reference: src/weights.rs:541)
* KV page formats V41 (FP8 + UE8M0/32) and V41Fp4 (e2m1 + e4m3/16) (reference: src/attention.rs:18-38)
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

E4M3_MAX = 448.0
E2M1_MAX = 6.0
# magnitudes representable by e2m1, indexed by the low three bits of the nibble
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


# ---------------------------------------------------------------- UE8M0
def ue8m0_decode(code: torch.Tensor) -> torch.Tensor:
    """byte -> fp32 power of two. 255 -> NaN; 0 -> 2^-127 (a subnormal); else 2^(s-127)."""
    c = code.to(torch.int32)
    bits = torch.where(c == 0, torch.full_like(c, 1 << 22), c << 23)
    out = bits.view(torch.float32).clone()
    out[c == 255] = float("nan")
    return out


def ue8m0_encode_ceil(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x (x > 0), as a UE8M0 byte; zeros map to 2^-127."""
    x = x.to(torch.float32)
    e = torch.ceil(torch.log2(torch.clamp(x, min=2.0 ** -127)))
    # log2 can be one ulp off for exact powers of two; fix by checking
    p = torch.exp2(e)
    e = torch.where(p < x, e + 1, e)
    e = torch.where(torch.exp2(e - 1) >= x, e - 1, e)
    return torch.clamp(e + 127, 0, 254).to(torch.uint8)


# ---------------------------------------------------------------- e4m3
def e4m3_quant(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even, saturate to +-448 (``cvt.rn.satfinite.e4m3``)."""
    return torch.clamp(x.to(torch.float32), -E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def mxfp8_quant(x: torch.Tensor, group: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """[..., K] -> (e4m3 [..., K], ue8m0 [..., K/group]); scale = 2^ceil(log2(amax/448))."""
    *lead, K = x.shape
    assert K % group == 0
    g = x.to(torch.float32).reshape(*lead, K // group, group)
    amax = g.abs().amax(-1)
    code = ue8m0_encode_ceil(amax / E4M3_MAX)
    s = ue8m0_decode(code)
    q = e4m3_quant(g / s.unsqueeze(-1)).reshape(*lead, K)
    return q, code


def mxfp8_dequant(q: torch.Tensor, code: torch.Tensor, group: int = 32) -> torch.Tensor:
    *lead, K = q.shape
    s = ue8m0_decode(code).unsqueeze(-1)
    return (q.to(torch.float32).reshape(*lead, K // group, group) * s).reshape(*lead, K)


def fp8_act_quant_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Activation quant with one fp32 scale per 128 along K (scale = amax/448)."""
    *lead, K = x.shape
    assert K % 128 == 0
    g = x.to(torch.float32).reshape(*lead, K // 128, 128)
    s = torch.clamp(g.abs().amax(-1), min=1e-12) / E4M3_MAX
    q = e4m3_quant(g / s.unsqueeze(-1)).reshape(*lead, K)
    return q, s


def fp8_block_quant(w: torch.Tensor, block: int = 128, ue8m0: bool = False
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Weight [N, K] -> (e4m3 [N, K], scale [ceil(N/b), ceil(K/b)]); fp32 scales, or UE8M0
    bytes when ``ue8m0`` (the 32x32 checkpoint layout)."""
    N, K = w.shape
    nb, kb = -(-N // block), -(-K // block)
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32)
    wp[:N, :K] = w.to(torch.float32)
    t = wp.reshape(nb, block, kb, block)
    amax = t.abs().amax(dim=(1, 3))
    if ue8m0:
        code = ue8m0_encode_ceil(amax / E4M3_MAX)
        s = ue8m0_decode(code)
        q = e4m3_quant(t / s[:, None, :, None]).reshape(nb * block, kb * block)[:N, :K]
        return q.contiguous(), code
    s = torch.clamp(amax, min=1e-12) / E4M3_MAX
    q = e4m3_quant(t / s[:, None, :, None]).reshape(nb * block, kb * block)[:N, :K]
    return q.contiguous(), s


def fp8_block_dequant(q: torch.Tensor, s: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    if s.dtype == torch.uint8:
        s = ue8m0_decode(s)
    se = s.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.to(torch.float32) * se


# ---------------------------------------------------------------- e2m1 / MXFP4
def e2m1_quant_codes(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit codes (sign<<3 | magnitude index), round to nearest, ties to even
    mantissa, saturating at 6."""
    a = x.abs().to(torch.float32)
    vals = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=x.device)
    # midpoints between consecutive magnitudes; ties go to the even code (index parity)
    mids = (vals[1:] + vals[:-1]) / 2
    idx = torch.zeros_like(a, dtype=torch.int64)
    for i in range(7):
        up = (a > mids[i]) | ((a == mids[i]) & ((i + 1) % 2 == 0))
        idx = torch.where(up, torch.full_like(idx, i + 1), idx)
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return (idx | (sign.to(torch.int64) << 3)).to(torch.uint8)


def e2m1_decode_codes(c: torch.Tensor) -> torch.Tensor:
    vals = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=c.device)
    c = c.to(torch.int64)
    mag = vals[c & 7]
    return torch.where((c & 8) != 0, -mag, mag)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] 4-bit codes -> [..., K/2] bytes, even element in the low nibble."""
    lo, hi = codes[..., 0::2], codes[..., 1::2]
    return (lo | (hi << 4)).to(torch.uint8)


def unpack_nibbles(p: torch.Tensor) -> torch.Tensor:
    lo, hi = p & 0xF, p >> 4
    return torch.stack([lo, hi], -1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def mxfp4_quant(w: torch.Tensor, group: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """[..., K] -> (packed e2m1 [..., K/2], ue8m0 [..., K/group]); scale = 2^ceil(log2(amax/6))."""
    *lead, K = w.shape
    assert K % group == 0
    g = w.to(torch.float32).reshape(*lead, K // group, group)
    code = ue8m0_encode_ceil(g.abs().amax(-1) / E2M1_MAX)
    code = torch.clamp(code, max=247)            # loader contract: scale byte <= 247
    s = ue8m0_decode(code)
    q = e2m1_quant_codes(g / s.unsqueeze(-1)).reshape(*lead, K)
    return pack_nibbles(q), code


def mxfp4_dequant(p: torch.Tensor, code: torch.Tensor, group: int = 32) -> torch.Tensor:
    v = e2m1_decode_codes(unpack_nibbles(p))
    *lead, K = v.shape
    s = ue8m0_decode(code).unsqueeze(-1)
    return (v.reshape(*lead, K // group, group) * s).reshape(*lead, K)


# ---------------------------------------------------------------- KV page rows
def kv_v41_encode(k: torch.Tensor) -> torch.Tensor:
    """Window-cache row: [..., D] -> bytes [..., D + D/32] (D e4m3 then D/32 ue8m0).
    528 bytes at D=512 (reference runtime/kernels/kv-v41-v1/kv_store.cu:33-150)."""
    q, code = mxfp8_quant(k.to(torch.bfloat16).to(torch.float32), 32)
    return torch.cat([q.view(torch.uint8), code], -1)


def kv_v41_decode(row: torch.Tensor, dim: int) -> torch.Tensor:
    q = row[..., :dim].contiguous().view(torch.float8_e4m3fn)
    return mxfp8_dequant(q, row[..., dim:dim + dim // 32], 32)


def kv_fp4_scale(amax: torch.Tensor) -> torch.Tensor:
    """Compressed-cache scale per 16 values: e4m3(amax/6), never below the smallest normal."""
    return e4m3_quant(torch.clamp(amax / E2M1_MAX, min=2.0 ** -6))


def kv_v41fp4_encode(k: torch.Tensor) -> torch.Tensor:
    """Compressed-cache row: [..., D] -> bytes [..., D/2 + D/16] (packed e2m1 then one e4m3
    scale per 16). 288 bytes at D=512 (reference runtime/kernels/compression-fp4-v1)."""
    *lead, D = k.shape
    g = k.to(torch.bfloat16).to(torch.float32).reshape(*lead, D // 16, 16)
    s8 = kv_fp4_scale(g.abs().amax(-1))
    s = s8.to(torch.float32).unsqueeze(-1)
    codes = e2m1_quant_codes(g / s).reshape(*lead, D)
    return torch.cat([pack_nibbles(codes), s8.view(torch.uint8)], -1)


def kv_v41fp4_decode(row: torch.Tensor, dim: int) -> torch.Tensor:
    v = e2m1_decode_codes(unpack_nibbles(row[..., :dim // 2]))
    s = row[..., dim // 2: dim // 2 + dim // 16].contiguous().view(torch.float8_e4m3fn).to(torch.float32)
    *lead, D = v.shape
    return (v.reshape(*lead, D // 16, 16) * s.unsqueeze(-1)).reshape(*lead, D)


def index_key_encode(k: torch.Tensor) -> torch.Tensor:
    """Index key: [..., Di] -> bytes [..., Di/2 + Di/32] (68 B at 128 dims;
    reference kernels/index_bf16.cu:8-10)."""
    p, code = mxfp4_quant(k, 32)
    return torch.cat([p, code], -1)


def index_key_decode(row: torch.Tensor, dim: int) -> torch.Tensor:
    return mxfp4_dequant(row[..., :dim // 2], row[..., dim // 2: dim // 2 + dim // 32], 32)


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)
