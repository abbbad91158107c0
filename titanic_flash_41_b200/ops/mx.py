"""Host-side helpers of the block-scaled tensor-core GEMM (``csrc/gemm_mx.cu``): buffers of UE8M0
scales in the kernel's unit layout, and the calls that fill them.

Unit layout: 128 bytes hold the scales of 32 consecutive rows x 128 inputs, byte
``(row % 32) * 4 + (k // 32) % 4``; units are ordered ``[k // 128][row // 32]``.
"""
from __future__ import annotations

import torch

from . import native

F8 = torch.float8_e4m3fn


def sf_units(rows: int, tile_rows: int) -> int:
    """Units per 128-input block for ``rows`` rows read in tiles of ``tile_rows`` rows."""
    return -(-rows // tile_rows) * tile_rows // 32


def empty_units(rows: int, K: int, tile_rows: int, device) -> torch.Tensor:
    return torch.zeros(K // 128, sf_units(rows, tile_rows), 128, dtype=torch.uint8, device=device)


def units_from_rowmajor(s: torch.Tensor, K: int, tile_rows: int = 256) -> torch.Tensor:
    """Row-major UE8M0 scales ``[rows, K/32]`` (a checkpoint's MXFP4 expert scales) -> unit layout."""
    s = s.reshape(-1, K // 32).contiguous()
    out = empty_units(s.shape[0], K, tile_rows, s.device)
    native.call("tf_mx_sf_to_units", s, out, s.shape[0], K, out.shape[1])
    return out


def units_from_block_scales(s: torch.Tensor, rows: int, K: int, tile_rows: int = 256):
    """fp32 scales per 128 x 128 block -> unit layout, or None when some scale is not an exact power
    of two in the UE8M0 range (such a matrix stays on the fp32-scaled GEMM)."""
    out = empty_units(rows, K, tile_rows, s.device)
    bad = torch.zeros(1, dtype=torch.int32, device=s.device)
    native.call("tf_mx_block_scales_to_units", s, s.stride(0), out, rows, K, out.shape[1], bad)
    return out if int(bad.item()) == 0 else None


def quant_rows(x: torch.Tensor, M: int, K: int, q: torch.Tensor, sf: torch.Tensor, x_div: int = 1, pair_dst=None) -> None:
    """Rows of ``x`` (f32 / f16 / bf16) -> MXFP8 values ``q`` + unit-layout scales ``sf``."""
    kind = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x.dtype]
    native.call("tf_quant_rows_mx_units", x, kind, x.stride(0), x_div, pair_dst, q, sf, sf.shape[1], M, K)


def gemm(a_q: torch.Tensor, sfa: torch.Tensor, b_q: torch.Tensor, sfb: torch.Tensor, out: torch.Tensor, M: int, N: int,
         K: int, status, b_fp4: bool = False, b_rows: int = 0, tile_expert=None, num_m_tiles=None) -> None:
    okind = {torch.float32: 0, torch.bfloat16: 2}[out.dtype]
    native.call("tf_gemm_mx", a_q, K, b_q, K // 2 if b_fp4 else K, b_rows or N, 1 if b_fp4 else 0, sfa, sfa.shape[1], sfb,
                sfb.shape[1], out, out.stride(0), okind, M, N, K, tile_expert, num_m_tiles, status)


def units_to_rowmajor(sf: torch.Tensor, rows: int) -> torch.Tensor:
    """Inverse of the unit layout (tests, debugging): -> ``[rows, K/32]`` uint8."""
    kb, units, _ = sf.shape
    return sf.view(kb, units, 32, 4).permute(1, 2, 0, 3).reshape(units * 32, kb * 4)[:rows]
