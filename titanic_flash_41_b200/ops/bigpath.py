"""Large-row-count (prefill) execution of the linear layers and routed experts on the tcgen05
GEMMs.

Block-scaled form (``EngineConfig.prefill_mx``, the default): activations are quantised to MXFP8
(one UE8M0 scale per row and 32 inputs), dense FP8 weights keep their values with their
power-of-two block scales re-expressed per 32 inputs, and MXFP4 expert weights are read as stored;
the tensor core applies both scale vectors (``csrc/gemm_mx.cu``).

fp32-scaled form (weights whose scales are not powers of two, or ``prefill_mx`` off): activations
get one fp32 scale per (row, 128), dense weights are block-128 FP8, MXFP4 expert weights are
re-expressed per chunk as block-scaled FP8, and partial sums are promoted per 128 inputs in software
(``csrc/gemm_tc.cu``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import mx, native


class BigPath:
    def __init__(self, engine):
        self.e = engine
        self.buf = {}
        self._converted = None      # layer whose experts currently sit in the FP8 staging copy
        self._mx_layer = None       # layer whose expert scales currently sit in the block-scaled layout
        self._mx_u = []
        self.resident = engine.world >= 4          # per-layer FP8 expert copies stay on the device
        self._resident = {}

    def _get(self, name, shape, dtype):
        t = self.buf.get(name)
        n = 1
        for s in shape:
            n *= s
        if t is None or t.numel() < n or t.dtype != dtype:
            t = torch.empty(n, dtype=dtype, device=self.e.dev)
            self.buf[name] = t
        return t[:n].view(*shape)

    # ---- dense ----------------------------------------------------------------------------
    def _units(self, w):
        """UE8M0 scales of a dense weight in the block-scaled kernel's layout (cached on the weight)."""
        if w.sfu is None:
            u = mx.units_from_block_scales(w.s, w.q.shape[0], w.q.shape[1])
            w.sfu = u if u is not None else False
        return w.sfu if w.sfu is not False else None

    def _gemm_mx(self, eng, x16: torch.Tensor, w, out: torch.Tensor, M: int, w3=None) -> bool:
        if not eng.ecfg.prefill_mx:
            return False
        sfb = self._units(w)
        sfb3 = self._units(w3) if w3 is not None else None
        if sfb is None or (w3 is not None and sfb3 is None):
            return False
        N, K = w.q.shape
        xq = self._get("xq_mx", (M, K), torch.uint8)
        sfa = self._get("sfa_mx", (K // 128, mx.sf_units(M, 128), 128), torch.uint8)
        mx.quant_rows(x16, M, K, xq, sfa)
        st = eng.status.t
        if w3 is None:
            if out.dtype in (torch.float32, torch.bfloat16):
                mx.gemm(xq, sfa, w.q, sfb, out, M, N, K, st)
            else:
                tmp = self._get("gemm_tmp", (M, N), torch.bfloat16)
                mx.gemm(xq, sfa, w.q, sfb, tmp, M, N, K, st)
                out[:M, :N].copy_(tmp)
            return True
        y = self._get("dual_y", (M, 2 * N), torch.bfloat16)
        mx.gemm(xq, sfa, w.q, sfb, y, M, N, K, st)
        mx.gemm(xq, sfa, w3.q, sfb3, y[:, N:], M, N, K, st)
        assert out.dtype == torch.float16
        native.call("tf_swiglu_rows", y, 2, 2 * N, out, out.stride(0), None, None, M, N, eng.cfg.swiglu_limit, None)
        return True

    def gemm(self, eng, x16: torch.Tensor, w, out: torch.Tensor, M: int, w3=None) -> None:
        if self._gemm_mx(eng, x16, w, out, M, w3):
            return
        N, K = w.q.shape
        xq = self._get("xq", (M, K), torch.uint8)
        xs = self._get("xs", (M, K // 128), torch.float32)
        xk = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x16.dtype]
        native.call("tf_quant_rows", x16, xk, x16.stride(0), None, 1, None, xq, xs, M, K)
        st = eng.status.t
        if w3 is None:
            if out.dtype in (torch.float32, torch.bfloat16):
                okind = 0 if out.dtype == torch.float32 else 2
                native.call("tf_gemm_tc", 2, xq, K, w.q, K, out, out.stride(0), M, N, K, xs, K // 128, w.s,
                            K // 128, okind, None, None, 0, st)
            else:
                tmp = self._get("gemm_tmp", (M, N), torch.bfloat16)
                native.call("tf_gemm_tc", 2, xq, K, w.q, K, tmp, N, M, N, K, xs, K // 128, w.s, K // 128, 2,
                            None, None, 0, st)
                out[:M, :N].copy_(tmp)
            return
        # dual: gate and up projections side by side, then the clamped SwiGLU
        y = self._get("dual_y", (M, 2 * N), torch.bfloat16)
        native.call("tf_gemm_tc", 2, xq, K, w.q, K, y, 2 * N, M, N, K, xs, K // 128, w.s, K // 128, 2, None, None, 0, st)
        native.call("tf_gemm_tc", 2, xq, K, w3.q, K, y[:, N:], 2 * N, M, N, K, xs, K // 128, w3.s, K // 128, 2,
                    None, None, 0, st)
        assert out.dtype == torch.float16
        native.call("tf_swiglu_rows", y, 2, 2 * N, out, out.stride(0), None, None, M, N, eng.cfg.swiglu_limit, None)

    # ---- routed experts ---------------------------------------------------------------------
    def moe(self, eng, L, T: int, b: dict, with_shared: bool = True, out: Optional[torch.Tensor] = None) -> None:
        """Routed experts of this rank (+ the shared expert) over the T rows in ``b`` -> ``b['delta']``
        (fp32), or -> ``out`` (bf16 or fp32 [T, hidden]) when given."""
        cfg = eng.cfg
        d, I, El, k = cfg.hidden, cfg.moe_inter, eng.El, cfg.topk
        npairs = T * k
        cap = npairs + El * 127
        cap = -(-cap // 128) * 128
        max_tiles = cap // 128
        i32 = torch.int32
        z = self.buf.get("counts")
        if z is None:
            z = torch.zeros(El, dtype=i32, device=eng.dev)
            self.buf["counts"] = z
        offsets = self._get("offsets", (El + 1,), i32)
        cursor = self._get("cursor", (El,), i32)
        tile_e = self._get("tile_e", (max_tiles,), i32)
        ntile = self._get("ntile", (2,), i32)
        pair_dst = self._get("pair_dst", (npairs,), i32)
        e_lo = eng.rank * El
        native.call("tf_moe_plan", b["ids"], npairs, e_lo, El, z, offsets, cursor, tile_e, max_tiles, ntile[0:1],
                    ntile[1:2], pair_dst)
        st = eng.status.t
        if eng.ecfg.prefill_mx and d % 128 == 0 and I % 256 == 0 and d % 256 == 0:
            # block-scaled form: the packed e2m1 weights are read as stored; their UE8M0 scales are
            # re-ordered into the kernel's layout once per layer visit (a few hundred MB of traffic
            # against the GBs of the FP8 re-expression below)
            if self._mx_layer is not L:
                u = self._get("mx_units", (3, (d // 128) * mx.sf_units(El * I, 256) * 128), torch.uint8)
                self._mx_u = []
                for j, (sc, rows, kk) in enumerate(((L.es1, El * I, d), (L.es3, El * I, d), (L.es2, El * d, I))):
                    uu = u[j][: (kk // 128) * mx.sf_units(rows, 256) * 128].view(kk // 128, mx.sf_units(rows, 256), 128)
                    native.call("tf_mx_sf_to_units", sc, uu, rows, kk, uu.shape[1])
                    self._mx_u.append(uu)
                self._mx_layer = L
            u1, u3, u2 = self._mx_u
            xp = self._get("xp", (cap, d), torch.uint8)
            sfx = self._get("sfx_mx", (d // 128, cap // 32, 128), torch.uint8)
            mx.quant_rows(b["h16"], npairs, d, xp, sfx, x_div=k, pair_dst=pair_dst)
            y1 = self._get("y1", (cap, 2 * I), torch.bfloat16)
            mx.gemm(xp, sfx, L.ew1, u1, y1, cap, I, d, st, b_fp4=True, b_rows=El * I, tile_expert=tile_e,
                    num_m_tiles=ntile[0:1])
            mx.gemm(xp, sfx, L.ew3, u3, y1[:, I:], cap, I, d, st, b_fp4=True, b_rows=El * I, tile_expert=tile_e,
                    num_m_tiles=ntile[0:1])
            aq = self._get("aq", (cap, I), torch.uint8)
            sfq = self._get("sfq_mx", (I // 128, cap // 32, 128), torch.uint8)
            native.call("tf_swiglu_rows_mx_units", y1, 2 * I, aq, sfq, cap // 32, cap, I, cfg.swiglu_limit, ntile[1:2])
            y2 = self._get("y2", (cap, d), torch.bfloat16)
            mx.gemm(aq, sfq, L.ew2, u2, y2, cap, d, I, st, b_fp4=True, b_rows=El * d, tile_expert=tile_e,
                    num_m_tiles=ntile[0:1])
            self._moe_tail(eng, L, T, b, y2, pair_dst, with_shared, out)
            return
        # expert weights of this layer as block-scaled FP8: [El, 2I, d] (w1 | w3) and [El, d, I]
        def convert(w13, s13, w2, s2):
            native.call("tf_mxfp4_to_fp8_block", L.ew1, L.es1, w13, s13, El, I, d, 0, 2 * I)
            native.call("tf_mxfp4_to_fp8_block", L.ew3, L.es3, w13, s13, El, I, d, I, 2 * I)
            native.call("tf_mxfp4_to_fp8_block", L.ew2, L.es2, w2, s2, El, d, I, 0, d)
        if self.resident:
            # enough HBM per rank (experts split over >= 4 ranks): every layer keeps its FP8 copy
            keep = self._resident.get(id(L))
            if keep is None:
                keep = (torch.empty(El, 2 * I, d, dtype=torch.uint8, device=eng.dev),
                        torch.empty(El * 2 * I // 128, d // 128, dtype=torch.float32, device=eng.dev),
                        torch.empty(El, d, I, dtype=torch.uint8, device=eng.dev),
                        torch.empty(El * d // 128, I // 128, dtype=torch.float32, device=eng.dev))
                convert(*keep)
                self._resident[id(L)] = keep
            w13, s13, w2, s2 = keep
        else:
            w13 = self._get("w13", (El, 2 * I, d), torch.uint8)
            s13 = self._get("s13", (El * 2 * I // 128, d // 128), torch.float32)
            w2 = self._get("w2", (El, d, I), torch.uint8)
            s2 = self._get("s2", (El * d // 128, I // 128), torch.float32)
            if self._converted is not L:
                # consecutive chunks of one layer (layer-major prefill) reuse the converted copy
                convert(w13, s13, w2, s2)
                self._converted = L
        # gather + quantise token rows into the expert-sorted padded matrix
        xp = self._get("xp", (cap, d), torch.uint8)
        xps = self._get("xps", (cap, d // 128), torch.float32)
        native.call("tf_quant_rows", b["h16"], 1, d, None, k, pair_dst, xp, xps, npairs, d)
        y1 = self._get("y1", (cap, 2 * I), torch.bfloat16)
        native.call("tf_gemm_tc", 2, xp, d, w13, d, y1, 2 * I, cap, 2 * I, d, xps, d // 128, s13, d // 128, 2,
                    tile_e, ntile[0:1], El, st)
        aq = self._get("aq", (cap, I), torch.uint8)
        aqs = self._get("aqs", (cap, I // 128), torch.float32)
        native.call("tf_swiglu_rows", y1, 2, 2 * I, None, 0, aq, aqs, cap, I, cfg.swiglu_limit, ntile[1:2])
        y2 = self._get("y2", (cap, d), torch.bfloat16)
        native.call("tf_gemm_tc", 2, aq, I, w2, I, y2, d, cap, d, I, aqs, I // 128, s2, I // 128, 2,
                    tile_e, ntile[0:1], El, st)
        self._moe_tail(eng, L, T, b, y2, pair_dst, with_shared, out)

    def _moe_tail(self, eng, L, T: int, b: dict, y2, pair_dst, with_shared: bool, out) -> None:
        """Shared expert, then the weighted sum of every row's expert outputs (+ shared) -> delta / out."""
        cfg = eng.cfg
        shared = None
        if cfg.n_shared and with_shared:
            eng._linear(b["h16"], L.sw1, b["s_act"], T, w3=L.sw3)
            eng._linear(b["s_act"], L.sw2, b["s_y"], T)
            shared = b["s_y"]
        dst = b["delta"] if out is None else out
        native.call("tf_moe_combine_perm", y2, 2, cfg.hidden, pair_dst, b["wts"], shared, dst,
                    2 if dst.dtype == torch.bfloat16 else 0, T, cfg.hidden, cfg.topk)


def attach(engine) -> BigPath:
    """Route rows beyond the small-M limit through the tensor-core path."""
    bp = BigPath(engine)
    engine.big_gemm = bp.gemm
    engine.big_moe_full = bp.moe
    return bp
