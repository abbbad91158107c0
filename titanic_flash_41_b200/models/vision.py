"""Vision tower: ViT over 14x14 patches -> 3x3 unfold -> two-layer aligner -> image token span.

``VisionOracle`` is the fp32 PyTorch definition; ``VisionTower`` runs the same network on the
device with the tcgen05 bf16 GEMM for every projection and for both attention products
(QK^T and PV per head) and the glue kernels of ``csrc/vision.cu`` in between
(reference: src/vision.rs:139 Vision, :481 encode, :386 encode_split; kernels/vision.cu).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config import VisionConfig

HEAD = 64


def init_vision_weights(vc: VisionConfig, d_model: int, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    w, pk = vc.hidden, 3 * vc.patch * vc.patch

    def mat(n, k, std=None):
        return torch.randn(n, k, generator=g) * (std or 1.0 / math.sqrt(k))
    W = {"patch.weight": mat(w, pk), "patch.bias": torch.randn(w, generator=g) * 0.02,
         "norm.weight": 1 + 0.05 * torch.randn(w, generator=g),
         "align1.weight": mat(d_model, w * vc.downsample ** 2), "align1.bias": torch.randn(d_model, generator=g) * 0.02,
         "align2.weight": mat(d_model, d_model), "align2.bias": torch.randn(d_model, generator=g) * 0.02,
         "start": torch.randn(d_model, generator=g) * 0.02, "newline": torch.randn(d_model, generator=g) * 0.02,
         "end": torch.randn(d_model, generator=g) * 0.02}
    for l in range(vc.layers):
        p = f"blocks.{l}."
        W[p + "norm1.weight"] = 1 + 0.05 * torch.randn(w, generator=g)
        W[p + "qkv.weight"], W[p + "qkv.bias"] = mat(3 * w, w), torch.randn(3 * w, generator=g) * 0.02
        W[p + "proj.weight"], W[p + "proj.bias"] = mat(w, w), torch.randn(w, generator=g) * 0.02
        W[p + "norm2.weight"] = 1 + 0.05 * torch.randn(w, generator=g)
        W[p + "gate_up.weight"] = mat(2 * vc.intermediate, w)
        W[p + "down.weight"] = mat(w, vc.intermediate)
    return {k: v.bfloat16().float() for k, v in W.items()}


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope2d(t: torch.Tensor, grid_w: int) -> torch.Tensor:
    """t [n, heads, 64]: pairs (c, c+32); the first 16 pairs follow the patch row, the rest the column."""
    n = t.shape[0]
    rows = torch.arange(n)
    pair = torch.arange(32)
    freq = 1.0 / (10000.0 ** ((pair % 16).float() / 16.0))
    pos = torch.where(pair[None, :] < 16, (rows[:, None] // grid_w).float(), (rows[:, None] % grid_w).float())
    ang = pos * freq[None, :]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = t[..., :32], t[..., 32:]
    return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)


class VisionOracle:
    def __init__(self, vc: VisionConfig, d_model: int, W: Dict[str, torch.Tensor], eps: float = 1e-6):
        self.vc, self.d, self.W, self.eps = vc, d_model, W, eps

    def encode(self, patches: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        """patches [gh*gw, 588] -> span [tokens, d_model] (fp32)."""
        vc, W = self.vc, self.W
        heads = vc.hidden // HEAD
        x = patches.float() @ W["patch.weight"].t() + W["patch.bias"]
        n = x.shape[0]
        for l in range(vc.layers):
            p = f"blocks.{l}."
            h = _rms(x, W[p + "norm1.weight"], self.eps)
            qkv = h @ W[p + "qkv.weight"].t() + W[p + "qkv.bias"]
            q, k, v = (qkv[:, i * vc.hidden:(i + 1) * vc.hidden].view(n, heads, HEAD) for i in range(3))
            q, k = _rope2d(q, gw), _rope2d(k, gw)
            att = torch.softmax(torch.einsum("nhd,mhd->hnm", q, k) / math.sqrt(HEAD), -1)
            o = torch.einsum("hnm,mhd->nhd", att, v).reshape(n, vc.hidden)
            x = x + o @ W[p + "proj.weight"].t() + W[p + "proj.bias"]
            h = _rms(x, W[p + "norm2.weight"], self.eps)
            gu = h @ W[p + "gate_up.weight"].t()
            act = torch.nn.functional.silu(gu[:, :vc.intermediate]) * gu[:, vc.intermediate:]
            x = x + act @ W[p + "down.weight"].t()
        x = _rms(x, W["norm.weight"], self.eps)
        ds = vc.downsample
        oh, ow = -(-gh // ds), -(-gw // ds)
        img = torch.zeros(oh * ds, ow * ds, vc.hidden)
        img[:gh, :gw] = x.view(gh, gw, vc.hidden)
        # channel-major, then dy, dx (the order of F.unfold)
        u = img.view(oh, ds, ow, ds, vc.hidden).permute(0, 2, 4, 1, 3).reshape(oh * ow, vc.hidden * ds * ds)
        f = torch.nn.functional.gelu(u @ W["align1.weight"].t() + W["align1.bias"])
        f = f @ W["align2.weight"].t() + W["align2.bias"]
        rows = [W["start"][None]]
        for y in range(oh):
            rows += [f[y * ow:(y + 1) * ow], W["newline"][None]]
        rows.append(W["end"][None])
        return torch.cat(rows, 0)


class VisionTower:
    """Device implementation.  All projections run through ``tf_gemm_tc`` (bf16 x bf16)."""

    def __init__(self, vc: VisionConfig, d_model: int, W: Dict[str, torch.Tensor], device="cuda", eps: float = 1e-6):
        from ..ops import native
        self.n, self.vc, self.d, self.eps, self.dev = native, vc, d_model, eps, torch.device(device)
        self.pk = 3 * vc.patch * vc.patch
        self.pk_pad = -(-self.pk // 64) * 64
        bf = lambda t: t.to(self.dev, torch.bfloat16).contiguous()
        self.W = {k: bf(v) for k, v in W.items()}
        pw = torch.zeros(vc.hidden, self.pk_pad)
        pw[:, :self.pk] = W["patch.weight"]
        self.W["patch.weight"] = bf(pw)
        self.status = native.StatusWord(self.dev)

    def _gemm(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        M, K = a.shape
        N = w.shape[0]
        self.n.call("tf_gemm_tc", 0, a, a.stride(0), w, w.stride(0), out, out.stride(0), M, N, K, None, 0, None, 0,
                    2 if out.dtype == torch.bfloat16 else 0, None, None, 0, self.status.t)
        return out

    def _linear(self, a, name, bias=True):
        w = self.W[name + ".weight"]
        out = torch.empty(a.shape[0], w.shape[0], dtype=torch.bfloat16, device=self.dev)
        self._gemm(a, w, out)
        if bias:
            self.n.call("tf_vis_bias", out, self.W[name + ".bias"], out, out.numel(), w.shape[0])
        return out

    def encode(self, patches: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        """patches [gh*gw, 588] bf16 -> span [tokens, d_model] bf16."""
        vc, nat, dev = self.vc, self.n, self.dev
        n, width = gh * gw, vc.hidden
        heads = width // HEAD
        n_pad = -(-n // 128) * 128
        bf = dict(dtype=torch.bfloat16, device=dev)
        pp = torch.zeros(n, self.pk_pad, **bf)
        pp[:, :self.pk] = patches.to(dev, torch.bfloat16)
        x = self._linear(pp, "patch")
        h = torch.empty(n, width, **bf)
        q, k, v = (torch.zeros(heads, n_pad, HEAD, **bf) for _ in range(3))
        vt = torch.empty(128, n_pad, **bf)
        scores = torch.empty(n, n_pad, dtype=torch.float32, device=dev)
        probs = torch.empty(n, n_pad, **bf)
        o128 = torch.empty(n, 128, **bf)
        att = torch.empty(n, width, **bf)
        delta = None
        for l in range(vc.layers):
            p = f"blocks.{l}."
            nat.call("tf_vis_norm", x, delta, self.W[p + "norm1.weight"], h, n, width, self.eps)
            qkv = self._linear(h, p + "qkv")
            nat.call("tf_vis_rope_split", qkv, q, k, v, n, n_pad, gw, heads)
            for hd in range(heads):
                self._gemm(q[hd, :n], k[hd], scores)
                nat.call("tf_vis_softmax", scores, probs, n, n, n_pad, 1.0 / math.sqrt(HEAD))
                nat.call("tf_vis_transpose_pad", v[hd], vt, n, n_pad)
                self._gemm(probs, vt, o128)
                att[:, hd * HEAD:(hd + 1) * HEAD].copy_(o128[:, :HEAD])
            d1 = self._linear(att, p + "proj")
            nat.call("tf_vis_norm", x, d1, self.W[p + "norm2.weight"], h, n, width, self.eps)
            gu = self._linear(h, p + "gate_up", bias=False)
            act = torch.empty(n, vc.intermediate, **bf)
            nat.call("tf_vis_swiglu", gu, act, n, vc.intermediate)
            delta = self._linear(act, p + "down", bias=False)
        nat.call("tf_vis_norm", x, delta, self.W["norm.weight"], h, n, width, self.eps)
        ds = vc.downsample
        oh, ow = -(-gh // ds), -(-gw // ds)
        u = torch.empty(oh * ow, width * ds * ds, **bf)
        nat.call("tf_vis_unfold", h, u, gh, gw, width)
        f1 = self._linear(u, "align1")
        nat.call("tf_vis_gelu", f1, f1, f1.numel())
        f2 = self._linear(f1, "align2")
        tokens = oh * (ow + 1) + 2
        span = torch.empty(tokens, self.d, **bf)
        nat.call("tf_vis_span", f2, self.W["start"], self.W["newline"], self.W["end"], span, ow, tokens, self.d)
        self.status.check()
        return span
