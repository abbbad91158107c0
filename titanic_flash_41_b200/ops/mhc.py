"""mHC boundary ops on the device (kernels: csrc/mhc.cu; fp32 reference: models/oracle.py)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import native


class HcBoundary:
    """Per-sublayer boundary of the multi-copy residual: ``prepare`` collapses the H copies into
    the sublayer input (and normalises it), ``finish`` mixes the sublayer output back."""

    def __init__(self, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, H: int, d: int, iters: int = 20,
                 eps: float = 1e-6, rms_eps: float = 1e-6):
        self.fn, self.base, self.scale = fn.float().contiguous(), base.float().contiguous(), scale.float().contiguous()
        self.H, self.d, self.iters, self.eps, self.rms_eps = H, d, iters, eps, rms_eps
        self._coef: Optional[torch.Tensor] = None

    def prepare(self, x: torch.Tensor, norm_w: Optional[torch.Tensor] = None
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """x [T, H, d] bf16 -> (collapsed [T, d] bf16, normalised f16 or None)."""
        T = x.shape[0]
        nb = native.lib().tf_hc_coef_bytes()
        if self._coef is None or self._coef.shape[0] < T:
            self._coef = torch.empty(T, nb, dtype=torch.uint8, device=x.device)
        v = torch.empty(T, self.d, dtype=torch.bfloat16, device=x.device)
        h16 = torch.empty(T, self.d, dtype=torch.float16, device=x.device) if norm_w is not None else None
        native.call("tf_hc_prepare", x.contiguous(), self.fn, self.base, self.scale, self._coef, v, norm_w, h16, None,
                    T, self.H, self.d, self.iters, self.eps, self.rms_eps)
        return v, h16

    def finish(self, x: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
        """x [T, H, d] bf16 residual copies, a [T, d] fp32 sublayer output -> new copies [T, H, d] bf16."""
        T = x.shape[0]
        y = torch.empty_like(x)
        native.call("tf_hc_post", x.contiguous(), a.float().contiguous(), self._coef, y, T, self.H, self.d)
        return y

    def coefficients(self, T: int):
        """(pre [T,H], post [T,H], comb [T,H,H]) of the last ``prepare`` (for tests / tracing)."""
        c = self._coef[:T].view(torch.float32).view(T, -1)
        H = self.H
        return c[:, 0:H], c[:, 4:4 + H], c[:, 8:24].view(T, 4, 4)[:, :H, :H]
