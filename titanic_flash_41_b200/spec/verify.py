"""CPU (fp64) restatement of sampling and block verification: the oracle of ``csrc/sampling.cu``
and the path the CPU/gloo runs use.

Temperature and nucleus truncation are applied to BOTH the target and the draft law before the
recurrence, so the committed tokens follow the modified target law exactly (the reference only
admits T in {0,1}, top-p = 1: src/protocol.rs:253-262; block verification:
kernels/block_rejection.cuh:1-63, Sun et al. arXiv:2403.10444).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def modified_law(logits: torch.Tensor, temperature: float, top_p: float) -> torch.Tensor:
    """Row-wise softmax(logits / T) restricted to the smallest set of most likely tokens whose
    mass reaches top_p (ties at the cut are all kept), renormalised.  fp64."""
    x = logits.double()
    if temperature <= 0:
        p = torch.zeros_like(x)
        p.scatter_(-1, x.argmax(-1, keepdim=True), 1.0)
        return p
    p = torch.softmax(x / temperature, -1)
    if top_p < 1.0:
        srt, _ = torch.sort(p, -1, descending=True)
        cs = torch.cumsum(srt, -1)
        n_in = (cs < top_p).sum(-1, keepdim=True).clamp(max=p.shape[-1] - 1)
        thr = torch.gather(srt, -1, n_in)
        p = torch.where(p >= thr, p, torch.zeros_like(p))
        p = p / p.sum(-1, keepdim=True)
    return p


def sample_from(p: torch.Tensor, u: float) -> int:
    """Inverse-CDF draw in index order with the target kept strictly inside the mass."""
    cdf = torch.cumsum(p.double(), -1)
    total = float(cdf[-1])
    t = min(u * total, float(torch.nextafter(cdf[-1], torch.zeros((), dtype=torch.float64))))
    idx = int(torch.searchsorted(cdf, torch.tensor(t, dtype=torch.float64), right=True))
    idx = min(idx, p.numel() - 1)
    while idx > 0 and p[idx] <= 0:
        idx -= 1
    return idx


def block_verify(P: torch.Tensor, Q: Optional[torch.Tensor], proposals: Sequence[int],
                 u_accept: Sequence[float], u_final: float) -> Tuple[int, int]:
    """P [g+1, V] target laws, Q [g, V] draft laws (None: point masses at the proposals).
    Returns (accepted prefix length tau, token emitted after the accepted prefix)."""
    g = len(proposals)
    V = P.shape[-1]
    w = [1.0]
    for i in range(1, g + 1):
        x = proposals[i - 1]
        pt = float(P[i - 1, x])
        q = 1.0 if Q is None else float(Q[i - 1, x])
        ratio = w[-1] * pt / q if q > 0 else (1.0 if pt > 0 else 0.0)
        w.append(min(1.0, ratio))

    def residual(i: int) -> torch.Tensor:
        r = w[i] * P[i].double()
        if i < g:
            if Q is None:
                r = r.clone()
                r[proposals[i]] -= 1.0
            else:
                r = r - Q[i].double()
        return r.clamp_min(0.0)

    tau = 0
    for i in range(1, g + 1):
        if i < g:
            R = float(residual(i).sum())
            den = R + 1.0 - w[i]
            h = R / den if den > 0 else 0.0
        else:
            h = w[g]
        if u_accept[i - 1] < h:
            tau = i
    return tau, sample_from(residual(tau), u_final)


def causal_rows(confidences: Sequence[float], ladder: Sequence[float]) -> int:
    """How many proposals to verify.  Confidence j precedes proposal j (it is computed from what the
    drafter saw before sampling it): proposal 1 is always verified, proposal j >= 2 only while every
    running product c_1 ... c_i, i <= j, stays at or above its threshold ``ladder[i - 2]`` (the last
    threshold repeats).  The first failed threshold stops and a NaN stops, so the length never
    depends on later confidences or on excluded proposals (reference:
    src/dspark_generation.rs causal_ladder_rows)."""
    if not len(confidences):
        return 0
    n, prod = 1, float(confidences[0])
    for j in range(1, len(confidences)):
        prod *= float(confidences[j])
        thr = ladder[min(j - 1, len(ladder) - 1)]
        if not (prod >= thr):
            break
        n = j + 1
    return n
