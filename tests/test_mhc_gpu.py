"""mHC boundary kernels against the oracle's fp32 functions."""
import pytest
import torch

from titanic_flash_41_b200.models import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H,d", [(1, 4, 512), (13, 4, 1280), (5, 2, 256)])
def test_prepare_and_post_match_oracle(T, H, d):
    from titanic_flash_41_b200.ops.mhc import HcBoundary
    dev = "cuda"
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, H, d, generator=g).bfloat16()
    fn = torch.randn(H * (2 + H), H * d, generator=g) * 0.05
    base = torch.randn(H * (2 + H), generator=g) * 0.3
    scale = torch.tensor([0.7, 1.3, 0.9])
    nw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    hb = HcBoundary(fn.to(dev), base.to(dev), scale.to(dev), H, d, iters=20, eps=1e-6, rms_eps=1e-6)
    v, h16 = hb.prepare(x.to(dev), nw.to(dev))
    pre, post, comb = oracle.hc_coefficients(x.float(), fn, base, scale, 20, 1e-6, 1e-6)
    gp, gq, gc = (t.float().cpu() for t in hb.coefficients(T))
    assert (gp - pre).abs().max() < 2e-3 and (gq - post).abs().max() < 2e-3 and (gc - comb).abs().max() < 2e-3
    want_v = oracle.hc_collapse(x.float(), pre)
    assert (v.float().cpu() - want_v).abs().max() < 0.03 * want_v.abs().max() + 1e-2
    want_h = oracle.rmsnorm(want_v.bfloat16().float(), nw.float(), 1e-6)
    assert (h16.float().cpu() - want_h).abs().max() < 0.05
    a = torch.randn(T, d, generator=g)
    y = hb.finish(x.to(dev), a.to(dev)).float().cpu()
    want_y = oracle.hc_post(x.float(), a, post, comb)
    assert (y - want_y).abs().max() < 0.03 * want_y.abs().max() + 1e-2
