"""tcgen05 GEMM against fp32 PyTorch references."""
import pytest
import torch

from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 512), (300, 256, 1024), (1000, 384, 4096)])
def test_gemm_bf16(M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    st = native.StatusWord(DEV)
    for okind, dt in ((2, torch.bfloat16), (0, torch.float32)):
        c = torch.zeros(M, N, device=DEV, dtype=dt)
        native.call("tf_gemm_tc", 0, a, K, b, K, c, N, M, N, K, None, 0, None, 0, okind, None, None, 0, st.t)
        torch.cuda.synchronize()
        st.check()
        assert _rel(c, a.float() @ b.float().t()) < 5e-3


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (200, 256, 1024), (1024, 512, 4096)])
def test_gemm_fp8_block_scaled(M, N, K):
    torch.manual_seed(1)
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV) * 0.05
    fw = E.quant_fp8_device(w)
    g = x.view(M, K // 128, 128)
    sa = g.abs().amax(-1).clamp_min(1e-12) / 448.0
    xq = (g / sa[:, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(M, K)
    xd = (xq.float().view(M, K // 128, 128) * sa[:, :, None]).view(M, K)
    st = native.StatusWord(DEV)
    c = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    native.call("tf_gemm_tc", 2, xq, K, fw.q, K, c, N, M, N, K, sa.contiguous(), K // 128, fw.s, K // 128, 2, None, None, 0, st.t)
    torch.cuda.synchronize()
    st.check()
    assert _rel(c, xd @ E.dequant_fp8(fw).t()) < 5e-3
    # unscaled fp8
    c2 = torch.zeros(M, N, device=DEV)
    native.call("tf_gemm_tc", 1, xq, K, fw.q, K, c2, N, M, N, K, None, 0, None, 0, 0, None, None, 0, st.t)
    torch.cuda.synchronize()
    st.check()
    assert _rel(c2, xq.float() @ fw.q.float().t()) < 1e-3
