"""tcgen05 GEMM against fp32 PyTorch references."""
import pytest
import torch

from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 512), (300, 256, 1024), (1000, 384, 4096),
                                   (4096, 2048, 512), (5000, 1024, 256)])   # the last two take 128x256 tiles
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


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (200, 256, 1024), (1024, 512, 4096), (4736, 1024, 1024)])
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


def _one_rank_workspace(nbytes):
    buf = torch.zeros(int(nbytes), dtype=torch.uint8, device=DEV)
    return buf, torch.tensor([buf.data_ptr()], dtype=torch.int64, device=DEV)


@pytest.mark.parametrize("kind,M,N,K", [(0, 512, 256, 1024), (2, 384, 128, 2048), (0, 2048, 384, 512),
                                        (2, 4864, 1024, 512)])
def test_allgather_gemm_single_rank(kind, M, N, K):
    """The all-gather form with one rank: copy CTAs move the shard into the gathered buffer with
    bulk copies, GEMM CTAs wait for each 128-row block.  Two calls exercise both slot parities."""
    torch.manual_seed(2)
    L = native.lib()
    buf, peers = _one_rank_workspace(L.tf_gemm_ag_workspace_bytes(kind, M, K, 1))
    st = native.StatusWord(DEV)
    w = torch.randn(N, K, device=DEV) * 0.05
    for epoch in (1, 2):
        x = torch.randn(M, K, device=DEV)
        off = int(L.tf_gemm_ag_shard_offset(kind, M, K, 1, epoch))
        c = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        if kind == 0:
            buf[off:off + M * K * 2].view(torch.bfloat16).view(M, K).copy_(x.bfloat16())
            wb = w.bfloat16()
            native.call("tf_gemm_ag", 0, wb, K, c, N, M, N, K, None, 0, 2, peers, buf, 1, 0, epoch, 4, 1000000, st.t)
            want = x.bfloat16().float() @ wb.float().t()
        else:
            fw = E.quant_fp8_device(w)
            g = x.view(M, K // 128, 128)
            sa = (g.abs().amax(-1).clamp_min(1e-12) / 448.0).contiguous()
            xq = (g / sa[:, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(M, K)
            buf[off:off + M * K].view(torch.float8_e4m3fn).view(M, K).copy_(xq)
            buf[off + M * K:off + M * K + M * (K // 128) * 4].view(torch.float32).view(M, K // 128).copy_(sa)
            native.call("tf_gemm_ag", 2, fw.q, K, c, N, M, N, K, fw.s, K // 128, 2, peers, buf, 1, 0, epoch, 4, 1000000, st.t)
            want = (xq.float().view(M, K // 128, 128) * sa[:, :, None]).view(M, K) @ E.dequant_fp8(fw).t()
        torch.cuda.synchronize()
        st.check()
        assert _rel(c, want) < 5e-3, epoch


def test_gemm_reduce_scatter_single_rank():
    """Reduce-scatter form with one rank: staged (transposed) tile stores into the receive slot and
    the owner-side sum must reproduce the plain GEMM."""
    torch.manual_seed(3)
    _rs_case(512, 256, 512)
    _rs_case(4864, 1024, 256)          # 128x256 tiles: two owner-side counters per tile


def _rs_case(M, N, K):
    L = native.lib()
    buf, peers = _one_rank_workspace(L.tf_gemm_rs_workspace_bytes(M, N, 1))
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    st = native.StatusWord(DEV)
    for epoch in (1, 2, 3):
        out = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        native.call("tf_gemm_rs", 0, a, K, b, K, M, N, K, None, 0, None, 0, peers, 1, 0, epoch, out, N, 1000000, st.t)
        torch.cuda.synchronize()
        st.check()
        assert _rel(out, a.float() @ b.float().t()) < 5e-3
