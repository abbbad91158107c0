"""Block-scaled tcgen05 GEMM (UE8M0 scales per 32 inputs applied by the tensor core) against fp32
PyTorch references of the same operands."""
import pytest
import torch

from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import mx, native

pytestmark = pytest.mark.gpu
DEV = "cuda"
F8 = torch.float8_e4m3fn


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def _mx_reference(x):
    """MXFP8 of rows: power-of-two scale per 32 inputs, smallest with amax / scale <= 448."""
    M, K = x.shape
    g = x.float().view(M, K // 32, 32)
    amax = g.abs().amax(-1)
    e = torch.ceil(torch.log2(amax.clamp_min(1e-38) / 448.0)).clamp(-127, 127)
    e = torch.where(amax > 0, e, torch.full_like(e, -127.0))
    q = (g * torch.exp2(-e)[:, :, None]).clamp(-448, 448).to(F8)
    return q.view(M, K), (e + 127).to(torch.uint8)


def _random_fp8(n, k, gen):
    b = torch.randint(0, 256, (n, k), device=DEV, dtype=torch.uint8, generator=gen)
    b[(b & 0x7F) == 0x7F] = 0x38                 # no NaN codes
    return b


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_quantiser_matches_the_mx_definition(dtype):
    torch.manual_seed(0)
    M, K = 70, 512
    x = (torch.randn(M, K, device=DEV) * torch.logspace(-3, 2, K, device=DEV)).to(dtype)
    x[3] = 0
    q = torch.zeros(M, K, dtype=torch.uint8, device=DEV)
    sf = mx.empty_units(M, K, 128, DEV)
    mx.quant_rows(x, M, K, q, sf)
    torch.cuda.synchronize()
    rq, rs = _mx_reference(x)
    assert torch.equal(mx.units_to_rowmajor(sf, M), rs)
    assert torch.equal(q.view(F8).float(), rq.float())


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 512), (1000, 2048, 4096), (4200, 1024, 1024)])
def test_gemm_mx_fp8_weights(M, N, K):
    gen = torch.Generator(device=DEV).manual_seed(M + N)
    x = torch.randn(M, K, device=DEV, generator=gen) * 2
    aq = torch.zeros(M, K, dtype=torch.uint8, device=DEV)
    sfa = mx.empty_units(M, K, 128, DEV)
    mx.quant_rows(x, M, K, aq, sfa)
    a_deq = aq.view(F8).float().view(M, K // 32, 32) * torch.exp2(mx.units_to_rowmajor(sfa, M).float() - 127)[:, :, None]
    bq = _random_fp8(N, K, gen)
    bs = torch.randint(118, 126, (N, K // 32), device=DEV, dtype=torch.uint8, generator=gen)
    sfb = mx.units_from_rowmajor(bs, K)
    b_deq = bq.view(F8).float().view(N, K // 32, 32) * torch.exp2(bs.float() - 127)[:, :, None]
    want = a_deq.view(M, K).double() @ b_deq.view(N, K).double().t()
    st = native.StatusWord(DEV)
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 4e-3)):
        c = torch.full((M, N + 8), 7.0, device=DEV, dtype=dt)          # row pitch wider than N: the edge must stay untouched
        mx.gemm(aq, sfa, bq, sfb, c, M, N, K, st.t)
        torch.cuda.synchronize()
        st.check()
        assert _rel(c[:, :N], want) < tol
        assert bool((c[:, N:] == 7.0).all())


def test_gemm_mx_block_scales_of_dense_weights():
    """A dense FP8 matrix whose 128 x 128 scales are powers of two runs unchanged on the block-scaled
    path: same values as the fp32-scaled GEMM's operands."""
    torch.manual_seed(3)
    M, N, K = 256, 512, 1024
    w = torch.randn(N, K, device=DEV) * 0.05
    blk = w.view(N // 128, 128, K // 128, 128)
    s = torch.exp2(torch.ceil(torch.log2(blk.abs().amax(dim=(1, 3)) / 448.0)))
    wq = (blk / s[:, None, :, None]).clamp(-448, 448).to(F8).view(N, K)
    sfb = mx.units_from_block_scales(s.contiguous(), N, K)
    assert sfb is not None
    assert mx.units_from_block_scales((s * 1.5).contiguous(), N, K) is None
    x = torch.randn(M, K, device=DEV)
    aq = torch.zeros(M, K, dtype=torch.uint8, device=DEV)
    sfa = mx.empty_units(M, K, 128, DEV)
    mx.quant_rows(x, M, K, aq, sfa)
    a_deq = (aq.view(F8).float().view(M, K // 32, 32) * torch.exp2(mx.units_to_rowmajor(sfa, M).float() - 127)[:, :, None])
    w_deq = (wq.float().view(N // 128, 128, K // 128, 128) * s[:, None, :, None]).view(N, K)
    c = torch.zeros(M, N, device=DEV)
    st = native.StatusWord(DEV)
    mx.gemm(aq, sfa, wq.view(torch.uint8), sfb, c, M, N, K, st.t)
    torch.cuda.synchronize()
    st.check()
    assert _rel(c, a_deq.view(M, K).double() @ w_deq.double().t()) < 2e-5


def test_gemm_mx_grouped_mxfp4_experts():
    """Expert-sorted padded rows x packed e2m1 expert weights read as stored (no conversion pass)."""
    gen = torch.Generator(device=DEV).manual_seed(9)
    El, N, K = 3, 512, 1024
    tiles = torch.tensor([2, 0, 0, 1], dtype=torch.int32, device=DEV)        # expert of each 128-row tile
    ntile = torch.tensor([4], dtype=torch.int32, device=DEV)
    cap = 6 * 128                                                            # two tiles beyond num_m_tiles stay untouched
    x = torch.randn(cap, K, device=DEV, generator=gen)
    aq = torch.zeros(cap, K, dtype=torch.uint8, device=DEV)
    sfa = mx.empty_units(cap, K, 128, DEV)
    mx.quant_rows(x, cap, K, aq, sfa)
    a_deq = (aq.view(F8).float().view(cap, K // 32, 32) * torch.exp2(mx.units_to_rowmajor(sfa, cap).float() - 127)[:, :, None])
    pk = torch.randint(0, 256, (El, N, K // 2), device=DEV, dtype=torch.uint8, generator=gen)
    sc = torch.randint(118, 126, (El, N, K // 32), device=DEV, dtype=torch.uint8, generator=gen)
    w = E.dequant_mxfp4(pk, sc)                                              # [El, N, K]
    sfb = mx.units_from_rowmajor(sc, K)
    c = torch.full((cap, N), 5.0, device=DEV, dtype=torch.bfloat16)
    st = native.StatusWord(DEV)
    mx.gemm(aq, sfa, pk, sfb, c, cap, N, K, st.t, b_fp4=True, b_rows=El * N, tile_expert=tiles, num_m_tiles=ntile)
    torch.cuda.synchronize()
    st.check()
    for i, e in enumerate(tiles.tolist()):
        rows = slice(i * 128, (i + 1) * 128)
        assert _rel(c[rows], a_deq.view(cap, K)[rows].double() @ w[e].double().t()) < 4e-3
    assert bool((c[4 * 128:] == 5.0).all())


def test_gemm_mx_refuses_bad_arguments():
    st = native.StatusWord(DEV)
    a = torch.zeros(128, 128, dtype=torch.uint8, device=DEV)
    sf = mx.empty_units(128, 128, 128, DEV)
    sfb = mx.empty_units(256, 128, 256, DEV)
    c = torch.zeros(128, 256, device=DEV)
    with pytest.raises(native.NativeError):
        native.call("tf_gemm_mx", a, 128, a, 128, 256, 0, sf, sf.shape[1], sfb, sfb.shape[1], c, 256, 0, 128, 256, 96, None,
                    None, st.t)                                            # K not a multiple of 128
    with pytest.raises(native.NativeError):
        native.call("tf_gemm_mx", a, 128, a, 128, 256, 0, sf, 1, sfb, sfb.shape[1], c, 256, 0, 128, 256, 128, None, None,
                    st.t)                                                  # too few scale units for the rows
