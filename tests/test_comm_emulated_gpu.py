"""The one-shot all-reduce protocol (csrc/comm.cuh) with several ranks emulated on ONE GPU by a
single cooperative launch: push of {payload, epoch} words, bounded polling, rank-ordered fp32 sum,
residual update and the fused boundary (RMSNorm + f16 / bf16 / MXFP8 rows), against PyTorch fp32
references and against the single-GPU boundary kernel."""
import pytest
import torch

from titanic_flash_41_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _emu(world, N, max_rows=32):
    from titanic_flash_41_b200.parallel.symm import EmulatedRanks
    return EmulatedRanks(world, N, max_rows, device=DEV)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_plain_sum_is_exact_and_identical_on_every_rank(world):
    """fp32 transport: the result is the rank-ordered fp32 sum, bit for bit, on every emulated rank,
    over many epochs back to back (both parities, rows changing between calls)."""
    N = 1024                                    # 32 column tiles: one row owner per row up to 32 rows
    emu = _emu(world, N)
    st = native.StatusWord(DEV)
    for it, rows in enumerate([1, 5, 16, 32, 7, 7, 7, 32, 3]):
        g = torch.Generator(device=DEV).manual_seed(100 * it + world)
        part = torch.randn(world, 32, N, device=DEV, generator=g)
        out = torch.full((world, 32, N), -7.0, device=DEV)
        emu.allreduce(part, rows, st.t, out=out)
        torch.cuda.synchronize()
        st.check()
        ref = torch.zeros(rows, N, device=DEV)
        for r in range(world):
            ref = ref + part[r, :rows]
        for r in range(world):
            assert torch.equal(out[r, :rows], ref), (it, r)
            assert (out[r, rows:] == -7.0).all()           # rows beyond the live count are untouched


@pytest.mark.parametrize("world,N", [(2, 512), (8, 512), (2, 4096)])
def test_residual_update_and_fused_boundary(world, N):
    """bf16 transport + residual + boundary: the residual equals bf16(x + sum of the bf16-rounded
    partials in rank order); the normalised rows equal what the boundary kernel of the single-GPU
    path (tf_add_norm_fused) makes of the same residual and sum."""
    torch.manual_seed(world * 7 + N)
    rows, RA = 11, 16
    emu = _emu(world, N)
    st = native.StatusWord(DEV)
    w = (1 + 0.1 * torch.randn(N, device=DEV)).bfloat16()
    x0 = torch.randn(RA, N, device=DEV).bfloat16()
    for it in range(3):
        part = torch.randn(world, RA, N, device=DEV) * (0.5 + it)
        resid = x0[None].repeat(world, 1, 1).contiguous()
        h16 = torch.zeros(world, RA, N, device=DEV, dtype=torch.float16)
        hb = torch.zeros(world, RA, N, device=DEV, dtype=torch.bfloat16)
        x8 = torch.zeros(world, RA, N, device=DEV, dtype=torch.uint8)
        x8s = torch.zeros(world, RA, N // 32, device=DEV, dtype=torch.uint8)
        emu.allreduce(part, rows, st.t, resid=resid, norm=dict(w=w, h16=h16, hb=hb, x8=x8, x8s=x8s, eps=1e-6))
        torch.cuda.synchronize()
        st.check()
        delta = torch.zeros(rows, N, device=DEV)
        for r in range(world):
            delta = delta + part[r, :rows].bfloat16().float()
        # the single-GPU boundary kernel on the same residual and sum
        xa = x0[:rows].clone()
        h16a = torch.zeros(rows, N, device=DEV, dtype=torch.float16)
        hba = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16)
        qa = torch.zeros(rows, N, device=DEV, dtype=torch.uint8)
        sa = torch.zeros(rows, N // 32, device=DEV, dtype=torch.uint8)
        native.call("tf_add_norm_fused", xa, delta, None, None, None, None, 0, 0, 0, w, h16a, hba, qa, sa, rows, N, 1e-6)
        torch.cuda.synchronize()
        assert torch.equal(xa, (x0[:rows].float() + delta).bfloat16())
        deq = lambda q, s_: (q.view(torch.float8_e4m3fn).float().view(rows, N // 32, 32)
                             * torch.exp2(s_.float() - 127)[..., None])
        for r in range(world):
            assert torch.equal(resid[r, :rows], xa), (it, r)
            assert torch.equal(resid[r, rows:], x0[rows:])
            for a, b_ in ((h16a, h16[r, :rows]), (hba, hb[r, :rows])):
                assert (a.float() - b_.float()).abs().max() <= 0.01 * a.float().abs().max()
                assert (a == b_).float().mean() > 0.98
            assert (deq(qa, sa) - deq(x8[r, :rows], x8s[r, :rows])).abs().max() <= 0.07 * h16a.float().abs().max()
            # every emulated rank holds bit-identical rows
            assert torch.equal(h16[r], h16[0]) and torch.equal(x8[r], x8[0]) and torch.equal(x8s[r], x8s[0])
        x0 = torch.cat([xa, x0[rows:]])


def test_bad_arguments_are_refused_on_the_host():
    emu = _emu(2, 512)
    st = native.StatusWord(DEV)
    part = torch.zeros(2, 32, 512, device=DEV)
    out = torch.zeros(2, 32, 512, device=DEV)
    with pytest.raises(native.NativeError):
        emu.allreduce(part, 33, st.t, out=out)              # more rows than the workspace holds
    with pytest.raises(native.NativeError):
        emu.allreduce(part, 4, st.t)                        # neither a residual nor an output
    with pytest.raises(native.NativeError):
        native.call("tf_wait_probe", None, 1, 10, st.t)


def test_wait_that_nothing_satisfies_reports_timeout():
    """Failure detection on the device without a fault: a bounded wait on a flag that nothing sets
    returns TF_TIMEOUT through the status word and the context stays usable."""
    st = native.StatusWord(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    native.call("tf_wait_probe", flag, 1, 2000, st.t)
    torch.cuda.synchronize()
    code, kern, _, spins = st.read()
    assert (code, kern) == (2, 201) and spins > 2000
    with pytest.raises(native.NativeError):
        st.check()
    assert st.read()[0] == 0
    assert float(torch.ones(4, device=DEV).sum()) == 4.0       # the context still works
