"""Expert-parallel MoE kernels on one GPU (world = 1: every peer pointer is the rank's own workspace)
against an fp32 reference on the dequantised weights."""
import pytest
import torch

from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(x, ids, wts, w1, w3, w2, limit):
    out = torch.zeros(x.shape[0], x.shape[1], device=x.device)
    for t in range(x.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            gate = (w1[e] @ x[t]).clamp(max=limit)
            up = (w3[e] @ x[t]).clamp(-limit, limit)
            out[t] += wts[t, j] * (w2[e] @ (torch.nn.functional.silu(gate) * up))
    return out


@pytest.mark.parametrize("Tl", [1, 37, 200])
def test_ep_moe_single_rank_matches_reference(Tl):
    from titanic_flash_41_b200.parallel.ep import EpMoE
    torch.manual_seed(0)
    d, I, Eg, k = 512, 256, 8, 2
    w1 = torch.randn(Eg, I, d, device=DEV) * 0.06
    w3 = torch.randn(Eg, I, d, device=DEV) * 0.06
    w2 = torch.randn(Eg, d, I, device=DEV) * 0.06
    q1, q3, q2 = (E.quant_mxfp4_device(w) for w in (w1, w3, w2))
    moe = EpMoE(d, I, Eg, k, 256, q1[0], q1[1], q3[0], q3[1], q2[0], q2[1], device=DEV)
    st = native.StatusWord(DEV)
    g = torch.Generator(device=DEV).manual_seed(1)
    for call in range(2):                                       # flags carry the epoch: nothing to clear
        x = torch.randn(Tl, d, device=DEV, generator=g).bfloat16()
        ids = torch.stack([torch.randperm(Eg, device=DEV, generator=g)[:k] for _ in range(Tl)]).int().contiguous()
        wts = torch.rand(Tl, k, device=DEV, generator=g).contiguous()
        out = torch.zeros(Tl, d, device=DEV, dtype=torch.bfloat16)
        moe.forward(x, ids, wts, out, st.t)
        torch.cuda.synchronize()
        st.check()
        want = _ref(x.float(), ids, wts, *(E.dequant_mxfp4(*q) for q in (q1, q3, q2)), 10.0)
        rel = float((out.float() - want).norm() / want.norm())
        assert rel < 0.06, (call, rel)


def test_ep_wait_times_out_cleanly():
    """A receive whose sources never published (epoch ahead of every flag) must report TF_TIMEOUT
    through the status word and leave the context usable."""
    from titanic_flash_41_b200.parallel.ep import EpMoE
    d, I, Eg, k = 512, 256, 8, 2
    z = lambda *s: torch.zeros(*s, dtype=torch.uint8, device=DEV)
    moe = EpMoE(d, I, Eg, k, 16, z(Eg, I, d // 2), z(Eg, I, d // 32), z(Eg, I, d // 2), z(Eg, I, d // 32),
                z(Eg, d, I // 2), z(Eg, d, I // 32), device=DEV, spin_limit=2000)
    st = native.StatusWord(DEV)
    native.call("tf_ep_recv_ids", moe.peers, 1, 0, moe.cap, d, k, moe.El, 16, 7, moe.ids_recv, 2000, st.t)
    torch.cuda.synchronize()
    with pytest.raises(native.NativeError, match="timeout"):
        st.check()
    assert int((moe.ids_recv >= 0).sum()) == 0
    assert torch.ones(4, device=DEV).sum().item() == 4.0        # the context still works
