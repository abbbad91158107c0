"""Rank-local (chunked) sampling and block verification, csrc/sample_chunks.cu: row statistics against
the full-row kernels, identical results for 1, 2, 4 and 8 (emulated) ranks, preservation of the
target law, nucleus truncation, and per-conversation settings inside one launch."""
import pytest
import torch

from titanic_flash_41_b200.ops import native
from titanic_flash_41_b200.parallel.symm import SampleWorkspace

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _split(full, world):
    """[rows, V] -> [world, rows, V / world]: rank r holds columns [r * Vl, (r + 1) * Vl)."""
    rows, V = full.shape
    return full.view(rows, world, V // world).transpose(0, 1).contiguous()


class Flow:
    """Draft draws (g launches with g = 0) followed by one verification launch, on `world` ranks
    (1 = a plain launch; > 1 = ranks emulated on this GPU)."""

    def __init__(self, V, S, g, world):
        self.V, self.S, self.g, self.world = V, S, g, world
        self.R = g + 1
        self.ws = SampleWorkspace(V, S * self.R, DEV, emulate=world if world > 1 else 1)
        self.sb = native.lib().tf_rowstat_bytes()
        self.st = native.StatusWord(DEV)

    def run(self, tl, dl, u_draft, u_ver, temp, topp, point_props=None, sess_g=None):
        """tl [S, g+1, V], dl [S, g, V] full rows.  Returns (props, dstat, tstat, n_accept, token) of
        rank 0 after checking that every rank produced the same."""
        S, g, R, V, W, sb = self.S, self.g, self.R, self.V, self.world, self.sb
        Vl = V // W
        gs = max(g, 1)
        i32 = dict(dtype=torch.int32, device=DEV)
        props = torch.zeros(W, S, gs, **i32)
        dstat = torch.zeros(W, S, gs, sb, dtype=torch.uint8, device=DEV)
        tstat = torch.zeros(W, S * R, sb, dtype=torch.uint8, device=DEV)
        nacc, tok = torch.zeros(W, S, **i32), torch.zeros(W, S, **i32)
        tls = _split(tl.reshape(S * R, V), W)                      # [W, S*R, Vl]
        point = point_props is not None
        dls = None
        if g > 0 and not point:
            dls = _split(dl.reshape(S * g, V), W).view(W, S, g, Vl)
            for j in range(g):
                lg = dls[:, :, j].contiguous()                     # [W, S, Vl]
                self.ws.sample(lg, None, None, None, u_draft[:, j:], gs, temp, topp, S, 0, Vl,
                               dstat[:, :, j], gs, None, props[:, :, j:], gs, self.st.t,
                               emu_strides=(S * Vl, 0, S * gs, S * gs, 0))
            torch.cuda.synchronize()
            for r in range(W):
                assert torch.equal(props[r], props[0]) and torch.equal(dstat[r], dstat[0])
        elif point:
            props[:] = point_props[None]
        self.ws.sample(tls, dls, dstat[0] if (g > 0 and not point) else None, props[0] if g > 0 else None, u_ver, g + 2,
                       temp, topp, S, g, Vl, tstat, 1, nacc, tok, 1, self.st.t, point_mass=point,
                       emu_strides=(S * R * Vl, S * g * Vl, S * R, S, S), sess_g=sess_g)
        torch.cuda.synchronize()
        self.st.check()
        for r in range(W):
            assert torch.equal(tstat[r], tstat[0]) and torch.equal(nacc[r], nacc[0]) and torch.equal(tok[r], tok[0])
        return props[0].clone(), dstat[0].clone(), tstat[0].clone(), nacc[0].clone(), tok[0].clone()


def _inputs(S, g, V, seed, scale=3.0):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    tl = torch.randn(S, g + 1, V, device=DEV, generator=gen) * scale
    dl = tl[:, :max(g, 1)] + 0.7 * torch.randn(S, max(g, 1), V, device=DEV, generator=gen)
    u_d = torch.rand(S, max(g, 1), dtype=torch.float64, device=DEV, generator=gen)
    u_v = torch.rand(S, g + 2, dtype=torch.float64, device=DEV, generator=gen)
    return tl, dl[:, :g].contiguous() if g else dl[:, :0], u_d, u_v


@pytest.mark.parametrize("V,rows", [(4096, 9), (129280, 5)])
def test_row_statistics_equal_the_full_row_kernels(V, rows):
    """max, nucleus threshold key and normaliser: bit-identical to tf_rowstats (integer mass sums do
    not depend on how the vocabulary is cut)."""
    torch.manual_seed(3)
    st = native.StatusWord(DEV)
    sb = native.lib().tf_rowstat_bytes()
    for temp, top_p in ((0.6, 0.95), (1.3, 1.0), (0.8, 0.3)):
        lg = (torch.randn(rows, V, device=DEV) * 3).contiguous()
        want = torch.zeros(rows, sb, dtype=torch.uint8, device=DEV)
        scr = torch.zeros(native.lib().tf_rowstats_scratch_bytes(rows), dtype=torch.uint8, device=DEV)
        native.call("tf_rowstats", lg, V, V, rows, temp, top_p, want, scr, st.t)
        f = Flow(V, rows, 0, 1)
        t = torch.full((rows,), temp, device=DEV)
        p = torch.full((rows,), top_p, device=DEV)
        u = torch.rand(rows, 2, dtype=torch.float64, device=DEV)
        _, _, got, _, tok = f.run(lg.view(rows, 1, V), None, None, u, t, p)
        assert torch.equal(got, want)
        assert ((tok >= 0) & (tok < V)).all()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("V", [4096, 129280])
def test_emulated_ranks_commit_what_one_rank_commits(world, V):
    S, g = (4, 3) if V == 4096 else (2, 3)
    temp = torch.tensor([0.6, 1.0, 0.6, 1e-3][:S], device=DEV)
    topp = torch.tensor([0.95, 1.0, 0.5, 1.0][:S], device=DEV)
    one, many = Flow(V, S, g, 1), Flow(V, S, g, world)
    for it in range(4):                                      # consecutive calls: both buffer parities
        tl, dl, u_d, u_v = _inputs(S, g, V, 50 + it)
        a = one.run(tl, dl, u_d, u_v, temp, topp)
        b = many.run(tl, dl, u_d, u_v, temp, topp)
        for x, y in zip(a, b):
            assert torch.equal(x, y), it


def test_block_verification_preserves_the_target_law():
    """The first committed token (accepted proposal or the resampled one) follows the target law,
    whatever the draft law (Sun et al., arXiv:2403.10444)."""
    V, S, g, T = 1024, 4, 2, 1.0
    gen = torch.Generator(device=DEV).manual_seed(5)
    base_t = torch.randn(g + 1, V, device=DEV, generator=gen) * 2.5
    base_d = base_t[:g] + 1.0 * torch.randn(g, V, device=DEV, generator=gen)
    tl, dl = base_t[None].repeat(S, 1, 1).contiguous(), base_d[None].repeat(S, 1, 1).contiguous()
    temp, topp = torch.full((S,), T, device=DEV), torch.ones(S, device=DEV)
    f = Flow(V, S, g, 1)
    first, accepted = [], 0
    n_calls = 1500
    for it in range(n_calls):
        u_d = torch.rand(S, g, dtype=torch.float64, device=DEV, generator=gen)
        u_v = torch.rand(S, g + 2, dtype=torch.float64, device=DEV, generator=gen)
        props, _, _, nacc, tok = f.run(tl, dl, u_d, u_v, temp, topp)
        first.append(torch.where(nacc > 0, props[:, 0], tok))
        accepted += int((nacc > 0).sum())
    first = torch.cat(first).long().cpu()
    emp = torch.bincount(first, minlength=V).double() / first.numel()
    p0 = torch.softmax(base_t[0].double().cpu(), -1)
    assert float((emp - p0).abs().max()) < 0.012
    assert 0.2 < accepted / (n_calls * S) < 1.0


def test_nucleus_and_per_conversation_settings():
    """Conversation 0 is greedy (temperature -> 0), 1 samples at T = 1 from the 50 % nucleus, 2 from
    the full law, all in ONE launch; the draws of 1 never leave its nucleus."""
    V, S = 1024, 3
    gen = torch.Generator(device=DEV).manual_seed(9)
    lg = (torch.randn(S, 1, V, device=DEV, generator=gen) * 2.0).contiguous()
    temp = torch.tensor([1e-3, 1.0, 1.0], device=DEV)
    topp = torch.tensor([1.0, 0.5, 1.0], device=DEV)
    f = Flow(V, S, 0, 1)
    p = torch.softmax(lg[:, 0].double(), -1)
    srt, idx = p[1].sort(descending=True)
    k = int((srt.cumsum(0) < 0.5).sum()) + 1
    nucleus = set(idx[:k].tolist())
    seen1, seen2 = set(), set()
    for it in range(300):
        u = torch.rand(S, 2, dtype=torch.float64, device=DEV, generator=gen)
        _, _, _, _, tok = f.run(lg, None, None, u, temp, topp)
        t = tok.tolist()
        assert t[0] == int(lg[0, 0].argmax())
        assert t[1] in nucleus
        seen1.add(t[1])
        seen2.add(t[2])
    assert len(seen1) > 1 and len(seen2) > len(seen1)


def test_point_mass_proposals_and_bad_arguments():
    """Copy proposals (a point-mass draft law) verify through the same launch; malformed calls are
    refused on the host."""
    V, S, g = 1024, 2, 2
    tl, _, _, u_v = _inputs(S, g, V, 77)
    props = torch.stack([tl[s, :g].argmax(-1) for s in range(S)]).int()       # the target's own favourites
    temp, topp = torch.full((S,), 1e-3, device=DEV), torch.ones(S, device=DEV)
    f = Flow(V, S, g, 1)
    _, _, _, nacc, tok = f.run(tl, None, None, u_v, temp, topp, point_props=props)
    assert nacc.tolist() == [g, g]                      # a greedy target accepts its own argmax every time
    assert tok.tolist() == [int(tl[s, g].argmax()) for s in range(S)]
    ws = f.ws
    z = torch.zeros(S, dtype=torch.int32, device=DEV)
    stat = torch.zeros(S * (g + 1), f.sb, dtype=torch.uint8, device=DEV)
    with pytest.raises(native.NativeError):            # rows beyond the workspace
        ws.sample(tl, None, None, props, u_v, g + 2, temp, topp, S + 1, g, V, stat, 1, z, z, 1, f.st.t, point_mass=True)
    with pytest.raises(native.NativeError):            # proposals without draft rows or the point-mass flag
        ws.sample(tl, None, None, props, u_v, g + 2, temp, topp, S, g, V, stat, 1, z, z, 1, f.st.t)
    with pytest.raises(native.NativeError):            # no logits
        ws.sample(None, None, None, None, u_v, g + 2, temp, topp, S, 0, V, stat, 1, z, z, 1, f.st.t)
    assert native.lib().tf_sample_chunks_count(1000) == 0      # 1000 / 8 = 125 is not a multiple of 4
    with pytest.raises(ValueError):
        SampleWorkspace(1000, 4, DEV)


@pytest.mark.parametrize("world", [1, 2])
def test_per_conversation_block_lengths_equal_shorter_blocks(world):
    """Causal stopping: a conversation that verifies only its first k proposals commits exactly what a
    block of k proposals commits (row k is its bonus row, later rows are ignored), inside one launch
    with conversations of other lengths."""
    V, S, g = 4096, 4, 3
    tl, dl, u_d, u_v = _inputs(S, g, V, seed=11)
    temp = torch.full((S,), 0.8, device=DEV)
    topp = torch.full((S,), 0.95, device=DEV)
    lens = torch.tensor([1, 2, 3, 2], dtype=torch.int32, device=DEV)
    props, _, _, nacc, tok = Flow(V, S, g, world).run(tl, dl, u_d, u_v, temp, topp, sess_g=lens)
    full = Flow(V, S, g, world).run(tl, dl, u_d, u_v, temp, topp)
    assert bool((nacc <= lens).all())
    differs = False
    for s in range(S):
        k = int(lens[s])
        uv = torch.cat([u_v[s:s + 1, :k], u_v[s:s + 1, g:g + 1], u_v[s:s + 1, g + 1:g + 2]], 1).contiguous()
        p1, _, _, n1, t1 = Flow(V, 1, k, world).run(tl[s:s + 1, :k + 1].contiguous(), dl[s:s + 1, :k].contiguous(),
                                                      u_d[s:s + 1].contiguous(), uv, temp[s:s + 1], topp[s:s + 1])
        assert torch.equal(p1[0, :k], props[s, :k])
        assert int(n1[0]) == int(nacc[s]) and int(t1[0]) == int(tok[s]), (s, k)
        differs |= k < g and (int(full[3][s]) != int(nacc[s]) or int(full[4][s]) != int(tok[s]))
    assert differs            # the shorter blocks are not what the full blocks would have committed
