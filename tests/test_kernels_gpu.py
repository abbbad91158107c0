"""Numerics of the CUDA kernels against plain PyTorch fp32 references (one B200)."""
import math

import numpy as np
import pytest
import torch

from titanic_flash_41_b200.formats import codecs
from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("M", [1, 5, 8, 16, 27, 32])
def test_smallm_fp8_dense(M):
    torch.manual_seed(M)
    N, K = 384, 1024
    w = torch.randn(N, K, device=DEV) * 0.05
    fw = E.quant_fp8_device(w)
    x = torch.randn(M, K, device=DEV).half()
    out = torch.zeros(M, N, device=DEV)
    native.call("tf_smallm_gemm", 0, fw.q, None, fw.s, None, 0, 0, K, K // 128, x, K, out, N, 0, N, K, M,
                None, None, None, None, None, 1, 0, M, 0.0)
    ref = x.float() @ E.dequant_fp8(fw).t()
    assert _rel(out, ref) < 2e-3


@pytest.mark.parametrize("M,N,K", [(16, 256, 2048), (9, 384, 4096), (16, 128, 2176)])
def test_smallm_fp8_dense_eight_way_k_split(M, N, K):
    """Dense matrices with few 32-feature tiles and long rows split K over eight warps per CTA
    (K not a multiple of 8 x 128 leaves the last warps short or idle); results are run-to-run identical."""
    torch.manual_seed(K + M)
    fw = E.quant_fp8_device(torch.randn(N, K, device=DEV) * 0.05)
    x = torch.randn(M, K, device=DEV).half()
    outs = []
    for _ in range(2):
        out = torch.zeros(M, N, device=DEV)
        native.call("tf_smallm_gemm", 0, fw.q, None, fw.s, None, 0, 0, K, K // 128, x, K, out, N, 0, N, K, M,
                    None, None, None, None, None, 1, 0, M, 0.0)
        outs.append(out)
    ref = x.float() @ E.dequant_fp8(fw).t()
    assert _rel(outs[0], ref) < 2e-3
    assert torch.equal(outs[0], outs[1])


def test_smallm_fp8_dual_swiglu_and_kslice():
    torch.manual_seed(0)
    N, K, M = 256, 512, 7
    w1, w3 = (E.quant_fp8_device(torch.randn(N, K, device=DEV) * 0.1) for _ in range(2))
    x = torch.randn(M, K, device=DEV).half()
    out = torch.zeros(M, N, device=DEV, dtype=torch.float16)
    native.call("tf_smallm_gemm", 0, w1.q, w3.q, w1.s, w3.s, 0, 0, K, K // 128, x, K, out, N, 1, N, K, M,
                None, None, None, None, None, 1, 0, M, 10.0)
    g = torch.clamp(x.float() @ E.dequant_fp8(w1).t(), max=10.0)
    u = torch.clamp(x.float() @ E.dequant_fp8(w3).t(), -10.0, 10.0)
    assert _rel(out, g * torch.sigmoid(g) * u) < 3e-3


def test_smallm_bf16_head():
    torch.manual_seed(1)
    N, K, M = 2048, 512, 9
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    x = torch.randn(M, K, device=DEV).bfloat16()
    out = torch.zeros(M, N, device=DEV)
    native.call("tf_smallm_gemm", 2, w, None, None, None, 0, 0, K * 2, 0, x, K, out, N, 0, N, K, M,
                None, None, None, None, None, 1, 0, M, 0.0)
    assert _rel(out, x.float() @ w.float().t()) < 1e-3


def _group_tables(ids, e_lo, e_hi):
    T, k = ids.shape
    i32 = dict(dtype=torch.int32, device=DEV)
    El = e_hi - e_lo
    t = dict(ge=torch.zeros(El, **i32), gs=torch.zeros(El, **i32), gc=torch.zeros(El, **i32),
             ng=torch.zeros(1, **i32), sp=torch.zeros(T * k, **i32), nl=torch.zeros(1, **i32))
    native.call("tf_route_group", ids, T * k, e_lo, e_hi, t["ge"], t["gs"], t["gc"], t["ng"], t["sp"], t["nl"])
    return t


def test_grouped_mxfp4_experts():
    torch.manual_seed(2)
    El, I, d, T, k = 6, 256, 512, 11, 2
    w1, w3 = torch.randn(El, I, d, device=DEV) * 0.05, torch.randn(El, I, d, device=DEV) * 0.05
    w2 = torch.randn(El, d, I, device=DEV) * 0.05
    (p1, s1), (p3, s3), (p2, s2) = (E.quant_mxfp4_device(w) for w in (w1, w3, w2))
    ids = torch.stack([torch.randperm(8, device=DEV)[:k] for _ in range(T)]).int()   # experts 0..7, local 1..6
    e_lo, e_hi = 1, 7
    t = _group_tables(ids, e_lo, e_hi)
    h = torch.randn(T, d, device=DEV).half()
    act = torch.zeros(T * k, I, device=DEV, dtype=torch.float16)
    y = torch.zeros(T * k, d, device=DEV)
    native.call("tf_smallm_gemm", 1, p1, p3, s1, s3, I * d // 2, I * d // 32, d // 2, d // 32, h, d, act, I,
                1, I, d, 0, t["ge"], t["gs"], t["gc"], t["ng"], t["sp"], k, El, 16, 10.0)
    native.call("tf_smallm_gemm", 1, p2, None, s2, None, d * I // 2, d * I // 32, I // 2, I // 32, act, I, y, d,
                0, d, I, 0, t["ge"], t["gs"], t["gc"], t["ng"], t["sp"], 1, El, 16, 0.0)
    d1, d3, d2 = E.dequant_mxfp4(p1, s1), E.dequant_mxfp4(p3, s3), E.dequant_mxfp4(p2, s2)
    for r in range(T):
        for j in range(k):
            e = int(ids[r, j]) - e_lo
            if not 0 <= e < El:
                continue
            g = torch.clamp(h[r].float() @ d1[e].t(), max=10.0)
            u = torch.clamp(h[r].float() @ d3[e].t(), -10.0, 10.0)
            a = (g * torch.sigmoid(g) * u)
            assert _rel(act[r * k + j], a) < 5e-3
            assert _rel(y[r * k + j], act[r * k + j].float() @ d2[e].t()) < 5e-3


def test_add_norm_and_fp8_quant():
    torch.manual_seed(3)
    T, d = 5, 512
    x = torch.randn(T, d, device=DEV).bfloat16()
    delta = torch.randn(T, d, device=DEV)
    w = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    x0 = x.clone()
    h16 = torch.zeros(T, d, device=DEV, dtype=torch.float16)
    q8 = torch.zeros(T, d, device=DEV, dtype=torch.uint8)
    qs = torch.zeros(T, d // 128, device=DEV)
    native.call("tf_add_norm", x, delta, 0, d, w, h16, None, q8, qs, T, d, 1e-6)
    xr = (x0.float() + delta).bfloat16().float()
    assert torch.equal(x.float(), xr)
    ref = (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
    assert _rel(h16, ref) < 5e-3
    deq = q8.view(torch.float8_e4m3fn).float().view(T, d // 128, 128) * qs[:, :, None]
    assert _rel(deq.view(T, d), ref) < 4e-2


def test_router_matches_oracle():
    from titanic_flash_41_b200.config import tiny_config
    from titanic_flash_41_b200.models.oracle import route
    torch.manual_seed(4)
    T, Ex, d, k = 13, 64, 512, 6
    cfg = tiny_config(n_experts=Ex, topk=k, scoring="sqrtsoftplus", router_bias=True, route_scale=1.5)
    h = torch.randn(T, d, device=DEV).half()
    gate = (torch.randn(Ex, d, device=DEV) / math.sqrt(d)).bfloat16()
    bias = torch.randn(Ex, device=DEV) * 0.1
    logits = torch.zeros(T, Ex, device=DEV)
    ids = torch.zeros(T, k, device=DEV, dtype=torch.int32)
    wts = torch.zeros(T, k, device=DEV)
    native.call("tf_router", h, gate, bias, None, None, -1, logits, ids, wts, T, Ex, d, k, 1, 1, 1.5)
    ref_logits = h.float() @ gate.float().t()
    assert _rel(logits, ref_logits) < 1e-4
    rid, rw = route(logits.cpu(), cfg, bias.cpu())
    assert torch.equal(ids.cpu().long(), rid)
    assert torch.allclose(wts.cpu(), rw, atol=1e-5)


@pytest.mark.parametrize("Hi", [4, 8, 16, 32])
def test_index_scores_and_topk(Hi):
    torch.manual_seed(5)
    T, Di, C, k = 8, 128, 700, 64
    keys_f = torch.randn(2, C, Di)
    krow = Di // 2 + Di // 32
    enc = codecs.index_key_encode(keys_f)                          # [2, C, 68]
    kd = codecs.index_key_decode(enc, Di)
    keys = enc.to(DEV).contiguous()
    q = torch.randn(T, Hi, Di, device=DEV).bfloat16()
    w = torch.rand(T, Hi, device=DEV)
    region = torch.tensor([0] * 4 + [1] * 4, dtype=torch.int32, device=DEV)
    nvalid = torch.tensor([700, 650, 3, 0, 129, 128, 127, 64], dtype=torch.int32, device=DEV)
    scores = torch.full((T, 1024), 7.0, device=DEV)
    native.call("tf_index_scores", q, w, region, nvalid, keys, C * krow, krow, T, Hi, Di, 4, scores, 1024, 0, 700)
    ref = torch.einsum("thd,tcd->thc", q.float().cpu(), kd[region.cpu().long()]).relu()
    ref = (ref * w.cpu()[:, :, None]).sum(1)
    for r in range(T):
        n = int(nvalid[r])
        assert torch.allclose(scores[r, :n].cpu(), ref[r, :n], atol=2e-2, rtol=2e-3)
    sel = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(T, dtype=torch.int32, device=DEV)
    # duplicate values to exercise ties
    scores[0, 10:20] = scores[0, 5].item()
    native.call("tf_topk_select", scores, 1024, nvalid, k, sel, cnt, None, 0, T)
    for r in range(T):
        n = int(nvalid[r])
        s = scores[r, :n].cpu()
        got = sel[r].cpu().tolist()
        if n <= k:
            assert got == list(range(n)) + [-1] * (k - n) and int(cnt[r]) == n
            continue
        order = torch.sort(s, descending=True, stable=True).indices[:k]
        assert got == sorted(order.tolist())


@pytest.mark.parametrize("Dh,Hl", [(128, 4), (512, 4), (512, 20), (256, 16)])
def test_sparse_attention_matches_reference(Dh, Hl):
    """Dh 128 runs the register-resident kernel, 256 / 512 the wide-latent one (head dim split over warps)."""
    torch.manual_seed(6)
    T, window, ring, C, k = 6, 16, 64, 50, 12
    win_row, comp_row = -(-(Dh + Dh // 32) // 16) * 16, -(-(Dh // 2 + Dh // 16) // 16) * 16
    kv = torch.randn(2, ring, Dh) * 1.5
    win = torch.zeros(2, ring, win_row, dtype=torch.uint8)
    win[:, :, :Dh + Dh // 32] = codecs.kv_v41_encode(kv)
    kvd = codecs.kv_v41_decode(win, Dh)
    ck = torch.randn(2, C, Dh)
    comp = torch.zeros(2, C, comp_row, dtype=torch.uint8)
    comp[:, :, :Dh // 2 + Dh // 16] = codecs.kv_v41fp4_encode(ck)
    ckd = codecs.kv_v41fp4_decode(comp, Dh)
    pos = torch.tensor([3, 20, 70, 100, 5, 64], dtype=torch.int32)
    region = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    sel = torch.full((T, k), -1, dtype=torch.int32)
    for r in range(T):
        n = [0, 3, 12, 12, 1, 7][r]
        sel[r, :n] = torch.sort(torch.randperm(C)[:n]).values.int()
    q = (torch.randn(T, Hl, Dh) * 0.5).bfloat16()
    sink = torch.randn(Hl) * 0.5
    freqs = torch.tensor([10000.0 ** (-2.0 * j / 64) for j in range(32)])
    nsplit = 3
    dev = lambda t: t.to(DEV).contiguous()
    part_o = torch.zeros(T, nsplit, Hl, Dh, device=DEV)
    part_lse = torch.zeros(T, nsplit, Hl, device=DEV)
    out = torch.zeros(T, Hl * Dh, device=DEV, dtype=torch.float16)
    st = native.StatusWord(DEV)
    native.call("tf_sparse_attention", dev(q), T, Hl, Dh, dev(pos), dev(region), None, dev(win), ring * win_row,
                win_row, ring, window, dev(comp), C * comp_row, comp_row, dev(sel), k, None, C,
                1 / math.sqrt(Dh), nsplit, part_o, part_lse, dev(sink), dev(freqs), 64, out, None, Hl * Dh, st.t)
    st.check()
    from titanic_flash_41_b200.models.oracle import apply_rope
    for r in range(T):
        p, rg = int(pos[r]), int(region[r])
        nw = min(p + 1, window)
        ks = [kvd[rg, (p - nw + 1 + i) % ring] for i in range(nw)]
        ks += [ckd[rg, int(c)] for c in sel[r] if c >= 0]
        Kmat = torch.stack(ks)
        lg = q[r].float() @ Kmat.t() / math.sqrt(Dh)
        lg = torch.cat([lg, sink[:, None]], 1)
        P = torch.softmax(lg, -1)[:, :-1]
        o = apply_rope((P @ Kmat)[None], torch.tensor([p]), freqs, inverse=True)[0]
        assert _rel(out[r].cpu().view(Hl, Dh), o) < 1e-2, r


@pytest.mark.parametrize("Hl", [64, 20])
def test_sparse_attention_of_prefill_rows_on_tcgen05_matches_reference(Hl):
    """64 rows or more of one split (head dim 128) run on the tcgen05 kernel (heads as M, 128-key
    chunks, S / O in tensor memory): same result as the fp32 reference and as the mma.sync kernel,
    for short rows (window only), rows with several chunks and a partly filled last chunk."""
    torch.manual_seed(8 + Hl)
    T, Dh, window, ring, C, k = 200, 128, 128, 512, 700, 320
    win_row, comp_row = -(-(Dh + Dh // 32) // 16) * 16, -(-(Dh // 2 + Dh // 16) // 16) * 16
    kv = torch.randn(2, ring, Dh) * 1.5
    win = torch.zeros(2, ring, win_row, dtype=torch.uint8)
    win[:, :, :Dh + Dh // 32] = codecs.kv_v41_encode(kv)
    kvd = codecs.kv_v41_decode(win, Dh)
    ck = torch.randn(2, C, Dh)
    comp = torch.zeros(2, C, comp_row, dtype=torch.uint8)
    comp[:, :, :Dh // 2 + Dh // 16] = codecs.kv_v41fp4_encode(ck)
    ckd = codecs.kv_v41fp4_decode(comp, Dh)
    pos = torch.cat([torch.arange(0, 100), torch.arange(300, 400)]).int()            # short windows, then full ones
    region = torch.cat([torch.zeros(100), torch.ones(100)]).int()
    sel = torch.full((T, k), -1, dtype=torch.int32)
    cnt = torch.zeros(T, dtype=torch.int32)
    for r in range(T):
        n = [0, 1, 37, 128, 129, 255, 320][r % 7]
        sel[r, :n] = torch.sort(torch.randperm(C)[:n]).values.int()
        cnt[r] = n
    q = (torch.randn(T, Hl, Dh) * 0.5).bfloat16()
    sink = torch.randn(Hl) * 0.5
    freqs = torch.tensor([10000.0 ** (-2.0 * j / 64) for j in range(32)])
    dev = lambda t: t.to(DEV).contiguous()
    st = native.StatusWord(DEV)
    outs = []
    for tc_on, counts in ((1, None), (1, dev(cnt)), (0, None)):
        native.lib().tf_sparse_attention_set_tc(tc_on)
        part_o = torch.zeros(T, 1, Hl, Dh, device=DEV)
        part_lse = torch.zeros(T, 1, Hl, device=DEV)
        out = torch.zeros(T, Hl * Dh, device=DEV, dtype=torch.float16)
        try:
            native.call("tf_sparse_attention", dev(q), T, Hl, Dh, dev(pos), dev(region), None, dev(win), ring * win_row,
                        win_row, ring, window, dev(comp), C * comp_row, comp_row, dev(sel), k, counts, C,
                        1 / math.sqrt(Dh), 1, part_o, part_lse, dev(sink), dev(freqs), 64, out, None, Hl * Dh, st.t)
            torch.cuda.synchronize()
        finally:
            native.lib().tf_sparse_attention_set_tc(1)
        st.check()
        outs.append(out.cpu().view(T, Hl, Dh).float())
    from titanic_flash_41_b200.models.oracle import apply_rope
    worst = 0.0
    for r in range(T):
        p, rg = int(pos[r]), int(region[r])
        nw = min(p + 1, window)
        ks = [kvd[rg, (p - nw + 1 + i) % ring] for i in range(nw)]
        ks += [ckd[rg, int(c)] for c in sel[r] if c >= 0]
        Kmat = torch.stack(ks)
        lg = q[r].float() @ Kmat.t() / math.sqrt(Dh)
        lg = torch.cat([lg, sink[:, None]], 1)
        P = torch.softmax(lg, -1)[:, :-1]
        o = apply_rope((P @ Kmat)[None], torch.tensor([p]), freqs, inverse=True)[0]
        for got in outs:
            worst = max(worst, _rel(got[r], o))
    assert worst < 1.5e-2, worst
    assert _rel(outs[0], outs[2]) < 1e-2 and torch.equal(outs[0], outs[1])


def test_sampling_kernels():
    torch.manual_seed(7)
    V, rows = 5000, 4
    lg = torch.randn(rows, V, device=DEV) * 3
    am = torch.zeros(rows, dtype=torch.int32, device=DEV)
    native.call("tf_argmax", lg, V, V, rows, am, None)
    assert am.cpu().tolist() == lg.argmax(-1).cpu().tolist()
    sb = native.lib().tf_rowstat_bytes()
    stat = torch.zeros(rows, sb, dtype=torch.uint8, device=DEV)
    st = native.StatusWord(DEV)
    T, top_p = 0.6, 0.95
    scr = torch.zeros(native.lib().tf_rowstats_scratch_bytes(rows), dtype=torch.uint8, device=DEV)
    native.call("tf_rowstats", lg, V, V, rows, T, top_p, stat, scr, st.t)
    assert int(scr.sum()) == 0          # every call leaves its scratch zeroed
    st.check()
    raw = stat.cpu().numpy().view(np.dtype([("m", "<f4"), ("thr", "<u4"), ("z", "<f8")]))
    pr = torch.softmax(lg.double().cpu() / T, -1)
    for r in range(rows):
        srt, _ = torch.sort(pr[r], descending=True)
        cs = torch.cumsum(srt, 0)
        n_in = int((cs < top_p).sum()) + 1
        mass = float(srt[:n_in].sum())
        z_total = float(torch.exp((lg[r].double().cpu() - lg[r].max().item()) / T).sum())
        assert abs(raw["z"][r][0] / z_total - mass) < 1e-6
    # plain sampling (g = 0): empirical law of the drawn tokens follows the nucleus distribution
    S = 4096
    lg1 = lg[:1].expand(S, V).contiguous()
    stat1 = stat[:1].expand(S, sb).contiguous()
    u = torch.rand(S, 2, dtype=torch.float64, device=DEV)
    R = torch.zeros(native.lib().tf_spec_verify_scratch_doubles(S, 0, V), dtype=torch.float64, device=DEV)
    w = torch.zeros(S, 1, dtype=torch.float64, device=DEV)
    nacc = torch.zeros(S, dtype=torch.int32, device=DEV)
    tok = torch.zeros(S, dtype=torch.int32, device=DEV)
    native.call("tf_spec_verify", lg1, None, stat1, None, None, u, S, 0, V, V, T, T, None, 0, R, w, nacc, tok, st.t)
    st.check()
    srt, idx = torch.sort(pr[0], descending=True)
    n_in = int((torch.cumsum(srt, 0) < top_p).sum()) + 1
    allowed = set(idx[:n_in].tolist())
    toks = tok.cpu().tolist()
    assert set(toks) <= allowed
    top = int(idx[0])
    want = float(srt[0] / srt[:n_in].sum())
    got = toks.count(top) / S
    assert abs(got - want) < 4 * math.sqrt(want * (1 - want) / S) + 1e-3


def test_block_verification_preserves_target_law():
    """Proposals from a draft law, verified against a target law: accepted/corrected first tokens
    must follow the target law (chi-square-style tolerance)."""
    torch.manual_seed(8)
    V, S, g = 64, 20000, 2
    tl = torch.randn(g + 1, V, device=DEV) * 1.5
    dl = tl[:g] + torch.randn(g, V, device=DEV) * 0.8
    T = 1.0
    sb = native.lib().tf_rowstat_bytes()
    st = native.StatusWord(DEV)
    tstat = torch.zeros(g + 1, sb, dtype=torch.uint8, device=DEV)
    dstat = torch.zeros(g, sb, dtype=torch.uint8, device=DEV)
    scr = torch.zeros(native.lib().tf_rowstats_scratch_bytes(g + 1), dtype=torch.uint8, device=DEV)
    native.call("tf_rowstats", tl, V, V, g + 1, T, 1.0, tstat, scr, st.t)
    native.call("tf_rowstats", dl, V, V, g, T, 1.0, dstat, scr, st.t)
    q = torch.softmax(dl.double(), -1)
    props = torch.stack([torch.multinomial(q[i], S, replacement=True) for i in range(g)], 1).int().contiguous()
    tlS = tl[None].expand(S, g + 1, V).contiguous()
    dlS = dl[None].expand(S, g, V).contiguous()
    u = torch.rand(S, g + 2, dtype=torch.float64, device=DEV)
    R = torch.zeros(native.lib().tf_spec_verify_scratch_doubles(S, g, V), dtype=torch.float64, device=DEV)
    w = torch.zeros(S, g + 1, dtype=torch.float64, device=DEV)
    nacc = torch.zeros(S, dtype=torch.int32, device=DEV)
    tok = torch.zeros(S, dtype=torch.int32, device=DEV)
    native.call("tf_spec_verify", tlS, dlS, tstat[None].expand(S, g + 1, sb).contiguous(),
                dstat[None].expand(S, g, sb).contiguous(), props, u, S, g, V, V, T, T, None, 0, R, w, nacc, tok, st.t)
    st.check()
    first = torch.where(nacc > 0, props[:, 0], tok).long().cpu()
    emp = torch.bincount(first, minlength=V).double() / S
    p0 = torch.softmax(tl[0].double().cpu(), -1)
    assert float((emp - p0).abs().max()) < 0.012
    assert 0.2 < float((nacc > 0).double().mean()) < 1.0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_key_sharded_selection_equals_unsharded(world):
    """Scoring split over `world` key shards (run one after the other here) + gather + merge gives
    exactly the ids of the unsharded selection."""
    from titanic_flash_41_b200.parallel import key_sharded as KS
    torch.manual_seed(9)
    T, Hi, Di, C, k = 6, 8, 128, 5000, 256
    krow = Di // 2 + Di // 32
    keys = codecs.index_key_encode(torch.randn(1, C, Di)).to(DEV).contiguous()
    q = torch.randn(T, Hi, Di, device=DEV).bfloat16()
    w = torch.rand(T, Hi, device=DEV)
    region = torch.zeros(T, dtype=torch.int32, device=DEV)
    nvalid = torch.tensor([5000, 4097, 300, 0, 129, 2600], dtype=torch.int32, device=DEV)
    lds = 5120
    scores = torch.zeros(T, lds, device=DEV)
    native.call("tf_index_scores", q, w, region, nvalid, keys, C * krow, krow, T, Hi, Di, 2, scores, lds, 0, C)
    want = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    wcnt = torch.zeros(T, dtype=torch.int32, device=DEV)
    native.call("tf_topk_select", scores, lds, nvalid, k, want, wcnt, None, 0, T)
    parts = [KS.local_candidates(q, w, region, nvalid, keys, C * krow, krow, T, Hi, Di, 2,
                                 torch.zeros(T, lds, device=DEV), C, k, r, world) for r in range(world)]
    ids, cnt = KS.merge(torch.cat([p[0] for p in parts], 1), torch.cat([p[1] for p in parts], 1), k)
    torch.cuda.synchronize()
    assert torch.equal(cnt, wcnt)
    assert torch.equal(ids, want)


@pytest.mark.parametrize("T", [1, 5, 16, 19])
def test_router_logits_small_matches_fp32(T):
    torch.manual_seed(T)
    E_, d = 72, 1024
    x = torch.randn(T, d, device=DEV).bfloat16()
    gate = (torch.randn(E_, d, device=DEV) / 32).bfloat16()
    out = torch.zeros(T, E_, device=DEV)
    native.call("tf_router_logits_small", x, d, gate, out, E_, T, E_, d)
    again = torch.zeros(T, E_, device=DEV)
    native.call("tf_router_logits_small", x, d, gate, again, E_, T, E_, d)
    torch.cuda.synchronize()
    want = x.float() @ gate.float().t()
    assert (out - want).abs().max() <= 1e-4 * want.abs().max() + 1e-5
    assert torch.equal(out, again)


def test_route_group_many_experts_is_sorted_and_stable():
    torch.manual_seed(9)
    El, T, k, e_lo = 200, 16, 6, 56
    ids = torch.stack([torch.randperm(256, device=DEV)[:k] for _ in range(T)]).int().contiguous()
    n = T * k
    i32 = lambda m: torch.zeros(m, dtype=torch.int32, device=DEV)
    ge, gs, gc, ng, sp, nl = i32(El), i32(El), i32(El), i32(1), i32(n), i32(1)
    native.call("tf_route_group", ids, n, e_lo, e_lo + El, ge, gs, gc, ng, sp, nl)
    torch.cuda.synchronize()
    flat = ids.flatten().cpu() - e_lo
    local = [(int(e), i) for i, e in enumerate(flat.tolist()) if 0 <= e < El]
    want_sorted = [i for _, i in sorted(local)]                      # by expert, then pair order
    assert int(nl) == len(local) and sp[: len(local)].tolist() == want_sorted
    experts = sorted({e for e, _ in local})
    assert int(ng) == len(experts) and ge[: len(experts)].tolist() == experts
    counts = [sum(1 for e, _ in local if e == x) for x in experts]
    assert gc[: len(experts)].tolist() == counts
    starts = [sum(counts[:j]) for j in range(len(experts))]
    assert gs[: len(experts)].tolist() == starts


@pytest.mark.parametrize("d", [512, 4096])
def test_fused_boundary_equals_combine_then_norm_then_quantiser(d):
    """tf_add_norm_fused against tf_moe_combine + tf_add_norm + tf_quant_rows_mx8: the residual is
    bit-identical; the mean square is summed in another order, so a normalised value may land on the
    neighbouring bf16 value."""
    torch.manual_seed(12)
    T, k, El, e_lo = 9, 3, 6, 2
    x0 = torch.randn(T, d, device=DEV).bfloat16()
    y_pair = torch.randn(T * k, d, device=DEV)
    ids = torch.randint(0, 10, (T, k), device=DEV, dtype=torch.int32)
    wts = torch.rand(T, k, device=DEV)
    shared = torch.randn(T, d, device=DEV)
    w = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    # separate kernels
    xa, delta = x0.clone(), torch.zeros(T, d, device=DEV)
    h16a, hba = torch.zeros(T, d, device=DEV, dtype=torch.float16), torch.zeros(T, d, device=DEV, dtype=torch.bfloat16)
    qa, sa = torch.zeros(T, d, dtype=torch.uint8, device=DEV), torch.zeros(T, d // 32, dtype=torch.uint8, device=DEV)
    native.call("tf_moe_combine", y_pair, ids, wts, shared, delta, T, d, k, e_lo, e_lo + El)
    native.call("tf_add_norm", xa, delta, 0, d, w, h16a, hba, None, None, T, d, 1e-6)
    native.call("tf_quant_rows_mx8", h16a, d, qa, sa, T, d)
    # one kernel
    xb = x0.clone()
    h16b, hbb, qb, sb = torch.zeros_like(h16a), torch.zeros_like(hba), torch.zeros_like(qa), torch.zeros_like(sa)
    native.call("tf_add_norm_fused", xb, None, y_pair, ids, wts, shared, k, e_lo, e_lo + El, w, h16b, hbb, qb, sb, T, d, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(xa, xb)
    for a, b_ in ((h16a, h16b), (hba, hbb)):
        assert (a.float() - b_.float()).abs().max() <= 0.01 * a.float().abs().max()
        assert (a == b_).float().mean() > 0.98
    deq = lambda q, s_: (q.view(torch.float8_e4m3fn).float().view(T, d // 32, 32) * torch.exp2(s_.float() - 127)[..., None])
    assert (deq(qa, sa) - deq(qb, sb)).abs().max() <= 0.07 * h16a.float().abs().max()
    assert (sa == sb).float().mean() > 0.98
    again = [torch.zeros_like(t) for t in (h16b, qb, sb)]
    xb2 = x0.clone()
    native.call("tf_add_norm_fused", xb2, None, y_pair, ids, wts, shared, k, e_lo, e_lo + El, w, again[0], None, again[1],
                again[2], T, d, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(again[0], h16b) and torch.equal(again[1], qb) and torch.equal(again[2], sb)   # run to run
    # plain delta source, no quantised copy
    xc, h16c = x0.clone(), torch.zeros_like(h16a)
    native.call("tf_add_norm_fused", xc, delta, None, None, None, None, 0, 0, 0, w, h16c, None, None, None, T, d, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(xc, xa) and (h16c == h16a).float().mean() > 0.98


@pytest.mark.parametrize("M", [3, 16, 27])
def test_router_topk_group_equals_the_two_launches(M):
    torch.manual_seed(M)
    E_, k, e_lo, El = 64, 6, 16, 32
    logits = torch.randn(M, E_, device=DEV)
    bias = torch.randn(E_, device=DEV) * 0.1
    i32 = lambda *s_: torch.zeros(*s_, dtype=torch.int32, device=DEV)
    out = []
    for fused in (False, True):
        ids, wts = i32(M, k), torch.zeros(M, k, device=DEV)
        ge, gs, gc, ng, sp, nl = i32(El), i32(El), i32(El), i32(1), i32(M * k), i32(1)
        if fused:
            native.call("tf_router_topk_group", logits, bias, None, None, -1, ids, wts, M, E_, k, 1, 1, 1.5, e_lo, e_lo + El,
                        ge, gs, gc, ng, sp, nl)
        else:
            native.call("tf_router_topk", logits, bias, None, None, -1, ids, wts, M, E_, k, 1, 1, 1.5)
            native.call("tf_route_group", ids, M * k, e_lo, e_lo + El, ge, gs, gc, ng, sp, nl)
        torch.cuda.synchronize()
        n, g = int(nl), int(ng)
        out.append((ids, wts, ge[:g].clone(), gs[:g].clone(), gc[:g].clone(), sp[:n].clone(), n, g))
    for a, b_ in zip(*out):
        assert torch.equal(a, b_) if isinstance(a, torch.Tensor) else a == b_


@pytest.mark.parametrize("T,n_max", [(4, 32768), (16, 20000), (3, 65536), (40, 30000), (36, 60000), (34, 70000)])
def test_topk_select_of_few_long_rows_matches_a_stable_sort(T, n_max):
    """A few long rows take the cluster-per-row kernel, more rows (or longer ones) the CTA-per-row
    kernel: same contract (exact, ties to the lower position, ids ascending, -1 padding, optional scores)."""
    torch.manual_seed(T)
    k, lds = 2048, n_max
    scores = (torch.randn(T, lds, device=DEV) * 0.3 + 5).relu()        # crowded exponents, like index scores
    scores[:, ::7] = scores[:, :1]                                      # many exact ties, some at the cut
    scores[0, :] = 1.25                                                 # a row of one value
    nvalid = torch.tensor([n_max, n_max - 13, 5000, 100][:T] + [n_max // 2 + i for i in range(max(0, T - 4))],
                          dtype=torch.int32, device=DEV)[:T]
    sel = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(T, dtype=torch.int32, device=DEV)
    osc = torch.zeros(T, k, device=DEV)
    native.call("tf_topk_select", scores, lds, nvalid, k, sel, cnt, osc, 100, T)
    torch.cuda.synchronize()
    for r in range(T):
        n = int(nvalid[r])
        s = scores[r, :n].cpu()
        got = sel[r].cpu().tolist()
        if n <= k:
            assert got == [100 + i for i in range(n)] + [-1] * (k - n) and int(cnt[r]) == n
            continue
        order = sorted(torch.sort(s, descending=True, stable=True).indices[:k].tolist())
        assert got == [100 + i for i in order] and int(cnt[r]) == k
        assert torch.equal(osc[r].cpu(), s[order])


@pytest.mark.parametrize("T", [1, 4, 16, 27])
def test_router_topk_group_in_registers_equals_the_shared_memory_form(T):
    """256 experts or fewer: the single-launch kernel keeps each row in registers; selection bias per
    row (image-token rows use the second bias), same ids, weights and groups as the two launches."""
    torch.manual_seed(40 + T)
    E_, k, e_lo, El = 256, 6, 64, 64
    logits = torch.randn(T, E_, device=DEV)
    bias, bias_vl = torch.randn(E_, device=DEV) * 0.1, torch.randn(E_, device=DEV) * 0.1
    tokens = torch.randint(0, 3, (T,), dtype=torch.int32, device=DEV)
    i32 = lambda *s_: torch.zeros(*s_, dtype=torch.int32, device=DEV)
    out = []
    for fused in (False, True):
        ids, wts = i32(T, k), torch.zeros(T, k, device=DEV)
        ge, gs, gc, ng, sp, nl = i32(El), i32(El), i32(El), i32(1), i32(T * k), i32(1)
        if fused:
            native.call("tf_router_topk_group", logits, bias, bias_vl, tokens, 1, ids, wts, T, E_, k, 1, 1, 1.5, e_lo,
                        e_lo + El, ge, gs, gc, ng, sp, nl)
        else:
            native.call("tf_router_topk", logits, bias, bias_vl, tokens, 1, ids, wts, T, E_, k, 1, 1, 1.5)
            native.call("tf_route_group", ids, T * k, e_lo, e_lo + El, ge, gs, gc, ng, sp, nl)
        torch.cuda.synchronize()
        n, g = int(nl), int(ng)
        out.append((ids, wts, ge[:g].clone(), gs[:g].clone(), gc[:g].clone(), sp[:n].clone(), n, g))
    for a, b_ in zip(*out):
        assert torch.equal(a, b_) if isinstance(a, torch.Tensor) else a == b_


def test_mxfp4_to_fp8_block_conversion_is_exact_where_representable():
    """e2m1 x 2^e re-expressed as e4m3 with one power-of-two scale per 128 x 128 block: exact while a
    group's scale is within 2^-6 of the block's largest (e4m3 holds the shifted magnitudes), rounded
    to nearest below that, signs kept."""
    torch.manual_seed(21)
    E_, N, K = 2, 256, 512
    pk = torch.randint(0, 256, (E_, N, K // 2), device=DEV, dtype=torch.uint8)
    sc = torch.randint(118, 126, (E_, N, K // 32), device=DEV, dtype=torch.uint8)
    sc[0, :5, :3] = 100                                   # far below the block maximum: rounds towards zero
    out = torch.zeros(E_, N, K, dtype=torch.uint8, device=DEV)
    out_s = torch.zeros(E_ * N // 128, K // 128, device=DEV)
    native.call("tf_mxfp4_to_fp8_block", pk, sc, out, out_s, E_, N, K, 0, N)
    torch.cuda.synchronize()
    want = E.dequant_mxfp4(pk, sc)                        # [E, N, K] fp32
    got = out.view(torch.float8_e4m3fn).float().view(E_, N // 128, 128, K // 128, 128) \
        * out_s.view(E_, N // 128, 1, K // 128, 1)
    got = got.reshape(E_, N, K)
    close = sc.view(E_, N // 128, 128, K // 128, 4).float()
    top = close.amax(dim=(2, 4), keepdim=True)
    exact = ((top - close) <= 6).expand_as(close).reshape(E_, N, K // 32).repeat_interleave(32, dim=2)
    assert torch.equal(got[exact], want[exact])
    blk_max = want.abs().view(E_, N // 128, 128, K // 128, 128).amax(dim=(2, 4), keepdim=True).expand(
        E_, N // 128, 128, K // 128, 128).reshape(E_, N, K)
    assert ((got - want).abs() <= blk_max * 2.0 ** -9).all()
    nz = got != 0
    assert torch.equal(torch.signbit(got[nz]), torch.signbit(want[nz]))


def test_mx8_row_quantiser_matches_codec():
    """e4m3 values with one UE8M0 scale per 32 inputs: same bytes as the host codec."""
    torch.manual_seed(5)
    x = (torch.randn(7, 512, device=DEV) * torch.rand(7, 1, device=DEV) * 4).half()
    x[3, 64:96] = 0
    q = torch.zeros(7, 512, dtype=torch.uint8, device=DEV)
    s = torch.zeros(7, 16, dtype=torch.uint8, device=DEV)
    native.call("tf_quant_rows_mx8", x, 512, q, s, 7, 512)
    torch.cuda.synchronize()
    wq, ws = codecs.mxfp8_quant(x.float().cpu(), 32)
    assert torch.equal(s.cpu()[ws != 0], ws[ws != 0])          # an all-zero group may carry any scale
    back = q.view(torch.float8_e4m3fn).float().view(7, 16, 32) * torch.exp2(s.float() - 127)[..., None]
    assert (back.view(7, 512) - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    assert torch.equal(q.cpu().view(7, 16, 32)[ws != 0], wq.view(torch.uint8).view(7, 16, 32)[ws != 0])


@pytest.mark.parametrize("dual,T", [(True, 16), (True, 5), (False, 16), (False, 3), (True, 24), (True, 32), (False, 24),
                                    (False, 32), (True, 17)])
def test_block_scaled_expert_gemv_matches_reference(dual, T):
    """MXFP4 weights x MXFP8 activations on tcgen05 block-scaled MMAs (scales applied by the tensor
    core) against fp32 math on the dequantised operands.  17..32 rows run the 32-column form."""
    from titanic_flash_41_b200.models import engine as E
    torch.manual_seed(7)
    El, N, K, k = 6, 256, 1024, 2
    w1 = torch.randn(El, N, K, device=DEV) * 0.1 * (1 + 3 * torch.rand(El, N, 1, device=DEV))
    w3 = torch.randn(El, N, K, device=DEV) * 0.1
    p1, s1 = E.quant_mxfp4_device(w1)
    p3, s3 = E.quant_mxfp4_device(w3)
    d1, d3 = E.dequant_mxfp4(p1, s1), E.dequant_mxfp4(p3, s3)
    ids = torch.stack([torch.randperm(El, device=DEV)[:k] for _ in range(T)]).int().contiguous()
    npairs = T * k
    i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=DEV)
    ge, gs, gc, ng, sp, nl = i32(El), i32(El), i32(El), i32(1), i32(npairs), i32(1)
    native.call("tf_route_group", ids, npairs, 0, El, ge, gs, gc, ng, sp, nl)
    rows = T if dual else npairs                       # plain form: one activation row per sorted pair
    x = (torch.randn(rows, K, device=DEV) * (0.2 + 2 * torch.rand(rows, 1, device=DEV))).half()
    xq = torch.zeros(rows, K, dtype=torch.uint8, device=DEV)
    xs = torch.zeros(rows, K // 32, dtype=torch.uint8, device=DEV)
    native.call("tf_quant_rows_mx8", x, K, xq, xs, rows, K)
    xd = (xq.view(torch.float8_e4m3fn).float().view(rows, K // 32, 32)
          * torch.exp2(xs.float() - 127)[..., None]).view(rows, K)
    st = native.StatusWord(DEV)
    if dual:
        y = torch.zeros(npairs, N, device=DEV, dtype=torch.float16)
    else:
        y = torch.zeros(npairs, N, device=DEV)
    y8 = torch.zeros(npairs, N, dtype=torch.uint8, device=DEV)
    y8s = torch.zeros(npairs, N // 32, dtype=torch.uint8, device=DEV)
    native.call("tf_moe_gemv_mx", p1, p3 if dual else None, s1, s3 if dual else None, El, xq, xs, rows, y, N,
                y8 if dual else None, y8s if dual else None, N, K, k, ge, gs, gc, ng, sp, min(El, npairs),
                10.0 if dual else 0.0, 0, 0, T, st.t)
    torch.cuda.synchronize()
    st.check()
    if dual:
        # the MXFP8 copy of the fused output equals quantising the f16 rows (up to f16 rounding of the input)
        back = (y8.view(torch.float8_e4m3fn).float().view(npairs, N // 32, 32)
                * torch.exp2(y8s.float() - 127)[..., None]).view(npairs, N)
        assert (back - y.float()).abs().max() <= 0.07 * y.float().abs().max() + 1e-3
    order = sp.tolist()
    for pos, pair in enumerate(order):
        t, j = divmod(pair, k)
        e = int(ids[t, j])
        if dual:
            a = d1[e] @ xd[t]
            up = (d3[e] @ xd[t]).clamp(-10, 10)
            want = torch.nn.functional.silu(a.clamp(max=10)) * up
            got = y[pos].float()                       # fused form writes rows in sorted pair order
            tol = 2e-3 * want.abs().max() + 2e-3
        else:
            want = d1[e] @ xd[pos]
            got = y[pair]
            tol = 1e-3 * want.abs().max() + 1e-4
        assert (got - want).abs().max() <= tol, (pos, pair, float((got - want).abs().max()), float(want.abs().max()))


def test_two_level_candidates_match_dense_selection():
    """Sparse scores equal the dense ones at the candidate keys, and selecting among the published
    blocks gives the dense top-k whenever all of it lies inside them."""
    from titanic_flash_41_b200.ops import two_level as TL
    torch.manual_seed(11)
    T, Hi, Di, C, k = 5, 8, 128, 4000, 64
    krow = Di // 2 + Di // 32
    keys = codecs.index_key_encode(torch.randn(1, C, Di)).to(DEV).contiguous()
    q = torch.randn(T, Hi, Di, device=DEV).bfloat16()
    w = torch.rand(T, Hi, device=DEV)
    region = torch.zeros(T, dtype=torch.int32, device=DEV)
    nvalid = torch.tensor([4000, 3001, 517, 64, 9], dtype=torch.int32, device=DEV)
    lds = 4096
    scores = torch.zeros(T, lds, device=DEV)
    native.call("tf_index_scores", q, w, region, nvalid, keys, C * krow, krow, T, Hi, Di, 1, scores, lds, 0, C)
    want = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    wcnt = torch.zeros(T, dtype=torch.int32, device=DEV)
    native.call("tf_topk_select", scores, lds, nvalid, k, want, wcnt, None, 0, T)
    cand = TL.publish(scores[:, :C], nvalid, n_blocks=128, T=T)
    assert cand.shape == (T, 1024)
    for r in range(T):
        c = cand[r][cand[r] >= 0]
        assert bool((c[1:] > c[:-1]).all()) and int(c.max()) < int(nvalid[r])
    sc = torch.empty(T, cand.shape[1], device=DEV)
    native.call("tf_index_scores_sparse", q, w, region, cand, cand.stride(0), keys, C * krow, krow, T, Hi, Di,
                cand.shape[1], sc, cand.shape[1])
    torch.cuda.synchronize()
    ok = cand >= 0
    dense_at = torch.gather(scores, 1, cand.clamp_min(0).long())
    assert (sc[ok] - dense_at[ok]).abs().max() <= 1e-3 * dense_at[ok].abs().max() + 1e-5
    assert bool(torch.isinf(sc[~ok]).all())
    ids, cnt = TL.consume(q, w, region, cand, keys, C * krow, krow, T, Hi, Di, k)
    assert torch.equal(cnt, wcnt)
    # the best 64 keys sit in the best 128 blocks of 8 (every top key's block maximum is at least its own
    # score); the two scorings may only disagree about keys that tie with the cut within rounding
    for r in range(T):
        a, b = set(ids[r][ids[r] >= 0].tolist()), set(want[r][want[r] >= 0].tolist())
        if a != b:
            cut = min(float(scores[r, i]) for i in b)
            assert all(abs(float(scores[r, i]) - cut) <= 1e-3 * abs(cut) + 1e-5 for i in a ^ b), r
