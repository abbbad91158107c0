"""Small, self-ending cases of single kernels for a profiler capture (one GPU, a few launches, well
under a GB on the device).  Each target prints the CUDA-event time of its launches.

    python benchmarks/profile_targets.py allreduce     # one-shot all-reduce + boundary, 2 emulated ranks, 16 x 4096
    python benchmarks/profile_targets.py sampler       # chunked sampler: verification of 4 x (3 + 1) rows, vocabulary 129,280
    python benchmarks/profile_targets.py attention     # sparse attention: 2,048 prefill rows, 64 heads x 128, 128 window + 2,048 selected keys
    python benchmarks/profile_targets.py index         # index scores + exact top-2048 of 2,048 prefill rows over 32,768 keys, 8 heads x 128
    python benchmarks/profile_targets.py prep          # attention prep of 2,048 prefill rows (RoPE, FP8 window rows, pooling, FP4 entries, index keys)
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from titanic_flash_41_b200.ops import native  # noqa: E402

DEV = "cuda"


def timed(fn, n=5, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) * 1e3)
    return sorted(out)[len(out) // 2]


def allreduce():
    from titanic_flash_41_b200.parallel.symm import EmulatedRanks
    world, N, rows = 2, 4096, 16
    emu = EmulatedRanks(world, N, 32, device=DEV)
    st = native.StatusWord(DEV)
    part = torch.randn(world, rows, N, device=DEV)
    resid = torch.randn(world, rows, N, device=DEV).bfloat16()
    w = torch.ones(N, device=DEV, dtype=torch.bfloat16)
    h16 = torch.zeros(world, rows, N, device=DEV, dtype=torch.float16)
    hb = torch.zeros(world, rows, N, device=DEV, dtype=torch.bfloat16)
    x8 = torch.zeros(world, rows, N, device=DEV, dtype=torch.uint8)
    x8s = torch.zeros(world, rows, N // 32, device=DEV, dtype=torch.uint8)
    us = timed(lambda: emu.allreduce(part, rows, st.t, resid=resid, norm=dict(w=w, h16=h16, hb=hb, x8=x8, x8s=x8s, eps=1e-6)))
    st.check()
    print(f"allreduce+boundary, {world} emulated ranks, {rows} x {N}: {us:.1f} us per launch")


def sampler():
    from titanic_flash_41_b200.parallel.symm import SampleWorkspace
    V, S, g = 129280, 4, 3
    ws = SampleWorkspace(V, S * (g + 1), DEV)
    st = native.StatusWord(DEV)
    sb = native.lib().tf_rowstat_bytes()
    gen = torch.Generator(device=DEV).manual_seed(1)
    tl = torch.randn(S * (g + 1), V, device=DEV, generator=gen) * 3
    dl = tl.view(S, g + 1, V)[:, :g].contiguous() + torch.randn(S, g, V, device=DEV, generator=gen)
    temp, topp = torch.full((S,), 0.6, device=DEV), torch.full((S,), 0.95, device=DEV)
    dstat = torch.zeros(S, g, sb, dtype=torch.uint8, device=DEV)
    props = torch.zeros(S, g, dtype=torch.int32, device=DEV)
    ud = torch.rand(S, g, dtype=torch.float64, device=DEV, generator=gen)
    for j in range(g):
        ws.sample(dl[:, j].contiguous(), None, None, None, ud[:, j:], g, temp, topp, S, 0, V, dstat[:, j], g, None,
                  props[:, j:], g, st.t)
    tstat = torch.zeros(S * (g + 1), sb, dtype=torch.uint8, device=DEV)
    nacc, tok = torch.zeros(S, dtype=torch.int32, device=DEV), torch.zeros(S, dtype=torch.int32, device=DEV)
    u = torch.rand(S, g + 2, dtype=torch.float64, device=DEV, generator=gen)
    us = timed(lambda: ws.sample(tl, dl, dstat, props, u, g + 2, temp, topp, S, g, V, tstat, 1, nacc, tok, 1, st.t))
    st.check()
    print(f"chunked sampler, verification of {S} x {g + 1} rows of {V} logits: {us:.1f} us per launch")


def attention():
    from titanic_flash_41_b200.formats import codecs
    T, Hl, Dh, window, C, k = 2048, 64, 128, 128, 32768, 2048
    ring = 16384 + 256
    win_row, comp_row = -(-(Dh + Dh // 32) // 16) * 16, -(-(Dh // 2 + Dh // 16) // 16) * 16
    gen = torch.Generator(device=DEV).manual_seed(2)
    win = torch.zeros(1, ring, win_row, dtype=torch.uint8, device=DEV)
    win[:, :, :Dh + Dh // 32] = codecs.kv_v41_encode(torch.randn(1, ring, Dh)).to(DEV)
    comp = torch.zeros(1, C, comp_row, dtype=torch.uint8, device=DEV)
    comp[:, :, :Dh // 2 + Dh // 16] = codecs.kv_v41fp4_encode(torch.randn(1, C, Dh)).to(DEV)
    pos = (torch.arange(T, dtype=torch.int32) + 131072 - T).to(DEV)
    region = torch.zeros(T, dtype=torch.int32, device=DEV)
    sel = torch.stack([torch.sort(torch.randperm(C, device=DEV, generator=gen)[:k]).values for _ in range(64)]).int()
    sel = sel.repeat(T // 64, 1).contiguous()
    cnt = torch.full((T,), k, dtype=torch.int32, device=DEV)
    q = (torch.randn(T, Hl, Dh, device=DEV, generator=gen) * 0.5).bfloat16()
    sink = torch.zeros(Hl, device=DEV)
    freqs = torch.tensor([10000.0 ** (-2.0 * j / 64) for j in range(32)], device=DEV)
    part_o = torch.zeros(T, 1, Hl, Dh, device=DEV)
    part_lse = torch.zeros(T, 1, Hl, device=DEV)
    out = torch.zeros(T, Hl * Dh, device=DEV, dtype=torch.float16)
    st = native.StatusWord(DEV)
    us = timed(lambda: native.call("tf_sparse_attention", q, T, Hl, Dh, pos, region, None, win, ring * win_row, win_row, ring,
                                   window, comp, C * comp_row, comp_row, sel, k, cnt, C, 1 / math.sqrt(Dh), 1, part_o,
                                   part_lse, sink, freqs, 64, out, None, Hl * Dh, st.t), n=3, warm=1)
    st.check()
    flops = 4.0 * T * Hl * Dh * (window + k)
    print(f"sparse attention, {T} rows x {Hl} heads x {Dh}, {window}+{k} keys: {us:.0f} us per launch, "
          f"{flops / us / 1e6:.1f} TFLOP/s")


def index():
    T, Hi, Di, C, k = 2048, 8, 128, 32768, 2048
    krow = Di // 2 + Di // 32
    gen = torch.Generator(device=DEV).manual_seed(3)
    keys = torch.randint(0, 256, (1, C, krow), dtype=torch.uint8, device=DEV, generator=gen)
    keys[:, :, Di // 2:] = 120                                  # UE8M0 scales near 2^-7
    q = torch.randn(T, Hi, Di, device=DEV, generator=gen).bfloat16()
    w = torch.rand(T, Hi, device=DEV, generator=gen)
    region = torch.zeros(T, dtype=torch.int32, device=DEV)
    nvalid = ((torch.arange(T, device=DEV) + 131072 - T + 1) // 4).int()
    scores = torch.zeros(T, C, device=DEV)
    sel = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(T, dtype=torch.int32, device=DEV)
    us = timed(lambda: native.call("tf_index_scores", q, w, region, nvalid, keys, C * krow, krow, T, Hi, Di, 32, scores, C, 0,
                                   C), n=3, warm=1)
    print(f"index scores, {T} rows x {C} keys, {Hi} heads x {Di}: {us:.0f} us per launch, "
          f"{2.0 * T * C * Hi * Di / us / 1e6:.1f} TFLOP/s")
    us = timed(lambda: native.call("tf_topk_select", scores, C, nvalid, k, sel, cnt, None, 0, T), n=3, warm=1)
    print(f"top-{k} select of {T} rows x {C} scores: {us:.0f} us per launch")


def prep():
    T, Hl, Dh, Di, Hi, ratio, rope = 2048, 64, 128, 128, 8, 4, 64
    ring, maxC = 16384 + 256, 32768 + 8
    win_row, comp_row = -(-(Dh + Dh // 32) // 16) * 16, -(-(Dh // 2 + Dh // 16) // 16) * 16
    krow = Di // 2 + Di // 32
    C = Dh + Di
    offs, o = {}, 0
    for nm, wd in (("q", Hl * Dh), ("kv", Dh), ("cv", C), ("cg", C), ("iq", Hi * Di), ("iw", Hi)):
        offs[nm] = o
        o += wd
    W = -(-o // 8) * 8
    gen = torch.Generator(device=DEV).manual_seed(4)
    P = torch.randn(T, W, device=DEV, generator=gen).bfloat16()
    pos = (torch.arange(T, dtype=torch.int32) + 131072 - T).to(DEV)
    region = torch.zeros(T, dtype=torch.int32, device=DEV)
    first = torch.zeros(T, dtype=torch.int32, device=DEV)
    last = torch.full((T,), 131071, dtype=torch.int32, device=DEV)
    freqs = torch.tensor([10000.0 ** (-2.0 * j / rope) for j in range(rope // 2)], device=DEV)
    norm = torch.ones(Dh, device=DEV, dtype=torch.bfloat16)
    qo = torch.zeros(T, Hl * Dh, device=DEV, dtype=torch.bfloat16)
    win = torch.zeros(1, ring, win_row, dtype=torch.uint8, device=DEV)
    comp = torch.zeros(1, maxC, comp_row, dtype=torch.uint8, device=DEV)
    keys = torch.zeros(1, maxC, krow, dtype=torch.uint8, device=DEV)
    carry = torch.zeros(1, ratio + 32, 2 * C, device=DEV)
    iq = torch.zeros(T, Hi * Di, device=DEV, dtype=torch.bfloat16)
    iw = torch.zeros(T, Hi, device=DEV)
    st = native.StatusWord(DEV)
    us = timed(lambda: native.call("tf_attn_prep", P, 1, W, T, pos, region, first, last, Hl, Dh, rope, freqs, freqs, norm, 1e-6,
                                   qo, win, ring * win_row, win_row, comp_row, krow, ring, offs["q"], offs["kv"], offs["cv"],
                                   offs["cg"], offs["iq"], offs["iw"], ratio, Di, Hi, norm, carry, carry.shape[1], comp, keys, maxC, iq, iw,
                                   st.t), n=3, warm=1)
    st.check()
    print(f"attention prep, {T} rows ({W} projected columns): {us:.0f} us per launch, "
          f"{(T * W * 2 + T * Hl * Dh * 2) / us / 1e3:.0f} GB/s of rows read + queries written")


if __name__ == "__main__":
    targets = {"allreduce": allreduce, "sampler": sampler, "attention": attention, "index": index, "prep": prep}
    if len(sys.argv) != 2 or sys.argv[1] not in targets:
        sys.exit("usage: python benchmarks/profile_targets.py {" + " | ".join(sorted(targets)) + "}")
    targets[sys.argv[1]]()
