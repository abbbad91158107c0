"""Small, self-ending cases of single kernels for a profiler capture (one GPU, a few launches, well
under a GB on the device).  Each target prints the CUDA-event time of its launches.

    python benchmarks/profile_targets.py allreduce     # one-shot all-reduce + boundary, 2 emulated ranks, 16 x 4096
    python benchmarks/profile_targets.py sampler       # chunked sampler: verification of 4 x (3 + 1) rows, vocabulary 129,280
    python benchmarks/profile_targets.py attention     # sparse attention: 2,048 prefill rows, 64 heads x 128, 128 window + 2,048 selected keys
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
    q = (torch.randn(T, Hl, Dh, device=DEV, generator=gen) * 0.5).bfloat16()
    sink = torch.zeros(Hl, device=DEV)
    freqs = torch.tensor([10000.0 ** (-2.0 * j / 64) for j in range(32)], device=DEV)
    part_o = torch.zeros(T, 1, Hl, Dh, device=DEV)
    part_lse = torch.zeros(T, 1, Hl, device=DEV)
    out = torch.zeros(T, Hl * Dh, device=DEV, dtype=torch.float16)
    st = native.StatusWord(DEV)
    us = timed(lambda: native.call("tf_sparse_attention", q, T, Hl, Dh, pos, region, None, win, ring * win_row, win_row, ring,
                                   window, comp, C * comp_row, comp_row, sel, k, None, C, 1 / math.sqrt(Dh), 1, part_o,
                                   part_lse, sink, freqs, 64, out, None, Hl * Dh, st.t), n=3, warm=1)
    st.check()
    flops = 4.0 * T * Hl * Dh * (window + k)
    print(f"sparse attention, {T} rows x {Hl} heads x {Dh}, {window}+{k} keys: {us:.0f} us per launch, "
          f"{flops / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    {"allreduce": allreduce, "sampler": sampler, "attention": attention}[sys.argv[1]]()
