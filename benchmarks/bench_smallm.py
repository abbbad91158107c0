"""Weight-streaming small-M GEMMs of the decode step, standalone: routed-expert FC1 (MXFP4, dual
w1/w3 + SwiGLU), FC2 (MXFP4) and a dense FP8 block-scaled projection, each against its HBM
roofline (bytes of weights + scales that must be read once).

    python benchmarks/bench_smallm.py [--experts 64] [--tokens 16] [--hidden 4096] [--inter 2048]
"""
import argparse

import torch

from common import peaks, time_cuda
from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import native


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=16)
    ap.add_argument("--topk", type=int, default=6)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--graph", action="store_true", help="time the replay of a captured CUDA graph")
    ap.add_argument("--only", default="", help="run only the variants whose name contains this")
    a = ap.parse_args()
    dev, pk = "cuda", peaks()
    El, T, k, d, I = a.experts, a.tokens, a.topk, a.hidden, a.inter
    g = torch.Generator(device=dev).manual_seed(0)

    def fp4(n, kk):
        return (torch.randint(0, 256, (El, n, kk // 2), device=dev, dtype=torch.uint8, generator=g),
                torch.full((El, n, kk // 32), 120, device=dev, dtype=torch.uint8))
    w1, s1 = fp4(I, d)
    w3, s3 = fp4(I, d)
    w2, s2 = fp4(d, I)
    ids = torch.stack([torch.randperm(El, device=dev, generator=g)[:k] for _ in range(T)]).int().contiguous()
    npairs = T * k
    i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
    g_expert, g_start, g_count, n_groups, sorted_pairs, n_local = i32(El), i32(El), i32(El), i32(1), i32(npairs), i32(1)
    native.call("tf_route_group", ids, npairs, 0, El, g_expert, g_start, g_count, n_groups, sorted_pairs, n_local)
    h16 = (torch.randn(T, d, device=dev, generator=g) * 0.5).half()
    act = torch.zeros(npairs, I, device=dev, dtype=torch.float16)
    y = torch.zeros(npairs, d, device=dev, dtype=torch.float32)      # the FC2 calls below ask for fp32 output
    slots = min(El, npairs)
    used = int(n_groups.item())

    def fc1():
        native.call("tf_smallm_gemm", 1, w1, w3, s1, s3, I * (d // 2), I * (d // 32), d // 2, d // 32, h16, d, act, I, 1,
                    I, d, 0, g_expert, g_start, g_count, n_groups, sorted_pairs, k, slots, min(T, 16), 10.0)

    def fc2():
        native.call("tf_smallm_gemm", 1, w2, None, s2, None, d * (I // 2), d * (I // 32), I // 2, I // 32, act, I, y, d, 0,
                    d, I, 0, g_expert, g_start, g_count, n_groups, sorted_pairs, 1, slots, min(T, 16), 0.0)

    fw = E.quant_fp8_device(torch.randn(d * 2, d, device=dev, generator=g) * 0.02)
    yd = torch.zeros(T, d * 2, device=dev, dtype=torch.float16)

    def dense():
        native.call("tf_smallm_gemm", 0, fw.q, None, fw.s, None, 0, 0, d, fw.s.shape[1], h16, d, yd, d * 2, 0, d * 2, d, T,
                    None, None, None, None, None, 1, 0, T, 0.0)

    stw = native.StatusWord(dev)

    # block-scaled tensor-core form: MXFP8 activations, the MMA consumes nibbles and scales
    x8 = torch.zeros(T, d, dtype=torch.uint8, device=dev)
    x8s = torch.zeros(T, d // 32, dtype=torch.uint8, device=dev)
    a8 = torch.zeros(npairs, I, dtype=torch.uint8, device=dev)
    a8s = torch.zeros(npairs, I // 32, dtype=torch.uint8, device=dev)

    def fc1_mx(blocked=0):
        native.call("tf_quant_rows_mx8", h16, d, x8, x8s, T, d)
        native.call("tf_moe_gemv_mx", w1, w3, s1, s3, El, x8, x8s, T, None, I, a8, a8s, I, d, k, g_expert, g_start,
                    g_count, n_groups, sorted_pairs, slots, 10.0, 0, blocked, T, stw.t)

    def fc2_mx(blocked=0):
        native.call("tf_moe_gemv_mx", w2, None, s2, None, El, a8, a8s, npairs, y, d, None, None, d, I, 1, g_expert,
                    g_start, g_count, n_groups, sorted_pairs, slots, 0.0, 0, blocked, T, stw.t)

    print(f"# peaks ({pk['source']}): HBM {pk['hbm_gbs']} GB/s; {used} of {El} experts hit by {npairs} pairs")
    for name, fn, nbytes in (("moe_fc1_mxfp4_dual", fc1, used * 2 * I * (d // 2 + d // 32)),
                             ("moe_fc2_mxfp4", fc2, used * d * (I // 2 + I // 32)),
                             ("moe_fc1_mx_tcgen05_dual (+quant)", fc1_mx, used * 2 * I * (d // 2 + d // 32)),
                             ("moe_fc2_mx_tcgen05 (input quantised by FC1)", fc2_mx, used * d * (I // 2 + I // 32)),
                             # same bytes read as [128 x 128] blocks of 8 KB (random nibbles: timing only)
                             ("moe_fc1_mx_tcgen05 blocked", lambda: fc1_mx(1), used * 2 * I * (d // 2 + d // 32)),
                             ("moe_fc2_mx_tcgen05 blocked", lambda: fc2_mx(1), used * d * (I // 2 + I // 32)),
                             ("dense_fp8_block128", dense, 2 * d * d + fw.s.numel() * 4)):
        if a.only and a.only not in name:
            continue
        med, best = time_cuda(fn, iters=a.iters, graph=a.graph)
        stw.check()
        print(f"{name:32s} {med * 1e3:8.1f} us  {nbytes / med / 1e6:8.1f} GB/s = "
              f"{nbytes / med / 1e6 / pk['hbm_gbs']:.2f} of {pk['source']} HBM copy bandwidth (best {best * 1e3:.1f} us)")


if __name__ == "__main__":
    main()
