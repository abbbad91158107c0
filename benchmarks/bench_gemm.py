"""tcgen05 GEMM throughput (bf16, FP8, FP8 with fp32 block scales promoted in software, MXFP8 /
MXFP4 block-scaled by the tensor core) against torch.matmul (cuBLAS) bf16.

    python benchmarks/bench_gemm.py [--sizes 8192,4096 ...]
"""
import argparse

import torch

from common import peaks, time_cuda
from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.ops import mx, native


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192x8192x8192,16384x8192x4096,16384x4096x8192,4096x4096x4096,512x4096x4096")
    args = ap.parse_args()
    pk = peaks()
    st = native.StatusWord("cuda")
    print(f"# peaks ({pk['source']}): bf16 {pk['bf16_tflops']} TFLOP/s")
    for shp in args.shapes.split(","):
        M, N, K = map(int, shp.split("x"))
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        med, best = time_cuda(lambda: torch.matmul(a, b.t(), out=c))
        print(f"{shp} cublas-bf16   {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s (best {fl / best / 1e9:.1f})")
        med, best = time_cuda(lambda: native.call("tf_gemm_tc", 0, a, K, b, K, c, N, M, N, K, None, 0, None, 0, 2, None, None, 0, st.t))
        print(f"{shp} tcgen05-bf16  {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s (best {fl / best / 1e9:.1f}) "
              f"= {fl / med / 1e9 / pk['bf16_tflops']:.2f} of {pk['source']} bf16 peak")
        aq = a.to(torch.float8_e4m3fn)
        fw = E.quant_fp8_device(b.float())
        sa = torch.ones(M, K // 128, device="cuda")
        med, best = time_cuda(lambda: native.call("tf_gemm_tc", 1, aq, K, fw.q, K, c, N, M, N, K, None, 0, None, 0, 2, None, None, 0, st.t))
        print(f"{shp} tcgen05-fp8   {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s (best {fl / best / 1e9:.1f})")
        med, best = time_cuda(lambda: native.call("tf_gemm_tc", 2, aq, K, fw.q, K, c, N, M, N, K, sa, K // 128, fw.s, K // 128, 2, None, None, 0, st.t))
        print(f"{shp} tcgen05-fp8bs {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s (best {fl / best / 1e9:.1f}) "
              f"= {fl / med / 1e9 / pk['bf16_tflops']:.2f} x {pk['source']} bf16 peak")
        # block-scaled by the tensor core: MXFP8 activations x MXFP8 weights, and x packed MXFP4 weights
        xq = torch.zeros(M, K, dtype=torch.uint8, device="cuda")
        sfa = mx.empty_units(M, K, 128, "cuda")
        mx.quant_rows(a, M, K, xq, sfa)
        sfb = mx.units_from_rowmajor(torch.full((N, K // 32), 120, dtype=torch.uint8, device="cuda"), K)
        med, best = time_cuda(lambda: mx.gemm(xq, sfa, fw.q, sfb, c, M, N, K, st.t))
        print(f"{shp} tcgen05-mxfp8 {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s (best {fl / best / 1e9:.1f}) "
              f"= {fl / med / 1e9 / pk['bf16_tflops']:.2f} x {pk['source']} bf16 peak")
        w4 = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda")
        med, best = time_cuda(lambda: mx.gemm(xq, sfa, w4, sfb, c, M, N, K, st.t, b_fp4=True))
        print(f"{shp} tcgen05-mxfp8 x mxfp4 weights {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s (best {fl / best / 1e9:.1f})")
        med, best = time_cuda(lambda: mx.quant_rows(a, M, K, xq, sfa))
        print(f"{shp} mxfp8 quantiser of the activations {med:8.3f} ms  {(M * K * 3 + M * K / 32) / med / 1e6:8.1f} GB/s")
        native.lib().tf_gemm_tc_force_tile(128)
        med, best = time_cuda(lambda: native.call("tf_gemm_tc", 0, a, K, b, K, c, N, M, N, K, None, 0, None, 0, 2, None, None, 0, st.t))
        print(f"{shp} tcgen05-bf16 128x128 tiles  {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s")
        med, best = time_cuda(lambda: native.call("tf_gemm_tc", 2, aq, K, fw.q, K, c, N, M, N, K, sa, K // 128, fw.s, K // 128, 2, None, None, 0, st.t))
        print(f"{shp} tcgen05-fp8bs 128x128 tiles {med:8.3f} ms  {fl / med / 1e9:8.1f} TFLOP/s")
        native.lib().tf_gemm_tc_force_tile(0)
        st.check()


if __name__ == "__main__":
    main()
