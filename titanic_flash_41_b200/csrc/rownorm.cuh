// Tail of a sublayer boundary for one row held in shared memory: RMSNorm scale, norm weight, the
// f16 / bf16 copies and (optionally) the MXFP8 form read by the block-scaled expert GEMV.  Shared
// by the boundary kernel (fused_norm.cu) and by the epilogue of the one-shot all-reduce (comm.cuh),
// so both produce bit-identical rows from the same residual.
//   v = bf16(x * rsqrt(mean(x^2) + eps) * w)            (reference: kernels/core.cu:851 ca_rms_bf16)
//   MXFP8: e4m3 values + one UE8M0 scale per 32 inputs  (reference: kernels/moe_frontend.cuh:158-242)
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

// `row` holds the d residual values (already bf16-rounded) of row r; `ss` is their sum of squares
// as every thread of the CTA knows it.  Must be called by every thread of the CTA.
__device__ __forceinline__ void row_norm_store(float* row, int d, float ss, float eps, const __nv_bfloat16* w,
                                               __half* h16, __nv_bfloat16* hb, uint8_t* x8, uint8_t* x8s, long r) {
  const float inv = rsqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = bf16_round(row[i] * inv * __bfloat162float(w[i]));
    row[i] = v;
    if (h16) h16[r * d + i] = __float2half(v);
    if (hb) hb[r * d + i] = __float2bfloat16(v);
  }
  if (x8) {
    __syncthreads();
    // one warp per group of 32 inputs; values as the f16 copy holds them
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = warp; b < d / 32; b += nw) {
      const float v = __half2float(__float2half(row[b * 32 + lane]));
      const float amax = warp_max(fabsf(v));
      int ex = -127;
      if (amax > 0.f) {
        int e2;
        const float m = frexpf(amax * (1.f / 448.f), &e2);
        ex = max(-127, min(127, (m == 0.5f) ? e2 - 1 : e2));
      }
      x8[r * d + b * 32 + lane] = (uint8_t)__nv_cvt_float_to_fp8(v * exp2f((float)-ex), __NV_SATFINITE, __NV_E4M3);
      if (lane == 0) x8s[r * (d / 32) + b] = (uint8_t)(ex + 127);
    }
  }
}
