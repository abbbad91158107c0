// Router logits of the decode step: logits[r, e] = sum_k x[r, k] * gate[e, k] for a few rows.
//
// The gate matrix is small (experts x hidden bf16, 2 MB at 256 x 4096), so the generic
// weight-streaming GEMV, which gives one CTA 32 output features, would run it on 8 CTAs and wait
// on memory latency.  Here one CTA owns one expert row and its four warps a quarter of the inputs
// each: every lane walks its quarter in 16-byte steps with 16 row accumulators (the activation
// rows come out of L1 / L2), the warps' partial sums meet in shared memory and are added in warp
// order.  Fixed summation order: bitwise reproducible.
//
// Reference behaviour: router scores of kernels/moe_frontend.cuh (`ca_route_topk` takes these
// logits); the top-k itself stays in tf_router_topk.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

constexpr int kRowsPerPass = 16;

__device__ __forceinline__ void router_logits_body(const __nv_bfloat16* __restrict__ x, int ldx,
                                                   const __nv_bfloat16* __restrict__ gate, float* __restrict__ out,
                                                   int ldo, int T, int E, int d) {
  __shared__ float red[4][kRowsPerPass];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x;
  const uint4* wrow = reinterpret_cast<const uint4*>(gate + (long)e * d);
  const int steps = d / 8;                                   // 16-byte steps of a row
  const int per = (steps + 3) / 4, k_lo = warp * per, k_hi = min(steps, k_lo + per);
  // the first gate vectors (immutable) are requested before waiting for the kernel that writes x
  uint4 wpre[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int k8 = k_lo + lane + 32 * j;
    wpre[j] = k8 < k_hi ? __ldg(wrow + k8) : make_uint4(0u, 0u, 0u, 0u);
  }
  tf_pdl_sync();
  for (int t0 = 0; t0 < T; t0 += kRowsPerPass) {
    float acc[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) acc[r] = 0.f;
    int it = t0 == 0 ? 0 : 2;
#pragma unroll 2
    for (int k8 = k_lo + lane; k8 < k_hi; k8 += 32, ++it) {
      uint4 w;
      if (it == 0) w = wpre[0];
      else if (it == 1) w = wpre[1];
      else w = __ldg(wrow + k8);
      uint4 xv[kRowsPerPass];
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r)
        xv[r] = __ldg(reinterpret_cast<const uint4*>(x + (long)min(t0 + r, T - 1) * ldx) + k8);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
      float2 wf[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) wf[j] = __bfloat1622float2(wp[j]);
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r) {
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xf = __bfloat1622float2(xp[j]);
          acc[r] = fmaf(wf[j].x, xf.x, acc[r]);
          acc[r] = fmaf(wf[j].y, xf.y, acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) {
      const float v = warp_sum(acc[r]);
      if (lane == 0) red[warp][r] = v;
    }
    __syncthreads();
    if (threadIdx.x < kRowsPerPass && t0 + threadIdx.x < T) {
      const int r = threadIdx.x;
      out[(long)(t0 + r) * ldo + e] = ((red[0][r] + red[1][r]) + red[2][r]) + red[3][r];
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(128)
router_logits_small_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ gate,
                           float* __restrict__ out, int ldo, int T, int E, int d) {
  router_logits_body(x, ldx, gate, out, ldo, T, E, d);
}

}  // namespace

// x [T, d] bf16 (row pitch ldx elements), gate [E, d] bf16, out [T, E] f32 (row pitch ldo)
TF_API int tf_router_logits_small(const void* x, int ldx, const void* gate, void* out, int ldo, int T, int E, int d,
                                  cudaStream_t st) {
  if (T <= 0 || d % 8 || ldx % 8) return -1;
  tf_launch(router_logits_small_kernel, dim3(E), dim3(128), 0, st, reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                        reinterpret_cast<const __nv_bfloat16*>(gate),
                                                        reinterpret_cast<float*>(out), ldo, T, E, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
