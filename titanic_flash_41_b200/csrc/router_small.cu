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
#include "router.cuh"

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
  for (int t0 = 0; t0 < T; t0 += kRowsPerPass) {
    float acc[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) acc[r] = 0.f;
#pragma unroll 2
    for (int k8 = k_lo + lane; k8 < k_hi; k8 += 32) {
      const uint4 w = __ldg(wrow + k8);
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
      if (lane == 0 && warp < 4) red[warp][r] = v;   // (warps past the fourth only take part in the barriers)
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
  tf_pdl_sync();
  router_logits_body(x, ldx, gate, out, ldo, T, E, d);
}

struct RouteOut {
  int* ids;
  float* wts;
  int topk, scoring, renorm;
  float scale;
  int e_lo, e_hi;
  int *group_expert, *group_start, *group_count, *n_groups, *sorted_pairs, *n_local_pairs;
  unsigned* ticket;                                   // zero between launches
};

// Logits, top-k and grouping in ONE launch: every CTA computes its expert's column, and the CTA
// that finishes last (a ticket counter) selects, one warp per row, and groups from the finished
// logit rows.
__global__ void __launch_bounds__(128)
router_small_fused_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ gate,
                          float* __restrict__ logits, int T, int E, int d, const RouterBias rb, const RouteOut o) {
  tf_pdl_sync();
  extern __shared__ int route_sm[];                   // [e_hi - e_lo] counts / offsets, [T * topk] local experts
  __shared__ int s_last;
  router_logits_body(x, ldx, gate, logits, E, T, E, d);
  __threadfence();                                    // this CTA's column is visible before its ticket
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(o.ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // four warps: up to four rows each at once (16 rows in one pass), one row each for a few rows
  const int warp = threadIdx.x >> 5;
  if (T > 4) {
    for (int r0 = warp * 4; r0 < T; r0 += 16)
      router_topk_rows_reg<8, 4>(logits, E, rb, r0, T, o.ids, o.wts, E, o.topk, o.scoring, o.renorm, o.scale,
                                 route_sm + (o.e_hi - o.e_lo), o.e_lo, o.e_hi);
  } else if (warp < T) {
    router_topk_rows_reg<8, 1>(logits, E, rb, warp, T, o.ids, o.wts, E, o.topk, o.scoring, o.renorm, o.scale,
                               route_sm + (o.e_hi - o.e_lo), o.e_lo, o.e_hi);
  }
  __syncthreads();
  route_group_body(nullptr, T * o.topk, o.e_lo, o.e_hi, o.group_expert, o.group_start, o.group_count, o.n_groups,
                   o.sorted_pairs, o.n_local_pairs, route_sm);
  if (threadIdx.x == 0) *o.ticket = 0u;
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

// tf_router_logits_small followed by tf_router_topk_group in one launch (E <= 256, up to 32 rows).
// `ticket`: one zeroed 32-bit word that stays with this call site (left zero on return).
TF_API int tf_router_small_fused(const void* x, int ldx, const void* gate, float* logits, int T, int E, int d,
                                 const float* bias, const float* bias_vl, const int* tokens, int image_token, int* ids,
                                 float* wts, int topk, int scoring, int renorm, float scale, int e_lo, int e_hi,
                                 int* group_expert, int* group_start, int* group_count, int* n_groups,
                                 int* sorted_pairs, int* n_local_pairs, void* ticket, cudaStream_t st) {
  const size_t smem = (size_t)(e_hi - e_lo + T * topk) * sizeof(int);
  if (T <= 0 || T > 32 || d % 8 || ldx % 8 || E > 256 || topk > 32 || e_hi <= e_lo || !ticket || smem > 40 * 1024)
    return -1;
  const RouterBias rb{bias, bias_vl, tokens, image_token};
  const RouteOut o{ids, wts, topk, scoring, renorm, scale, e_lo, e_hi, group_expert, group_start, group_count,
                   n_groups, sorted_pairs, n_local_pairs, reinterpret_cast<unsigned*>(ticket)};
  tf_launch(router_small_fused_kernel, dim3(E), dim3(128), smem, st, reinterpret_cast<const __nv_bfloat16*>(x), ldx,
            reinterpret_cast<const __nv_bfloat16*>(gate), logits, T, E, d, rb, o);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
