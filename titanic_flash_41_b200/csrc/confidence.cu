// Confidence head of the drafter and the causal stopping rule, device side.
//
//   tf_draft_confidence   after draft pass j (0-based) of S conversations:
//                           c_j = sigmoid(<w[0:d], hidden_j> + <w[d:d+r], latent_j>)
//                         hidden_j = the drafter's residual stream of the pass before the final norm,
//                         latent_j = the Markov embedding of the token the pass was fed (r = 0: none)
//                         (reference: kernels/dspark_confidence_fused.cuh ca_confidence_fused_full,
//                         weight mtp.<last>.confidence_head.proj.weight [1, d + r] widened to fp32).
//                         Then the stopping rule, kept on the device so that the verification
//                         launch of the same CUDA graph can read it:
//                           cum_0 = c_0, verify = 1; pass j >= 1: cum_j = cum_{j-1} * c_j and
//                           proposal j + 1 is verified iff every earlier one is and cum_j >= ladder[j-1]
//                         (reference: src/dspark_generation.rs causal_ladder_rows: each confidence
//                         precedes the proposal it admits, the first failed threshold stops, a NaN
//                         stops; later confidences cannot change the length).
// Every rank of a tensor-parallel group holds the same residual rows bit for bit and sums in the
// same order, so all ranks reach the same counts without an exchange.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) draft_confidence_kernel(const void* __restrict__ x, int x_kind, int ldx,
                                                               const __nv_bfloat16* __restrict__ lat, int r,
                                                               const float* __restrict__ w,
                                                               const float* __restrict__ ladder, int n_ladder,
                                                               int j, int g, float* __restrict__ conf,
                                                               float* __restrict__ cum, int* __restrict__ verify,
                                                               int d) {
  tf_pdl_sync();
  __shared__ float part[8];
  const int s = blockIdx.x, t = threadIdx.x;
  float sum = 0.f;
  if (x_kind == 0) {
    const float* row = reinterpret_cast<const float*>(x) + (long)s * ldx;
    for (int i = t; i < d; i += 256) sum = fmaf(row[i], w[i], sum);
  } else {
    const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(x) + (long)s * ldx;
    for (int i = t; i < d; i += 256) sum = fmaf(__bfloat162float(row[i]), w[i], sum);
  }
  if (lat != nullptr)
    for (int i = t; i < r; i += 256) sum = fmaf(__bfloat162float(lat[(long)s * r + i]), w[d + i], sum);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
  if ((t & 31) == 0) part[t >> 5] = sum;
  __syncthreads();
  if (t == 0) {
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += part[k];
    const float c = 1.f / (1.f + expf(-tot));
    conf[(long)s * g + j] = c;
    if (j == 0) {
      cum[s] = c;
      verify[s] = 1;
    } else {
      const float cv = cum[s] * c;
      cum[s] = cv;
      const float thr = ladder[min(j - 1, n_ladder - 1)];
      if (verify[s] == j && cv >= thr) verify[s] = j + 1;
    }
  }
}

}  // namespace

// x: [S, ldx] rows of kind 0 = fp32, 1 = bf16; lat: [S, r] bf16 or null; w: [d + r] fp32;
// ladder: [n_ladder] thresholds of proposals 2, 3, ... (the last one repeats);
// conf: [S, g] out, cum: [S] running products, verify: [S] proposals to verify (1..g).
TF_API int tf_draft_confidence(const void* x, int x_kind, int ldx, const void* lat, int r, const float* w,
                               const float* ladder, int n_ladder, int j, int g, float* conf, float* cum,
                               int* verify, int S, int d, cudaStream_t st) {
  if (!x || !w || !conf || !cum || !verify || S < 1 || j < 0 || j >= g || (j > 0 && (!ladder || n_ladder < 1))) return -1;
  if (x_kind != 0 && x_kind != 1) return -1;
  tf_launch(draft_confidence_kernel, dim3(S), dim3(256), 0, st, x, x_kind, ldx, (const __nv_bfloat16*)lat,
            lat ? r : 0, w, ladder, n_ladder, j, g, conf, cum, verify, d);
  return (int)cudaGetLastError();
}
