// Sublayer boundary of decode rows with its neighbours folded in: one launch does
//   [combine]  delta[r, :] = sum_j wts[r, j] * y_pair[r * topk + j, :] (experts of this rank, in
//              slot order) + shared[r, :]                 -- what tf_moe_combine would have written
//   [residual] x[r, :] = bf16(x[r, :] + delta[r, :])
//   [norm]     v = bf16(x * rsqrt(mean(x^2) + eps) * w)   -> f16 and / or bf16 copies
//   [mx8]      the MXFP8 form of v (e4m3 + one UE8M0 scale per 32) for the block-scaled expert GEMV
// The arithmetic is that of tf_moe_combine + tf_add_norm + tf_quant_rows_mx8 run one after the
// other (same order of additions, same roundings), so results are bit-identical; what goes away
// is two launches and two dependent-launch gaps per layer of a captured decode step.
//
// Reference behaviour: the FFN sum with the shared expert (kernels/ffn_sum_shared.cuh:7-33), the
// residual RMSNorm (kernels/core.cu:851 ca_rms_bf16) and the MXFP8 K32 activation quantisation of
// the MoE front-end (kernels/moe_frontend.cuh).
#include "rownorm.cuh"

namespace {

struct FusedNormParams {
  __nv_bfloat16* x;            // [T, d] residual stream, updated in place
  const float* delta;          // [T, d] fp32 or null
  const float* y_pair;         // combine source (null: use delta)
  const int* ids;
  const float* wts;
  const float* shared_y;       // may be null
  int topk, e_lo, e_hi;
  const __nv_bfloat16* w;      // [d]
  __half* h16;
  __nv_bfloat16* hb;
  uint8_t* x8;                 // [T, d] e4m3 or null
  uint8_t* x8s;                // [T, d / 32] UE8M0
  int d;
  float eps;
};

__global__ void __launch_bounds__(1024) fused_norm_kernel(const FusedNormParams p) {
  tf_pdl_sync();
  extern __shared__ float row[];            // d floats
  __shared__ float scratch[32];
  const int r = blockIdx.x, d = p.d;
  __nv_bfloat16* xr = p.x + (long)r * d;
  float ss = 0.f;
  // four consecutive elements per thread and step: 16-byte loads of the expert outputs, all
  // independent, so a row's 7 x 16 KB of inputs are in flight at once
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    const uint2 xraw = *reinterpret_cast<const uint2*>(xr + i);
    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xraw);
    const float2 x01 = __bfloat1622float2(xb[0]), x23 = __bfloat1622float2(xb[1]);
    float v[4] = {x01.x, x01.y, x23.x, x23.y};
    bool add = false;
    float dv[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.y_pair) {
      for (int j = 0; j < p.topk; ++j) {
        const int e = p.ids[r * p.topk + j];
        if (e >= p.e_lo && e < p.e_hi) {
          const float wj = p.wts[r * p.topk + j];
          const float4 y = *reinterpret_cast<const float4*>(p.y_pair + (long)(r * p.topk + j) * d + i);
          dv[0] = fmaf(wj, y.x, dv[0]);
          dv[1] = fmaf(wj, y.y, dv[1]);
          dv[2] = fmaf(wj, y.z, dv[2]);
          dv[3] = fmaf(wj, y.w, dv[3]);
        }
      }
      if (p.shared_y) {
        const float4 y = *reinterpret_cast<const float4*>(p.shared_y + (long)r * d + i);
        dv[0] += y.x; dv[1] += y.y; dv[2] += y.z; dv[3] += y.w;
      }
      add = true;
    } else if (p.delta) {
      const float4 y = *reinterpret_cast<const float4*>(p.delta + (long)r * d + i);
      dv[0] = y.x; dv[1] = y.y; dv[2] = y.z; dv[3] = y.w;
      add = true;
    }
    if (add) {
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = bf16_round(v[c] + dv[c]);
      __nv_bfloat162 o[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
      *reinterpret_cast<uint2*>(xr + i) = *reinterpret_cast<uint2*>(o);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      row[i + c] = v[c];
      ss += v[c] * v[c];
    }
  }
  ss = block_sum(ss, scratch);
  row_norm_store(row, d, ss, p.eps, p.w, p.h16, p.hb, p.x8, p.x8s, r);
}

}  // namespace

// Exactly one of (delta) / (y_pair, ids, wts[, shared_y]) / neither feeds the residual add.
TF_API int tf_add_norm_fused(void* x, const void* delta, const void* y_pair, const int* ids, const void* wts,
                             const void* shared_y, int topk, int e_lo, int e_hi, const void* w, void* h16, void* hb,
                             void* x8, void* x8s, int T, int d, float eps, cudaStream_t st) {
  if (d % 128 || T <= 0 || (y_pair && (!ids || !wts || topk <= 0)) || (x8 && !x8s)) return -1;
  FusedNormParams p;
  p.x = (__nv_bfloat16*)x; p.delta = (const float*)delta; p.y_pair = (const float*)y_pair; p.ids = ids;
  p.wts = (const float*)wts; p.shared_y = (const float*)shared_y; p.topk = topk; p.e_lo = e_lo; p.e_hi = e_hi;
  p.w = (const __nv_bfloat16*)w; p.h16 = (__half*)h16; p.hb = (__nv_bfloat16*)hb; p.x8 = (uint8_t*)x8;
  p.x8s = (uint8_t*)x8s; p.d = d; p.eps = eps;
  tf_launch(fused_norm_kernel, dim3(T), dim3(d >= 4096 ? 1024 : 256), d * sizeof(float), st, p);
  return (int)cudaGetLastError();
}
