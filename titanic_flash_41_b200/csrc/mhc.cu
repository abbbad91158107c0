// mHC boundary (multi-stream residual with hc_mult = H copies), H <= 4.
//
//   tf_hc_prepare   one CTA per row: the H*(2+H) mixes of the flattened H x d row against `fn`
//                   (fp32 weights), all scaled by rsqrt(mean(x^2) + rms_eps); then
//                   pre_h = sigmoid(m_h*s0 + b_h) + eps, post_h = 2*sigmoid(m_{H+h}*s1 + b_{H+h}),
//                   comb = Sinkhorn(row-softmax + eps) (column step first, then iters-1 row/column
//                   pairs); finally the collapsed input v = sum_h pre_h * x_h (sequential fp32
//                   FMAs, rounded once to bf16) and, optionally, its RMSNorm in f16 / bf16 for the
//                   sublayer's first GEMM.  The coefficients stay in a small per-row record for
//                   tf_hc_post.
//   tf_hc_post      y_c = post_c * a + sum_k comb[k, c] * x_k for the sublayer output a.
// fp32 reference: the model oracle's hc_coefficients / hc_collapse / hc_post
// (reference arithmetic: kernels/core.cu:859-936, fused variant kernels/roce_oneshot_hc.cuh:52-63;
// Rust side src/mhc.rs:946 prepare, :1186 finish).
#include "common.cuh"

namespace {
constexpr int kMaxH = 4;
constexpr int kMaxMix = kMaxH * (2 + kMaxH);     // 24

struct HcCoef {                                    // per row, 32 floats
  float pre[kMaxH], post[kMaxH], comb[kMaxH * kMaxH], pad[8];
};

__global__ void __launch_bounds__(256) hc_prepare_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const float* __restrict__ fn,
                                                         const float* __restrict__ base,
                                                         const float* __restrict__ scale, HcCoef* __restrict__ coef,
                                                         __nv_bfloat16* __restrict__ v_out,
                                                         const __nv_bfloat16* __restrict__ norm_w,
                                                         __half* __restrict__ h16, __nv_bfloat16* __restrict__ hb,
                                                         int H, int d, int iters, float eps, float rms_eps) {
  tf_pdl_sync();
  __shared__ float red[kMaxMix + 1][8];
  __shared__ float mix[kMaxMix + 1];
  __shared__ float s_pre[kMaxH];
  __shared__ float s_vv[8];
  const int r = blockIdx.x, nmix = H * (2 + H), n = H * d;
  const __nv_bfloat16* xr = x + (long)r * n;
  float acc[kMaxMix + 1];
#pragma unroll
  for (int q = 0; q <= kMaxMix; ++q) acc[q] = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) {
    const float a = __bfloat162float(xr[i]);
    acc[kMaxMix] += a * a;
#pragma unroll
    for (int q = 0; q < kMaxMix; ++q)
      if (q < nmix) acc[q] = fmaf(a, fn[(long)q * n + i], acc[q]);
  }
#pragma unroll
  for (int q = 0; q <= kMaxMix; ++q) {
    float t = acc[q];
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if ((threadIdx.x & 31) == 0) red[q][threadIdx.x >> 5] = t;
  }
  __syncthreads();
  if (threadIdx.x <= kMaxMix) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[threadIdx.x][w];
    mix[threadIdx.x] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const float inv = rsqrtf(mix[kMaxMix] / n + rms_eps);
    HcCoef c;
    for (int h = 0; h < H; ++h) {
      c.pre[h] = 1.f / (1.f + expf(-(mix[h] * inv * scale[0] + base[h]))) + eps;
      c.post[h] = 2.f / (1.f + expf(-(mix[H + h] * inv * scale[1] + base[H + h])));
      s_pre[h] = c.pre[h];
    }
    float m[kMaxH][kMaxH];
    for (int i = 0; i < H; ++i) {
      float mx = -1e30f, sum = 0.f;
      for (int j = 0; j < H; ++j) {
        m[i][j] = mix[2 * H + i * H + j] * inv * scale[2] + base[2 * H + i * H + j];
        mx = fmaxf(mx, m[i][j]);
      }
      for (int j = 0; j < H; ++j) {
        m[i][j] = expf(m[i][j] - mx);
        sum += m[i][j];
      }
      for (int j = 0; j < H; ++j) m[i][j] = m[i][j] / sum + eps;
    }
    auto cols = [&]() {
      for (int j = 0; j < H; ++j) {
        float s = 0.f;
        for (int i = 0; i < H; ++i) s += m[i][j];
        for (int i = 0; i < H; ++i) m[i][j] /= (s + eps);
      }
    };
    auto rows = [&]() {
      for (int i = 0; i < H; ++i) {
        float s = 0.f;
        for (int j = 0; j < H; ++j) s += m[i][j];
        for (int j = 0; j < H; ++j) m[i][j] /= (s + eps);
      }
    };
    cols();
    for (int it = 1; it < iters; ++it) {
      rows();
      cols();
    }
    for (int i = 0; i < H; ++i)
      for (int j = 0; j < H; ++j) c.comb[i * kMaxH + j] = m[i][j];
    coef[r] = c;
  }
  __syncthreads();
  // collapse (+ optional RMSNorm of the collapsed row)
  float vv = 0.f;
  for (int i = threadIdx.x; i < d; i += 256) {
    float v = 0.f;
    for (int h = 0; h < H; ++h) v = fmaf(s_pre[h], __bfloat162float(xr[h * d + i]), v);
    const __nv_bfloat16 vb = __float2bfloat16_rn(v);
    v_out[(long)r * d + i] = vb;
    const float vr = __bfloat162float(vb);
    vv += vr * vr;
  }
  if (norm_w == nullptr) return;
#pragma unroll
  for (int o = 16; o; o >>= 1) vv += __shfl_xor_sync(0xffffffffu, vv, o);
  if ((threadIdx.x & 31) == 0) s_vv[threadIdx.x >> 5] = vv;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += s_vv[w];
  const float inv = rsqrtf(tot / d + rms_eps);
  for (int i = threadIdx.x; i < d; i += 256) {
    const float y = __bfloat162float(v_out[(long)r * d + i]) * inv * __bfloat162float(norm_w[i]);
    if (h16) h16[(long)r * d + i] = __float2half(y);
    if (hb) hb[(long)r * d + i] = __float2bfloat16_rn(y);
  }
}

// grid (rows, H)
__global__ void __launch_bounds__(256) hc_post_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ a,
                                                      const HcCoef* __restrict__ coef,
                                                      __nv_bfloat16* __restrict__ y, int H, int d) {
  tf_pdl_sync();
  const int r = blockIdx.x, c = blockIdx.y;
  const HcCoef k = coef[r];
  const __nv_bfloat16* xr = x + (long)r * H * d;
  for (int i = threadIdx.x; i < d; i += 256) {
    float v = k.post[c] * a[(long)r * d + i];
    for (int q = 0; q < H; ++q) v = fmaf(k.comb[q * kMaxH + c], __bfloat162float(xr[q * d + i]), v);
    y[((long)r * H + c) * d + i] = __float2bfloat16_rn(v);
  }
}
}  // namespace

TF_API int tf_hc_coef_bytes() { return (int)sizeof(HcCoef); }

// x [rows, H, d] bf16; fn [H*(2+H), H*d] f32; base [H*(2+H)], scale [3] f32; coef [rows] records;
// v [rows, d] bf16 collapsed input; norm_w (optional) [d] bf16 -> h16 / hb normalised copies
TF_API int tf_hc_prepare(const void* x, const float* fn, const float* base, const float* scale, void* coef, void* v,
                         const void* norm_w, void* h16, void* hb, int rows, int H, int d, int iters, float eps,
                         float rms_eps, cudaStream_t st) {
  if (H < 1 || H > kMaxH) return -1;
  if (rows <= 0) return 0;
  tf_launch(hc_prepare_kernel, dim3(rows), dim3(256), 0, st, (const __nv_bfloat16*)x, fn, base, scale, (HcCoef*)coef, (__nv_bfloat16*)v,
                                          (const __nv_bfloat16*)norm_w, (__half*)h16, (__nv_bfloat16*)hb, H, d, iters,
                                          eps, rms_eps);
  return (int)cudaGetLastError();
}

// y [rows, H, d] bf16 = post * a + comb^T x with a [rows, d] f32 (the reduced sublayer output)
TF_API int tf_hc_post(const void* x, const float* a, const void* coef, void* y, int rows, int H, int d,
                      cudaStream_t st) {
  if (H < 1 || H > kMaxH) return -1;
  if (rows <= 0) return 0;
  tf_launch(hc_post_kernel, dim3(dim3(rows, H)), dim3(256), 0, st, (const __nv_bfloat16*)x, a, (const HcCoef*)coef, (__nv_bfloat16*)y, H, d);
  return (int)cudaGetLastError();
}
