// Glue kernels of the vision tower (ViT): everything between its tensor-core GEMMs.
//
//   tf_vis_bias            y = x + bias (per column)
//   tf_vis_norm            RMSNorm rows, optionally after adding a delta into the residual
//   tf_vis_rope_split      qkv [n, 3*width] -> per-head q, k, v with 2-D rotary embedding: of each head's
//                          32 rotation pairs the first 16 turn with the patch row, the last 16
//                          with the patch column, frequency 10000^(-(c mod 16)/16)
//   tf_vis_softmax         row softmax of attention scores, scaled, over the first n columns
//   tf_vis_swiglu          silu(gate) rounded to bf16, times up
//   tf_vis_unfold          3x3 neighbourhoods (channel, dy, dx order; zero beyond the bottom/right edge)
//   tf_vis_gelu            exact (erf) GELU
//   tf_vis_span            start | feature rows each followed by a newline embedding | end
//   tf_vis_transpose_pad   V [n, 64] of one head -> [128, n_pad] (rows 64.. zero) for the P*V GEMM
// (reference: kernels/vision.cu:7-177, 12 kernels; encoder dataflow src/vision.rs:481 encode).
#include "common.cuh"

namespace {
typedef __nv_bfloat16 B;

__global__ void vis_bias_kernel(const B* x, const B* bias, B* y, long count, int width) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) y[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + __bfloat162float(bias[i % width]));
}

__global__ void __launch_bounds__(256) vis_norm_kernel(B* x, const B* delta, const B* w, B* y, int width, float eps) {
  tf_pdl_sync();
  __shared__ float red[8];
  const long row = blockIdx.x;
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += 256) {
    float v = __bfloat162float(x[row * width + c]);
    if (delta) {
      v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(delta[row * width + c])));
      x[row * width + c] = __float2bfloat16_rn(v);
    }
    s += v * v;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int q = 0; q < 8; ++q) t += red[q];
  const float inv = rsqrtf(t / width + eps);
  for (int c = threadIdx.x; c < width; c += 256)
    y[row * width + c] = __float2bfloat16_rn(__bfloat162float(x[row * width + c]) * inv * __bfloat162float(w[c]));
}

// q, k, v: [heads][n_pad][64]
__global__ void vis_rope_split_kernel(const B* qkv, B* q, B* k, B* v, int n, int n_pad, int grid_w, int heads) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int width = heads * 64;
  if (i >= (long)n * width) return;
  const int row = (int)(i / width), c = (int)(i % width), head = c / 64, half = c % 64;
  const int pair = half % 32;
  const float freq = 1.f / powf(10000.f, (float)(pair % 16) / 16.f);
  const float pos = (float)(pair < 16 ? row / grid_w : row % grid_w);
  float sn, cs;
  sincosf(pos * freq, &sn, &cs);
  const long src = (long)row * 3 * width + head * 64;
  const float q1 = __bfloat162float(qkv[src + pair]), q2 = __bfloat162float(qkv[src + pair + 32]);
  const float k1 = __bfloat162float(qkv[src + width + pair]), k2 = __bfloat162float(qkv[src + width + pair + 32]);
  const long dst = ((long)head * n_pad + row) * 64 + half;
  q[dst] = __float2bfloat16_rn(half < 32 ? q1 * cs - q2 * sn : q2 * cs + q1 * sn);
  k[dst] = __float2bfloat16_rn(half < 32 ? k1 * cs - k2 * sn : k2 * cs + k1 * sn);
  v[dst] = qkv[src + 2 * width + half];
}

// scores [rows, ld] f32 -> probs [rows, ld] bf16 over the first n columns (the rest zero)
__global__ void __launch_bounds__(256) vis_softmax_kernel(const float* s, B* p, int n, int ld, float scale) {
  tf_pdl_sync();
  __shared__ float red[8];
  const long row = blockIdx.x;
  const float* sr = s + row * ld;
  float mx = -1e30f;
  for (int c = threadIdx.x; c < n; c += 256) mx = fmaxf(mx, sr[c] * scale);
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int q = 1; q < 8; ++q) mx = fmaxf(mx, red[q]);
  __syncthreads();
  float sum = 0.f;
  for (int c = threadIdx.x; c < n; c += 256) sum += expf(sr[c] * scale - mx);
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int q = 0; q < 8; ++q) tot += red[q];
  const float inv = 1.f / tot;
  for (int c = threadIdx.x; c < ld; c += 256)
    p[row * ld + c] = __float2bfloat16_rn(c < n ? expf(sr[c] * scale - mx) * inv : 0.f);
}

__global__ void vis_swiglu_kernel(const B* gu, B* y, long count, int inter) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long row = i / inter;
  const int c = (int)(i % inter);
  const float g = __bfloat162float(gu[row * 2 * inter + c]);
  const B act = __float2bfloat16_rn(g / (1.f + expf(-g)));
  y[i] = __float2bfloat16_rn(__bfloat162float(act) * __bfloat162float(gu[row * 2 * inter + inter + c]));
}

__global__ void vis_unfold_kernel(const B* x, B* y, int h, int w, int width, long count) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int cols = width * 9, out_w = (w + 2) / 3;
  const int row = (int)(i / cols), col = (int)(i % cols);
  const int sy = (row / out_w) * 3 + (col % 9) / 3, sx = (row % out_w) * 3 + col % 3;
  y[i] = (sy < h && sx < w) ? x[((long)sy * w + sx) * width + col / 9] : __float2bfloat16_rn(0.f);
}

__global__ void vis_gelu_kernel(const B* x, B* y, long count) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const float v = __bfloat162float(x[i]);
  y[i] = __float2bfloat16_rn((v * 0.5f) * (1.f + erff(v * 0.70710678118654752440f)));
}

__global__ void vis_span_kernel(const B* f, const B* start, const B* newline, const B* end, B* out, int width,
                                int tokens, int d) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)tokens * d) return;
  const int row = (int)(i / d), col = (int)(i % d);
  if (row == 0) out[i] = start[col];
  else if (row + 1 == tokens) out[i] = end[col];
  else {
    const int r = row - 1, x = r % (width + 1), y = r / (width + 1);
    out[i] = x == width ? newline[col] : f[((long)y * width + x) * d + col];
  }
}

// v [n_pad, 64] -> vt [128, n_pad]: vt[c][r] = v[r][c] for c < 64 and r < n, zero elsewhere
__global__ void vis_transpose_pad_kernel(const B* v, B* vt, int n, int n_pad) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 128L * n_pad) return;
  const int c = (int)(i / n_pad), r = (int)(i % n_pad);
  vt[i] = (c < 64 && r < n) ? v[(long)r * 64 + c] : __float2bfloat16_rn(0.f);
}

inline unsigned blocks(long n) { return (unsigned)((n + 255) / 256); }
}  // namespace

TF_API int tf_vis_bias(const void* x, const void* bias, void* y, long count, int width, cudaStream_t st) {
  tf_launch(vis_bias_kernel, dim3(blocks(count)), dim3(256), 0, st, (const B*)x, (const B*)bias, (B*)y, count, width);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_norm(void* x, const void* delta, const void* w, void* y, int rows, int width, float eps,
                       cudaStream_t st) {
  tf_launch(vis_norm_kernel, dim3(rows), dim3(256), 0, st, (B*)x, (const B*)delta, (const B*)w, (B*)y, width, eps);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_rope_split(const void* qkv, void* q, void* k, void* v, int n, int n_pad, int grid_w, int heads,
                             cudaStream_t st) {
  tf_launch(vis_rope_split_kernel, dim3(blocks((long)n * heads * 64)), dim3(256), 0, st, (const B*)qkv, (B*)q, (B*)k, (B*)v, n, n_pad,
                                                                      grid_w, heads);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_softmax(const float* s, void* p, int rows, int n, int ld, float scale, cudaStream_t st) {
  tf_launch(vis_softmax_kernel, dim3(rows), dim3(256), 0, st, s, (B*)p, n, ld, scale);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_swiglu(const void* gu, void* y, long rows, int inter, cudaStream_t st) {
  tf_launch(vis_swiglu_kernel, dim3(blocks(rows * inter)), dim3(256), 0, st, (const B*)gu, (B*)y, rows * inter, inter);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_unfold(const void* x, void* y, int h, int w, int width, cudaStream_t st) {
  const long count = (long)((h + 2) / 3) * ((w + 2) / 3) * width * 9;
  tf_launch(vis_unfold_kernel, dim3(blocks(count)), dim3(256), 0, st, (const B*)x, (B*)y, h, w, width, count);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_gelu(const void* x, void* y, long count, cudaStream_t st) {
  tf_launch(vis_gelu_kernel, dim3(blocks(count)), dim3(256), 0, st, (const B*)x, (B*)y, count);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_span(const void* f, const void* start, const void* newline, const void* end, void* out, int width,
                       int tokens, int d, cudaStream_t st) {
  tf_launch(vis_span_kernel, dim3(blocks((long)tokens * d)), dim3(256), 0, st, (const B*)f, (const B*)start, (const B*)newline,
                                                            (const B*)end, (B*)out, width, tokens, d);
  return (int)cudaGetLastError();
}
TF_API int tf_vis_transpose_pad(const void* v, void* vt, int n, int n_pad, cudaStream_t st) {
  tf_launch(vis_transpose_pad_kernel, dim3(blocks(128L * n_pad)), dim3(256), 0, st, (const B*)v, (B*)vt, n, n_pad);
  return (int)cudaGetLastError();
}
