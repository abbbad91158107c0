// Kernels around the tensor-core GEMMs for large row counts (prefill chunks):
//   * row-wise FP8 quantisation with one fp32 scale per 128 (activations entering an FP8 GEMM)
//   * clamped SwiGLU (+ optional FP8 quantisation) over a [rows, 2I] GEMM output
//   * routed-expert bookkeeping without a host round trip: histogram of (token, slot) pairs per
//     local expert, 128-row-padded segment offsets, per-M-tile expert table, destination row of
//     every pair
//   * gather + quantise token rows into the expert-sorted, padded activation matrix
//   * MXFP4 (e2m1 + UE8M0/32) expert weights re-expressed as FP8 with one power-of-two scale per
//     128x128 block, the operand format of the block-scaled tcgen05 GEMM
//   * weighted combine of the expert outputs in fixed top-k order (+ shared expert)
// Reference counterparts: kernels/moe_frontend.cuh (route grouping tables), kernels/
// shared_swiglu_quant.cuh, kernels/ffn_sum_shared.cuh, src/expert_packing.rs (weight repack).
#include "common.cuh"

namespace {

// one warp per (row, 128-block): x f16/bf16/f32 -> e4m3 + scale
template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
// four consecutive elements in one load (the address is a multiple of four elements)
template <typename T>
__device__ __forceinline__ void ld4(const T* p, float v[4]);
template <> __device__ __forceinline__ void ld4<__half>(const __half* p, float v[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <> __device__ __forceinline__ void ld4<__nv_bfloat16>(const __nv_bfloat16* p, float v[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <> __device__ __forceinline__ void ld4<float>(const float* p, float v[4]) {
  const float4 raw = *reinterpret_cast<const float4*>(p);
  v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
}

template <typename T>
__global__ void quant_rows_kernel(const T* __restrict__ x, long ldx, const int* __restrict__ row_src,
                                  int src_div, const int* __restrict__ row_dst, uint8_t* __restrict__ q,
                                  float* __restrict__ s, int rows, int K) {
  tf_pdl_sync();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_per_row = K / 128;
  const long item = (long)blockIdx.x * warps + warp;
  if (item >= (long)rows * kb_per_row) return;
  const int r = (int)(item / kb_per_row), kb = (int)(item % kb_per_row);
  const long src = row_src ? row_src[r] / src_div : (src_div > 1 ? r / src_div : r);
  const long dst = row_dst ? row_dst[r] : r;
  if (dst < 0) return;
  const T* xp = x + src * ldx + kb * 128 + lane * 4;
  float v[4], am = 0.f;
  ld4<T>(xp, v);
#pragma unroll
  for (int j = 0; j < 4; ++j) am = fmaxf(am, fabsf(v[j]));
  am = warp_max(am);
  const float sc = fmaxf(am, 1e-12f) / 448.f;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) packed |= (uint32_t)float_to_e4m3(v[j] / sc) << (8 * j);
  reinterpret_cast<uint32_t*>(q + dst * K + kb * 128)[lane] = packed;
  if (lane == 0) s[dst * kb_per_row + kb] = sc;
}

// y [rows, 2I] (gate | up halves) -> act: f16 [rows, I] and/or fp8 + scales
template <typename T>
__global__ void swiglu_rows_kernel(const T* __restrict__ y, long ldy, __half* __restrict__ out16, long ldo,
                                   uint8_t* __restrict__ q, float* __restrict__ s, int rows, int I, float limit,
                                   const int* __restrict__ n_rows_dev) {
  tf_pdl_sync();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_per_row = I / 128;
  const long item = (long)blockIdx.x * warps + warp;
  if (n_rows_dev) rows = min(rows, *n_rows_dev);
  if (item >= (long)rows * kb_per_row) return;
  const int r = (int)(item / kb_per_row), kb = (int)(item % kb_per_row);
  const T* g = y + (long)r * ldy + kb * 128 + lane * 4;
  const T* u = g + I;
  float v[4], am = 0.f, gv[4], uv[4];
  ld4<T>(g, gv);
  ld4<T>(u, uv);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float gate = gv[j], up = uv[j];
    if (limit > 0.f) {
      gate = fminf(gate, limit);
      up = fminf(fmaxf(up, -limit), limit);
    }
    v[j] = __half2float(__float2half(gate / (1.f + __expf(-gate)) * up));
    am = fmaxf(am, fabsf(v[j]));
  }
  if (out16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) out16[(long)r * ldo + kb * 128 + lane * 4 + j] = __float2half(v[j]);
  }
  if (q) {
    am = warp_max(am);
    const float sc = fmaxf(am, 1e-12f) / 448.f;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= (uint32_t)float_to_e4m3(v[j] / sc) << (8 * j);
    reinterpret_cast<uint32_t*>(q + (long)r * I + kb * 128)[lane] = packed;
    if (lane == 0) s[(long)r * kb_per_row + kb] = sc;
  }
}

// ---- routed-expert bookkeeping ------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_pairs, int e_lo, int El, int* counts) {
  tf_pdl_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = ids[i] - e_lo;
  if (e >= 0 && e < El) atomicAdd(&counts[e], 1);
}
// single CTA: padded offsets, tile table, cursors reset.  tile_expert has room for max_tiles ints.
__global__ void moe_offsets_kernel(int* counts, int El, int* offsets, int* cursor, int* tile_expert,
                                   int max_tiles, int* num_tiles, int* padded_rows) {
  tf_pdl_sync();
  if (threadIdx.x == 0) {
    int off = 0, t = 0;
    for (int e = 0; e < El; ++e) {
      offsets[e] = off;
      cursor[e] = 0;
      const int tiles = (counts[e] + 127) / 128;
      for (int j = 0; j < tiles && t < max_tiles; ++j) tile_expert[t++] = e;
      off += tiles * 128;
      counts[e] = 0;            // ready for the next launch
    }
    offsets[El] = off;
    *num_tiles = t;
    *padded_rows = off;
  }
}
__global__ void moe_place_kernel(const int* __restrict__ ids, int n_pairs, int e_lo, int El,
                                 const int* __restrict__ offsets, int* cursor, int* pair_dst) {
  tf_pdl_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = ids[i] - e_lo;
  pair_dst[i] = (e >= 0 && e < El) ? offsets[e] + atomicAdd(&cursor[e], 1) : -1;
}

// ---- MXFP4 -> FP8 with one power-of-two scale per 128x128 block -----------------------------
// grid (K/128, N/128, experts), 128 threads.  A 32-input group whose
// UE8M0 scale is 2^-shift of the block's largest one turns into e4m3 through a table of the eight
// e2m1 magnitudes times 2^-shift (built per CTA with the same rounding as a direct conversion):
// one byte-permute per four weights, the sign bits moved from nibble to byte positions.
__device__ __forceinline__ uint32_t e2m1x4_signs_to_bytes(uint32_t half16) {
  const uint32_t s = half16 & 0x8888u;                               // sign bits at 3, 7, 11, 15
  const uint32_t z = (s & 0x00ffu) | ((s & 0xff00u) << 8);           // ... at 3, 7, 19, 23
  return ((z & 0x00080008u) << 4) | ((z & 0x00800080u) << 8);        // ... at 7, 15, 23, 31
}
__global__ void __launch_bounds__(128)
mxfp4_to_fp8_block_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ sc,
                          uint8_t* __restrict__ out, float* __restrict__ out_s, int N, int K,
                          long out_expert_stride, int out_row0, int out_N) {
  tf_pdl_sync();
  __shared__ int smax;
  __shared__ uint2 lut[16];                // [shift]: bytes 0..7 = e4m3 of magnitude code 0..7 times 2^-shift
  const int kb = blockIdx.x, nb = blockIdx.y, e = blockIdx.z, t = threadIdx.x;
  // four lanes share a row (one 32-input group = 16 packed bytes each): a warp reads 8 rows x 64
  // contiguous bytes and writes 8 rows x 128 contiguous bytes per step; four steps cover 128 rows
  const int g = t & 3, r0 = t >> 2;
  const long row0 = (long)e * N + nb * 128;
  if (t == 0) smax = 0;
  reinterpret_cast<uint8_t*>(lut)[t] = float_to_e4m3(e2m1_to_float(t & 7) * exp2f((float)-(t >> 3)));
  __syncthreads();
  int c[4], mx = 0;
  uint4 pk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long row = row0 + r0 + 32 * i;
    c[i] = sc[row * (K / 32) + kb * 4 + g];
    pk[i] = *reinterpret_cast<const uint4*>(w + row * (K / 2) + kb * 64 + g * 16);
    mx = max(mx, c[i]);
  }
  mx = __reduce_max_sync(0xffffffffu, mx);
  if ((t & 31) == 0) atomicMax(&smax, mx);
  __syncthreads();
  const int top = smax;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint2 L = lut[min(top - c[i], 15)];       // from 2^-15 on every magnitude rounds to zero
    const uint32_t words[4] = {pk[i].x, pk[i].y, pk[i].z, pk[i].w};
    uint32_t o[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t lo16 = words[q] & 0xffffu, hi16 = words[q] >> 16;
      o[2 * q] = __byte_perm(L.x, L.y, lo16 & 0x7777u) | e2m1x4_signs_to_bytes(lo16);
      o[2 * q + 1] = __byte_perm(L.x, L.y, hi16 & 0x7777u) | e2m1x4_signs_to_bytes(hi16);
    }
    uint8_t* orow = out + (long)e * out_expert_stride + ((long)out_row0 + nb * 128 + r0 + 32 * i) * K + kb * 128;
    uint4* dst = reinterpret_cast<uint4*>(orow + g * 32);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  if (t == 0) {
    const long srow_o = ((long)e * out_N + out_row0) / 128 + nb;
    out_s[srow_o * (K / 128) + kb] = ue8m0_to_float((uint8_t)top);
  }
}

// out[t,:] = sum_j wts[t,j] * y[pair_dst[t*k+j],:] (fixed j order) + shared[t,:]
template <typename T, typename O>
__global__ void moe_combine_perm_kernel(const T* __restrict__ y, long ldy, const int* __restrict__ pair_dst,
                                        const float* __restrict__ wts, const float* __restrict__ shared_y,
                                        O* __restrict__ out, int d, int topk) {
  tf_pdl_sync();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < topk; ++j) {
      const int dst = pair_dst[t * topk + j];
      if (dst >= 0) acc = fmaf(wts[t * topk + j], ldf<T>(y + (long)dst * ldy + i), acc);
    }
    if (shared_y) acc += shared_y[(long)t * d + i];
    stf(out + (long)t * d + i, acc);
  }
}

// The same sum for bf16 expert outputs, eight columns per thread (16-byte loads; d and ldy multiples
// of 8, 16-byte aligned rows): same order of additions per element.
template <typename O>
__global__ void __launch_bounds__(256) moe_combine_perm_vec_kernel(const __nv_bfloat16* __restrict__ y, long ldy,
                                                                   const int* __restrict__ pair_dst,
                                                                   const float* __restrict__ wts,
                                                                   const float* __restrict__ shared_y,
                                                                   O* __restrict__ out, int d, int topk) {
  tf_pdl_sync();
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = 0.f;
    for (int j = 0; j < topk; ++j) {
      const int dst = pair_dst[t * topk + j];
      if (dst < 0) continue;
      const float w = wts[t * topk + j];
      const uint4 raw = *reinterpret_cast<const uint4*>(y + (long)dst * ldy + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = __bfloat1622float2(h[c]);
        acc[2 * c] = fmaf(w, f.x, acc[2 * c]);
        acc[2 * c + 1] = fmaf(w, f.y, acc[2 * c + 1]);
      }
    }
    if (shared_y) {
      const float4 a = *reinterpret_cast<const float4*>(shared_y + (long)t * d + i);
      const float4 b = *reinterpret_cast<const float4*>(shared_y + (long)t * d + i + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    if (sizeof(O) == 4) {
      float4* o = reinterpret_cast<float4*>(out + (long)t * d + i);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      __nv_bfloat162 hh[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) hh[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
      *reinterpret_cast<uint4*>(out + (long)t * d + i) = *reinterpret_cast<uint4*>(hh);
    }
  }
}

// out[i] = sum over w (in order) of slices[w * stride + i] (bf16) + extra[i], for i < n: the owner of
// a row slice sums the partial outputs every rank sent for it, in rank order, in fp32
__global__ void sum_slices_kernel(const __nv_bfloat16* __restrict__ slices, int world, long stride,
                                  const float* __restrict__ extra, float* __restrict__ out, long n) {
  tf_pdl_sync();
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int w = 0; w < world; ++w) {
    const uint4 raw = *reinterpret_cast<const uint4*>(slices + (long)w * stride + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  if (extra) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += extra[i + j];
  }
  *reinterpret_cast<float4*>(out + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  *reinterpret_cast<float4*>(out + i + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

}  // namespace

// x_kind: 0 f32, 1 f16, 2 bf16.  row_src/row_dst optional (gather / scatter); src row = row_src[r] / src_div.
TF_API int tf_quant_rows(const void* x, int x_kind, long ldx, const int* row_src, int src_div,
                         const int* row_dst, void* q, float* s, int rows, int K, cudaStream_t st) {
  if (K % 128 || rows <= 0) return rows <= 0 ? 0 : -1;
  if (ldx % 4 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;      // rows are read four elements at a time
  const long items = (long)rows * (K / 128);
  const unsigned grid = (unsigned)((items + 7) / 8);
  if (src_div < 1) src_div = 1;
  if (x_kind == 0) tf_launch(quant_rows_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)x, ldx, row_src, src_div, row_dst, (uint8_t*)q, s, rows, K);
  else if (x_kind == 1) tf_launch(quant_rows_kernel<__half>, dim3(grid), dim3(256), 0, st, (const __half*)x, ldx, row_src, src_div, row_dst, (uint8_t*)q, s, rows, K);
  else tf_launch(quant_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, ldx, row_src, src_div, row_dst, (uint8_t*)q, s, rows, K);
  return (int)cudaGetLastError();
}

TF_API int tf_swiglu_rows(const void* y, int y_kind, long ldy, void* out16, long ldo, void* q, float* s,
                          int rows, int I, float limit, const int* n_rows_dev, cudaStream_t st) {
  if (I % 128 || rows <= 0) return rows <= 0 ? 0 : -1;
  if (ldy % 4 || (reinterpret_cast<uintptr_t>(y) & 15)) return -1;      // rows are read four elements at a time
  const long items = (long)rows * (I / 128);
  const unsigned grid = (unsigned)((items + 7) / 8);
  if (y_kind == 0) tf_launch(swiglu_rows_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)y, ldy, (__half*)out16, ldo, (uint8_t*)q, s, rows, I, limit, n_rows_dev);
  else if (y_kind == 2) tf_launch(swiglu_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)y, ldy, (__half*)out16, ldo, (uint8_t*)q, s, rows, I, limit, n_rows_dev);
  else return -1;
  return (int)cudaGetLastError();
}

// counts must be zero on entry (it is left zeroed).  tile_expert capacity = max_tiles.
TF_API int tf_moe_plan(const int* ids, int n_pairs, int e_lo, int El, int* counts, int* offsets, int* cursor,
                       int* tile_expert, int max_tiles, int* num_tiles, int* padded_rows, int* pair_dst,
                       cudaStream_t st) {
  const unsigned grid = (unsigned)((n_pairs + 255) / 256);
  tf_launch(moe_count_kernel, dim3(grid), dim3(256), 0, st, ids, n_pairs, e_lo, El, counts);
  tf_launch(moe_offsets_kernel, dim3(1), dim3(32), 0, st, counts, El, offsets, cursor, tile_expert, max_tiles, num_tiles, padded_rows);
  tf_launch(moe_place_kernel, dim3(grid), dim3(256), 0, st, ids, n_pairs, e_lo, El, offsets, cursor, pair_dst);
  return (int)cudaGetLastError();
}

// w [E, N, K/2], sc [E, N, K/32] -> out rows [out_row0, out_row0+N) of every expert's [out_N, K] fp8 matrix
TF_API int tf_mxfp4_to_fp8_block(const void* w, const void* sc, void* out, float* out_s, int E, int N, int K,
                                 int out_row0, int out_N, cudaStream_t st) {
  if (N % 128 || K % 128 || out_row0 % 128 || out_N % 128) return -1;
  dim3 grid(K / 128, N / 128, E);
  tf_launch(mxfp4_to_fp8_block_kernel, dim3(grid), dim3(128), 0, st, (const uint8_t*)w, (const uint8_t*)sc, (uint8_t*)out, out_s,
                                                  N, K, (long)out_N * K, out_row0, out_N);
  return (int)cudaGetLastError();
}

// out_kind: 0 = fp32, 2 = bf16
TF_API int tf_moe_combine_perm(const void* y, int y_kind, long ldy, const int* pair_dst, const float* wts,
                               const float* shared_y, void* out, int out_kind, int T, int d, int topk,
                               cudaStream_t st) {
  if (T <= 0) return 0;
  if (!y || !pair_dst || !wts || !out) return -1;
  const bool vec = y_kind == 2 && d % 8 == 0 && ldy % 8 == 0 && !(reinterpret_cast<uintptr_t>(y) & 15) &&
                   !(reinterpret_cast<uintptr_t>(out) & 15) && !(shared_y && (reinterpret_cast<uintptr_t>(shared_y) & 15));
  if (vec && out_kind == 0) tf_launch(moe_combine_perm_vec_kernel<float>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)y, ldy, pair_dst, wts, shared_y, (float*)out, d, topk);
  else if (vec && out_kind == 2) tf_launch(moe_combine_perm_vec_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)y, ldy, pair_dst, wts, shared_y, (__nv_bfloat16*)out, d, topk);
  else if (y_kind == 0 && out_kind == 0) tf_launch(moe_combine_perm_kernel<float, float>, dim3(T), dim3(256), 0, st, (const float*)y, ldy, pair_dst, wts, shared_y, (float*)out, d, topk);
  else if (y_kind == 2 && out_kind == 0) tf_launch(moe_combine_perm_kernel<__nv_bfloat16, float>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)y, ldy, pair_dst, wts, shared_y, (float*)out, d, topk);
  else if (y_kind == 2 && out_kind == 2) tf_launch(moe_combine_perm_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)y, ldy, pair_dst, wts, shared_y, (__nv_bfloat16*)out, d, topk);
  else return -1;
  return (int)cudaGetLastError();
}

// out[i] = sum_w slices[w][i] (bf16, fixed order w = 0..world-1, fp32 accumulation) + extra[i] (fp32, optional)
// for i < n; `stride` = elements between consecutive slices.  n, stride multiples of 8; 16-byte aligned.
TF_API int tf_sum_slices(const void* slices, int world, long stride, const float* extra, float* out, long n,
                         cudaStream_t st) {
  if (n <= 0) return 0;
  if (!slices || !out || world < 1 || n % 8 || stride % 8 || (reinterpret_cast<uintptr_t>(slices) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (extra && (reinterpret_cast<uintptr_t>(extra) & 15)))
    return -1;
  const long threads = n / 8;
  tf_launch(sum_slices_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)slices, world, stride, extra,
                                                                        out, n);
  return (int)cudaGetLastError();
}
