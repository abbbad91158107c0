// Engram (hashed n-gram embedding memory), device side.
//
//   tf_engram_dequant   packed rows (256 e4m3 values + 8 UE8M0 group scales = 264 B) -> bf16, with
//                       the ownership rule of a row-sharded table: ids outside this rank's
//                       [row_start, row_end) give zero rows, so the sum over ranks is the lookup
//                       (reference: kernels/core.cu:967 ca_engram_dequant).
//   tf_engram_gate      per residual copy h: gate = sigmoid(ssqrt(<rmsnorm(x_h) * qw_h * kw_h,
//                       rmsnorm(key_h)> / sqrt(d))), out_h = x_h + gate * value, where
//                       ssqrt(v) = sign(v) * sqrt(max(|v|, 1e-6)) (reference: kernels/core.cu:952
//                       ca_engram_gate; kv rows hold m keys followed by one value).
// On B200 the whole table shard lives in HBM (25 GB per GPU at 8 ranks for the 2 x 384 M-row
// tables), so the reference's SSD / io_uring row store becomes one gather from device memory.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) engram_dequant_kernel(const uint8_t* __restrict__ table,
                                                             const long long* __restrict__ ids,
                                                             __nv_bfloat16* __restrict__ out, int count,
                                                             long long row_start, long long row_end) {
  tf_pdl_sync();
  const int r = blockIdx.x;
  if (r >= count) return;
  const long long id = ids[r];
  const int i = threadIdx.x;
  float v = 0.f;
  if (id >= row_start && id < row_end) {
    const uint8_t* row = table + (id - row_start) * 264;
    v = e4m3_to_float(row[i]) * ue8m0_to_float(row[256 + i / 32]);
  }
  out[(long)r * 256 + i] = __float2bfloat16_rn(v);
}

// grid (rows, m), 256 threads
__global__ void __launch_bounds__(256) engram_gate_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ kv,
                                                          const __nv_bfloat16* __restrict__ qw,
                                                          const __nv_bfloat16* __restrict__ kw,
                                                          __nv_bfloat16* __restrict__ out, int m, int d, float eps) {
  tf_pdl_sync();
  __shared__ float red[3][8];
  const int r = blockIdx.x, h = blockIdx.y;
  const __nv_bfloat16* xr = x + ((long)r * m + h) * d;
  const __nv_bfloat16* kr = kv + ((long)r * (m + 1) + h) * d;
  const __nv_bfloat16* vr = kv + ((long)r * (m + 1) + m) * d;
  float xx = 0.f, kk = 0.f, dot = 0.f;
  for (int i = threadIdx.x; i < d; i += 256) {
    const float a = __bfloat162float(xr[i]), b = __bfloat162float(kr[i]);
    xx += a * a;
    kk += b * b;
    dot += (a * (__bfloat162float(qw[h * d + i]) * __bfloat162float(kw[h * d + i]))) * b;
  }
  float v[3] = {xx, kk, dot};
#pragma unroll
  for (int q = 0; q < 3; ++q) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v[q] += __shfl_xor_sync(0xffffffffu, v[q], o);
    if ((threadIdx.x & 31) == 0) red[q][threadIdx.x >> 5] = v[q];
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 3; ++q) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[q][w];        // fixed order
    v[q] = t;
  }
  float s = (v[2] * (rsqrtf(v[0] / d + eps) * rsqrtf(v[1] / d + eps))) * rsqrtf((float)d);
  s = copysignf(sqrtf(fmaxf(fabsf(s), 1e-6f)), s);
  const float g = 1.f / (1.f + expf(-s));
  __nv_bfloat16* o = out + ((long)r * m + h) * d;
  for (int i = threadIdx.x; i < d; i += 256)
    o[i] = __float2bfloat16_rn(__bfloat162float(xr[i]) + g * __bfloat162float(vr[i]));
}

}  // namespace

// table: this rank's rows [row_start, row_end) of 264 bytes each; ids [count] int64; out [count, 256] bf16
TF_API int tf_engram_dequant(const void* table, const void* ids, void* out, int count, long row_start, long row_end,
                             cudaStream_t st) {
  if (count <= 0) return 0;
  tf_launch(engram_dequant_kernel, dim3(count), dim3(256), 0, st, (const uint8_t*)table, (const long long*)ids, (__nv_bfloat16*)out, count,
                                               row_start, row_end);
  return (int)cudaGetLastError();
}

// x [rows, m, d], kv [rows, m + 1, d], qw / kw [m, d], out [rows, m, d], all bf16
TF_API int tf_engram_gate(const void* x, const void* kv, const void* qw, const void* kw, void* out, int rows, int m,
                          int d, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  tf_launch(engram_gate_kernel, dim3(dim3(rows, m)), dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)kv,
                                                    (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw,
                                                    (__nv_bfloat16*)out, m, d, eps);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// n-gram hash ids on the device.  A verification step samples its proposal tokens inside the
// captured graph, so the host cannot hash them; this kernel reads the tokens of the launch where
// the embedding reads them.  One thread per (row, table); same arithmetic as the host
// (models/engram.py HashHistory.prepare; reference: src/engram.rs hash history): compressed token
// ids, rolling = c0*m0 ^ c1*m1 ^ ... in 64 bits, id = rolling mod prime + offset per (order, head).
// `recent` holds, per row, the ngram-1 tokens before the row's conversation block, newest first.
namespace {
constexpr int kMaxNgram = 8;

__global__ void engram_hash_kernel(const int* __restrict__ tokens, const int* __restrict__ pos,
                                   const int* __restrict__ first_row, const int* __restrict__ recent,
                                   const long long* __restrict__ token_map, int vocab,
                                   const unsigned long long* __restrict__ mult,
                                   const unsigned long long* __restrict__ primes,
                                   const unsigned long long* __restrict__ offsets, long long* __restrict__ out,
                                   int T, long out_table_stride, int tables, int ngram, int heads, int pad_token,
                                   int image_token, TfStatusWord* st) {
  tf_pdl_sync();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * tables) return;
  const int i = idx / tables, t = idx % tables;
  const int in_block = i - first_row[i];
  const unsigned long long pad = (unsigned long long)token_map[pad_token];
  unsigned long long comp[kMaxNgram];
  bool blocked = false;
  for (int back = 0; back < ngram; ++back) {
    if (pos[i] < back) blocked = true;
    const int tok = back <= in_block ? tokens[i - back] : recent[i * (ngram - 1) + (back - in_block - 1)];
    if (tok == image_token) {
      blocked = true;
    } else if (tok < 0 || tok >= vocab) {
      tf_report(st, TF_BAD_INDEX, 140, i, tok);
      blocked = true;
    }
    comp[back] = blocked ? pad : (unsigned long long)token_map[tok];
  }
  const int ids = (ngram - 1) * heads;
  long long* o = out + (long)t * out_table_stride + (long)i * ids;
  unsigned long long rolling = comp[0] * mult[t * ngram];
  for (int back = 1; back < ngram; ++back) {
    rolling ^= comp[back] * mult[t * ngram + back];
    for (int head = 0; head < heads; ++head) {
      const int h = (back - 1) * heads + head;
      o[h] = (long long)(rolling % primes[t * ids + h] + offsets[t * ids + h]);
    }
  }
}
}  // namespace

// tokens / pos / first_row [T] int32; recent [T, ngram-1] int32; token_map [vocab] int64;
// mult [tables, ngram], primes / offsets [tables, (ngram-1)*heads] uint64; out [tables][T rows at
// out_table_stride elements per table][(ngram-1)*heads] int64
TF_API int tf_engram_hash(const int* tokens, const int* pos, const int* first_row, const int* recent,
                          const void* token_map, int vocab, const void* mult, const void* primes, const void* offsets,
                          void* out, int T, long out_table_stride, int tables, int ngram, int heads, int pad_token,
                          int image_token, void* status, cudaStream_t st) {
  if (T <= 0 || ngram < 2 || ngram > kMaxNgram || pad_token < 0 || pad_token >= vocab) return -1;
  const int n = T * tables;
  tf_launch(engram_hash_kernel, dim3((n + 127) / 128), dim3(128), 0, st, tokens, pos, first_row, recent, (const long long*)token_map, vocab, (const unsigned long long*)mult,
      (const unsigned long long*)primes, (const unsigned long long*)offsets, (long long*)out, T, out_table_stride,
      tables, ngram, heads, pad_token, image_token, (TfStatusWord*)status);
  return (int)cudaGetLastError();
}
