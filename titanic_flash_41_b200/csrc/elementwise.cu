// Row-wise kernels around the GEMMs: embedding gather, residual + RMSNorm (+FP8 quant),
// attention pre-processing (RoPE, KV norm/quant/store, compressor pooling, index keys),
// router + expert grouping, expert combine.  One CTA per row unless noted.
//
// Reference arithmetic restated here: RMSNorm kernels/core.cu:851-857; RoPE table
// kernels/core.cu:980-999; K store runtime/kernels/kv-v41-v1/kv_store.cu:33-150 (fp32 norm ->
// bf16 -> RoPE tail in fp32 -> bf16 -> e4m3 + UE8M0 per 32); gated pooling
// kernels/core.cu:944-950 generalised from pairs to groups of `ratio`; router
// kernels/moe_frontend.cuh:27-130; ordered route sum kernels/ffn_sum_shared.cuh:7-33.
#include "common.cuh"
#include "router.cuh"

namespace {

// --------------------------------------------------------------------------- embedding
__global__ void embed_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int d, int vocab, TfStatusWord* st) {
  tf_pdl_sync();
  const int r = blockIdx.x;
  int tok = tokens[r];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) tf_report(st, TF_BAD_INDEX, 1, r, tok);
    tok = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (long)tok * d);
  uint4* dst = reinterpret_cast<uint4*>(out + (long)r * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

// --------------------------------------------------------------------------- residual + norm
// x (bf16 residual stream) += delta (optional, f32 or bf16); then h = rmsnorm(x) * w written as
// f16 (decode GEMMs), bf16, and/or FP8 e4m3 with one fp32 scale per 128 along K (tensor-core
// GEMMs).  `sumsq_out` optionally receives the row's mean square.
__global__ void add_norm_kernel(__nv_bfloat16* __restrict__ x, const void* __restrict__ delta,
                                int delta_kind, int ldd, const __nv_bfloat16* __restrict__ w,
                                __half* __restrict__ h16, __nv_bfloat16* __restrict__ hb,
                                uint8_t* __restrict__ q8, float* __restrict__ qs, int d, float eps) {
  tf_pdl_sync();
  extern __shared__ float row[];            // d floats
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  __nv_bfloat16* xr = x + (long)r * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = __bfloat162float(xr[i]);
    if (delta) {
      float dv = delta_kind == 0 ? reinterpret_cast<const float*>(delta)[(long)r * ldd + i]
                                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(delta)[(long)r * ldd + i]);
      v = bf16_round(v + dv);
      xr[i] = __float2bfloat16(v);
    }
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = bf16_round(row[i] * inv * __bfloat162float(w[i]));
    row[i] = v;
    if (h16) h16[(long)r * d + i] = __float2half(v);
    if (hb) hb[(long)r * d + i] = __float2bfloat16(v);
  }
  if (q8) {
    __syncthreads();
    // one warp per 128-wide block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = warp; b < d / 128; b += nw) {
      float v[4], am = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = row[b * 128 + lane * 4 + j];
        am = fmaxf(am, fabsf(v[j]));
      }
      am = warp_max(am);
      const float s = fmaxf(am, 1e-12f) / 448.f;
      uint32_t packed = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) packed |= (uint32_t)float_to_e4m3(v[j] / s) << (8 * j);
      reinterpret_cast<uint32_t*>(q8 + (long)r * d + b * 128)[lane] = packed;
      if (lane == 0) qs[(long)r * (d / 128) + b] = s;
    }
  }
}

// --------------------------------------------------------------------------- attention prep
// The compressor inputs of an open group wait in a ring addressed by absolute position with
// at least `ratio + kCarrySpan` slots per conversation: a speculative row up to kCarrySpan positions
// past the committed length can then never overwrite a slot that a later, shorter re-run still needs.
// (Sources with different ratios may share one allocation sized for the largest: `carry_slots`.)
constexpr int kCarrySpan = 32;

struct PrepParams {
  const void* P;        // fused projection output [T, ldp]; kind 0 = f32, 1 = bf16
  int p_kind, ldp;
  int T;
  const int* pos;       // [T] absolute position
  const int* region;    // [T] conversation slot
  const int* first_row; // [T] first row of this row's conversation in the launch
  const int* last_pos;  // [T] last position of this row's conversation in the launch
  int Hl, Dh, rope_dim;
  const float* freqs;   // [rope_dim/2]
  const float* cfreqs;  // compressed-entry frequencies
  const __nv_bfloat16* kv_norm_w;
  float eps;
  // outputs
  __nv_bfloat16* q_out; // [T, Hl, Dh]
  uint8_t* win;         // window ring base for this layer: [regions][ring][Dh + Dh/32]
  long win_region_stride;
  int ring;
  int win_row, comp_row, key_row;   // row strides in bytes
  // column offsets inside P
  int off_q, off_kv, off_cv, off_cg, off_iq, off_iw;   // -1 = absent
  // compressor (source layers)
  int ratio, Di, Hi;
  const __nv_bfloat16* comp_norm_w;
  float* carry;         // [regions][carry_slots][2*(Dh+Di)]
  int carry_slots;
  uint8_t* comp;        // [regions][maxC][Dh/2 + Dh/16]
  uint8_t* keys;        // [regions][maxC][Di/2 + Di/32]
  int maxC;
  __nv_bfloat16* iq_out; // [T, Hi, Di]
  float* iw_out;         // [T, Hi]
  TfStatusWord* st;
};

// sin/cos of pos * freq.  The product (fp32, as the reference's frequency table defines the angle)
// is reduced to [0, 2*pi) in double before the fp32 sincos, which keeps the fast path even at
// positions near a million without changing the angle.
__device__ __forceinline__ void rope_sincos(int pos, float freq, float* sn, float* cs) {
  const float ang = (float)pos * freq;
  const double two_pi = 6.283185307179586476925286766559;
  const double red = (double)ang - two_pi * floor((double)ang / two_pi);
  sincosf((float)red, sn, cs);
}

__device__ __forceinline__ float ldp(const PrepParams& p, long row, int col) {
  return p.p_kind == 0 ? reinterpret_cast<const float*>(p.P)[row * p.ldp + col]
                       : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.P)[row * p.ldp + col]);
}

// encode Dh values (shared memory, already bf16-rounded) as a V41 window row
__device__ void store_v41(const float* v, uint8_t* dst, int D) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int b = warp; b < D / 32; b += nw) {
    float x = v[b * 32 + lane];
    float am = warp_max(fabsf(x));
    uint8_t code = ue8m0_ceil(am / 448.f);
    float s = ue8m0_to_float(code);
    dst[b * 32 + lane] = float_to_e4m3(x / s);
    if (lane == 0) dst[D + b] = code;
  }
}
// encode D values as a V41-FP4 compressed row: packed e2m1 + one e4m3 scale per 16
__device__ void store_v41fp4(const float* v, uint8_t* dst, int D) {
  for (int b = threadIdx.x; b < D / 16; b += blockDim.x) {
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) am = fmaxf(am, fabsf(v[b * 16 + j]));
    uint8_t sc = float_to_e4m3(fmaxf(am / 6.f, 0.015625f));
    float s = e4m3_to_float(sc);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t lo = float_to_e2m1(v[b * 16 + 2 * j] / s), hi = float_to_e2m1(v[b * 16 + 2 * j + 1] / s);
      dst[b * 8 + j] = (uint8_t)(lo | (hi << 4));
    }
    dst[D / 2 + b] = sc;
  }
}
// encode Di values as an index key: packed e2m1 + one UE8M0 per 32
__device__ void store_index_key(const float* v, uint8_t* dst, int D) {
  for (int b = threadIdx.x; b < D / 32; b += blockDim.x) {
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) am = fmaxf(am, fabsf(v[b * 32 + j]));
    uint8_t code = (uint8_t)min((int)ue8m0_ceil(am / 6.f), 247);
    float s = ue8m0_to_float(code);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t lo = float_to_e2m1(v[b * 32 + 2 * j] / s), hi = float_to_e2m1(v[b * 32 + 2 * j + 1] / s);
      dst[b * 16 + j] = (uint8_t)(lo | (hi << 4));
    }
    dst[D / 2 + b] = code;
  }
}

__global__ void attn_prep_kernel(PrepParams p) {
  tf_pdl_sync();
  extern __shared__ float sm[];     // max(Dh, Dh+Di) floats + scratch
  __shared__ float scratch[32];
  const int r = blockIdx.x, tid = threadIdx.x;
  const int pos = p.pos[r], reg = p.region[r];
  const int half_rd = p.rope_dim / 2, tail0 = p.Dh - p.rope_dim;
  // the row's rotation table, computed once (accurate sincos of large arguments is slow)
  __shared__ float s_sin[128], s_cos[128];
  if (tid < half_rd) rope_sincos(pos, p.freqs[tid], &s_sin[tid], &s_cos[tid]);
  __syncthreads();

  // ---- q: RoPE on the tail of every head.  With few rows the launch has gridDim.y > 1: the CTAs
  // with blockIdx.y > 0 share the query elements of the row, the CTA with blockIdx.y == 0 does the rest.
  const int qparts = gridDim.y > 1 ? gridDim.y - 1 : 1;
  const int qpart = gridDim.y > 1 ? (int)blockIdx.y - 1 : 0;
  const bool q_vec = p.p_kind != 0 && p.ldp % 8 == 0 && p.off_q % 8 == 0 && p.Dh % 8 == 0 && tail0 % 8 == 0 &&
                     !(reinterpret_cast<uintptr_t>(p.P) & 15) && !(reinterpret_cast<uintptr_t>(p.q_out) & 15);
  if (p.off_q >= 0 && qpart >= 0 && q_vec) {
    // bf16 rows, eight elements (four rotation pairs) per 16-byte load and store: same arithmetic as
    // the element-wise loop below
    const __nv_bfloat16* prow = reinterpret_cast<const __nv_bfloat16*>(p.P) + (long)r * p.ldp + p.off_q;
    __nv_bfloat16* qrow = p.q_out + (long)r * p.Hl * p.Dh;
    for (int v = qpart * blockDim.x + tid; v < p.Hl * p.Dh / 8; v += qparts * blockDim.x) {
      uint4 raw = *reinterpret_cast<const uint4*>(prow + v * 8);
      const int dd = (v * 8) % p.Dh;
      if (dd >= tail0) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int j = ((dd - tail0) >> 1) + k;
          const float sn = s_sin[j], cs = s_cos[j];
          const float2 f = __bfloat1622float2(h[k]);
          h[k] = __halves2bfloat162(__float2bfloat16(f.x * cs - f.y * sn), __float2bfloat16(f.x * sn + f.y * cs));
        }
      }
      *reinterpret_cast<uint4*>(qrow + v * 8) = raw;
    }
  } else if (p.off_q >= 0 && qpart >= 0) {
    for (int i = qpart * blockDim.x + tid; i < p.Hl * p.Dh; i += qparts * blockDim.x) {
      const int dd = i % p.Dh;
      float v = ldp(p, r, p.off_q + i);
      if (dd >= tail0) {
        const int j = (dd - tail0) >> 1;
        const float sn = s_sin[j], cs = s_cos[j];
        float other = ldp(p, r, p.off_q + (i ^ 1));
        v = ((dd - tail0) & 1) ? (other * sn + v * cs) : (v * cs - other * sn);
      }
      p.q_out[(long)r * p.Hl * p.Dh + i] = __float2bfloat16(v);
    }
  }
  if (gridDim.y > 1 && blockIdx.y > 0) return;      // query-only CTA
  // ---- kv latent: norm -> bf16 -> RoPE -> bf16 -> V41 row
  if (p.off_kv >= 0) {
    float ss = 0.f;
    for (int i = tid; i < p.Dh; i += blockDim.x) {
      float v = ldp(p, r, p.off_kv + i);
      sm[i] = v;
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)p.Dh + p.eps);
    for (int i = tid; i < p.Dh; i += blockDim.x)
      sm[i] = bf16_round(sm[i] * inv * __bfloat162float(p.kv_norm_w[i]));
    __syncthreads();
    float rot = 0.f;
    int ri = -1;
    if (tid < p.rope_dim) {
      const int dd = tail0 + tid, j = tid >> 1;
      const float sn = s_sin[j], cs = s_cos[j];
      float a = sm[dd], o = sm[dd ^ 1];
      rot = (tid & 1) ? (o * sn + a * cs) : (a * cs - o * sn);
      ri = dd;
    }
    __syncthreads();
    if (ri >= 0) sm[ri] = bf16_round(rot);
    __syncthreads();
    uint8_t* dst = p.win + (long)reg * p.win_region_stride + (long)(pos % p.ring) * p.win_row;
    store_v41(sm, dst, p.Dh);
    __syncthreads();
  }
  // ---- indexer query / weights
  if (p.off_iq >= 0) {
    for (int i = tid; i < p.Hi * p.Di; i += blockDim.x)
      p.iq_out[(long)r * p.Hi * p.Di + i] = __float2bfloat16(ldp(p, r, p.off_iq + i));
    for (int i = tid; i < p.Hi; i += blockDim.x) p.iw_out[(long)r * p.Hi + i] = ldp(p, r, p.off_iw + i);
  }
  // ---- compressor: pool the group this row completes
  if (p.off_cv >= 0 && ((pos + 1) % p.ratio) == 0) {
    const int C = p.Dh + p.Di, g = pos / p.ratio;
    if (g >= p.maxC) {
      if (tid == 0) tf_report(p.st, TF_BAD_INDEX, 2, r, g);
      return;
    }
    const int first = p.first_row[r];
    const int CS = p.carry_slots;
    const float* car = p.carry + (long)reg * CS * 2 * C;
    for (int c = tid; c < C; c += blockDim.x) {
      float mx = -INFINITY;
      for (int j = 0; j < p.ratio; ++j) {
        const int mr = r - (p.ratio - 1 - j);
        float gt = (mr >= first) ? ldp(p, mr, p.off_cg + c)
                                 : car[((pos - (p.ratio - 1 - j)) % CS) * 2 * C + C + c];
        mx = fmaxf(mx, gt);
      }
      float den = 0.f, num = 0.f;
      for (int j = 0; j < p.ratio; ++j) {
        const int mr = r - (p.ratio - 1 - j);
        float gt, vv;
        if (mr >= first) {
          gt = ldp(p, mr, p.off_cg + c);
          vv = ldp(p, mr, p.off_cv + c);
        } else {
          const float* cs = car + ((pos - (p.ratio - 1 - j)) % CS) * 2 * C;
          gt = cs[C + c];
          vv = cs[c];
        }
        float e = __expf(gt - mx);
        den += e;
        num += e * vv;
      }
      sm[c] = num / den;
    }
    __syncthreads();
    // index key from the pooled tail
    store_index_key(sm + p.Dh, p.keys + ((long)reg * p.maxC + g) * p.key_row, p.Di);
    // compressed latent: norm -> bf16 -> RoPE at the entry's own index -> bf16 -> FP4 row
    float ss = 0.f;
    for (int i = tid; i < p.Dh; i += blockDim.x) ss += sm[i] * sm[i];
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)p.Dh + p.eps);
    for (int i = tid; i < p.Dh; i += blockDim.x)
      sm[i] = bf16_round(sm[i] * inv * __bfloat162float(p.comp_norm_w[i]));
    __syncthreads();
    float rot = 0.f;
    int ri = -1;
    if (tid < p.rope_dim) {
      const int dd = tail0 + tid, j = tid >> 1;
      float sn, cs;
      rope_sincos(g, p.cfreqs[j], &sn, &cs);
      float a = sm[dd], o = sm[dd ^ 1];
      rot = (tid & 1) ? (o * sn + a * cs) : (a * cs - o * sn);
      ri = dd;
    }
    __syncthreads();
    if (ri >= 0) sm[ri] = bf16_round(rot);
    __syncthreads();
    store_v41fp4(sm, p.comp + ((long)reg * p.maxC + g) * p.comp_row, p.Dh);
  }
}

// Save the compressor inputs of rows whose group is still open at the end of the launch (they
// are read by a later launch).  Runs after attn_prep_kernel on the same stream, so no row of
// this launch still reads the slots being written.
__global__ void carry_save_kernel(PrepParams p) {
  tf_pdl_sync();
  const int r = blockIdx.x;
  const int pos = p.pos[r], reg = p.region[r];
  const int group_end = (pos / p.ratio + 1) * p.ratio - 1;
  if (group_end <= p.last_pos[r]) return;
  const int C = p.Dh + p.Di;
  const int CS = p.carry_slots;
  float* cs = p.carry + ((long)reg * CS + (pos % CS)) * 2 * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    cs[c] = ldp(p, r, p.off_cv + c);
    cs[C + c] = ldp(p, r, p.off_cg + c);
  }
}

// --------------------------------------------------------------------------- router
// logits[r, e] = h[r,:] . gate[e,:]  (f16 activations, bf16 gate), one warp per (expert, row-block)
__global__ void router_logits_kernel(const __half* __restrict__ h, const __nv_bfloat16* __restrict__ gate,
                                     float* __restrict__ logits, int M, int E, int d) {
  tf_pdl_sync();
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= E) return;
  const __nv_bfloat16* g = gate + (long)e * d;
  for (int r0 = 0; r0 < M; r0 += 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = lane * 8; k < d; k += 256) {
      uint4 gv = *reinterpret_cast<const uint4*>(g + k);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
      float gf[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(g2[q]);
        gf[2 * q] = f.x;
        gf[2 * q + 1] = f.y;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (r0 + j < M) {
          uint4 hv = *reinterpret_cast<const uint4*>(h + (long)(r0 + j) * d + k);
          const __half2* h2 = reinterpret_cast<const __half2*>(&hv);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float2 f = __half22float2(h2[q]);
            acc[j] = fmaf(f.x, gf[2 * q], acc[j]);
            acc[j] = fmaf(f.y, gf[2 * q + 1], acc[j]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = warp_sum(acc[j]);
      if (lane == 0 && r0 + j < M) logits[(long)(r0 + j) * E + e] = v;
    }
  }
}

__global__ void router_topk_kernel(const float* __restrict__ logits, const RouterBias bias,
                                   int* __restrict__ ids, float* __restrict__ wts, int M, int E, int topk,
                                   int scoring, int renorm, float scale) {
  tf_pdl_sync();
  extern __shared__ float sc[];                       // [warps][2][E]
  router_topk_rows(logits, bias, ids, wts, M, E, topk, scoring, renorm, scale, sc, blockIdx.x * (blockDim.x >> 5));
}

__global__ void route_group_kernel(const int* __restrict__ ids, int n_pairs, int e_lo, int e_hi,
                                   int* group_expert, int* group_start, int* group_count, int* n_groups,
                                   int* sorted_pairs, int* n_local_pairs) {
  tf_pdl_sync();
  extern __shared__ int cnt_smem[];
  route_group_body(ids, n_pairs, e_lo, e_hi, group_expert, group_start, group_count, n_groups, sorted_pairs,
                   n_local_pairs, cnt_smem);
}

// Decode rows: top-k of every row (one warp each, 16 rows per pass) and the grouping of the
// resulting pairs in ONE single-CTA launch.
__global__ void __launch_bounds__(512) router_topk_group_kernel(
    const float* __restrict__ logits, const RouterBias bias, int* __restrict__ ids, float* __restrict__ wts,
    int M, int E, int topk, int scoring, int renorm, float scale, int e_lo, int e_hi, int* group_expert,
    int* group_start, int* group_count, int* n_groups, int* sorted_pairs, int* n_local_pairs) {
  tf_pdl_sync();
  extern __shared__ float fsm[];                       // [16][2][E] floats, reused as ints by the grouping
  if (E <= 256 && topk <= 32) {
    // rows in registers; the local expert of every pair goes straight to the grouping's table
    int* cnt = reinterpret_cast<int*>(fsm);
    for (int r = threadIdx.x >> 5; r < M; r += blockDim.x >> 5)
      router_topk_rows_reg<8, 1>(logits, E, bias, r, M, ids, wts, E, topk, scoring, renorm, scale,
                                 cnt + (e_hi - e_lo), e_lo, e_hi);
    __syncthreads();
    route_group_body(nullptr, M * topk, e_lo, e_hi, group_expert, group_start, group_count, n_groups, sorted_pairs,
                     n_local_pairs, cnt);
    return;
  }
  for (int row0 = 0; row0 < M; row0 += 16)
    router_topk_rows(logits, bias, ids, wts, M, E, topk, scoring, renorm, scale, fsm, row0);
  __syncthreads();                                     // ids of every row are written (same CTA)
  route_group_body(ids, M * topk, e_lo, e_hi, group_expert, group_start, group_count, n_groups, sorted_pairs,
                   n_local_pairs, reinterpret_cast<int*>(fsm));
}

// out[r,:] = sum_j wts[r,j] * y_pair[r*topk+j,:] (experts of this rank only, fixed order) + shared[r,:]
__global__ void moe_combine_kernel(const float* __restrict__ y_pair, const int* __restrict__ ids,
                                   const float* __restrict__ wts, const float* __restrict__ shared_y,
                                   float* __restrict__ out, int d, int topk, int e_lo, int e_hi) {
  tf_pdl_sync();
  const int r = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < topk; ++j) {
      const int e = ids[r * topk + j];
      if (e >= e_lo && e < e_hi) acc = fmaf(wts[r * topk + j], y_pair[(long)(r * topk + j) * d + i], acc);
    }
    if (shared_y) acc += shared_y[(long)r * d + i];
    out[(long)r * d + i] = acc;
  }
}

__global__ void cast_f32_to_f16_kernel(const float* in, __half* out, long n) {
  tf_pdl_sync();
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2half(in[i]);
}

}  // namespace

TF_API int tf_embed(const int* tokens, const void* table, void* out, int T, int d, int vocab,
                    void* status, cudaStream_t st) {
  if (d % 8) return -1;
  tf_launch(embed_kernel, dim3(T), dim3(128), 0, st, tokens, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, d, vocab,
                                  (TfStatusWord*)status);
  return (int)cudaGetLastError();
}

TF_API int tf_add_norm(void* x, const void* delta, int delta_kind, int ldd, const void* w, void* h16,
                       void* hb, void* q8, void* qs, int T, int d, float eps, cudaStream_t st) {
  if (d % 128) return -1;
  tf_launch(add_norm_kernel, dim3(T), dim3(256), d * sizeof(float), st, (__nv_bfloat16*)x, delta, delta_kind, ldd,
                                                     (const __nv_bfloat16*)w, (__half*)h16,
                                                     (__nv_bfloat16*)hb, (uint8_t*)q8, (float*)qs, d, eps);
  return (int)cudaGetLastError();
}

TF_API int tf_attn_prep(const void* P, int p_kind, int ldp, int T, const int* pos, const int* region,
                        const int* first_row, const int* last_pos, int Hl, int Dh, int rope_dim,
                        const float* freqs, const float* cfreqs, const void* kv_norm_w, float eps,
                        void* q_out, void* win, long win_region_stride, int win_row, int comp_row,
                        int key_row, int ring, int off_q, int off_kv,
                        int off_cv, int off_cg, int off_iq, int off_iw, int ratio, int Di, int Hi,
                        const void* comp_norm_w, float* carry, int carry_slots, void* comp, void* keys,
                        int maxC, void* iq_out, float* iw_out, void* status, cudaStream_t st) {
  if (Dh % 32 || rope_dim > 256 || (off_cv >= 0 && Di % 32)) return -1;
  if (carry_slots <= 0) carry_slots = ratio + kCarrySpan;
  if (carry_slots < ratio + kCarrySpan) return -1;
  PrepParams p;
  p.P = P; p.p_kind = p_kind; p.ldp = ldp; p.T = T; p.pos = pos; p.region = region;
  p.first_row = first_row; p.last_pos = last_pos; p.Hl = Hl; p.Dh = Dh; p.rope_dim = rope_dim;
  p.freqs = freqs; p.cfreqs = cfreqs; p.kv_norm_w = (const __nv_bfloat16*)kv_norm_w; p.eps = eps;
  p.q_out = (__nv_bfloat16*)q_out; p.win = (uint8_t*)win; p.win_region_stride = win_region_stride;
  p.ring = ring; p.win_row = win_row; p.comp_row = comp_row; p.key_row = key_row; p.off_q = off_q; p.off_kv = off_kv; p.off_cv = off_cv; p.off_cg = off_cg;
  p.off_iq = off_iq; p.off_iw = off_iw; p.ratio = ratio; p.Di = Di; p.Hi = Hi;
  p.comp_norm_w = (const __nv_bfloat16*)comp_norm_w; p.carry = carry; p.carry_slots = carry_slots; p.comp = (uint8_t*)comp;
  p.keys = (uint8_t*)keys; p.maxC = maxC; p.iq_out = (__nv_bfloat16*)iq_out; p.iw_out = iw_out;
  p.st = (TfStatusWord*)status;
  const int smf = (off_cv >= 0 ? Dh + Di : Dh);
  // few rows (decode): eight more CTAs per row share the query heads
  tf_launch(attn_prep_kernel, dim3(dim3(T, (T <= 64 && off_q >= 0) ? 9 : 1)), dim3(256), smf * sizeof(float), st, p);
  if (off_cv >= 0) tf_launch(carry_save_kernel, dim3(T), dim3(128), 0, st, p);
  return (int)cudaGetLastError();
}

// bias_vl / tokens / image_token (all optional): rows whose token is the image token are selected
// with bias_vl (reference: kernels/moe_frontend.cuh:140).
TF_API int tf_router(const void* h16, const void* gate, const float* bias, const float* bias_vl, const int* tokens,
                     int image_token, float* logits, int* ids, float* wts, int M, int E, int d, int topk, int scoring,
                     int renorm, float scale, cudaStream_t st) {
  if (d % 256) return -1;
  const RouterBias rb{bias, bias_vl, tokens, image_token};
  tf_launch(router_logits_kernel, dim3((E + 7) / 8), dim3(256), 0, st, (const __half*)h16, (const __nv_bfloat16*)gate,
                                                    logits, M, E, d);
  const int nw = 4;
  tf_launch(router_topk_kernel, dim3((M + nw - 1) / nw), dim3(nw * 32), nw * 2 * E * sizeof(float), st, logits, rb, ids, wts, M, E, topk, scoring, renorm, scale);
  return (int)cudaGetLastError();
}

// top-k + weights only, for logits produced elsewhere (large row counts: tensor-core GEMM)
TF_API int tf_router_topk(const float* logits, const float* bias, const float* bias_vl, const int* tokens,
                          int image_token, int* ids, float* wts, int M, int E, int topk, int scoring, int renorm,
                          float scale, cudaStream_t st) {
  const int nw = 4;
  const RouterBias rb{bias, bias_vl, tokens, image_token};
  tf_launch(router_topk_kernel, dim3((M + nw - 1) / nw), dim3(nw * 32), nw * 2 * E * sizeof(float), st, logits, rb, ids, wts, M, E, topk, scoring, renorm, scale);
  return (int)cudaGetLastError();
}

// tf_router_topk followed by tf_route_group for up to 32 rows, one launch
TF_API int tf_router_topk_group(const float* logits, const float* bias, const float* bias_vl, const int* tokens,
                                int image_token, int* ids, float* wts, int M, int E, int topk,
                                int scoring, int renorm, float scale, int e_lo, int e_hi, int* group_expert,
                                int* group_start, int* group_count, int* n_groups, int* sorted_pairs,
                                int* n_local_pairs, cudaStream_t st) {
  const size_t smem = max((size_t)16 * 2 * E * sizeof(float), (size_t)(e_hi - e_lo + M * topk) * sizeof(int));
  if (M <= 0 || M > 32 || e_hi <= e_lo || smem > 48 * 1024) return -1;
  const RouterBias rb{bias, bias_vl, tokens, image_token};
  tf_launch(router_topk_group_kernel, dim3(1), dim3(512), smem, st, logits, rb, ids, wts, M, E, topk, scoring, renorm, scale, e_lo, e_hi,
                                                 group_expert, group_start, group_count, n_groups, sorted_pairs,
                                                 n_local_pairs);
  return (int)cudaGetLastError();
}

TF_API int tf_route_group(const int* ids, int n_pairs, int e_lo, int e_hi, int* group_expert,
                          int* group_start, int* group_count, int* n_groups, int* sorted_pairs,
                          int* n_local_pairs, cudaStream_t st) {
  if (n_pairs <= 0 || e_hi <= e_lo || (size_t)(e_hi - e_lo + n_pairs) * sizeof(int) > 48 * 1024) return -1;
  tf_launch(route_group_kernel, dim3(1), dim3(256), (e_hi - e_lo + n_pairs) * sizeof(int), st, ids, n_pairs, e_lo, e_hi, group_expert, group_start, group_count, n_groups, sorted_pairs,
      n_local_pairs);
  return (int)cudaGetLastError();
}

TF_API int tf_moe_combine(const float* y_pair, const int* ids, const float* wts, const float* shared_y,
                          float* out, int M, int d, int topk, int e_lo, int e_hi, cudaStream_t st) {
  tf_launch(moe_combine_kernel, dim3(dim3(M, M <= 64 ? (d + 255) / 256 : 1)), dim3(256), 0, st, y_pair, ids, wts, shared_y, out, d, topk, e_lo, e_hi);
  return (int)cudaGetLastError();
}

TF_API int tf_cast_f32_f16(const float* in, void* out, long n, cudaStream_t st) {
  tf_launch(cast_f32_to_f16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, in, (__half*)out, n);
  return (int)cudaGetLastError();
}
