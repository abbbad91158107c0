// Sparse MQA attention over the V4.1 caches: every query row attends to its sliding window
// (FP8 rows, e4m3 + UE8M0/32), to the compressed entries its indexer selected (FP4 rows, e2m1 +
// e4m3/16) and to a per-head sink.  One latent per key is both K and V.
//
// Layout of the work: a CTA owns one query row and walks 64-key chunks of that row's key list
// (split s takes chunks s, s+nsplit, ...).  Keys are dequantised once per chunk into shared
// memory, row-major; QK^T reads them as they lie and PV reads the same rows through
// ldmatrix.trans (heads up to 128 wide), so no transposed copy is written.  FP4 entries, 94 % of
// the keys of a long-context row, are unpacked eight at a time with the byte-permute form of
// common.cuh.  Each warp owns 16 heads and runs both contractions on m16n8k16 tensor-core tiles
// with an online base-2 softmax.  Partials
// (normalised output + log2-sum-exp) are merged with the sink as an extra zero-valued logit,
// then the inverse RoPE rotation is applied to the output tail (the value shares the key's
// rotated latent; reference src/layer_attention.rs:1416-1423).  Partial/merge arithmetic follows
// the reference's split decode (runtime/kernels/attention-dsv41-decode-v1/decode.cu:249-314):
// fp32 normalised partials, base-2 LSE, empty splits at -1e30.
#include "common.cuh"

namespace {

constexpr int kChunk = 64;
constexpr float kNegBig = -1e30f;

struct AttnParams {
  const __nv_bfloat16* q;     // [T, Hl, Dh] (RoPE applied)
  int T, Hl, Dh;
  const int* pos;             // [T]
  const int* region;          // [T]
  const int* min_pos;         // [T] or null: oldest position a row may attend in the window
  const uint8_t* win;         // [regions][ring][Dh + Dh/32]
  long win_region_stride;
  int ring, window;
  int win_row, comp_row;      // row strides in bytes (multiples of 16)
  const uint8_t* comp;        // [regions][maxC][Dh/2 + Dh/16] or null
  long comp_region_stride;
  const int* sel;             // [T, sel_stride] ascending ids, -1 = none
  int sel_stride;
  const int* sel_count;       // [T] or null (then scan for -1)
  int maxC;
  float scale_log2;           // softmax scale * log2(e)
  int nsplit;
  float* part_o;              // [T, nsplit, Hl, Dh]
  float* part_lse;            // [T, nsplit, Hl]  (log2 domain; kNegBig when empty)
  TfStatusWord* st;
  // the tcgen05 kernel finishes the row itself (sink, inverse rotation of the tail, f16 / bf16 rows)
  const float* sink;          // [Hl] or null
  const float* freqs;         // [rope_dim / 2]
  int rope_dim;
  __half* out16;
  __nv_bfloat16* outb;
  int ldo;
};

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

#include "attention_tc.cuh"     // sparse_attn_tc_kernel: prefill rows on tcgen05 (inside this namespace)

int g_attn_tc = 1;               // tf_sparse_attention_set_tc
int g_attn_sms = 0;

template <int DH>
__global__ void __launch_bounds__(128) sparse_attn_kernel(AttnParams p) {
  tf_pdl_sync();
  constexpr int KS = DH + 8;          // row stride of Ks (halfs): 16-byte rows shifted by one bank group per key
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* Ks = reinterpret_cast<__half*>(smem_raw);          // [64][KS]

  const int r = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int pos = p.pos[r], reg = p.region[r];
  const int nwin = min(pos + 1 - (p.min_pos ? p.min_pos[r] : 0), p.window);
  int nsel = 0;
  if (p.comp) {
    if (p.sel_count) nsel = p.sel_count[r];
    else {
      // ids are ascending with -1 padding at the end: binary search for the first -1
      int lo = 0, hi = p.sel_stride;
      const int* s = p.sel + (long)r * p.sel_stride;
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (s[mid] >= 0) lo = mid + 1; else hi = mid;
      }
      nsel = lo;
    }
  }
  const int nkeys = nwin + nsel;
  const int nchunks = (nkeys + kChunk - 1) / kChunk;
  const int h0 = warp * 16;
  const bool warp_active = h0 < p.Hl;

  // ---- Q fragments (pre-scaled)
  uint32_t qf[DH / 16][4];
  if (warp_active) {
    const __nv_bfloat16* q0 = p.q + ((long)r * p.Hl + min(h0 + g, p.Hl - 1)) * DH;
    const __nv_bfloat16* q8 = p.q + ((long)r * p.Hl + min(h0 + g + 8, p.Hl - 1)) * DH;
    const bool v0 = h0 + g < p.Hl, v8 = h0 + g + 8 < p.Hl;
#pragma unroll
    for (int ks = 0; ks < DH / 16; ++ks) {
      const int k = ks * 16 + 2 * t;
      float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q0 + k));
      float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q8 + k));
      float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q0 + k + 8));
      float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q8 + k + 8));
      const float s0 = v0 ? p.scale_log2 : 0.f, s8 = v8 ? p.scale_log2 : 0.f;
      qf[ks][0] = pack_h2(a.x * s0, a.y * s0);
      qf[ks][1] = pack_h2(b.x * s8, b.y * s8);
      qf[ks][2] = pack_h2(c.x * s0, c.y * s0);
      qf[ks][3] = pack_h2(d.x * s8, d.y * s8);
    }
  }
  float o[DH / 8][4];
#pragma unroll
  for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = kNegBig, m8 = kNegBig, l0 = 0.f, l8 = 0.f;

  const int wrow = p.win_row, crow = p.comp_row;
  const uint8_t* win = p.win + (long)reg * p.win_region_stride;
  const uint8_t* comp = p.comp ? p.comp + (long)reg * p.comp_region_stride : nullptr;
  const uint32_t kfrag = (uint32_t)__cvta_generic_to_shared(Ks + (lane & 7) * KS + (lane >> 3) * 8);

  // Gather pipeline.  Thread tid serves key tid % 64 of every chunk and NI = DH / 32 of its 16-value
  // segments (tid / 64 + 2j).  The raw bytes of the NEXT chunk's rows (and the key ids of the chunk
  // after it) are requested before this chunk's MMAs and converted after them, so the two dependent
  // global loads of a gathered row (id -> row) overlap the tensor work instead of preceding it.
  constexpr int NI = DH / 32;
  const int my_key = threadIdx.x & (kChunk - 1), seg0 = threadIdx.x >> 6;
  auto load_src = [&](int c) -> int {
    const int i = c * kChunk + my_key;
    if (c >= nchunks || i >= nkeys) return 0x7fffffff;
    if (i < nwin) return (pos - nwin + 1 + i) % p.ring;
    int id = p.sel[(long)r * p.sel_stride + (i - nwin)];
    if (id < 0 || id >= p.maxC) {
      tf_report(p.st, TF_BAD_INDEX, 10, r, id);
      id = 0;
    }
    return ~id;
  };
  uint4 raw[NI];
  uint8_t rsc[NI];
  auto load_raw = [&](int src) {
    if (src == 0x7fffffff) return;
    if (src >= 0) {
      const uint8_t* row = win + (long)src * wrow;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        raw[j] = *reinterpret_cast<const uint4*>(row + (seg0 + 2 * j) * 16);
        rsc[j] = row[DH + j];                        // (seg0 + 2j) >> 1 == j
      }
    } else {
      const uint8_t* row = comp + (long)(~src) * crow;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const uint2 v = *reinterpret_cast<const uint2*>(row + (seg0 + 2 * j) * 8);
        raw[j] = make_uint4(v.x, v.y, 0u, 0u);
        rsc[j] = row[DH / 2 + seg0 + 2 * j];
      }
    }
  };
  int src_cur = load_src(split), src_next = load_src(split + p.nsplit);
  load_raw(src_cur);

  for (int c = split; c < nchunks; c += p.nsplit) {
    const int kbase = c * kChunk;
    __syncthreads();                                   // the previous chunk's MMAs have read Ks
    // convert this chunk's rows: sixteen f16 values per segment
#pragma unroll
    for (int j = 0; j < NI; ++j) {
      uint32_t hv[8];
      if (src_cur == 0x7fffffff) {
#pragma unroll
        for (int q = 0; q < 8; ++q) hv[q] = 0u;
      } else if (src_cur >= 0) {
        const float sc = ue8m0_to_float(rsc[j]);
        const uint16_t* h = reinterpret_cast<const uint16_t*>(&raw[j]);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint32_t h2 = e4m3x2_to_h2(h[q]);
          float2 f = __half22float2(*reinterpret_cast<__half2*>(&h2));
          hv[q] = pack_h2(f.x * sc, f.y * sc);
        }
      } else {
        // the unpacked halves hold value * 2^-14: fold 2^14 into the group's scale (fp32: no overflow)
        const float sc = e4m3_to_float(rsc[j]) * 16384.f;
        uint32_t lo4[4], hi4[4];
        e2m1x8_to_h2x4_scaled(raw[j].x, lo4);
        e2m1x8_to_h2x4_scaled(raw[j].y, hi4);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo4[q]));
          const float2 cc = __half22float2(*reinterpret_cast<__half2*>(&hi4[q]));
          hv[q] = pack_h2(a.x * sc, a.y * sc);
          hv[4 + q] = pack_h2(cc.x * sc, cc.y * sc);
        }
      }
      uint4* kd = reinterpret_cast<uint4*>(Ks + my_key * KS + (seg0 + 2 * j) * 16);
      kd[0] = make_uint4(hv[0], hv[1], hv[2], hv[3]);
      kd[1] = make_uint4(hv[4], hv[5], hv[6], hv[7]);
    }
    // request the next chunk's rows and the ids of the chunk after it
    src_cur = src_next;
    load_raw(src_cur);
    src_next = load_src(c + 2 * p.nsplit);
    __syncthreads();
    if (!warp_active) continue;

    // ---- S = Q K^T for 8 key tiles
    float s[kChunk / 8][4];
#pragma unroll
    for (int nt = 0; nt < kChunk / 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      // one ldmatrix.x4 = the B fragments of two 16-deep steps (lane l: row l % 8 of block l / 8)
      const uint32_t kaddr = kfrag + nt * (8 * KS * 2);
#pragma unroll
      for (int k2 = 0; k2 < DH / 32; ++k2) {
        uint32_t b4[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b4[0]), "=r"(b4[1]), "=r"(b4[2]), "=r"(b4[3])
                     : "r"(kaddr + k2 * 64));
        mma_f16_16816(s[nt], qf[2 * k2], b4);
        mma_f16_16816(s[nt], qf[2 * k2 + 1], b4 + 2);
      }
    }
    // mask keys beyond the list
    const int valid = nkeys - kbase;
    float cm0 = kNegBig, cm8 = kNegBig;
#pragma unroll
    for (int nt = 0; nt < kChunk / 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = nt * 8 + 2 * t + (i & 1);
        if (key >= valid) s[nt][i] = kNegBig;
      }
      cm0 = fmaxf(cm0, fmaxf(s[nt][0], s[nt][1]));
      cm8 = fmaxf(cm8, fmaxf(s[nt][2], s[nt][3]));
    }
    cm0 = fmaxf(cm0, __shfl_xor_sync(0xffffffffu, cm0, 1));
    cm0 = fmaxf(cm0, __shfl_xor_sync(0xffffffffu, cm0, 2));
    cm8 = fmaxf(cm8, __shfl_xor_sync(0xffffffffu, cm8, 1));
    cm8 = fmaxf(cm8, __shfl_xor_sync(0xffffffffu, cm8, 2));
    const float nm0 = fmaxf(m0, cm0), nm8 = fmaxf(m8, cm8);
    const float f0 = exp2f(m0 - nm0), f8 = exp2f(m8 - nm8);
    m0 = nm0;
    m8 = nm8;
    l0 *= f0;
    l8 *= f8;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      o[i][0] *= f0;
      o[i][1] *= f0;
      o[i][2] *= f8;
      o[i][3] *= f8;
    }
    uint32_t pf[kChunk / 16][4];
#pragma unroll
    for (int nt = 0; nt < kChunk / 8; ++nt) {
      float p0 = exp2f(s[nt][0] - m0), p1 = exp2f(s[nt][1] - m0);
      float p2 = exp2f(s[nt][2] - m8), p3 = exp2f(s[nt][3] - m8);
      if (s[nt][0] <= kNegBig) p0 = 0.f;
      if (s[nt][1] <= kNegBig) p1 = 0.f;
      if (s[nt][2] <= kNegBig) p2 = 0.f;
      if (s[nt][3] <= kNegBig) p3 = 0.f;
      l0 += p0 + p1;
      l8 += p2 + p3;
      // C tiles (2j, 2j+1) of S become the A fragment of k16 step j
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(p2, p3);
    }
    // ---- O += P V: the B fragments (keys along k, dims along n) come out of the row-major key
    // tile through ldmatrix.trans, four 8x8 blocks (two k16 steps) per instruction
    {
      const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks);
      const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
      for (int dt = 0; dt < DH / 8; ++dt) {
#pragma unroll
        for (int kp = 0; kp < kChunk / 32; ++kp) {
          const int key = (2 * kp + (lm >> 1)) * 16 + (lm & 1) * 8 + lr;
          const uint32_t addr = ks_base + (uint32_t)(key * KS + dt * 8) * 2u;
          uint32_t b0[2], b1[2];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0[0]), "=r"(b0[1]), "=r"(b1[0]), "=r"(b1[1])
                       : "r"(addr));
          mma_f16_16816(o[dt], pf[2 * kp], b0);
          mma_f16_16816(o[dt], pf[2 * kp + 1], b1);
        }
      }
    }
  }
  if (!warp_active) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l8 += __shfl_xor_sync(0xffffffffu, l8, 1);
  l8 += __shfl_xor_sync(0xffffffffu, l8, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i8 = l8 > 0.f ? 1.f / l8 : 0.f;
  const long base = ((long)r * p.nsplit + split) * p.Hl;
  if (h0 + g < p.Hl) {
    float* po = p.part_o + (base + h0 + g) * DH;
#pragma unroll
    for (int dt = 0; dt < DH / 8; ++dt)
      *reinterpret_cast<float2*>(po + dt * 8 + 2 * t) = make_float2(o[dt][0] * i0, o[dt][1] * i0);
    if (t == 0) p.part_lse[base + h0 + g] = l0 > 0.f ? m0 + log2f(l0) : kNegBig;
  }
  if (h0 + g + 8 < p.Hl) {
    float* po = p.part_o + (base + h0 + g + 8) * DH;
#pragma unroll
    for (int dt = 0; dt < DH / 8; ++dt)
      *reinterpret_cast<float2*>(po + dt * 8 + 2 * t) = make_float2(o[dt][2] * i8, o[dt][3] * i8);
    if (t == 0) p.part_lse[base + h0 + g + 8] = l8 > 0.f ? m8 + log2f(l8) : kNegBig;
  }
}

// ---------------------------------------------------------------------------------------------
// Wide latent (head_dim 256 / 512, the reference model's 512-wide MLA latent): the head dimension is
// split over the four warps.  Each warp forms the partial scores of all 16 heads of a head tile over
// its DH/4 dims, the partials are summed through shared memory, every warp then runs the same
// online softmax and accumulates P.V for its own DH/4 output dims, so the per-warp register
// footprint is that of a 128-wide head.  Head tiles of 16 are processed one after the other.
// ---------------------------------------------------------------------------------------------
template <int DH>
__global__ void __launch_bounds__(128) sparse_attn_wide_kernel(AttnParams p) {
  tf_pdl_sync();
  constexpr int SL = DH / 4;          // dims owned by one warp
  constexpr int KS = DH + 8;
  constexpr int VS = kChunk + 8;
  constexpr int SP = kChunk + 4;      // row stride of the partial-score tiles (floats)
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* Ks = reinterpret_cast<__half*>(smem_raw);                    // [64][KS]
  __half* Vt = Ks + kChunk * KS;                                       // [DH][VS]
  float* Sp = reinterpret_cast<float*>(Vt + DH * VS);                  // [4 warps][16][SP]
  __shared__ int key_src[kChunk];

  const int r = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int pos = p.pos[r], reg = p.region[r];
  const int nwin = min(pos + 1 - (p.min_pos ? p.min_pos[r] : 0), p.window);
  int nsel = 0;
  if (p.comp) {
    if (p.sel_count) nsel = p.sel_count[r];
    else {
      int lo = 0, hi = p.sel_stride;
      const int* sidx = p.sel + (long)r * p.sel_stride;
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (sidx[mid] >= 0) lo = mid + 1; else hi = mid;
      }
      nsel = lo;
    }
  }
  const int nkeys = nwin + nsel;
  const int nchunks = (nkeys + kChunk - 1) / kChunk;
  const int wrow = p.win_row, crow = p.comp_row;
  const uint8_t* win = p.win + (long)reg * p.win_region_stride;
  const uint8_t* comp = p.comp ? p.comp + (long)reg * p.comp_region_stride : nullptr;
  const int d0 = warp * SL;

  for (int h0 = 0; h0 < p.Hl; h0 += 16) {
    // ---- this warp's slice of the (pre-scaled) Q fragments of the head tile
    uint32_t qf[SL / 16][4];
    {
      const __nv_bfloat16* q0 = p.q + ((long)r * p.Hl + min(h0 + g, p.Hl - 1)) * DH + d0;
      const __nv_bfloat16* q8 = p.q + ((long)r * p.Hl + min(h0 + g + 8, p.Hl - 1)) * DH + d0;
      const float s0 = h0 + g < p.Hl ? p.scale_log2 : 0.f, s8 = h0 + g + 8 < p.Hl ? p.scale_log2 : 0.f;
#pragma unroll
      for (int ks = 0; ks < SL / 16; ++ks) {
        const int k = ks * 16 + 2 * t;
        float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q0 + k));
        float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q8 + k));
        float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q0 + k + 8));
        float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q8 + k + 8));
        qf[ks][0] = pack_h2(a.x * s0, a.y * s0);
        qf[ks][1] = pack_h2(b.x * s8, b.y * s8);
        qf[ks][2] = pack_h2(c.x * s0, c.y * s0);
        qf[ks][3] = pack_h2(d.x * s8, d.y * s8);
      }
    }
    float o[SL / 8][4];
#pragma unroll
    for (int i = 0; i < SL / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = kNegBig, m8 = kNegBig, l0 = 0.f, l8 = 0.f;

    for (int c = split; c < nchunks; c += p.nsplit) {
      const int kbase = c * kChunk;
      __syncthreads();
      for (int kk = threadIdx.x; kk < kChunk; kk += blockDim.x) {
        const int i = kbase + kk;
        int src = 0x7fffffff;
        if (i < nwin) {
          src = (pos - nwin + 1 + i) % p.ring;
        } else if (i < nkeys) {
          int id = p.sel[(long)r * p.sel_stride + (i - nwin)];
          if (id < 0 || id >= p.maxC) {
            tf_report(p.st, TF_BAD_INDEX, 11, r, id);
            id = 0;
          }
          src = ~id;
        }
        key_src[kk] = src;
      }
      __syncthreads();
      for (int it = threadIdx.x; it < kChunk * (DH / 16); it += blockDim.x) {
        const int key = it % kChunk, seg = it / kChunk;
        const int src = key_src[key];
        float v[16];
        if (src == 0x7fffffff) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        } else if (src >= 0) {
          const uint8_t* row = win + (long)src * wrow;
          uint4 raw = *reinterpret_cast<const uint4*>(row + seg * 16);
          const float sc = ue8m0_to_float(row[DH + (seg >> 1)]);
          const uint16_t* h = reinterpret_cast<const uint16_t*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t h2 = e4m3x2_to_h2(h[j]);
            float2 f = __half22float2(*reinterpret_cast<__half2*>(&h2));
            v[2 * j] = f.x * sc;
            v[2 * j + 1] = f.y * sc;
          }
        } else {
          const uint8_t* row = comp + (long)(~src) * crow;
          uint2 raw = *reinterpret_cast<const uint2*>(row + seg * 8);
          const float sc = e4m3_to_float(row[DH / 2 + seg]);
          const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = e2m1_to_float((w[j >> 3] >> (4 * (j & 7))) & 0xfu) * sc;
        }
        __half* kd = Ks + key * KS + seg * 16;
#pragma unroll
        for (int j = 0; j < 16; j += 2) *reinterpret_cast<__half2*>(kd + j) = __floats2half2_rn(v[j], v[j + 1]);
#pragma unroll
        for (int j = 0; j < 16; ++j) Vt[(seg * 16 + j) * VS + key] = __float2half(v[j]);
      }
      __syncthreads();
      // ---- partial S over this warp's dims, summed through shared memory
      float s[kChunk / 8][4];
#pragma unroll
      for (int nt = 0; nt < kChunk / 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const __half* kr = Ks + (nt * 8 + g) * KS + d0 + 2 * t;
#pragma unroll
        for (int ks = 0; ks < SL / 16; ++ks) {
          uint32_t b[2];
          b[0] = *reinterpret_cast<const uint32_t*>(kr + ks * 16);
          b[1] = *reinterpret_cast<const uint32_t*>(kr + ks * 16 + 8);
          mma_f16_16816(s[nt], qf[ks], b);
        }
        float* sp = Sp + (warp * 16) * SP + nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(sp + g * SP) = make_float2(s[nt][0], s[nt][1]);
        *reinterpret_cast<float2*>(sp + (g + 8) * SP) = make_float2(s[nt][2], s[nt][3]);
      }
      __syncthreads();
#pragma unroll
      for (int nt = 0; nt < kChunk / 8; ++nt) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {                   // fixed order: every warp gets the same sums
          const float* sp = Sp + (w * 16) * SP + nt * 8 + 2 * t;
          const float2 x = *reinterpret_cast<const float2*>(sp + g * SP);
          const float2 y = *reinterpret_cast<const float2*>(sp + (g + 8) * SP);
          a0 += x.x; a1 += x.y; a2 += y.x; a3 += y.y;
        }
        s[nt][0] = a0; s[nt][1] = a1; s[nt][2] = a2; s[nt][3] = a3;
      }
      const int valid = nkeys - kbase;
      float cm0 = kNegBig, cm8 = kNegBig;
#pragma unroll
      for (int nt = 0; nt < kChunk / 8; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = nt * 8 + 2 * t + (i & 1);
          if (key >= valid) s[nt][i] = kNegBig;
        }
        cm0 = fmaxf(cm0, fmaxf(s[nt][0], s[nt][1]));
        cm8 = fmaxf(cm8, fmaxf(s[nt][2], s[nt][3]));
      }
      cm0 = fmaxf(cm0, __shfl_xor_sync(0xffffffffu, cm0, 1));
      cm0 = fmaxf(cm0, __shfl_xor_sync(0xffffffffu, cm0, 2));
      cm8 = fmaxf(cm8, __shfl_xor_sync(0xffffffffu, cm8, 1));
      cm8 = fmaxf(cm8, __shfl_xor_sync(0xffffffffu, cm8, 2));
      const float nm0 = fmaxf(m0, cm0), nm8 = fmaxf(m8, cm8);
      const float f0 = exp2f(m0 - nm0), f8 = exp2f(m8 - nm8);
      m0 = nm0;
      m8 = nm8;
      l0 *= f0;
      l8 *= f8;
#pragma unroll
      for (int i = 0; i < SL / 8; ++i) {
        o[i][0] *= f0;
        o[i][1] *= f0;
        o[i][2] *= f8;
        o[i][3] *= f8;
      }
      uint32_t pf[kChunk / 16][4];
#pragma unroll
      for (int nt = 0; nt < kChunk / 8; ++nt) {
        float p0 = exp2f(s[nt][0] - m0), p1 = exp2f(s[nt][1] - m0);
        float p2 = exp2f(s[nt][2] - m8), p3 = exp2f(s[nt][3] - m8);
        if (s[nt][0] <= kNegBig) p0 = 0.f;
        if (s[nt][1] <= kNegBig) p1 = 0.f;
        if (s[nt][2] <= kNegBig) p2 = 0.f;
        if (s[nt][3] <= kNegBig) p3 = 0.f;
        l0 += p0 + p1;
        l8 += p2 + p3;
        pf[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(p0, p1);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(p2, p3);
      }
      // ---- O[:, this warp's dims] += P V
#pragma unroll
      for (int dt = 0; dt < SL / 8; ++dt) {
        const __half* vr = Vt + (d0 + dt * 8 + g) * VS + 2 * t;
#pragma unroll
        for (int ks = 0; ks < kChunk / 16; ++ks) {
          uint32_t b[2];
          b[0] = *reinterpret_cast<const uint32_t*>(vr + ks * 16);
          b[1] = *reinterpret_cast<const uint32_t*>(vr + ks * 16 + 8);
          mma_f16_16816(o[dt], pf[ks], b);
        }
      }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l8 += __shfl_xor_sync(0xffffffffu, l8, 1);
    l8 += __shfl_xor_sync(0xffffffffu, l8, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i8 = l8 > 0.f ? 1.f / l8 : 0.f;
    const long base = ((long)r * p.nsplit + split) * p.Hl;
    if (h0 + g < p.Hl) {
      float* po = p.part_o + (base + h0 + g) * DH + d0;
#pragma unroll
      for (int dt = 0; dt < SL / 8; ++dt)
        *reinterpret_cast<float2*>(po + dt * 8 + 2 * t) = make_float2(o[dt][0] * i0, o[dt][1] * i0);
      if (t == 0 && warp == 0) p.part_lse[base + h0 + g] = l0 > 0.f ? m0 + log2f(l0) : kNegBig;
    }
    if (h0 + g + 8 < p.Hl) {
      float* po = p.part_o + (base + h0 + g + 8) * DH + d0;
#pragma unroll
      for (int dt = 0; dt < SL / 8; ++dt)
        *reinterpret_cast<float2*>(po + dt * 8 + 2 * t) = make_float2(o[dt][2] * i8, o[dt][3] * i8);
      if (t == 0 && warp == 0) p.part_lse[base + h0 + g + 8] = l8 > 0.f ? m8 + log2f(l8) : kNegBig;
    }
  }
}

// merge splits + sink, inverse RoPE on the tail, write f16 and/or bf16.  grid (T, Hl), block Dh.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                  const float* __restrict__ sink, const int* __restrict__ pos,
                                  const float* __restrict__ freqs, int nsplit, int Hl, int Dh, int rope_dim,
                                  __half* __restrict__ out16, __nv_bfloat16* __restrict__ outb, int ldo) {
  tf_pdl_sync();
  extern __shared__ float vals[];   // Dh
  const int r = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float* lse = part_lse + ((long)r * nsplit) * Hl + h;
  float mx = sink ? sink[h] * 1.4426950408889634f : kNegBig;
  for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, lse[(long)s * Hl]);
  float den = sink ? exp2f(sink[h] * 1.4426950408889634f - mx) : 0.f;
  float acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float l = lse[(long)s * Hl];
    if (l <= kNegBig) continue;
    const float w = exp2f(l - mx);
    den += w;
    acc += w * part_o[(((long)r * nsplit + s) * Hl + h) * Dh + d];
  }
  vals[d] = den > 0.f ? acc / den : 0.f;
  __syncthreads();
  float v = vals[d];
  const int tail0 = Dh - rope_dim;
  if (d >= tail0) {
    const int j = (d - tail0) >> 1;
    float sn, cs;
    {
      const float ang = (float)pos[r] * freqs[j];
      const double two_pi = 6.283185307179586476925286766559;
      sincosf((float)((double)ang - two_pi * floor((double)ang / two_pi)), &sn, &cs);
    }
    const float other = vals[d ^ 1];
    // inverse rotation: angle -> -angle
    v = ((d - tail0) & 1) ? (-other * sn + v * cs) : (v * cs + other * sn);
  }
  const long off = (long)r * ldo + (long)h * Dh + d;
  if (out16) out16[off] = __float2half(v);
  if (outb) outb[off] = __float2bfloat16(v);
}

}  // namespace

// 1 (default): prefill rows (one split, head dim 128, 64 rows or more) run on the tcgen05 kernel;
// 0: always the mma.sync kernels.  Returns the previous setting.
TF_API int tf_sparse_attention_set_tc(int on) {
  const int old = g_attn_tc;
  g_attn_tc = on ? 1 : 0;
  return old;
}

TF_API int tf_sparse_attention(const void* q, int T, int Hl, int Dh, const int* pos, const int* region,
                               const int* min_pos,
                               const void* win, long win_region_stride, int win_row, int ring, int window,
                               const void* comp, long comp_region_stride, int comp_row, const int* sel, int sel_stride,
                               const int* sel_count, int maxC, float scale, int nsplit, float* part_o,
                               float* part_lse, const float* sink, const float* freqs, int rope_dim,
                               void* out16, void* outb, int ldo, void* status, cudaStream_t st) {
  if (Dh != 128 && Dh != 64 && Dh != 256 && Dh != 512) return -1;
  if (Hl > 64 || nsplit < 1 || (win_row % 16) || (comp && (comp_row % 16))) return -1;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.T = T; p.Hl = Hl; p.Dh = Dh; p.pos = pos; p.region = region; p.min_pos = min_pos;
  p.win = (const uint8_t*)win; p.win_region_stride = win_region_stride; p.ring = ring; p.window = window; p.win_row = win_row; p.comp_row = comp_row;
  p.comp = (const uint8_t*)comp; p.comp_region_stride = comp_region_stride; p.sel = sel;
  p.sel_stride = sel_stride; p.sel_count = sel_count; p.maxC = maxC;
  p.scale_log2 = scale * 1.4426950408889634f; p.nsplit = nsplit; p.part_o = part_o; p.part_lse = part_lse;
  p.st = (TfStatusWord*)status;
  // four warps always: all of them dequantise the key chunk, those that own heads run the MMAs
  const int warps = 4;
  dim3 grid(T, nsplit);
  p.sink = sink; p.freqs = freqs; p.rope_dim = rope_dim; p.out16 = (__half*)out16; p.outb = (__nv_bfloat16*)outb; p.ldo = ldo;
  if (g_attn_tc && Dh == 128 && nsplit == 1 && T >= 64 && Hl <= 64 && !(reinterpret_cast<uintptr_t>(q) & 15) &&
      rope_dim <= 64 && rope_dim % 2 == 0 && ldo % 8 == 0 && !(reinterpret_cast<uintptr_t>(out16) & 15) &&
      !(reinterpret_cast<uintptr_t>(outb) & 15)) {
    // prefill rows: persistent CTAs on the tcgen05 tensor cores, one query row at a time
    if (!g_attn_sms) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&g_attn_sms, cudaDevAttrMultiProcessorCount, dev);
      cudaFuncSetAttribute(sparse_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem);
    }
    tf_launch(sparse_attn_tc_kernel, dim3(T < g_attn_sms ? T : g_attn_sms), dim3(kTcThreads), kTcSmem, st, p);
    return (int)cudaGetLastError();      // (sink, inverse rotation and the output rows are part of that kernel)
  } else if (Dh == 512 || Dh == 256) {
    const int smem = (kChunk * (Dh + 8) + Dh * (kChunk + 8)) * 2 + 4 * 16 * (kChunk + 4) * 4;
    static bool attr_set = false;
    if (!attr_set) {
      cudaFuncSetAttribute(sparse_attn_wide_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (kChunk * (512 + 8) + 512 * (kChunk + 8)) * 2 + 4 * 16 * (kChunk + 4) * 4);
      cudaFuncSetAttribute(sparse_attn_wide_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (kChunk * (256 + 8) + 256 * (kChunk + 8)) * 2 + 4 * 16 * (kChunk + 4) * 4);
      attr_set = true;
    }
    if (Dh == 512) tf_launch(sparse_attn_wide_kernel<512>, dim3(grid), dim3(warps * 32), smem, st, p);
    else tf_launch(sparse_attn_wide_kernel<256>, dim3(grid), dim3(warps * 32), smem, st, p);
  } else if (Dh == 128) {
    const int smem = kChunk * (128 + 8) * 2;
    tf_launch(sparse_attn_kernel<128>, dim3(grid), dim3(warps * 32), smem, st, p);
  } else {
    const int smem = kChunk * (64 + 8) * 2;
    tf_launch(sparse_attn_kernel<64>, dim3(grid), dim3(warps * 32), smem, st, p);
  }
  dim3 mg(T, Hl);
  tf_launch(attn_merge_kernel, dim3(mg), dim3(Dh), Dh * sizeof(float), st, part_o, part_lse, sink, pos, freqs, nsplit, Hl, Dh,
                                                        rope_dim, (__half*)out16, (__nv_bfloat16*)outb, ldo);
  return (int)cudaGetLastError();
}
