// Indexer: scores of query rows against the FP4 index keys of their conversation, and exact
// top-k selection.
//
//   score(row, key) = sum_h relu(q[row,h,:] . k[key,:]) * w[row,h]
//
// Keys are packed e2m1 + one UE8M0 per 32 (68 bytes at 128 dims; reference
// kernels/index_bf16.cu:8-10); queries are bf16, accumulation is fp32 on m16n8k16 tiles with the
// (padded) heads of one row as the MMA's M.  Row `r` scores keys [0, nvalid[r]); the rest of its
// score row is -inf.  Selection is exact: ties at the cut go to the lower position and the
// output ids are ascending (reference contract: kernels/index_bf16.cu:1-21, src/topk.rs).
#include <cooperative_groups.h>

#include "common.cuh"

namespace {

constexpr int kKeysPerCta = 128;

struct ScoreParams {
  const __nv_bfloat16* q;   // [T, Hi, Di]
  const float* w;           // [T, Hi]
  const int* region;        // [T]
  const int* nvalid;        // [T]
  const uint8_t* keys;      // [regions][maxC][key_row]
  long key_region_stride;
  int key_row;
  int T, Hi, Di;
  int rows_per_group;       // consecutive rows sharing a region handled by one CTA
  float* scores;            // [T, lds]
  int lds;
  int key_lo, key_hi;       // this rank's key shard [lo, hi) (key-sharded scoring)
};

template <int DI>
__global__ void __launch_bounds__(128, 3) index_score_kernel(ScoreParams p) {
  tf_pdl_sync();
  constexpr int KS = DI + 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* Ks = reinterpret_cast<__half*>(smem_raw);   // [128][KS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.y * p.rows_per_group;
  const int nrows = min(p.rows_per_group, p.T - row0);
  const int key0 = p.key_lo + blockIdx.x * kKeysPerCta;
  int maxvalid = 0;
  for (int i = 0; i < nrows; ++i) maxvalid = max(maxvalid, p.nvalid[row0 + i]);
  maxvalid = min(maxvalid, p.key_hi);
  if (key0 >= maxvalid) {
    // still have to blank the tail of the score rows this CTA covers
    for (int i = 0; i < nrows; ++i)
      for (int k = threadIdx.x; k < kKeysPerCta; k += blockDim.x)
        if (key0 + k < p.lds && key0 + k < p.key_hi) p.scores[(long)(row0 + i) * p.lds + key0 + k] = -INFINITY;
    return;
  }
  const uint8_t* kb = p.keys + (long)p.region[row0] * p.key_region_stride;
  // dequantise 128 keys: one thread per (key, 32-block)
  for (int it = threadIdx.x; it < kKeysPerCta * (DI / 32); it += blockDim.x) {
    const int key = it % kKeysPerCta, blk = it / kKeysPerCta;
    __half* dst = Ks + key * KS + blk * 32;
    if (key0 + key < maxvalid) {
      const uint8_t* row = kb + (long)(key0 + key) * p.key_row;
      const float sc = ue8m0_to_float(row[DI / 2 + blk]);
      // unpacked halves hold value * 2^-14: the block scale takes the 2^14 (in fp32: no overflow)
      const uint32_t* wv = reinterpret_cast<const uint32_t*>(row + blk * 16);   // key rows are 4-byte aligned
      const float s14 = sc * 16384.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t h4[4], o[4];
        e2m1x8_to_h2x4_scaled(wv[q], h4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h4[j]));
          const __half2 h = __floats2half2_rn(f.x * s14, f.y * s14);
          o[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 2) *reinterpret_cast<__half2*>(dst + j) = __floats2half2_rn(0.f, 0.f);
    }
  }
  __syncthreads();
  // One m16 MMA tile holds 16 (query row, head) pairs: with 16+ heads a row spans whole tiles,
  // with fewer heads 16/Hi consecutive rows share one tile.
  const int rpt = p.Hi >= 16 ? 1 : 16 / p.Hi;
  const int head_tiles = p.Hi >= 16 ? (p.Hi + 15) / 16 : 1;
  const int units = (nrows + rpt - 1) / rpt;
  const uint32_t kfrag = (uint32_t)__cvta_generic_to_shared(Ks + (lane & 7) * KS + (lane >> 3) * 8);
  for (int u = warp; u < units; u += 4) {
    float tot0[kKeysPerCta / 8][2], tot8[kKeysPerCta / 8][2];
#pragma unroll
    for (int nt = 0; nt < kKeysPerCta / 8; ++nt) tot0[nt][0] = tot0[nt][1] = tot8[nt][0] = tot8[nt][1] = 0.f;
    int ra = 0, rb = 0;
    for (int ht = 0; ht < head_tiles; ++ht) {
      int ha, hb;
      if (p.Hi >= 16) {
        ra = rb = u;
        ha = ht * 16 + g;
        hb = ha + 8;
      } else {
        ra = u * rpt + g / p.Hi;
        ha = g % p.Hi;
        rb = u * rpt + (g + 8) / p.Hi;
        hb = (g + 8) % p.Hi;
      }
      const bool v0 = ra < nrows && ha < p.Hi, v8 = rb < nrows && hb < p.Hi;
      const long pa = (long)(row0 + min(ra, nrows - 1)) * p.Hi + min(ha, p.Hi - 1);
      const long pb = (long)(row0 + min(rb, nrows - 1)) * p.Hi + min(hb, p.Hi - 1);
      const __nv_bfloat16* q0 = p.q + pa * DI;
      const __nv_bfloat16* q8 = p.q + pb * DI;
      const float w0 = v0 ? p.w[pa] : 0.f, w8 = v8 ? p.w[pb] : 0.f;
      uint32_t qf[DI / 16][4];
#pragma unroll
      for (int ks = 0; ks < DI / 16; ++ks) {
        const int k = ks * 16 + 2 * t;
        float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q0 + k));
        float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q8 + k));
        float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q0 + k + 8));
        float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q8 + k + 8));
        __half2 ha2 = __floats2half2_rn(a.x, a.y), hb2 = __floats2half2_rn(b.x, b.y);
        __half2 hc2 = __floats2half2_rn(c.x, c.y), hd2 = __floats2half2_rn(d.x, d.y);
        qf[ks][0] = *reinterpret_cast<uint32_t*>(&ha2);
        qf[ks][1] = *reinterpret_cast<uint32_t*>(&hb2);
        qf[ks][2] = *reinterpret_cast<uint32_t*>(&hc2);
        qf[ks][3] = *reinterpret_cast<uint32_t*>(&hd2);
      }
#pragma unroll
      for (int nt = 0; nt < kKeysPerCta / 8; ++nt) {
        float sacc[4] = {0.f, 0.f, 0.f, 0.f};
        // one ldmatrix.x4 brings the B fragments of two 16-deep k steps (lane l: row l % 8 of
        // matrix l / 8; matrices = k 0-7, 8-15, 16-23, 24-31 of this 32-deep piece)
        const uint32_t kaddr = kfrag + nt * (8 * KS * 2);
#pragma unroll
        for (int k2 = 0; k2 < DI / 32; ++k2) {
          uint32_t b4[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b4[0]), "=r"(b4[1]), "=r"(b4[2]), "=r"(b4[3])
                       : "r"(kaddr + k2 * 64));
          mma_f16_16816(sacc, qf[2 * k2], b4);
          mma_f16_16816(sacc, qf[2 * k2 + 1], b4 + 2);
        }
        tot0[nt][0] += fmaxf(sacc[0], 0.f) * w0;
        tot0[nt][1] += fmaxf(sacc[1], 0.f) * w0;
        tot8[nt][0] += fmaxf(sacc[2], 0.f) * w8;
        tot8[nt][1] += fmaxf(sacc[3], 0.f) * w8;
      }
    }
    // sum over the heads of one query row: lanes that differ in the low log2(min(Hi,8)) bits of g
    if (p.Hi >= 8) {
      // Eight fragment rows (g) per query row.  Halving exchange instead of a butterfly per value:
      // in each of three rounds a lane keeps the half of its values whose key-tile bit equals its
      // own bit of g and hands the other half to its partner, so 64 values cost 32 + 16 + 8
      // shuffles (not 192) and every lane ends with the finished sums of key tiles g and g + 8,
      // which it stores itself.  Same pairing order as a butterfly: bitwise the same sums.
      const int nh = p.Hi >= 16 ? 1 : 2;                 // 16+ heads: tot0 and tot8 are the same query row
      const bool g0 = g & 1, g1 = g & 2, g2 = g & 4;
      float A[8][2][2], B[4][2][2], C[2][2][2];
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            if (h < nh) {
              float lo = h ? tot8[2 * m][i] : tot0[2 * m][i], hi = h ? tot8[2 * m + 1][i] : tot0[2 * m + 1][i];
              if (nh == 1) {
                lo += tot8[2 * m][i];
                hi += tot8[2 * m + 1][i];
              }
              A[m][h][i] = (g0 ? hi : lo) + __shfl_xor_sync(0xffffffffu, g0 ? lo : hi, 4);
            }
          }
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 2; ++i)
            if (h < nh)
              B[n][h][i] = (g1 ? A[2 * n + 1][h][i] : A[2 * n][h][i]) +
                           __shfl_xor_sync(0xffffffffu, g1 ? A[2 * n][h][i] : A[2 * n + 1][h][i], 8);
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 2; ++i)
            if (h < nh)
              C[q][h][i] = (g2 ? B[2 * q + 1][h][i] : B[2 * q][h][i]) +
                           __shfl_xor_sync(0xffffffffu, g2 ? B[2 * q][h][i] : B[2 * q + 1][h][i], 16);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int ri = h == 0 ? ra : rb;
        if (h >= nh || ri >= nrows) continue;
        const int r = row0 + ri;
        const int nv = min(p.nvalid[r], p.key_hi);
        float* out = p.scores + (long)r * p.lds;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int k = key0 + (8 * q + g) * 8 + 2 * t;   // this lane holds key tile 8q + g
          if (k < p.lds && k < p.key_hi) out[k] = k < nv ? C[q][h][0] : -INFINITY;
          if (k + 1 < p.lds && k + 1 < p.key_hi) out[k + 1] = k + 1 < nv ? C[q][h][1] : -INFINITY;
        }
      }
      continue;
    }
    const int span = p.Hi;                               // fewer than 8 heads: fragment rows of one query row within g
    const bool writer = (g % span) == 0;
#pragma unroll
    for (int nt = 0; nt < kKeysPerCta / 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float a = tot0[nt][i], b = tot8[nt][i];
        for (int m = 4; m < 4 * span; m <<= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, m);
          b += __shfl_xor_sync(0xffffffffu, b, m);
        }
        tot0[nt][i] = a;
        tot8[nt][i] = b;
      }
      if (writer) {
        const int k = key0 + nt * 8 + 2 * t;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int ri = half == 0 ? ra : rb;
          if (ri >= nrows) continue;
          const int r = row0 + ri;
          const int nv = min(p.nvalid[r], p.key_hi);
          const float* tv = half == 0 ? tot0[nt] : tot8[nt];
          float* out = p.scores + (long)r * p.lds;
          if (k < p.lds && k < p.key_hi) out[k] = k < nv ? tv[0] : -INFINITY;
          if (k + 1 < p.lds && k + 1 < p.key_hi) out[k + 1] = k + 1 < nv ? tv[1] : -INFINITY;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// exact top-k per row by radix select on the order-preserving integer image of the float
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// scores [T, lds]; n[r] valid entries; out ids [T, k] ascending, -1 padded; count[r] = min(n, k).
// `base` is added to every id (key-sharded scoring passes the shard offset).
__global__ void __launch_bounds__(1024) topk_select_kernel(const float* __restrict__ scores, int lds,
                                                           const int* __restrict__ nvalid, int k,
                                                           int* __restrict__ out, int* __restrict__ count,
                                                           float* __restrict__ out_scores, int base) {
  tf_pdl_sync();
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need, s_run, s_tie_run;
  __shared__ int warp_tot[32][2];
  const int r = blockIdx.x, tid = threadIdx.x;
  const int n = min(nvalid[r], lds);
  const float* s = scores + (long)r * lds;
  int* o = out + (long)r * k;
  if (n <= k) {
    for (int i = tid; i < k; i += blockDim.x) {
      o[i] = i < n ? base + i : -1;
      if (out_scores) out_scores[(long)r * k + i] = i < n ? s[i] : -INFINITY;
    }
    if (tid == 0 && count) count[r] = n;
    return;
  }
  // find the k-th largest key: MSB-first radix over 4 bytes
  if (tid == 0) {
    s_prefix = 0;
    s_need = k;
  }
  uint32_t mask = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    if (pass == 0) {
      // index scores crowd into a few exponent bytes: one shared atomic per warp and distinct bin
      for (int i0 = 0; i0 < n; i0 += blockDim.x) {
        const int i = i0 + tid;
        const bool in = i < n;
        const int bin = in ? (int)(float_key(s[i]) >> 24) : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        if (in && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
      }
    } else {
      for (int i = tid; i < n; i += blockDim.x) {
        const uint32_t key = float_key(s[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
      }
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_need = need;                     // how many to take from bin b (at deeper levels)
      s_prefix = prefix | ((uint32_t)b << shift);
    }
    __syncthreads();
    mask |= 0xffu << shift;
  }
  const uint32_t thr = s_prefix;         // key of the k-th largest
  const int need_ties = s_need;          // elements equal to thr to keep (lowest positions first)
  if (tid == 0) {
    s_run = 0;
    s_tie_run = 0;
  }
  __syncthreads();
  // ordered compaction in position order
  const int lane = tid & 31, warp = tid >> 5;
  for (int base_i = 0; base_i < n; base_i += blockDim.x) {
    const int i = base_i + tid;
    uint32_t key = i < n ? float_key(s[i]) : 0;
    const int gt = (i < n && key > thr) ? 1 : 0;
    const int eq = (i < n && key == thr) ? 1 : 0;
    // inclusive scans of gt and eq within the block
    int sg = gt, se = eq;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int a = __shfl_up_sync(0xffffffffu, sg, d), b = __shfl_up_sync(0xffffffffu, se, d);
      if (lane >= d) {
        sg += a;
        se += b;
      }
    }
    if (lane == 31) {
      warp_tot[warp][0] = sg;
      warp_tot[warp][1] = se;
    }
    __syncthreads();
    int og = 0, oe = 0;
    for (int w2 = 0; w2 < warp; ++w2) {
      og += warp_tot[w2][0];
      oe += warp_tot[w2][1];
    }
    const int run = s_run, tie_run = s_tie_run;
    const int eq_rank = tie_run + oe + se - eq;           // ties before this element
    const int take_eq = eq && (eq_rank < need_ties);
    // position among kept elements = kept gt before + kept eq before
    const int gt_before = run + og + sg - gt;
    const int eq_before = min(eq_rank, need_ties);
    if (gt || take_eq) {
      const int dst = gt_before + eq_before - 0;
      // run counts only gt; ties tracked separately: final index = gt_before + eq_before
      if (dst < k) {
        o[dst] = base + i;
        if (out_scores) out_scores[(long)r * k + dst] = s[i];
      }
    }
    __syncthreads();
    if (tid == blockDim.x - 1) {
      s_run = run + og + sg;
      s_tie_run = tie_run + oe + se;
    }
    __syncthreads();
  }
  if (tid == 0 && count) count[r] = k;
}

// The same selection for a few rows (decode): one CLUSTER of 8 CTAs per row.  Every thread keeps its
// run of consecutive keys in registers, the byte histograms are built with warp-aggregated shared
// atomics (scores crowd into a few exponent bytes, which serialises plain atomics) and read by all
// eight CTAs over distributed shared memory; the compaction needs only the totals of the CTAs
// before this one.  Output identical to topk_select_kernel.
// (Measured for the many rows of a prefill chunk too, as 2 CTAs x 32 keys per thread: 1,058 us for
// 2,048 rows x 32,768 scores against 816 us of the one-CTA kernel above, which therefore keeps them.)
constexpr int kSelThreads = 512;

template <int kSelCluster, int kSelKeysPerThread>
__global__ void __cluster_dims__(kSelCluster, 1, 1) __launch_bounds__(kSelThreads)
topk_select_cluster_kernel(const float* __restrict__ scores, int lds, const int* __restrict__ nvalid, int k,
                           int* __restrict__ out, int* __restrict__ count, float* __restrict__ out_scores,
                           int base) {
  tf_pdl_sync();
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ int hist[4][256];                      // one histogram per radix pass: no reuse, no second barrier
  __shared__ int wsum[kSelThreads / 32][2];
  __shared__ int cta_tot[2];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  const int r = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = (int)cluster.block_rank();
  const int n = min(nvalid[r], lds);
  const float* s = scores + (long)r * lds;
  int* o = out + (long)r * k;
  if (n <= k) {                                     // uniform over the cluster: nobody waits for anybody
    if (c == 0) {
      for (int i = tid; i < k; i += kSelThreads) {
        o[i] = i < n ? base + i : -1;
        if (out_scores) out_scores[(long)r * k + i] = i < n ? s[i] : -INFINITY;
      }
      if (tid == 0 && count) count[r] = n;
    }
    return;
  }
  const int chunk = (n + kSelCluster - 1) / kSelCluster;
  const int per = (chunk + kSelThreads - 1) / kSelThreads;       // <= kSelKeysPerThread (host check)
  const int lo = min(n, c * chunk), hi = min(n, lo + chunk);
  const int i0 = lo + tid * per;
  uint32_t key[kSelKeysPerThread];
#pragma unroll
  for (int j = 0; j < kSelKeysPerThread; ++j) key[j] = (j < per && i0 + j < hi) ? float_key(s[i0 + j]) : 0u;
  for (int i = tid; i < 4 * 256; i += kSelThreads) (&hist[0][0])[i] = 0;
  __syncthreads();
  uint32_t prefix = 0, mask = 0;
  int need = k;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
#pragma unroll
    for (int j = 0; j < kSelKeysPerThread; ++j) {
      if (j < per) {                                 // uniform over the warp
        const bool in = i0 + j < hi && (key[j] & mask) == prefix;
        const int bin = in ? (int)((key[j] >> shift) & 0xffu) : -1;
        if (pass == 0) {                             // the first byte is crowded: one atomic per warp and bin
          const unsigned peers = __match_any_sync(0xffffffffu, bin);
          if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[pass][bin], __popc(peers));
        } else if (in) {
          atomicAdd(&hist[pass][bin], 1);
        }
      }
    }
    cluster.sync();
    // thread t < 256 owns bin 255 - t: an inclusive scan over t is the count of keys in bins >= its own
    int h = 0;
    if (tid < 256) {
#pragma unroll
      for (int q = 0; q < kSelCluster; ++q) h += cluster.map_shared_rank(&hist[pass][0], q)[255 - tid];
    }
    int inc = h;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += v;
    }
    if (lane == 31) wsum[warp][0] = inc;
    __syncthreads();
    if (tid < 256) {
      for (int w2 = 0; w2 < warp; ++w2) inc += wsum[w2][0];
      if (inc >= need && inc - h < need) {           // exactly one bin holds the k-th largest
        s_prefix = prefix | ((uint32_t)(255 - tid) << shift);
        s_need = need - (inc - h);
      }
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    mask |= 0xffu << shift;
  }
  const uint32_t thr = prefix;                       // key of the k-th largest
  const int need_ties = need;                        // keys equal to it that are kept (lowest positions first)
  int cgt = 0, ceq = 0;
#pragma unroll
  for (int j = 0; j < kSelKeysPerThread; ++j) {
    if (j < per && i0 + j < hi) {
      cgt += key[j] > thr;
      ceq += key[j] == thr;
    }
  }
  int sg = cgt, se = ceq;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, sg, d), b = __shfl_up_sync(0xffffffffu, se, d);
    if (lane >= d) {
      sg += a;
      se += b;
    }
  }
  if (lane == 31) {
    wsum[warp][0] = sg;
    wsum[warp][1] = se;
  }
  __syncthreads();
  int og = sg - cgt, oe = se - ceq;                  // keys before this thread's run, inside the CTA
  for (int w2 = 0; w2 < warp; ++w2) {
    og += wsum[w2][0];
    oe += wsum[w2][1];
  }
  if (tid == kSelThreads - 1) {
    cta_tot[0] = og + cgt;
    cta_tot[1] = oe + ceq;
  }
  cluster.sync();
  for (int q = 0; q < c; ++q) {                      // ... and in the CTAs before this one
    const int* t = cluster.map_shared_rank(&cta_tot[0], q);
    og += t[0];
    oe += t[1];
  }
#pragma unroll
  for (int j = 0; j < kSelKeysPerThread; ++j) {
    if (j < per && i0 + j < hi) {
      const bool gt = key[j] > thr, eq = key[j] == thr;
      if (gt || (eq && oe < need_ties)) {
        const int dst = og + min(oe, need_ties);
        if (dst < k) {
          o[dst] = base + i0 + j;
          if (out_scores) out_scores[(long)r * k + dst] = s[i0 + j];
        }
      }
      og += gt;
      oe += eq;
    }
  }
  if (c == 0 && tid == 0 && count) count[r] = k;
  cluster.sync();                                    // nobody leaves while its totals may still be read
}

// Merge per-rank candidate lists (key-sharded scoring): cand_scores/cand_ids [T, ranks*k] -> top-k
// ids ascending.  Reuses the selection kernel on the gathered scores, then maps positions to ids.
__global__ void map_ids_kernel(const int* __restrict__ picked, const int* __restrict__ cand_ids, int ldc,
                               int k, int* __restrict__ out) {
  tf_pdl_sync();
  const int r = blockIdx.x;
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const int p = picked[(long)r * k + i];
    out[(long)r * k + i] = p >= 0 ? cand_ids[(long)r * ldc + p] : -1;
  }
}

// ---------------------------------------------------------------------------------------------
// two-level selection: block maxima of a source layer's scores, and scoring of candidate keys only
// ---------------------------------------------------------------------------------------------
// bmax[r, j] = max of scores[r, 8j .. 8j+7] over valid keys (-inf when none)
__global__ void __launch_bounds__(256) index_block_max_kernel(const float* __restrict__ scores, int lds,
                                                              const int* __restrict__ nvalid,
                                                              float* __restrict__ bmax, int ldb, int nblk) {
  tf_pdl_sync();
  const int r = blockIdx.y, j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= nblk) return;
  const int nv = nvalid[r];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = 8 * j + i;
    if (k < nv) m = fmaxf(m, scores[(long)r * lds + k]);
  }
  bmax[(long)r * ldb + j] = m;
}

// one warp per (row, candidate): the key is decoded exactly as in the dense kernel (value * scale
// rounded to f16, query rounded to f16), products accumulate in fp32
template <int DI>
__global__ void __launch_bounds__(256) index_scores_sparse_kernel(const __nv_bfloat16* __restrict__ q,
                                                                  const float* __restrict__ w,
                                                                  const int* __restrict__ region,
                                                                  const int* __restrict__ cand, int ldc,
                                                                  const uint8_t* __restrict__ keys,
                                                                  long key_region_stride, int key_row, int Hi,
                                                                  int C, float* __restrict__ out, int ldo) {
  tf_pdl_sync();
  constexpr int PER = DI / 32;                       // dims per lane
  const int r = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 8 + warp;
  if (c >= C) return;
  const int id = cand[(long)r * ldc + c];
  if (id < 0) {
    if (lane == 0) out[(long)r * ldo + c] = -INFINITY;
    return;
  }
  const uint8_t* row = keys + (long)region[r] * key_region_stride + (long)id * key_row;
  float kv[PER];
  const int d0 = lane * PER;
  const float sc = ue8m0_to_float(row[DI / 2 + d0 / 32]);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = d0 + i;
    const uint8_t b = row[d >> 1];
    kv[i] = __half2float(__float2half_rn(e2m1_to_float((d & 1) ? (b >> 4) : (b & 0xf)) * sc));
  }
  float total = 0.f;
  for (int h = 0; h < Hi; ++h) {
    const __nv_bfloat16* qh = q + ((long)r * Hi + h) * DI + d0;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc = fmaf(__half2float(__float2half_rn(__bfloat162float(qh[i]))), kv[i], acc);
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    total += fmaxf(acc, 0.f) * w[(long)r * Hi + h];
  }
  if (lane == 0) out[(long)r * ldo + c] = total;
}

}  // namespace

TF_API int tf_index_scores(const void* q, const float* w, const int* region, const int* nvalid,
                           const void* keys, long key_region_stride, int key_row, int T, int Hi, int Di,
                           int rows_per_group, float* scores, int lds, int key_lo, int key_hi,
                           cudaStream_t st) {
  if ((Di != 128 && Di != 64 && Di != 32) || key_row % 4 || rows_per_group < 1) return -1;
  if (key_hi <= key_lo) return 0;
  ScoreParams p;
  p.q = (const __nv_bfloat16*)q; p.w = w; p.region = region; p.nvalid = nvalid;
  p.keys = (const uint8_t*)keys; p.key_region_stride = key_region_stride; p.key_row = key_row;
  p.T = T; p.Hi = Hi; p.Di = Di; p.rows_per_group = rows_per_group; p.scores = scores; p.lds = lds;
  p.key_lo = key_lo; p.key_hi = key_hi;
  dim3 grid((key_hi - key_lo + kKeysPerCta - 1) / kKeysPerCta, (T + rows_per_group - 1) / rows_per_group);
  const int smem = kKeysPerCta * (Di + 8) * 2;
  if (Di == 128) tf_launch(index_score_kernel<128>, dim3(grid), dim3(128), smem, st, p);
  else if (Di == 64) tf_launch(index_score_kernel<64>, dim3(grid), dim3(128), smem, st, p);
  else tf_launch(index_score_kernel<32>, dim3(grid), dim3(128), smem, st, p);
  return (int)cudaGetLastError();
}

TF_API int tf_topk_select(const float* scores, int lds, const int* nvalid, int k, int* out, int* count,
                          float* out_scores, int base, int T, cudaStream_t st) {
  // a few long rows (decode): one cluster of CTAs per row; many rows: one CTA per row fills the GPU
  if (T <= 32 && lds > 4096 && lds <= 8 * kSelThreads * 16)
    tf_launch(topk_select_cluster_kernel<8, 16>, dim3(8, T), dim3(kSelThreads), 0, st, scores, lds, nvalid, k, out,
              count, out_scores, base);
  else
    tf_launch(topk_select_kernel, dim3(T), dim3(1024), 0, st, scores, lds, nvalid, k, out, count, out_scores, base);
  return (int)cudaGetLastError();
}

TF_API int tf_map_ids(const int* picked, const int* cand_ids, int ldc, int k, int* out, int T,
                      cudaStream_t st) {
  tf_launch(map_ids_kernel, dim3(T), dim3(256), 0, st, picked, cand_ids, ldc, k, out);
  return (int)cudaGetLastError();
}

// block maxima over blocks of 8 keys (two-level candidates: reference src/candidates.rs:1-20)
TF_API int tf_index_block_max(const float* scores, int lds, const int* nvalid, float* bmax, int ldb, int nblk, int T,
                              cudaStream_t st) {
  if (T <= 0 || nblk <= 0) return 0;
  tf_launch(index_block_max_kernel, dim3(dim3((nblk + 255) / 256, T)), dim3(256), 0, st, scores, lds, nvalid, bmax, ldb, nblk);
  return (int)cudaGetLastError();
}

// scores of candidate keys only: cand [T, C] key ids (-1 = none) -> out [T, C] (-inf for none)
TF_API int tf_index_scores_sparse(const void* q, const float* w, const int* region, const int* cand, int ldc,
                                  const void* keys, long key_region_stride, int key_row, int T, int Hi, int Di, int C,
                                  float* out, int ldo, cudaStream_t st) {
  if (T <= 0 || C <= 0) return 0;
  dim3 grid((C + 7) / 8, T);
  if (Di == 128)
    tf_launch(index_scores_sparse_kernel<128>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)q, w, region, cand, ldc,
                                                          (const uint8_t*)keys, key_region_stride, key_row, Hi, C, out, ldo);
  else if (Di == 64)
    tf_launch(index_scores_sparse_kernel<64>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)q, w, region, cand, ldc,
                                                         (const uint8_t*)keys, key_region_stride, key_row, Hi, C, out, ldo);
  else return -1;
  return (int)cudaGetLastError();
}
