// Router pieces shared by the single-launch decode router kernels: top-k of a row of router logits
// (smem and register forms) and the counting sort of (token, slot) pairs by local expert.
// Reference behaviour: kernels/moe_frontend.cuh (`ca_route_topk`, selection bias, image-token bias).
#pragma once
#include "common.cuh"

// top-k per row (one warp per row) + weights.  scoring 0 = softmax, 1 = sqrtsoftplus.
// Ties go to the lowest expert id; NaN keys count as +inf.
// The selection bias is chosen per row: rows whose token is `image_token` use bias_vl (when given).
struct RouterBias {
  const float* bias;
  const float* bias_vl;
  const int* tokens;
  int image_token;
};
__device__ __forceinline__ void router_topk_rows(const float* __restrict__ logits, const RouterBias rb,
                                                 int* __restrict__ ids, float* __restrict__ wts, int M, int E, int topk,
                                                 int scoring, int renorm, float scale, float* sc, int row0) {
  // sc: [warps][2][E] floats of shared memory; warp w serves row row0 + w
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = row0 + warp;
  if (r >= M) return;
  float* score = sc + (long)warp * 2 * E;
  float* key = score + E;
  const float* lg = logits + (long)r * E;
  const float* bias = (rb.bias_vl && rb.tokens && rb.tokens[r] == rb.image_token) ? rb.bias_vl : rb.bias;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
  mx = warp_max(mx);
  float den = 0.f;
  for (int e = lane; e < E; e += 32) {
    float x = lg[e], s;
    if (scoring == 1) {
      float sp = x > 20.f ? x : log1pf(expf(x));
      s = sqrtf(sp);
    } else {
      s = expf(x - mx);
      den += s;
    }
    score[e] = s;
  }
  den = warp_sum(den);
  for (int e = lane; e < E; e += 32) {
    if (scoring == 0) score[e] /= den;
    float k = score[e] + (bias ? bias[e] : 0.f);
    key[e] = isnan(k) ? INFINITY : k;
  }
  __syncwarp();
  float wsum = 0.f;
  for (int j = 0; j < topk; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      float k = key[e];
      if (k > best || (k == best && e < bi)) {
        best = k;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = 0;
    if (lane == 0) {
      ids[(long)r * topk + j] = bi;
      wts[(long)r * topk + j] = score[bi];
      key[bi] = -INFINITY;
    }
    wsum += score[bi];
    __syncwarp();
  }
  if (lane == 0) {
    for (int j = 0; j < topk; ++j) {
      float w = wts[(long)r * topk + j];
      if (renorm) w = w / (wsum + 1e-20f);
      wts[(long)r * topk + j] = w * scale;
    }
  }
}


// The same top-k with rows in registers (E <= 32 * NPL): lane l holds experts l, l + 32, ... of R
// rows at once (rows r0 .. r0 + R - 1; the independent rows hide each other's load and shuffle
// latency).  Lane j < topk ends up with the j-th pick; ids/wts are written once.  `loc`
// (optional, shared memory) receives the local expert of every pair (-1 outside [e_lo, e_hi)) for
// the grouping that follows in the same CTA.  Bitwise the same scores, picks and weights as
// router_topk_rows.
template <int NPL, int R>
__device__ __forceinline__ void router_topk_rows_reg(const float* __restrict__ logits, int ldl, const RouterBias rb,
                                                     int r0, int M, int* __restrict__ ids, float* __restrict__ wts,
                                                     int E, int topk, int scoring, int renorm, float scale, int* loc,
                                                     int e_lo, int e_hi) {
  const int lane = threadIdx.x & 31;
  const float* bias[R];
#pragma unroll
  for (int q = 0; q < R; ++q) {
    const int r = min(r0 + q, M - 1);
    bias[q] = (rb.bias_vl && rb.tokens && rb.tokens[r] == rb.image_token) ? rb.bias_vl : rb.bias;
  }
  float sc[R][NPL], ky[R][NPL];
#pragma unroll
  for (int q = 0; q < R; ++q) {
    const float* lg = logits + (long)min(r0 + q, M - 1) * ldl;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      sc[q][i] = e < E ? __ldcg(lg + e) : -INFINITY;               // the logit, for now
      ky[q][i] = (bias[q] && e < E) ? bias[q][e] : 0.f;            // the bias, for now
    }
  }
#pragma unroll
  for (int q = 0; q < R; ++q) {
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPL; ++i) mx = fmaxf(mx, sc[q][i]);
    mx = warp_max(mx);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      const float x = sc[q][i];
      float s = 0.f;
      if (e < E) {
        if (scoring == 1) {
          const float sp = x > 20.f ? x : log1pf(expf(x));
          s = sqrtf(sp);
        } else {
          s = expf(x - mx);
          den += s;
        }
      }
      sc[q][i] = s;
    }
    den = warp_sum(den);
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (scoring == 0) sc[q][i] /= den;
      const float k = sc[q][i] + ky[q][i];
      ky[q][i] = e < E ? (isnan(k) ? INFINITY : k) : -INFINITY;
    }
  }
  float wsum[R], my_w[R];
  int my_id[R];
#pragma unroll
  for (int q = 0; q < R; ++q) {
    wsum[q] = my_w[q] = 0.f;
    my_id[q] = 0;
  }
  for (int j = 0; j < topk; ++j) {
    float best[R];
    int bi[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      best[q] = -INFINITY;
      bi[q] = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int e = lane + 32 * i;
        if (e < E && (ky[q][i] > best[q] || (ky[q][i] == best[q] && e < bi[q]))) {
          best[q] = ky[q][i];
          bi[q] = e;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const float ob = __shfl_xor_sync(0xffffffffu, best[q], o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi[q], o);
        if (ob > best[q] || (ob == best[q] && oi < bi[q])) {
          best[q] = ob;
          bi[q] = oi;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < R; ++q) {
      if (bi[q] == 0x7fffffff) bi[q] = 0;
      float mine = 0.f;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        if (lane + 32 * i == bi[q]) {
          mine = sc[q][i];
          ky[q][i] = -INFINITY;
        }
      }
      const float w = __shfl_sync(0xffffffffu, mine, bi[q] & 31);
      if (lane == j) {
        my_id[q] = bi[q];
        my_w[q] = w;
      }
      wsum[q] += w;
    }
  }
#pragma unroll
  for (int q = 0; q < R; ++q) {
    const int r = r0 + q;
    if (r < M && lane < topk) {
      const float w = renorm ? my_w[q] / (wsum[q] + 1e-20f) : my_w[q];
      ids[(long)r * topk + lane] = my_id[q];
      wts[(long)r * topk + lane] = w * scale;
      if (loc) {
        const int e = my_id[q] - e_lo;
        loc[r * topk + lane] = (e >= 0 && e < e_hi - e_lo) ? e : -1;
      }
    }
  }
}

// Group (token, slot) pairs by expert for the experts this rank owns: counting sort in one CTA.
// Outputs: group_expert/start/count for the compacted active experts, n_groups, sorted_pairs.
__device__ __forceinline__ void route_group_body(const int* __restrict__ ids, int n_pairs, int e_lo, int e_hi,
                                                 int* group_expert, int* group_start, int* group_count,
                                                 int* n_groups, int* sorted_pairs, int* n_local_pairs, int* cnt) {
  // cnt: [E_local] counts, then offsets; then the local expert of every pair (shared memory)
  // (ids == nullptr: the caller has filled loc already and synchronised the CTA)
  const int El = e_hi - e_lo;
  int* loc = cnt + El;
  if (ids) {
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
      const int e = ids[i] - e_lo;
      loc[i] = (e >= 0 && e < El) ? e : -1;
    }
    __syncthreads();
  }
  // one thread per expert counts its pairs out of shared memory (no atomics: fixed order)
  for (int e = threadIdx.x; e < El; e += blockDim.x) {
    int c = 0;
    for (int i = 0; i < n_pairs; ++i) c += (loc[i] == e);
    cnt[e] = c;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // warp 0: exclusive scan of the counts and compaction of the active experts, 32 at a time
    const int lane = threadIdx.x;
    int off = 0, ng = 0;
    for (int base = 0; base < El; base += 32) {
      const int e = base + lane;
      const int c = e < El ? cnt[e] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      const unsigned act = __ballot_sync(0xffffffffu, c > 0);
      const int start = off + inc - c;
      if (c > 0) {
        const int gi = ng + __popc(act & ((1u << lane) - 1u));
        group_expert[gi] = e;
        group_start[gi] = start;
        group_count[gi] = c;
      }
      if (e < El) cnt[e] = start;
      off += __shfl_sync(0xffffffffu, inc, 31);
      ng += __popc(act);
    }
    if (lane == 0) {
      *n_groups = ng;
      *n_local_pairs = off;
    }
  }
  __syncthreads();
  // stable placement in pair order (single thread per expert keeps the order deterministic)
  for (int e = threadIdx.x; e < El; e += blockDim.x) {
    int off = cnt[e];
    for (int i = 0; i < n_pairs; ++i)
      if (loc[i] == e) sorted_pairs[off++] = i;
  }
}

