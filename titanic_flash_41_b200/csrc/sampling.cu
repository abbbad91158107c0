// Sampling and speculative verification on fp32 logits.
//
//  * argmax (greedy; ties to the lowest id; reference kernels/core.cu:631-643)
//  * row statistics for temperature + nucleus (top-p) sampling: max, the order-preserving key of
//    the smallest logit inside the nucleus, and the nucleus mass, all in fp64
//  * block verification (Sun et al., arXiv:2403.10444; reference kernels/block_rejection.cuh:1-63):
//      w_0 = 1, w_i = min(1, w_{i-1} p_{i-1}(x_i) / q_{i-1}(x_i)),
//      R_i = sum_v max(w_i p_i(v) - q_i(v), 0),  h_i = R_i / (R_i + 1 - w_i) (i < g), h_g = w_g,
//      tau = max{ i : u_i <= h_i } (0 if none); token at tau from the normalised residual (or from
//      p_g when tau = g).  p and q are the temperature- and nucleus-modified distributions, so the
//      output law is exactly the modified target law.  Masses are fp64; non-finite logits or
//      negative masses raise a status word instead of producing a token.
//  * the same draw kernel samples plain rows (no proposals): tau = g = 0.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct RowStat {
  float m;          // max logit
  uint32_t thr;     // smallest key inside the nucleus (0 = everything)
  double z;         // sum over the nucleus of exp((x - m) / T)
};

__device__ double block_sum_d(double v, double* scratch) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[w] = v;
  __syncthreads();
  double t = lane < nw ? scratch[lane] : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int ldl, int V, int* __restrict__ out,
                              float* __restrict__ out_val) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int r = blockIdx.x;
  const float* x = logits + (long)r * ldl;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = x[i];
    if (v > best || (v == best && i < idx)) {
      best = v;
      idx = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) {
    bv[w] = best;
    bi[w] = idx;
  }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? bv[lane] : -INFINITY;
    idx = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
      }
    }
    if (lane == 0) {
      out[r] = idx == 0x7fffffff ? 0 : idx;
      if (out_val) out_val[r] = best;
    }
  }
}

__global__ void __launch_bounds__(1024) rowstat_kernel(const float* __restrict__ logits, int ldl, int V,
                                                       float temp, float top_p, RowStat* __restrict__ out,
                                                       TfStatusWord* st) {
  __shared__ float fscr[32];
  const int r = blockIdx.x;
  const float* x = logits + (long)r * ldl;
  float m = -INFINITY;
  int bad = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = x[i];
    if (isnan(v) || v == INFINITY) bad = 1;
    m = fmaxf(m, v);
  }
  m = block_max(m, fscr);
  if (__syncthreads_or(bad)) {
    if (threadIdx.x == 0) {
      tf_report(st, TF_NONFINITE, 20, r, 0);
      out[r].m = 0.f;
      out[r].thr = 0xffffffffu;
      out[r].z = 1.0;
    }
    return;
  }
  // Masses are accumulated as 2^-40 fixed point so that the (unordered) shared-memory atomics give
  // the same sums on every run and on every rank that samples the same row.
  __shared__ unsigned long long hist[4096];
  __shared__ unsigned long long chunk[32];
  __shared__ unsigned long long s_above, s_total, s_inbin;
  __shared__ uint32_t s_prefix;
  const float inv_t = 1.f / temp;
  const double kFix = 1099511627776.0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t prefix = 0, mask = 0;
  unsigned long long target = 0;
  if (threadIdx.x == 0) s_above = 0;
  // radix levels over the order-preserving key: 12 + 12 + 8 bits
  for (int level = 0; level < 3; ++level) {
    const int shift = level == 0 ? 20 : (level == 1 ? 8 : 0);
    const int nb = level == 2 ? 256 : 4096;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = x[i];
      const uint32_t key = fkey(v);
      if ((key & mask) == prefix)
        atomicAdd(&hist[(key >> shift) & (nb - 1)], (unsigned long long)((double)expf((v - m) * inv_t) * kFix));
    }
    __syncthreads();
    // per-warp sums of nb/32 consecutive bins
    {
      const int per = nb / 32;
      unsigned long long sacc = 0;
      for (int j = lane; j < per; j += 32) sacc += hist[warp * per + j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
      if (lane == 0) chunk[warp] = sacc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (level == 0) {
        unsigned long long tot = 0;
        for (int w = 0; w < 32; ++w) tot += chunk[w];
        s_total = tot;
        target = top_p < 1.f ? (unsigned long long)((double)top_p * (double)tot) : 0ull;
        if (target == 0) target = 1;
      }
      // first bin from the top whose inclusive cumulative mass reaches the target
      const int per = nb / 32;
      unsigned long long cum = s_above;
      int w = 31;
      for (; w > 0; --w) {
        if (cum + chunk[w] >= target) break;
        cum += chunk[w];
      }
      int b = w * per + per - 1;
      for (; b > w * per; --b) {
        if (cum + hist[b] >= target) break;
        cum += hist[b];
      }
      s_above = cum;
      s_inbin = hist[b];
      s_prefix = prefix | ((uint32_t)b << shift);
    }
    __syncthreads();
    prefix = s_prefix;
    mask |= (uint32_t)(nb - 1) << shift;
    if (top_p >= 1.f) break;
  }
  uint32_t thr = 0;
  double z = (double)s_total / kFix;
  if (top_p < 1.f) {
    thr = prefix;
    z = (double)(s_above + s_inbin) / kFix;
  }
  if (threadIdx.x == 0) {
    out[r].m = m;
    out[r].thr = thr;
    out[r].z = z;
  }
}

__device__ __forceinline__ double prob_of(const float* x, const RowStat& s, float inv_t, int v) {
  const float l = x[v];
  if (fkey(l) < s.thr) return 0.0;
  return (double)expf((l - s.m) * inv_t) / s.z;
}

struct VerifyParams {
  const float* tlogits;     // [S, g+1, V] target rows
  const float* dlogits;     // [S, g, V] draft rows (null with point-mass proposals)
  const RowStat* tstat;     // [S*(g+1)]
  const RowStat* dstat;     // [S*g]
  const int* proposals;     // [S, g]
  const double* uniforms;   // [S, g+2]: u_1..u_g (acceptance), u_draw at index g, spare
  int S, g, V, ldl;
  float t_temp, d_temp;
  int point_mass;           // 1: q_i is a point mass at the proposal (text-lookup proposals)
  double* R;                // [S, g+1] scratch: residual masses
  double* w;                // [S, g+1] scratch
  int* n_accept;            // [S]
  int* next_token;          // [S]
  TfStatusWord* st;
};

// residual value at token v of row i: max(w_i p_i(v) - q_i(v), 0); bonus row (i == g) has q = 0
__device__ __forceinline__ double residual_at(const VerifyParams& p, int s, int i, double wi, int v) {
  const float* tx = p.tlogits + ((long)s * (p.g + 1) + i) * p.ldl;
  double val = wi * prob_of(tx, p.tstat[s * (p.g + 1) + i], 1.f / p.t_temp, v);
  if (i < p.g) {
    if (p.point_mass) {
      if (v == p.proposals[s * p.g + i]) val -= 1.0;
    } else {
      const float* dx = p.dlogits + ((long)s * p.g + i) * p.ldl;
      val -= prob_of(dx, p.dstat[s * p.g + i], 1.f / p.d_temp, v);
    }
  }
  return val > 0.0 ? val : 0.0;
}

// grid (S, g+1): w_i and R_i
__global__ void __launch_bounds__(1024) verify_mass_kernel(VerifyParams p) {
  __shared__ double scratch[32];
  __shared__ double s_w;
  const int s = blockIdx.x, i = blockIdx.y;
  if (threadIdx.x == 0) {
    double w = 1.0;
    for (int j = 1; j <= i; ++j) {
      const int x = p.proposals[s * p.g + j - 1];
      const float* tx = p.tlogits + ((long)s * (p.g + 1) + j - 1) * p.ldl;
      double pt = prob_of(tx, p.tstat[s * (p.g + 1) + j - 1], 1.f / p.t_temp, x);
      double q = 1.0;
      if (!p.point_mass) {
        const float* dx = p.dlogits + ((long)s * p.g + j - 1) * p.ldl;
        q = prob_of(dx, p.dstat[s * p.g + j - 1], 1.f / p.d_temp, x);
      }
      double ratio = q > 0.0 ? w * pt / q : (pt > 0.0 ? 1.0 : 0.0);
      w = ratio < 1.0 ? ratio : 1.0;
    }
    s_w = w;
    p.w[s * (p.g + 1) + i] = w;
  }
  __syncthreads();
  const double wi = s_w;
  double acc = 0.0;
  for (int v = threadIdx.x; v < p.V; v += blockDim.x) acc += residual_at(p, s, i, wi, v);
  acc = block_sum_d(acc, scratch);
  if (threadIdx.x == 0) {
    p.R[s * (p.g + 1) + i] = acc;
    if (!(acc >= 0.0) || isinf(acc)) tf_report(p.st, TF_NONFINITE, 21, s, i);
  }
}

// grid S: decide tau and draw the token
__global__ void __launch_bounds__(1024) verify_decide_kernel(VerifyParams p) {
  constexpr int kTile = 1024;
  __shared__ double tile_mass[512];
  __shared__ double scan[1024];
  __shared__ int s_tau, s_tile, s_tok;
  __shared__ double s_target;
  const int s = blockIdx.x, g = p.g;
  const double* R = p.R + s * (g + 1);
  const double* w = p.w + s * (g + 1);
  const double* u = p.uniforms + (long)s * (g + 2);
  if (threadIdx.x == 0) {
    int tau = 0;
    for (int i = 1; i <= g; ++i) {
      double h = (i < g) ? (R[i] + 1.0 - w[i] > 0.0 ? R[i] / (R[i] + 1.0 - w[i]) : 0.0) : w[g];
      if (u[i - 1] <= h) tau = i;
    }
    s_tau = tau;
    s_tok = -1;
  }
  __syncthreads();
  const int tau = s_tau;
  const double wi = w[tau];
  const int ntiles = (p.V + kTile - 1) / kTile;
  if (ntiles > 512) {
    if (threadIdx.x == 0) tf_report(p.st, TF_BAD_ARG, 22, ntiles, 0);
    return;
  }
  // tile masses: one warp per tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int tl = warp; tl < ntiles; tl += nw) {
    double acc = 0.0;
    for (int v = tl * kTile + lane; v < min(p.V, (tl + 1) * kTile); v += 32) acc += residual_at(p, s, tau, wi, v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) tile_mass[tl] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int tl = 0; tl < ntiles; ++tl) total += tile_mass[tl];
    double target = u[g] * total;
    // keep the target strictly inside the mass so that a token is always found
    if (target >= total) target = nextafter(total, 0.0);
    int tl = 0;
    double before = 0.0;
    for (; tl < ntiles - 1; ++tl) {
      if (before + tile_mass[tl] > target) break;
      before += tile_mass[tl];
    }
    s_tile = tl;
    s_target = target - before;
    if (!(total > 0.0)) tf_report(p.st, TF_NONFINITE, 23, s, tau);
  }
  __syncthreads();
  const int v = s_tile * kTile + threadIdx.x;
  double val = (threadIdx.x < kTile && v < p.V) ? residual_at(p, s, tau, wi, v) : 0.0;
  scan[threadIdx.x] = val;
  __syncthreads();
  // inclusive scan (Hillis-Steele over 1024 entries)
  for (int d = 1; d < 1024; d <<= 1) {
    double add = threadIdx.x >= d ? scan[threadIdx.x - d] : 0.0;
    __syncthreads();
    scan[threadIdx.x] += add;
    __syncthreads();
  }
  const double cdf = scan[threadIdx.x], prev = threadIdx.x ? scan[threadIdx.x - 1] : 0.0;
  if (val > 0.0 && prev <= s_target && s_target < cdf) s_tok = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tok = s_tok;
    if (tok < 0) {
      // rounding pushed the target past the last positive entry: take the last positive one
      for (int j = min(kTile, p.V - s_tile * kTile) - 1; j >= 0; --j) {
        double pv = j ? scan[j] - scan[j - 1] : scan[0];
        if (pv > 0.0) {
          tok = s_tile * kTile + j;
          break;
        }
      }
      if (tok < 0) {
        tf_report(p.st, TF_NONFINITE, 24, s, tau);
        tok = 0;
      }
    }
    p.n_accept[s] = tau;
    p.next_token[s] = tok;
  }
}

}  // namespace

TF_API int tf_argmax(const float* logits, int ldl, int V, int rows, int* out, float* out_val,
                     cudaStream_t st) {
  argmax_kernel<<<rows, 1024, 0, st>>>(logits, ldl, V, out, out_val);
  return (int)cudaGetLastError();
}

TF_API int tf_rowstat_bytes() { return (int)sizeof(RowStat); }

TF_API int tf_rowstats(const float* logits, int ldl, int V, int rows, float temp, float top_p, void* out,
                       void* status, cudaStream_t st) {
  if (!(temp > 0.f)) return -1;
  rowstat_kernel<<<rows, 1024, 0, st>>>(logits, ldl, V, temp, top_p, (RowStat*)out, (TfStatusWord*)status);
  return (int)cudaGetLastError();
}

// Block verification of g proposals per conversation (g may be 0: plain sampling of one row).
TF_API int tf_spec_verify(const float* tlogits, const float* dlogits, const void* tstat, const void* dstat,
                          const int* proposals, const double* uniforms, int S, int g, int V, int ldl,
                          float t_temp, float d_temp, int point_mass, double* R, double* w, int* n_accept,
                          int* next_token, void* status, cudaStream_t st) {
  VerifyParams p;
  p.tlogits = tlogits; p.dlogits = dlogits; p.tstat = (const RowStat*)tstat; p.dstat = (const RowStat*)dstat;
  p.proposals = proposals; p.uniforms = uniforms; p.S = S; p.g = g; p.V = V; p.ldl = ldl;
  p.t_temp = t_temp; p.d_temp = d_temp; p.point_mass = point_mass; p.R = R; p.w = w;
  p.n_accept = n_accept; p.next_token = next_token; p.st = (TfStatusWord*)status;
  dim3 grid(S, g + 1);
  verify_mass_kernel<<<grid, 1024, 0, st>>>(p);
  verify_decide_kernel<<<S, 1024, 0, st>>>(p);
  return (int)cudaGetLastError();
}
