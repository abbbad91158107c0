// Sampling and speculative verification on fp32 logits.
//
//  * argmax (greedy; ties to the lowest id; reference kernels/core.cu:631-643)
//  * row statistics for temperature + nucleus (top-p) sampling: max, the order-preserving key of
//    the smallest logit inside the nucleus, and the nucleus mass, all in fp64
//  * block verification (Sun et al., arXiv:2403.10444; reference kernels/block_rejection.cuh:1-63):
//      w_0 = 1, w_i = min(1, w_{i-1} p_{i-1}(x_i) / q_{i-1}(x_i)),
//      R_i = sum_v max(w_i p_i(v) - q_i(v), 0),  h_i = R_i / (R_i + 1 - w_i) (i < g), h_g = w_g,
//      tau = max{ i : u_i < h_i } (0 if none); token at tau from the normalised residual (or from
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
  tf_pdl_sync();
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

// ---------------------------------------------------------------------------------------------
// Row statistics for temperature + nucleus sampling, spread over the whole GPU.
//
// A row of 129,280 logits is too long for one CTA to walk several times at decode latency, so
// every pass is a (rows x slices) grid and the passes talk through a small scratch area:
//   max pass      -> scratch.maxkey[row]          (atomicMax on the order-preserving key)
//   3 radix levels over the key (12 + 12 + 8 bits): a histogram pass adds each slice's
//     shared-memory histogram of MASS into scratch.hist[row][4096]; a pick pass (one CTA per
//     row) finds the first bin from the top whose inclusive cumulative mass reaches top_p * Z,
//     records the prefix, and clears the histogram for the next level / next call.
// Masses are 2^-40 fixed point: integer atomics make the sums independent of arrival order, so
// every rank that samples the same row derives bit-identical statistics.
// Scratch layout per row: RowScratch header (64 B) followed by 4096 uint64 bins; it must be
// zero before the first call and is left zero by every call.
// ---------------------------------------------------------------------------------------------
constexpr int kSlices = 16;
constexpr double kFix = 1099511627776.0;     // 2^40

struct RowScratch {
  unsigned int maxkey;       // fkey of the row maximum (0 = not yet computed)
  unsigned int prefix;       // key bits fixed so far
  unsigned int mask;         // which bits of the key are fixed
  int bad;                   // non-finite logit seen
  unsigned long long above;  // mass strictly above the current prefix bin
  unsigned long long total;  // Z in fixed point
  unsigned long long target; // top_p * Z in fixed point
  unsigned long long inbin;  // mass of the chosen bin at the last level
  unsigned long long pad[2];
};
static_assert(sizeof(RowScratch) == 64, "RowScratch is 64 bytes");
constexpr size_t kRowScratchBytes = sizeof(RowScratch) + 4096 * sizeof(unsigned long long);

__device__ __forceinline__ RowScratch* row_scratch(void* base, int r) {
  return reinterpret_cast<RowScratch*>(reinterpret_cast<uint8_t*>(base) + (size_t)r * kRowScratchBytes);
}
__device__ __forceinline__ unsigned long long* row_hist(void* base, int r) {
  return reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(base) + (size_t)r * kRowScratchBytes +
                                               sizeof(RowScratch));
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// slice bounds in units of float4
__device__ __forceinline__ void slice_range(int V4, int& lo, int& hi) {
  const int per = (V4 + gridDim.y - 1) / gridDim.y;
  lo = blockIdx.y * per;
  hi = min(V4, lo + per);
}

__global__ void __launch_bounds__(256) rowmax_kernel(const float* __restrict__ logits, int ldl, int V,
                                                     void* scratch) {
  tf_pdl_sync();
  const int r = blockIdx.x;
  const float4* x4 = reinterpret_cast<const float4*>(logits + (long)r * ldl);
  int lo, hi;
  slice_range(V / 4, lo, hi);
  float m = -INFINITY;
  int bad = 0;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float4 v = x4[i];
    const float a = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
    if (!(a < INFINITY) || isnan(v.x + v.y + v.z + v.w)) bad = 1;
    m = fmaxf(m, a);
  }
  if (blockIdx.y == gridDim.y - 1)
    for (int i = (V / 4) * 4 + threadIdx.x; i < V; i += blockDim.x) {
      const float v = logits[(long)r * ldl + i];
      if (!(v < INFINITY) || isnan(v)) bad = 1;
      m = fmaxf(m, v);
    }
  m = warp_max(m);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) {
    RowScratch* rs = row_scratch(scratch, r);
    if (m > -INFINITY) atomicMax(&rs->maxkey, fkey(m));
    if (bad) atomicExch(&rs->bad, 1);
  }
}

// level 0/1/2: shift 20/8/0, bins 4096/4096/256
__global__ void __launch_bounds__(256) rowhist_kernel(const float* __restrict__ logits, int ldl, int V,
                                                      float inv_t, const float* __restrict__ sess_temp, int rps,
                                                      int level, void* scratch) {
  tf_pdl_sync();
  __shared__ unsigned long long sh[4096];
  const int r = blockIdx.x;
  if (sess_temp) inv_t = __frcp_rn(sess_temp[r / rps]);    // IEEE reciprocal, as the host computes 1 / T
  RowScratch* rs = row_scratch(scratch, r);
  const int shift = level == 0 ? 20 : (level == 1 ? 8 : 0);
  const int nb = level == 2 ? 256 : 4096;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const float m = key_to_float(rs->maxkey);
  const uint32_t prefix = rs->prefix, mask = rs->mask;
  const float* x = logits + (long)r * ldl;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  int lo, hi;
  slice_range(V / 4, lo, hi);
  auto add = [&](float v) {
    const uint32_t key = fkey(v);
    if ((key & mask) == prefix)
      atomicAdd(&sh[(key >> shift) & (nb - 1)], (unsigned long long)((double)expf((v - m) * inv_t) * kFix));
  };
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float4 v = x4[i];
    add(v.x);
    add(v.y);
    add(v.z);
    add(v.w);
  }
  if (blockIdx.y == gridDim.y - 1)
    for (int i = (V / 4) * 4 + threadIdx.x; i < V; i += blockDim.x) add(x[i]);
  __syncthreads();
  unsigned long long* gh = row_hist(scratch, r);
  for (int i = threadIdx.x; i < nb; i += blockDim.x)
    if (sh[i]) atomicAdd(&gh[i], sh[i]);
}

// one CTA (1024 threads) per row: choose the bin, clear the histogram
__global__ void __launch_bounds__(1024) rowpick_kernel(int level, float top_p, const float* __restrict__ sess_top_p,
                                                       int rps, int last, RowStat* __restrict__ out, void* scratch,
                                                       TfStatusWord* st) {
  tf_pdl_sync();
  __shared__ unsigned long long chunk[32];
  const int r = blockIdx.x;
  if (sess_top_p) top_p = sess_top_p[r / rps];
  RowScratch* rs = row_scratch(scratch, r);
  unsigned long long* gh = row_hist(scratch, r);
  const int shift = level == 0 ? 20 : (level == 1 ? 8 : 0);
  const int nb = level == 2 ? 256 : 4096;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = nb / 32;
  unsigned long long sacc = 0;
  for (int j = lane; j < per; j += 32) sacc += gh[warp * per + j];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
  if (lane == 0) chunk[warp] = sacc;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (level == 0) {
      unsigned long long tot = 0;
      for (int w = 0; w < 32; ++w) tot += chunk[w];
      rs->total = tot;
      unsigned long long tg = top_p < 1.f ? (unsigned long long)((double)top_p * (double)tot) : 0ull;
      rs->target = tg ? tg : 1ull;
      rs->above = 0;
    }
    const unsigned long long target = rs->target;
    unsigned long long cum = rs->above;
    int w = 31;
    for (; w > 0; --w) {
      if (cum + chunk[w] >= target) break;
      cum += chunk[w];
    }
    int b = w * per + per - 1;
    for (; b > w * per; --b) {
      if (cum + gh[b] >= target) break;
      cum += gh[b];
    }
    rs->above = cum;
    rs->inbin = gh[b];
    rs->prefix |= (uint32_t)b << shift;
    rs->mask |= (uint32_t)(nb - 1) << shift;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nb; i += blockDim.x) gh[i] = 0;
  if (last && threadIdx.x == 0) {
    RowStat o;
    o.m = key_to_float(rs->maxkey);
    if (rs->bad) {
      tf_report(st, TF_NONFINITE, 20, r, 0);
      o.m = 0.f;
      o.thr = 0xffffffffu;
      o.z = 1.0;
    } else if (top_p < 1.f) {
      o.thr = rs->prefix;
      o.z = (double)(rs->above + rs->inbin) / kFix;
    } else {
      o.thr = 0;
      o.z = (double)rs->total / kFix;
    }
    out[r] = o;
    rs->maxkey = 0;
    rs->prefix = 0;
    rs->mask = 0;
    rs->bad = 0;
    rs->above = rs->total = rs->target = rs->inbin = 0;
  }
}

// ---------------------------------------------------------------------------------------------
// block verification
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ double prob_of(const float* x, const RowStat& s, float inv_t, int v) {
  const float l = x[v];
  if (fkey(l) < s.thr) return 0.0;
  return (double)expf((l - s.m) * inv_t) / s.z;
}

constexpr int kTile = 1024;

struct VerifyParams {
  const float* tlogits;     // [S, g+1, V] target rows
  const float* dlogits;     // [S, g, V] draft rows (null with point-mass proposals)
  const RowStat* tstat;     // [S*(g+1)]
  const RowStat* dstat;     // [S*g]
  const int* proposals;     // [S, g]
  const double* uniforms;   // [S, g+2]: u_1..u_g (acceptance), u_draw at index g, spare
  int S, g, V, ldl;
  float t_temp, d_temp;
  const float* sess_temp;   // [S] or null: temperature of conversation s for its target AND draft rows
  int point_mass;           // 1: q_i is a point mass at the proposal (text-lookup proposals)
  double* tile_mass;        // [S, g+1, ntiles] scratch: residual mass of every 1024-token tile
  double* w;                // [S, g+1] scratch
  int* n_accept;            // [S]
  int* next_token;          // [S]
  TfStatusWord* st;
};

// acceptance weight after i accepted proposals: w_0 = 1, w_i = min(1, w_{i-1} p_{i-1}(x_i) / q_{i-1}(x_i))
__device__ double weight_chain(const VerifyParams& p, int s, int i) {
  double w = 1.0;
  for (int j = 1; j <= i; ++j) {
    const int x = p.proposals[s * p.g + j - 1];
    const float* tx = p.tlogits + ((long)s * (p.g + 1) + j - 1) * p.ldl;
    const double pt = prob_of(tx, p.tstat[s * (p.g + 1) + j - 1], __frcp_rn(p.sess_temp ? p.sess_temp[s] : p.t_temp), x);
    double q = 1.0;
    if (!p.point_mass) {
      const float* dx = p.dlogits + ((long)s * p.g + j - 1) * p.ldl;
      q = prob_of(dx, p.dstat[s * p.g + j - 1], __frcp_rn(p.sess_temp ? p.sess_temp[s] : p.d_temp), x);
    }
    const double ratio = q > 0.0 ? w * pt / q : (pt > 0.0 ? 1.0 : 0.0);
    w = ratio < 1.0 ? ratio : 1.0;
  }
  return w;
}

// residual value at token v of row i: max(w_i p_i(v) - q_i(v), 0); the bonus row (i == g) has q = 0.
// wz = w_i / Z_target, qz = 1 / Z_draft are hoisted by the callers.
struct RowCtx {
  const float* tx;
  const float* dx;
  float tm, dm, t_inv, d_inv;
  uint32_t tthr, dthr;
  double wz, qz;
  int point_tok;            // >= 0: point-mass proposal at this token
};
__device__ __forceinline__ RowCtx row_ctx(const VerifyParams& p, int s, int i, double wi) {
  RowCtx c;
  const RowStat ts = p.tstat[s * (p.g + 1) + i];
  c.tx = p.tlogits + ((long)s * (p.g + 1) + i) * p.ldl;
  c.tm = ts.m;
  c.tthr = ts.thr;
  c.t_inv = __frcp_rn(p.sess_temp ? p.sess_temp[s] : p.t_temp);
  c.wz = wi / ts.z;
  c.dx = nullptr;
  c.point_tok = -1;
  c.dm = 0.f;
  c.dthr = 0;
  c.d_inv = __frcp_rn(p.sess_temp ? p.sess_temp[s] : p.d_temp);
  c.qz = 0.0;
  if (i < p.g) {
    if (p.point_mass) c.point_tok = p.proposals[s * p.g + i];
    else {
      const RowStat ds = p.dstat[s * p.g + i];
      c.dx = p.dlogits + ((long)s * p.g + i) * p.ldl;
      c.dm = ds.m;
      c.dthr = ds.thr;
      c.qz = 1.0 / ds.z;
    }
  }
  return c;
}
__device__ __forceinline__ double residual(const RowCtx& c, int v) {
  const float l = c.tx[v];
  double val = fkey(l) >= c.tthr ? c.wz * (double)expf((l - c.tm) * c.t_inv) : 0.0;
  if (c.dx) {
    const float d = c.dx[v];
    if (fkey(d) >= c.dthr) val -= c.qz * (double)expf((d - c.dm) * c.d_inv);
  } else if (v == c.point_tok) {
    val -= 1.0;
  }
  return val > 0.0 ? val : 0.0;
}

// grid (S * (g+1), ntiles), 256 threads: residual mass of one 1024-token tile of one row
__global__ void __launch_bounds__(256) verify_tiles_kernel(VerifyParams p) {
  tf_pdl_sync();
  __shared__ double s_w;
  __shared__ double wsum[8];
  const int row = blockIdx.x, s = row / (p.g + 1), i = row % (p.g + 1), tile = blockIdx.y;
  if (threadIdx.x == 0) s_w = weight_chain(p, s, i);
  __syncthreads();
  const RowCtx c = row_ctx(p, s, i, s_w);
  double acc = 0.0;
  const int v0 = tile * kTile + threadIdx.x * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (v0 + j < p.V) acc += residual(c, v0 + j);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int k = 0; k < 8; ++k) t += wsum[k];
    p.tile_mass[(long)row * gridDim.y + tile] = t;
  }
}

// grid S, 1024 threads: acceptance length and the emitted token
__global__ void __launch_bounds__(1024) verify_decide_kernel(VerifyParams p, int ntiles) {
  tf_pdl_sync();
  __shared__ double scan[1024];
  __shared__ double Rrow[64], wrow[64];
  __shared__ int s_tau, s_tile, s_tok;
  __shared__ double s_target;
  const int s = blockIdx.x, g = p.g;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // R_i: fixed-order sums of the tile masses (one warp per row)
  for (int i = warp; i <= g; i += 32) {
    const double* tm = p.tile_mass + ((long)s * (g + 1) + i) * ntiles;
    double acc = 0.0;
    for (int t = lane; t < ntiles; t += 32) acc += tm[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) Rrow[i] = acc;
  }
  if (threadIdx.x == 0)
    for (int i = 0; i <= g; ++i) {
      wrow[i] = weight_chain(p, s, i);
      p.w[s * (g + 1) + i] = wrow[i];
    }
  __syncthreads();
  if (threadIdx.x == 0) {
    const double* u = p.uniforms + (long)s * (g + 2);
    int tau = 0;
    for (int i = 1; i <= g; ++i) {
      const double R = Rrow[i], w = wrow[i];
      if (!(R >= 0.0) || isinf(R)) tf_report(p.st, TF_NONFINITE, 21, s, i);
      const double h = (i < g) ? (R + 1.0 - w > 0.0 ? R / (R + 1.0 - w) : 0.0) : w;
      if (u[i - 1] < h) tau = i;
    }
    s_tau = tau;
    s_tok = -1;
    const double* tm = p.tile_mass + ((long)s * (g + 1) + tau) * ntiles;
    const double total = Rrow[tau];
    double target = u[g] * total;
    if (target >= total) target = nextafter(total, 0.0);
    int tl = 0;
    double before = 0.0;
    for (; tl < ntiles - 1; ++tl) {
      if (before + tm[tl] > target) break;
      before += tm[tl];
    }
    s_tile = tl;
    s_target = target - before;
    if (!(total > 0.0)) tf_report(p.st, TF_NONFINITE, 23, s, tau);
  }
  __syncthreads();
  const int tau = s_tau;
  const RowCtx c = row_ctx(p, s, tau, wrow[tau]);
  const int v = s_tile * kTile + threadIdx.x;
  const double val = v < p.V ? residual(c, v) : 0.0;
  scan[threadIdx.x] = val;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const double add = threadIdx.x >= d ? scan[threadIdx.x - d] : 0.0;
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
        const double pv = j ? scan[j] - scan[j - 1] : scan[0];
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
  tf_launch(argmax_kernel, dim3(rows), dim3(1024), 0, st, logits, ldl, V, out, out_val);
  return (int)cudaGetLastError();
}

TF_API int tf_rowstat_bytes() { return (int)sizeof(RowStat); }

// bytes of zero-initialised scratch tf_rowstats needs for `rows` rows
TF_API long tf_rowstats_scratch_bytes(int rows) { return (long)rows * (long)kRowScratchBytes; }

// scratch: tf_rowstats_scratch_bytes(rows) bytes, zero before the first call (left zero by each call).
// sess_temp / sess_top_p (device arrays, may be null): per-conversation settings, row r belonging to
// conversation r / rows_per_sess; they override the scalars, so requests with different sampling
// settings share one launch (and one captured graph).  The host must have validated them
// (temperature > 0, 0 < top_p <= 1).
static int rowstats_launch(const float* logits, int ldl, int V, int rows, float temp, float top_p,
                           const float* sess_temp, const float* sess_top_p, int rows_per_sess, void* out,
                           void* scratch, void* status, cudaStream_t st) {
  if (logits == nullptr || out == nullptr || scratch == nullptr || rows <= 0 || V <= 0 || ldl < V) return -1;
  if (!(temp > 0.f) || !(top_p > 0.f && top_p <= 1.f) || (ldl % 4) != 0 || (((uintptr_t)logits) & 15) != 0) return -1;
  if ((sess_temp || sess_top_p) && rows_per_sess <= 0) return -1;
  const float inv_t = 1.f / temp;
  const int rps = rows_per_sess > 0 ? rows_per_sess : 1;
  dim3 grid(rows, kSlices);
  tf_launch(rowmax_kernel, dim3(grid), dim3(256), 0, st, logits, ldl, V, scratch);
  const int levels = (sess_top_p || top_p < 1.f) ? 3 : 1;
  for (int level = 0; level < levels; ++level) {
    tf_launch(rowhist_kernel, dim3(grid), dim3(256), 0, st, logits, ldl, V, inv_t, sess_temp, rps, level, scratch);
    tf_launch(rowpick_kernel, dim3(rows), dim3(1024), 0, st, level, top_p, sess_top_p, rps, level == levels - 1, (RowStat*)out, scratch,
                                          (TfStatusWord*)status);
  }
  return (int)cudaGetLastError();
}

TF_API int tf_rowstats(const float* logits, int ldl, int V, int rows, float temp, float top_p, void* out,
                       void* scratch, void* status, cudaStream_t st) {
  return rowstats_launch(logits, ldl, V, rows, temp, top_p, nullptr, nullptr, 1, out, scratch, status, st);
}

// tf_rowstats with per-conversation temperature / top-p arrays (see rowstats_launch)
TF_API int tf_rowstats_per_session(const float* logits, int ldl, int V, int rows, const float* sess_temp,
                                   const float* sess_top_p, int rows_per_sess, void* out, void* scratch,
                                   void* status, cudaStream_t st) {
  if (!sess_temp || !sess_top_p) return -1;
  return rowstats_launch(logits, ldl, V, rows, 1.f, 1.f, sess_temp, sess_top_p, rows_per_sess, out, scratch, status, st);
}

// doubles of scratch tf_spec_verify needs in `tile_mass`
TF_API long tf_spec_verify_scratch_doubles(int S, int g, int V) {
  return (long)S * (g + 1) * ((V + kTile - 1) / kTile);
}

// Block verification of g proposals per conversation (g may be 0: plain sampling of one row).
TF_API int tf_spec_verify(const float* tlogits, const float* dlogits, const void* tstat, const void* dstat,
                          const int* proposals, const double* uniforms, int S, int g, int V, int ldl,
                          float t_temp, float d_temp, const float* sess_temp, int point_mass, double* tile_mass,
                          double* w, int* n_accept, int* next_token, void* status, cudaStream_t st) {
  if (g > 62 || g < 0 || S <= 0 || V <= 0 || !tlogits || !tstat || !uniforms || !tile_mass || !w || !n_accept ||
      !next_token)
    return -1;
  if (g > 0 && (!proposals || (!point_mass && (!dlogits || !dstat)))) return -1;
  if (!sess_temp && (!(t_temp > 0.f) || !(d_temp > 0.f))) return -1;
  VerifyParams p;
  p.tlogits = tlogits; p.dlogits = dlogits; p.tstat = (const RowStat*)tstat; p.dstat = (const RowStat*)dstat;
  p.proposals = proposals; p.uniforms = uniforms; p.S = S; p.g = g; p.V = V; p.ldl = ldl;
  p.t_temp = t_temp; p.d_temp = d_temp; p.sess_temp = sess_temp; p.point_mass = point_mass; p.tile_mass = tile_mass; p.w = w;
  p.n_accept = n_accept; p.next_token = next_token; p.st = (TfStatusWord*)status;
  const int ntiles = (V + kTile - 1) / kTile;
  dim3 grid(S * (g + 1), ntiles);
  tf_launch(verify_tiles_kernel, dim3(grid), dim3(256), 0, st, p);
  tf_launch(verify_decide_kernel, dim3(S), dim3(1024), 0, st, p, ntiles);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// tf_rowstats with library-owned scratch (contract in rowstats_static.h)
// ---------------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>

#include "rowstats_static.h"

static __device__ __align__(256) unsigned char g_rowstats_static_scratch[TF_ROWSTATS_STATIC_MAX_ROWS * kRowScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

// address of this device's copy of the array; looked up once per device
cudaError_t static_scratch(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_rowstats_static_scratch);
    if (e != cudaSuccess) return e;
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return cudaSuccess;
}
}  // namespace

TF_API int tf_rowstats_static(const float* logits, int ldl, int V, int rows, float temp, float top_p, void* out,
                              void* status, cudaStream_t st) {
  if (rows > TF_ROWSTATS_STATIC_MAX_ROWS) {
    fprintf(stderr, "tf_rowstats_static: %d rows exceed the built-in scratch of %d rows; use tf_rowstats\n", rows,
            TF_ROWSTATS_STATIC_MAX_ROWS);
    return TF_ROWSTATS_STATIC_TOO_MANY_ROWS;
  }
  if (rows <= 0 || V <= 0 || out == nullptr || logits == nullptr || ldl < V) return -1;
  if (!(temp > 0.f) || !(top_p > 0.f && top_p <= 1.f) || (ldl % 4) != 0 || (((uintptr_t)logits) & 15) != 0) return -1;
  void* scratch = nullptr;
  cudaError_t e = static_scratch(&scratch);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(scratch, 0, (size_t)rows * kRowScratchBytes, st);
  if (e != cudaSuccess) return (int)e;
  return tf_rowstats(logits, ldl, V, rows, temp, top_p, out, scratch, status, st);
}
