// Rank-local sampling and block verification over a vocabulary that is split into chunks.
//
// The vocabulary is cut into P chunks of at most 16,384 logits (P a multiple of 8, so 1, 2, 4 or 8
// ranks own whole chunks: rank k holds chunks [k * P / world, (k + 1) * P / world) of every row).
// One CTA per (row, chunk) stages its chunk in shared memory once and then takes part in a short
// series of exchanges with the other chunks of the row -- CTAs of the same GPU and of the peer GPUs
// alike -- through 8-byte {payload, tag} words pushed into every rank's workspace (the in-band-epoch
// protocol of comm.cuh).  Nothing else crosses NVLink: no rank ever sees another rank's logits.
//
//   1. row maximum                       (1 word per chunk)
//   2. nucleus threshold by a 4 x 8-bit radix select over the order-preserving key, on histograms
//      of 2^-40 fixed-point MASS: integer sums, independent of arrival order and of the number of
//      ranks                              (256 bins per chunk and level)
//   3. probabilities of the proposals under the target and the draft law (the chunk that owns the
//      proposed token publishes them)
//   4. residual mass of every chunk, R_i = sum_v max(w_i p_i(v) - q_i(v), 0), fp64, fixed order
//   5. the emitted token (the chunk that holds it publishes it)
//
// Every rank derives the same acceptance length from the same exchanged numbers, so all ranks
// commit identical tokens; and because the chunking does not depend on the number of ranks, a
// conversation samples the same tokens on 1, 2, 4 or 8 GPUs for the same logits and seeds.
// With g = 0 the kernel is the plain temperature / top-p sampler of a row (used for the draft
// proposals); it also leaves the row statistics (max, threshold key, normaliser) for a later
// verification launch.
//
// Arithmetic contract: block verification of Sun et al. (arXiv:2403.10444) on the temperature- and
// nucleus-modified laws, as csrc/sampling.cu (reference: kernels/block_rejection.cuh:1-63,
// kernels/categorical.cuh:14-60; rank-local form src/sharded_block.rs:111-161,
// src/rejection_sharded.rs, src/hierarchical_categorical.rs:70-183, kernels/sharded_block.cuh).
//
// Every wait is bounded; a wait that runs out records TF_TIMEOUT (kernel id 210, detail = (exchange,
// row)) and the CTA returns.  The grid always spans max_rows rows so that the call counters of all
// CTAs advance together; rows beyond the live count return at once.
#include "comm.cuh"

namespace {

constexpr int kChunkMax = 16384;
constexpr int kThreads = 1024;
constexpr int kMaxP = 16;          // chunks per row
constexpr int kMaxG = 15;          // proposals per conversation
constexpr double kFix = 1099511627776.0;     // 2^40

struct RowStat {                   // same layout as csrc/sampling.cu
  float m;
  uint32_t thr;
  double z;
};

__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct ChunkParams {
  const float* tlogits;     // [S * (g+1), ldl] this rank's columns of the target rows
  const float* dlogits;     // [S * g, ldl] draft rows (null: none / point-mass proposals)
  const RowStat* dstat;     // [S * g] statistics of the draft rows (from earlier g = 0 launches)
  const int* proposals;     // [S, g]
  const double* uniforms;   // conversation s: acceptance draws u[s * u_stride + 0..g-1], final draw at + g
  int u_stride;
  const float* sess_temp;   // [S]
  const float* sess_top_p;  // [S]
  int S, g, V, ldl, chunk, P, csplit;
  int point_mass;
  const int* sess_point;    // [S] or null: 1 = this conversation's proposals are point masses (copy proposals)
  const int* forced;        // g = 0 only, [S] at forced[s * tok_stride] or null: conversations flagged in
                            // sess_point emit this token instead of the draw (their proposal is known)
  const int* sess_g;        // [S] or null: conversation s verifies only its first sess_g[s] proposals (1..g); the
                            // row after them is its bonus row and later rows are ignored (causal stopping)
  RowStat* tstat;           // out: statistics of the target rows, row r at tstat[r * stat_stride]
  int stat_stride;
  int* n_accept;            // out [S] (may be null)
  int* next_token;          // out: conversation s at next_token[s * tok_stride]
  int tok_stride;
  // exchange
  const unsigned long long* peers;   // [world] workspace bases
  int world, rank, max_rows;
  unsigned int* ctr;        // [grid.z][max_rows * csplit] call counters of this rank's CTAs
  int spin_limit;
  TfStatusWord* st;
  // emulated ranks (grid.z > 1): element strides between ranks of the local arrays
  long emu_tl, emu_dl, emu_stat, emu_tok, emu_acc;
};

// workspace areas, in 64-bit words from the base (every area double-buffered)
struct Areas {
  long maxw, hist, prop, mass, tok, total;
};
__host__ __device__ inline Areas areas(int P, int R) {
  Areas a;
  a.maxw = 0;
  a.hist = a.maxw + 2L * P * R * 2;
  a.prop = a.hist + 2L * P * R * 256 * 2;
  a.mass = a.prop + 2L * R * 4;
  a.tok = a.mass + 2L * P * R * 2;
  a.total = a.tok + 2L * R * 2;
  return a;
}

struct Waiter {
  int spin_limit;
  TfStatusWord* st;
  long long t0;
  int* fail;
  __device__ __forceinline__ ulonglong2 wait(const unsigned long long* p, unsigned int tag, int what, int row) const {
    ulonglong2 v = ld_ll2(p);
    int spins = 0;
    while (!ll_ready(v, tag)) {
      if (*fail || ++spins > spin_limit || clock64() - t0 > 2000000000LL) {
        tf_report(st, TF_TIMEOUT, 210, what, row);
        *fail = 1;
        break;
      }
      v = ld_ll2(p);
    }
    return v;
  }
};

__device__ __forceinline__ void push2(const ChunkParams& p, long word, uint32_t a, uint32_t b, unsigned int tag) {
  for (int r = 0; r < p.world; ++r) {
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.peers[r]) + word;
    st_ll(dst, a, tag);
    st_ll(dst + 1, b, tag);
  }
}
__device__ __forceinline__ void push_double(const ChunkParams& p, long word, double v, unsigned int tag) {
  const unsigned long long b = (unsigned long long)__double_as_longlong(v);
  push2(p, word, (uint32_t)b, (uint32_t)(b >> 32), tag);
}
__device__ __forceinline__ double pair_double(const ulonglong2& v) {
  return __longlong_as_double((long long)(((v.y & 0xffffffffull) << 32) | (v.x & 0xffffffffull)));
}
__device__ __forceinline__ unsigned long long pair_u64(const ulonglong2& v) {
  return ((v.y & 0xffffffffull) << 32) | (v.x & 0xffffffffull);
}

__device__ __forceinline__ double prob_of(float l, const RowStat& s, float inv_t) {
  if (fkey(l) < s.thr) return 0.0;
  return (double)expf((l - s.m) * inv_t) / s.z;
}

__global__ void __launch_bounds__(kThreads, 1) sample_chunks_kernel(const ChunkParams p) {
  tf_pdl_sync();
  extern __shared__ __align__(16) unsigned char smem[];
  float* tbuf = reinterpret_cast<float*>(smem);
  float* dbuf = tbuf + p.chunk;
  unsigned long long* whist = reinterpret_cast<unsigned long long*>(dbuf + p.chunk);   // [32][256]
  __shared__ unsigned long long gbins[256], gpart[4][256];
  __shared__ double wm[32], cm[(kMaxG + 1) * kMaxP], Rrow[kMaxG + 1], wrow[kMaxG + 1], ptq[2 * kMaxG];
  __shared__ float redf[32];
  __shared__ int redi[32];
  __shared__ unsigned int s_call, s_key[kMaxP], s_bad[kMaxP];
  __shared__ unsigned int s_prefix, s_mask;
  __shared__ unsigned long long s_above, s_total, s_target, s_inbin;
  __shared__ int s_fail, s_tau, s_chunk, s_warp;
  __shared__ double s_draw;

  const int row = blockIdx.x, lc = blockIdx.y, ez = blockIdx.z;
  const int rank = p.rank + ez, part = rank * p.csplit + lc;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = p.g, R1 = g + 1, P = p.P;
  if (threadIdx.x == 0) {
    s_call = ++p.ctr[((long)ez * p.max_rows + row) * p.csplit + lc];
    s_fail = 0;
  }
  __syncthreads();
  if (row >= p.S * R1) return;
  const unsigned int call = s_call, par = call & 1;
  const unsigned int tag0 = call << 4;
  const int s = row / R1, i = row % R1;
  const Areas A = areas(P, p.max_rows);
  const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(p.peers[rank]);
  Waiter W{p.spin_limit, p.st, clock64(), &s_fail};

  // ---- stage this chunk of the target row (and of the draft row it is verified against)
  const int n = p.chunk;
  const float* trow = p.tlogits + ez * p.emu_tl + (long)row * p.ldl + (long)lc * n;
  const bool point = p.point_mass || (p.sess_point && p.sess_point[s]);
  // proposals this conversation verifies: rows past its bonus row still publish (every CTA of the
  // block takes part in the exchanges) but nothing reads what they publish
  const int gs = (g > 0 && p.sess_g) ? min(max(p.sess_g[s], 1), g) : g;
  const bool has_d = (i < gs) && p.dlogits != nullptr && !point;
  const float* drow = has_d ? p.dlogits + ez * p.emu_dl + (long)(s * g + i) * p.ldl + (long)lc * n : nullptr;
  for (int k = threadIdx.x * 4; k < n; k += kThreads * 4) {
    *reinterpret_cast<float4*>(tbuf + k) = *reinterpret_cast<const float4*>(trow + k);
    if (has_d) *reinterpret_cast<float4*>(dbuf + k) = *reinterpret_cast<const float4*>(drow + k);
  }
  __syncthreads();
  // IEEE reciprocal (not the fast-math approximation): every kernel and the host agree on 1 / T bit for bit
  const float inv_t = __frcp_rn(p.sess_temp[s]);
  const float top_p = p.sess_top_p[s];

  // ---- 1. row maximum
  float m = -INFINITY;
  int bad = 0;
  for (int k = threadIdx.x; k < n; k += kThreads) {
    const float v = tbuf[k];
    if (!(v < INFINITY) || isnan(v)) bad = 1;
    m = fmaxf(m, v);
  }
  m = warp_max(m);
  bad = __any_sync(0xffffffffu, bad);
  if (lane == 0) {
    redf[warp] = m;
    redi[warp] = bad;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = -INFINITY;
    int b2 = 0;
    for (int w = 0; w < 32; ++w) {
      b2 |= redi[w];
      if (!redi[w]) mm = fmaxf(mm, redf[w]);
    }
    push2(p, A.maxw + (((long)par * P + part) * p.max_rows + row) * 2, mm > -INFINITY ? fkey(mm) : 0u, (uint32_t)b2, tag0);
  }
  if (threadIdx.x < P) {
    const ulonglong2 v = W.wait(mine + A.maxw + (((long)par * P + threadIdx.x) * p.max_rows + row) * 2, tag0, 0, row);
    s_key[threadIdx.x] = (uint32_t)v.x;
    s_bad[threadIdx.x] = (uint32_t)v.y;
  }
  __syncthreads();
  if (s_fail) return;
  uint32_t mkey = 0;
  int anybad = 0;
  for (int q = 0; q < P; ++q) {
    mkey = max(mkey, s_key[q]);
    anybad |= (int)s_bad[q];
  }
  RowStat stat;
  stat.m = key_to_float(mkey);

  // ---- 2. nucleus threshold: radix select on mass histograms (levels of 8 key bits, top first)
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_mask = 0;
    s_above = 0;
  }
  const int levels = anybad ? 0 : (top_p < 1.f ? 4 : 1);
  for (int level = 0; level < levels; ++level) {
    const int shift = 24 - 8 * level;
    const unsigned int tag = tag0 + 1 + level;
    for (int k = threadIdx.x; k < 32 * 256; k += kThreads) whist[k] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    {
      // a thread's consecutive elements mostly fall into the same few bins (the top key bits are the
      // sign and the exponent): add up a run privately and touch shared memory once per run
      int cur = -1;
      unsigned long long run = 0;
      for (int k = threadIdx.x; k < n; k += kThreads) {
        const float v = tbuf[k];
        const uint32_t key = fkey(v);
        if ((key & mask) != prefix) continue;
        const int bin = (key >> shift) & 255;
        const unsigned long long mass = (unsigned long long)((double)expf((v - stat.m) * inv_t) * kFix);
        if (bin != cur) {
          if (cur >= 0) atomicAdd(&whist[warp * 256 + cur], run);
          cur = bin;
          run = 0;
        }
        run += mass;
      }
      if (cur >= 0) atomicAdd(&whist[warp * 256 + cur], run);
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      unsigned long long acc = 0;
      for (int w = 0; w < 32; ++w) acc += whist[w * 256 + threadIdx.x];
      push2(p, A.hist + ((((long)(level & 1) * P + part) * p.max_rows + row) * 256 + threadIdx.x) * 2, (uint32_t)acc,
            (uint32_t)(acc >> 32), tag);
    }
    {
      // every thread polls one bin of up to four source chunks, all loads in flight at once
      const int bin = threadIdx.x & 255, qg = threadIdx.x >> 8;
      const unsigned long long* src0 = mine + A.hist + ((((long)(level & 1) * P) * p.max_rows + row) * 256 + bin) * 2;
      const long qstride = (long)p.max_rows * 256 * 2;
      ulonglong2 v[4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
        if (qg + 4 * t < P) v[t] = ld_ll2(src0 + (qg + 4 * t) * qstride);
      unsigned long long tot = 0;
#pragma unroll
      for (int t = 0; t < 4; ++t)
        if (qg + 4 * t < P) {
          if (!ll_ready(v[t], tag)) v[t] = W.wait(src0 + (qg + 4 * t) * qstride, tag, 1 + level, row);
          tot += pair_u64(v[t]);
        }
      gpart[qg][bin] = tot;
    }
    __syncthreads();
    if (s_fail) return;
    if (threadIdx.x < 256)
      gbins[threadIdx.x] = gpart[0][threadIdx.x] + gpart[1][threadIdx.x] + gpart[2][threadIdx.x] + gpart[3][threadIdx.x];
    __syncthreads();
    if (threadIdx.x == 0) {
      if (level == 0) {
        unsigned long long tot = 0;
        for (int b = 0; b < 256; ++b) tot += gbins[b];
        s_total = tot;
        const unsigned long long tg = top_p < 1.f ? (unsigned long long)((double)top_p * (double)tot) : 0ull;
        s_target = tg ? tg : 1ull;
      }
      const unsigned long long target = s_target;
      unsigned long long cum = s_above;
      int b = 255;
      for (; b > 0; --b) {
        if (cum + gbins[b] >= target) break;
        cum += gbins[b];
      }
      s_above = cum;
      s_inbin = gbins[b];
      s_prefix |= (uint32_t)b << shift;
      s_mask |= 255u << shift;
    }
    __syncthreads();
  }
  if (anybad) {
    if (threadIdx.x == 0 && lc == 0) tf_report(p.st, TF_NONFINITE, 20, row, 0);
    stat.m = 0.f;
    stat.thr = 0xffffffffu;
    stat.z = 1.0;
  } else if (top_p < 1.f) {
    stat.thr = s_prefix;
    stat.z = (double)(s_above + s_inbin) / kFix;
  } else {
    stat.thr = 0;
    stat.z = (double)s_total / kFix;
  }
  if (threadIdx.x == 0 && lc == 0) p.tstat[ez * p.emu_stat + (long)row * p.stat_stride] = stat;

  // ---- 3. probabilities of the proposals (published by the chunk that owns the token)
  const long base = (long)part * n;
  RowStat ds;
  float d_inv = inv_t;
  ds.m = 0.f; ds.thr = 0; ds.z = 1.0;
  if (has_d && p.dstat) ds = p.dstat[s * g + i];
  if (g > 0) {
    if (i < g && threadIdx.x == 0) {
      const int x = p.proposals[s * g + i];
      if (x >= base && x < base + n) {
        const double pt = prob_of(tbuf[x - base], stat, inv_t);
        const double q = (point || !has_d) ? 1.0 : prob_of(dbuf[x - base], ds, d_inv);
        const long w0 = A.prop + ((long)par * p.max_rows + row) * 4;
        push_double(p, w0, pt, tag0 + 5);
        push_double(p, w0 + 2, q, tag0 + 5);
      }
    }
    if (threadIdx.x < 2 * g) {
      const int j = threadIdx.x >> 1, h = threadIdx.x & 1;
      ptq[threadIdx.x] = pair_double(W.wait(mine + A.prop + ((long)par * p.max_rows + s * R1 + j) * 4 + 2 * h, tag0 + 5, 5,
                                            row));
    }
    __syncthreads();
    if (s_fail) return;
  }
  if (threadIdx.x == 0) {
    // w_0 = 1, w_j = min(1, w_{j-1} p_{j-1}(x_j) / q_{j-1}(x_j))
    double w = 1.0;
    wrow[0] = 1.0;
    for (int j = 1; j <= g; ++j) {
      const double pt = ptq[2 * (j - 1)], q = ptq[2 * (j - 1) + 1];
      const double ratio = q > 0.0 ? w * pt / q : (pt > 0.0 ? 1.0 : 0.0);
      w = ratio < 1.0 ? ratio : 1.0;
      wrow[j] = w;
    }
  }
  __syncthreads();

  // ---- 4. residual mass of this chunk: max(w_i p_i(v) - q_i(v), 0); the bonus row has q = 0
  const double wz = wrow[i] / stat.z;
  const double qz = has_d ? 1.0 / ds.z : 0.0;
  const int point_tok = (i < gs && point) ? p.proposals[s * g + i] : -1;
  auto residual = [&](int k) -> double {
    const float l = tbuf[k];
    double val = fkey(l) >= stat.thr ? wz * (double)expf((l - stat.m) * inv_t) : 0.0;
    if (qz > 0.0) {
      const float d = dbuf[k];
      if (fkey(d) >= ds.thr) val -= qz * (double)expf((d - ds.m) * d_inv);
    } else if (base + k == point_tok) {
      val -= 1.0;
    }
    return val > 0.0 ? val : 0.0;
  };
  double my_mass = 0.0;
  for (int k = threadIdx.x; k < n; k += kThreads) my_mass += residual(k);
  double wsum = my_mass;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
  if (lane == 0) wm[warp] = wsum;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 32; ++w) t += wm[w];
    push_double(p, A.mass + (((long)par * P + part) * p.max_rows + row) * 2, t, tag0 + 6);
  }
  if (threadIdx.x < R1 * P) {
    const int ii = threadIdx.x / P, q = threadIdx.x % P;
    cm[ii * kMaxP + q] = pair_double(W.wait(mine + A.mass + (((long)par * P + q) * p.max_rows + s * R1 + ii) * 2, tag0 + 6,
                                            6, row));
  }
  __syncthreads();
  if (s_fail) return;
  if (threadIdx.x == 0) {
    for (int ii = 0; ii <= g; ++ii) {
      double t = 0.0;
      for (int q = 0; q < P; ++q) t += cm[ii * kMaxP + q];
      Rrow[ii] = t;
    }
    const double* u = p.uniforms + (long)s * p.u_stride;
    int tau = 0;
    for (int ii = 1; ii <= gs; ++ii) {
      const double Rr = Rrow[ii], w = wrow[ii];
      if (!(Rr >= 0.0) || isinf(Rr)) tf_report(p.st, TF_NONFINITE, 21, s, ii);
      const double h = (ii < gs) ? (Rr + 1.0 - w > 0.0 ? Rr / (Rr + 1.0 - w) : 0.0) : w;
      if (u[ii - 1] < h) tau = ii;
    }
    s_tau = tau;
    const double total = Rrow[tau];
    double target = u[g] * total;
    if (target >= total) target = nextafter(total, 0.0);
    int q = 0;
    double before = 0.0;
    for (; q < P - 1; ++q) {
      if (before + cm[tau * kMaxP + q] > target) break;
      before += cm[tau * kMaxP + q];
    }
    s_chunk = q;
    s_draw = target - before;
    if (!(total > 0.0) && i == 0 && lc == 0) tf_report(p.st, TF_NONFINITE, 23, s, tau);
  }
  __syncthreads();
  const int tau = s_tau;

  // ---- 5. the chunk that holds the draw finds the token: warp, lane, element
  if (i == tau && part == s_chunk) {
    if (threadIdx.x == 0) {
      double before = 0.0;
      int w = 0;
      for (; w < 31; ++w) {
        if (before + wm[w] > s_draw) break;
        before += wm[w];
      }
      // rounding can leave the draw past the last positive warp: step back to one that has mass
      while (w > 0 && !(wm[w] > 0.0)) --w;
      s_warp = w;
      s_draw -= before;
    }
    __syncthreads();
    if (warp == s_warp) {
      // inclusive scan of the lane masses in lane order
      double incl = my_mass;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const double excl = incl - my_mass, draw = s_draw;
      const bool hit = my_mass > 0.0 && excl <= draw && draw < incl;
      unsigned int hits = __ballot_sync(0xffffffffu, hit);
      if (!hits) {
        // rounding left the draw past the last positive lane: take that lane
        const unsigned int pos = __ballot_sync(0xffffffffu, my_mass > 0.0);
        hits = pos ? (1u << (31 - __clz(pos))) : 1u;
      }
      const int winner = __ffs(hits) - 1;
      if (lane == winner) {
        double rest = draw - excl, acc = 0.0;
        int tok = -1, last_pos = -1;
        for (int k = threadIdx.x; k < n; k += kThreads) {
          const double v = residual(k);
          if (v > 0.0) {
            last_pos = k;
            if (acc + v > rest) {
              tok = k;
              break;
            }
            acc += v;
          }
        }
        if (tok < 0) tok = last_pos;
        if (tok < 0) {
          tf_report(p.st, TF_NONFINITE, 24, s, tau);
          tok = 0;
        }
        push2(p, A.tok + ((long)par * p.max_rows + s) * 2, (uint32_t)(base + tok), (uint32_t)tau, tag0 + 7);
      }
    }
  }
  if (i == 0 && lc == 0 && threadIdx.x == 0) {
    const ulonglong2 v = W.wait(mine + A.tok + ((long)par * p.max_rows + s) * 2, tag0 + 7, 7, row);
    if (!s_fail) {
      int tok = (int)(uint32_t)v.x;
      if (g == 0 && p.forced && p.sess_point && p.sess_point[s]) tok = p.forced[(long)s * p.tok_stride];
      p.next_token[ez * p.emu_tok + (long)s * p.tok_stride] = tok;
      if (p.n_accept) p.n_accept[ez * p.emu_acc + s] = (int)(uint32_t)v.y;
    }
  }
}

}  // namespace

// chunks per row and logits per chunk for a vocabulary of V (0 = this V cannot be chunked: V must be
// a multiple of 32 * P)
TF_API int tf_sample_chunks_count(int V) {
  if (V <= 0) return 0;
  const int P = 8 * ((V + 8 * kChunkMax - 1) / (8 * kChunkMax));
  if (P > kMaxP || V % P != 0 || (V / P) % 4 != 0) return 0;
  return P;
}

// bytes of (symmetric, zero-initialised) workspace per rank
TF_API long tf_sample_chunks_workspace_bytes(int V, int max_rows) {
  const int P = tf_sample_chunks_count(V);
  return P ? areas(P, max_rows).total * 8 : 0;
}

// One launch = row statistics + block verification (g > 0) or plain sampling (g = 0) of S
// conversations; see the header of this file.  sess_point [S] (optional) flags conversations whose
// proposals are point masses (copy proposals found on the host); in a g = 0 launch such a
// conversation emits forced[s * tok_stride] instead of its draw.  sess_g [S] (optional, g > 0): how many of its
// proposals each conversation verifies (1..g).  `ctr`: world_emulated * max_rows * (P / world) zeroed
// ints of this rank.  ranks_emulated > 1 runs that many ranks in one cooperative launch on this GPU
// (peers then names areas of this device; emu_* are the element strides between the ranks' logits and
// output arrays; proposals and dstat are shared by the emulated ranks).
TF_API int tf_sample_chunks(const float* tlogits, const float* dlogits, const void* dstat, const int* proposals,
                            const double* uniforms, int u_stride, const float* sess_temp, const float* sess_top_p,
                            int S, int g, int V, int ldl, int point_mass, const int* sess_point, const int* forced,
                            const int* sess_g, void* tstat, int stat_stride, int* n_accept,
                            int* next_token, int tok_stride, const void* peers, int world, int rank, int max_rows,
                            void* ctr, int spin_limit, void* status, int ranks_emulated, long emu_tl, long emu_dl,
                            long emu_stat, long emu_tok, long emu_acc, cudaStream_t st) {
  const int P = tf_sample_chunks_count(V);
  if (!P || world < 1 || world > kCommMaxWorld || P % world || S < 1 || g < 0 || g > kMaxG || S * (g + 1) > max_rows)
    return -1;
  if (!tlogits || !uniforms || !sess_temp || !sess_top_p || !tstat || !next_token || !peers || !ctr) return -1;
  if (g > 0 && (!proposals || (!point_mass && (!dlogits || !dstat)))) return -1;
  const int csplit = P / world, chunk = V / P;
  if (ldl < csplit * chunk || ldl % 4 || (((uintptr_t)tlogits) & 15) || (dlogits && (((uintptr_t)dlogits) & 15))) return -1;
  if (ranks_emulated > 1 && ranks_emulated != world) return -1;
  if ((g + 1) * P > kThreads || u_stride < g + 1 || stat_stride < 1 || tok_stride < 1) return -1;
  ChunkParams p;
  p.tlogits = tlogits; p.dlogits = dlogits; p.dstat = (const RowStat*)dstat; p.proposals = proposals;
  p.uniforms = uniforms; p.u_stride = u_stride; p.sess_temp = sess_temp; p.sess_top_p = sess_top_p;
  p.S = S; p.g = g; p.V = V; p.ldl = ldl; p.chunk = chunk; p.P = P; p.csplit = csplit; p.point_mass = point_mass;
  p.sess_point = sess_point; p.forced = forced; p.sess_g = sess_g;
  p.tstat = (RowStat*)tstat; p.stat_stride = stat_stride; p.n_accept = n_accept; p.next_token = next_token;
  p.tok_stride = tok_stride; p.peers = (const unsigned long long*)peers; p.world = world; p.rank = rank;
  p.max_rows = max_rows; p.ctr = (unsigned int*)ctr; p.spin_limit = spin_limit; p.st = (TfStatusWord*)status;
  p.emu_tl = emu_tl; p.emu_dl = emu_dl; p.emu_stat = emu_stat; p.emu_tok = emu_tok; p.emu_acc = emu_acc;
  const size_t dyn = (size_t)chunk * 8 + 32 * 256 * 8;
  cudaError_t e = cudaFuncSetAttribute(sample_chunks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
  if (e != cudaSuccess) return (int)e;
  const int ez = ranks_emulated > 1 ? ranks_emulated : 1;
  dim3 grid(max_rows, csplit, ez);
  if (ez > 1 || csplit > 1) {
    // CTAs of one GPU wait for each other: all of them must be resident
    int dev = 0, per_sm = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sample_chunks_kernel, kThreads, dyn);
    if ((long)per_sm * sms < (long)S * (g + 1) * csplit * ez) return -1;
  }
  tf_launch(sample_chunks_kernel, dim3(grid), dim3(kThreads), dyn, st, p);
  return (int)cudaGetLastError();
}
