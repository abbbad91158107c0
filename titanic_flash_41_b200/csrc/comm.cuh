// One-shot all-reduce over NVLink peer memory, used as the epilogue of the producing kernel, with
// the sublayer boundary that follows the sum computed before the row leaves the SM.
//
// Every rank runs the same kernel with the same grid.  CTA j owns columns [32j, 32j+32) of a
// [rows, N] fp32 partial.
//   (1) push   CTA j stores its tile into the receive area of EVERY rank (its own included) as
//              8-byte words {payload, epoch}: the epoch travels in the same naturally aligned
//              64-bit store as the data it guards, so a reader that sees the epoch sees the data.
//              No fence, no separate flag, no second round trip.  Payload: two bf16 columns
//              (residual path: the transport precision of the reference's one-shot sum,
//              kernels/roce_oneshot_twin.cuh:95-167) or one fp32 column (WIDE, plain sums).
//   (2) reduce CTA r (r < rows) then turns into the owner of row r: it polls the words of that row
//              from every source rank (16-byte volatile loads, all sources in flight at once, each
//              wait bounded), sums the `world` partials in rank order in fp32 -- every rank adds
//              the same numbers in the same order, so all ranks hold bit-identical results --
//   (3) boundary  and, while the row sits in shared memory, adds it to the residual stream and
//              computes the RMSNorm, the f16 / bf16 copies and the MXFP8 row that the next
//              sublayer reads: the launch that used to follow every collective is gone
//              (reference: kernels/roce_oneshot_hc.cuh:27-77, caller src/mhc.rs:1276 finish_fused).
// The other CTAs leave after their push.  No CPU proxy, no second launch, no NCCL.
//
// Symmetric workspace layout (same offsets on every rank; base addresses of all ranks in `peers`):
//   u64 [2 parity][world src][max_rows][N]      (bf16 payloads use the first N/2 words of a row)
// Slots alternate by epoch parity.  A rank can run at most one epoch ahead of the slowest rank:
// finishing epoch e needs every rank's words of epoch e, which a rank only sends from the launch
// after the one that read epoch e-1.  Words of epoch e-2 in the same slot carry the wrong epoch
// and are never mistaken for data.
//
// A wait that runs out records TF_TIMEOUT (kernel id 200, detail = (source rank, row)) in the
// status word and the CTA returns without touching the residual: no trap, no endless spin.
//
// Several ranks can be emulated by one launch on one GPU (grid.y = ranks, `peers` pointing at
// `world` areas of the same device): the launch must then be cooperative, because row owners wait
// for CTAs of the other emulated ranks.
#pragma once
#include "rownorm.cuh"

constexpr int kCommMaxWorld = 8;

struct CommParams {
  const unsigned long long* peers;   // [world] base address of every rank's workspace (device array)
  int world, rank;                   // rank of blockIdx.y == 0 (emulation: rank + blockIdx.y)
  int tiles;                         // N / 32
  int max_rows;
  int N;
  unsigned int* epoch;               // [grid.y][tiles] local counters (plain device memory)
  int spin_limit;
  TfStatusWord* st;
};

// what the owner of a reduced row does with it
struct RowEpilogue {
  __nv_bfloat16* resid;        // [rows, N] residual stream, updated in place (may be null)
  float* ar_out;               // [rows, N] the reduced fp32 sum (may be null)
  const __nv_bfloat16* norm_w; // [N] RMSNorm weight of the boundary that follows (null: no norm)
  __half* h16;                 // [rows, N] normalised row, f16 (may be null)
  __nv_bfloat16* hb;           // [rows, N] normalised row, bf16 (may be null)
  uint8_t* x8;                 // [rows, N] MXFP8 values (may be null)
  uint8_t* x8s;                // [rows, N / 32] UE8M0 scales
  float eps;
};

__device__ __forceinline__ void st_ll(unsigned long long* p, uint32_t data, uint32_t flag) {
  const unsigned long long v = ((unsigned long long)flag << 32) | (unsigned long long)data;
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ ulonglong2 ld_ll2(const unsigned long long* p) {
  ulonglong2 v;
  asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool ll_ready(const ulonglong2& v, unsigned int e) {
  return (unsigned int)(v.x >> 32) == e && (unsigned int)(v.y >> 32) == e;
}

// (1) tile[r * 32 + c] (fp32, shared memory) of this CTA's 32 columns -> every rank's receive area
template <bool WIDE>
__device__ __forceinline__ void comm_push_tile(const CommParams& c, int rank, const float* tile, int rows, int j,
                                               unsigned int e) {
  constexpr int WPT = WIDE ? 32 : 16;          // words per tile row
  const int par = e & 1;
  const int per_peer = rows * WPT;
  for (int i = threadIdx.x; i < c.world * per_peer; i += blockDim.x) {
    const int pi = i / per_peer, rem = i - pi * per_peer, r = rem / WPT, q = rem - r * WPT;
    int peer = rank + 1 + pi;                  // start with the neighbour so that the ranks spread over the links
    if (peer >= c.world) peer -= c.world;
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(c.peers[peer]) +
                              ((long)(par * c.world + rank) * c.max_rows + r) * c.N + j * WPT + q;
    uint32_t data;
    if (WIDE) {
      data = __float_as_uint(tile[r * 32 + q]);
    } else {
      const __nv_bfloat162 b = __floats2bfloat162_rn(tile[r * 32 + 2 * q], tile[r * 32 + 2 * q + 1]);
      data = *reinterpret_cast<const uint32_t*>(&b);
    }
    st_ll(dst, data, e);
  }
}

// (2) + (3): owner of `row`.  rowbuf: N floats of shared memory.  Called by every thread of the CTA.
template <bool WIDE>
__device__ __forceinline__ bool comm_reduce_row(const CommParams& c, int rank, int row, unsigned int e,
                                                const RowEpilogue& ep, float* rowbuf, float* scratch, int* s_fail) {
  constexpr int LPQ = WIDE ? 2 : 1;            // 16-byte loads per source and column quad
  const int par = e & 1;
  const unsigned long long* base = reinterpret_cast<const unsigned long long*>(c.peers[rank]) +
                                   ((long)par * c.world * c.max_rows + row) * c.N;
  const long src_stride = (long)c.max_rows * c.N;
  const int nquads = c.N / 4;
  const long long t0 = clock64();
  bool failed = false;
  float ss = 0.f;
  for (int q = threadIdx.x; q < nquads && !failed; q += blockDim.x) {
    ulonglong2 v[kCommMaxWorld][LPQ];
#pragma unroll
    for (int s = 0; s < kCommMaxWorld; ++s)
      if (s < c.world) {
#pragma unroll
        for (int l = 0; l < LPQ; ++l) v[s][l] = ld_ll2(base + s * src_stride + (long)q * (2 * LPQ) + 2 * l);
      }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < kCommMaxWorld; ++s)
      if (s < c.world && !failed) {
#pragma unroll
        for (int l = 0; l < LPQ; ++l) {
          int spins = 0;
          // the wait gives up after spin_limit polls or about one second of SM clocks
          while (!ll_ready(v[s][l], e)) {
            if (++spins > c.spin_limit || clock64() - t0 > 2000000000LL) {
              tf_report(c.st, TF_TIMEOUT, 200, s, row);
              *s_fail = 1;
              failed = true;
              break;
            }
            v[s][l] = ld_ll2(base + s * src_stride + (long)q * (2 * LPQ) + 2 * l);
          }
        }
        if (WIDE) {
          acc[0] += __uint_as_float((uint32_t)v[s][0].x);
          acc[1] += __uint_as_float((uint32_t)v[s][0].y);
          acc[2] += __uint_as_float((uint32_t)v[s][LPQ - 1].x);
          acc[3] += __uint_as_float((uint32_t)v[s][LPQ - 1].y);
        } else {
          const uint32_t lo = (uint32_t)v[s][0].x, hi = (uint32_t)v[s][0].y;
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi));
          acc[0] += a.x;
          acc[1] += a.y;
          acc[2] += b.x;
          acc[3] += b.y;
        }
      }
#pragma unroll
    for (int k = 0; k < 4; ++k) rowbuf[4 * q + k] = acc[k];
  }
  __syncthreads();
  if (*s_fail) return false;
  const long r = row;
  for (int q = threadIdx.x; q < nquads; q += blockDim.x) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = rowbuf[4 * q + k];
    if (ep.ar_out) *reinterpret_cast<float4*>(ep.ar_out + r * c.N + 4 * q) = make_float4(v[0], v[1], v[2], v[3]);
    if (ep.resid) {
      __nv_bfloat16* xr = ep.resid + r * c.N + 4 * q;
      const uint2 xraw = *reinterpret_cast<const uint2*>(xr);
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xraw);
      const float2 x01 = __bfloat1622float2(xb[0]), x23 = __bfloat1622float2(xb[1]);
      v[0] = bf16_round(x01.x + v[0]);
      v[1] = bf16_round(x01.y + v[1]);
      v[2] = bf16_round(x23.x + v[2]);
      v[3] = bf16_round(x23.y + v[3]);
      __nv_bfloat162 o[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
      *reinterpret_cast<uint2*>(xr) = *reinterpret_cast<uint2*>(o);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        rowbuf[4 * q + k] = v[k];
        ss += v[k] * v[k];
      }
    }
  }
  if (ep.norm_w && ep.resid) {
    ss = block_sum(ss, scratch);
    row_norm_store(rowbuf, c.N, ss, ep.eps, ep.norm_w, ep.h16, ep.hb, ep.x8, ep.x8s, r);
  }
  return true;
}

// tile: this CTA's partial values, tile[r * 32 + c] for r < rows (shared memory, fp32); rowbuf: N
// floats of shared memory.  blockIdx.x is the tile, blockIdx.y the emulated rank offset.  Must be
// called by every thread of the CTA; the caller passes epilogue pointers of ITS rank.
template <bool WIDE>
__device__ __forceinline__ void comm_allreduce_rows(const CommParams& c, const float* tile, int rows,
                                                    const RowEpilogue& ep, float* rowbuf) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  __shared__ float s_scratch[32];
  const int j = blockIdx.x, rank = c.rank + blockIdx.y;
  if (threadIdx.x == 0) {
    s_epoch = ++c.epoch[(long)blockIdx.y * c.tiles + j];
    s_fail = 0;
  }
  __syncthreads();
  const unsigned int e = s_epoch;
  comm_push_tile<WIDE>(c, rank, tile, rows, j, e);
  if (j < rows) comm_reduce_row<WIDE>(c, rank, j, e, ep, rowbuf, s_scratch, &s_fail);
}
