// Weight-streaming GEMM for small row counts (decode / verification: M <= 32 rows per group).
//
//   Y[r, n] = sum_k X[r, k] * W[n, k]     W: FP8 e4m3 with 128x128 fp32 block scales (kind 0),
//                                            MXFP4 = packed e2m1 + one UE8M0 per 32 along K (kind 1),
//                                            or bf16 (kind 2, bf16 activations)
//
// At these row counts the op is bound by reading W once from HBM, so the kernel is organised
// around the weight stream: every lane issues 16-byte loads of consecutive K of one weight row,
// converts in registers (cvt e4m3x2->f16x2; e2m1 through an exponent-field trick) and feeds
// m16n8k16 tensor-core tiles in which 16 weight rows are the MMA's M and the (few) activation
// rows its N.  The K index of an MMA slot is a permutation chosen so that the 16-byte weight load
// IS the A fragment; the activation fragment follows the same permutation.  Per K step a warp
// first issues the loads of ALL its weight tiles (two 16-row tiles, times two matrices in the
// dual form: 8 x 16 B per lane in flight), then the activation fragments once, then the MMAs,
// which keeps enough bytes in flight to follow HBM.  K is split over the warps of a CTA and
// reduced through shared memory in a fixed order: results are run-to-run deterministic.
//
// Grouped form (routed experts): blockIdx.y walks a compacted list of active experts; rows of a
// group are gathered through `sorted_pairs`.  `dual` computes W1 and W3 tiles together and
// applies the clamped SwiGLU before storing (reference kernels/core.cu:938-942).
//
// Replaces, for the B200 build: kernels/direct_gemv_fp8.cu (FP8 GEMV, M<=8) and the b12x
// `moe.w4a8.compact_micro` bundles of the reference.
#include "comm.cuh"

namespace {

constexpr int kWarps = 4;   // K is split four ways inside a CTA; four CTAs fit on an SM
constexpr int kMaxWarps = 8;   // dense matrices with few 32-feature tiles split K eight ways instead (more warps per SM)
constexpr int kTileN = 32;   // output columns per CTA (two m16 tiles per warp)

struct SmallMParams {
  const uint8_t* W;          // [groups][N][ldw bytes]
  const uint8_t* W3;         // dual mode: second matrix (same layout), else null
  const void* S;             // fp8: float [N/128][lds]; fp4: uint8 [N][lds]
  const void* S3;
  long w_group_stride;       // bytes
  long s_group_stride;       // elements of S
  int ldw;                   // bytes per weight row
  int lds;                   // scale row stride (elements)
  const __half* X;           // activations f16 (bf16 for kind 2)
  int ldx;                   // elements
  void* Y;                   // output
  int ldy;                   // elements
  int out_kind;              // 0 = f32, 1 = f16, 2 = bf16
  int N, K;                  // K in elements
  int M;                     // rows (dense form)
  // grouped form
  const int* group_expert;   // [slots] expert id of each active group (null = dense)
  const int* group_start;    // [slots] offset into sorted_pairs
  const int* group_count;    // [slots]
  const int* n_groups;       // device scalar
  const int* sorted_pairs;   // pair ids sorted by expert
  int x_div;                 // x row = pair / x_div
  float swiglu_limit;
  int k_per_warp;            // multiple of 128
  // fused tensor-parallel epilogue (dense form, M <= 32): all-reduce the [M, N] partial over the
  // peers' memory, add it to the residual stream and run the boundary that follows (comm.cuh)
  int use_comm;              // 0 = off, 1 = bf16 transport, 2 = fp32 transport
  CommParams comm;
  RowEpilogue ep;
};

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// streaming (evict-first) 16-byte load: weights are read exactly once per launch
__device__ __forceinline__ uint4 ld_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// One group (dense matrix or one expert): NT = 2 (or 4 in the dual form) weight tiles of 16 rows.
template <int KIND, int MT, bool DUAL>
__device__ __forceinline__ void run_rows(const SmallMParams& p, const uint8_t* Wg, const uint8_t* W3g,
                                         const void* Sg, const void* S3g, int rows, const int* pairs,
                                         int row_base, float (*red)[32][4], float* tile_out, bool& need_wait) {
  // need_wait: the kernel has not yet waited for its predecessor in the stream.  The dense forms
  // request their first weight block (immutable data) before they wait, so that the weight stream
  // starts while the kernel before this one is still finishing; activations are read after.
  auto wait_once = [&]() {
    if (need_wait) {
      tf_pdl_sync();
      need_wait = false;
    }
  };
  constexpr int NM = DUAL ? 2 : 1;
  constexpr int NT = 2 * NM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * kTileN;
  const int k0 = warp * p.k_per_warp, k1 = min(p.K, k0 + p.k_per_warp);

  if (pairs) wait_once();                  // (grouped forms have waited already: their lists are kernel outputs)
  const __half* xrow[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int r = min(row_base + m * 8 + g, rows - 1);
    const int xr = pairs ? pairs[r] / p.x_div : r;
    xrow[m] = p.X + (long)xr * p.ldx;
  }
  // tile ti -> matrix (ti >> 1), 16-row half (ti & 1)
  const uint8_t* wrow0[NT];
  const uint8_t* wrow8[NT];
#pragma unroll
  for (int ti = 0; ti < NT; ++ti) {
    const uint8_t* base = (ti >> 1) ? W3g : Wg;
    wrow0[ti] = base + (long)(n0 + 16 * (ti & 1) + g) * p.ldw;
    wrow8[ti] = wrow0[ti] + 8L * p.ldw;
  }
  float acc[NT][MT][4];
#pragma unroll
  for (int ti = 0; ti < NT; ++ti)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[ti][m][0] = acc[ti][m][1] = acc[ti][m][2] = acc[ti][m][3] = 0.f;

  if (KIND == 0) {
    // ---------------- FP8, fp32 scale per 128x128 block: accumulate a block, then promote
    const float* S = reinterpret_cast<const float*>(Sg) + (long)(n0 >> 7) * p.lds;
    const float* S3 = DUAL ? reinterpret_cast<const float*>(S3g) + (long)(n0 >> 7) * p.lds : nullptr;
    // The weights of the NEXT 128-k block are requested before the MMAs of this one (plain form;
    // the fused form already has twice the loads per step): with N / 32 CTAs on the grid only a
    // few warps run per SM, so the bytes each keeps in flight decide how well the stream follows HBM.
    constexpr bool kPrefetch = !DUAL;
    uint4 w0[2][NT], w8[2][NT], w0n[2][NT], w8n[2][NT];
    auto load_block = [&](int kb, uint4 (&a0)[2][NT], uint4 (&a8)[2][NT]) {
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int ti = 0; ti < NT; ++ti) {
          a0[s][ti] = ld_stream(wrow0[ti] + kb + s * 64 + t * 16);
          a8[s][ti] = ld_stream(wrow8[ti] + kb + s * 64 + t * 16);
        }
    };
    if (kPrefetch && k0 < k1) load_block(k0, w0, w8);
    if (kPrefetch) wait_once();
    for (int kb = k0; kb < k1; kb += 128) {
      float blk[NT][MT][4];
#pragma unroll
      for (int ti = 0; ti < NT; ++ti)
#pragma unroll
        for (int m = 0; m < MT; ++m) blk[ti][m][0] = blk[ti][m][1] = blk[ti][m][2] = blk[ti][m][3] = 0.f;
      if (!kPrefetch) {
        load_block(kb, w0, w8);
        wait_once();
      } else if (kb + 128 < k1) {
        load_block(kb + 128, w0n, w8n);
      }
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int k = kb + s * 64 + t * 16;
        uint4 xv[MT][2];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4* xp = reinterpret_cast<const uint4*>(xrow[m] + k);
          xv[m][0] = xp[0];
          xv[m][1] = xp[1];
        }
#pragma unroll
        for (int ti = 0; ti < NT; ++ti) {
          const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0[s][ti]);
          const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8[s][ti]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t a[4];
            a[0] = e4m3x2_to_h2((uint16_t)(a0w[j] & 0xffffu));
            a[1] = e4m3x2_to_h2((uint16_t)(a8w[j] & 0xffffu));
            a[2] = e4m3x2_to_h2((uint16_t)(a0w[j] >> 16));
            a[3] = e4m3x2_to_h2((uint16_t)(a8w[j] >> 16));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[m][0]);
              uint32_t b[2] = {xw[2 * j], xw[2 * j + 1]};
              mma_f16_16816(blk[ti][m], a, b);
            }
          }
        }
      }
      const float sc = __ldg(S + (kb >> 7));
      const float sc3 = DUAL ? __ldg(S3 + (kb >> 7)) : 0.f;
#pragma unroll
      for (int ti = 0; ti < NT; ++ti)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[ti][m][i] = fmaf((ti >> 1) ? sc3 : sc, blk[ti][m][i], acc[ti][m][i]);
      if (kPrefetch) {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int ti = 0; ti < NT; ++ti) {
            w0[s][ti] = w0n[s][ti];
            w8[s][ti] = w8n[s][ti];
          }
      }
    }
  } else if (KIND == 2) {
    // ---------------- bf16 weights: a 16-byte load holds 8 consecutive k; 64 k per step
    for (int kb = k0; kb < k1; kb += 64) {
      uint4 w0[NT][2], w8[NT][2];
#pragma unroll
      for (int ti = 0; ti < NT; ++ti)
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          w0[ti][s] = ld_stream(wrow0[ti] + 2 * (kb + s * 32 + t * 8));
          w8[ti][s] = ld_stream(wrow8[ti] + 2 * (kb + s * 32 + t * 8));
        }
      wait_once();
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        uint4 xv[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) xv[m] = *reinterpret_cast<const uint4*>(xrow[m] + kb + s * 32 + t * 8);
#pragma unroll
        for (int ti = 0; ti < NT; ++ti) {
          const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0[ti][s]);
          const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8[ti][s]);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint32_t a[4] = {a0w[2 * j], a8w[2 * j], a0w[2 * j + 1], a8w[2 * j + 1]};
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[m]);
              uint32_t b[2] = {xw[2 * j], xw[2 * j + 1]};
              mma_bf16_16816(acc[ti][m], a, b);
            }
          }
        }
      }
    }
  } else {
    // ---------------- MXFP4: 32 nibbles per 16-byte load = one scale group of one row; 128 k per step
    const uint8_t* srow0[NT];
    const uint8_t* srow8[NT];
#pragma unroll
    for (int ti = 0; ti < NT; ++ti) {
      const uint8_t* sb = reinterpret_cast<const uint8_t*>((ti >> 1) ? S3g : Sg);
      srow0[ti] = sb + (long)(n0 + 16 * (ti & 1) + g) * p.lds;
      srow8[ti] = srow0[ti] + 8L * p.lds;
    }
    for (int kb = k0; kb < k1; kb += 128) {
      uint4 w0[NT], w8[NT];
      uint8_t c0[NT], c8[NT];
      const int sbi = (kb >> 5) + t;
#pragma unroll
      for (int ti = 0; ti < NT; ++ti) {
        w0[ti] = ld_stream(wrow0[ti] + (kb >> 1) + t * 16);
        w8[ti] = ld_stream(wrow8[ti] + (kb >> 1) + t * 16);
        c0[ti] = __ldg(srow0[ti] + sbi);
        c8[ti] = __ldg(srow8[ti] + sbi);
      }
      uint4 xv[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4* xp = reinterpret_cast<const uint4*>(xrow[m] + kb + t * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) xv[m][q] = xp[q];
      }
#pragma unroll
      for (int ti = 0; ti < NT; ++ti) {
        // factor = 2^14 * 2^(s-127) as f16x2 (exact for s in [99,142]; the loader checks the range)
        __half2 h0 = __float2half2_rn(ue8m0_to_float(c0[ti]) * 16384.f);
        __half2 h8 = __float2half2_rn(ue8m0_to_float(c8[ti]) * 16384.f);
        const uint32_t s0 = *reinterpret_cast<uint32_t*>(&h0), s8 = *reinterpret_cast<uint32_t*>(&h8);
        const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0[ti]);
        const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8[ti]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t h0x[4], h8x[4];
          e2m1x8_to_h2x4_scaled(a0w[i], h0x);
          e2m1x8_to_h2x4_scaled(a8w[i], h8x);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            h0x[q] = h2_mul(h0x[q], s0);
            h8x[q] = h2_mul(h8x[q], s8);
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int j = 2 * i + half;
            uint32_t a[4] = {h0x[2 * half], h8x[2 * half], h0x[2 * half + 1], h8x[2 * half + 1]};
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[m][0]);
              uint32_t b[2] = {xw[2 * j], xw[2 * j + 1]};
              mma_f16_16816(acc[ti][m], a, b);
            }
          }
        }
      }
    }
  }

  // ---- fixed-order reduction over the K-splitting warps, then the epilogue
  // red is [kWarps * NT * MT][32][4]
  wait_once();                             // (a warp whose K range is empty has not waited yet)
  __syncthreads();
#pragma unroll
  for (int ti = 0; ti < NT; ++ti)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[(warp * NT + ti) * MT + m][lane][i] = acc[ti][m][i];
  __syncthreads();
  constexpr int kSlots = 2 * MT * 32 * 4;
  const int nwarps = blockDim.x >> 5;
  for (int s = threadIdx.x; s < kSlots; s += blockDim.x) {
    const int i = s & 3, ln = (s >> 2) & 31, m = (s >> 7) % MT, h = (s >> 7) / MT;
    float v = 0.f, v3 = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      v += red[(w * NT + h) * MT + m][ln][i];
      if (DUAL) v3 += red[(w * NT + 2 + h) * MT + m][ln][i];
    }
    // C fragment: weight row = g (+8 for i >= 2); activation row = 2t + (i & 1)
    const int gg = ln >> 2, tt = ln & 3;
    const int n = n0 + 16 * h + gg + ((i & 2) ? 8 : 0);
    const int r = row_base + m * 8 + 2 * tt + (i & 1);
    if (r < rows && n < p.N) {
      float o = v;
      if (DUAL) {
        float gate = v, up = v3;
        if (p.swiglu_limit > 0.f) {
          gate = fminf(gate, p.swiglu_limit);
          up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit);
        }
        o = gate / (1.f + __expf(-gate)) * up;
      }
      const long orow = pairs ? pairs[r] : r;
      const long off = orow * p.ldy + n;
      if (tile_out) tile_out[r * 32 + (n - n0)] = o;
      else if (p.out_kind == 0) reinterpret_cast<float*>(p.Y)[off] = o;
      else if (p.out_kind == 1) reinterpret_cast<__half*>(p.Y)[off] = __float2half(o);
      else reinterpret_cast<__nv_bfloat16*>(p.Y)[off] = __float2bfloat16(o);
    }
  }
  __syncthreads();
}

template <int KIND, bool DUAL>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
smallm_gemm_kernel(SmallMParams p) {
  // grouped forms read kernel outputs (the group lists) first; dense forms wait inside run_rows
  bool need_wait = p.group_expert == nullptr;
  if (!need_wait) tf_pdl_sync();
  __shared__ float red[kMaxWarps * (DUAL ? 4 : 2) * 2][32][4];
  __shared__ __align__(16) float ctile[(KIND == 0 && !DUAL) ? 32 * 32 : 4];
  float* tile_out = (KIND == 0 && !DUAL && p.use_comm) ? ctile : nullptr;
  int rows;
  const uint8_t *Wg = p.W, *W3g = p.W3;
  const void *Sg = p.S, *S3g = p.S3;
  const int* pairs = nullptr;
  if (p.group_expert) {
    const int slot = blockIdx.y;
    if (slot >= *p.n_groups) return;
    const int e = p.group_expert[slot];
    rows = p.group_count[slot];
    pairs = p.sorted_pairs + p.group_start[slot];
    Wg += (long)e * p.w_group_stride;
    const long sbytes = (long)e * p.s_group_stride * (KIND == 0 ? 4 : 1);   // kinds 1 and 3: one byte per scale
    Sg = reinterpret_cast<const uint8_t*>(Sg) + sbytes;
    if (DUAL) {
      W3g += (long)e * p.w_group_stride;
      S3g = reinterpret_cast<const uint8_t*>(S3g) + sbytes;
    }
  } else {
    rows = p.M;
  }
  // 8 activation rows per MMA tile: one tile when the group has at most 8 rows, else 16 at a time
  int row_base = 0;
  while (row_base < rows) {
    if (rows - row_base <= 8) {
      run_rows<KIND, 1, DUAL>(p, Wg, W3g, Sg, S3g, rows, pairs, row_base, red, tile_out, need_wait);
      row_base += 8;
    } else {
      run_rows<KIND, 2, DUAL>(p, Wg, W3g, Sg, S3g, rows, pairs, row_base, red, tile_out, need_wait);
      row_base += 16;
    }
  }
  if (need_wait) tf_pdl_sync();            // (no rows: nothing has waited)
  if (KIND == 0 && !DUAL) {
    if (p.use_comm) {
      extern __shared__ float rowbuf[];      // N floats, comm form only
      if (p.use_comm == 2) comm_allreduce_rows<true>(p.comm, ctile, rows, p.ep, rowbuf);
      else comm_allreduce_rows<false>(p.comm, ctile, rows, p.ep, rowbuf);
    }
  }
}

template <int KIND, bool DUAL>
cudaError_t launch(const SmallMParams& p, int slots, cudaStream_t st, int warps = kWarps) {
  dim3 grid((p.N + kTileN - 1) / kTileN, slots > 0 ? slots : 1);
  tf_launch(smallm_gemm_kernel<KIND, DUAL>, dim3(grid), dim3(warps * 32), 0, st, p);
  return cudaGetLastError();
}

}  // namespace

// kind: 0 = FP8 block-128, 1 = MXFP4, 2 = bf16 weights (X is then bf16, not f16).
// Returns a cudaError_t (0 = ok) or -1 for a bad argument.  `max_rows` is accepted for ABI
// stability; the kernel sizes its row tiles from the actual group sizes.
TF_API int tf_smallm_gemm(int kind, const void* W, const void* W3, const void* S, const void* S3,
                          long w_group_stride, long s_group_stride, int ldw, int lds, const void* X,
                          int ldx, void* Y, int ldy, int out_kind, int N, int K, int M,
                          const int* group_expert, const int* group_start, const int* group_count,
                          const int* n_groups, const int* sorted_pairs, int x_div, int slots,
                          int max_rows, float swiglu_limit, cudaStream_t stream) {
  (void)max_rows;
  if (N % kTileN != 0 || K % 128 != 0 || (ldx % 8) != 0 || (ldw % 16) != 0) return -1;
  SmallMParams p;
  p.W = (const uint8_t*)W; p.W3 = (const uint8_t*)W3; p.S = S; p.S3 = S3;
  p.w_group_stride = w_group_stride; p.s_group_stride = s_group_stride;
  p.ldw = ldw; p.lds = lds; p.X = (const __half*)X; p.ldx = ldx; p.Y = Y; p.ldy = ldy;
  p.out_kind = out_kind; p.N = N; p.K = K; p.M = M;
  p.group_expert = group_expert; p.group_start = group_start; p.group_count = group_count;
  p.n_groups = n_groups; p.sorted_pairs = sorted_pairs; p.x_div = x_div > 0 ? x_div : 1;
  p.swiglu_limit = swiglu_limit;
  p.k_per_warp = ((K + kWarps - 1) / kWarps + 127) / 128 * 128;
  p.use_comm = 0;
  const bool dual = W3 != nullptr;
  cudaError_t e;
  // dense FP8 with so few tiles that an SM gets two CTAs or fewer: eight K-splitting warps per CTA
  int warps = kWarps;
  if (kind == 0 && !dual && !group_expert && N / kTileN <= 320 && K >= 8 * 256) {
    warps = kMaxWarps;
    p.k_per_warp = ((K + warps - 1) / warps + 127) / 128 * 128;
  }
  if (kind == 0) e = dual ? launch<0, true>(p, slots, stream) : launch<0, false>(p, slots, stream, warps);
  else if (kind == 1) e = dual ? launch<1, true>(p, slots, stream) : launch<1, false>(p, slots, stream);
  else if (kind == 2) e = launch<2, false>(p, slots, stream);
  else return -1;
  return (int)e;
}

// Dense FP8 GEMV (M <= 32) fused with the tensor-parallel all-reduce, the residual update and the
// boundary that follows:
//   resid[M, N] += sum over ranks of X_rank[M, K] * W_rank[N, K]^T      (and/or ar_out = the sum)
//   norm_w given: h16 / hb / (x8, x8s) = RMSNorm(resid) * norm_w in f16 / bf16 / MXFP8
// `peers` is a device array of `world` workspace base addresses (see comm.cuh for the layout),
// `epoch` a zero-initialised device array of N/32 counters owned by this rank.  With a residual the
// partials travel as bf16, without one (ar_out only) as fp32.
TF_API int tf_smallm_gemm_allreduce(const void* W, const void* S, int ldw, int lds, const void* X, int ldx,
                                    int N, int K, int M, const void* peers, int world, int rank,
                                    int max_rows, void* epoch, void* resid, float* ar_out, const void* norm_w,
                                    void* h16, void* hb, void* x8, void* x8s, float eps, int spin_limit,
                                    void* status, cudaStream_t stream) {
  if (N % kTileN != 0 || K % 128 != 0 || (ldx % 8) != 0 || (ldw % 16) != 0 || N % 128 != 0) return -1;
  if (M < 1 || M > 32 || M > max_rows || world < 1 || world > kCommMaxWorld || N / kTileN < M) return -1;
  if (!W || !S || !X || !peers || !epoch || (!resid && !ar_out) || (x8 && !x8s) || (norm_w && !resid)) return -1;
  SmallMParams p;
  p.W = (const uint8_t*)W; p.W3 = nullptr; p.S = S; p.S3 = nullptr;
  p.w_group_stride = 0; p.s_group_stride = 0; p.ldw = ldw; p.lds = lds;
  p.X = (const __half*)X; p.ldx = ldx; p.Y = nullptr; p.ldy = N; p.out_kind = 0; p.N = N; p.K = K; p.M = M;
  p.group_expert = nullptr; p.group_start = nullptr; p.group_count = nullptr; p.n_groups = nullptr;
  p.sorted_pairs = nullptr; p.x_div = 1; p.swiglu_limit = 0.f;
  p.k_per_warp = ((K + kMaxWarps - 1) / kMaxWarps + 127) / 128 * 128;
  p.use_comm = resid ? 1 : 2;
  p.comm.peers = (const unsigned long long*)peers; p.comm.world = world; p.comm.rank = rank;
  p.comm.tiles = N / kTileN; p.comm.max_rows = max_rows; p.comm.N = N; p.comm.epoch = (unsigned int*)epoch;
  p.comm.spin_limit = spin_limit; p.comm.st = (TfStatusWord*)status;
  p.ep.resid = (__nv_bfloat16*)resid; p.ep.ar_out = ar_out; p.ep.norm_w = (const __nv_bfloat16*)norm_w;
  p.ep.h16 = (__half*)h16; p.ep.hb = (__nv_bfloat16*)hb; p.ep.x8 = (uint8_t*)x8; p.ep.x8s = (uint8_t*)x8s;
  p.ep.eps = eps;
  const size_t dyn = (size_t)N * sizeof(float);
  if (dyn > 24 * 1024) {
    cudaError_t a = cudaFuncSetAttribute(smallm_gemm_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)dyn);
    if (a != cudaSuccess) return (int)a;
  }
  dim3 grid(N / kTileN, 1);
  tf_launch(smallm_gemm_kernel<0, false>, dim3(grid), dim3(kMaxWarps * 32), dyn, stream, p);
  return (int)cudaGetLastError();
}
