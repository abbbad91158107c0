// Weight-streaming GEMM for small row counts (decode / verification: M <= 32 rows per group).
//
//   Y[r, n] = sum_k X[r, k] * W[n, k]          W: FP8 e4m3 with 128x128 fp32 block scales, or
//                                                 MXFP4 (packed e2m1 + one UE8M0 per 32 along K)
//
// At these row counts the op is bound by reading W once from HBM, so the kernel is organised
// around the weight stream: every lane issues 16-byte loads of consecutive K of one weight row,
// converts in registers (cvt e4m3x2->f16x2; e2m1 through an exponent-field trick) and feeds
// m16n8k16 tensor-core tiles in which the 16 weight rows are the MMA's M and the (few)
// activation rows its N.  The K index of an MMA slot is a permutation chosen so that the
// 16-byte weight load IS the A fragment; the activation fragment follows the same permutation.
// K is split over the warps of a CTA and reduced through shared memory in a fixed order, so
// results are run-to-run deterministic.
//
// Grouped form (routed experts): blockIdx.y walks a compacted list of active experts; rows of a
// group are gathered through `sorted_pairs`.  `dual` computes W1 and W3 tiles together and
// applies the clamped SwiGLU before storing (reference kernels/core.cu:938-942).
//
// Replaces, for the B200 build: kernels/direct_gemv_fp8.cu (FP8 GEMV, M<=8) and the b12x
// `moe.w4a8.compact_micro` bundles of the reference.
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
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
  const __half* X;           // activations f16
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
};

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int KIND>  // 0 = fp8 block128, 1 = mxfp4, 2 = bf16 weights with bf16 activations
struct Loader;

// ---- FP8: one step = 64 k -----------------------------------------------------------------
template <>
struct Loader<0> {
  static constexpr int kStep = 64;
  static __device__ __forceinline__ void load(const uint8_t* row0, const uint8_t* row8, int k, int t,
                                              uint4& w0, uint4& w8) {
    w0 = __ldg(reinterpret_cast<const uint4*>(row0 + k + t * 16));
    w8 = __ldg(reinterpret_cast<const uint4*>(row8 + k + t * 16));
  }
};
template <>
struct Loader<1> {
  static constexpr int kStep = 128;
  static __device__ __forceinline__ void load(const uint8_t* row0, const uint8_t* row8, int k, int t,
                                              uint4& w0, uint4& w8) {
    w0 = __ldg(reinterpret_cast<const uint4*>(row0 + (k >> 1) + t * 16));
    w8 = __ldg(reinterpret_cast<const uint4*>(row8 + (k >> 1) + t * 16));
  }
};

__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Accumulate one 16-row weight tile over k in [k0, k1) against MT activation tiles.
template <int KIND, int MT>
__device__ __forceinline__ void stream_tile(const SmallMParams& p, const uint8_t* Wg, const void* Sg,
                                            int n0, int k0, int k1, const __half* const xrow[MT],
                                            float acc[MT][4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint8_t* row0 = Wg + (long)(n0 + g) * p.ldw;
  const uint8_t* row8 = Wg + (long)(n0 + g + 8) * p.ldw;
  if (KIND == 0) {
    const float* S = reinterpret_cast<const float*>(Sg) + (long)(n0 >> 7) * p.lds;
    for (int kb = k0; kb < k1; kb += 128) {
      float blk[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) blk[m][0] = blk[m][1] = blk[m][2] = blk[m][3] = 0.f;
      uint4 w0[2], w8[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) Loader<0>::load(row0, row8, kb + s * 64, t, w0[s], w8[s]);
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0[s]);
        const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8[s]);
        uint4 xv[MT][2];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4* xp = reinterpret_cast<const uint4*>(xrow[m] + kb + s * 64 + t * 16);
          xv[m][0] = xp[0];
          xv[m][1] = xp[1];
        }
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
            mma_f16_16816(blk[m], a, b);
          }
        }
      }
      const float sc = __ldg(S + (kb >> 7));
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][i] = fmaf(sc, blk[m][i], acc[m][i]);
    }
  } else if (KIND == 2) {
    // bf16: a 16-byte load holds 8 consecutive k of one row; one step = 32 k = two MMAs
    for (int kb = k0; kb < k1; kb += 32) {
      const uint4 w0 = __ldg(reinterpret_cast<const uint4*>(row0 + 2 * (kb + t * 8)));
      const uint4 w8 = __ldg(reinterpret_cast<const uint4*>(row8 + 2 * (kb + t * 8)));
      const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0);
      const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xrow[m] + kb + t * 8);
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t a[4] = {a0w[2 * j], a8w[2 * j], a0w[2 * j + 1], a8w[2 * j + 1]};
          uint32_t b[2] = {xw[2 * j], xw[2 * j + 1]};
          mma_bf16_16816(acc[m], a, b);
        }
      }
    }
  } else {
    const uint8_t* S0 = reinterpret_cast<const uint8_t*>(Sg) + (long)(n0 + g) * p.lds;
    const uint8_t* S8 = reinterpret_cast<const uint8_t*>(Sg) + (long)(n0 + g + 8) * p.lds;
    for (int kb = k0; kb < k1; kb += 128) {
      uint4 w0, w8;
      Loader<1>::load(row0, row8, kb, t, w0, w8);
      // factor = 2^14 * 2^(s-127) as f16x2 (exact for s in [99,142]; the loader checks the range)
      const int sb = (kb >> 5) + t;
      float f0 = ue8m0_to_float(__ldg(S0 + sb)) * 16384.f, f8 = ue8m0_to_float(__ldg(S8 + sb)) * 16384.f;
      __half2 h0 = __float2half2_rn(f0), h8 = __float2half2_rn(f8);
      const uint32_t s0 = *reinterpret_cast<uint32_t*>(&h0), s8 = *reinterpret_cast<uint32_t*>(&h8);
      const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0);
      const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8);
      uint4 xv[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4* xp = reinterpret_cast<const uint4*>(xrow[m] + kb + t * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) xv[m][q] = xp[q];
      }
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
            mma_f16_16816(acc[m], a, b);
          }
        }
      }
    }
  }
}

template <int KIND, int MT, bool DUAL>
__global__ void __launch_bounds__(kWarps * 32) smallm_gemm_kernel(SmallMParams p) {
  constexpr int NM = DUAL ? 2 : 1;
  __shared__ float red[kWarps][NM][2][MT][32][4];   // [warp][matrix][m16 tile][n8 tile][lane][4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  int rows, row_base = 0;
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
    const long sbytes = (long)e * p.s_group_stride * (KIND == 0 ? 4 : 1);
    Sg = reinterpret_cast<const uint8_t*>(Sg) + sbytes;
    if (DUAL) {
      W3g += (long)e * p.w_group_stride;
      S3g = reinterpret_cast<const uint8_t*>(S3g) + sbytes;
    }
  } else {
    rows = p.M;
  }
  const int n0 = blockIdx.x * kTileN;
  const int k0 = warp * p.k_per_warp, k1 = min(p.K, k0 + p.k_per_warp);

  for (; row_base < rows; row_base += 8 * MT) {
    const __half* xrow[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int r = min(row_base + m * 8 + g, rows - 1);
      int xr = pairs ? pairs[r] / p.x_div : r;
      xrow[m] = p.X + (long)xr * p.ldx;
    }
    float acc[NM][2][MT][4];
#pragma unroll
    for (int a = 0; a < NM; ++a)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[a][h][m][0] = acc[a][h][m][1] = acc[a][h][m][2] = acc[a][h][m][3] = 0.f;
    if (k0 < k1) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        stream_tile<KIND, MT>(p, Wg, Sg, n0 + 16 * h, k0, k1, xrow, acc[0][h]);
        if (DUAL) stream_tile<KIND, MT>(p, W3g, S3g, n0 + 16 * h, k0, k1, xrow, acc[NM - 1][h]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < NM; ++a)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) red[warp][a][h][m][lane][i] = acc[a][h][m][i];
    __syncthreads();
    // fixed-order reduction over warps; thread -> (h, m, lane, i) slots
    constexpr int kSlots = 2 * MT * 32 * 4;
    for (int s = threadIdx.x; s < kSlots; s += kWarps * 32) {
      const int i = s & 3, ln = (s >> 2) & 31, m = (s >> 7) % MT, h = (s >> 7) / MT;
      float v = 0.f, v3 = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        v += red[w][0][h][m][ln][i];
        if (DUAL) v3 += red[w][NM - 1][h][m][ln][i];
      }
      // C fragment: rows (weight row) = g or g+8 for i>=2 ; cols (activation row) = 2t + (i&1)
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
        if (p.out_kind == 0) reinterpret_cast<float*>(p.Y)[off] = o;
        else if (p.out_kind == 1) reinterpret_cast<__half*>(p.Y)[off] = __float2half(o);
        else reinterpret_cast<__nv_bfloat16*>(p.Y)[off] = __float2bfloat16(o);
      }
    }
    __syncthreads();
  }
}

template <int KIND, bool DUAL>
cudaError_t launch(const SmallMParams& p, int max_rows, int slots, cudaStream_t st) {
  dim3 grid((p.N + kTileN - 1) / kTileN, slots > 0 ? slots : 1);
  dim3 block(kWarps * 32);
  if (max_rows <= 8) smallm_gemm_kernel<KIND, 1, DUAL><<<grid, block, 0, st>>>(p);
  else smallm_gemm_kernel<KIND, 2, DUAL><<<grid, block, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

// kind: 0 = FP8 block-128, 1 = MXFP4, 2 = bf16 weights (X is then bf16, not f16).  Returns a cudaError_t (0 = ok) or -1 for a bad argument.
TF_API int tf_smallm_gemm(int kind, const void* W, const void* W3, const void* S, const void* S3,
                          long w_group_stride, long s_group_stride, int ldw, int lds, const void* X,
                          int ldx, void* Y, int ldy, int out_kind, int N, int K, int M,
                          const int* group_expert, const int* group_start, const int* group_count,
                          const int* n_groups, const int* sorted_pairs, int x_div, int slots,
                          int max_rows, float swiglu_limit, cudaStream_t stream) {
  if (N % kTileN != 0 || K % 128 != 0 || (ldx % 8) != 0) return -1;
  if (kind == 0 && (ldw % 16) != 0) return -1;
  if (kind == 1 && (ldw % 16) != 0) return -1;
  SmallMParams p;
  p.W = (const uint8_t*)W; p.W3 = (const uint8_t*)W3; p.S = S; p.S3 = S3;
  p.w_group_stride = w_group_stride; p.s_group_stride = s_group_stride;
  p.ldw = ldw; p.lds = lds; p.X = (const __half*)X; p.ldx = ldx; p.Y = Y; p.ldy = ldy;
  p.out_kind = out_kind; p.N = N; p.K = K; p.M = M;
  p.group_expert = group_expert; p.group_start = group_start; p.group_count = group_count;
  p.n_groups = n_groups; p.sorted_pairs = sorted_pairs; p.x_div = x_div > 0 ? x_div : 1;
  p.swiglu_limit = swiglu_limit;
  int kpw = ((K + kWarps - 1) / kWarps + 127) / 128 * 128;
  p.k_per_warp = kpw;
  const bool dual = W3 != nullptr;
  cudaError_t e;
  if (kind == 0) e = dual ? launch<0, true>(p, max_rows, slots, stream) : launch<0, false>(p, max_rows, slots, stream);
  else if (kind == 1) e = dual ? launch<1, true>(p, max_rows, slots, stream) : launch<1, false>(p, max_rows, slots, stream);
  else if (kind == 2) e = launch<2, false>(p, max_rows, slots, stream);
  else return -1;
  return (int)e;
}
