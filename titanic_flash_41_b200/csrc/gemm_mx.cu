// Block-scaled tensor-core GEMM for sm_100a (prefill rows):
//
//   C[M, N] = (A * sfa) (B * sfb)^T      A [M, K] e4m3 (MXFP8 activations)
//                                         B [N, K] e4m3, or packed e2m1 (MXFP4 experts, K/2 bytes per row)
//                                         sfa / sfb: one UE8M0 scale per (row, 32 k)
//
// `tcgen05.mma kind::mxf8f6f4.block_scale` applies both scale vectors inside the tensor core, so a
// whole K runs into ONE accumulator in tensor memory: no per-128-k promotion through registers
// (which holds the fp32-scaled form at about half the FP8 rate) and no conversion pass for MXFP4
// weights (TMA expands the nibbles to the padded shared-memory form the instruction reads).
//
// Scale layout in global memory ("units"): 128 bytes hold the scales of 32 consecutive rows x 128 k,
// byte (row % 32) * 4 + (k / 32) % 4; units are ordered [k / 128][row / 32].  The scales a tile
// needs for one 128-deep k block are then contiguous (512 B for 128 rows of A, 1 KB for 256 rows of
// B): one bulk copy each per stage, and a warp moves them to tensor memory with one 4-byte shared
// load per lane and column (tcgen05.st; columns j = rows 32j..32j+31, byte = which 32-k group).
//
// One persistent CTA per SM walks 128 x 256 output tiles:
//   warp 0       TMA producer (A, B tiles with 128-byte swizzle + the two scale pieces; 4 stages)
//   warp 1       MMA issuer (one thread), owns the tensor-memory allocation
//   warps 2-5    scale movers: shared memory -> tensor memory, one per 32-lane quadrant
//   warps 6-13   epilogue: tensor memory -> registers -> bf16 / f32 rows
// The accumulator (256 columns) is single: the epilogue frees it as soon as its tcgen05.ld's have
// landed, before converting and storing, so the next tile's MMAs wait for the drain only.
// Grouped form (routed experts): A rows are expert-sorted in 128-row padded segments and M tile i
// uses the weights of expert tile_expert[i] (rows [e * N, (e + 1) * N) of B).
// Every wait is bounded: on a time-out the CTA raises its abort flag, records TF_TIMEOUT, lets
// copies in flight land, frees its tensor memory and returns.
//
// Reference behaviour: block-scaled dense and expert GEMMs of the prefill path
// (src/blockscaled.rs:21-87 scale format; src/fp8_linear.rs:122 call site; the b12x
// `gemm.dense` / `moe.grouped` bundles).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kStages = 4;
constexpr int kSfaBytes = BM / 32 * 128;                       // 512
constexpr int kSfbBytes = BN / 32 * 128;                       // 1024
constexpr int kStageBytes = BM * 128 + BN * 128 + 2048;        // tiles, scale pieces, pad to 1 KB multiple
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + 4 + kEpiWarps) * 32;
constexpr int kAccCols = BN;                                   // accumulator columns [0, 256)
constexpr int kSfCols = 16;                                    // per stage: 4 (A) + 8 (B), padded
constexpr int kTmemCols = 512;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;

struct MxGemmParams {
  int M, N, K;
  int b_fp4;                 // B is packed e2m1
  const uint8_t* sfa;        // units [K/128][sfa_units]
  const uint8_t* sfb;        // units [K/128][sfb_units]
  int sfa_units, sfb_units;  // units per k block (rows / 32, padded)
  void* C;
  int ldc;
  int out_kind;              // 0 f32, 2 bf16
  const int* tile_expert;
  const int* num_m_tiles;
  TfStatusWord* status;
};

__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t v[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t v[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= (A * sfa) (B * sfb)^T, scales read from tensor memory; ONE thread issues
__device__ __forceinline__ void mma_mx(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// block-scaled instruction descriptor: A = e4m3 (0), B = e4m3 (0) or e2m1 (5), both K-major, UE8M0
// scales, `sf` = which byte of the 32-bit scale columns this 32-k step uses (A and B alike)
__device__ __forceinline__ uint32_t idesc_mx(uint32_t bfmt, uint32_t sf) {
  return (sf << 4) | (0u << 7) | (bfmt << 10) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) |
         ((uint32_t)(BM >> 4) << 24) | (sf << 29);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const MxGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;            // swizzled tiles need 1024-byte alignment
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t bar0 = base + kStages * kStageBytes;
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto sf_full = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
  const uint32_t tfull = bar0 + 8u * (3 * kStages), tempty = tfull + 8u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + kStages * kStageBytes + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + kStages * kStageBytes + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = p.K / BK;
  const int nt = (p.N + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(full(s), 1);
      tc::mbar_init(empty(s), 1);
      tc::mbar_init(sf_full(s), 4);
    }
    tc::mbar_init(tfull, 1);
    tc::mbar_init(tempty, kEpiWarps);
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tc::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // set-up done: wait for the kernel before this one (operands and tile lists are its outputs)
  tf_pdl_sync();
  const int mt = p.tile_expert ? *p.num_m_tiles : (p.M + BM - 1) / BM;
  const int tiles = mt * nt;
  const int stride = gridDim.x;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc::prefetch_tmap(&mapA);
      tc::prefetch_tmap(&mapB);
      const uint32_t tx = BM * 128 + (p.b_fp4 ? BN * 64 : BN * 128) + kSfaBytes + kSfbBytes;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += stride) {
        const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
        const int nb0 = n0 + (p.tile_expert ? p.tile_expert[tile % mt] * p.N : 0);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          if (!(ok = tc::mbar_wait(empty(s), ((it / kStages) & 1) ^ 1, abort_flag))) break;
          tc::mbar_expect_tx(full(s), tx);
          const uint32_t sa = base + s * kStageBytes;
          tc::tma_load_2d(sa, &mapA, kb * BK, m0, full(s));
          tc::tma_load_2d(sa + BM * 128, &mapB, kb * BK, nb0, full(s));
          tc::bulk_g2s(sa + (BM + BN) * 128, p.sfa + ((long)kb * p.sfa_units + m0 / 32) * 128, kSfaBytes, full(s));
          tc::bulk_g2s(sa + (BM + BN) * 128 + kSfaBytes, p.sfb + ((long)kb * p.sfb_units + nb0 / 32) * 128,
                       kSfbBytes, full(s));
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) {}       // copies in flight land before the smem goes back
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t bfmt = p.b_fp4 ? 5u : 0u;
      int it = 0, n_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += stride, ++n_tile) {
        if (!(ok = tc::mbar_wait(tempty, (n_tile & 1) ^ 1, abort_flag))) break;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = tc::mbar_wait(full(s), ph, abort_flag))) break;
          if (!(ok = tc::mbar_wait(sf_full(s), ph, abort_flag))) break;
          tc::tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint64_t da = tc::smem_desc_sw128(sa), db = tc::smem_desc_sw128(sa + BM * 128);
          const uint32_t sfa = tmem_base + kAccCols + s * kSfCols, sfb = sfa + 4;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_mx(tmem_base, da + 2 * k, db + 2 * k, idesc_mx(bfmt, k), sfa, sfb, (kb == 0 && k == 0) ? 0u : 1u);
          tc::mma_commit(empty(s));          // frees the stage and, with it, the stage's scale columns
        }
        if (ok) tc::mma_commit(tfull);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ scale movers
    // When full(s) completes for lap r of the ring, the MMAs that read scale columns s in lap r - 1 are
    // done (the producer refilled the stage only after their commit): the columns are free.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += stride) {
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % kStages;
        if (!(ok = tc::mbar_wait(full(s), (it / kStages) & 1, abort_flag))) break;
        const uint8_t* sf = aligned + s * kStageBytes + (BM + BN) * 128;
        uint32_t va[4], vb[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) va[j] = *reinterpret_cast<const uint32_t*>(sf + j * 128 + lane * 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) vb[j] = *reinterpret_cast<const uint32_t*>(sf + kSfaBytes + j * 128 + lane * 4);
        const uint32_t t = tmem_base + lane_base + kAccCols + s * kSfCols;
        tmem_st4(t, va);
        tmem_st8(t + 4, vb);
        tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(sf_full(s));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int ew = warp - 6;
    const int quad = warp & 3;                 // TMEM lanes this warp may touch: [32*quad, 32*quad+32)
    const int half = ew >> 2;                  // which 128 of the tile's 256 columns
    int n_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += stride, ++n_tile) {
      const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
      const int row = m0 + quad * 32 + lane;
      const int col0 = n0 + half * 128;
      if (!(ok = tc::mbar_wait(tfull, n_tile & 1, abort_flag))) break;
      tc::tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + half * 128;
#pragma unroll
      for (int c = 0; c < 128; c += 64) {
        uint32_t v0[32], v1[32];
        tc::tmem_ld32(taddr + c, v0);
        tc::tmem_ld32(taddr + c + 32, v1);
        tc::tmem_ld_wait();
        if (c == 64) {
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(tempty);
        }
        if (row < p.M) {
          const long off = (long)row * p.ldc + col0 + c;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t* v = h ? v1 : v0;
            if (p.out_kind == 0) {
              float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + off + h * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col0 + c + h * 32 + 4 * i < p.N)
                  dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
            } else {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + off + h * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 hh[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  hh[j] = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                if (col0 + c + h * 32 + 8 * i < p.N) dst[i] = *reinterpret_cast<uint4*>(hh);
              }
            }
          }
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) tf_report(p.status, TF_TIMEOUT, 140, blockIdx.x, p.b_fp4);
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// MXFP8 quantiser of activation rows with the scales in the unit layout.
// One thread per (row, 32 inputs).  dst row = pair_dst[r] when given (expert-sorted padded rows),
// source row = r / x_div.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ int mx_exponent(float amax) {
  // smallest power of two >= amax / 448 (so the scaled values fit e4m3)
  if (!(amax > 0.f)) return -127;
  int e2;
  const float m = frexpf(amax * (1.f / 448.f), &e2);       // value = m * 2^e2, m in [0.5, 1)
  return max(-127, min(127, (m == 0.5f) ? e2 - 1 : e2));
}

template <typename T>
__global__ void __launch_bounds__(128) quant_rows_mx_units_kernel(const T* __restrict__ x, int ldx, int x_div,
                                                                  const int* __restrict__ pair_dst,
                                                                  uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                  int sf_units, int rows, int K) {
  tf_pdl_sync();
  const int ks = K / 32;
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * ks) return;
  const int r = (int)(i / ks), b = (int)(i % ks);
  const int dst = pair_dst ? pair_dst[r] : r;
  if (dst < 0) return;
  const T* src = x + (long)(r / x_div) * ldx + b * 32;
  // 32 inputs = 64 (or 128) contiguous bytes, 16-byte aligned (ldx is a multiple of 8 elements)
  constexpr int kVec = 16 / sizeof(T);
  T raw[32];
#pragma unroll
  for (int j = 0; j < 32 / kVec; ++j)
    *reinterpret_cast<uint4*>(raw + j * kVec) = *reinterpret_cast<const uint4*>(src + j * kVec);
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v[j] = to_f<T>(raw[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const int ex = mx_exponent(amax);
  const float inv = exp2f((float)-ex);
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi =
        __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    o[j] = lo | (hi << 16);
  }
  uint4* out = reinterpret_cast<uint4*>(q + (long)dst * K + b * 32);
  out[0] = make_uint4(o[0], o[1], o[2], o[3]);
  out[1] = make_uint4(o[4], o[5], o[6], o[7]);
  sf[((long)(b >> 2) * sf_units + (dst >> 5)) * 128 + (dst & 31) * 4 + (b & 3)] = (uint8_t)(ex + 127);
}

// Clamped SwiGLU of [rows, 2I] bf16 (gate | up) -> MXFP8 rows [rows, I] + unit-layout scales.
// One thread per (row, 32 outputs).  `num_rows` (device, optional) bounds the rows at run time.
__global__ void __launch_bounds__(128) swiglu_rows_mx_units_kernel(const __nv_bfloat16* __restrict__ y, int ldy,
                                                                   uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                   int sf_units, int rows, int I, float limit,
                                                                   const int* __restrict__ num_rows) {
  tf_pdl_sync();
  const int ks = I / 32;
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int live = num_rows ? min(rows, *num_rows) : rows;
  if (i >= (long)live * ks) return;
  const int r = (int)(i / ks), b = (int)(i % ks);
  const __nv_bfloat16* g = y + (long)r * ldy + b * 32;
  const __nv_bfloat16* u = g + I;
  __nv_bfloat16 gr[32], ur[32];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    *reinterpret_cast<uint4*>(gr + 8 * j) = *reinterpret_cast<const uint4*>(g + 8 * j);
    *reinterpret_cast<uint4*>(ur + 8 * j) = *reinterpret_cast<const uint4*>(u + 8 * j);
  }
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float gate = __bfloat162float(gr[j]), up = __bfloat162float(ur[j]);
    if (limit > 0.f) {
      gate = fminf(gate, limit);
      up = fminf(fmaxf(up, -limit), limit);
    }
    v[j] = gate / (1.f + __expf(-gate)) * up;
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const int ex = mx_exponent(amax);
  const float inv = exp2f((float)-ex);
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * inv, v[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi =
        __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * inv, v[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    o[j] = lo | (hi << 16);
  }
  uint4* out = reinterpret_cast<uint4*>(q + (long)r * I + b * 32);
  out[0] = make_uint4(o[0], o[1], o[2], o[3]);
  out[1] = make_uint4(o[4], o[5], o[6], o[7]);
  sf[((long)(b >> 2) * sf_units + (r >> 5)) * 128 + (r & 31) * 4 + (b & 3)] = (uint8_t)(ex + 127);
}

// row-major UE8M0 scales [rows, K/32] -> unit layout [K/128][units][128]
__global__ void __launch_bounds__(256) sf_to_units_kernel(const uint8_t* __restrict__ s, uint8_t* __restrict__ out,
                                                          long rows, int ks, int units) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * ks) return;
  const long r = i / ks;
  const int b = (int)(i % ks);
  out[((long)(b >> 2) * units + (r >> 5)) * 128 + (r & 31) * 4 + (b & 3)] = s[i];
}

// fp32 power-of-two scales per 128 x 128 block [rows/128, K/128] -> unit layout (every 32 x 32
// sub-block of a block carries the block's exponent).  `bad` counts scales that are not powers of two
// in the UE8M0 range.
__global__ void __launch_bounds__(256) block_scales_to_units_kernel(const float* __restrict__ s, int lds,
                                                                    uint8_t* __restrict__ out, long rows, int kb_n,
                                                                    int units, int* __restrict__ bad) {
  tf_pdl_sync();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;      // (row, k block)
  if (i >= rows * kb_n) return;
  const long r = i / kb_n;
  const int kb = (int)(i % kb_n);
  const float v = s[(r >> 7) * lds + kb];
  int e2;
  const float m = frexpf(v, &e2);                                  // v = m * 2^e2
  int ex = e2 - 1;
  if (!(v > 0.f) || m != 0.5f || ex < -127 || ex > 127) {
    if (bad) atomicAdd(bad, 1);
    ex = -127;
  }
  const uint32_t byte = (uint32_t)(ex + 127);
  *reinterpret_cast<uint32_t*>(out + ((long)kb * units + (r >> 5)) * 128 + (r & 31) * 4) = byte * 0x01010101u;
}

int g_sms = 0;

inline bool make_map_fp4(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K) {
  auto fn = tc::encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 31) || ((K / 2) & 31) || (K & 127)) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K / 2};
  cuuint32_t box[2] = {128, (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Scale units needed for `rows` rows that tiles of `tile_rows` rows may touch (whole tiles).
TF_API long tf_mx_sf_units(long rows, int tile_rows) {
  return (rows + tile_rows - 1) / tile_rows * tile_rows / 32;
}

// C[M, N] (ldc elements per row; out_kind 0 = f32, 2 = bf16) = A (e4m3 [M, K], row pitch lda bytes) x
// B^T.  B: e4m3 [b_rows, K] (row pitch ldb bytes) or, with b_fp4, packed e2m1 [b_rows, K / 2].
// sfa / sfb: unit-layout scales with sfa_units / sfb_units units per 128-deep k block
// (tf_mx_sf_units(M, 128) and tf_mx_sf_units(b_rows, 256) or more).  Grouped form: tile_expert /
// num_m_tiles as in tf_gemm_tc, b_rows = experts * N, N a multiple of 256.
TF_API int tf_gemm_mx(const void* A, long lda, const void* B, long ldb, long b_rows, int b_fp4, const void* sfa,
                      int sfa_units, const void* sfb, int sfb_units, void* C, int ldc, int out_kind, int M, int N,
                      int K, const int* tile_expert, const int* num_m_tiles, void* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || K % BK || N % 8 || (out_kind != 0 && out_kind != 2)) return -1;
  if (!A || !B || !sfa || !sfb || !C) return -1;
  if (tile_expert && (N % BN || !num_m_tiles)) return -1;
  const long m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  if (sfa_units < m_tiles * (BM / 32)) return -1;
  if (sfb_units < (tile_expert ? b_rows / 32 : n_tiles * (BN / 32))) return -1;
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15)) return -1;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc * (out_kind == 0 ? 4 : 2)) % 16) return -1;
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  }
  CUtensorMap mA, mB;
  if (!tc::make_map_2d(&mA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM)) return -4;
  if (b_fp4) {
    if (ldb != K / 2 || !make_map_fp4(&mB, B, b_rows, K)) return -4;
  } else if (!tc::make_map_2d(&mB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_rows, K, ldb, BN)) {
    return -4;
  }
  MxGemmParams p;
  p.M = M; p.N = N; p.K = K; p.b_fp4 = b_fp4 ? 1 : 0;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.sfa_units = sfa_units; p.sfb_units = sfb_units;
  p.C = C; p.ldc = ldc; p.out_kind = out_kind;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles;
  p.status = reinterpret_cast<TfStatusWord*>(status);
  const long tiles = m_tiles * n_tiles;
  const int grid = (int)(tiles < g_sms ? tiles : g_sms);
  tf_launch(gemm_mx_kernel, dim3(grid), dim3(kThreads), kSmemBytes, st, mA, mB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// x [rows / x_div source rows, K] (xkind 0 f32, 1 f16, 2 bf16; row pitch ldx elements) -> q e4m3
// [dst rows, K] + unit-layout scales.  pair_dst (optional): destination row of every source pair.
TF_API int tf_quant_rows_mx_units(const void* x, int xkind, int ldx, int x_div, const int* pair_dst, void* q, void* sf,
                                  int sf_units, int rows, int K, cudaStream_t st) {
  if (rows <= 0 || K % 128 || x_div <= 0 || !x || !q || !sf || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  const long n = (long)rows * (K / 32);
  const dim3 grid((unsigned)((n + 127) / 128));
  uint8_t* qq = reinterpret_cast<uint8_t*>(q);
  uint8_t* ss = reinterpret_cast<uint8_t*>(sf);
  if (xkind == 0)
    tf_launch(quant_rows_mx_units_kernel<float>, grid, dim3(128), 0, st, reinterpret_cast<const float*>(x), ldx, x_div,
              pair_dst, qq, ss, sf_units, rows, K);
  else if (xkind == 1)
    tf_launch(quant_rows_mx_units_kernel<__half>, grid, dim3(128), 0, st, reinterpret_cast<const __half*>(x), ldx,
              x_div, pair_dst, qq, ss, sf_units, rows, K);
  else if (xkind == 2)
    tf_launch(quant_rows_mx_units_kernel<__nv_bfloat16>, grid, dim3(128), 0, st,
              reinterpret_cast<const __nv_bfloat16*>(x), ldx, x_div, pair_dst, qq, ss, sf_units, rows, K);
  else
    return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

TF_API int tf_swiglu_rows_mx_units(const void* y, int ldy, void* q, void* sf, int sf_units, int rows, int I,
                                   float limit, const int* num_rows, cudaStream_t st) {
  if (rows <= 0 || I % 128 || !y || !q || !sf || ldy % 8 || (reinterpret_cast<uintptr_t>(y) & 15)) return -1;
  const long n = (long)rows * (I / 32);
  tf_launch(swiglu_rows_mx_units_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st,
            reinterpret_cast<const __nv_bfloat16*>(y), ldy, reinterpret_cast<uint8_t*>(q),
            reinterpret_cast<uint8_t*>(sf), sf_units, rows, I, limit, num_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// row-major UE8M0 scales [rows, K / 32] -> unit layout (`out` holds K / 128 * units * 128 bytes, zeroed by the caller)
TF_API int tf_mx_sf_to_units(const void* s, void* out, long rows, int K, int units, cudaStream_t st) {
  if (rows <= 0 || K % 128 || units * 32L < rows) return -1;
  const long n = rows * (K / 32);
  tf_launch(sf_to_units_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st,
            reinterpret_cast<const uint8_t*>(s), reinterpret_cast<uint8_t*>(out), rows, K / 32, units);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// fp32 scales per 128 x 128 block (row pitch lds) -> unit layout; *bad (device, optional) counts
// scales that are not exact powers of two in range (such a matrix cannot take this path)
TF_API int tf_mx_block_scales_to_units(const float* s, int lds, void* out, long rows, int K, int units, int* bad,
                                       cudaStream_t st) {
  if (rows <= 0 || K % 128 || units * 32L < rows) return -1;
  const long n = rows * (K / 128);
  tf_launch(block_scales_to_units_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, s, lds,
            reinterpret_cast<uint8_t*>(out), rows, K / 128, units, bad);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
