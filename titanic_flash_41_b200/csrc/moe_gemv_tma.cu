// Routed-expert GEMV of the decode step, weights streamed by TMA.
//
//   Y[pair, n] = sum_k X[row(pair), k] * W[expert][n, k]      MXFP4 weights (quad-packed layout),
//                                                             e4m3 activations with one scale per row
//
// The register-fed form of this op (smallm_gemm.cu) keeps one step of loads in flight per warp
// and reaches ~0.4 of HBM bandwidth.  Here a producer warp issues TMA tile loads (this GPU's own
// memory, 128-byte swizzle, no multicast) of 32 weight rows x 256 k into a ring of shared-memory
// stages, so the bytes in flight per SM are set by the ring (3 CTAs x 6 stages x 8 KB), not by
// registers; four consumer warps take the stages in turn (a K split), read their fragments with
// conflict-free 16-byte shared loads, convert e2m1 -> e4m3 with two shifts and two masks per four
// weights and issue m16n8k32 tensor-core steps, one 32-wide scale group per step.  Partial sums of
// the four warps are added in a fixed order.  The dual form computes w1 and w3 tiles together and
// applies the clamped SwiGLU.  Every mbarrier wait is bounded; a time-out raises the CTA's abort
// flag, records TF_TIMEOUT and the CTA leaves without storing.
//
// Replaces for the B200 build the b12x `moe.w4a8.compact_micro` / `integration.tp_moe.dynamic`
// decode bundles of the reference (src/moe.rs:997 run_live_for_ffn).
#include "tc.cuh"

namespace {

constexpr int kConsumers = 4;
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kTileN = 32;                 // weight rows (output columns) per CTA
constexpr int kStages = 4;
constexpr int kBoxBytes = kTileN * 128;    // 32 rows x 128 bytes (256 k of packed e2m1), 128-byte swizzle
// per matrix and stage: two boxes (512 k) + 32 rows x 16 scale bytes, padded so every stage of the
// dual form keeps the boxes 1024-byte aligned
constexpr int kMatStage = 2 * kBoxBytes + 1024;
constexpr int kRedBytes = kConsumers * 4 * 2 * 32 * 4 * 4;   // [warps][NT<=4][MT<=2][32 lanes][4] floats

struct MoeTmaParams {
  const uint8_t* S;          // [experts][N][lds] UE8M0, one per 32 k
  const uint8_t* S3;
  long s_group_stride;       // bytes between experts
  int lds;
  const uint8_t* X;          // e4m3, 8-run order (see tf_quant_rows_e4m3_perm), ldx bytes per row
  int ldx;
  const float* x_scale;
  void* Y;
  int ldy, out_kind;         // 0 f32, 1 f16, 2 bf16
  int N, K;
  const int* group_expert;
  const int* group_start;
  const int* group_count;
  const int* n_groups;
  const int* sorted_pairs;
  int x_div;
  float swiglu_limit;
  TfStatusWord* status;
};

__device__ __forceinline__ void mma_e4m3(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  const float z = 0.f;
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}
// barrier among the four consumer warps only (the producer runs ahead on its own schedule)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ uint32_t cvt4(uint32_t x) { return ((x << 4) & 0x80808080u) | ((x << 2) & 0x1c1c1c1cu); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// one 512-k stage for one consumer warp: four 128-k parts, NT tiles of 16 weight rows; weights and
// their scale bytes both come from the stage
template <int MT, bool DUAL>
__device__ __forceinline__ void consume_stage(uint32_t stage, int k_base, const uint8_t* const xb[MT],
                                              float (&acc)[DUAL ? 4 : 2][MT][4]) {
  constexpr int NT = DUAL ? 4 : 2;
  constexpr int NM = DUAL ? 2 : 1;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t sc_base = stage + NM * 2 * kBoxBytes;       // [NM][32 rows][16 scale bytes]
#pragma unroll
  for (int part = 0; part < 4; ++part) {
    const int kb = k_base + part * 128;
    uint4 w0[NT], w8[NT];
    uint32_t c0[NT], c8[NT];
#pragma unroll
    for (int ti = 0; ti < NT; ++ti) {
      const uint32_t box = stage + ((ti >> 1) * 2 + (part >> 1)) * kBoxBytes;
      const int r0 = 16 * (ti & 1) + g, r8 = r0 + 8, c = (part & 1) * 4 + t;
      w0[ti] = lds128(box + r0 * 128 + ((c ^ (r0 & 7)) << 4));
      w8[ti] = lds128(box + r8 * 128 + ((c ^ (r8 & 7)) << 4));
      const uint32_t sc = sc_base + (ti >> 1) * (kTileN * 16) + part * 4;
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(c0[ti]) : "r"(sc + r0 * 16));
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(c8[ti]) : "r"(sc + r8 * 16));
    }
    uint2 xv[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) xv[m][j] = *reinterpret_cast<const uint2*>(xb[m] + kb + 32 * j + 8 * t);
#pragma unroll
    for (int ti = 0; ti < NT; ++ti) {
      const uint32_t* a0w = reinterpret_cast<const uint32_t*>(&w0[ti]);
      const uint32_t* a8w = reinterpret_cast<const uint32_t*>(&w8[ti]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a0 = cvt4(a0w[j] & 0x0f0f0f0fu), a2 = cvt4((a0w[j] >> 4) & 0x0f0f0f0fu);
        const uint32_t a1 = cvt4(a8w[j] & 0x0f0f0f0fu), a3 = cvt4((a8w[j] >> 4) & 0x0f0f0f0fu);
        const float s0 = __uint_as_float(((c0[ti] >> (8 * j)) & 0xffu) << 23);
        const float s8 = __uint_as_float(((c8[ti] >> (8 * j)) & 0xffu) << 23);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float dd[4];
          mma_e4m3(dd, a0, a1, a2, a3, xv[m][j].x, xv[m][j].y);
          acc[ti][m][0] = fmaf(s0, dd[0], acc[ti][m][0]);
          acc[ti][m][1] = fmaf(s0, dd[1], acc[ti][m][1]);
          acc[ti][m][2] = fmaf(s8, dd[2], acc[ti][m][2]);
          acc[ti][m][3] = fmaf(s8, dd[3], acc[ti][m][3]);
        }
      }
    }
  }
}

// Persistent: every CTA walks (expert group, 32-row tile) work items; the producer streams the
// stages of one item after another without draining the ring in between.
template <bool DUAL>
__global__ void __launch_bounds__(kThreads) moe_gemv_tma_kernel(const __grid_constant__ CUtensorMap mapW,
                                                                const __grid_constant__ CUtensorMap mapW3,
                                                                const __grid_constant__ CUtensorMap mapS,
                                                                const __grid_constant__ CUtensorMap mapS3,
                                                                const MoeTmaParams p) {
  constexpr int NT = DUAL ? 4 : 2;
  constexpr int NM = DUAL ? 2 : 1;
  constexpr int kStageBytes = NM * kMatStage;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t bar0 = base + kStages * kStageBytes;                       // full[kStages], empty[kStages]
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + kStages * kStageBytes + 8 * 2 * kStages);
  float(*red)[32][4] = reinterpret_cast<float(*)[32][4]>(aligned + kStages * kStageBytes + 256);

  const int ntiles = p.N / kTileN;
  const int items = *p.n_groups * ntiles;
  const int nsteps = p.K / 512;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(full(s), 1);
      tc::mbar_init(empty(s), 1);
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();

  if (warp == kConsumers) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc::prefetch_tmap(&mapW);
      tc::prefetch_tmap(&mapS);
      if (DUAL) {
        tc::prefetch_tmap(&mapW3);
        tc::prefetch_tmap(&mapS3);
      }
      bool ok = true;
      int it = 0;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int slot = item / ntiles, n0 = (item % ntiles) * kTileN;
        const int e = p.group_expert[slot], rows = p.group_count[slot];
        const int passes = rows <= 8 ? 1 : (rows + 15) / 16;
        const int row = e * p.N + n0;
        for (int q = 0; q < passes * nsteps && ok; ++q, ++it) {
          const int s = q % nsteps, st = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = tc::mbar_wait(empty(st), ph ^ 1, abort_flag))) break;
          tc::mbar_expect_tx(full(st), NM * (2 * kBoxBytes + kTileN * 16));
          const uint32_t dst = base + st * kStageBytes;
          tc::tma_load_2d(dst, &mapW, s * 256, row, full(st));
          tc::tma_load_2d(dst + kBoxBytes, &mapW, s * 256 + 128, row, full(st));
          tc::tma_load_2d(dst + NM * 2 * kBoxBytes, &mapS, s * 16, row, full(st));
          if (DUAL) {
            tc::tma_load_2d(dst + 2 * kBoxBytes, &mapW3, s * 256, row, full(st));
            tc::tma_load_2d(dst + 3 * kBoxBytes, &mapW3, s * 256 + 128, row, full(st));
            tc::tma_load_2d(dst + 4 * kBoxBytes + kTileN * 16, &mapS3, s * 16, row, full(st));
          }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) {}          // let copies in flight land before the CTA exits
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers (K split by stage)
    const int g = lane >> 2;
    bool ok = true;
    int it0 = 0;                                     // stage counter at the start of the current pass
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int slot = item / ntiles, n0 = (item % ntiles) * kTileN;
      const int rows = p.group_count[slot];
      const int* pairs = p.sorted_pairs + p.group_start[slot];
      const int passes = rows <= 8 ? 1 : (rows + 15) / 16;
      for (int pass = 0; pass < passes; ++pass, it0 += nsteps) {
        const int row_base = (rows <= 8) ? 0 : pass * 16;
        const bool two = rows - row_base > 8;           // MT = 2 when more than 8 rows remain
        const uint8_t* xb[2];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const int r = min(row_base + m * 8 + g, rows - 1);
          xb[m] = p.X + (long)(pairs[r] / p.x_div) * p.ldx;
        }
        float acc[NT][2][4];
#pragma unroll
        for (int ti = 0; ti < NT; ++ti)
#pragma unroll
          for (int m = 0; m < 2; ++m) acc[ti][m][0] = acc[ti][m][1] = acc[ti][m][2] = acc[ti][m][3] = 0.f;
        for (int s = warp; s < nsteps; s += kConsumers) {
          const int it = it0 + s, st = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (ok) ok = tc::mbar_wait(full(st), ph, abort_flag);
          if (ok) {
            const uint32_t stage = base + st * kStageBytes;
            if (two) {
              consume_stage<2, DUAL>(stage, s * 512, xb, acc);
            } else {
              float a1[NT][1][4];
              const uint8_t* x1[1] = {xb[0]};
#pragma unroll
              for (int ti = 0; ti < NT; ++ti)
#pragma unroll
                for (int i = 0; i < 4; ++i) a1[ti][0][i] = acc[ti][0][i];
              consume_stage<1, DUAL>(stage, s * 512, x1, a1);
#pragma unroll
              for (int ti = 0; ti < NT; ++ti)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[ti][0][i] = a1[ti][0][i];
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(empty(st));
          }
        }
        // ---- fixed-order sum over the four warps, then the epilogue
#pragma unroll
        for (int ti = 0; ti < NT; ++ti)
#pragma unroll
          for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[(warp * NT + ti) * 2 + m][lane][i] = acc[ti][m][i];
        consumer_sync();
        const bool good = *abort_flag == 0;
        constexpr int kSlots = 2 * 2 * 32 * 4;
        for (int sidx = threadIdx.x; good && sidx < kSlots; sidx += kConsumers * 32) {
          const int i = sidx & 3, ln = (sidx >> 2) & 31, m = (sidx >> 7) % 2, h = (sidx >> 7) / 2;
          if (m == 1 && !two) continue;
          float v = 0.f, v3 = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumers; ++w) {
            v += red[(w * NT + h) * 2 + m][ln][i];
            if (DUAL) v3 += red[(w * NT + 2 + h) * 2 + m][ln][i];
          }
          const int gg = ln >> 2, tt = ln & 3;
          const int n = n0 + 16 * h + gg + ((i & 2) ? 8 : 0);
          const int r = row_base + m * 8 + 2 * tt + (i & 1);
          if (r < rows && n < p.N) {
            const float xs = p.x_scale[pairs[r] / p.x_div] * 64.f;   // row scale and the e2m1 -> e4m3 offset 2^6
            v *= xs;
            v3 *= xs;
            float o = v;
            if (DUAL) {
              float gate = v, up = v3;
              if (p.swiglu_limit > 0.f) {
                gate = fminf(gate, p.swiglu_limit);
                up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit);
              }
              o = gate / (1.f + __expf(-gate)) * up;
            }
            const long off = (long)pairs[r] * p.ldy + n;
            if (p.out_kind == 0) reinterpret_cast<float*>(p.Y)[off] = o;
            else if (p.out_kind == 1) reinterpret_cast<__half*>(p.Y)[off] = __float2half(o);
            else reinterpret_cast<__nv_bfloat16*>(p.Y)[off] = __float2bfloat16(o);
          }
        }
        consumer_sync();
      }
    }
  }
  if (*abort_flag && threadIdx.x == 0) tf_report(p.status, TF_TIMEOUT, 130, blockIdx.x, 0);
}

}  // namespace

// W / W3: [experts][N][K/2] quad-packed e2m1 (row pitch ldw bytes, experts contiguous); S / S3: UE8M0
// [experts][N][lds] with lds % 16 == 0; X / x_scale from tf_quant_rows_e4m3_perm.  N % 32 == 0, K % 512 == 0.
TF_API int tf_moe_gemv_w4a8_tma(const void* W, const void* W3, const void* S, const void* S3, int experts, int ldw,
                                int lds, long s_group_stride, const void* X, int ldx, const float* x_scale, void* Y,
                                int ldy, int out_kind, int N, int K, const int* group_expert, const int* group_start,
                                const int* group_count, const int* n_groups, const int* sorted_pairs, int x_div,
                                int slots, float swiglu_limit, void* status, cudaStream_t stream) {
  if (N % kTileN != 0 || K % 512 != 0 || (ldx % 8) != 0 || (ldw % 16) != 0 || (lds % 16) != 0 || !x_scale || slots < 1)
    return -1;
  if (s_group_stride != (long)N * lds) return -1;       // scales of all experts form one [experts*N, lds] matrix
  CUtensorMap mw, mw3, ms, ms3;
  const uint64_t rows = (uint64_t)experts * N;
  if (!tc::make_map_2d(&mw, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, (uint64_t)K / 2, (uint64_t)ldw, kTileN)) return -2;
  if (!tc::make_map_2d_plain(&ms, S, rows, (uint64_t)K / 32, (uint64_t)lds, 16, kTileN)) return -2;
  mw3 = mw;
  ms3 = ms;
  if (W3 && (!tc::make_map_2d(&mw3, W3, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, (uint64_t)K / 2, (uint64_t)ldw, kTileN) ||
             !tc::make_map_2d_plain(&ms3, S3, rows, (uint64_t)K / 32, (uint64_t)lds, 16, kTileN)))
    return -2;
  MoeTmaParams p;
  p.S = (const uint8_t*)S; p.S3 = (const uint8_t*)S3; p.s_group_stride = s_group_stride; p.lds = lds;
  p.X = (const uint8_t*)X; p.ldx = ldx; p.x_scale = x_scale; p.Y = Y; p.ldy = ldy; p.out_kind = out_kind;
  p.N = N; p.K = K; p.group_expert = group_expert; p.group_start = group_start; p.group_count = group_count;
  p.n_groups = n_groups; p.sorted_pairs = sorted_pairs; p.x_div = x_div > 0 ? x_div : 1;
  p.swiglu_limit = swiglu_limit; p.status = (TfStatusWord*)status;
  const bool dual = W3 != nullptr;
  const int smem = kStages * (dual ? 2 : 1) * kMatStage + 1024 + 256 + kRedBytes;
  static bool attr_set = false;
  static int sms = 0;
  if (!attr_set) {
    cudaFuncSetAttribute(moe_gemv_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         kStages * 2 * kMatStage + 1024 + 256 + kRedBytes);
    cudaFuncSetAttribute(moe_gemv_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         kStages * kMatStage + 1024 + 256 + kRedBytes);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    attr_set = true;
  }
  const long items = (long)slots * (N / kTileN);
  const int per_sm = dual ? 2 : 3;
  const int grid = (int)(items < (long)sms * per_sm ? items : (long)sms * per_sm);
  if (dual) moe_gemv_tma_kernel<true><<<grid, kThreads, smem, stream>>>(mw, mw3, ms, ms3, p);
  else moe_gemv_tma_kernel<false><<<grid, kThreads, smem, stream>>>(mw, mw3, ms, ms3, p);
  return (int)cudaGetLastError();
}
