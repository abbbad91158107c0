// Routed-expert GEMV of the decode step on the block-scaled tensor cores.
//
// The experts are stored as MXFP4 (packed e2m1, one UE8M0 scale per 32 inputs).  Unpacking the
// nibbles on the CUDA cores costs about three instructions per weight, which holds a
// register-fed kernel at ~0.4 of the HBM rate.  Here the tensor core consumes the nibbles and the
// scales itself: `tcgen05.mma kind::mxf8f6f4.block_scale` with
//   A = 128 output features x 32 inputs of e2m1, brought by TMA in the padded form (sixteen
//       4-bit values per 16 bytes of shared memory) the instruction expects, 128-byte swizzle;
//   B = 16 (or 32: verification blocks of 17..32 rows) activation rows x 32 inputs of e4m3 (MXFP8:
//       UE8M0 scale per 32 inputs);
//   scale factors in tensor memory: for A four 32-bit columns per 128 inputs (column j holds
//       rows 32j..32j+31, byte b the b-th group of 32 inputs), for B one column per 128 inputs;
//   D = f32 in tensor memory, 128 lanes x 16 (32) columns.
// The CUDA cores touch only the scales (16 bytes per row and 512 inputs: TMA stages them in shared
// memory with the data, the four warps that later run the epilogue rearrange them and write them
// to tensor memory with tcgen05.st) and the 16 x 128 results.
//
// Work item = (active expert, 128 output features); persistent CTAs, one per SM:
//   warp 0  TMA producer   (ring of 128-input stages: weights of w1 [and w3] + activation rows;
//                           ring of scale blocks, one per 512 inputs)
//   warp 1  MMA issuer     (owns the TMEM allocation)
//   warps 2-5  scale loaders, then epilogue (clamped SwiGLU for the fused w1/w3 form)
// Every wait is bounded: on a time-out the CTA raises its abort flag, reports TF_TIMEOUT, frees its
// tensor memory and returns.
//
// Reference behaviour: the routed-expert decode path of the reference's MoE kernels
// (runtime/kernels/moe: grouped MXFP4 expert matvec with clamped SwiGLU).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "tc.cuh"

namespace {

constexpr int kThreads = 192;
constexpr int kTile = 128;          // output features per work item
constexpr int kRows = 16;           // activation rows (MMA N) of the narrow form; the wide form takes 32
constexpr int kBK = 128;            // inputs per stage
constexpr int kSuper = 512;         // inputs per scale load (4 stages)
constexpr int kSfBufs = 4;          // scale-factor slots in tensor memory (loaders run ahead of the MMAs)

struct MxParams {
  const int* g_expert;
  const int* g_start;
  const int* g_count;
  const int* n_groups;
  const int* sorted_pairs;
  const uint8_t* sw1;               // [experts, N, K/32] UE8M0
  const uint8_t* sw3;
  const uint8_t* sx;                // [x_rows, K/32] UE8M0
  void* out;
  uint8_t* q_out;                   // fused form: MXFP8 copy of the output rows (values, then scales)
  uint8_t* q_scale;
  int ldo, N, K, topk, x_rows, a_tx_bytes, blocked;
  float limit;
  TfStatusWord* status;
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t v[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t v[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// D[tmem] (+)= (A * scale_A) (B * scale_B)^T, scales read from tensor memory; ONE thread issues
__device__ __forceinline__ void mma_mx(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// block-scaled instruction descriptor: A = e2m1 (5), B = e4m3 (0), both K-major, UE8M0 scales,
// `sf` = which byte of the 32-bit scale columns this 32-input step uses (same for A and B)
__device__ __forceinline__ uint32_t idesc_mx(uint32_t sf, int rows) {
  return (sf << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(rows >> 3) << 17) | (1u << 23) |
         ((uint32_t)(kTile >> 4) << 24) | (sf << 29);
}

// stages of the weight ring: what fits beside the scale slots in 227 KB
__host__ __device__ constexpr int mx_stages(int dual, int rows) { return dual ? (rows > 16 ? 5 : 6) : (rows > 16 ? 10 : 11); }

template <int DUAL, int ROWS>
__global__ void __launch_bounds__(kThreads, 1)
moe_mx_kernel(const __grid_constant__ CUtensorMap mapW1, const __grid_constant__ CUtensorMap mapW3,
              const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapS1,
              const __grid_constant__ CUtensorMap mapS3, const __grid_constant__ CUtensorMap mapSX, const MxParams p) {
  constexpr int kMats = DUAL ? 2 : 1;
  constexpr int kRows = ROWS;
  constexpr int kStages = mx_stages(DUAL, ROWS);
  // tensor-memory columns: accumulators [0, kAccCols) = buf * 2 * kRows + mat * kRows; A scales
  // [kAccCols, kAccCols + 128) = slot * 32 + mat * 16; B scales after them = slot * 16
  constexpr int kAccCols = 4 * kRows, kSfaCol = kAccCols, kSfbCol = kAccCols + 128;
  constexpr int kTmemCols = kRows > 16 ? 512 : 256;
  // scale bytes of one 512-input block: [128 rows][16] per matrix, then [kRows][16] of the activations
  constexpr int kSfsBytes = (kMats * kTile * 16 + kRows * 16 + 127) / 128 * 128;
  constexpr int kStageBytes = kMats * kTile * 128 + kRows * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t sfs0 = base + kStages * kStageBytes;                    // kSfBufs staging slots for scales
  const uint32_t bar0 = sfs0 + kSfBufs * kSfsBytes;
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto sf_full = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto sf_empty = [&](int b) { return bar0 + 8u * (2 * kStages + kSfBufs + b); };
  auto acc_full = [&](int b) { return bar0 + 8u * (2 * kStages + 2 * kSfBufs + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (2 * kStages + 2 * kSfBufs + 2 + b); };
  auto sfs_full = [&](int b) { return bar0 + 8u * (2 * kStages + 2 * kSfBufs + 4 + b); };
  auto sfs_empty = [&](int b) { return bar0 + 8u * (2 * kStages + 3 * kSfBufs + 4 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      aligned + kStages * kStageBytes + kSfBufs * kSfsBytes + 8 * (2 * kStages + 4 * kSfBufs + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(const_cast<uint32_t*>(tmem_slot) + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // DUAL: 0 = one weight tile per item; 1 = w1 and w3 tiles + SwiGLU; 2 = two adjacent tiles of ONE
  // matrix per item (half as many items, each streaming twice the bytes: the second GEMV of the experts)
  constexpr int kItemN = DUAL == 2 ? 2 * kTile : kTile;
  const int tiles_n = p.N / kItemN;
  const int kchunks = p.K / kBK, nsuper = p.K / kSuper;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(full(s), 1);
      tc::mbar_init(empty(s), 1);
    }
    for (int b = 0; b < kSfBufs; ++b) {
      tc::mbar_init(sf_full(b), 4);
      tc::mbar_init(sf_empty(b), 1);
      tc::mbar_init(sfs_full(b), 1);
      tc::mbar_init(sfs_empty(b), 4);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(acc_full(b), 1);
      tc::mbar_init(acc_empty(b), 4);
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tc::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // barriers and tensor memory are set up; only now wait for the kernel before this one (its
  // outputs, the group list first of all, are read from here on)
  tf_pdl_sync();
  const int items = *p.n_groups * tiles_n;
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc::prefetch_tmap(&mapW1);
      if (DUAL) tc::prefetch_tmap(&mapW3);
      tc::prefetch_tmap(&mapX);
      tc::prefetch_tmap(&mapS1);
      tc::prefetch_tmap(&mapSX);
      const uint32_t tx = kMats * p.a_tx_bytes + kRows * 128;
      int it = 0, fsf = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int g = item / tiles_n, n0 = (item % tiles_n) * kItemN;
        const int wrow = p.g_expert[g] * p.N + n0;
        const int xrow = DUAL == 1 ? 0 : p.g_start[g];
        for (int kc = 0; kc < kchunks; ++kc, ++it) {
          if (kc % (kSuper / kBK) == 0) {
            // the scale bytes of the next 512 inputs travel with the data: the four loader warps
            // find them in shared memory instead of waiting on first-touch global loads
            const int sl = fsf % kSfBufs, sc = kc / (kSuper / kBK);
            if (!(ok = tc::mbar_wait(sfs_empty(sl), ((fsf / kSfBufs) & 1) ^ 1, abort_flag))) break;
            tc::mbar_expect_tx(sfs_full(sl), kMats * kTile * 16 + kRows * 16);
            const uint32_t d = sfs0 + sl * kSfsBytes;
            tc::tma_load_2d(d, &mapS1, sc * 16, wrow, sfs_full(sl));
            if (DUAL == 1) tc::tma_load_2d(d + kTile * 16, &mapS3, sc * 16, wrow, sfs_full(sl));
            if (DUAL == 2) tc::tma_load_2d(d + kTile * 16, &mapS1, sc * 16, wrow + kTile, sfs_full(sl));
            tc::tma_load_2d(d + kMats * kTile * 16, &mapSX, sc * 16, xrow, sfs_full(sl));
            ++fsf;
          }
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = tc::mbar_wait(empty(s), ph ^ 1, abort_flag))) break;
          tc::mbar_expect_tx(full(s), tx);
          const uint32_t sa = base + s * kStageBytes;
          // row-major weights: box = 128 rows x 64 bytes at the row pitch; blocked weights: the
          // [128 x 128] block of this (tile, stage) is 8 KB contiguous
          const int wx = p.blocked ? 0 : kc * kBK;
          const int wy = p.blocked ? ((wrow / kTile) * kchunks + kc) * kTile : wrow;
          tc::tma_load_2d(sa, &mapW1, wx, wy, full(s));
          if (DUAL == 1) tc::tma_load_2d(sa + kTile * 128, &mapW3, wx, wy, full(s));
          if (DUAL == 2)
            tc::tma_load_2d(sa + kTile * 128, &mapW1, wx, p.blocked ? wy + kchunks * kTile : wy + kTile, full(s));
          tc::tma_load_2d(sa + kMats * kTile * 128, &mapX, kc * kBK, xrow, full(s));
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
      int it = 0, sfit = 0, n_item = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++n_item) {
        const int ab = n_item & 1;
        if (!(ok = tc::mbar_wait(acc_empty(ab), ((n_item >> 1) & 1) ^ 1, abort_flag))) break;
        const uint32_t td = tmem_base + ab * 2 * kRows;
        for (int sc = 0; sc < nsuper && ok; ++sc, ++sfit) {
          const int sb = sfit % kSfBufs;
          if (!(ok = tc::mbar_wait(sf_full(sb), (sfit / kSfBufs) & 1, abort_flag))) break;
          tc::tc_fence_after();
          const uint32_t sfa = tmem_base + kSfaCol + sb * 32, sfb = tmem_base + kSfbCol + sb * 16;
          for (int c = 0; c < kSuper / kBK; ++c, ++it) {
            const int s = it % kStages;
            if (!(ok = tc::mbar_wait(full(s), (it / kStages) & 1, abort_flag))) break;
            tc::tc_fence_after();
            const uint32_t sa = base + s * kStageBytes;
            const uint64_t da1 = tc::smem_desc_sw128(sa), da3 = tc::smem_desc_sw128(sa + kTile * 128),
                           db = tc::smem_desc_sw128(sa + kMats * kTile * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t acc = (sc == 0 && c == 0 && k == 0) ? 0u : 1u;
              const uint32_t id = idesc_mx(k, kRows);
              mma_mx(td, da1 + 2 * k, db + 2 * k, id, sfa + c * 4, sfb + c * 4, acc);
              if (DUAL) mma_mx(td + kRows, da3 + 2 * k, db + 2 * k, id, sfa + 16 + c * 4, sfb + c * 4, acc);
            }
            tc::mma_commit(empty(s));
          }
          if (ok) tc::mma_commit(sf_empty(sb));
        }
        if (ok) tc::mma_commit(acc_full(ab));
      }
    }
  } else {
    // ------------------------------------------------------------------ scale loaders + epilogue
    // One flat sequence of (item, 512-input block) runs through the loaders: the scale bytes of a
    // block arrive in shared memory by TMA (requested a ring ahead by the producer), each warp
    // rearranges them into the tensor-memory layout for its own lane quadrant, and the epilogue of
    // an item runs only after the first block of the NEXT item has been delivered, so the MMA warp
    // never waits for an epilogue.
    const int quad = warp & 3;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    auto epilogue = [&](int item, int n_item) -> bool {
      const int g = item / tiles_n, n0 = (item % tiles_n) * kItemN;
      const int gs = p.g_start[g], gc = p.g_count[g];
      const int ab = n_item & 1;
      // output row of accumulator column `lane` (-1: nobody routed there)
      int orow = -1;
      if (lane < kRows) {
        if (DUAL == 1) {
          for (int i = 0; i < gc; ++i)
            if (p.sorted_pairs[gs + i] / p.topk == lane) orow = gs + i;
        } else if (lane < gc) {
          orow = p.sorted_pairs[gs + lane];
        }
      }
      if (!tc::mbar_wait(acc_full(ab), (n_item >> 1) & 1, abort_flag)) return false;
      tc::tc_fence_after();
      uint32_t a1[kRows], a3[kRows];
#pragma unroll
      for (int h = 0; h < kRows / 16; ++h) {
        tmem_ld16(tmem_base + lane_base + ab * 2 * kRows + h * 16, a1 + h * 16);
        if (DUAL) tmem_ld16(tmem_base + lane_base + ab * 2 * kRows + kRows + h * 16, a3 + h * 16);
      }
      tc::tmem_ld_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(acc_empty(ab));
      const int n = n0 + quad * 32 + lane;
#pragma unroll
      for (int c = 0; c < kRows; ++c) {
        const int r = __shfl_sync(0xffffffffu, orow, c);
        if (r < 0) continue;
        float o = __uint_as_float(a1[c]);
        if (DUAL == 1) {
          float gate = o, up = __uint_as_float(a3[c]);
          if (p.limit > 0.f) {
            gate = fminf(gate, p.limit);
            up = fminf(fmaxf(up, -p.limit), p.limit);
          }
          o = gate / (1.f + __expf(-gate)) * up;
          if (p.out) reinterpret_cast<__half*>(p.out)[(long)r * p.ldo + n] = __float2half(o);
          if (p.q_out) {
            // the warp's 32 features are one scale group of the next GEMV's input
            float amax = fabsf(o);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            int ex = -127;
            if (amax > 0.f) {
              int e2;
              const float m = frexpf(amax * (1.f / 448.f), &e2);
              ex = max(-127, min(127, (m == 0.5f) ? e2 - 1 : e2));
            }
            const float q = o * exp2f((float)-ex);
            p.q_out[(long)r * p.N + n] = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
            if (lane == 0) p.q_scale[(long)r * (p.N / 32) + n / 32] = (uint8_t)(ex + 127);
          }
        } else {
          reinterpret_cast<float*>(p.out)[(long)r * p.ldo + n] = o;
          if (DUAL == 2) reinterpret_cast<float*>(p.out)[(long)r * p.ldo + n + kTile] = __uint_as_float(a3[c]);
        }
      }
      return true;
    };
    int f = 0, n_item = 0, item = blockIdx.x, sc = 0, pend_item = -1, pend_n = 0;
    bool ok = true;
    while (item < items && ok) {
      int nitem = item, nsc = sc + 1;
      if (nsc == nsuper) {
        nitem += gridDim.x;
        nsc = 0;
      }
      const int sb = f % kSfBufs;
      const uint32_t par = (f / kSfBufs) & 1;
      if (!(ok = tc::mbar_wait(sfs_full(sb), par, abort_flag))) break;
      // rows lane, lane+32, lane+64, lane+96 of each matrix: 16 scale bytes = four 128-input words
      const uint8_t* sl = aligned + kStages * kStageBytes + sb * kSfsBytes;
      uint4 w[kMats][4];
#pragma unroll
      for (int m = 0; m < kMats; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          w[m][j] = *reinterpret_cast<const uint4*>(sl + m * kTile * 16 + (lane + 32 * j) * 16);
      const uint4 xa = *reinterpret_cast<const uint4*>(sl + kMats * kTile * 16 + (lane & (kRows - 1)) * 16);
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(sfs_empty(sb));
      if (!(ok = tc::mbar_wait(sf_empty(sb), par ^ 1, abort_flag))) break;
      tc::tc_fence_after();
#pragma unroll
      for (int m = 0; m < kMats; ++m) {
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[0 + j] = w[m][j].x;       // inputs   0..127 of this block: column j = rows 32j..32j+31
          v[4 + j] = w[m][j].y;       // inputs 128..255
          v[8 + j] = w[m][j].z;
          v[12 + j] = w[m][j].w;
        }
        tmem_st16(tmem_base + lane_base + kSfaCol + sb * 32 + m * 16, v);
      }
      {
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0;
        v[0] = xa.x; v[4] = xa.y; v[8] = xa.z; v[12] = xa.w;
        tmem_st16(tmem_base + lane_base + kSfbCol + sb * 16, v);
      }
      tmem_st_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(sf_full(sb));
      ++f;
      if (pend_item >= 0) {
        ok = epilogue(pend_item, pend_n);
        pend_item = -1;
      }
      if (sc == nsuper - 1) {
        pend_item = item;
        pend_n = n_item++;
      }
      item = nitem;
      sc = nsc;
    }
    if (ok && pend_item >= 0) epilogue(pend_item, pend_n);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) tf_report(p.status, TF_TIMEOUT, 130 + DUAL + (ROWS > 16 ? 4 : 0), blockIdx.x, items);
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// one thread per group of 32 inputs: e4m3 values and the UE8M0 scale 2^ceil(log2(amax / 448))
__global__ void quant_rows_mx8_kernel(const __half* __restrict__ x, int ldx, uint8_t* __restrict__ q,
                                      uint8_t* __restrict__ s, int rows, int K) {
  tf_pdl_sync();
  const int ks = K / 32;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * ks) return;
  const int r = i / ks, b = i % ks;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long)r * ldx + b * 32);
  uint4 v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = src[j];
  const __half2* h = reinterpret_cast<const __half2*>(v);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float2 f = __half22float2(h[j]);
    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  int ex = -127;
  if (amax > 0.f) {
    // smallest power of two >= amax / 448
    int e2;
    const float m = frexpf(amax * (1.f / 448.f), &e2);       // value = m * 2^e2, m in [0.5, 1)
    ex = (m == 0.5f) ? e2 - 1 : e2;
    ex = max(-127, min(127, ex));
  }
  const float inv = exp2f((float)-ex);
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f0 = __half22float2(h[2 * j]), f1 = __half22float2(h[2 * j + 1]);
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f0.x * inv, f0.y * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f1.x * inv, f1.y * inv), __NV_SATFINITE, __NV_E4M3);
    o[j] = lo | (hi << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(q + (long)r * K + b * 32);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  s[(long)r * ks + b] = (uint8_t)(ex + 127);
}

int g_mx_sms = 0;

inline bool make_map_fp4(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K) {
  auto fn = tc::encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 31) || ((K / 2) & 31) || (K & 127)) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K / 2};
  cuuint32_t box[2] = {128, (cuuint32_t)kTile};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// x [rows, K] f16 -> q [rows, K] e4m3 + s [rows, K/32] UE8M0
TF_API int tf_quant_rows_mx8(const void* x, int ldx, void* q, void* s, int rows, int K, cudaStream_t st) {
  if (K % 32 || ldx % 8 || rows <= 0) return -1;
  const int n = rows * (K / 32);
  tf_launch(quant_rows_mx8_kernel, dim3((n + 127) / 128), dim3(128), 0, st, reinterpret_cast<const __half*>(x), ldx,
                                                        reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(s),
                                                        rows, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Routed experts over the groups of tf_route_group.
//   w1 (and w3: fused clamped SwiGLU, f16 output rows in SORTED pair order) or w1 alone (f32 output
//   rows by pair index); weights [experts, N, K/2] packed e2m1, scales [experts, N, K/32] UE8M0.
//   q_out / q_scale (fused form, optional): the same output rows as MXFP8 [rows, N] + [rows, N/32],
//   ready to be the plain form's input; `out` may then be null.
//   x8 / sx: MXFP8 activation rows.  Fused form: the T token rows (T <= 32), one accumulator
//   column per token.  Plain form: rows in sorted pair order, the group's rows are consecutive;
//   x8 needs no padding rows (a box that runs past the last row reads zeros), sx is clamped.
//   group_rows: the most rows one group can hold (the token rows of the step; 0 = 16): above 16
//   the 32-column form of the kernel runs.
//   a_tx_bytes: bytes a [128 x 128] e2m1 box adds to the mbarrier's transaction count (0: the
//   packed size).  blocked: the weights are stored block by block ([128 rows x 128 inputs] = 8 KB
//   contiguous, blocks of one row tile consecutive) instead of row-major.
TF_API int tf_moe_gemv_mx(const void* w1, const void* w3, const void* s1, const void* s3, int experts,
                          const void* x8, const void* sx, int x_rows, void* out, int ldo, void* q_out,
                          void* q_scale, int N, int K, int topk,
                          const int* g_expert, const int* g_start, const int* g_count, const int* n_groups,
                          const int* sorted_pairs, int max_groups, float limit, int a_tx_bytes, int blocked,
                          int group_rows, void* status, cudaStream_t st) {
  if (N % kTile || K % kSuper || x_rows <= 0 || max_groups <= 0) return -1;
  const bool dual = w3 != nullptr;
  if (group_rows <= 0) group_rows = kRows;
  if (dual && x_rows > group_rows) group_rows = x_rows;
  if (group_rows > 32) return -1;
  const int rows = group_rows > kRows ? 32 : kRows;
  if (!g_mx_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_mx_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(moe_mx_kernel<0, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(moe_mx_kernel<1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(moe_mx_kernel<2, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(moe_mx_kernel<0, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(moe_mx_kernel<1, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(moe_mx_kernel<2, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  }
  CUtensorMap m1, m3, mx, ms1, ms3, msx;
  if (!tc::make_map_2d_plain(&ms1, s1, (uint64_t)experts * N, K / 32, K / 32, 16, kTile)) return -4;
  if (!tc::make_map_2d_plain(&ms3, dual ? s3 : s1, (uint64_t)experts * N, K / 32, K / 32, 16, kTile)) return -4;
  if (!tc::make_map_2d_plain(&msx, sx, x_rows, K / 32, K / 32, 16, rows)) return -4;
  // blocked: [experts * N/128 * K/128] blocks of [128 rows x 128 inputs], each 8 KB contiguous
  const uint64_t wrows = blocked ? (uint64_t)experts * N * (K / kBK) : (uint64_t)experts * N;
  const uint64_t wcols = blocked ? kBK : K;
  if (!make_map_fp4(&m1, w1, wrows, wcols)) return -4;
  if (!make_map_fp4(&m3, dual ? w3 : w1, wrows, wcols)) return -4;
  if (!tc::make_map_2d(&mx, x8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x_rows, K, K, rows)) return -4;
  MxParams p;
  p.g_expert = g_expert; p.g_start = g_start; p.g_count = g_count; p.n_groups = n_groups;
  p.sorted_pairs = sorted_pairs;
  p.sw1 = reinterpret_cast<const uint8_t*>(s1);
  p.sw3 = reinterpret_cast<const uint8_t*>(dual ? s3 : s1);
  p.sx = reinterpret_cast<const uint8_t*>(sx);
  p.out = out; p.ldo = ldo;
  p.q_out = reinterpret_cast<uint8_t*>(q_out);
  p.q_scale = reinterpret_cast<uint8_t*>(q_scale); p.N = N; p.K = K; p.topk = topk; p.x_rows = x_rows;
  p.a_tx_bytes = a_tx_bytes > 0 ? a_tx_bytes : kTile * kBK / 2;
  p.limit = limit;
  p.blocked = blocked;
  p.status = reinterpret_cast<TfStatusWord*>(status);
  const bool pair = !dual && N % (2 * kTile) == 0;         // plain form, two adjacent tiles per work item
  const int grid = min(g_mx_sms, max_groups * (N / (pair ? 2 * kTile : kTile)));
  const int stages = mx_stages(dual || pair, rows), mats = (dual || pair) ? 2 : 1;
  const int sfs = (mats * kTile * 16 + rows * 16 + 127) / 128 * 128;
  const int smem = stages * (mats * kTile * 128 + rows * 128) + kSfBufs * sfs + 1024 + 512;
  if (smem > 227 * 1024) return -3;
  const dim3 g(grid), t(kThreads);
  if (rows == kRows) {
    if (dual) tf_launch(moe_mx_kernel<1, 16>, g, t, smem, st, m1, m3, mx, ms1, ms3, msx, p);
    else if (pair) tf_launch(moe_mx_kernel<2, 16>, g, t, smem, st, m1, m3, mx, ms1, ms3, msx, p);
    else tf_launch(moe_mx_kernel<0, 16>, g, t, smem, st, m1, m3, mx, ms1, ms3, msx, p);
  } else {
    if (dual) tf_launch(moe_mx_kernel<1, 32>, g, t, smem, st, m1, m3, mx, ms1, ms3, msx, p);
    else if (pair) tf_launch(moe_mx_kernel<2, 32>, g, t, smem, st, m1, m3, mx, ms1, ms3, msx, p);
    else tf_launch(moe_mx_kernel<0, 32>, g, t, smem, st, m1, m3, mx, ms1, ms3, msx, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
