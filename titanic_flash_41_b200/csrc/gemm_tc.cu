// Tensor-core GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (both operands K-major)
//
//   kind 0  bf16 x bf16            tcgen05.mma kind::f16
//   kind 1  e4m3 x e4m3            tcgen05.mma kind::f8f6f4, unscaled
//   kind 2  e4m3 x e4m3 block-scaled: A carries one fp32 scale per (row, 128 k), B one per
//           (128 rows, 128 k).  Each 128-deep K block is accumulated by the tensor core into its
//           own TMEM buffer and promoted into fp32 registers with the product of the two scales
//           by the epilogue warps (software promotion; four TMEM buffers keep the MMA pipe fed
//           while earlier blocks are being promoted).
//
// One persistent CTA per SM walks 128x128 output tiles.  Warp 0 issues TMA loads (tensor maps over
// this GPU's memory, 128-byte swizzle, no multicast) into a 6-stage shared-memory ring; one
// elected thread of warp 1 issues tcgen05.mma with accumulators in tensor memory; warps 2-9 drain
// TMEM with tcgen05.ld (two warps per 32-lane quadrant, 64 columns each), scale, convert and
// store.  Every wait is bounded: on a time-out the CTA raises its abort flag, records TF_TIMEOUT
// in the status word, lets copies in flight land, frees its TMEM and returns.
//
// Replaces for the B200 build: the b12x `gemm.dense` / FlashInfer MXFP8 bundles and the cuBLAS
// GemmEx calls of the reference (src/fp8_linear.rs:122, src/blas.rs:24).
#include "tc.cuh"

namespace {

constexpr int BM = 128, BN = 128;
constexpr int kStages = 6;
constexpr int kStageBytes = (BM + BN) * 128;       // rows of 128 bytes
constexpr int kAccBufs = 4;                        // TMEM accumulator buffers of BN columns
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;

struct GemmParams {
  int M, N, K;
  int kind;                 // 0 bf16, 1 fp8, 2 fp8 block-scaled
  const float* sa;          // [M, K/128]
  int ldsa;
  const float* sb;          // [N/128, K/128]
  int ldsb;
  void* C;
  int ldc;
  int out_kind;             // 0 f32, 2 bf16
  TfStatusWord* status;
  // grouped form (routed experts): A rows are expert-sorted in 128-row padded segments; M tile i
  // belongs to expert tile_expert[i] whose weights are rows [e*N, (e+1)*N) of B
  const int* tile_expert;
  const int* num_m_tiles;
  // reduce-scatter form (tensor-parallel partial products): the bf16 tile of rows owned by rank o
  // is stored straight into rank o's receive slot for this rank over NVLink and the tile's
  // arrival counter on rank o is bumped; tf_rs_reduce on rank o sums the `world` slots.
  const unsigned long long* rs_peers;   // [world] workspace bases (null = plain store)
  int rs_world, rs_rank, rs_rows;       // rs_rows = M / world (multiple of 128)
  long rs_recv_off;                     // byte offset of this parity's receive area in a workspace
  long rs_flag_off;                     // byte offset of the arrival counters
};

template <int KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;            // swizzled tiles need 1024-byte alignment
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t bar0 = base + kStages * kStageBytes;      // full[kStages], empty[kStages], tfull[4], tempty[4]
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto tempty = [&](int b) { return bar0 + 8u * (2 * kStages + kAccBufs + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + kStages * kStageBytes + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + kStages * kStageBytes + 208);
  unsigned int* rs_done = reinterpret_cast<unsigned int*>(aligned + kStages * kStageBytes + 216);   // [8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int BK = (KIND == 0) ? 64 : 128;               // elements per 128-byte row
  const int kblocks = (p.K + BK - 1) / BK;
  const int mt = p.tile_expert ? *p.num_m_tiles : (p.M + BM - 1) / BM, nt = p.N / BN;
  const int tiles = mt * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(full(s), 1);
      tc::mbar_init(empty(s), 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      tc::mbar_init(tfull(b), 1);
      tc::mbar_init(tempty(b), kEpiWarps / 2 * 0 + kEpiWarps);
    }
    *abort_flag = 0;
    for (int i = 0; i < 8; ++i) rs_done[i] = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tc::smem_u32(const_cast<uint32_t*>(tmem_slot)), kAccBufs * BN);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc::prefetch_tmap(&mapA);
      tc::prefetch_tmap(&mapB);
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
        const int nb0 = n0 + (p.tile_expert ? p.tile_expert[tile % mt] * p.N : 0);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = tc::mbar_wait(empty(s), ph ^ 1, abort_flag))) break;
          tc::mbar_expect_tx(full(s), kStageBytes);
          const uint32_t sa = base + s * kStageBytes;
          tc::tma_load_2d(sa, &mapA, kb * BK, m0, full(s));
          tc::tma_load_2d(sa + BM * 128, &mapB, kb * BK, nb0, full(s));
        }
      }
      if (!ok) {
        // let copies in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (KIND == 0) ? tc::instr_desc(1, 1, BM, BN) : tc::instr_desc(0, 0, BM, BN);
      int it = 0, grp = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const bool grp_start = (KIND == 2) || kb == 0;
          const bool grp_end = (KIND == 2) || kb == kblocks - 1;
          const int buf = grp % kAccBufs;
          if (grp_start) {
            const uint32_t gph = (grp / kAccBufs) & 1;
            if (!(ok = tc::mbar_wait(tempty(buf), gph ^ 1, abort_flag))) break;
          }
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = tc::mbar_wait(full(s), ph, abort_flag))) break;
          tc::tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint64_t da = tc::smem_desc_sw128(sa), db = tc::smem_desc_sw128(sa + BM * 128);
          const uint32_t td = tmem_base + buf * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t acc = (grp_start && k == 0) ? 0u : 1u;
            if (KIND == 0) tc::mma_f16(td, da + 2 * k, db + 2 * k, idesc, acc);
            else tc::mma_f8(td, da + 2 * k, db + 2 * k, idesc, acc);
          }
          tc::mma_commit(empty(s));
          if (grp_end) {
            tc::mma_commit(tfull(buf));
            ++grp;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int ew = warp - 2;
    const int quad = warp & 3;                 // TMEM lanes this warp may touch: [32*quad, 32*quad+32)
    const int half = ew >> 2;                  // which 64 of the tile's 128 columns
    int grp = 0, tile_iter = -1;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      ++tile_iter;
      const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
      const int row = m0 + quad * 32 + lane;
      float acc[64];
      if (KIND == 2) {
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      }
      const int groups = (KIND == 2) ? kblocks : 1;
      const float* sa_row = (KIND == 2 && row < p.M) ? p.sa + (long)row * p.ldsa : nullptr;
      const int nb0 = n0 + (p.tile_expert ? p.tile_expert[tile % mt] * p.N : 0);
      const float* sb_row = (KIND == 2) ? p.sb + (long)(nb0 >> 7) * p.ldsb : nullptr;
      float s_next = (KIND == 2) ? (sa_row ? sa_row[0] : 0.f) * sb_row[0] : 1.f;
      for (int g = 0; g < groups && ok; ++g, ++grp) {
        const int buf = grp % kAccBufs;
        const uint32_t gph = (grp / kAccBufs) & 1;
        const float s = s_next;
        if (KIND == 2 && g + 1 < groups) s_next = (sa_row ? sa_row[g + 1] : 0.f) * sb_row[g + 1];
        if (!(ok = tc::mbar_wait(tfull(buf), gph, abort_flag))) break;
        tc::tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + half * 64;
        uint32_t v0[32], v1[32];
        tc::tmem_ld32(taddr, v0);
        tc::tmem_ld32(taddr + 32, v1);
        tc::tmem_ld_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(tempty(buf));
        if (KIND == 2) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            acc[i] = fmaf(s, __uint_as_float(v0[i]), acc[i]);
            acc[32 + i] = fmaf(s, __uint_as_float(v1[i]), acc[32 + i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            acc[i] = __uint_as_float(v0[i]);
            acc[32 + i] = __uint_as_float(v1[i]);
          }
        }
      }
      if (p.rs_peers) {
        // ---- GEMM -> reduce-scatter: push the tile to the rank that owns these rows
        const int owner = m0 / p.rs_rows;
        if (ok && row < p.M) {
          __nv_bfloat16* recv = reinterpret_cast<__nv_bfloat16*>(p.rs_peers[owner] + p.rs_recv_off);
          uint4* dst = reinterpret_cast<uint4*>(
              recv + ((long)p.rs_rank * p.rs_rows + (row - owner * p.rs_rows)) * p.N + n0 + half * 64);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[8 * i + 2 * j], acc[8 * i + 2 * j + 1]);
            dst[i] = *reinterpret_cast<uint4*>(h);
          }
        }
        __threadfence_system();
        // the last of the eight epilogue warps to finish this tile publishes it (no blocking barrier:
        // a warp that gave up on a time-out must not strand the others)
        __syncwarp();
        if (lane == 0) {
          unsigned int* done = rs_done + (tile_iter & 7);
          if (atomicAdd(done, 1u) == kEpiWarps - 1) {
            *done = 0;
            __threadfence_system();
            if (ok) {
              unsigned int* cnt = reinterpret_cast<unsigned int*>(p.rs_peers[owner] + p.rs_flag_off) +
                                  ((m0 - owner * p.rs_rows) / BM) * (p.N / BN) + n0 / BN;
              asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
            }
          }
        }
      } else if (ok && row < p.M) {
        const long off = (long)row * p.ldc + n0 + half * 64;
        if (p.out_kind == 0) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + off);
#pragma unroll
          for (int i = 0; i < 16; ++i) dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + off);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[8 * i + 2 * j], acc[8 * i + 2 * j + 1]);
            dst[i] = *reinterpret_cast<uint4*>(h);
          }
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) tf_report(p.status, TF_TIMEOUT, 100 + KIND, blockIdx.x, 0);
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, kAccBufs * BN);
  }
}

int g_sms = 0;

struct RsConfig {
  const unsigned long long* peers = nullptr;
  int world = 0, rank = 0;
  long recv_off = 0, flag_off = 0;
} g_rs;   // set by tf_gemm_rs around the launch; plain calls leave it empty

// sum the `world` received slots of every 128x128 tile in rank order once all of them arrived
__global__ void __launch_bounds__(256) rs_reduce_kernel(const unsigned long long* peers, int rank, int world,
                                                        int rows, int N, long recv_off, long flag_off,
                                                        unsigned int want, __nv_bfloat16* out, int ldo,
                                                        int spin_limit, TfStatusWord* st) {
  __shared__ int s_fail;
  const int nt = N / BN, tile = blockIdx.x, mt_i = tile / nt, nt_i = tile % nt;
  const unsigned int* cnt = reinterpret_cast<const unsigned int*>(peers[rank] + flag_off) + tile;
  if (threadIdx.x == 0) {
    s_fail = 0;
    int spins = 0;
    const long long t0 = clock64();
    unsigned int v;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
      if ((int)(v - want) >= 0) break;
      if (++spins > spin_limit || clock64() - t0 > 4000000000LL) {
        tf_report(st, TF_TIMEOUT, 110, tile, (int)v);
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (s_fail) return;
  const __nv_bfloat16* recv = reinterpret_cast<const __nv_bfloat16*>(peers[rank] + recv_off);
  // 128 x 128 tile: 256 threads x (8 columns x 8 rows-strided)
  for (int i = threadIdx.x; i < BM * (BN / 8); i += blockDim.x) {
    const int r = mt_i * BM + i / (BN / 8), c = nt_i * BN + (i % (BN / 8)) * 8;
    if (r >= rows) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int src = 0; src < world; ++src) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(recv + ((long)src * rows + r) * N + c));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    __nv_bfloat162 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + (long)r * ldo + c) = *reinterpret_cast<uint4*>(o);
  }
}

}  // namespace

// kind 0: A,B bf16; kind 1/2: A,B e4m3 (2 = block scales sa [M,K/128], sb [N/128,K/128]).
// lda/ldb in elements, ldc in elements.  N must be a multiple of 128, K of 128 (64 for bf16).
// Grouped form: `experts` > 0, B holds experts*N rows, M is the capacity of the padded A matrix,
// tile_expert/num_m_tiles come from tf_moe_plan.
TF_API int tf_gemm_tc(int kind, const void* A, long lda, const void* B, long ldb, void* C, int ldc, int M,
                      int N, int K, const float* sa, int ldsa, const float* sb, int ldsb, int out_kind,
                      const int* tile_expert, const int* num_m_tiles, int experts, void* status,
                      cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N % BN != 0 || (kind == 0 ? K % 64 : K % 128) != 0) return -1;
  if (out_kind != 0 && out_kind != 2) return -1;
  if ((out_kind == 0 ? ldc % 4 : ldc % 8) != 0) return -1;
  if (kind == 2 && (!sa || !sb)) return -1;
  CUtensorMap ma, mb;
  const int es = kind == 0 ? 2 : 1;
  const CUtensorMapDataType dt = kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (!tc::make_map_2d(&ma, A, dt, es, M, K, (uint64_t)lda * es, BM)) return -2;
  if (!tc::make_map_2d(&mb, B, dt, es, (uint64_t)N * (experts > 0 ? experts : 1), K, (uint64_t)ldb * es, BN)) return -2;
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.kind = kind; p.sa = sa; p.ldsa = ldsa; p.sb = sb; p.ldsb = ldsb;
  p.C = C; p.ldc = ldc; p.out_kind = out_kind; p.status = (TfStatusWord*)status;
  p.tile_expert = experts > 0 ? tile_expert : nullptr; p.num_m_tiles = num_m_tiles;
  p.rs_peers = g_rs.peers; p.rs_world = g_rs.world; p.rs_rank = g_rs.rank; p.rs_rows = g_rs.world ? M / g_rs.world : 0;
  p.rs_recv_off = g_rs.recv_off; p.rs_flag_off = g_rs.flag_off;
  if (p.rs_peers && (M % (g_rs.world * BM) != 0)) return -1;
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  const int grid = tiles < g_sms ? tiles : g_sms;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    attr_set = true;
  }
  if (kind == 0) gemm_tc_kernel<0><<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, p);
  else if (kind == 1) gemm_tc_kernel<1><<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, p);
  else gemm_tc_kernel<2><<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

// bytes of the symmetric workspace of the GEMM -> reduce-scatter form: two receive areas (epoch
// parity) of [world][M/world][N] bf16 plus the arrival counters
TF_API long tf_gemm_rs_flag_bytes(int M, int N, int world) {
  return ((long)(M / world / BM) * (N / BN) * 4 + 255) / 256 * 256;
}
TF_API long tf_gemm_rs_workspace_bytes(int M, int N, int world) {
  return tf_gemm_rs_flag_bytes(M, N, world) + 2L * M * N * 2;
}

// C_rank[M/world, N] = sum over ranks of (A_r[M, K] * B_r[N, K]^T)[rows of this rank].
// One tcgen05 GEMM whose epilogue stores every tile into its owner's memory while the next tile is
// being multiplied, followed by the owner-side rank-ordered sum.  `epoch` counts calls on this
// workspace (1, 2, ...): arrival counters are monotonic and receive areas alternate by parity.
TF_API int tf_gemm_rs(int kind, const void* A, long lda, const void* B, long ldb, int M, int N, int K,
                      const float* sa, int ldsa, const float* sb, int ldsb, const void* peers, int world,
                      int rank, int epoch, void* out, int ldo, int spin_limit, void* status, cudaStream_t stream) {
  if (world < 1 || M % (world * BM) != 0 || N % BN != 0 || (ldo % 8) != 0) return -1;
  const long flag_bytes = tf_gemm_rs_flag_bytes(M, N, world);
  g_rs.peers = (const unsigned long long*)peers; g_rs.world = world; g_rs.rank = rank;
  g_rs.flag_off = 0;
  g_rs.recv_off = flag_bytes + (long)(epoch & 1) * M * N * 2;
  const int rc = tf_gemm_tc(kind, A, lda, B, ldb, nullptr, N, M, N, K, sa, ldsa, sb, ldsb, 2, nullptr, nullptr, 0,
                            status, stream);
  const long recv_off = g_rs.recv_off;
  g_rs = RsConfig();
  if (rc != 0) return rc;
  const int rows = M / world;
  const int tiles = (rows / BM) * (N / BN);
  rs_reduce_kernel<<<tiles, 256, 0, stream>>>((const unsigned long long*)peers, rank, world, rows, N, recv_off, 0,
                                              (unsigned int)epoch * (unsigned int)world, (__nv_bfloat16*)out, ldo,
                                              spin_limit, (TfStatusWord*)status);
  return (int)cudaGetLastError();
}
