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

constexpr int BM = 128;
constexpr int kRingBytes = 6 * 32768;              // operand ring: 6 x 32 KB (BN 128) or 4 x 48 KB (BN 256)
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr int kStagingBytes = kEpiWarps * 4096;     // per-warp 32 x 128 B transpose buffers (reduce-scatter stores)
constexpr int kSmemBytes = kRingBytes + 1024 /*align*/ + 256 /*barriers*/ + kStagingBytes;
constexpr int kCopyPiece = 32768;                  // all-gather role: bytes per bulk copy
constexpr int kCopyDepth = 3;                      // loads issued ahead of their stores

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
  // all-gather form (sequence-parallel activations): A is row-sharded over the ranks.  The last
  // ag_copy_ctas CTAs pull every rank's shard (rows, then their block scales) from its workspace
  // into this GPU's gathered buffer with bulk copies, 128 rows at a time, and publish one flag per
  // 128-row block; the TMA producer of a GEMM CTA waits for the flag of the block it is about to
  // read.  Blocks are visited own shard first, then rank+1, rank+2, ...
  const unsigned long long* ag_peers;   // [world] workspace bases (null = A is local)
  int ag_world, ag_rank, ag_rows;       // ag_rows = M / world (multiple of 128)
  int ag_copy_ctas;
  int ag_row_bytes, ag_srow_bytes;      // bytes per row of A and of its scales (0 = none)
  long ag_shard_off;                    // this parity's shard area in every workspace
  long ag_gath_off;                     // gathered A, then gathered scales, in the own workspace
  long ag_flag_off;                     // [world] shard-ready words (peers write), then [M/128] block flags
  unsigned int ag_epoch;
  int spin_limit;
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// wait until *p >= want (wrap-safe); false after spin_limit polls or ~1 s
template <bool SYS>
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int want, int spin_limit) {
  const long long t0 = clock64();
  for (int spins = 0;; ++spins) {
    const unsigned int v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int)(v - want) >= 0) return true;
    if (spins > spin_limit || clock64() - t0 > 2000000000LL) return false;
  }
}

constexpr int kCopyStages = 6;
// The all-gather role of one CTA: a single thread drives a ring of kCopyStages 32 KB buffers; loads run
// kCopyDepth pieces ahead of the stores.
__device__ void ag_copy_role(const GemmParams& p, uint32_t base, uint32_t bar0, int cta, int n_ctas) {
  if (threadIdx.x != 0) return;
  unsigned int* flags = reinterpret_cast<unsigned int*>(p.ag_peers[p.ag_rank] + p.ag_flag_off);
  if (cta == 0) {
    // our shard was written by earlier work on this stream: tell every rank it may be read
    for (int r = 0; r < p.ag_world; ++r) {
      unsigned int* f = reinterpret_cast<unsigned int*>(p.ag_peers[r] + p.ag_flag_off) + p.ag_rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(p.ag_epoch) : "memory");
    }
  }
  for (int s = 0; s < kCopyStages; ++s) tc::mbar_init(bar0 + 8u * s, 1);
  tc::fence_barrier_init();
  volatile int abort_local = 0;
  const int tpr = p.ag_rows / BM;
  uint8_t* gath = reinterpret_cast<uint8_t*>(p.ag_peers[p.ag_rank] + p.ag_gath_off);
  uint8_t* gath_s = gath + (long)p.M * p.ag_row_bytes;
  long issued = 0, stored = 0;          // pieces over the whole kernel (ring position / parity)
  bool ok = true;
  for (int q = cta; q < p.ag_world * tpr && ok; q += n_ctas) {
    const int src = (p.ag_rank + q / tpr) % p.ag_world, blk = q % tpr;
    if (!wait_flag<true>(flags + src, p.ag_epoch, p.spin_limit)) {
      tf_report(p.status, TF_TIMEOUT, 120, src, q);
      break;
    }
    const uint8_t* shard = reinterpret_cast<const uint8_t*>(p.ag_peers[src] + p.ag_shard_off);
    // two segments: 128 rows of A, then their scale rows
    for (int seg = 0; seg < 2 && ok; ++seg) {
      const long seg_bytes = (long)BM * (seg == 0 ? p.ag_row_bytes : p.ag_srow_bytes);
      if (seg_bytes == 0) continue;
      const uint8_t* from = seg == 0 ? shard + (long)blk * seg_bytes
                                     : shard + (long)p.ag_rows * p.ag_row_bytes + (long)blk * seg_bytes;
      uint8_t* to = seg == 0 ? gath + ((long)src * p.ag_rows + (long)blk * BM) * p.ag_row_bytes
                             : gath_s + ((long)src * p.ag_rows + (long)blk * BM) * p.ag_srow_bytes;
      const int n = (int)((seg_bytes + kCopyPiece - 1) / kCopyPiece);
      for (int i = 0; i < n + kCopyDepth && ok; ++i) {
        if (i < n) {
          const int sl = (int)(issued % kCopyStages);
          // the store that last used this buffer is kCopyStages pieces back: at most
          // kCopyStages - kCopyDepth - 1 younger store groups may still be reading shared memory
          tc::bulk_wait_read<kCopyStages - kCopyDepth - 1>();
          const uint32_t bytes = (uint32_t)min((long)kCopyPiece, seg_bytes - (long)i * kCopyPiece);
          tc::mbar_expect_tx(bar0 + 8u * sl, bytes);
          tc::bulk_g2s(base + sl * kCopyPiece, from + (long)i * kCopyPiece, bytes, bar0 + 8u * sl);
          ++issued;
        }
        const int j = i - kCopyDepth;
        if (j >= 0) {
          const int sl = (int)(stored % kCopyStages);
          if (!(ok = tc::mbar_wait(bar0 + 8u * sl, (uint32_t)((stored / kCopyStages) & 1), &abort_local))) break;
          const uint32_t bytes = (uint32_t)min((long)kCopyPiece, seg_bytes - (long)j * kCopyPiece);
          tc::bulk_s2g(to + (long)j * kCopyPiece, base + sl * kCopyPiece, bytes);
          tc::bulk_commit();
          ++stored;
        }
      }
    }
    tc::bulk_wait_all<0>();
    if (!ok) {
      tf_report(p.status, TF_TIMEOUT, 121, src, q);
      break;
    }
    tc::fence_proxy_async_global();
    __threadfence();
    unsigned int* bf = flags + p.ag_world + (src * tpr + blk);
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bf), "r"(p.ag_epoch) : "memory");
  }
  tc::bulk_wait_all<0>();
}

template <int KIND, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const GemmParams p) {
  tf_pdl_sync();
  // BN = 128: six 32 KB stages, four TMEM buffers; BN = 256: four 48 KB stages, two TMEM buffers
  // (a third less operand traffic from L2 per FLOP)
  constexpr int kStages = (BN == 128) ? 6 : 4;
  constexpr int kStageBytes = (BM + BN) * 128;
  constexpr int kAccBufs = 512 / BN;
  constexpr int CH = BN / 2;                               // output columns per epilogue warp
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

  uint8_t* stage_out = aligned + kStages * kStageBytes + 256;                                        // [8][4096]

  const int n_copy = p.ag_peers ? p.ag_copy_ctas : 0;
  const int n_gemm = gridDim.x - n_copy;
  if ((int)blockIdx.x >= n_gemm) {
    ag_copy_role(p, base, bar0, blockIdx.x - n_gemm, n_copy);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int BK = (KIND == 0) ? 64 : 128;               // elements per 128-byte row
  const int kblocks = (p.K + BK - 1) / BK;
  const int mt = p.tile_expert ? *p.num_m_tiles : (p.M + BM - 1) / BM, nt = p.N / BN;
  const int tiles = mt * nt;
  // tile -> (row block, column block).  Plain: row blocks fastest (one weight panel stays hot in L2).
  // All-gather: column blocks fastest and row blocks in arrival order (own shard, rank+1, ...).
  const int ag_tpr = p.ag_peers ? p.ag_rows / BM : 1;
  auto tile_m = [&](int tile) {
    if (!p.ag_peers) return tile % mt;
    const int mi = tile / nt;
    return ((p.ag_rank + mi / ag_tpr) % p.ag_world) * ag_tpr + mi % ag_tpr;
  };
  auto tile_n = [&](int tile) { return p.ag_peers ? tile % nt : tile / mt; };

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
      const unsigned int* blk_flags =
          p.ag_peers ? reinterpret_cast<const unsigned int*>(p.ag_peers[p.ag_rank] + p.ag_flag_off) + p.ag_world
                     : nullptr;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += n_gemm) {
        const int m0 = tile_m(tile) * BM, n0 = tile_n(tile) * BN;
        const int nb0 = n0 + (p.tile_expert ? p.tile_expert[tile % mt] * p.N : 0);
        if (blk_flags) {
          // rows of this block arrive through the copy CTAs (bulk stores): wait, then order the
          // TMA reads after what the flag published
          if (!wait_flag<false>(blk_flags + m0 / BM, p.ag_epoch, p.spin_limit)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc::fence_proxy_async_global();
        }
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
      for (int tile = blockIdx.x; tile < tiles && ok; tile += n_gemm) {
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
    for (int tile = blockIdx.x; tile < tiles && ok; tile += n_gemm) {
      ++tile_iter;
      const int m0 = tile_m(tile) * BM, n0 = tile_n(tile) * BN;
      const int row = m0 + quad * 32 + lane;
      if (KIND == 2 && p.ag_peers) {
        // the scale rows of this block come with the gathered rows: wait for the block as well
        int good = 1;
        if (lane == 0) {
          const unsigned int* bf =
              reinterpret_cast<const unsigned int*>(p.ag_peers[p.ag_rank] + p.ag_flag_off) + p.ag_world + m0 / BM;
          good = wait_flag<false>(bf, p.ag_epoch, p.spin_limit) ? 1 : 0;
          if (!good) *abort_flag = 1;
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
      }
      float acc[CH];
      if (KIND == 2) {
#pragma unroll
        for (int i = 0; i < CH; ++i) acc[i] = 0.f;
      }
      const int groups = (KIND == 2) ? kblocks : 1;
      const float* sa_row = (KIND == 2 && row < p.M) ? p.sa + (long)row * p.ldsa : nullptr;
      const int nb0 = n0 + (p.tile_expert ? p.tile_expert[tile % mt] * p.N : 0);
      const float* sb_row = (KIND == 2) ? p.sb + (long)((nb0 + half * CH) >> 7) * p.ldsb : nullptr;
      float s_next = (KIND == 2) ? (sa_row ? sa_row[0] : 0.f) * sb_row[0] : 1.f;
      for (int g = 0; g < groups && ok; ++g, ++grp) {
        const int buf = grp % kAccBufs;
        const uint32_t gph = (grp / kAccBufs) & 1;
        const float s = s_next;
        if (KIND == 2 && g + 1 < groups) s_next = (sa_row ? sa_row[g + 1] : 0.f) * sb_row[g + 1];
        if (!(ok = tc::mbar_wait(tfull(buf), gph, abort_flag))) break;
        tc::tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + half * CH;
#pragma unroll
        for (int c = 0; c < CH; c += 64) {
          uint32_t v0[32], v1[32];
          tc::tmem_ld32(taddr + c, v0);
          tc::tmem_ld32(taddr + c + 32, v1);
          tc::tmem_ld_wait();
          if (c + 64 >= CH) {
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tempty(buf));
          }
          if (KIND == 2) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              acc[c + i] = fmaf(s, __uint_as_float(v0[i]), acc[c + i]);
              acc[c + 32 + i] = fmaf(s, __uint_as_float(v1[i]), acc[c + 32 + i]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              acc[c + i] = __uint_as_float(v0[i]);
              acc[c + 32 + i] = __uint_as_float(v1[i]);
            }
          }
        }
      }
      if (p.rs_peers) {
        // ---- GEMM -> reduce-scatter: push the tile to the rank that owns these rows
        const int owner = m0 / p.rs_rows;
        if (ok) {
          // transpose the warp's 32 x 64 bf16 block through its private shared-memory buffer so
          // that each store instruction covers four whole 128-byte row segments of the peer's
          // memory (16-byte chunks XOR-swizzled by row: conflict-free both ways)
          uint8_t* buf = stage_out + ew * 4096;
          __nv_bfloat16* recv = reinterpret_cast<__nv_bfloat16*>(p.rs_peers[owner] + p.rs_recv_off);
          const int rbase = m0 + quad * 32;
#pragma unroll
          for (int c = 0; c < CH; c += 64) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              __nv_bfloat162 h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                h[j] = __floats2bfloat162_rn(acc[c + 8 * i + 2 * j], acc[c + 8 * i + 2 * j + 1]);
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((i ^ (lane & 7)) << 4)) = *reinterpret_cast<uint4*>(h);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3), ch = lane & 7;
              const uint4 v = *reinterpret_cast<const uint4*>(buf + rr * 128 + ((ch ^ (rr & 7)) << 4));
              const int grow = rbase + rr;
              if (grow < p.M)
                *reinterpret_cast<uint4*>(recv + ((long)p.rs_rank * p.rs_rows + (grow - owner * p.rs_rows)) * p.N + n0 +
                                          half * CH + c + ch * 8) = v;
            }
            __syncwarp();
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
                                  ((m0 - owner * p.rs_rows) / BM) * (p.N / 128) + n0 / 128;
              for (int j = 0; j < BN / 128; ++j)      // the owner sums 128-column tiles
                asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt + j) : "memory");
            }
          }
        }
      } else if (ok && row < p.M) {
        const long off = (long)row * p.ldc + n0 + half * CH;
        if (p.out_kind == 0) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + off);
#pragma unroll
          for (int i = 0; i < CH / 4; ++i) dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + off);
#pragma unroll
          for (int i = 0; i < CH / 8; ++i) {
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
  if (*abort_flag && threadIdx.x == 0) tf_report(p.status, TF_TIMEOUT, 100 + KIND, blockIdx.x, BN);
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, kAccBufs * BN);
  }
}

int g_sms = 0;
int g_force_bn = 0;   // tests: 128 pins the small tile

struct RsConfig {
  const unsigned long long* peers = nullptr;
  int world = 0, rank = 0;
  long recv_off = 0, flag_off = 0;
} g_rs;   // set by tf_gemm_rs around the launch; plain calls leave it empty

struct AgConfig {
  const unsigned long long* peers = nullptr;
  int world = 0, rank = 0, copy_ctas = 0, spin_limit = 0;
  long shard_off = 0, gath_off = 0;
  unsigned int epoch = 0;
} g_ag;   // set by tf_gemm_ag around the launch

// sum the `world` received slots of every 128x128 tile in rank order once all of them arrived
__global__ void __launch_bounds__(256) rs_reduce_kernel(const unsigned long long* peers, int rank, int world,
                                                        int rows, int N, long recv_off, long flag_off,
                                                        unsigned int want, __nv_bfloat16* out, int ldo,
                                                        int spin_limit, TfStatusWord* st) {
  tf_pdl_sync();
  __shared__ int s_fail;
  const int nt = N / 128, tile = blockIdx.x, mt_i = tile / nt, nt_i = tile % nt;
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
  for (int i = threadIdx.x; i < BM * (128 / 8); i += blockDim.x) {
    const int r = mt_i * BM + i / (128 / 8), c = nt_i * 128 + (i % (128 / 8)) * 8;
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
  if (N % 128 != 0 || (kind == 0 ? K % 64 : K % 128) != 0) return -1;
  if (out_kind != 0 && out_kind != 2) return -1;
  if ((out_kind == 0 ? ldc % 4 : ldc % 8) != 0) return -1;
  if (kind == 2 && (!sa || !sb)) return -1;
  CUtensorMap ma, mb;
  const int es = kind == 0 ? 2 : 1;
  const CUtensorMapDataType dt = kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // 128x256 tiles once they still fill the machine; 128x128 otherwise
  const int BN = (N % 256 == 0 && (long)((M + BM - 1) / BM) * (N / 256) >= g_sms && g_force_bn != 128) ? 256 : 128;
  if (!tc::make_map_2d(&ma, A, dt, es, M, K, (uint64_t)lda * es, BM)) return -2;
  if (!tc::make_map_2d(&mb, B, dt, es, (uint64_t)N * (experts > 0 ? experts : 1), K, (uint64_t)ldb * es, BN)) return -2;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.kind = kind; p.sa = sa; p.ldsa = ldsa; p.sb = sb; p.ldsb = ldsb;
  p.C = C; p.ldc = ldc; p.out_kind = out_kind; p.status = (TfStatusWord*)status;
  p.tile_expert = experts > 0 ? tile_expert : nullptr; p.num_m_tiles = num_m_tiles;
  p.rs_peers = g_rs.peers; p.rs_world = g_rs.world; p.rs_rank = g_rs.rank; p.rs_rows = g_rs.world ? M / g_rs.world : 0;
  p.rs_recv_off = g_rs.recv_off; p.rs_flag_off = g_rs.flag_off;
  if (p.rs_peers && (M % (g_rs.world * BM) != 0)) return -1;
  p.ag_peers = g_ag.peers; p.ag_world = g_ag.world; p.ag_rank = g_ag.rank; p.ag_rows = g_ag.world ? M / g_ag.world : 0;
  p.ag_copy_ctas = g_ag.copy_ctas; p.ag_row_bytes = K * es; p.ag_srow_bytes = kind == 2 ? (K / 128) * 4 : 0;
  p.ag_shard_off = g_ag.shard_off; p.ag_gath_off = g_ag.gath_off; p.ag_flag_off = 0; p.ag_epoch = g_ag.epoch;
  p.spin_limit = g_ag.spin_limit;
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  int grid = tiles < g_sms ? tiles : g_sms;
  if (p.ag_peers) {
    if (M % (g_ag.world * BM) != 0 || experts > 0 || g_ag.copy_ctas < 1 || g_ag.copy_ctas >= g_sms) return -1;
    const int gemm_ctas = g_sms - g_ag.copy_ctas;
    grid = (tiles < gemm_ctas ? tiles : gemm_ctas) + g_ag.copy_ctas;   // every CTA is resident: one per SM
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_tc_kernel<0, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<1, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<2, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<0, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<1, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaFuncSetAttribute(gemm_tc_kernel<2, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    attr_set = true;
  }
  if (BN == 128) {
    if (kind == 0) tf_launch(gemm_tc_kernel<0, 128>, dim3(grid), dim3(kThreads), kSmemBytes, stream, ma, mb, p);
    else if (kind == 1) tf_launch(gemm_tc_kernel<1, 128>, dim3(grid), dim3(kThreads), kSmemBytes, stream, ma, mb, p);
    else tf_launch(gemm_tc_kernel<2, 128>, dim3(grid), dim3(kThreads), kSmemBytes, stream, ma, mb, p);
  } else {
    if (kind == 0) tf_launch(gemm_tc_kernel<0, 256>, dim3(grid), dim3(kThreads), kSmemBytes, stream, ma, mb, p);
    else if (kind == 1) tf_launch(gemm_tc_kernel<1, 256>, dim3(grid), dim3(kThreads), kSmemBytes, stream, ma, mb, p);
    else tf_launch(gemm_tc_kernel<2, 256>, dim3(grid), dim3(kThreads), kSmemBytes, stream, ma, mb, p);
  }
  return (int)cudaGetLastError();
}

// bytes of the symmetric workspace of the GEMM -> reduce-scatter form: two receive areas (epoch
// parity) of [world][M/world][N] bf16 plus the arrival counters
TF_API long tf_gemm_rs_flag_bytes(int M, int N, int world) {
  return ((long)(M / world / BM) * (N / 128) * 4 + 255) / 256 * 256;
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
  if (world < 1 || M % (world * BM) != 0 || N % 128 != 0 || (ldo % 8) != 0) return -1;
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
  const int tiles = (rows / BM) * (N / 128);
  tf_launch(rs_reduce_kernel, dim3(tiles), dim3(256), 0, stream, (const unsigned long long*)peers, rank, world, rows, N, recv_off, 0,
                                              (unsigned int)epoch * (unsigned int)world, (__nv_bfloat16*)out, ldo,
                                              spin_limit, (TfStatusWord*)status);
  return (int)cudaGetLastError();
}

// ---- all-gather -> GEMM.  Workspace (symmetric, same layout on every rank):
//   [0, 4096)            flags: [world] shard-ready words, then [M/128] block flags
//   two shard areas      (epoch parity) of M/world rows of A followed by their scale rows
//   gathered A [M rows], gathered scales [M rows]
static long ag_shard_bytes(int kind, int M, int K, int world) {
  const long es = kind == 0 ? 2 : 1;
  return ((long)(M / world) * (K * es + (kind == 2 ? (K / 128) * 4 : 0)) + 255) / 256 * 256;
}
TF_API long tf_gemm_ag_shard_offset(int kind, int M, int K, int world, int epoch) {
  return 4096 + (long)(epoch & 1) * ag_shard_bytes(kind, M, K, world);
}
TF_API long tf_gemm_ag_workspace_bytes(int kind, int M, int K, int world) {
  const long es = kind == 0 ? 2 : 1;
  return 4096 + 2 * ag_shard_bytes(kind, M, K, world) + (long)M * (K * es + (kind == 2 ? (K / 128) * 4 : 0)) + 256;
}

// C[M, N] = allgather_rows(A_shards)[M, K] * B[N, K]^T with B, C local.  The caller has written its
// M/world rows of A (and, for kind 2, their [rows, K/128] fp32 scales right behind them) at
// tf_gemm_ag_shard_offset(..., epoch) of its own workspace before this call on the same stream.
// `epoch` counts calls on this workspace (1, 2, ...).  M/128 must not exceed 1024 - world.
TF_API int tf_gemm_ag(int kind, const void* B, long ldb, void* C, int ldc, int M, int N, int K, const float* sb,
                      int ldsb, int out_kind, const void* peers, const void* own_base, int world, int rank,
                      int epoch, int copy_ctas, int spin_limit, void* status, cudaStream_t stream) {
  if (world < 1 || M % (world * BM) != 0 || M / BM + world > 1024 || kind == 1) return -1;
  const long es = kind == 0 ? 2 : 1;
  g_ag.peers = (const unsigned long long*)peers; g_ag.world = world; g_ag.rank = rank; g_ag.copy_ctas = copy_ctas;
  g_ag.spin_limit = spin_limit; g_ag.epoch = (unsigned int)epoch;
  g_ag.shard_off = tf_gemm_ag_shard_offset(kind, M, K, world, epoch);
  g_ag.gath_off = 4096 + 2 * ag_shard_bytes(kind, M, K, world);
  const uint8_t* gath = reinterpret_cast<const uint8_t*>(own_base) + g_ag.gath_off;
  const float* sa = kind == 2 ? reinterpret_cast<const float*>(gath + (long)M * K * es) : nullptr;
  const int rc = tf_gemm_tc(kind, gath, K, B, ldb, C, ldc, M, N, K, sa, K / 128, sb, ldsb, out_kind, nullptr, nullptr,
                            0, status, stream);
  g_ag = AgConfig();
  return rc;
}

// tests / benchmarks: 128 pins the 128x128 tile, 0 restores the automatic choice
TF_API int tf_gemm_tc_force_tile(int bn) {
  g_force_bn = bn;
  return 0;
}
