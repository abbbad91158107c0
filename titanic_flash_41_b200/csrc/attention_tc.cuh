// Sparse attention of prefill rows on the tcgen05 tensor cores (head dim 128, up to 64 heads, one
// split).  Included by attention.cu inside its anonymous namespace (AttnParams, kNegBig).
//
// A persistent CTA takes one query row at a time.  All heads of the row read the same latent keys,
// so the heads are the M of both contractions and a chunk of 128 gathered keys is N of the first and
// K of the second:
//
//   S[head, key]  = Q[head, :] . K[key, :]        A = Q [128 x 128 dims]   B = key tile, K-major
//   O[head, dim] += P[head, key] * K[key, dim]     A = P [ 64 x 128 keys]   B = the same tile, MN-major
//
// Operands are f16 in shared memory with the 128-byte swizzle (two 64-column sub-tiles each): a latent
// value times its scale is exact in f16 (FP4 rows: five mantissa bits at most, FP8 rows: four), and
// Q is bf16 converted once per row.  S (two buffers) and O (two buffers, alternating rows) live in
// tensor memory.  Q's 64 head rows are stored twice, so accumulator lanes 64..127 of S repeat lanes
// 0..63 and a softmax thread owns one lane and HALF of the chunk's key columns.
//
//   warps 0-7   gather: two threads per key of the chunk (64 dims each) fetch its FP8 window row or
//               FP4 compressed row (the next chunk's bytes are requested before this chunk is
//               converted; ids are decoded a chunk after they are loaded) and write it as a row of the
//               key tile; three tiles in flight
//   warps 8-11  softmax: base-2 online softmax with a stale reference maximum (O is rescaled, and
//               the previous PV waited for, only when a score exceeds it by 2^8), P as f16 into
//               shared memory (two buffers); the two threads of a head meet at a named barrier of
//               their warp pair; warps 8-9 finish the row: sink as an extra zero-valued logit, inverse
//               rotation of the tail, f16 / bf16 output
//   warp 12     one thread issues the MMAs: QK of chunk c + 1 before PV of chunk c
// Every mbarrier wait is bounded; on a time-out the CTA raises its abort flag, reports TF_TIMEOUT,
// frees its tensor memory and returns (softmax warps stop waiting but keep walking their named
// barriers, so no warp is left behind at one).
//
// Output: the finished rows, i.e. what the mma.sync kernel and attn_merge_kernel produce together with
// one split.
#pragma once
#include "tc.cuh"

constexpr int kTcKeys = 128;
constexpr int kTcProd = 8;                           // gather warps: two threads per key row (64 dims each)
constexpr int kTcThreads = (kTcProd + 5) * 32;      // gather warps, 4 softmax warps, 1 MMA warp
constexpr int kTcSub = 16384;                       // one [128 rows x 128 B] sub-tile
constexpr int kTcQSub = 16384;                      // Q: rows 0..63 the heads, rows 64..127 the heads again; two buffers
constexpr int kTcPSub = 8192;                       // P: 64 rows (the heads); two buffers
constexpr int kTcStage = 2 * kTcSub;                // the key tile: two 64-dim sub-tiles of [128 keys x 128 B]
constexpr int kTcStages = 3;                        // key tiles in flight (the gather runs ahead of the MMAs)
constexpr int kTcSmem = 4 * kTcQSub /*Q x2*/ + 4 * kTcPSub /*P x2*/ + kTcStages * kTcStage + 1024 + 2048;

// byte offset of (row, byte column) inside a 128-byte-swizzled sub-tile
__device__ __forceinline__ uint32_t sw128(int row, int colb) {
  return (uint32_t)(row * 128 + ((((colb >> 4) ^ (row & 7)) << 4) | (colb & 15)));
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t v[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
// MN-major operand (the contiguous direction is M / N, here the 128 dims of a key row) in the same
// 128-byte-swizzled tile of 128-byte rows: 8 k-rows form a 1,024-byte group (stride offset), the
// second 64 columns live one sub-tile further (leading offset)
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(kTcSub >> 4) << 16;              // leading byte offset: next 64 columns
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset: next 8 k-rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void tmem_st_wait_tc() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ int attn_row_keys(const AttnParams& p, int r, int* nwin_out) {
  const int pos = p.pos[r];
  const int nwin = min(pos + 1 - (p.min_pos ? p.min_pos[r] : 0), p.window);
  int nsel = 0;
  if (p.comp) {
    if (p.sel_count) nsel = p.sel_count[r];
    else {
      int lo = 0, hi = p.sel_stride;
      const int* s = p.sel + (long)r * p.sel_stride;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s[mid] >= 0) lo = mid + 1; else hi = mid;
      }
      nsel = lo;
    }
  }
  *nwin_out = nwin;
  return nwin + nsel;
}

__global__ void __launch_bounds__(kTcThreads, 1) sparse_attn_tc_kernel(AttnParams p) {
  tf_pdl_sync();
  constexpr int DH = 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw0 = tc::smem_u32(smem_raw);
  const uint32_t base = (raw0 + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw0);
  // Q: two buffers of two 128-row sub-tiles; rows 64..127 repeat the heads, so accumulator lanes
  // 64..127 of S hold the same scores and a second pair of softmax warps can take half the columns.
  // P: two buffers of two 64-row sub-tiles.  The PV MMA reads 128 rows of A: rows 64..127 of a P
  // sub-tile alias the shared memory behind it (finite or not, they only reach accumulator lanes
  // 64..127 of O, which nobody reads).
  constexpr int kQBytes = 4 * kTcQSub, kOpBytes = kQBytes + 4 * kTcPSub;
  const uint32_t q_s = base, p_s = base + kQBytes, st_s = base + kOpBytes;
  uint8_t* q_g = aligned;
  uint8_t* p_g = aligned + kQBytes;
  uint8_t* st_g = aligned + kOpBytes;
  const uint32_t bar0 = base + kOpBytes + kTcStages * kTcStage;
  auto full = [&](int s) { return bar0 + 8u * s; };              // gather -> MMA            (4 warps)
  auto empty = [&](int s) { return bar0 + 8u * (4 + s); };       // PV done: stage free        (commit)
  auto s_ready = [&](int b) { return bar0 + 8u * (8 + b); };     // QK done                    (commit)
  auto s_free = [&](int b) { return bar0 + 8u * (10 + b); };     // softmax has read S         (2 warps)
  const uint32_t p_ready = bar0 + 8u * 12;                       // P written, O rescaled      (2 warps)
  const uint32_t o_ready = bar0 + 8u * 13;                       // PV done                    (commit)
  auto o_free = [&](int b) { return bar0 + 8u * (21 + b); };     // softmax has read O[b]      (2 warps)
  auto q_ready = [&](int b) { return bar0 + 8u * (15 + b); };    // Q buffer written           (4 warps)
  auto q_free = [&](int b) { return bar0 + 8u * (17 + b); };     // the row's QK MMAs are done (commit)
  auto p_free = [&](int b) { return bar0 + 8u * (19 + b); };     // the PV that read P[b] is done (commit)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + kOpBytes + kTcStages * kTcStage + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + kOpBytes + kTcStages * kTcStage + 200);
  float* xch = reinterpret_cast<float*>(aligned + kOpBytes + kTcStages * kTcStage + 256);      // [3][128] softmax exchange

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      tc::mbar_init(full(s), kTcProd);
      tc::mbar_init(empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      tc::mbar_init(s_ready(s), 1);
      tc::mbar_init(s_free(s), 4);
      tc::mbar_init(q_ready(s), kTcProd);
      tc::mbar_init(q_free(s), 1);
      tc::mbar_init(p_free(s), 1);
      tc::mbar_init(o_free(s), 2);
    }
    tc::mbar_init(p_ready, 4);
    tc::mbar_init(o_ready, 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  // Q and P start as zeros: rows 64..127 of P (no heads there) stay zero for the whole launch
  for (int i = threadIdx.x; i < kOpBytes / 16; i += kTcThreads)
    reinterpret_cast<uint4*>(q_g)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (warp == kTcProd + 4) tc::tmem_alloc(tc::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128u};
  const uint32_t tOb[2] = {tmem_base + 256u, tmem_base + 384u};     // O of even / odd rows of this CTA

  if (warp < kTcProd) {
    // ------------------------------------------------------------------ gather + convert
    const int tid = threadIdx.x & 127;              // key of the chunk served by this thread ...
    const int hh = threadIdx.x >> 7;                // ... and which 64 of its 128 dims
    uint4 rawv[4];
    uint32_t rsc[1];
    int it = 0, n_row = 0;
    bool ok = true;
    for (int r = blockIdx.x; r < p.T && ok; r += gridDim.x, ++n_row) {
      int nwin;
      const int nkeys = attn_row_keys(p, r, &nwin);
      const int nchunks = (nkeys + kTcKeys - 1) / kTcKeys;
      const int pos = p.pos[r], reg = p.region[r];
      const uint8_t* win = p.win + (long)reg * p.win_region_stride;
      const uint8_t* comp = p.comp ? p.comp + (long)reg * p.comp_region_stride : nullptr;
      // A key is (kind, value): kind 0 = padding, 1 = window ring slot, 2 = compressed entry id.  The
      // id is only looked at when its row is fetched, a chunk later: nothing waits for the id load.
      auto key_kind = [&](int c) -> int {
        const int i = c * kTcKeys + tid;
        return (c >= nchunks || i >= nkeys) ? 0 : (i < nwin ? 1 : 2);
      };
      auto key_val = [&](int c, int kind) -> int {
        const int i = c * kTcKeys + tid;
        if (kind == 1) return (pos - nwin + 1 + i) % p.ring;
        if (kind == 2) return p.sel[(long)r * p.sel_stride + (i - nwin)];
        return 0;
      };
      auto load_raw = [&](int kind, int val) {
        if (kind == 1) {
          const uint8_t* row = win + (long)val * p.win_row;
#pragma unroll
          for (int j = 0; j < 4; ++j) rawv[j] = *reinterpret_cast<const uint4*>(row + hh * 64 + j * 16);
          rsc[0] = *reinterpret_cast<const uint32_t*>(row + DH) >> (16 * hh);       // the half's two scale bytes
        } else if (kind == 2) {
          int id = val;
          if (id < 0 || id >= p.maxC) {
            tf_report(p.st, TF_BAD_INDEX, 11, r, id);
            id = 0;
          }
          const uint8_t* row = comp + (long)id * p.comp_row;
#pragma unroll
          for (int j = 0; j < 2; ++j) rawv[j] = *reinterpret_cast<const uint4*>(row + hh * 32 + j * 16);
          rsc[0] = *reinterpret_cast<const uint32_t*>(row + DH / 2 + hh * 4);       // the half's four scale bytes
        }
      };
      int kind_cur = key_kind(0), kind_next = key_kind(1);
      int val_cur = key_val(0, kind_cur), val_next = key_val(1, kind_next);
      load_raw(kind_cur, val_cur);
      // Q of this row into buffer n_row & 1: free once the QK MMAs of the row before last are done
      const int qb = n_row & 1;
      if (!(ok = tc::mbar_wait(q_free(qb), ((n_row >> 1) & 1) ^ 1, abort_flag))) break;
      {
        // 64 heads x 128 dims bf16 = 1,024 16-byte pieces over 128 threads
        const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + (long)r * p.Hl * DH);
#pragma unroll
        for (int j = 0; j < 1024 / (kTcProd * 32); ++j) {
          const int piece = (int)threadIdx.x + kTcProd * 32 * j;
          const int h = piece >> 4, c16 = piece & 15;           // 16 pieces per head row
          uint4 v = h < p.Hl ? qsrc[piece] : make_uint4(0u, 0u, 0u, 0u);
          uint32_t* vw = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int e = 0; e < 4; ++e) {                          // bf16 pair -> f16 pair (exact in range)
            const float2 f2 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&vw[e]));
            vw[e] = pack_h2(f2.x, f2.y);
          }
          uint8_t* qsub = q_g + (qb * 2 + (c16 >> 3)) * kTcQSub;
          *reinterpret_cast<uint4*>(qsub + sw128(h, (c16 & 7) * 16)) = v;
          *reinterpret_cast<uint4*>(qsub + sw128(h + 64, (c16 & 7) * 16)) = v;
        }
        tc::fence_proxy_async();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(q_ready(qb));
      }
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int s = it % kTcStages;
        if (!(ok = tc::mbar_wait(empty(s), ((it / kTcStages) & 1) ^ 1, abort_flag))) break;
        uint8_t* kt = st_g + s * kTcStage;
        // The key row as f16 (what a latent value times its scale is exactly: at most five mantissa
        // bits for FP4 rows, four for FP8 rows), sixteen values = one 32-byte piece at a time.  One
        // branch per row kind, not per piece: the FP4 body (all but the window rows) stays small.
        auto put = [&](int seg, const uint32_t (&hv)[8]) {          // seg: 16-value piece of this thread's half
          const int d0 = hh * 64 + seg * 16;
          uint8_t* ksub = kt + (d0 >> 6) * kTcSub;
          *reinterpret_cast<uint4*>(ksub + sw128(tid, (d0 & 63) * 2)) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
          *reinterpret_cast<uint4*>(ksub + sw128(tid, (d0 & 63) * 2 + 16)) = make_uint4(hv[4], hv[5], hv[6], hv[7]);
        };
        if (kind_cur == 0) {
          const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
          for (int seg = 0; seg < 4; ++seg) put(seg, z);
        } else if (kind_cur == 1) {
#pragma unroll
          for (int seg = 0; seg < 4; ++seg) {
            uint32_t hv[8];
            const float sc = ue8m0_to_float((rsc[0] >> (8 * (seg >> 1))) & 0xffu);
            const uint16_t* h = reinterpret_cast<const uint16_t*>(&rawv[seg]);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              uint32_t h2 = e4m3x2_to_h2(h[q]);
              const float2 v = __half22float2(*reinterpret_cast<__half2*>(&h2));
              hv[q] = pack_h2(v.x * sc, v.y * sc);
            }
            put(seg, hv);
          }
        } else {
          // the unpacked halves hold value * 2^-14; two packed f16 multiplies (by 2^14, exact, then by
          // the group's e4m3 scale, exact) instead of a trip through fp32 and back
          const __half2 k14 = __floats2half2_rn(16384.f, 16384.f);
#pragma unroll
          for (int seg = 0; seg < 4; ++seg) {
            uint32_t hv[8];
            const uint32_t sb = (rsc[0] >> (8 * seg)) & 0xffu;
            const uint32_t sh = e4m3x2_to_h2((uint16_t)(sb | (sb << 8)));
            const __half2 sc2 = *reinterpret_cast<const __half2*>(&sh);
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&rawv[seg >> 1]) + 2 * (seg & 1);
            e2m1x8_to_h2x4_scaled(w[0], hv);
            e2m1x8_to_h2x4_scaled(w[1], hv + 4);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const __half2 x = __hmul2(__hmul2(*reinterpret_cast<__half2*>(&hv[q]), k14), sc2);
              hv[q] = *reinterpret_cast<const uint32_t*>(&x);
            }
            put(seg, hv);
          }
        }
        // request the next chunk's rows and the ids of the chunk after it, then hand the stage over
        kind_cur = kind_next;
        val_cur = val_next;
        load_raw(kind_cur, val_cur);
        kind_next = key_kind(c + 2);
        val_next = key_val(c + 2, kind_next);
        tc::fence_proxy_async();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(full(s));
      }
    }
  } else if (warp == kTcProd + 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc(0, 0, 128, 128);      // f16 x f16, M 128, N 128, both K-major
      constexpr uint32_t idesc_pv = idesc | (1u << 16);               // B (the key tile as V) MN-major
      int it = 0, n_row = 0;
      bool ok = true;
      auto qk = [&](int i, int qb) -> bool {                         // S[i & 1] = Q[qb] . Kt(stage i & 1)^T
        const int s = i & 1, stg = i % kTcStages;
        if (!tc::mbar_wait(full(stg), (i / kTcStages) & 1, abort_flag)) return false;
        if (!tc::mbar_wait(s_free(s), ((i >> 1) & 1) ^ 1, abort_flag)) return false;
        tc::tc_fence_after();
        const uint32_t kt = st_s + stg * kTcStage;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc::mma_f16(tS[s], tc::smem_desc_sw128(q_s + (qb * 2 + j) * kTcQSub) + 2 * k,
                        tc::smem_desc_sw128(kt + j * kTcSub) + 2 * k, idesc, (j | k) ? 1u : 0u);
        tc::mma_commit(s_ready(s));
        return true;
      };
      for (int r = blockIdx.x; r < p.T && ok; r += gridDim.x, ++n_row) {
        int nwin;
        const int nkeys = attn_row_keys(p, r, &nwin);
        const int nchunks = (nkeys + kTcKeys - 1) / kTcKeys;
        const int qb = n_row & 1;
        if (!(ok = tc::mbar_wait(q_ready(qb), (n_row >> 1) & 1, abort_flag))) break;
        if (!(ok = qk(it, qb))) break;
        if (nchunks == 1) tc::mma_commit(q_free(qb));
        for (int c = 0; c < nchunks; ++c, ++it) {
          if (c + 1 < nchunks) {
            if (!(ok = qk(it + 1, qb))) break;
            if (c + 2 == nchunks) tc::mma_commit(q_free(qb));      // the row's last QK is issued
          }
          if (!(ok = tc::mbar_wait(p_ready, it & 1, abort_flag))) break;
          // the first PV of a row overwrites O[n_row & 1]: the result of the row before last must have been read
          if (c == 0 && !(ok = tc::mbar_wait(o_free(n_row & 1), ((n_row >> 1) & 1) ^ 1, abort_flag))) break;
          tc::tc_fence_after();
          // B = the same key tile read MN-major (dims contiguous): 16 keys per step = 2,048 bytes
          const uint32_t kt = st_s + (it % kTcStages) * kTcStage;
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc::mma_f16(tOb[n_row & 1], tc::smem_desc_sw128(p_s + ((it & 1) * 2 + j) * kTcPSub) + 2 * k, smem_desc_sw128_mn(kt) + 128u * (4 * j + k),
                          idesc_pv, (c | j | k) ? 1u : 0u);
          tc::mma_commit(empty(it % kTcStages));
          tc::mma_commit(p_free(it & 1));
          tc::mma_commit(o_ready);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax
    // Thread L of the four warps reads accumulator lane L: head L % 64, key columns 64 (L / 64) ..
    // + 63 of the chunk (lanes 64..127 of S repeat lanes 0..63).  The two threads of a head share
    // the reference maximum (chunk maxima and the row sum meet in shared memory under a named
    // barrier of the 128 softmax threads); only the first two warps touch O.
    const int L = (warp - kTcProd) * 32 + lane;
    const int h = L & 63, half = L >> 6;
    const uint32_t lane_off = (uint32_t)((warp - kTcProd) * 32) << 16;
    const uint32_t col0 = (uint32_t)half * 64u;
    // (the two warps that share a set of heads meet at a named barrier of their own, 64 threads)
    const int pair_bar = 1 + ((warp - kTcProd) & 1);
    auto sm_bar = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
    // A wait that runs out raises the CTA's abort flag.  The warp then stops waiting but keeps walking
    // the same sequence of named barriers as its partner (nobody is left behind at a barrier); the
    // results of such a launch are void and the status word says so.
    bool fail = false;
    auto wait = [&](uint32_t bar, uint32_t parity) {
      if (!fail && !tc::mbar_wait(bar, parity, abort_flag)) fail = true;
    };
    int it = 0, n_row = 0;
    for (int r = blockIdx.x; r < p.T; r += gridDim.x, ++n_row) {
      int nwin;
      const int nkeys = attn_row_keys(p, r, &nwin);
      const int nchunks = (nkeys + kTcKeys - 1) / kTcKeys;
      float m = kNegBig, l = 0.f;
      const uint32_t tO = tOb[n_row & 1];
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int sb = it & 1;
        const int valid = nkeys - c * kTcKeys - (int)col0;           // own columns >= valid are padding
        float* xc = xch + (it & 1) * 128;
        wait(s_ready(sb), (it >> 1) & 1);
        tc::tc_fence_after();
        // The reference maximum m is the first chunk's; it moves only when some head finds a score
        // more than 2^8 above it (then O is rescaled, which has to wait for the PV before, and the
        // chunk is exponentiated again).  Until then exp2(s - m) <= 256 is harmless in f16 / fp32,
        // the ratio O / l does not depend on m, and one short loop over the thread's two pieces of 32
        // scores does everything (small code: the instruction cache, not the arithmetic, was the limit).
        if (c == 0) {
          float cm = kNegBig;
#pragma unroll 1
          for (int q = 0; q < 2; ++q) {
            uint32_t v[32];
            tc::tmem_ld32(tS[sb] + lane_off + col0 + q * 32, v);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (q * 32 + i < valid) cm = fmaxf(cm, __uint_as_float(v[i]));
          }
          xch[256 + L] = cm;
          sm_bar();
          m = fmaxf(cm, xch[256 + (L ^ 64)]) * p.scale_log2;
        }
        // the PV that read this P buffer two chunks ago is done
        wait(p_free(it & 1), ((it >> 1) & 1) ^ 1);
        bool again = false;
        do {
          float cm = kNegBig, ls = 0.f;
          uint8_t* psub = p_g + ((it & 1) * 2 + half) * kTcPSub;     // keys 64 half .. of this chunk
#pragma unroll 1
          for (int q = 0; q < 2; ++q) {
            uint32_t v[32];
            tc::tmem_ld32(tS[sb] + lane_off + col0 + q * 32, v);
            tc::tmem_ld_wait();
            uint32_t pk[16];
            if (valid >= 64) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float x0 = __uint_as_float(v[2 * i]), x1 = __uint_as_float(v[2 * i + 1]);
                cm = fmaxf(cm, fmaxf(x0, x1));
                const float a = exp2f(fmaf(x0, p.scale_log2, -m)), b = exp2f(fmaf(x1, p.scale_log2, -m));
                ls += a + b;
                pk[i] = pack_h2(a, b);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const bool in0 = q * 32 + 2 * i < valid, in1 = q * 32 + 2 * i + 1 < valid;
                const float x0 = in0 ? __uint_as_float(v[2 * i]) : kNegBig, x1 = in1 ? __uint_as_float(v[2 * i + 1]) : kNegBig;
                cm = fmaxf(cm, fmaxf(x0, x1));
                const float a = in0 ? exp2f(fmaf(x0, p.scale_log2, -m)) : 0.f;
                const float b = in1 ? exp2f(fmaf(x1, p.scale_log2, -m)) : 0.f;
                ls += a + b;
                pk[i] = pack_h2(a, b);
              }
            }
            // 32 keys = 64 bytes = four 16-byte pieces of row h
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(psub + sw128(h, q * 64 + i * 16)) =
                  make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
          // both threads of a head must take the same decision: exchange the chunk maxima
          xc[L] = cm;
          sm_bar();
          cm = fmaxf(cm, xc[L ^ 64]) * p.scale_log2;
          again = __any_sync(0xffffffffu, cm > m + 8.f);
          if (!again) {
            l += ls;
          } else {
            // rare: move the maximum, rescale O and l, exponentiate the chunk again
            const float nm = fmaxf(m, cm);
            const float f = exp2f(m - nm);
            m = nm;
            l *= f;
            if (c > 0 && half == 0) {
              wait(o_ready, (it & 1) ^ 1);
              tc::tc_fence_after();
#pragma unroll 1
              for (int q = 0; q < 4; ++q) {
                uint32_t o[32];
                tc::tmem_ld32(tO + lane_off + q * 32, o);
                tc::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                tmem_st32(tO + lane_off + q * 32, o);
              }
              tmem_st_wait_tc();
            }
            sm_bar();                                             // (the exchange slots are written again)
          }
        } while (again);
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(s_free(sb));
        tc::fence_proxy_async();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(p_ready);
      }
      // ---- the row's result: both halves' sums, then the first two warps wait for the last PV,
      // normalise and write the partial
      float* xr = xch + 256;
      sm_bar();                                                   // (first-chunk maxima have been read)
      xr[L] = l;
      sm_bar();
      l += xr[L ^ 64];
      if (half == 0) {
        wait(o_ready, (it & 1) ^ 1);
        tc::tc_fence_after();
        // The sink is one more logit with a zero value: the row is scaled by w / (w + w_sink) as the
        // split merge would.  Then the inverse rotation of the tail (the value shares the key's rotated
        // latent) and the f16 / bf16 row.  Lane j holds the sine and cosine of pair j of the tail.
        float scale_o = 0.f;
        if (l > 0.f) {
          const float lse = m + log2f(l);
          const float s2 = p.sink ? p.sink[min(h, p.Hl - 1)] * 1.4426950408889634f : kNegBig;
          const float mx = fmaxf(s2, lse);
          const float w = exp2f(lse - mx);
          scale_o = w / (w + (p.sink ? exp2f(s2 - mx) : 0.f)) / l;
        }
        float sn = 0.f, cs = 1.f;
        if (lane < p.rope_dim / 2) {
          const float ang = (float)p.pos[r] * p.freqs[lane];
          const double two_pi = 6.283185307179586476925286766559;
          sincosf((float)((double)ang - two_pi * floor((double)ang / two_pi)), &sn, &cs);
        }
        const int tail0 = DH - p.rope_dim;
        const long orow = (long)r * p.ldo + (long)h * DH;
#pragma unroll 1
        for (int q = 0; q < 4; ++q) {
          uint32_t v[32];
          tc::tmem_ld32(tO + lane_off + q * 32, v);
          tc::tmem_ld_wait();
          float o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]) * scale_o;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int d = q * 32 + i;
            const int j = (d - tail0) >> 1;                       // pair of the tail (uniform over the warp)
            const float sj = __shfl_sync(0xffffffffu, sn, j & 31), cj = __shfl_sync(0xffffffffu, cs, j & 31);
            if (d >= tail0) {
              const float a = o[i], b2 = o[i + 1];
              o[i] = a * cj + b2 * sj;                            // inverse rotation: angle -> -angle
              o[i + 1] = -a * sj + b2 * cj;
            }
          }
          if (h < p.Hl) {
            if (p.out16) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(p.out16 + orow + q * 32 + 8 * i) =
                    make_uint4(pack_h2(o[8 * i], o[8 * i + 1]), pack_h2(o[8 * i + 2], o[8 * i + 3]),
                               pack_h2(o[8 * i + 4], o[8 * i + 5]), pack_h2(o[8 * i + 6], o[8 * i + 7]));
            }
            if (p.outb) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(p.outb + orow + q * 32 + 8 * i) =
                    make_uint4(pack_bf2(o[8 * i], o[8 * i + 1]), pack_bf2(o[8 * i + 2], o[8 * i + 3]),
                               pack_bf2(o[8 * i + 4], o[8 * i + 5]), pack_bf2(o[8 * i + 6], o[8 * i + 7]));
            }
          }
        }
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(o_free(n_row & 1));
      }
      sm_bar();                                                   // the sums have been read before the next row writes them
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) tf_report(p.st, TF_TIMEOUT, 150, blockIdx.x, 0);
  if (warp == kTcProd + 4) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 512);
  }
}
