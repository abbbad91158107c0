// One-shot all-reduce over NVLink peer memory, used as the epilogue of the producing kernel.
//
// Every rank runs the same kernel with the same grid.  CTA j owns columns [32j, 32j+32) of a
// [rows, N] fp32 partial.  It (1) stores its tile into the receive buffer of EVERY rank (plain
// peer stores through NVSwitch), (2) publishes the tile with a release store of its epoch number
// to a flag word on every rank, (3) waits -- with a bound -- for the same tile from every rank,
// (4) sums the `world` partials in rank order in fp32, so all ranks hold bit-identical results,
// and (5) applies the epilogue (residual update).  No CPU proxy, no second launch, no NCCL.
// This is the B200 counterpart of the reference's fused one-shot all-reduce + boundary epilogue
// (kernels/roce_oneshot_hc.cuh:27-77, kernels/roce_oneshot_twin.cuh:95-167).
//
// Symmetric workspace layout (same offsets on every rank; base addresses of all ranks in `peers`):
//   [0, flag_bytes)          flags   uint32 [world src][tiles]        epoch last published
//   [flag_bytes, ...)        recv    float  [2 parity][world src][max_rows][N]
// Receive slots alternate by epoch parity; a rank can run at most one epoch ahead of the slowest
// rank because finishing epoch e needs every rank's tile of epoch e, which a rank only sends after
// it has finished reading epoch e-1.
//
// A wait that runs out records TF_TIMEOUT (kernel id 200, detail = (peer, tile)) in the status
// word and the CTA returns without touching the residual: no trap, no endless spin.
#pragma once
#include "common.cuh"

struct CommParams {
  const unsigned long long* peers;   // [world] base address of every rank's workspace (device array)
  int world, rank;
  int tiles;                         // N / 32
  int max_rows;
  int N;
  unsigned int* epoch;               // [tiles] local counters (plain device memory)
  long flag_bytes;
  int spin_limit;
  TfStatusWord* st;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// tile: this CTA's partial values, tile[r * 32 + c] for r < rows (shared memory, fp32).
// On return (true) tile[] holds the rank-ordered sum.  Must be called by every thread of the CTA.
__device__ __forceinline__ bool comm_allreduce_tile(const CommParams& c, float* tile, int rows, int j) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  if (threadIdx.x == 0) {
    s_epoch = ++c.epoch[j];
    s_fail = 0;
  }
  __syncthreads();
  const unsigned int e = s_epoch;
  const int par = e & 1;
  const int n0 = j * 32;
  // (1) push the tile to every rank (own rank included)
  for (int i = threadIdx.x; i < c.world * rows * 8; i += blockDim.x) {
    const int peer = i / (rows * 8), rem = i % (rows * 8), r = rem >> 3, q = rem & 7;
    float* recv = reinterpret_cast<float*>(c.peers[peer] + c.flag_bytes);
    float4* dst = reinterpret_cast<float4*>(recv + ((long)(par * c.world + c.rank) * c.max_rows + r) * c.N + n0) + q;
    *dst = *reinterpret_cast<const float4*>(tile + r * 32 + q * 4);
  }
  __threadfence_system();
  __syncthreads();
  // (2) publish
  if (threadIdx.x < c.world) {
    unsigned int* flags = reinterpret_cast<unsigned int*>(c.peers[threadIdx.x]);
    st_release_sys(flags + c.rank * c.tiles + j, e);
  }
  // (3) bounded wait for every rank's tile
  if (threadIdx.x < c.world) {
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(c.peers[c.rank]) + threadIdx.x * c.tiles + j;
    int spins = 0;
    const long long t0 = clock64();
    // epochs only grow; (int) difference handles wrap-around.  The wait gives up after spin_limit
    // polls or about one second of SM clocks, whichever comes first.
    while ((int)(ld_acquire_sys(mine) - e) < 0) {
      if (++spins > c.spin_limit || clock64() - t0 > 2000000000LL) {
        tf_report(c.st, TF_TIMEOUT, 200, threadIdx.x, j);
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (s_fail) return false;
  // (4) rank-ordered fp32 sum (L1 bypassed: the slots are rewritten by peers every other epoch)
  const float* recv = reinterpret_cast<const float*>(c.peers[c.rank] + c.flag_bytes);
  for (int i = threadIdx.x; i < rows * 8; i += blockDim.x) {
    const int r = i >> 3, q = i & 7;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int src = 0; src < c.world; ++src) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(
                                  recv + ((long)(par * c.world + src) * c.max_rows + r) * c.N + n0) + q);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    *reinterpret_cast<float4*>(tile + r * 32 + q * 4) = acc;
  }
  __syncthreads();
  return true;
}

// residual update shared by the fused kernels: x[r, n0 + c] = bf16(x + tile)
__device__ __forceinline__ void comm_residual_update(__nv_bfloat16* x, int ldx, float* out, int ldo,
                                                     const float* tile, int rows, int j) {
  const int n0 = j * 32;
  for (int i = threadIdx.x; i < rows * 32; i += blockDim.x) {
    const int r = i >> 5, cc = i & 31;
    const float v = tile[i];
    if (out) out[(long)r * ldo + n0 + cc] = v;
    if (x) {
      __nv_bfloat16* px = x + (long)r * ldx + n0 + cc;
      *px = __float2bfloat16(bf16_round(__bfloat162float(*px) + v));
    }
  }
}
