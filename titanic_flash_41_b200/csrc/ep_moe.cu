// Expert-parallel MoE over NVLink peer memory: token-sharded ranks, experts split whole across ranks.
//
//   dispatch  every rank quantises its token rows to FP8 (one fp32 scale per 128 values) and stores
//             each (token, chosen expert) pair -- row, scales, (expert, source pair index) -- straight
//             into the receive area that the expert's rank keeps for this source.  Slots inside a
//             (source, destination) area come from a local counter; when the last CTA has finished,
//             the counts and an epoch flag are published to every destination (release, system scope).
//   receive   the destination waits (bounded) for all sources' flags, turns the received metadata
//             into the id list that the grouped-GEMM planner understands, and gathers the rows
//             into the expert-sorted, 128-row padded matrix the tcgen05 grouped GEMM reads.
//   return    expert outputs go back with plain peer stores into the source's combine buffer,
//             indexed by the source's own pair number; a flag per destination rank follows.
//   combine   the source waits for every rank's flag and sums its k rows per token in slot order
//             with the router weights (fixed order: run-to-run identical), plus the shared expert.
//
// No NCCL call, no host synchronisation and no atomics across NVLink: every cross-GPU access is a
// plain store or an acquire load of a flag.  Flags carry the call's epoch, so nothing is cleared
// between calls.  Every wait gives up after `spin_limit` polls or ~1 s and records TF_TIMEOUT.
//
// The reference has no expert parallelism (its experts are column-sliced over 4 ranks and the
// "transport" is an all-gather of quantised rows: src/ffn.rs:789-878, src/moe_transport.rs); this
// is the B200 replacement for that transport.
#include "comm.cuh"

namespace {

struct EpParams {
  const unsigned long long* peers;   // [world] workspace bases
  int world, rank;
  int cap;                           // rows a source may send to one destination
  int d, k, El;
  long off_meta, off_s, off_x, off_ret;
  unsigned int epoch;
  int spin_limit;
  TfStatusWord* st;
};

// control block at offset 0 of every workspace (uint32 words)
constexpr int kMaxWorld = 16;
constexpr int kWalkCtas = 148 * 8;               // grid of the kernels that walk received entries
constexpr int W_DISP_FLAG = 0;                 // [world] written by sources
constexpr int W_DISP_CNT = kMaxWorld;          // [world] written by sources
constexpr int W_RET_FLAG = 2 * kMaxWorld;      // [world] written by destinations
constexpr int W_SEND_CNT = 3 * kMaxWorld;      // [world] local slot counters
constexpr int W_DONE = 4 * kMaxWorld;          // [2] local last-CTA counters

__device__ __forceinline__ unsigned int* ctrl(const EpParams& p, int r) {
  return reinterpret_cast<unsigned int*>(p.peers[r]);
}
__device__ __forceinline__ bool wait_epoch(const unsigned int* f, unsigned int want, int spin_limit) {
  const long long t0 = clock64();
  for (int spins = 0;; ++spins) {
    if ((int)(ld_acquire_sys(f) - want) >= 0) return true;
    if (spins > spin_limit || clock64() - t0 > 2000000000LL) return false;
  }
}

// one CTA (256 threads) per local token
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpParams p, const __nv_bfloat16* __restrict__ x, long ldx,
                                                          const int* __restrict__ ids, int Tl) {
  tf_pdl_sync();
  extern __shared__ uint8_t sm[];
  uint8_t* q = sm;                                         // [d]
  float* sc = reinterpret_cast<float*>(sm + p.d);          // [d / 128]
  __shared__ int s_slot[16], s_dst[16];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool live = t < Tl;                                // a rank without tokens launches one idle CTA
  const __nv_bfloat16* row = x + (long)t * ldx;
  for (int b = warp; live && b < p.d / 128; b += 8) {
    const uint2 raw = *reinterpret_cast<const uint2*>(row + b * 128 + lane * 4);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), c = __bfloat1622float2(h[1]);
    float m = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y)));
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float s = fmaxf(m, 1e-12f) / 448.f, inv = 1.f / s;
    const uint32_t pk = (uint32_t)float_to_e4m3(a.x * inv) | ((uint32_t)float_to_e4m3(a.y * inv) << 8) |
                        ((uint32_t)float_to_e4m3(c.x * inv) << 16) | ((uint32_t)float_to_e4m3(c.y * inv) << 24);
    *reinterpret_cast<uint32_t*>(q + b * 128 + lane * 4) = pk;
    if (lane == 0) sc[b] = s;
  }
  unsigned int* mine = ctrl(p, p.rank);
  if (threadIdx.x < p.k) s_dst[threadIdx.x] = -1;
  if (live && threadIdx.x < p.k) {
    const int e = ids[t * p.k + threadIdx.x];
    const int dst = (e >= 0 && e < p.El * p.world) ? e / p.El : -1;
    s_dst[threadIdx.x] = dst;
    s_slot[threadIdx.x] = dst >= 0 ? (int)atomicAdd(mine + W_SEND_CNT + dst, 1u) : -1;
  }
  __syncthreads();
  for (int j = 0; j < p.k; ++j) {
    const int dst = s_dst[j], slot = s_slot[j];
    if (dst < 0) continue;
    if (slot >= p.cap) {
      if (threadIdx.x == 0) tf_report(p.st, TF_BAD_INDEX, 300, dst, slot);
      continue;
    }
    const long entry = (long)p.rank * p.cap + slot;
    uint8_t* base = reinterpret_cast<uint8_t*>(p.peers[dst]);
    uint4* dx = reinterpret_cast<uint4*>(base + p.off_x + entry * p.d);
    for (int i = threadIdx.x; i < p.d / 16; i += 256) dx[i] = reinterpret_cast<const uint4*>(q)[i];
    uint4* ds = reinterpret_cast<uint4*>(base + p.off_s + entry * (p.d / 128) * 4);
    if (threadIdx.x < p.d / 512) ds[threadIdx.x] = reinterpret_cast<const uint4*>(sc)[threadIdx.x];
    if (threadIdx.x == 0)
      *reinterpret_cast<int2*>(base + p.off_meta + entry * 8) = make_int2(ids[t * p.k + j], t * p.k + j);
  }
  // last CTA publishes the counts
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(mine + W_DONE, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x < p.world) {
    __threadfence();
    const int r = threadIdx.x;
    const unsigned int cnt = atomicExch(mine + W_SEND_CNT + r, 0u);
    unsigned int* theirs = ctrl(p, r);
    theirs[W_DISP_CNT + p.rank] = cnt < (unsigned)p.cap ? cnt : (unsigned)p.cap;
    st_release_sys(theirs + W_DISP_FLAG + p.rank, p.epoch);
    if (r == 0) mine[W_DONE] = 0;
  }
}

// ids_out[src * cap + i] = expert id of entry i from source src, -1 beyond what arrived
__global__ void __launch_bounds__(256) ep_recv_ids_kernel(EpParams p, int* __restrict__ ids_out) {
  tf_pdl_sync();
  __shared__ int s_cnt[kMaxWorld];
  __shared__ int s_fail;
  unsigned int* mine = ctrl(p, p.rank);
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!wait_epoch(mine + W_DISP_FLAG + threadIdx.x, p.epoch, p.spin_limit)) {
      tf_report(p.st, TF_TIMEOUT, 301, threadIdx.x, blockIdx.x);
      s_fail = 1;
      s_cnt[threadIdx.x] = 0;
    } else {
      s_cnt[threadIdx.x] = (int)mine[W_DISP_CNT + threadIdx.x];
    }
  }
  __syncthreads();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)p.world * p.cap) return;
  const int src = (int)(i / p.cap), slot = (int)(i % p.cap);
  int e = -1;
  if (!s_fail && slot < s_cnt[src])
    e = reinterpret_cast<const int2*>(reinterpret_cast<const uint8_t*>(p.peers[p.rank]) + p.off_meta)[i].x;
  ids_out[i] = e;
}

// rows that arrived -> their place in the expert-sorted padded matrix.  A fixed grid walks only
// the entries that arrived (counts were published with the dispatch flags, which the receive
// kernel of this call has already waited for).
__global__ void __launch_bounds__(256) ep_gather_kernel(EpParams p, const int* __restrict__ pair_dst,
                                                        uint8_t* __restrict__ xp, float* __restrict__ xps) {
  tf_pdl_sync();
  const unsigned int* mine = ctrl(p, p.rank);
  const uint8_t* base = reinterpret_cast<const uint8_t*>(p.peers[p.rank]);
  for (int src = 0; src < p.world; ++src) {
    const int cnt = (int)mine[W_DISP_CNT + src];
    for (int slot = blockIdx.x; slot < cnt; slot += gridDim.x) {
      const long i = (long)src * p.cap + slot;
      const int dst = pair_dst[i];
      if (dst < 0) continue;
      const uint4* sx = reinterpret_cast<const uint4*>(base + p.off_x + i * p.d);
      uint4* dx = reinterpret_cast<uint4*>(xp + (long)dst * p.d);
      for (int j = threadIdx.x; j < p.d / 16; j += 256) dx[j] = sx[j];
      const float* ss = reinterpret_cast<const float*>(base + p.off_s + i * (p.d / 128) * 4);
      if (threadIdx.x < p.d / 128) xps[(long)dst * (p.d / 128) + threadIdx.x] = ss[threadIdx.x];
    }
  }
}

// expert outputs back to the rank that owns the token
__global__ void __launch_bounds__(256) ep_return_kernel(EpParams p, const int* __restrict__ pair_dst,
                                                        const __nv_bfloat16* __restrict__ y, long ldy) {
  tf_pdl_sync();
  unsigned int* mine = ctrl(p, p.rank);
  for (int src = 0; src < p.world; ++src) {
    const int cnt = (int)mine[W_DISP_CNT + src];
    for (int slot = blockIdx.x; slot < cnt; slot += gridDim.x) {
      const long i = (long)src * p.cap + slot;
      const int dst = pair_dst[i];
      if (dst < 0) continue;
      const int2 meta = reinterpret_cast<const int2*>(reinterpret_cast<const uint8_t*>(p.peers[p.rank]) + p.off_meta)[i];
      const uint4* sy = reinterpret_cast<const uint4*>(y + (long)dst * ldy);
      uint4* dy =
          reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peers[src]) + p.off_ret + (long)meta.y * p.d * 2);
      for (int j = threadIdx.x; j < p.d / 8; j += 256) dy[j] = sy[j];
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(mine + W_DONE + 1, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x < p.world) {
    __threadfence();
    st_release_sys(ctrl(p, threadIdx.x) + W_RET_FLAG + p.rank, p.epoch);
    if (threadIdx.x == 0) mine[W_DONE + 1] = 0;
  }
}

// out[t] = sum_j w[t,j] * returned[t*k+j] (+ shared[t]) in slot order
__global__ void __launch_bounds__(256) ep_combine_kernel(EpParams p, const int* __restrict__ ids,
                                                         const float* __restrict__ wts,
                                                         const float* __restrict__ shared_y,
                                                         __nv_bfloat16* __restrict__ out, long ldo) {
  tf_pdl_sync();
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!wait_epoch(ctrl(p, p.rank) + W_RET_FLAG + threadIdx.x, p.epoch, p.spin_limit)) {
      tf_report(p.st, TF_TIMEOUT, 302, threadIdx.x, blockIdx.x);
      s_fail = 1;
    }
  }
  __syncthreads();
  if (s_fail) return;
  const int t = blockIdx.x;
  const __nv_bfloat16* ret =
      reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const uint8_t*>(p.peers[p.rank]) + p.off_ret);
  for (int c = threadIdx.x * 2; c < p.d; c += 512) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < p.k; ++j) {
      const int e = ids[t * p.k + j];
      if (e < 0 || e >= p.El * p.world) continue;
      const float w = wts[t * p.k + j];
      const float2 v = __bfloat1622float2(
          __ldcg(reinterpret_cast<const __nv_bfloat162*>(ret + ((long)t * p.k + j) * p.d + c)));
      a0 = fmaf(w, v.x, a0);
      a1 = fmaf(w, v.y, a1);
    }
    if (shared_y) {
      a0 += shared_y[(long)t * p.d + c];
      a1 += shared_y[(long)t * p.d + c + 1];
    }
    *reinterpret_cast<__nv_bfloat162*>(out + (long)t * ldo + c) = __floats2bfloat162_rn(a0, a1);
  }
}

EpParams make_params(const void* peers, int world, int rank, int cap, int d, int k, int El, int Tl_max, int epoch,
                     int spin_limit, void* status) {
  EpParams p;
  p.peers = (const unsigned long long*)peers; p.world = world; p.rank = rank; p.cap = cap; p.d = d; p.k = k; p.El = El;
  p.off_meta = 4096;
  p.off_s = p.off_meta + (((long)world * cap * 8 + 255) / 256) * 256;
  p.off_x = p.off_s + (((long)world * cap * (d / 128) * 4 + 255) / 256) * 256;
  p.off_ret = p.off_x + (((long)world * cap * d + 255) / 256) * 256;
  p.epoch = (unsigned int)epoch; p.spin_limit = spin_limit; p.st = (TfStatusWord*)status;
  (void)Tl_max;
  return p;
}

}  // namespace

// cap: rows one source may send to one destination (worst case: local tokens * k)
TF_API long tf_ep_workspace_bytes(int world, int cap, int d, int Tl_max, int k) {
  EpParams p = make_params(nullptr, world, 0, cap, d, k, 1, Tl_max, 0, 0, nullptr);
  return p.off_ret + (long)Tl_max * k * d * 2 + 256;
}

TF_API int tf_ep_dispatch(const void* peers, int world, int rank, int cap, int d, int k, int El, int Tl_max, int epoch,
                          const void* x, long ldx, const int* ids, int Tl, void* status, cudaStream_t st) {
  if (world > kMaxWorld || k > 16 || d % 512 != 0 || Tl > Tl_max) return -1;
  if (Tl <= 0) Tl = 0;
  EpParams p = make_params(peers, world, rank, cap, d, k, El, Tl_max, epoch, 0, status);
  // a rank without tokens still has to publish its (zero) counts: one CTA with no pairs
  const int grid = Tl > 0 ? Tl : 1;
  tf_launch(ep_dispatch_kernel, dim3(grid), dim3(256), d + (d / 128) * 4, st, p, (const __nv_bfloat16*)x, ldx, ids, Tl);
  return (int)cudaGetLastError();
}

TF_API int tf_ep_recv_ids(const void* peers, int world, int rank, int cap, int d, int k, int El, int Tl_max, int epoch,
                          int* ids_out, int spin_limit, void* status, cudaStream_t st) {
  EpParams p = make_params(peers, world, rank, cap, d, k, El, Tl_max, epoch, spin_limit, status);
  const long n = (long)world * cap;
  tf_launch(ep_recv_ids_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, p, ids_out);
  return (int)cudaGetLastError();
}

TF_API int tf_ep_gather(const void* peers, int world, int rank, int cap, int d, int k, int El, int Tl_max,
                        const int* pair_dst, void* xp, float* xps, cudaStream_t st) {
  EpParams p = make_params(peers, world, rank, cap, d, k, El, Tl_max, 0, 0, nullptr);
  tf_launch(ep_gather_kernel, dim3(kWalkCtas), dim3(256), 0, st, p, pair_dst, (uint8_t*)xp, xps);
  return (int)cudaGetLastError();
}

TF_API int tf_ep_return(const void* peers, int world, int rank, int cap, int d, int k, int El, int Tl_max, int epoch,
                        const int* pair_dst, const void* y, long ldy, void* status, cudaStream_t st) {
  EpParams p = make_params(peers, world, rank, cap, d, k, El, Tl_max, epoch, 0, status);
  tf_launch(ep_return_kernel, dim3(kWalkCtas), dim3(256), 0, st, p, pair_dst, (const __nv_bfloat16*)y, ldy);
  return (int)cudaGetLastError();
}

TF_API int tf_ep_combine(const void* peers, int world, int rank, int cap, int d, int k, int El, int Tl_max, int epoch,
                         const int* ids, const float* wts, const float* shared_y, void* out, long ldo, int Tl,
                         int spin_limit, void* status, cudaStream_t st) {
  if (Tl <= 0) return 0;
  EpParams p = make_params(peers, world, rank, cap, d, k, El, Tl_max, epoch, spin_limit, status);
  tf_launch(ep_combine_kernel, dim3(Tl), dim3(256), 0, st, p, ids, wts, shared_y, (__nv_bfloat16*)out, ldo);
  return (int)cudaGetLastError();
}
