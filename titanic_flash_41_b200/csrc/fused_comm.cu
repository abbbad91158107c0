// Expert combine fused with the tensor/expert-parallel all-reduce and the residual update:
//   resid[r, :] += sum over ranks of ( sum_j w[r,j] * y_pair[r*k+j, :] (this rank's experts, fixed
//                  slot order) + shared_rank[r, :] )
// One CTA per 32 output columns, the same tiling as the fused GEMV, so both kinds of call share
// one symmetric workspace and one epoch sequence.  Also exports a plain one-shot all-reduce of a
// [rows, N] fp32 matrix (rows <= 32) for the remaining small exchanges, and a wait-limit probe
// used by the failure-detection test (a wait that nothing satisfies must return TF_TIMEOUT).
// Reference counterparts: kernels/ffn_sum_shared.cuh + kernels/roce_oneshot_hc.cuh.
#include "comm.cuh"

namespace {

__global__ void __launch_bounds__(256) combine_allreduce_kernel(
    const float* __restrict__ y_pair, const int* __restrict__ ids, const float* __restrict__ wts,
    const float* __restrict__ shared_y, int rows, int d, int topk, int e_lo, int e_hi, CommParams c,
    __nv_bfloat16* resid, float* ar_out) {
  __shared__ __align__(16) float tile[32 * 32];
  const int j = blockIdx.x, n0 = j * 32;
  for (int i = threadIdx.x; i < rows * 32; i += blockDim.x) {
    const int r = i >> 5, cc = i & 31;
    float acc = 0.f;
    if (y_pair) {
      for (int k = 0; k < topk; ++k) {
        const int e = ids[r * topk + k];
        if (e >= e_lo && e < e_hi) acc = fmaf(wts[r * topk + k], y_pair[(long)(r * topk + k) * d + n0 + cc], acc);
      }
    }
    if (shared_y) acc += shared_y[(long)r * d + n0 + cc];
    tile[i] = acc;
  }
  __syncthreads();
  if (comm_allreduce_tile(c, tile, rows, j)) comm_residual_update(resid, d, ar_out, d, tile, rows, j);
}

// Wait on a flag nobody sets: exercises the bounded-wait path in isolation.
__global__ void wait_probe_kernel(const unsigned int* flag, unsigned int want, int spin_limit, TfStatusWord* st) {
  int spins = 0;
  while ((int)(ld_acquire_sys(flag) - want) < 0) {
    if (++spins > spin_limit) {
      tf_report(st, TF_TIMEOUT, 201, 0, spins);
      return;
    }
  }
}

CommParams make_comm(const void* peers, int world, int rank, int N, int max_rows, long flag_bytes, void* epoch,
                     int spin_limit, void* status) {
  CommParams c;
  c.peers = (const unsigned long long*)peers; c.world = world; c.rank = rank; c.tiles = N / 32;
  c.max_rows = max_rows; c.N = N; c.epoch = (unsigned int*)epoch; c.flag_bytes = flag_bytes;
  c.spin_limit = spin_limit; c.st = (TfStatusWord*)status;
  return c;
}

}  // namespace

// bytes of the symmetric workspace every rank must allocate for width N and up to max_rows rows
TF_API long tf_comm_flag_bytes(int world, int N) { return ((long)world * (N / 32) * 4 + 255) / 256 * 256; }
TF_API long tf_comm_workspace_bytes(int world, int N, int max_rows) {
  return tf_comm_flag_bytes(world, N) + 2L * world * max_rows * N * 4;
}

// y_pair may be null (then only `shared_y` -- any [rows, d] fp32 partial -- is reduced)
TF_API int tf_moe_combine_allreduce(const float* y_pair, const int* ids, const float* wts, const float* shared_y,
                                    int rows, int d, int topk, int e_lo, int e_hi, const void* peers, int world,
                                    int rank, int max_rows, long flag_bytes, void* epoch, void* resid,
                                    float* ar_out, int spin_limit, void* status, cudaStream_t st) {
  if (d % 32 || rows < 1 || rows > 32 || rows > max_rows || world < 1 || world > 32) return -1;
  CommParams c = make_comm(peers, world, rank, d, max_rows, flag_bytes, epoch, spin_limit, status);
  combine_allreduce_kernel<<<d / 32, 256, 0, st>>>(y_pair, ids, wts, shared_y, rows, d, topk, e_lo, e_hi, c,
                                                   (__nv_bfloat16*)resid, ar_out);
  return (int)cudaGetLastError();
}

TF_API int tf_wait_probe(const void* flag, int want, int spin_limit, void* status, cudaStream_t st) {
  wait_probe_kernel<<<1, 1, 0, st>>>((const unsigned int*)flag, (unsigned int)want, spin_limit, (TfStatusWord*)status);
  return (int)cudaGetLastError();
}
