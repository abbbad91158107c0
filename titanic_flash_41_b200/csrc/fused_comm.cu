// Expert combine fused with the tensor/expert-parallel all-reduce, the residual update and the
// boundary of the next sublayer:
//   resid[r, :] += sum over ranks of ( sum_j w[r,j] * y_pair[r*k+j, :] (this rank's experts, fixed
//                  slot order) + shared_rank[r, :] )
//   norm_w given: h16 / hb / (x8, x8s) = RMSNorm(resid) * norm_w
// One CTA per 32 output columns, the same tiling as the fused GEMV, so both kinds of call share
// one symmetric workspace and one epoch sequence.  Also exports a plain one-shot all-reduce of a
// [rows, N] fp32 matrix (rows <= 32) for the remaining small exchanges, a form that emulates
// several ranks in one cooperative launch on one GPU (protocol tests on a single device), and a
// wait-limit probe used by the failure-detection test (a wait that nothing satisfies must return
// TF_TIMEOUT).
// Reference counterparts: kernels/ffn_sum_shared.cuh + kernels/roce_oneshot_hc.cuh.
#include "comm.cuh"

namespace {

struct CombineParams {
  const float* y_pair;
  const int* ids;
  const float* wts;
  const float* shared_y;
  int rows, d, topk, e_lo, e_hi;
  CommParams c;
  RowEpilogue ep;
  int wide;
  // emulated ranks (grid.y > 1): rank y reads its partial at shared_y + y * emu_stride and writes its
  // outputs at the same element offset (x8s: emu_stride / 32)
  long emu_stride;
};

__global__ void __launch_bounds__(256) combine_allreduce_kernel(const CombineParams p) {
  tf_pdl_sync();
  __shared__ __align__(16) float tile[32 * 32];
  extern __shared__ float rowbuf[];
  const int j = blockIdx.x, n0 = j * 32, rows = p.rows, d = p.d, topk = p.topk;
  const long off = (long)blockIdx.y * p.emu_stride;
  const float* shared_y = p.shared_y ? p.shared_y + off : nullptr;
  for (int i = threadIdx.x; i < rows * 32; i += blockDim.x) {
    const int r = i >> 5, cc = i & 31;
    float acc = 0.f;
    if (p.y_pair) {
      for (int k = 0; k < topk; ++k) {
        const int e = p.ids[r * topk + k];
        if (e >= p.e_lo && e < p.e_hi)
          acc = fmaf(p.wts[r * topk + k], p.y_pair[(long)(r * topk + k) * d + n0 + cc], acc);
      }
    }
    if (shared_y) acc += shared_y[(long)r * d + n0 + cc];
    tile[i] = acc;
  }
  __syncthreads();
  RowEpilogue ep = p.ep;
  if (off) {
    if (ep.resid) ep.resid += off;
    if (ep.ar_out) ep.ar_out += off;
    if (ep.h16) ep.h16 += off;
    if (ep.hb) ep.hb += off;
    if (ep.x8) ep.x8 += off;
    if (ep.x8s) ep.x8s += off / 32;
  }
  if (p.wide) comm_allreduce_rows<true>(p.c, tile, rows, ep, rowbuf);
  else comm_allreduce_rows<false>(p.c, tile, rows, ep, rowbuf);
}

// Wait on a flag nobody sets: exercises the bounded-wait path in isolation.
__global__ void wait_probe_kernel(const unsigned int* flag, unsigned int want, int spin_limit, TfStatusWord* st) {
  tf_pdl_sync();
  int spins = 0;
  while ((int)(ld_acquire_sys(flag) - want) < 0) {
    if (++spins > spin_limit) {
      tf_report(st, TF_TIMEOUT, 201, 0, spins);
      return;
    }
  }
}

bool fill(CombineParams& p, const float* y_pair, const int* ids, const float* wts, const float* shared_y, int rows,
          int d, int topk, int e_lo, int e_hi, const void* peers, int world, int rank, int max_rows, void* epoch,
          void* resid, float* ar_out, const void* norm_w, void* h16, void* hb, void* x8, void* x8s, float eps,
          int spin_limit, void* status) {
  if (d % 128 || rows < 1 || rows > 32 || rows > max_rows || world < 1 || world > kCommMaxWorld || d / 32 < rows)
    return false;
  if (!peers || !epoch || (!resid && !ar_out) || (!y_pair && !shared_y) || (y_pair && (!ids || !wts)) ||
      (x8 && !x8s) || (norm_w && !resid))
    return false;
  p.y_pair = y_pair; p.ids = ids; p.wts = wts; p.shared_y = shared_y; p.rows = rows; p.d = d; p.topk = topk;
  p.e_lo = e_lo; p.e_hi = e_hi;
  p.c.peers = (const unsigned long long*)peers; p.c.world = world; p.c.rank = rank; p.c.tiles = d / 32;
  p.c.max_rows = max_rows; p.c.N = d; p.c.epoch = (unsigned int*)epoch; p.c.spin_limit = spin_limit;
  p.c.st = (TfStatusWord*)status;
  p.ep.resid = (__nv_bfloat16*)resid; p.ep.ar_out = ar_out; p.ep.norm_w = (const __nv_bfloat16*)norm_w;
  p.ep.h16 = (__half*)h16; p.ep.hb = (__nv_bfloat16*)hb; p.ep.x8 = (uint8_t*)x8; p.ep.x8s = (uint8_t*)x8s;
  p.ep.eps = eps;
  p.wide = resid ? 0 : 1;
  p.emu_stride = 0;
  return true;
}

cudaError_t dyn_smem(size_t dyn) {
  if (dyn <= 40 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(combine_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
}

}  // namespace

// bytes of the symmetric workspace every rank must allocate for width N and up to max_rows rows
TF_API long tf_comm_workspace_bytes(int world, int N, int max_rows) { return 2L * world * max_rows * N * 8; }

// y_pair may be null (then only `shared_y` -- any [rows, d] fp32 partial -- is reduced).  With a
// residual the partials travel as bf16, without one (ar_out only) as fp32.
TF_API int tf_moe_combine_allreduce(const float* y_pair, const int* ids, const float* wts, const float* shared_y,
                                    int rows, int d, int topk, int e_lo, int e_hi, const void* peers, int world,
                                    int rank, int max_rows, void* epoch, void* resid, float* ar_out,
                                    const void* norm_w, void* h16, void* hb, void* x8, void* x8s, float eps,
                                    int spin_limit, void* status, cudaStream_t st) {
  CombineParams p;
  if (!fill(p, y_pair, ids, wts, shared_y, rows, d, topk, e_lo, e_hi, peers, world, rank, max_rows, epoch, resid,
            ar_out, norm_w, h16, hb, x8, x8s, eps, spin_limit, status))
    return -1;
  const size_t dyn = (size_t)d * sizeof(float);
  cudaError_t a = dyn_smem(dyn);
  if (a != cudaSuccess) return (int)a;
  tf_launch(combine_allreduce_kernel, dim3(d / 32), dim3(256), dyn, st, p);
  return (int)cudaGetLastError();
}

// `world` ranks emulated by ONE cooperative launch on one GPU: rank y reduces partial[y] (fp32
// [world][rows_alloc][d], rank stride = rows_alloc * d elements) and writes its outputs at the same
// per-rank offset of resid / ar_out / h16 / hb / x8 (x8s: stride / 32); `peers` holds `world`
// workspace areas of this device, `epoch` world * d/32 counters.  For protocol tests on one device.
TF_API int tf_comm_allreduce_emulated(const float* partial, int rows, int rows_alloc, int d, const void* peers,
                                      int world, int max_rows, void* epoch, void* resid, float* ar_out,
                                      const void* norm_w, void* h16, void* hb, void* x8, void* x8s, float eps,
                                      int spin_limit, void* status, cudaStream_t st) {
  CombineParams p;
  if (rows_alloc < rows ||
      !fill(p, nullptr, nullptr, nullptr, partial, rows, d, 0, 0, 0, peers, world, 0, max_rows, epoch, resid, ar_out,
            norm_w, h16, hb, x8, x8s, eps, spin_limit, status))
    return -1;
  p.emu_stride = (long)rows_alloc * d;
  const size_t dyn = (size_t)d * sizeof(float);
  cudaError_t a = dyn_smem(dyn);
  if (a != cudaSuccess) return (int)a;
  // every CTA of every emulated rank must be resident: a cooperative launch fails instead of waiting
  int dev = 0, coop = 0, per_sm = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, combine_allreduce_kernel, 256, dyn);
  if (!coop || (long)per_sm * sms < (long)(d / 32) * world) return -1;
  void* args[] = {(void*)&p};
  return (int)cudaLaunchCooperativeKernel((const void*)combine_allreduce_kernel, dim3(d / 32, world), dim3(256), args,
                                          dyn, st);
}

TF_API int tf_wait_probe(const void* flag, int want, int spin_limit, void* status, cudaStream_t st) {
  if (!flag) return -1;
  tf_launch(wait_probe_kernel, dim3(1), dim3(1), 0, st, (const unsigned int*)flag, (unsigned int)want, spin_limit, (TfStatusWord*)status);
  return (int)cudaGetLastError();
}
