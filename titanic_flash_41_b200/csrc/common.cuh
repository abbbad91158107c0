// Shared device helpers for the sm_100a kernels: status words, bounded waits, number-format
// conversions, warp/block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TF_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  A decode step is several hundred short kernels, each of which
// waits for the launch latency of its successor after it has finished.  Every kernel here begins
// with tf_pdl_sync(): it waits until the kernel before it in the stream has completed and its
// writes are visible (so the usual ordering holds for every read AND write that follows), then
// lets the kernel after it be launched.  With the launch attribute set (tf_set_pdl), the next
// kernel's CTAs are therefore already resident and parked at their own tf_pdl_sync() while this
// one runs, and start the moment it ends.  Without the attribute both instructions are no-ops.
// (Reference: launch_pdl, src/cuda.rs:2209.)
// ---------------------------------------------------------------------------------------
// A kernel whose first loads are of data no kernel writes (weights) may issue those loads before
// tf_pdl_sync(): they then overlap the tail of the kernel before it.
__device__ __forceinline__ void tf_pdl_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

extern int g_tf_pdl;     // set through tf_set_pdl (launch.cu)

template <typename... KArgs, typename... Args>
inline cudaError_t tf_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_tf_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------------
// Status words.  No kernel traps, asserts or spins without a limit: a kernel that meets a
// bad argument or a wait that runs out records (code, detail) here and returns; the host
// reads the word after the step (the reference records a poison word + (peer, slot, seq)
// the same way: kernels/roce_oneshot_twin.cuh:108-140).
// ---------------------------------------------------------------------------------------
enum TfStatus : int {
  TF_OK = 0,
  TF_BAD_ARG = 1,
  TF_TIMEOUT = 2,       // a bounded wait ran out
  TF_BAD_INDEX = 3,     // an index outside its table (candidate remap, page map)
  TF_NONFINITE = 4,     // NaN/inf where a probability was expected
};

struct TfStatusWord {
  int code;     // first non-zero code wins
  int kernel;   // kernel id
  int detail0;  // e.g. peer / stage / row
  int detail1;
};

__device__ __forceinline__ void tf_report(TfStatusWord* st, int code, int kernel, int d0, int d1) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->kernel = kernel;
    st->detail0 = d0;
    st->detail1 = d1;
  }
}

// ---------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; `scratch` holds >= 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[w] = v;
  __syncthreads();
  float t = (lane < nw) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[w] = v;
  __syncthreads();
  float t = (lane < nw) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// ---------------------------------------------------------------------------------------
// number formats
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float ue8m0_to_float(uint8_t s) {
  // 255 -> NaN, 0 -> 2^-127, else 2^(s-127)
  uint32_t bits = (s == 255) ? 0x7fc00000u : (s == 0 ? (1u << 22) : ((uint32_t)s << 23));
  return __uint_as_float(bits);
}
// smallest power of two >= x (x >= 0) as a UE8M0 byte
__device__ __forceinline__ uint8_t ue8m0_ceil(float x) {
  uint32_t b = __float_as_uint(fmaxf(x, 1.1754944e-38f));
  int e = (int)(b >> 23) & 0xff;
  if (b & 0x7fffffu) e += 1;
  return (uint8_t)min(max(e, 0), 254);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t float_to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
// two e4m3 bytes (low byte = first element) -> f16x2
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
  uint32_t e = (nib >> 1) & 3u, m = nib & 1u;
  float mag = e ? (float)(2u + m) * 0.5f * (float)(1u << (e - 1)) : 0.5f * (float)m;
  return (nib & 8u) ? -mag : mag;
}
// round-to-nearest-even e2m1 code of x (saturating at 6)
__device__ __forceinline__ uint32_t float_to_e2m1(float x) {
  float a = fabsf(x);
  uint32_t c;
  if (a <= 0.25f) c = 0;                 // tie 0.25 -> 0 (even)
  else if (a < 0.75f) c = 1;             // tie 0.75 -> 1.0 (code 2, even)
  else if (a <= 1.25f) c = 2;            // tie 1.25 -> 1.0 (even)
  else if (a < 1.75f) c = 3;             // tie 1.75 -> 2.0
  else if (a <= 2.5f) c = 4;             // tie 2.5 -> 2.0
  else if (a < 3.5f) c = 5;              // tie 3.5 -> 4.0
  else if (a <= 5.0f) c = 6;             // tie 5.0 -> 4.0
  else c = 7;
  return c | ((x < 0.f || (x == 0.f && signbit(x))) ? 8u : 0u);
}
// 8 packed e2m1 nibbles (element i in bits [4i,4i+4)) -> four f16x2 holding value * 2^-14
// (the nibble's exponent/mantissa bits dropped into the f16 exponent field; subnormal exact).
__device__ __forceinline__ void e2m1x8_to_h2x4_scaled(uint32_t w, uint32_t out[4]) {
  // one nibble per byte: t = elements 0,2,4,6 ; u = elements 1,3,5,7
  const uint32_t t = w & 0x0f0f0f0fu, u = (w >> 4) & 0x0f0f0f0fu;
  // high byte of the f16 image of a nibble n: sign -> bit 7, (n & 7) -> bits 1..3
  const uint32_t ht = ((t << 4) & 0x80808080u) | ((t << 1) & 0x0e0e0e0eu);
  const uint32_t hu = ((u << 4) & 0x80808080u) | ((u << 1) & 0x0e0e0e0eu);
  out[0] = __byte_perm(ht, hu, 0x4000) & 0xff00ff00u;
  out[1] = __byte_perm(ht, hu, 0x5111) & 0xff00ff00u;
  out[2] = __byte_perm(ht, hu, 0x6222) & 0xff00ff00u;
  out[3] = __byte_perm(ht, hu, 0x7333) & 0xff00ff00u;
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// m16n8k16 f16 x f16 -> f32
__device__ __forceinline__ void mma_f16_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
