// Process-wide switch of programmatic dependent launches (see tf_pdl_sync / tf_launch in common.cuh).
#include "common.cuh"

int g_tf_pdl = 0;

// on != 0: every kernel of this library is launched with the programmatic-stream-serialization
// attribute, in eager launches and under stream capture alike.  Returns the previous setting.
TF_API int tf_set_pdl(int on) {
  const int old = g_tf_pdl;
  g_tf_pdl = on ? 1 : 0;
  return old;
}

TF_API int tf_get_pdl() { return g_tf_pdl; }

namespace {
__global__ void stamp_kernel(unsigned long long* ring, int slot) {
  tf_pdl_sync();
  if (threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    ring[slot] = t;
  }
}
}  // namespace

// Device timestamp (nanoseconds of the GPU's global timer) into ring[slot], in stream order.  A
// stamp is an ordinary one-thread kernel, so it can be captured in a CUDA graph: replaying the
// graph refreshes the ring, which is how kernels are timed INSIDE a graph without a profiler
// (reference: the globaltimer marks of src/layer_clock.rs).
TF_API int tf_stamp(void* ring, int slot, int capacity, cudaStream_t st) {
  if (!ring || slot < 0 || slot >= capacity) return -1;
  tf_launch(stamp_kernel, dim3(1), dim3(32), 0, st, reinterpret_cast<unsigned long long*>(ring), slot);
  return (int)cudaGetLastError();
}
