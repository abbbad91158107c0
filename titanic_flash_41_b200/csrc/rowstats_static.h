// tf_rowstats_static: the row statistics of tf_rowstats (row maximum, softmax normaliser and the
// nucleus cut-off of each logits row) for a caller that has no device memory to give as scratch.
//
// This entry point has no counterpart in the reference engine; it exists for hosts of this
// library that cannot allocate: a plain C program that links the shared object and owns no
// allocator, or a sampling thread that runs while the engine's pools already hold nearly all of
// the device memory, where a fresh device allocation can fail or stall every stream of the device.
//
// The scratch area is one file-scope device array inside the library, sized for
// TF_ROWSTATS_STATIC_MAX_ROWS rows (32,832 bytes per row; 525,312 bytes in all).  Consequences:
//   * rows > TF_ROWSTATS_STATIC_MAX_ROWS is refused with TF_ROWSTATS_STATIC_TOO_MANY_ROWS and a
//     line on stderr; nothing is launched.
//   * The first call on each device looks the array's address up once (cudaGetSymbolAddress) and
//     keeps it; that lookup can load the module, so make one call on every device before any
//     stream capture begins.  Later calls only enqueue a clear of the part they use and kernels.
//   * Every call clears rows * 32,832 bytes of the array on `st` before its kernels, so an earlier
//     call that was abandoned half-way cannot leak counters into this one.
//   * There is ONE array per device: two calls whose kernels can overlap in time (different
//     streams, or different host threads on different streams) race on it and return garbage.
//     Issue the calls of one device on one stream, or order them with events.
//   * Nothing is allocated or freed, here or later: no cudaMalloc / cudaFree / cudaMallocAsync,
//     no library call that allocates.
//
// Arguments are those of tf_rowstats without `scratch`: logits [rows, ldl] fp32 (16-byte aligned,
// ldl % 4 == 0), V valid columns, temp > 0, top_p in (0, 1], out = rows * tf_rowstat_bytes() bytes,
// status = the device status word (may be null).  Returns 0, -1 (bad argument),
// TF_ROWSTATS_STATIC_TOO_MANY_ROWS, or a cudaError_t value.
#pragma once
#include <cuda_runtime.h>

#define TF_ROWSTATS_STATIC_MAX_ROWS 16
#define TF_ROWSTATS_STATIC_TOO_MANY_ROWS (-3)

extern "C" __attribute__((visibility("default"))) int tf_rowstats_static(
    const float* logits, int ldl, int V, int rows, float temp, float top_p, void* out, void* status,
    cudaStream_t st);
