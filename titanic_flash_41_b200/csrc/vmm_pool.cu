// Fixed pool of physical memory chunks mapped on demand into contiguous virtual ranges.
//
//   pool      n chunks of `chunk` bytes (a multiple of the allocation granularity, 16 MiB by
//             default) created once with cuMemCreate: snapshots of session state are carved from
//             it, so saving and dropping images never fragments or grows the device heap
//   range     tf_vmm_alloc reserves a virtual range, maps ceil(bytes / chunk) free chunks into it
//             and returns its address; tf_vmm_free unmaps and gives the chunks back
//   elastic   tf_vmm_reserve reserves a large range with nothing mapped; tf_vmm_resize maps or
//             unmaps chunks at its tail, so a region's buffers keep their addresses (captured CUDA
//             graphs stay valid) while only the occupied part costs memory
// Running out of chunks is an error code, not an exception or a device fault.
// (reference: src/cuda.rs:418 ChunkPool, :435 ElasticAllocation, :499 PooledAllocation,
//  :1137 create_image_pool, :1208 allocate_pooled, :1236 allocate_elastic, :1724 elastic_map)
#include <cuda.h>
#include <cudaTypedefs.h>

#include <map>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace {

struct Driver {
  PFN_cuMemCreate_v10020 create = nullptr;
  PFN_cuMemRelease_v10020 release = nullptr;
  PFN_cuMemAddressReserve_v10020 reserve = nullptr;
  PFN_cuMemAddressFree_v10020 afree = nullptr;
  PFN_cuMemMap_v10020 map = nullptr;
  PFN_cuMemUnmap_v10020 unmap = nullptr;
  PFN_cuMemSetAccess_v10020 access = nullptr;
  PFN_cuMemGetAllocationGranularity_v10020 gran = nullptr;
  bool ok = false;
};

template <typename F>
bool entry(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return false;
  *out = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = entry("cuMemCreate", &d.create) && entry("cuMemRelease", &d.release) &&
           entry("cuMemAddressReserve", &d.reserve) && entry("cuMemAddressFree", &d.afree) &&
           entry("cuMemMap", &d.map) && entry("cuMemUnmap", &d.unmap) && entry("cuMemSetAccess", &d.access) &&
           entry("cuMemGetAllocationGranularity", &d.gran);
  });
  return d;
}

struct Range {
  size_t reserved = 0;              // bytes of virtual address space
  std::vector<int> chunks;          // pool chunks mapped from the start of the range, in order
};

struct Pool {
  int device = 0;
  size_t chunk = 0;
  std::vector<CUmemGenericAllocationHandle> handles;
  std::vector<int> free_list;
  std::map<CUdeviceptr, Range> ranges;
  std::mutex mu;
};

int map_tail(Pool* p, CUdeviceptr base, Range& r, size_t want_chunks) {
  Driver& d = driver();
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = p->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  while (r.chunks.size() < want_chunks) {
    if (p->free_list.empty()) return -2;
    const int c = p->free_list.back();
    const CUdeviceptr at = base + r.chunks.size() * p->chunk;
    if (d.map(at, p->chunk, 0, p->handles[c], 0) != CUDA_SUCCESS) return -3;
    if (d.access(at, p->chunk, &acc, 1) != CUDA_SUCCESS) {
      d.unmap(at, p->chunk);
      return -3;
    }
    p->free_list.pop_back();
    r.chunks.push_back(c);
  }
  while (r.chunks.size() > want_chunks) {
    const CUdeviceptr at = base + (r.chunks.size() - 1) * p->chunk;
    if (d.unmap(at, p->chunk) != CUDA_SUCCESS) return -3;
    p->free_list.push_back(r.chunks.back());
    r.chunks.pop_back();
  }
  return 0;
}

}  // namespace

// returns a pool handle (0 on failure); *chunk_out = the chunk size actually used
TF_API long tf_vmm_pool_create(int device, long chunk_bytes, int n_chunks, long* chunk_out) {
  Driver& d = driver();
  if (!d.ok || n_chunks <= 0 || chunk_bytes <= 0) return 0;
  cudaSetDevice(device);
  cudaFree(nullptr);                                   // make sure the primary context exists
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  size_t g = 0;
  if (d.gran(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) return 0;
  Pool* p = new Pool;
  p->device = device;
  p->chunk = ((size_t)chunk_bytes + g - 1) / g * g;
  for (int i = 0; i < n_chunks; ++i) {
    CUmemGenericAllocationHandle h;
    if (d.create(&h, p->chunk, &prop, 0) != CUDA_SUCCESS) break;      // a smaller pool is still a pool
    p->handles.push_back(h);
    p->free_list.push_back(i);
  }
  if (p->handles.empty()) {
    delete p;
    return 0;
  }
  if (chunk_out) *chunk_out = (long)p->chunk;
  return (long)reinterpret_cast<uintptr_t>(p);
}

TF_API int tf_vmm_pool_chunks(long pool, int* total, int* free_chunks) {
  Pool* p = reinterpret_cast<Pool*>((uintptr_t)pool);
  if (!p) return -1;
  std::lock_guard<std::mutex> lock(p->mu);
  *total = (int)p->handles.size();
  *free_chunks = (int)p->free_list.size();
  return 0;
}

// reserve `max_bytes` of address space with `mapped_bytes` mapped at its start; returns the address or 0
// (*err: 0 ok, -1 bad argument, -2 pool exhausted, -3 driver error)
TF_API long tf_vmm_reserve(long pool, long max_bytes, long mapped_bytes, int* err) {
  Pool* p = reinterpret_cast<Pool*>((uintptr_t)pool);
  Driver& d = driver();
  *err = -1;
  if (!p || max_bytes <= 0 || mapped_bytes < 0 || mapped_bytes > max_bytes) return 0;
  std::lock_guard<std::mutex> lock(p->mu);
  const size_t chunks_max = ((size_t)max_bytes + p->chunk - 1) / p->chunk;
  const size_t want = ((size_t)mapped_bytes + p->chunk - 1) / p->chunk;
  if (want > p->free_list.size()) {
    *err = -2;
    return 0;
  }
  CUdeviceptr base = 0;
  if (d.reserve(&base, chunks_max * p->chunk, p->chunk, 0, 0) != CUDA_SUCCESS) {
    *err = -3;
    return 0;
  }
  Range r;
  r.reserved = chunks_max * p->chunk;
  const int rc = map_tail(p, base, r, want);
  if (rc != 0) {
    map_tail(p, base, r, 0);
    d.afree(base, r.reserved);
    *err = rc;
    return 0;
  }
  p->ranges[base] = r;
  *err = 0;
  return (long)base;
}

TF_API long tf_vmm_alloc(long pool, long bytes, int* err) { return tf_vmm_reserve(pool, bytes, bytes, err); }

// grow or shrink the mapped prefix of a reserved range; contents of what stays mapped are kept
TF_API int tf_vmm_resize(long pool, long base, long mapped_bytes) {
  Pool* p = reinterpret_cast<Pool*>((uintptr_t)pool);
  if (!p) return -1;
  std::lock_guard<std::mutex> lock(p->mu);
  auto it = p->ranges.find((CUdeviceptr)base);
  if (it == p->ranges.end() || mapped_bytes < 0 || (size_t)mapped_bytes > it->second.reserved) return -1;
  const size_t want = ((size_t)mapped_bytes + p->chunk - 1) / p->chunk;
  const size_t have = it->second.chunks.size();
  if (want > have && want - have > p->free_list.size()) return -2;
  return map_tail(p, (CUdeviceptr)base, it->second, want);
}

TF_API int tf_vmm_free(long pool, long base) {
  Pool* p = reinterpret_cast<Pool*>((uintptr_t)pool);
  Driver& d = driver();
  if (!p) return -1;
  std::lock_guard<std::mutex> lock(p->mu);
  auto it = p->ranges.find((CUdeviceptr)base);
  if (it == p->ranges.end()) return -1;
  const int rc = map_tail(p, (CUdeviceptr)base, it->second, 0);
  if (rc != 0) return rc;
  d.afree((CUdeviceptr)base, it->second.reserved);
  p->ranges.erase(it);
  return 0;
}

// the caller has synchronised the device and dropped every view of the pool's ranges
TF_API int tf_vmm_pool_destroy(long pool) {
  Pool* p = reinterpret_cast<Pool*>((uintptr_t)pool);
  Driver& d = driver();
  if (!p) return -1;
  {
    std::lock_guard<std::mutex> lock(p->mu);
    for (auto& kv : p->ranges) {
      map_tail(p, kv.first, kv.second, 0);
      d.afree(kv.first, kv.second.reserved);
    }
    p->ranges.clear();
    for (auto h : p->handles) d.release(h);
  }
  delete p;
  return 0;
}
