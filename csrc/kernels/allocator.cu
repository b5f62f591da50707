// Caching memory pools: device memory and page-locked host memory, per device, in power-of-two size classes.
//
// cudaMalloc and cudaHostAlloc synchronise the device and cost tens to hundreds of microseconds; a serving process
// that stages a request in pinned memory and hands tensors between stages cannot pay that per request. A freed block
// goes back to its size class together with an event recorded on the stream that last used it, and is handed out
// again only when that event has completed, so a block is never reused under a copy or kernel still in flight.
//
// The reference has the same two roles as FDHostAllocator / FDDeviceAllocator / FDDeviceHostAllocator
// (fastdeploy/core/allocate.h:26-56) without caching; its back ends bring their own pools.
#include "fdb_common.h"

#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace fdb {

struct PoolBlock {
  void* ptr;
  size_t bytes;       // size class
  int device;
  int kind;           // 0 device, 1 pinned host
  cudaEvent_t ev;     // recorded at free time on the caller's stream (null when freed without a stream)
};

struct Pool {
  std::mutex mu;
  // (kind, device, size class) -> cached blocks
  std::map<std::tuple<int, int, size_t>, std::vector<PoolBlock>> cache;
  std::unordered_map<void*, PoolBlock> live;
  long long allocated[2] = {0, 0};      // bytes handed out now
  long long cached[2] = {0, 0};         // bytes sitting in the cache
  long long high_water[2] = {0, 0};
  long long driver_calls[2] = {0, 0};   // cudaMalloc / cudaHostAlloc calls made
  long long hits[2] = {0, 0};           // allocations served from the cache
};

static Pool& pool() {
  static Pool p;
  return p;
}

static size_t size_class(size_t bytes) {
  size_t c = 512;
  while (c < bytes) c <<= 1;
  return c;
}

}  // namespace fdb

using namespace fdb;

// kind 0: device memory of `device`; kind 1: page-locked host memory (portable, usable from every device).
FDB_API void* fdb_pool_alloc(int kind, int device, long long bytes) {
  if (kind < 0 || kind > 1 || bytes <= 0) { set_error("pool_alloc: bad kind or size"); return nullptr; }
  Pool& p = pool();
  const size_t cls = size_class(static_cast<size_t>(bytes));
  const int dev_key = kind == 1 ? -1 : device;
  {
    std::lock_guard<std::mutex> lk(p.mu);
    auto it = p.cache.find({kind, dev_key, cls});
    if (it != p.cache.end()) {
      auto& v = it->second;
      for (size_t i = 0; i < v.size(); ++i) {
        if (v[i].ev != nullptr && cudaEventQuery(v[i].ev) != cudaSuccess) continue;    // still in use by its stream
        PoolBlock b = v[i];
        v.erase(v.begin() + i);
        if (b.ev != nullptr) { cudaEventDestroy(b.ev); b.ev = nullptr; }
        p.cached[kind] -= static_cast<long long>(cls);
        p.allocated[kind] += static_cast<long long>(cls);
        p.high_water[kind] = std::max(p.high_water[kind], p.allocated[kind]);
        p.hits[kind] += 1;
        p.live[b.ptr] = b;
        return b.ptr;
      }
    }
  }
  void* ptr = nullptr;
  cudaError_t e;
  if (kind == 0) {
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != device) cudaSetDevice(device);
    e = cudaMalloc(&ptr, cls);
    if (prev != device) cudaSetDevice(prev);
  } else {
    e = cudaHostAlloc(&ptr, cls, cudaHostAllocPortable);
  }
  if (e != cudaSuccess) {
    set_error(std::string("pool_alloc: ") + cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(p.mu);
  p.driver_calls[kind] += 1;
  p.allocated[kind] += static_cast<long long>(cls);
  p.high_water[kind] = std::max(p.high_water[kind], p.allocated[kind]);
  p.live[ptr] = PoolBlock{ptr, cls, dev_key, kind, nullptr};
  return ptr;
}

// Returns a block to the cache. `stream` (may be null with use_stream = 0) is the stream whose work last touched it.
FDB_API int fdb_pool_free(void* ptr, void* stream, int use_stream) {
  Pool& p = pool();
  std::lock_guard<std::mutex> lk(p.mu);
  auto it = p.live.find(ptr);
  if (it == p.live.end()) { set_error("pool_free: pointer was not allocated by this pool"); return -1; }
  PoolBlock b = it->second;
  p.live.erase(it);
  if (use_stream) {
    if (cudaEventCreateWithFlags(&b.ev, cudaEventDisableTiming) == cudaSuccess) {
      if (cudaEventRecord(b.ev, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        cudaEventDestroy(b.ev);
        b.ev = nullptr;
        cudaGetLastError();
      }
    } else {
      b.ev = nullptr;
      cudaGetLastError();
    }
  }
  p.allocated[b.kind] -= static_cast<long long>(b.bytes);
  p.cached[b.kind] += static_cast<long long>(b.bytes);
  p.cache[{b.kind, b.device, b.bytes}].push_back(b);
  return 0;
}

// Releases every cached block whose last use has completed back to the driver. Returns the bytes released.
FDB_API long long fdb_pool_trim() {
  Pool& p = pool();
  std::lock_guard<std::mutex> lk(p.mu);
  long long released = 0;
  for (auto& kv : p.cache) {
    auto& v = kv.second;
    for (size_t i = 0; i < v.size();) {
      if (v[i].ev != nullptr && cudaEventQuery(v[i].ev) != cudaSuccess) { ++i; continue; }
      if (v[i].ev != nullptr) cudaEventDestroy(v[i].ev);
      if (v[i].kind == 0) cudaFree(v[i].ptr); else cudaFreeHost(v[i].ptr);
      p.cached[v[i].kind] -= static_cast<long long>(v[i].bytes);
      released += static_cast<long long>(v[i].bytes);
      v.erase(v.begin() + i);
    }
  }
  cudaGetLastError();
  return released;
}

// out[0..9] = for kind 0 then kind 1: allocated, cached, high water, driver calls, cache hits
FDB_API void fdb_pool_stats(long long* out) {
  Pool& p = pool();
  std::lock_guard<std::mutex> lk(p.mu);
  for (int k = 0; k < 2; ++k) {
    out[5 * k + 0] = p.allocated[k];
    out[5 * k + 1] = p.cached[k];
    out[5 * k + 2] = p.high_water[k];
    out[5 * k + 3] = p.driver_calls[k];
    out[5 * k + 4] = p.hits[k];
  }
}
