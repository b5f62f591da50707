// Allocation-free global average pooling; see gap_noalloc.h for who needs it and the rules of use.
// The per-split partial sums go to a file-scope device array instead of a caller-provided buffer.
#include "gap_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace {

// Scratch for the partial sums, part of the library image on every device that loads it.
// In host code this name is only a handle: the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_gap_scratch[FDB_GAP_NOALLOC_MAX_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t;
    if (BF16) t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
    else t = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

// One block = one image, one pixel split, 64 channels; 256 threads = 8 channel groups x 32 pixel lanes.
template <bool BF16>
__global__ void gap_partial_noalloc(const uint8_t* __restrict__ x, float* __restrict__ part, int HW, int C,
                                    int x_ld, int S, long long x_n_stride) {
  const int n = blockIdx.y, split = blockIdx.z;
  const int cg = threadIdx.x & 7, pl = threadIdx.x >> 3;
  const int c0 = (blockIdx.x * 8 + cg) * 8;
  const int per = (HW + S - 1) / S;
  const int p_begin = split * per, p_end = min(HW, p_begin + per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < C) {
    const uint8_t* base = x + (static_cast<size_t>(n) * x_n_stride + c0) * 2;
    for (int p = p_begin + pl; p < p_end; p += 32) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(p) * x_ld * 2));
      float f[8];
      unpack8<BF16>(u, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
  __shared__ float red[32][8][8];
#pragma unroll
  for (int j = 0; j < 8; ++j) red[pl][cg][j] = acc[j];
  __syncthreads();
  if (threadIdx.x < 64) {
    const int g = threadIdx.x >> 3, j = threadIdx.x & 7;
    float s = 0.f;
    for (int l = 0; l < 32; ++l) s += red[l][g][j];
    const int c = (blockIdx.x * 8 + g) * 8 + j;
    // every (n, split, c) element read by the second kernel is written here: no clearing needed
    if (c < C) part[(static_cast<size_t>(n) * S + split) * C + c] = s;
  }
}

__global__ void gap_finalize_noalloc(const float* __restrict__ part, void* __restrict__ out, int N, int C, int S,
                                     int out_dtype, int out_ld, float scale) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * C) return;
  const int n = idx / C, c = idx - n * C;
  float s = 0.f;
  for (int k = 0; k < S; ++k) s += part[(static_cast<size_t>(n) * S + k) * C + c];
  s *= scale;
  const size_t o = static_cast<size_t>(n) * out_ld + c;
  if (out_dtype == 2) reinterpret_cast<float*>(out)[o] = s;
  else if (out_dtype == 1) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(s);
  else reinterpret_cast<__half*>(out)[o] = __float2half_rn(s);
}

// Device address of the scratch array for the current device; resolved once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FDB_GAP_NOALLOC_CUDA_ERROR;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_gap_scratch);
    if (e != cudaSuccess || ptr == nullptr) return FDB_GAP_NOALLOC_CUDA_ERROR;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return FDB_GAP_NOALLOC_OK;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int fdb_global_avgpool_noalloc(const void* x, void* out, int n, int hw, int c, int x_ld, long long x_n_stride,
                               int splits, int is_bf16, int out_dtype, int out_ld, void* stream) {
  if (x == nullptr || out == nullptr || n <= 0 || hw <= 0 || c <= 0 || splits <= 0 || c % 8 != 0 || x_ld % 8 != 0 ||
      x_ld < c || out_ld < c || out_dtype < 0 || out_dtype > 2 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return FDB_GAP_NOALLOC_BAD_ARGUMENT;
  // Every image starts at x + i * x_n_stride and is read with 16-byte loads: the image stride must keep
  // that alignment, and a non-zero stride may not be shorter than one image (overlapping images are
  // legal reads but never what a caller means).
  if (x_n_stride < 0 || x_n_stride % 8 != 0 ||
      (x_n_stride > 0 && x_n_stride < static_cast<long long>(hw - 1) * x_ld + c))
    return FDB_GAP_NOALLOC_BAD_ARGUMENT;
  const long long need = static_cast<long long>(n) * splits * c;
  if (need > FDB_GAP_NOALLOC_MAX_SCRATCH_FLOATS) return FDB_GAP_NOALLOC_TOO_LARGE;
  if (splits > 65535 || n > 65535) return FDB_GAP_NOALLOC_BAD_ARGUMENT;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FDB_GAP_NOALLOC_OK) return rc;
  const long long xns = x_n_stride > 0 ? x_n_stride : static_cast<long long>(hw) * x_ld;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((c + 63) / 64, n, splits);
  // Launch errors are read with cudaPeekAtLastError straight after each launch, so that this call
  // reports its own launches only and leaves an earlier, unrelated error where its owner will find it.
  if (cudaPeekAtLastError() != cudaSuccess) return FDB_GAP_NOALLOC_CUDA_ERROR;
  if (is_bf16)
    gap_partial_noalloc<true><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(x), scratch, hw, c, x_ld, splits, xns);
  else
    gap_partial_noalloc<false><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(x), scratch, hw, c, x_ld, splits, xns);
  gap_finalize_noalloc<<<(n * c + 255) / 256, 256, 0, s>>>(scratch, out, n, c, splits, out_dtype, out_ld, 1.0f / hw);
  return cudaPeekAtLastError() == cudaSuccess ? FDB_GAP_NOALLOC_OK : FDB_GAP_NOALLOC_CUDA_ERROR;
}

extern "C" __attribute__((visibility("default")))
const char* fdb_global_avgpool_noalloc_strerror(int code) {
  switch (code) {
    case FDB_GAP_NOALLOC_OK: return "ok";
    case FDB_GAP_NOALLOC_BAD_ARGUMENT: return "bad argument: null pointer, x not 16-byte aligned, non-positive size, c / x_ld / x_n_stride not a "
                                              "multiple of 8, x_ld or out_ld below c, x_n_stride shorter than one image, or out_dtype outside 0..2";
    case FDB_GAP_NOALLOC_TOO_LARGE: return "n * splits * c exceeds the built-in scratch of 1048576 floats";
    case FDB_GAP_NOALLOC_CUDA_ERROR: return "CUDA error: pending before the call, while resolving the scratch address, or at launch";
    default: return "unknown code";
  }
}
