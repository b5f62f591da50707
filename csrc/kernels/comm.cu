// Peer-memory communication layer for one process per GPU.
//
// * symmetric heap: every rank allocates the same-sized device buffer here and publishes its CUDA
//   IPC handle; peers open it and get a plain device pointer that their kernels load from and store
//   to over NVLink (no library kernel ever receives such a pointer);
// * signals: 32-bit counters inside the heap, bumped with system-scope atomics after the data they
//   cover, waited for with a clock budget; a wait that runs out records kStatusTimeoutPeer in the
//   status word and the kernel returns, so the context stays usable;
// * collectives written directly on top: barrier, all-gather (pull), reduce-scatter and all-reduce
//   (pull + sum), and the slot reduction that finishes the fused GEMM -> reduce-scatter.
//
// The reference has no communication layer at all (it scales by independent instances,
// serving/src/fastdeploy_runtime.cc); this file has no counterpart there.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "fdb_common.h"

namespace fdb {

constexpr int kMaxPeers = 8;
constexpr long long kPeerWaitClocks = 2000000000LL;   // about one second at 1.9 GHz
constexpr int kStatusTimeoutPeerCode = 4;

// Device barriers and the fused peer-mode GEMMs take their epoch as a launch parameter that the host
// increments per launch, so these launches must not be captured into a CUDA graph (a replay would wait
// for an epoch that has already passed): the Python layer launches them eagerly.
struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spins until *flag >= target or the budget runs out (then the status word gets the peer code).
// A status word that already holds an error ends the wait at once: after one lost peer every later wait
// of the queued forward would otherwise spin for its whole budget on data that will never come.
__device__ __forceinline__ bool wait_ge(const unsigned* flag, unsigned target, int* status) {
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    if (static_cast<int>(ld_acquire_sys(flag) - target) >= 0) return true;
    if ((it & 63u) == 63u) {
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
      if (clock64() - t0 > kPeerWaitClocks) {
        if (status != nullptr) atomicExch(status, kStatusTimeoutPeerCode);
        return false;
      }
      __nanosleep(200);
    }
  }
}

// ------------------------------------------------------------------ barrier
// flags[r] on every rank counts arrivals of rank r. Each rank bumps its slot on all peers, then waits
// until all slots of its own array reach the epoch.
__global__ void comm_barrier_kernel(PeerPtrs flags, int world, int rank, unsigned epoch, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    red_release_sys_add(static_cast<unsigned*>(flags.p[t]) + rank, 1u);
    wait_ge(static_cast<const unsigned*>(flags.p[rank]) + t, epoch, status);
  }
}

// ------------------------------------------------------------------ pull collectives (16-bit or fp32 payloads)
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// out[r * count + i] = src_r[i] for every rank r (16-byte vectors; count * sizeof(T) % 16 == 0)
__global__ void allgather_pull_kernel(PeerPtrs src, uint4* out, long long vecs_per_rank, int world, int rank) {
  const long long total = vecs_per_rank * world;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    // start with the next rank so that the ranks do not all read the same peer at once
    const int step = static_cast<int>(i / vecs_per_rank);
    const int r = (rank + 1 + step) % world;
    const long long k = i - step * vecs_per_rank;
    out[r * vecs_per_rank + k] = static_cast<const uint4*>(src.p[r])[k];
  }
}

// out[i] = sum_r src_r[offset + i], i < count: reduce-scatter with offset = rank * count, all-reduce with
// offset = 0 and count = everything. Eight 16-bit (or four fp32) elements per thread step.
template <typename T>
__global__ void reduce_pull_kernel(PeerPtrs src, T* out, long long offset, long long count, int world, int rank) {
  constexpr int kVec = 16 / sizeof(T);
  const long long vecs = count / kVec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) acc[j] = 0.f;
    for (int s = 0; s < world; ++s) {
      const int r = (rank + s) % world;
      const uint4 v = reinterpret_cast<const uint4*>(static_cast<const T*>(src.p[r]) + offset)[i];
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) acc[j] += to_f<T>(e[j]);
    }
    uint4 o;
    T* e = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < kVec; ++j) e[j] = from_f<T>(acc[j]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// ------------------------------------------------------------------ slot reduction of the fused GEMM -> reduce-scatter
// slots: [world][rows][ld] partial results written by the ranks' GEMM epilogues into this rank's heap;
// counters[b] counts the stores that have landed for 128-row block b. One CTA per (row block, column
// chunk) waits for its block, then sums the world slots in fp32, adds the bias and writes the output.
template <typename T>
__global__ void __launch_bounds__(256) slot_reduce_kernel(const T* slots, const unsigned* counters, unsigned target,
                                                          T* out, const float* bias, int rows, int cols, int ld,
                                                          int out_ld, int world, int* status,
                                                          const T* residual, int res_ld) {
  __shared__ int ok;
  const int blk = blockIdx.x;
  if (threadIdx.x == 0) ok = wait_ge(counters + blk, target, status) ? 1 : 0;
  __syncthreads();
  if (!ok) return;
  constexpr int kVec = 16 / sizeof(T);
  const int row0 = blk * 128;
  const int nrow = min(128, rows - row0);
  const int vec_cols = cols / kVec;
  const int chunk = blockIdx.y, chunks = gridDim.y;
  for (int idx = threadIdx.x + chunk * blockDim.x; idx < nrow * vec_cols; idx += blockDim.x * chunks) {
    const int r = idx / vec_cols, c = (idx - r * vec_cols) * kVec;
    float acc[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) acc[j] = bias != nullptr ? bias[c + j] : 0.f;
    if (residual != nullptr) {   // may alias out: each element is read and written by the same thread
      const uint4 v = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row0 + r) * res_ld + c);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) acc[j] += to_f<T>(e[j]);
    }
    for (int s = 0; s < world; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(slots + (static_cast<size_t>(s) * rows + row0 + r) * ld + c);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) acc[j] += to_f<T>(e[j]);
    }
    uint4 o;
    T* e = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < kVec; ++j) e[j] = from_f<T>(acc[j]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(row0 + r) * out_ld + c) = o;
  }
}


// Slot reduction fused with the residual addition and the LayerNorm that follows it in a pre-norm transformer
// block: x = x + bias + sum of the world partial blocks (written back in place), y = LayerNorm(x) * gamma + beta.
// One warp per row keeps the whole row (cols <= 2048) in registers, so x is read once and the normalised row
// leaves in the same pass. Two CTAs share each 128-row block (64 rows each) and both wait for its counter.
__device__ __forceinline__ void ld8f(const float* p, float (&f)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// OUT8: y is e4m3 (one byte per element, y_ld in bytes), the normalised row is multiplied by out_scale first.
// The partial results come from `src`: src.p[s] is the first of this rank's rows in rank s's buffer - slots in
// this rank's own memory for the push form of the reduce-scatter, or the peers' own result buffers, read
// straight over NVLink, for the pull form (every load of a row chunk is issued before the first use, so a
// thread keeps WORLD 16-byte peer loads in flight per chunk and a CTA well over 100 KB).
template <typename T, int WORLD, bool OUT8>
__global__ void __launch_bounds__(256) slot_reduce_ln_kernel(PeerPtrs src, const unsigned* counters, unsigned target,
                                                             T* x, const float* bias, int rows, int cols,
                                                             int* status, const float* gamma, const float* beta,
                                                             float eps, void* y_, int y_ld, float out_scale) {
  T* y = static_cast<T*>(y_);
  __shared__ int ok;
  const int blk = blockIdx.x >> 2;                 // four CTAs share a 128-row block, 32 rows each
  if (threadIdx.x == 0) ok = wait_ge(counters + blk, target, status) ? 1 : 0;
  __syncthreads();
  if (!ok) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row_lo = blk * 128 + (blockIdx.x & 3) * 32;
  const int row_hi = min(rows, row_lo + 32);
  for (int row = row_lo + warp; row < row_hi; row += 8) {
    float v[8][8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = lane * 8 + k * 256;
      if (c < cols) {
        // every load of this chunk is issued before the first use
        uint4 raw[WORLD + 1];
        raw[0] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * cols + c);
#pragma unroll
        for (int s = 0; s < WORLD; ++s)
          raw[s + 1] = *reinterpret_cast<const uint4*>(static_cast<const T*>(src.p[s]) + static_cast<size_t>(row) * cols + c);
        float bv[8];
        if (bias != nullptr) ld8f(bias + c, bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] = bias != nullptr ? bv[j] : 0.f;
#pragma unroll
        for (int s = 0; s <= WORLD; ++s) {
          const T* e = reinterpret_cast<const T*>(&raw[s]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[k][j] += to_f<T>(e[j]);
        }
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) { oe[j] = from_f<T>(v[k][j]); v[k][j] = to_f<T>(oe[j]); }   // normalise what was stored
        *reinterpret_cast<uint4*>(x + static_cast<size_t>(row) * cols + c) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] = 0.f;
      }
    }
    float s1 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) s1 += v[k][j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    const float mean = s1 / cols;
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (lane * 8 + k * 256 < cols) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[k][j] - mean; s2 += d * d; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    const float rstd = rsqrtf(s2 / cols + eps);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = lane * 8 + k * 256;
      if (c < cols) {
        float g[8], bt[8];
        ld8f(gamma + c, g);
        ld8f(beta + c, bt);
        if (OUT8) {
          uint32_t w[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float t[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) t[j] = ((v[k][4 * h + j] - mean) * rstd * g[4 * h + j] + bt[4 * h + j]) * out_scale;
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(t[0], t[1]), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(t[2], t[3]), __NV_SATFINITE, __NV_E4M3);
            w[h] = lo | (hi << 16);
          }
          *reinterpret_cast<uint2*>(static_cast<uint8_t*>(y_) + static_cast<size_t>(row) * y_ld + c) = make_uint2(w[0], w[1]);
        } else {
          uint4 o;
          T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
          for (int j = 0; j < 8; ++j) oe[j] = from_f<T>((v[k][j] - mean) * rstd * g[j] + bt[j]);
          *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * y_ld + c) = o;
        }
      }
    }
  }
}

}  // namespace fdb

using namespace fdb;

// ------------------------------------------------------------------ heap + IPC
FDB_API void* fdb_comm_alloc(long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) { set_error("comm: cudaMalloc failed"); return nullptr; }
  cudaMemset(p, 0, static_cast<size_t>(bytes));
  return p;
}
FDB_API int fdb_comm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
FDB_API int fdb_comm_ipc_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { set_error("comm: cudaIpcGetMemHandle failed"); return -1; }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return 0;
}
FDB_API void* fdb_comm_ipc_open(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return nullptr; }
  return p;
}
FDB_API int fdb_comm_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

static int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
  (void)what;
  return 0;
}

FDB_API int fdb_comm_barrier(void* const* flag_ptrs, int world, int rank, unsigned epoch, int* status, void* stream) {
  if (world < 1 || world > kMaxPeers) { set_error("comm: 1..8 ranks"); return -1; }
  PeerPtrs f{};
  for (int i = 0; i < world; ++i) f.p[i] = flag_ptrs[i];
  comm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, epoch, status);
  return check_launch("barrier");
}

FDB_API int fdb_comm_allgather(void* const* src_ptrs, void* out, long long bytes_per_rank, int world, int rank,
                               void* stream) {
  if (world < 1 || world > kMaxPeers || bytes_per_rank % 16 != 0) { set_error("comm: all-gather needs 16-byte multiples"); return -1; }
  PeerPtrs s{};
  for (int i = 0; i < world; ++i) s.p[i] = src_ptrs[i];
  const long long vecs = bytes_per_rank / 16;
  const int grid = static_cast<int>(std::min<long long>((vecs * world + 255) / 256, 4 * sm_count()));
  allgather_pull_kernel<<<std::max(grid, 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(s, static_cast<uint4*>(out), vecs,
                                                                                       world, rank);
  return check_launch("allgather");
}

// dtype: kF16 | kBF16 | kF32; out[i] = sum over ranks of src_r[offset + i]
FDB_API int fdb_comm_reduce(void* const* src_ptrs, void* out, long long offset, long long count, int dtype, int world,
                            int rank, void* stream) {
  const int es = dtype == kF32 ? 4 : 2;
  if (world < 1 || world > kMaxPeers || (count * es) % 16 != 0 || (offset * es) % 16 != 0) {
    set_error("comm: reduce needs 16-byte multiples"); return -1;
  }
  PeerPtrs s{};
  for (int i = 0; i < world; ++i) s.p[i] = src_ptrs[i];
  const long long vecs = count * es / 16;
  const int grid = std::max(1, static_cast<int>(std::min<long long>((vecs + 255) / 256, 4 * sm_count())));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == kF32) reduce_pull_kernel<float><<<grid, 256, 0, st>>>(s, static_cast<float*>(out), offset, count, world, rank);
  else if (dtype == kBF16) reduce_pull_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(s, static_cast<__nv_bfloat16*>(out), offset, count, world, rank);
  else reduce_pull_kernel<__half><<<grid, 256, 0, st>>>(s, static_cast<__half*>(out), offset, count, world, rank);
  return check_launch("reduce");
}

// out = sum over slots + bias + residual (bias and residual optional; residual may be the same buffer as out).
FDB_API int fdb_comm_slot_reduce_res(const void* slots, const unsigned* counters, unsigned target, void* out,
                                     const float* bias, const void* residual, int res_ld, int rows, int cols, int ld,
                                     int out_ld, int world, int dtype, int* status, void* stream) {
  if (cols % 8 != 0 || ld % 8 != 0 || out_ld % 8 != 0 || (residual != nullptr && res_ld % 8 != 0)) { set_error("comm: slot reduce needs 8-element multiples"); return -1; }
  const dim3 grid((rows + 127) / 128, std::max(1, std::min(8, cols / 256)));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    slot_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(slots), counters, target,
                                                           static_cast<__nv_bfloat16*>(out), bias, rows, cols, ld, out_ld, world, status,
                                                           static_cast<const __nv_bfloat16*>(residual), res_ld);
  else if (dtype == kF16)
    slot_reduce_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(slots), counters, target,
                                                    static_cast<__half*>(out), bias, rows, cols, ld, out_ld, world, status,
                                                    static_cast<const __half*>(residual), res_ld);
  else { set_error("comm: slot reduce takes fp16 or bf16"); return -1; }
  return check_launch("slot_reduce");
}

FDB_API int fdb_comm_slot_reduce(const void* slots, const unsigned* counters, unsigned target, void* out,
                                 const float* bias, int rows, int cols, int ld, int out_ld, int world, int dtype,
                                 int* status, void* stream) {
  return fdb_comm_slot_reduce_res(slots, counters, target, out, bias, nullptr, 0, rows, cols, ld, out_ld, world, dtype,
                                  status, stream);
}

// x [rows, cols] += bias + sum of slots [world, rows, cols]; y [rows, y_ld] = LayerNorm(x) * gamma + beta.
// out_fp8 != 0: y is e4m3 with row pitch y_ld bytes, the normalised rows are scaled by out_scale first.
FDB_API int fdb_comm_slot_reduce_ln(const void* slots, const unsigned* counters, unsigned target, void* x,
                                    const float* bias, int rows, int cols, int world, int dtype, int* status,
                                    const float* gamma, const float* beta, float eps, void* y, int y_ld, void* stream,
                                    int out_fp8, float out_scale) {
  if (cols % 8 != 0 || cols > 2048 || y_ld % 8 != 0 || gamma == nullptr || beta == nullptr) {
    set_error("comm: fused slot reduce + LayerNorm needs cols a multiple of 8 up to 2048, gamma and beta"); return -1;
  }
  auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  if (!al16(gamma) || !al16(beta) || (bias != nullptr && !al16(bias))) { set_error("comm: bias, gamma and beta must be 16-byte aligned"); return -1; }
  const int grid = 4 * ((rows + 127) / 128);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PeerPtrs src{};
  for (int s2 = 0; s2 < world && s2 < kMaxPeers; ++s2)
    src.p[s2] = const_cast<uint8_t*>(static_cast<const uint8_t*>(slots)) + static_cast<size_t>(s2) * rows * cols * 2;
#define FDB_SRLN(T, W)                                                                                              \
  if (out_fp8)                                                                                                      \
    slot_reduce_ln_kernel<T, W, true><<<grid, 256, 0, st>>>(src, counters, target, static_cast<T*>(x),              \
                                                            bias, rows, cols, status, gamma, beta, eps, y, y_ld, out_scale);     \
  else                                                                                                              \
    slot_reduce_ln_kernel<T, W, false><<<grid, 256, 0, st>>>(src, counters, target, static_cast<T*>(x),             \
                                                             bias, rows, cols, status, gamma, beta, eps, y, y_ld, 1.f)
#define FDB_SRLN_W(T)                                              \
  switch (world) {                                                 \
    case 1: FDB_SRLN(T, 1); break;                                 \
    case 2: FDB_SRLN(T, 2); break;                                 \
    case 4: FDB_SRLN(T, 4); break;                                 \
    case 8: FDB_SRLN(T, 8); break;                                 \
    default: set_error("comm: fused slot reduce + LayerNorm takes 1, 2, 4 or 8 ranks"); return -1; \
  }
  if (dtype == kBF16) { FDB_SRLN_W(__nv_bfloat16) }
  else if (dtype == kF16) { FDB_SRLN_W(__half) }
  else { set_error("comm: slot reduce takes fp16 or bf16"); return -1; }
#undef FDB_SRLN_W
#undef FDB_SRLN
  return check_launch("slot_reduce_ln");
}

// Pull form: part_ptrs[s] points at this rank's rows inside rank s's partial-result buffer ([rows][cols], peer
// memory for s != this rank). Everything else as fdb_comm_slot_reduce_ln.
FDB_API int fdb_comm_slot_reduce_ln_pull(void* const* part_ptrs, const unsigned* counters, unsigned target, void* x,
                                         const float* bias, int rows, int cols, int world, int dtype, int* status,
                                         const float* gamma, const float* beta, float eps, void* y, int y_ld,
                                         void* stream, int out_fp8, float out_scale) {
  if (cols % 8 != 0 || cols > 2048 || y_ld % 8 != 0 || gamma == nullptr || beta == nullptr) {
    set_error("comm: fused slot reduce + LayerNorm needs cols a multiple of 8 up to 2048, gamma and beta"); return -1;
  }
  auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  if (!al16(gamma) || !al16(beta) || (bias != nullptr && !al16(bias))) { set_error("comm: bias, gamma and beta must be 16-byte aligned"); return -1; }
  PeerPtrs src{};
  for (int s2 = 0; s2 < world && s2 < kMaxPeers; ++s2) {
    if (part_ptrs[s2] == nullptr || !al16(part_ptrs[s2])) { set_error("comm: partial-result pointers must be set and 16-byte aligned"); return -1; }
    src.p[s2] = part_ptrs[s2];
  }
  const int grid = 4 * ((rows + 127) / 128);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FDB_SRLN(T, W)                                                                                              \
  if (out_fp8)                                                                                                      \
    slot_reduce_ln_kernel<T, W, true><<<grid, 256, 0, st>>>(src, counters, target, static_cast<T*>(x),              \
                                                            bias, rows, cols, status, gamma, beta, eps, y, y_ld, out_scale);     \
  else                                                                                                              \
    slot_reduce_ln_kernel<T, W, false><<<grid, 256, 0, st>>>(src, counters, target, static_cast<T*>(x),             \
                                                             bias, rows, cols, status, gamma, beta, eps, y, y_ld, 1.f)
#define FDB_SRLN_W(T)                                              \
  switch (world) {                                                 \
    case 1: FDB_SRLN(T, 1); break;                                 \
    case 2: FDB_SRLN(T, 2); break;                                 \
    case 4: FDB_SRLN(T, 4); break;                                 \
    case 8: FDB_SRLN(T, 8); break;                                 \
    default: set_error("comm: fused slot reduce + LayerNorm takes 1, 2, 4 or 8 ranks"); return -1; \
  }
  if (dtype == kBF16) { FDB_SRLN_W(__nv_bfloat16) }
  else if (dtype == kF16) { FDB_SRLN_W(__half) }
  else { set_error("comm: slot reduce takes fp16 or bf16"); return -1; }
#undef FDB_SRLN_W
#undef FDB_SRLN
  return check_launch("slot_reduce_ln_pull");
}
