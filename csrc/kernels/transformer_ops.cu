// Row-wise kernels of the transformer path: LayerNorm, fused embedding-sum + LayerNorm,
// masked scaled softmax over attention scores, per-head transpose of V.
// The GEMMs around them (QKV / output projection / FFN and the two batched attention
// products) run on the tcgen05 kernel in conv_gemm_sm100.cu.
//
// In the reference these are whatever Paddle Inference / TensorRT pick for ERNIE and ViT
// (fastdeploy/runtime/backends/paddle/paddle_backend.cc:426 predictor_->Run()).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <functional>

#include "fdb_common.h"

namespace fdb {

struct TfDesc {
  void* p[10];
  long long i[16];
  float f[4];
};

struct TfOp : Op {
  std::function<int(cudaStream_t)> fn;
  int launch(cudaStream_t s) override { return fn(s); }
};

enum TfKind : int { kLayerNorm = 0, kEmbedLayerNorm = 1, kMaskedSoftmax = 2, kHeadTranspose = 3 };

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
template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (BF16) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

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

// ---- LayerNorm over the last dimension: one warp per row --------------------------------
// p0 x, p1 y, p2 gamma fp32 (or null), p3 beta fp32 (or null); i0 rows, i1 C, i2 x_ld, i3 y_ld, i4 bf16; f0 eps
template <bool BF16>
__global__ void layernorm_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ gamma,
                                 const float* __restrict__ beta, long long rows, int C, int x_ld, int y_ld, float eps) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint8_t* xr = x + row * x_ld * 2;
  float s = 0.f, ss = 0.f;
  for (int c = lane * 8; c < C; c += 256) {
    float f[8];
    unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(xr + c * 2)), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j];
  }
  const float mean = warp_sum(s) / C;
  for (int c = lane * 8; c < C; c += 256) {
    float f[8];
    unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(xr + c * 2)), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float d = f[j] - mean; ss += d * d; }
  }
  const float rstd = rsqrtf(warp_sum(ss) / C + eps);
  uint8_t* yr = y + row * y_ld * 2;
  for (int c = lane * 8; c < C; c += 256) {
    float f[8];
    unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(xr + c * 2)), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = (f[j] - mean) * rstd;
      if (gamma) v *= gamma[c + j];
      if (beta) v += beta[c + j];
      f[j] = v;
    }
    *reinterpret_cast<uint4*>(yr + c * 2) = pack8<BF16>(f);
  }
}

// ---- LayerNorm with the row held in registers (C <= 2048): every load of the row is in flight before the
// first use, the row is read from memory once, and the statistics take two register passes.
// Eight floats -> eight e4m3 bytes (saturating).
__device__ __forceinline__ uint2 pack8_e4m3(const float (&f)[8]) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h], f[4 * h + 1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h + 2], f[4 * h + 3]), __NV_SATFINITE, __NV_E4M3);
    w[h] = lo | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

// OUT8: the normalised row is multiplied by out_scale (the reciprocal of the consumer GEMM's activation
// scale) and stored as e4m3, one byte per element (y_ld counts bytes then).
// NK = 256-column chunks a lane holds (C <= NK * 256): sized to the row so that short rows keep few registers.
template <bool BF16, bool OUT8, int NK>
__global__ void __launch_bounds__(256) layernorm_reg_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y,
                                                            const float* __restrict__ gamma, const float* __restrict__ beta,
                                                            long long rows, int C, int x_ld, int y_ld, float eps,
                                                            float out_scale) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint8_t* xr = x + row * x_ld * 2;
  uint4 raw[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int c = lane * 8 + k * 256;
    raw[k] = c < C ? __ldg(reinterpret_cast<const uint4*>(xr + c * 2)) : make_uint4(0, 0, 0, 0);
  }
  float v[NK][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    unpack8<BF16>(raw[k], v[k]);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[k][j];
  }
  const float mean = warp_sum(s) / C;
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    if (lane * 8 + k * 256 < C) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = v[k][j] - mean; ss += d * d; }
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / C + eps);
  uint8_t* yr = y + row * y_ld * (OUT8 ? 1 : 2);
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int c = lane * 8 + k * 256;
    if (c < C) {
      float g[8], b[8];
      if (gamma) {
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
        g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
      }
      if (beta) {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + c)), b1 = __ldg(reinterpret_cast<const float4*>(beta + c + 4));
        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
      }
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = (v[k][j] - mean) * rstd;
        if (gamma) t *= g[j];
        if (beta) t += b[j];
        f[j] = OUT8 ? t * out_scale : t;
      }
      if (OUT8) *reinterpret_cast<uint2*>(yr + c) = pack8_e4m3(f);
      else *reinterpret_cast<uint4*>(yr + c * 2) = pack8<BF16>(f);
    }
  }
}

// ---- sum of up to 4 embedding lookups + LayerNorm: one warp per token ---------------------
// p0..p3 ids (int64 [rows]) (null = position index row % i3), p4..p7 tables (16-bit [V][C]), p8 y;
// gamma/beta fp32 are passed in a second descriptor call? No: p9 points at a fp32 block [gamma(C) | beta(C)].
// i0 rows, i1 C, i2 num tables, i3 seq_len (for implicit positions), i4 bf16, i5 y_ld, i6..i9 rows of each table
// (0 = not given); f0 eps. An id outside its table is clamped into it (a checked build also counts it).
template <bool BF16>
__global__ void embed_layernorm_kernel(const long long* const* __restrict__ ids4, const uint8_t* const* __restrict__ tabs4,
                                       uint8_t* __restrict__ y, const float* __restrict__ gb, long long rows, int C,
                                       int ntab, int seq, int y_ld, float eps, int4 table_rows) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  long long idx[4];
  const int vrows[4] = {table_rows.x, table_rows.y, table_rows.z, table_rows.w};
  for (int t = 0; t < ntab; ++t) {
    idx[t] = ids4[t] ? ids4[t][row] : (row % seq);
    if (vrows[t] > 0) {
      if (lane == 0) FDB_NOTE_OOB(2, idx[t], static_cast<long long>(vrows[t]));
      idx[t] = idx[t] < 0 ? 0 : (idx[t] >= vrows[t] ? vrows[t] - 1 : idx[t]);
    }
  }
  float s = 0.f, ss = 0.f;
  // C <= 8 * 32 * 6 = 1536 keeps the row in registers
  float v[6][8];
  int nv = 0;
  for (int c = lane * 8; c < C; c += 256, ++nv) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[nv][j] = 0.f;
    for (int t = 0; t < ntab; ++t) {
      float f[8];
      unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(tabs4[t] + (idx[t] * C + c) * 2)), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[nv][j] += f[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[nv][j];
  }
  const float mean = warp_sum(s) / C;
  for (int k = 0; k < nv; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float d = v[k][j] - mean; ss += d * d; }
  const float rstd = rsqrtf(warp_sum(ss) / C + eps);
  uint8_t* yr = y + row * y_ld * 2;
  int k = 0;
  for (int c = lane * 8; c < C; c += 256, ++k) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = (v[k][j] - mean) * rstd * gb[c + j] + gb[C + c + j];
    *reinterpret_cast<uint4*>(yr + c * 2) = pack8<BF16>(f);
  }
}

// ---- softmax(scale * s + mask) in place over attention scores: one warp per row ---------------
// scores [B][H][S][ld] 16-bit, valid columns Sk, columns [Sk, ld) are written as zero (they pad the
// K dimension of the following P.V product). mask fp32, element (b, s, k) at b*m_b + s*m_s + k (m_s may
// be 0 for a key-padding mask [B][Sk]); null = no mask.
// p0 scores, p1 mask; i0 B, i1 H, i2 S, i3 Sk, i4 ld, i5 bf16, i6 m_b, i7 m_s; f0 scale
template <bool BF16>
__global__ void masked_softmax_kernel(uint8_t* __restrict__ sc, const float* __restrict__ mask, long long rows, int H,
                                      int S, int Sk, int ld, long long m_b, long long m_s, float scale) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int s_idx = static_cast<int>(row % S);
  const long long b = row / (static_cast<long long>(S) * H);
  uint8_t* r = sc + row * ld * 2;
  const float* mrow = mask ? mask + b * m_b + s_idx * m_s : nullptr;
  // Sk <= 8 * 32 * 4 = 1024 keeps the row in registers
  float v[4][8];
  int nv = 0;
  float mx = -INFINITY;
  for (int c = lane * 8; c < ld; c += 256, ++nv) {
    unpack8<BF16>(*reinterpret_cast<const uint4*>(r + c * 2), v[nv]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = (c + j < Sk) ? v[nv][j] * scale + (mrow ? mrow[c + j] : 0.f) : -INFINITY;
      v[nv][j] = t;
      mx = fmaxf(mx, t);
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int k = 0; k < nv; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float e = v[k][j] == -INFINITY ? 0.f : __expf(v[k][j] - mx);
      v[k][j] = e;
      sum += e;
    }
  const float inv = 1.f / warp_sum(sum);
  int k = 0;
  for (int c = lane * 8; c < ld; c += 256, ++k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[k][j] *= inv;
    *reinterpret_cast<uint4*>(r + c * 2) = pack8<BF16>(v[k]);
  }
}

// ---- V [B][S][H*D] (row stride ld) -> V^T [B][H][D][Sp], zero padded to Sp ------------------------
// p0 v, p1 vt; i0 B, i1 S, i2 H, i3 D, i4 v_ld, i5 Sp
__global__ void head_transpose_kernel(const uint16_t* __restrict__ v, uint16_t* __restrict__ vt, int B, int S, int H,
                                      int D, int v_ld, int Sp) {
  __shared__ uint16_t tile[32][33];
  const int bh = blockIdx.z, b = bh / H, h = bh - b * H;
  const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int s = s0 + i, d = d0 + threadIdx.x;
    tile[i][threadIdx.x] = (s < S && d < D) ? v[(static_cast<size_t>(b) * S + s) * v_ld + h * D + d] : 0;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int d = d0 + i, s = s0 + threadIdx.x;
    if (d < D && s < Sp) vt[((static_cast<size_t>(b) * H + h) * D + d) * Sp + s] = tile[threadIdx.x][i];
  }
}

// Same transpose with 16-byte accesses on both sides: one CTA per (b, h, 64 keys). Needs D, v_ld and Sp to be
// multiples of 8 and 16-byte aligned bases.
__global__ void __launch_bounds__(256) head_transpose_vec_kernel(const uint16_t* __restrict__ v, uint16_t* __restrict__ vt,
                                                                 int B, int S, int H, int D, int v_ld, int Sp) {
  extern __shared__ uint16_t tp_tile[];          // [64][D + 2]
  const int pitch = D + 2;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int s0 = blockIdx.x * 64;
  const int dv = D / 8;
  for (int i = threadIdx.x; i < 64 * dv; i += blockDim.x) {
    const int r = i / dv, c = (i - r * dv) * 8;
    const int sidx = s0 + r;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (sidx < S) val = __ldg(reinterpret_cast<const uint4*>(v + (static_cast<size_t>(b) * S + sidx) * v_ld + h * D + c));
    uint32_t* dst = reinterpret_cast<uint32_t*>(tp_tile + r * pitch + c);     // pitch and c are even: 4-byte aligned
    dst[0] = val.x; dst[1] = val.y; dst[2] = val.z; dst[3] = val.w;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D * 8; i += blockDim.x) {
    const int sv = (i & 7) * 8, d = i >> 3;     // eight consecutive threads write one 128-byte row segment
    if (s0 + sv >= Sp) continue;
    uint16_t e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = tp_tile[(sv + j) * pitch + d];
    uint4 o;
    o.x = e[0] | (static_cast<uint32_t>(e[1]) << 16); o.y = e[2] | (static_cast<uint32_t>(e[3]) << 16);
    o.z = e[4] | (static_cast<uint32_t>(e[5]) << 16); o.w = e[6] | (static_cast<uint32_t>(e[7]) << 16);
    *reinterpret_cast<uint4*>(vt + ((static_cast<size_t>(b) * H + h) * D + d) * Sp + s0 + sv) = o;
  }
}

}  // namespace fdb
FDB_BOUNDS_TU("transformer_ops")
namespace fdb {

#define FDB_TF_CHECK()                              \
  do {                                              \
    cudaError_t _e = cudaGetLastError();            \
    if (_e != cudaSuccess) {                        \
      set_error(cudaGetErrorString(_e));            \
      return -1;                                    \
    }                                               \
    return 0;                                       \
  } while (0)

}  // namespace fdb

using namespace fdb;

FDB_API void* fdb_transformer_create(int kind, const TfDesc* dp) {
  const TfDesc d = *dp;
  auto* op = new TfOp();
  switch (kind) {
    case kLayerNorm: {
      const long long rows = d.i[0];
      const int C = d.i[1], x_ld = d.i[2], y_ld = d.i[3];
      const bool bf = d.i[4] != 0;
      const bool out8 = d.i[5] != 0;        // e4m3 output, scaled by f1
      const float eps = d.f[0], out_scale = d.f[1];
      if (C % 8 || x_ld % 8 || y_ld % 8) { set_error("layernorm: C/ld must be multiples of 8"); delete op; return nullptr; }
      if (out8 && (C > 2048 || reinterpret_cast<uintptr_t>(d.p[2]) % 16 || reinterpret_cast<uintptr_t>(d.p[3]) % 16)) {
        set_error("layernorm: the e4m3 output form needs C <= 2048 and aligned gamma / beta"); delete op; return nullptr;
      }
      op->fn = [=](cudaStream_t s) {
        const int grid = static_cast<int>((rows * 32 + 255) / 256);
        const bool regs = C <= 2048 && (reinterpret_cast<uintptr_t>(d.p[2]) % 16 == 0) && (reinterpret_cast<uintptr_t>(d.p[3]) % 16 == 0);
        if (out8 || regs) {
          const int nk = (C + 255) / 256;
#define FDB_LN_LAUNCH(NK)                                                                                              \
  do {                                                                                                                 \
    if (out8 && bf) layernorm_reg_kernel<true, true, NK><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (const float*)d.p[2], (const float*)d.p[3], rows, C, x_ld, y_ld, eps, out_scale); \
    else if (out8) layernorm_reg_kernel<false, true, NK><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (const float*)d.p[2], (const float*)d.p[3], rows, C, x_ld, y_ld, eps, out_scale); \
    else if (bf) layernorm_reg_kernel<true, false, NK><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (const float*)d.p[2], (const float*)d.p[3], rows, C, x_ld, y_ld, eps, 1.f); \
    else layernorm_reg_kernel<false, false, NK><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (const float*)d.p[2], (const float*)d.p[3], rows, C, x_ld, y_ld, eps, 1.f); \
  } while (0)
          if (nk <= 1) FDB_LN_LAUNCH(1);
          else if (nk == 2) FDB_LN_LAUNCH(2);
          else if (nk == 3) FDB_LN_LAUNCH(3);
          else if (nk == 4) FDB_LN_LAUNCH(4);
          else if (nk <= 6) FDB_LN_LAUNCH(6);
          else FDB_LN_LAUNCH(8);
#undef FDB_LN_LAUNCH
        }
        else if (bf) layernorm_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (const float*)d.p[2], (const float*)d.p[3], rows, C, x_ld, y_ld, eps);
        else layernorm_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (const float*)d.p[2], (const float*)d.p[3], rows, C, x_ld, y_ld, eps);
        FDB_TF_CHECK();
      };
      break;
    }
    case kEmbedLayerNorm: {
      // p0 = device array of 4 id pointers, p1 = device array of 4 table pointers, p2 = y, p3 = gamma|beta block
      const long long rows = d.i[0];
      const int C = d.i[1], ntab = d.i[2], seq = d.i[3], y_ld = d.i[5];
      const bool bf = d.i[4] != 0;
      const float eps = d.f[0];
      const int4 vr = make_int4(d.i[6], d.i[7], d.i[8], d.i[9]);
      if (C % 8 || C > 1536 || ntab < 1 || ntab > 4 || y_ld % 8) { set_error("embed_layernorm: C multiple of 8 and <= 1536, 1..4 tables"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        const int grid = static_cast<int>((rows * 32 + 255) / 256);
        if (bf) embed_layernorm_kernel<true><<<grid, 256, 0, s>>>((const long long* const*)d.p[0], (const uint8_t* const*)d.p[1], (uint8_t*)d.p[2], (const float*)d.p[3], rows, C, ntab, seq, y_ld, eps, vr);
        else embed_layernorm_kernel<false><<<grid, 256, 0, s>>>((const long long* const*)d.p[0], (const uint8_t* const*)d.p[1], (uint8_t*)d.p[2], (const float*)d.p[3], rows, C, ntab, seq, y_ld, eps, vr);
        FDB_TF_CHECK();
      };
      break;
    }
    case kMaskedSoftmax: {
      const int B = d.i[0], H = d.i[1], S = d.i[2], Sk = d.i[3], ld = d.i[4];
      const bool bf = d.i[5] != 0;
      const long long m_b = d.i[6], m_s = d.i[7];
      const float scale = d.f[0];
      if (ld % 8 || ld > 1024 || Sk > ld) { set_error("masked_softmax: ld multiple of 8, <= 1024, >= Sk"); delete op; return nullptr; }
      const long long rows = static_cast<long long>(B) * H * S;
      op->fn = [=](cudaStream_t s) {
        const int grid = static_cast<int>((rows * 32 + 255) / 256);
        if (bf) masked_softmax_kernel<true><<<grid, 256, 0, s>>>((uint8_t*)d.p[0], (const float*)d.p[1], rows, H, S, Sk, ld, m_b, m_s, scale);
        else masked_softmax_kernel<false><<<grid, 256, 0, s>>>((uint8_t*)d.p[0], (const float*)d.p[1], rows, H, S, Sk, ld, m_b, m_s, scale);
        FDB_TF_CHECK();
      };
      break;
    }
    case kHeadTranspose: {
      const int B = d.i[0], S = d.i[1], H = d.i[2], D = d.i[3], v_ld = d.i[4], Sp = d.i[5];
      op->fn = [=](cudaStream_t s) {
        const bool vec = D % 8 == 0 && v_ld % 8 == 0 && Sp % 8 == 0 && B * H <= 65535 &&
                         reinterpret_cast<uintptr_t>(d.p[0]) % 16 == 0 && reinterpret_cast<uintptr_t>(d.p[1]) % 16 == 0;
        if (vec) {
          head_transpose_vec_kernel<<<dim3((Sp + 63) / 64, B * H), 256, 64 * (D + 2) * 2, s>>>(
              (const uint16_t*)d.p[0], (uint16_t*)d.p[1], B, S, H, D, v_ld, Sp);
          FDB_TF_CHECK();
        }
        dim3 grid((Sp + 31) / 32, (D + 31) / 32, B * H), block(32, 8);
        head_transpose_kernel<<<grid, block, 0, s>>>((const uint16_t*)d.p[0], (uint16_t*)d.p[1], B, S, H, D, v_ld, Sp);
        FDB_TF_CHECK();
      };
      break;
    }
    default:
      set_error("fdb_transformer_create: unknown kind");
      delete op;
      return nullptr;
  }
  return op;
}
