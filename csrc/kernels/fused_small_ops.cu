// Small fused kernels around the convolutions of detection / classification networks:
//
//  * gap_partial_v2: per-split channel sums of an NHWC tensor with four 16-byte loads in flight per
//    thread and enough blocks to fill the machine (the pooled tensor of an effective-squeeze-excite
//    block is often larger than L2, so this is a pure bandwidth kernel);
//  * ese_gate: finishes the average, multiplies by the 1x1 "excite" weights, adds the bias and
//    applies the gate activation - the three launches (finalise, a 1-row GEMM, activation) that a
//    squeeze-excite block otherwise costs collapse into one;
//  * spp_maxpool: the stride-1 max pools of a spatial-pyramid-pooling block (kernel sizes 5 / 9 / 13
//    or any odd sizes) from ONE read of the input: the image tile sits in shared memory, row maxima
//    then column maxima (max pooling is separable), each result written to its own destination
//    (normally channel slices of the concatenated buffer).
//
// The reference gets all of this from TensorRT / Paddle Inference (trt_backend.cc:347 enqueueV2); its
// own pooling kernel is the adaptive pool of runtime/backends/common/cuda/adaptive_pool2d_kernel.cu:20-59.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <functional>

#include "fdb_common.h"

namespace fdb {

struct FusedDesc {
  void* p[8];
  long long i[24];
  float f[8];
};

struct FusedOp : Op {
  std::function<int(cudaStream_t)> fn;
  int launch(cudaStream_t s) override { return fn(s); }
};

#define FDB_FUSED_CHECK()                               \
  do {                                                  \
    cudaError_t e_ = cudaGetLastError();                \
    if (e_ != cudaSuccess) {                            \
      set_error(cudaGetErrorString(e_));                \
      return -1;                                        \
    }                                                   \
    return 0;                                           \
  } while (0)

template <bool BF16>
__device__ __forceinline__ void unpack8f(const uint4& u, float (&f)[8]) {
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

__device__ __forceinline__ float gate_act(float x, int act, float alpha, float beta) {
  switch (act) {
    case kActRelu: return fmaxf(x, 0.f);
    case kActSilu: return __fdividef(x, 1.f + __expf(-x));
    case kActHardSwish: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) * (1.f / 6.f);
    case kActHardSigmoid: return fminf(fmaxf(alpha * x + beta, 0.f), 1.f);
    case kActSigmoid: return __fdividef(1.f, 1.f + __expf(-x));
    case kActRelu6: return fminf(fmaxf(x, 0.f), 6.f);
    case kActLeakyRelu: return x > 0.f ? x : alpha * x;
    case kActTanh: return tanhf(x);
    default: return x;
  }
}

// ---- channel sums per pixel split ---------------------------------------------------------------
// part[n][split][c] = sum over the split's pixels of x[n][p][c]. One block: one image, one split, 64
// channels; 256 threads = 8 channel groups x 32 pixel lanes, four pixels in flight per lane.
template <bool BF16>
__global__ void __launch_bounds__(256) gap_partial_v2_kernel(const uint8_t* __restrict__ x, float* __restrict__ part,
                                                             int HW, int C, int x_ld, int S, long long x_n_stride) {
  const int n = blockIdx.y, split = blockIdx.z;
  const int cg = threadIdx.x & 7, pl = threadIdx.x >> 3;
  const int c0 = (blockIdx.x * 8 + cg) * 8;
  const int per = (HW + S - 1) / S;
  const int p_begin = split * per, p_end = min(HW, p_begin + per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < C) {
    const uint8_t* base = x + (static_cast<size_t>(n) * x_n_stride + c0) * 2;
    const size_t pitch = static_cast<size_t>(x_ld) * 2;
    int p = p_begin + pl;
    for (; p + 96 < p_end; p += 128) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(base + p * pitch));
      const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(base + (p + 32) * pitch));
      const uint4 u2 = __ldg(reinterpret_cast<const uint4*>(base + (p + 64) * pitch));
      const uint4 u3 = __ldg(reinterpret_cast<const uint4*>(base + (p + 96) * pitch));
      float f0[8], f1[8], f2[8], f3[8];
      unpack8f<BF16>(u0, f0); unpack8f<BF16>(u1, f1); unpack8f<BF16>(u2, f2); unpack8f<BF16>(u3, f3);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += (f0[j] + f1[j]) + (f2[j] + f3[j]);
    }
    for (; p < p_end; p += 32) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(base + p * pitch));
      float f[8];
      unpack8f<BF16>(u, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
  __shared__ float red[32][8][9];
#pragma unroll
  for (int j = 0; j < 8; ++j) red[pl][cg][j] = acc[j];
  __syncthreads();
  if (threadIdx.x < 64) {
    const int g = threadIdx.x >> 3, j = threadIdx.x & 7;
    float s = 0.f;
#pragma unroll 8
    for (int l = 0; l < 32; ++l) s += red[l][g][j];
    const int c = (blockIdx.x * 8 + g) * 8 + j;
    if (c < C) part[(static_cast<size_t>(n) * S + split) * C + c] = s;
  }
}

// ---- squeeze-excite gate ------------------------------------------------------------------------
// gate[n][co] = act(bias[co] + sum_ci W[co][ci] * mean[n][ci]),  mean[n][ci] = scale * sum_s part[n][s][ci].
// Block (co chunk of 64, image n): the means of the image go to shared memory once, then each of the
// 8 warps produces 8 outputs with 16-byte weight loads and a shuffle reduction.
template <bool BF16>
__global__ void __launch_bounds__(256) ese_gate_kernel(const float* __restrict__ part, const uint8_t* __restrict__ W,
                                                       const float* __restrict__ bias, float* __restrict__ out,
                                                       int Cin, int Cout, int S, int w_ld, int out_ld, float scale,
                                                       int act, float alpha, float beta) {
  extern __shared__ float v[];
  const int n = blockIdx.y;
  const float* pn = part + static_cast<size_t>(n) * S * Cin;
  for (int ci = threadIdx.x; ci < Cin; ci += 256) {
    float s = 0.f;
    for (int k = 0; k < S; ++k) s += pn[static_cast<size_t>(k) * Cin + ci];
    v[ci] = s * scale;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int j = 0; j < 8; ++j) {
    const int co = blockIdx.x * 64 + warp * 8 + j;
    if (co >= Cout) break;
    const uint8_t* wr = W + static_cast<size_t>(co) * w_ld * 2;
    float s = 0.f;
    for (int c = lane * 8; c < Cin; c += 256) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(wr + c * 2));
      float f[8];
      unpack8f<BF16>(u, f);
      const float4 a0 = *reinterpret_cast<const float4*>(v + c);
      const float4 a1 = *reinterpret_cast<const float4*>(v + c + 4);
      s += f[0] * a0.x + f[1] * a0.y + f[2] * a0.z + f[3] * a0.w + f[4] * a1.x + f[5] * a1.y + f[6] * a1.z + f[7] * a1.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[static_cast<size_t>(n) * out_ld + co] = gate_act(s + (bias != nullptr ? bias[co] : 0.f), act, alpha, beta);
  }
}

// ---- several stride-1 max pools of one input ----------------------------------------------------
// Block: one image, kSppCg channel groups (8 channels each). The H x W tile and the row maxima of
// every kernel size live in shared memory as packed 16-bit pairs; max is exact in the storage type.
constexpr int kSppMaxK = 3;
struct SppParams {
  const uint8_t* x;
  uint8_t* y[kSppMaxK];
  int y_ld[kSppMaxK];
  long long y_n_stride[kSppMaxK];
  int radius[kSppMaxK];
  int nk;
  int H, W, C8, x_ld, cg_per_block;
  long long x_n_stride;
};

template <bool BF16>
__device__ __forceinline__ uint4 max8(const uint4& a, const uint4& b) {
  uint4 r;
  if (BF16) {
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r.x) : "r"(a.x), "r"(b.x));
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r.y) : "r"(a.y), "r"(b.y));
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r.z) : "r"(a.z), "r"(b.z));
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r.w) : "r"(a.w), "r"(b.w));
  } else {
    asm("max.f16x2 %0, %1, %2;" : "=r"(r.x) : "r"(a.x), "r"(b.x));
    asm("max.f16x2 %0, %1, %2;" : "=r"(r.y) : "r"(a.y), "r"(b.y));
    asm("max.f16x2 %0, %1, %2;" : "=r"(r.z) : "r"(a.z), "r"(b.z));
    asm("max.f16x2 %0, %1, %2;" : "=r"(r.w) : "r"(a.w), "r"(b.w));
  }
  return r;
}

template <bool BF16>
__global__ void __launch_bounds__(256) spp_maxpool_kernel(const SppParams p) {
  extern __shared__ __align__(16) uint8_t spp_smem[];
  const int n = blockIdx.y;
  const int cg0 = blockIdx.x * p.cg_per_block;
  const int ncg = min(p.cg_per_block, p.C8 - cg0);
  const int HW = p.H * p.W;
  const int items = HW * ncg;
  uint4* tile = reinterpret_cast<uint4*>(spp_smem);                 // [HW][ncg]
  uint4* rows = tile + static_cast<size_t>(HW) * p.cg_per_block;    // [nk][HW][ncg]
  const uint8_t* xn = p.x + static_cast<size_t>(n) * p.x_n_stride * 2;
  for (int it = threadIdx.x; it < items; it += 256) {
    const int px = it / ncg, g = it - px * ncg;
    tile[it] = __ldg(reinterpret_cast<const uint4*>(xn + (static_cast<size_t>(px) * p.x_ld + (cg0 + g) * 8) * 2));
  }
  __syncthreads();
  // row maxima: windows grow with the radius, so each size extends the previous one
  for (int it = threadIdx.x; it < items; it += 256) {
    const int px = it / ncg, g = it - px * ncg;
    const int h = px / p.W, w = px - h * p.W;
    uint4 m = tile[it];
    int done = 0;
    for (int k = 0; k < p.nk; ++k) {
      const int r = p.radius[k];
      for (int d = done + 1; d <= r; ++d) {
        if (w - d >= 0) m = max8<BF16>(m, tile[(px - d) * ncg + g]);
        if (w + d < p.W) m = max8<BF16>(m, tile[(px + d) * ncg + g]);
      }
      done = r;
      rows[(static_cast<size_t>(k) * HW + px) * ncg + g] = m;
    }
  }
  __syncthreads();
  for (int it = threadIdx.x; it < items; it += 256) {
    const int px = it / ncg, g = it - px * ncg;
    const int h = px / p.W;
    for (int k = 0; k < p.nk; ++k) {
      const int r = p.radius[k];
      const uint4* rk = rows + static_cast<size_t>(k) * HW * ncg;
      uint4 m = rk[it];
      for (int d = 1; d <= r; ++d) {
        if (h - d >= 0) m = max8<BF16>(m, rk[(px - d * p.W) * ncg + g]);
        if (h + d < p.H) m = max8<BF16>(m, rk[(px + d * p.W) * ncg + g]);
      }
      *reinterpret_cast<uint4*>(p.y[k] + (static_cast<size_t>(n) * p.y_n_stride[k] + static_cast<size_t>(px) * p.y_ld[k] +
                                          (cg0 + g) * 8) * 2) = m;
    }
  }
}

// ---- per-image weights: Wn[n][co][k] = W[co][k] * (gate[n][k] (+ 1)) ------------------------------
// Folds a channel gate (squeeze-excite) that multiplies the INPUT of a 1x1 convolution into that
// convolution's weights: conv(x * g) = conv_{W diag(g)}(x). The scaled feature map is then never
// written or read. 16-byte vectors of 8 input channels; columns past Cin are copied (zero padding).
template <bool BF16>
__global__ void __launch_bounds__(256) scale_weights_kernel(const uint8_t* __restrict__ W, const float* __restrict__ gate,
                                                            uint8_t* __restrict__ out, long long total, int Cout, int K8,
                                                            int Cin, int gate_ld, float plus) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int kg = static_cast<int>(idx % K8);
    const long long t = idx / K8;
    const int co = static_cast<int>(t % Cout);
    const int n = static_cast<int>(t / Cout);
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(W + (static_cast<size_t>(co) * K8 + kg) * 16));
    float f[8];
    unpack8f<BF16>(u, f);
    const int k0 = kg * 8;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g0 = k0 + 2 * j < Cin ? gate[static_cast<size_t>(n) * gate_ld + k0 + 2 * j] + plus : 1.f;
      const float g1 = k0 + 2 * j + 1 < Cin ? gate[static_cast<size_t>(n) * gate_ld + k0 + 2 * j + 1] + plus : 1.f;
      if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j] * g0, f[2 * j + 1] * g1);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(f[2 * j] * g0, f[2 * j + 1] * g1);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(out + ((static_cast<size_t>(n) * Cout + co) * K8 + kg) * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---- static quantisation to e4m3: y[r][c] = e4m3(x[r][c] * scale) ----------------------------------
// 16-bit rows in, byte rows out (8 elements per thread step). Used where a GEMM's fp8 input comes from a
// kernel that cannot quantise in its own epilogue (the attention output in front of the projection).
template <bool BF16>
__global__ void __launch_bounds__(256) quantize_e4m3_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y,
                                                            long long total, int C8, int x_ld, int y_ld, float scale) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx % C8);
    const long long r = idx / C8;
    float f[8];
    unpack8f<BF16>(__ldg(reinterpret_cast<const uint4*>(x + (r * x_ld + cg * 8) * 2)), f);
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h] * scale, f[4 * h + 1] * scale), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h + 2] * scale, f[4 * h + 3] * scale), __NV_SATFINITE, __NV_E4M3);
      w[h] = lo | (hi << 16);
    }
    *reinterpret_cast<uint2*>(y + r * y_ld + cg * 8) = make_uint2(w[0], w[1]);
  }
}

// Dynamic per-row (per-token) quantisation: one warp per row finds the row's absolute maximum, maps it onto 448 and
// writes e4m3 plus the fp32 scale the consuming GEMM multiplies back in its epilogue. Columns C..CP-1 (the padding up
// to the GEMM's K block) are written as zeros. The row is read twice; the second read hits L1 / L2.
template <bool BF16>
__global__ void __launch_bounds__(256) quantize_rows_e4m3_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y,
                                                                 float* __restrict__ scales, long long rows, int C8,
                                                                 int CP8, int x_ld, int y_ld) {
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  float amax = 0.f;
  for (int cg = lane; cg < C8; cg += 32) {
    float f[8];
    unpack8f<BF16>(__ldg(reinterpret_cast<const uint4*>(x + (r * x_ld + cg * 8) * 2)), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-12f);
  const float inv = 448.f / amax;
  if (lane == 0) scales[r] = amax / 448.f;
  for (int cg = lane; cg < CP8; cg += 32) {
    uint32_t w[2] = {0u, 0u};
    if (cg < C8) {
      float f[8];
      unpack8f<BF16>(__ldg(reinterpret_cast<const uint4*>(x + (r * x_ld + cg * 8) * 2)), f);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h] * inv, f[4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h + 2] * inv, f[4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        w[h] = lo | (hi << 16);
      }
    }
    *reinterpret_cast<uint2*>(y + r * y_ld + cg * 8) = make_uint2(w[0], w[1]);
  }
}

}  // namespace fdb

using namespace fdb;

// kind 0  gap_partial_v2 : p0 x, p1 part;  i0 N, i1 HW, i2 C, i3 x_ld, i4 S, i5 bf16, i6 x_n_stride
// kind 1  ese_gate       : p0 part, p1 W (16-bit [Cout][w_ld]), p2 bias fp32 or null, p3 out fp32 [N][out_ld];
//                          i0 N, i1 Cin, i2 Cout, i3 S, i4 w_ld, i5 out_ld, i6 act, i7 bf16; f0 scale, f1 alpha, f2 beta
// kind 2  spp_maxpool    : p0 x, p1..p3 outputs; i0 N, i1 H, i2 W, i3 C, i4 x_ld, i5 x_n_stride, i6 bf16, i7 nk,
//                          i8+3k kernel size, i9+3k y_ld, i10+3k y_n_stride
FDB_API void* fdb_fused_create(int kind, const FusedDesc* dp) {
  const FusedDesc d = *dp;
  auto* op = new FusedOp();
  switch (kind) {
    case 0: {
      const int N = d.i[0], HW = d.i[1], C = d.i[2], x_ld = d.i[3], S = d.i[4];
      const bool bf = d.i[5] != 0;
      const long long xns = d.i[6] > 0 ? d.i[6] : static_cast<long long>(HW) * x_ld;
      if (C % 8 || x_ld % 8 || xns % 8 || S < 1 || S > 65535 || N > 65535 ||
          (reinterpret_cast<uintptr_t>(d.p[0]) & 15)) {
        set_error("gap_partial: C, ld and image stride must be multiples of 8, x 16-byte aligned"); delete op; return nullptr;
      }
      op->fn = [=](cudaStream_t s) {
        dim3 grid((C + 63) / 64, N, S);
        if (bf) gap_partial_v2_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (float*)d.p[1], HW, C, x_ld, S, xns);
        else gap_partial_v2_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (float*)d.p[1], HW, C, x_ld, S, xns);
        FDB_FUSED_CHECK();
      };
      break;
    }
    case 1: {
      const int N = d.i[0], Cin = d.i[1], Cout = d.i[2], S = d.i[3], w_ld = d.i[4], out_ld = d.i[5], act = d.i[6];
      const bool bf = d.i[7] != 0;
      const float scale = d.f[0], al = d.f[1], be = d.f[2];
      if (Cin % 8 || w_ld % 8 || Cin > 8192 || N > 65535 || (reinterpret_cast<uintptr_t>(d.p[1]) & 15)) {
        set_error("ese_gate: Cin and w_ld must be multiples of 8 (Cin <= 8192), W 16-byte aligned"); delete op; return nullptr;
      }
      op->fn = [=](cudaStream_t s) {
        dim3 grid((Cout + 63) / 64, N);
        const size_t smem = static_cast<size_t>(Cin) * 4;
        if (bf) ese_gate_kernel<true><<<grid, 256, smem, s>>>((const float*)d.p[0], (const uint8_t*)d.p[1], (const float*)d.p[2], (float*)d.p[3], Cin, Cout, S, w_ld, out_ld, scale, act, al, be);
        else ese_gate_kernel<false><<<grid, 256, smem, s>>>((const float*)d.p[0], (const uint8_t*)d.p[1], (const float*)d.p[2], (float*)d.p[3], Cin, Cout, S, w_ld, out_ld, scale, act, al, be);
        FDB_FUSED_CHECK();
      };
      break;
    }
    case 2: {
      SppParams p{};
      const int N = d.i[0];
      p.H = d.i[1]; p.W = d.i[2];
      const int C = d.i[3];
      p.x_ld = d.i[4];
      p.x_n_stride = d.i[5] > 0 ? d.i[5] : static_cast<long long>(p.H) * p.W * p.x_ld;
      const bool bf = d.i[6] != 0;
      p.nk = d.i[7];
      p.x = static_cast<const uint8_t*>(d.p[0]);
      if (p.nk < 1 || p.nk > kSppMaxK || C % 8 || p.x_ld % 8 || p.x_n_stride % 8 || N > 65535) {
        set_error("spp_maxpool: 1..3 kernels, C / ld multiples of 8"); delete op; return nullptr;
      }
      int prev = 0;
      for (int k = 0; k < p.nk; ++k) {
        const int ks = d.i[8 + 3 * k];
        if (ks % 2 == 0 || ks / 2 <= prev) { set_error("spp_maxpool: kernel sizes must be odd and increasing"); delete op; return nullptr; }
        p.radius[k] = ks / 2;
        prev = ks / 2;
        p.y[k] = static_cast<uint8_t*>(d.p[1 + k]);
        p.y_ld[k] = d.i[9 + 3 * k];
        p.y_n_stride[k] = d.i[10 + 3 * k] > 0 ? d.i[10 + 3 * k] : static_cast<long long>(p.H) * p.W * p.y_ld[k];
        if (p.y_ld[k] % 8 || p.y_n_stride[k] % 8 || (reinterpret_cast<uintptr_t>(p.y[k]) & 15)) {
          set_error("spp_maxpool: output ld / stride must be multiples of 8, pointers 16-byte aligned"); delete op; return nullptr;
        }
      }
      p.C8 = C / 8;
      // channel groups per block: as many as fit 96 KB of shared memory (tile + one row-max plane per size), at most 4
      const size_t per_cg = static_cast<size_t>(p.H) * p.W * 16 * (1 + p.nk);
      int cgb = static_cast<int>((96 * 1024) / per_cg);
      if (cgb < 1) { set_error("spp_maxpool: feature map too large for the shared-memory tile"); delete op; return nullptr; }
      cgb = cgb > 4 ? 4 : cgb;
      if (cgb > p.C8) cgb = p.C8;
      p.cg_per_block = cgb;
      const size_t smem = per_cg * cgb;
      static size_t max_smem_dev[64][2] = {};
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("spp_maxpool: no current device"); delete op; return nullptr; }
      size_t* max_smem = max_smem_dev[dev];        // the opt-in limit is per function and per device
      if (smem > 48 * 1024 && smem > max_smem[bf ? 1 : 0]) {
        cudaError_t e = bf ? cudaFuncSetAttribute(spp_maxpool_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                           : cudaFuncSetAttribute(spp_maxpool_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); delete op; return nullptr; }
        max_smem[bf ? 1 : 0] = smem;
      }
      op->fn = [=](cudaStream_t s) {
        dim3 grid((p.C8 + p.cg_per_block - 1) / p.cg_per_block, N);
        if (bf) spp_maxpool_kernel<true><<<grid, 256, smem, s>>>(p);
        else spp_maxpool_kernel<false><<<grid, 256, smem, s>>>(p);
        FDB_FUSED_CHECK();
      };
      break;
    }
    case 3: {
      // scale_weights: p0 W 16-bit [Cout][K], p1 gate fp32 [N][gate_ld], p2 out 16-bit [N][Cout][K];
      // i0 N, i1 Cout, i2 K (multiple of 8), i3 Cin (<= K), i4 gate_ld, i5 bf16; f0 added to the gate
      const int N = d.i[0], Cout = d.i[1], Kp = d.i[2], Cin = d.i[3], gld = d.i[4];
      const bool bf = d.i[5] != 0;
      const float plus = d.f[0];
      if (Kp % 8 || Cin > Kp || (reinterpret_cast<uintptr_t>(d.p[0]) & 15) || (reinterpret_cast<uintptr_t>(d.p[2]) & 15)) {
        set_error("scale_weights: K must be a multiple of 8 covering Cin, pointers 16-byte aligned"); delete op; return nullptr;
      }
      const long long total = static_cast<long long>(N) * Cout * (Kp / 8);
      op->fn = [=](cudaStream_t s) {
        const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
        if (bf) scale_weights_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1], (uint8_t*)d.p[2], total, Cout, Kp / 8, Cin, gld, plus);
        else scale_weights_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1], (uint8_t*)d.p[2], total, Cout, Kp / 8, Cin, gld, plus);
        FDB_FUSED_CHECK();
      };
      break;
    }
    case 4: {
      // quantize_e4m3: p0 x 16-bit [rows][x_ld], p1 y e4m3 [rows][y_ld]; i0 rows, i1 C, i2 x_ld, i3 y_ld, i4 bf16; f0 scale
      const long long rows = d.i[0];
      const int C = d.i[1], x_ld = d.i[2], y_ld = d.i[3];
      const bool bf = d.i[4] != 0;
      const float scale = d.f[0];
      if (C % 8 || x_ld % 8 || y_ld % 8 || (reinterpret_cast<uintptr_t>(d.p[0]) & 15) || (reinterpret_cast<uintptr_t>(d.p[1]) & 7)) {
        set_error("quantize_e4m3: C and row pitches must be multiples of 8, pointers aligned"); delete op; return nullptr;
      }
      const long long total = rows * (C / 8);
      op->fn = [=](cudaStream_t s) {
        const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
        if (bf) quantize_e4m3_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, C / 8, x_ld, y_ld, scale);
        else quantize_e4m3_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, C / 8, x_ld, y_ld, scale);
        FDB_FUSED_CHECK();
      };
      break;
    }
    case 5: {
      // quantize_rows_e4m3: p0 x 16-bit [rows][x_ld], p1 y e4m3 [rows][y_ld], p2 scales fp32 [rows];
      //                     i0 rows, i1 C, i2 x_ld, i3 y_ld, i4 bf16, i5 CP (padded row length written, >= C)
      const long long rows = d.i[0];
      const int C = d.i[1], x_ld = d.i[2], y_ld = d.i[3], CP = d.i[5] > 0 ? d.i[5] : d.i[1];
      const bool bf = d.i[4] != 0;
      if (C % 8 || CP % 8 || CP < C || CP > y_ld || x_ld % 8 || y_ld % 8 || (reinterpret_cast<uintptr_t>(d.p[0]) & 15) ||
          (reinterpret_cast<uintptr_t>(d.p[1]) & 7)) {
        set_error("quantize_rows_e4m3: C, CP and row pitches must be multiples of 8, C <= CP <= y_ld, pointers aligned");
        delete op; return nullptr;
      }
      op->fn = [=](cudaStream_t s) {
        if (rows == 0) return 0;
        const int grid = static_cast<int>((rows * 32 + 255) / 256);
        if (bf) quantize_rows_e4m3_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (float*)d.p[2], rows, C / 8, CP / 8, x_ld, y_ld);
        else quantize_rows_e4m3_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], (float*)d.p[2], rows, C / 8, CP / 8, x_ld, y_ld);
        FDB_FUSED_CHECK();
      };
      break;
    }
    default:
      set_error("fdb_fused_create: unknown kind");
      delete op;
      return nullptr;
  }
  return op;
}
