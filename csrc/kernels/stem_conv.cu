// First-layer ("stem") convolution: 3x3, stride 2, padding 1, at most 4 real input channels
// (stored as 8-channel NHWC rows of 16 bytes) to 32 output channels, bias + activation fused.
//
// This layer is memory bound (27 multiply-adds per output value) and a poor fit for the tensor
// core pipeline, where K = 27 is padded to nine 64-wide slabs of almost only zeros. Here one
// thread produces one output pixel: it reads its 3x3 input pixels with nine 16-byte loads
// (neighbouring threads share them through L1) and keeps 32 fp32 accumulators. Weights and bias
// travel in the kernel parameter block, so after full unrolling every multiply-add takes its weight
// straight from the constant bank and no weight load is ever issued. The 64-byte output row of a
// pixel leaves as four 16-byte stores; a warp writes 2 KB of consecutive memory.
//
// The reference runs this layer inside its inference back ends (fastdeploy/runtime/backends/*),
// it has no kernel of its own for it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fdb_common.h"

namespace fdb {

constexpr int kStemCout = 32;
constexpr int kStemTaps = 9;
constexpr int kStemCin = 3;

struct StemConvDesc {
  const void* x;   // NHWC, 8 channels per pixel (16-bit), channels >= cin are ignored
  void* y;         // NHWC, 32 channels written per pixel
  int* status;
  int dtype;       // kF16 | kBF16 (input and output)
  int N, H, W, Ho, Wo;
  int x_ld, y_ld;  // elements per pixel row entry (x_ld = 8)
  long long x_n_stride, y_n_stride;   // elements between images
  int act;         // kActNone | kActRelu | kActSilu
  int cin;         // 1..3 real channels
  float w[kStemTaps * kStemCin * kStemCout];   // [kh][kw][ci][co]
  float bias[kStemCout];
};

template <bool BF16>
__device__ __forceinline__ void unpack3(const uint4& v, float& c0, float& c1, float& c2) {
  if (BF16) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    c0 = a.x; c1 = a.y; c2 = b.x;
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    c0 = a.x; c1 = a.y; c2 = b.x;
  }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <bool BF16, int ACT>
__global__ void __launch_bounds__(128) stem_conv_kernel(const __grid_constant__ StemConvDesc d) {
  const int ow = blockIdx.x * 128 + threadIdx.x;
  const int oh = blockIdx.y;
  const int n = blockIdx.z;
  if (ow >= d.Wo) return;
  float acc[kStemCout];
#pragma unroll
  for (int c = 0; c < kStemCout; ++c) acc[c] = d.bias[c];
  const uint8_t* xin = reinterpret_cast<const uint8_t*>(d.x) + static_cast<size_t>(n) * d.x_n_stride * 2;
#pragma unroll
  for (int kh = 0; kh < 3; ++kh) {
    const int ih = oh * 2 - 1 + kh;
    const bool row_ok = ih >= 0 && ih < d.H;
#pragma unroll
    for (int kw = 0; kw < 3; ++kw) {
      const int iw = ow * 2 - 1 + kw;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row_ok && iw >= 0 && iw < d.W) {
        v = __ldg(reinterpret_cast<const uint4*>(xin + (static_cast<size_t>(ih) * d.W + iw) * d.x_ld * 2));
      }
      float xc[3];
      unpack3<BF16>(v, xc[0], xc[1], xc[2]);
#pragma unroll
      for (int ci = 0; ci < kStemCin; ++ci) {
#pragma unroll
        for (int c = 0; c < kStemCout; ++c) {
          acc[c] = fmaf(xc[ci], d.w[((kh * 3 + kw) * kStemCin + ci) * kStemCout + c], acc[c]);
        }
      }
    }
  }
  uint32_t out[kStemCout / 2];
#pragma unroll
  for (int c = 0; c < kStemCout; c += 2) {
    float a = acc[c], b = acc[c + 1];
    if (ACT == kActRelu) { a = fmaxf(a, 0.f); b = fmaxf(b, 0.f); }
    if (ACT == kActSilu) {
      float ta, tb;
      asm("tanh.approx.f32 %0, %1;" : "=f"(ta) : "f"(0.5f * a));
      asm("tanh.approx.f32 %0, %1;" : "=f"(tb) : "f"(0.5f * b));
      a = fmaf(0.5f * a, ta, 0.5f * a);
      b = fmaf(0.5f * b, tb, 0.5f * b);
    }
    out[c / 2] = pack_pair<BF16>(a, b);
  }
  uint8_t* yrow = reinterpret_cast<uint8_t*>(d.y) +
                  (static_cast<size_t>(n) * d.y_n_stride + (static_cast<size_t>(oh) * d.Wo + ow) * d.y_ld) * 2;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    reinterpret_cast<uint4*>(yrow)[g] = make_uint4(out[4 * g], out[4 * g + 1], out[4 * g + 2], out[4 * g + 3]);
  }
}

struct StemConvOp : Op {
  StemConvDesc d;
  int launch(cudaStream_t s) override {
    const dim3 grid((d.Wo + 127) / 128, d.Ho, d.N);
    const bool bf16 = d.dtype == kBF16;
#define FDB_STEM_LAUNCH(B, A) stem_conv_kernel<B, A><<<grid, 128, 0, s>>>(d)
    if (bf16) {
      if (d.act == kActSilu) FDB_STEM_LAUNCH(true, kActSilu);
      else if (d.act == kActRelu) FDB_STEM_LAUNCH(true, kActRelu);
      else FDB_STEM_LAUNCH(true, kActNone);
    } else {
      if (d.act == kActSilu) FDB_STEM_LAUNCH(false, kActSilu);
      else if (d.act == kActRelu) FDB_STEM_LAUNCH(false, kActRelu);
      else FDB_STEM_LAUNCH(false, kActNone);
    }
#undef FDB_STEM_LAUNCH
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

}  // namespace fdb

using namespace fdb;

FDB_API void* fdb_stem_conv_create(const StemConvDesc* dp) {
  const StemConvDesc& d = *dp;
  if (d.dtype != kF16 && d.dtype != kBF16) { set_error("stem_conv: 16-bit input and output only"); return nullptr; }
  if (d.act != kActNone && d.act != kActRelu && d.act != kActSilu) { set_error("stem_conv: activation must be none, relu or silu"); return nullptr; }
  if (d.cin < 1 || d.cin > kStemCin) { set_error("stem_conv: 1 to 3 input channels"); return nullptr; }
  if (d.x_ld < 4 || (d.x_ld * 2) % 16 != 0 || (d.y_ld * 2) % 16 != 0 || d.y_ld < kStemCout) {
    set_error("stem_conv: pixel rows must be 16-byte multiples"); return nullptr;
  }
  if (reinterpret_cast<uintptr_t>(d.x) % 16 != 0 || reinterpret_cast<uintptr_t>(d.y) % 16 != 0 ||
      (d.x_n_stride * 2) % 16 != 0 || (d.y_n_stride * 2) % 16 != 0) {
    set_error("stem_conv: tensors must be 16-byte aligned"); return nullptr;
  }
  if (d.Ho != (d.H + 2 - 3) / 2 + 1 || d.Wo != (d.W + 2 - 3) / 2 + 1) { set_error("stem_conv: output size does not match 3x3 stride 2 pad 1"); return nullptr; }
  if (d.Ho > 65535 || d.N > 65535) { set_error("stem_conv: grid too large"); return nullptr; }
  auto* op = new StemConvOp();
  op->d = d;
  // channels past cin never contribute
  for (int t = 0; t < kStemTaps; ++t)
    for (int ci = d.cin; ci < kStemCin; ++ci)
      for (int c = 0; c < kStemCout; ++c) op->d.w[(t * kStemCin + ci) * kStemCout + c] = 0.f;
  return op;
}
