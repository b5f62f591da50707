// Memory-bound NHWC helper kernels of the native backend: pooling, squeeze-excite
// plumbing, nearest upsampling, channel-slice copies, elementwise ops, DFL box decode.
// All of them move 16-byte vectors (8 fp16/bf16 channels) per thread and accept a
// channel stride ("ld") on both sides so that concat / split are fused away by
// reading and writing channel slices of wider buffers.
//
// The reference gets these from TensorRT / Paddle Inference; its only own kernel in
// this family is the adaptive pool (runtime/backends/common/cuda/adaptive_pool2d_kernel.cu:20-59).
//
// Generic descriptor: every op is created with fdb_simple_create(kind, &SimpleDesc);
// the slot meaning per kind is documented at the kernel and mirrored in
// fastdeploy_b200/ops/nhwc.py.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <functional>

#include "fdb_common.h"

namespace fdb {

struct SimpleDesc {
  void* p[8];
  long long i[24];
  float f[8];
};

struct LambdaOp : Op {
  std::function<int(cudaStream_t)> fn;
  int launch(cudaStream_t s) override { return fn(s); }
};

enum SimpleKind : int {
  kGapPartial = 0,
  kGapFinalize = 1,
  kSeFc = 2,
  kScaleChannels = 3,
  kMaxPool = 4,
  kUpsampleNearest = 5,
  kCopyChannels = 6,
  kDflDecode = 7,
  kBinary = 8,
  kAvgPool = 9,
  kCast = 10,
  kUnary = 11,
  kDepthwiseConv = 12,
};

// ---- 16-bit pack helpers -----------------------------------------------------------
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

__device__ __forceinline__ float act_f32(float x, int act, float alpha, float beta) {
  switch (act) {
    case kActRelu: return fmaxf(x, 0.f);
    case kActSilu: return __fdividef(x, 1.f + __expf(-x));
    case kActHardSwish: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) * (1.f / 6.f);
    case kActHardSigmoid: return fminf(fmaxf(alpha * x + beta, 0.f), 1.f);
    case kActSigmoid: return __fdividef(1.f, 1.f + __expf(-x));
    case kActGelu: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case kActRelu6: return fminf(fmaxf(x, 0.f), 6.f);
    case kActLeakyRelu: return x > 0.f ? x : alpha * x;
    case kActTanh: return tanhf(x);
    default: return x;
  }
}

// ---- global average pool, phase 1 ---------------------------------------------------
// p0 x (16-bit NHWC), p1 partial fp32 [N][S][C];  i0 N, i1 HW, i2 C, i3 x_ld, i4 S (splits), i5 bf16,
// i6 x_n_stride (elements). Each block: one image, one split, 64 channels; 256 threads =
// 8 channel groups x 32 pixel lanes.
template <bool BF16>
__global__ void gap_partial_kernel(const uint8_t* __restrict__ x, float* __restrict__ part, int HW, int C,
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
    if (c < C) part[(static_cast<size_t>(n) * S + split) * C + c] = s;
  }
}

// phase 2: p0 partial, p1 out (fp32 or 16-bit [N][C] with ld); i0 N, i1 C, i2 S, i3 out dtype, i4 out_ld; f0 scale
__global__ void gap_finalize_kernel(const float* __restrict__ part, void* __restrict__ out, int N, int C, int S,
                                    int out_dtype, int out_ld, float scale) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * C) return;
  const int n = idx / C, c = idx - n * C;
  float s = 0.f;
  for (int k = 0; k < S; ++k) s += part[(static_cast<size_t>(n) * S + k) * C + c];
  s *= scale;
  const size_t o = static_cast<size_t>(n) * out_ld + c;
  if (out_dtype == kF32) reinterpret_cast<float*>(out)[o] = s;
  else if (out_dtype == kBF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(s);
  else reinterpret_cast<__half*>(out)[o] = __float2half_rn(s);
}

// ---- squeeze-excite fully connected ------------------------------------------------
// out[n][co] = act(b[co] + sum_ci W[co][ci] * v[n][ci]);  one warp per output.
// p0 v fp32 [N][Cin], p1 W 16-bit [Cout][Cin], p2 bias fp32 or null, p3 out fp32 [N][Cout];
// i0 N, i1 Cin, i2 Cout, i3 act, i4 bf16; f0 alpha, f1 beta
template <bool BF16>
__global__ void se_fc_kernel(const float* __restrict__ v, const uint8_t* __restrict__ W, const float* __restrict__ b,
                             float* __restrict__ out, int N, int Cin, int Cout, int act, float alpha, float beta) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= N * Cout) return;
  const int n = warp / Cout, co = warp - n * Cout;
  const float* vn = v + static_cast<size_t>(n) * Cin;
  const uint8_t* wr = W + static_cast<size_t>(co) * Cin * 2;
  float s = 0.f;
  for (int c = lane * 8; c < Cin; c += 256) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(wr + c * 2));
    float f[8];
    unpack8<BF16>(u, f);
    const float4 a0 = *reinterpret_cast<const float4*>(vn + c);
    const float4 a1 = *reinterpret_cast<const float4*>(vn + c + 4);
    s += f[0] * a0.x + f[1] * a0.y + f[2] * a0.z + f[3] * a0.w + f[4] * a1.x + f[5] * a1.y + f[6] * a1.z + f[7] * a1.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[warp] = act_f32(s + (b ? b[co] : 0.f), act, alpha, beta);
}

// ---- y = x * s[n][c] (+ r) -------------------------------------------------------------
// p0 x, p1 s fp32 [N][C], p2 y, p3 r (optional, same dtype);  i0 N, i1 HW, i2 C, i3 x_ld, i4 y_ld, i5 bf16,
// i6 x_n_stride, i7 y_n_stride, i8 r_ld, i9 r_n_stride
template <bool BF16>
__global__ void scale_channels_kernel(const uint8_t* __restrict__ x, const float* __restrict__ s, uint8_t* __restrict__ y,
                                      const uint8_t* __restrict__ r, long long total, int HW, int C8, int C, int x_ld,
                                      int y_ld, long long xns, long long yns, int r_ld, long long rns) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx % C8);
    const long long pn = idx / C8;
    const int p = static_cast<int>(pn % HW);
    const int n = static_cast<int>(pn / HW);
    const int c = cg * 8;
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(x + (n * xns + static_cast<long long>(p) * x_ld + c) * 2));
    float f[8];
    unpack8<BF16>(u, f);
    const float4 s0 = *reinterpret_cast<const float4*>(s + static_cast<size_t>(n) * C + c);
    const float4 s1 = *reinterpret_cast<const float4*>(s + static_cast<size_t>(n) * C + c + 4);
    f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w;
    f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
    if (r != nullptr) {
      const uint4 ur = __ldg(reinterpret_cast<const uint4*>(r + (n * rns + static_cast<long long>(p) * r_ld + c) * 2));
      float g[8];
      unpack8<BF16>(ur, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
    }
    *reinterpret_cast<uint4*>(y + (n * yns + static_cast<long long>(p) * y_ld + c) * 2) = pack8<BF16>(f);
  }
}

// ---- max / average pool -----------------------------------------------------------------
// p0 x, p1 y; i0 N, i1 H, i2 W, i3 C, i4 x_ld, i5 Ho, i6 Wo, i7 y_ld, i8 kh, i9 kw, i10 sh, i11 sw,
// i12 pad_top, i13 pad_left, i14 bf16, i15 x_n_stride, i16 y_n_stride, i17 mode (0 max, 1 avg exclusive,
// 2 avg inclusive)
template <bool BF16>
__global__ void pool_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, long long total, int H, int W,
                            int C8, int x_ld, int Ho, int Wo, int y_ld, int kh, int kw, int sh, int sw, int pt,
                            int pl, long long xns, long long yns, int mode) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx % C8);
    long long t = idx / C8;
    const int ow = static_cast<int>(t % Wo); t /= Wo;
    const int oh = static_cast<int>(t % Ho);
    const int n = static_cast<int>(t / Ho);
    const int h0 = max(oh * sh - pt, 0), h1 = min(oh * sh - pt + kh, H);
    const int w0 = max(ow * sw - pl, 0), w1 = min(ow * sw - pl + kw, W);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = mode == 0 ? -INFINITY : 0.f;
    for (int h = h0; h < h1; ++h) {
      const uint8_t* row = x + (n * xns + (static_cast<long long>(h) * W + w0) * x_ld + cg * 8) * 2;
      for (int w = w0; w < w1; ++w, row += x_ld * 2) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(row));
        float f[8];
        unpack8<BF16>(u, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = mode == 0 ? fmaxf(acc[j], f[j]) : acc[j] + f[j];
      }
    }
    if (mode != 0) {
      const int cnt = mode == 1 ? max((h1 - h0) * (w1 - w0), 1) : kh * kw;
      const float inv = 1.f / cnt;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= inv;
    }
    *reinterpret_cast<uint4*>(y + (n * yns + (static_cast<long long>(oh) * Wo + ow) * y_ld + cg * 8) * 2) =
        pack8<BF16>(acc);
  }
}

// ---- nearest upsample by integer factors / channel-slice copy ------------------------------------
// p0 x, p1 y; i0 N, i1 H, i2 W, i3 C, i4 x_ld, i5 y_ld, i6 fh, i7 fw, i8 x_n_stride, i9 y_n_stride
__global__ void upsample_nearest_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, long long total,
                                        int H, int W, int C8, int x_ld, int y_ld, int fh, int fw, long long xns,
                                        long long yns) {
  const int Ho = H * fh, Wo = W * fw;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx % C8);
    long long t = idx / C8;
    const int ow = static_cast<int>(t % Wo); t /= Wo;
    const int oh = static_cast<int>(t % Ho);
    const int n = static_cast<int>(t / Ho);
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(
        x + (n * xns + (static_cast<long long>(oh / fh) * W + ow / fw) * x_ld + cg * 8) * 2));
    *reinterpret_cast<uint4*>(y + (n * yns + (static_cast<long long>(oh) * Wo + ow) * y_ld + cg * 8) * 2) = u;
  }
}

// ---- binary elementwise with optional activation: y = act(a (op) b) ---------------------------------
// p0 a, p1 b, p2 y; i0 rows, i1 C, i2 a_ld, i3 b_ld, i4 y_ld, i5 bf16, i6 op (0 add, 1 mul, 2 sub, 3 max),
// i7 act, i8 b_mode (0 same shape, 1 b is [C] broadcast); f0 alpha, f1 beta
template <bool BF16>
__global__ void binary_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, uint8_t* __restrict__ y,
                              long long total, int C8, int a_ld, int b_ld, int y_ld, int op, int act, int b_mode,
                              float alpha, float beta) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx % C8);
    const long long r = idx / C8;
    const uint4 ua = __ldg(reinterpret_cast<const uint4*>(a + (r * a_ld + cg * 8) * 2));
    const uint4 ub = __ldg(reinterpret_cast<const uint4*>(b + ((b_mode ? 0 : r * b_ld) + cg * 8) * 2));
    float fa[8], fb[8];
    unpack8<BF16>(ua, fa);
    unpack8<BF16>(ub, fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = op == 0 ? fa[j] + fb[j] : op == 1 ? fa[j] * fb[j] : op == 2 ? fa[j] - fb[j] : fmaxf(fa[j], fb[j]);
      fa[j] = act_f32(v, act, alpha, beta);
    }
    *reinterpret_cast<uint4*>(y + (r * y_ld + cg * 8) * 2) = pack8<BF16>(fa);
  }
}

// ---- unary activation: y = act(x) -----------------------------------------------------------------
// p0 x, p1 y; i0 rows, i1 C, i2 x_ld, i3 y_ld, i4 bf16, i5 act; f0 alpha, f1 beta
template <bool BF16>
__global__ void unary_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, long long total, int C8, int x_ld,
                             int y_ld, int act, float alpha, float beta) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx % C8);
    const long long r = idx / C8;
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(x + (r * x_ld + cg * 8) * 2));
    float f[8];
    unpack8<BF16>(u, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = act_f32(f[j], act, alpha, beta);
    *reinterpret_cast<uint4*>(y + (r * y_ld + cg * 8) * 2) = pack8<BF16>(f);
  }
}

// ---- dtype cast of a dense buffer (fp32 <-> fp16/bf16, int64 <-> int32) -------------------------------
// p0 x, p1 y; i0 count, i1 src dtype, i2 dst dtype.  Successor of the reference's only function kernel,
// CudaCast (fastdeploy/function/cuda_cast.cu:20-41).
template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ x, D* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = static_cast<D>(x[i]);
}
template <>
__global__ void cast_kernel<float, __half>(const float* __restrict__ x, __half* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __float2half_rn(x[i]);
}
template <>
__global__ void cast_kernel<float, __nv_bfloat16>(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                  long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16_rn(x[i]);
}
template <>
__global__ void cast_kernel<__half, float>(const __half* __restrict__ x, float* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __half2float(x[i]);
}
template <>
__global__ void cast_kernel<__nv_bfloat16, float>(const __nv_bfloat16* __restrict__ x, float* __restrict__ y,
                                                  long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __bfloat162float(x[i]);
}

// ---- DFL box decode (PP-YOLOE ET-head) ----------------------------------------------------------------
// reg logits [N][A][4*(R+1)] (16-bit or fp32) -> boxes fp32 [N][A][4] = (x1,y1,x2,y2), divided by the
// per-image scale factor (h_ratio, w_ratio) so that boxes are in source-image pixels
// (fastdeploy/vision/detection/ppdet/postprocessor.cc:171-180).
// p0 reg, p1 boxes, p2 scale_factor fp32 [N][2] or null; i0 N, i1 A, i2 R+1 (bins), i3 reg dtype,
// i4 num levels, i5.. per level: start, W, stride (3 ints each, up to 5 levels), i20 elements between
// anchors of reg (0 = 4*bins); f0 grid cell offset
struct DflLevels {
  int n;
  int start[5], w[5], stride[5];
};
template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <> __device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_as_float<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

template <typename T>
__global__ void dfl_decode_kernel(const T* __restrict__ reg, float* __restrict__ boxes,
                                  const float* __restrict__ scale_factor, int N, int A, int bins, DflLevels lv,
                                  float offset, int reg_ld) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (n, a, side)
  if (idx >= N * A * 4) return;
  const int side = idx & 3;
  const int na = idx >> 2;
  const int n = na / A, a = na - n * A;
  const T* p = reg + static_cast<size_t>(na) * reg_ld + side * bins;
  float m = -INFINITY;
  for (int k = 0; k < bins; ++k) m = fmaxf(m, ld_as_float<T>(p + k));
  float den = 0.f, num = 0.f;
  for (int k = 0; k < bins; ++k) {
    const float e = __expf(ld_as_float<T>(p + k) - m);
    den += e;
    num += e * k;
  }
  const float dist = num / den;
  int l = 0;
  for (int k = 1; k < lv.n; ++k)
    if (a >= lv.start[k]) l = k;
  const int local = a - lv.start[l];
  const int gy = local / lv.w[l], gx = local - gy * lv.w[l];
  const float c = ((side & 1) ? gy : gx) + offset;
  float v = (side < 2 ? c - dist : c + dist) * lv.stride[l];
  if (scale_factor != nullptr) v /= scale_factor[n * 2 + ((side & 1) ? 0 : 1)];
  boxes[idx] = v;
}

// ------------------------------------------------------------------------------------------------
static inline int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

#define FDB_LAUNCH_CHECK()                          \
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

// ---- depthwise convolution -----------------------------------------------------------
// p0 x (16-bit NHWC), p1 w fp32 [KH*KW][C], p2 bias fp32 [C] or null, p3 y (16-bit NHWC);
// i0 N, i1 H, i2 W, i3 C, i4 x_ld, i5 Ho, i6 Wo, i7 y_ld, i8 KH, i9 KW, i10 stride_h, i11 stride_w,
// i12 pad_top, i13 pad_left, i14 bf16, i15 x_n_stride, i16 y_n_stride, i17 act; f0 alpha, f1 beta.
// One thread = one output pixel x 8 channels: KH*KW 16-byte input loads, weights through L1, fp32
// accumulation, bias + activation fused. Memory bound by construction (one MAC per loaded value).
template <bool BF16>
__global__ void depthwise_conv_kernel(const uint8_t* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                      uint8_t* __restrict__ y, long long total, int H, int W, int C8, int x_ld, int Ho, int Wo,
                                      int y_ld, int KH, int KW, int sh, int sw, int pt, int pl, long long xns, long long yns,
                                      int act, float alpha, float beta) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(i % C8);
    long long r = i / C8;
    const int ow = static_cast<int>(r % Wo); r /= Wo;
    const int oh = static_cast<int>(r % Ho);
    const int n = static_cast<int>(r / Ho);
    const int c0 = cg * 8, C = C8 * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = bias != nullptr ? bias[c0 + j] : 0.f;
    const uint8_t* xn = x + static_cast<size_t>(n) * xns * 2;
    for (int kh = 0; kh < KH; ++kh) {
      const int ih = oh * sh - pt + kh;
      if (ih < 0 || ih >= H) continue;
      for (int kw = 0; kw < KW; ++kw) {
        const int iw = ow * sw - pl + kw;
        if (iw < 0 || iw >= W) continue;
        const uint4 v = *reinterpret_cast<const uint4*>(xn + ((static_cast<size_t>(ih) * W + iw) * x_ld + c0) * 2);
        float f[8];
        unpack8<BF16>(v, f);
        const float4 w0 = *reinterpret_cast<const float4*>(w + static_cast<size_t>(kh * KW + kw) * C + c0);
        const float4 w1 = *reinterpret_cast<const float4*>(w + static_cast<size_t>(kh * KW + kw) * C + c0 + 4);
        acc[0] = fmaf(f[0], w0.x, acc[0]); acc[1] = fmaf(f[1], w0.y, acc[1]);
        acc[2] = fmaf(f[2], w0.z, acc[2]); acc[3] = fmaf(f[3], w0.w, acc[3]);
        acc[4] = fmaf(f[4], w1.x, acc[4]); acc[5] = fmaf(f[5], w1.y, acc[5]);
        acc[6] = fmaf(f[6], w1.z, acc[6]); acc[7] = fmaf(f[7], w1.w, acc[7]);
      }
    }
    if (act != kActNone) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = act_f32(acc[j], act, alpha, beta);
    }
    *reinterpret_cast<uint4*>(y + (static_cast<size_t>(n) * yns + (static_cast<size_t>(oh) * Wo + ow) * y_ld + c0) * 2) =
        pack8<BF16>(acc);
  }
}

// The 3x3 and 5x5 depthwise layers of the light backbones: one thread = 8 channels x 4 neighbouring output pixels of a
// row. Per filter row the K weight vectors sit in registers and every input column of the window is loaded once and
// fed to all the outputs it reaches, so a 5x5 layer issues 8 input loads per filter row for 4 outputs instead of 20,
// and the loops are unrolled at compile time (K and the horizontal stride are template parameters).
template <bool BF16, int K, int SW>
__global__ void __launch_bounds__(256) depthwise_conv_tiled_kernel(
    const uint8_t* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, uint8_t* __restrict__ y,
    long long total, int H, int W, int C8, int x_ld, int Ho, int Wo, int y_ld, int sh, int pt, int pl, long long xns,
    long long yns, int act, float alpha, float beta) {
  constexpr int TW = 4, WIN = (TW - 1) * SW + K;
  const int wt = (Wo + TW - 1) / TW;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(i % C8);
    long long r = i / C8;
    const int ot = static_cast<int>(r % wt); r /= wt;
    const int oh = static_cast<int>(r % Ho);
    const int n = static_cast<int>(r / Ho);
    const int c0 = cg * 8, C = C8 * 8, ow0 = ot * TW;
    float acc[TW][8];
#pragma unroll
    for (int t = 0; t < TW; ++t)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[t][j] = bias != nullptr ? bias[c0 + j] : 0.f;
    const uint8_t* xn = x + static_cast<size_t>(n) * xns * 2;
    const int iw0 = ow0 * SW - pl;
#pragma unroll
    for (int kh = 0; kh < K; ++kh) {
      const int ih = oh * sh - pt + kh;
      if (ih < 0 || ih >= H) continue;
      float wk[K][8];
#pragma unroll
      for (int kw = 0; kw < K; ++kw) {
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(kh * K + kw) * C + c0));
        const float4 w1 = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(kh * K + kw) * C + c0 + 4));
        wk[kw][0] = w0.x; wk[kw][1] = w0.y; wk[kw][2] = w0.z; wk[kw][3] = w0.w;
        wk[kw][4] = w1.x; wk[kw][5] = w1.y; wk[kw][6] = w1.z; wk[kw][7] = w1.w;
      }
      const uint8_t* xrow = xn + (static_cast<size_t>(ih) * W * x_ld + c0) * 2;
#pragma unroll
      for (int j = 0; j < WIN; ++j) {
        const int iw = iw0 + j;
        if (iw < 0 || iw >= W) continue;
        float f[8];
        unpack8<BF16>(__ldg(reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(iw) * x_ld * 2)), f);
#pragma unroll
        for (int t = 0; t < TW; ++t) {
          const int kw = j - t * SW;               // resolved at compile time: j, t and SW are constants here
          if (kw >= 0 && kw < K) {
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[t][q] = fmaf(f[q], wk[kw][q], acc[t][q]);
          }
        }
      }
    }
    uint8_t* yrow = y + (static_cast<size_t>(n) * yns + static_cast<size_t>(oh) * Wo * y_ld + c0) * 2;
#pragma unroll
    for (int t = 0; t < TW; ++t) {
      if (ow0 + t >= Wo) break;
      if (act != kActNone) {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[t][q] = act_f32(acc[t][q], act, alpha, beta);
      }
      *reinterpret_cast<uint4*>(yrow + static_cast<size_t>(ow0 + t) * y_ld * 2) = pack8<BF16>(acc[t]);
    }
  }
}

FDB_API void* fdb_simple_create(int kind, const SimpleDesc* dp) {
  const SimpleDesc d = *dp;
  auto* op = new LambdaOp();
  switch (kind) {
    case kGapPartial: {
      const int N = d.i[0], HW = d.i[1], C = d.i[2], x_ld = d.i[3], S = d.i[4];
      const bool bf = d.i[5] != 0;
      const long long xns = d.i[6] > 0 ? d.i[6] : static_cast<long long>(HW) * x_ld;
      if (C % 8 || x_ld % 8) { set_error("gap: C and ld must be multiples of 8"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        dim3 grid((C + 63) / 64, N, S);
        if (bf) gap_partial_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (float*)d.p[1], HW, C, x_ld, S, xns);
        else gap_partial_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (float*)d.p[1], HW, C, x_ld, S, xns);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kGapFinalize: {
      const int N = d.i[0], C = d.i[1], S = d.i[2], odt = d.i[3], old = d.i[4] > 0 ? d.i[4] : d.i[1];
      const float scale = d.f[0];
      op->fn = [=](cudaStream_t s) {
        gap_finalize_kernel<<<(N * C + 255) / 256, 256, 0, s>>>((const float*)d.p[0], d.p[1], N, C, S, odt, old, scale);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kSeFc: {
      const int N = d.i[0], Cin = d.i[1], Cout = d.i[2], act = d.i[3];
      const bool bf = d.i[4] != 0;
      const float al = d.f[0], be = d.f[1];
      if (Cin % 8) { set_error("se_fc: Cin must be a multiple of 8"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        const long long threads = static_cast<long long>(N) * Cout * 32;
        const int grid = static_cast<int>((threads + 255) / 256);
        if (bf) se_fc_kernel<true><<<grid, 256, 0, s>>>((const float*)d.p[0], (const uint8_t*)d.p[1], (const float*)d.p[2], (float*)d.p[3], N, Cin, Cout, act, al, be);
        else se_fc_kernel<false><<<grid, 256, 0, s>>>((const float*)d.p[0], (const uint8_t*)d.p[1], (const float*)d.p[2], (float*)d.p[3], N, Cin, Cout, act, al, be);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kScaleChannels: {
      const int N = d.i[0], HW = d.i[1], C = d.i[2], x_ld = d.i[3], y_ld = d.i[4];
      const bool bf = d.i[5] != 0;
      const long long xns = d.i[6] > 0 ? d.i[6] : static_cast<long long>(HW) * x_ld;
      const long long yns = d.i[7] > 0 ? d.i[7] : static_cast<long long>(HW) * y_ld;
      const int r_ld = d.i[8] > 0 ? static_cast<int>(d.i[8]) : C;
      const long long rns = d.i[9] > 0 ? d.i[9] : static_cast<long long>(HW) * r_ld;
      if (C % 8 || x_ld % 8 || y_ld % 8 || r_ld % 8) { set_error("scale_channels: C/ld must be multiples of 8"); delete op; return nullptr; }
      const long long total = static_cast<long long>(N) * HW * (C / 8);
      op->fn = [=](cudaStream_t s) {
        const int grid = grid_for(total, 256);
        if (bf) scale_channels_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1], (uint8_t*)d.p[2], (const uint8_t*)d.p[3], total, HW, C / 8, C, x_ld, y_ld, xns, yns, r_ld, rns);
        else scale_channels_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1], (uint8_t*)d.p[2], (const uint8_t*)d.p[3], total, HW, C / 8, C, x_ld, y_ld, xns, yns, r_ld, rns);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kMaxPool:
    case kAvgPool: {
      const int N = d.i[0], H = d.i[1], W = d.i[2], C = d.i[3], x_ld = d.i[4], Ho = d.i[5], Wo = d.i[6], y_ld = d.i[7];
      const int kh = d.i[8], kw = d.i[9], sh = d.i[10], sw = d.i[11], pt = d.i[12], pl = d.i[13];
      const bool bf = d.i[14] != 0;
      const long long xns = d.i[15] > 0 ? d.i[15] : static_cast<long long>(H) * W * x_ld;
      const long long yns = d.i[16] > 0 ? d.i[16] : static_cast<long long>(Ho) * Wo * y_ld;
      const int mode = kind == kMaxPool ? 0 : (d.i[17] == 2 ? 2 : 1);
      if (C % 8 || x_ld % 8 || y_ld % 8) { set_error("pool: C/ld must be multiples of 8"); delete op; return nullptr; }
      const long long total = static_cast<long long>(N) * Ho * Wo * (C / 8);
      op->fn = [=](cudaStream_t s) {
        const int grid = grid_for(total, 256);
        if (bf) pool_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, H, W, C / 8, x_ld, Ho, Wo, y_ld, kh, kw, sh, sw, pt, pl, xns, yns, mode);
        else pool_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, H, W, C / 8, x_ld, Ho, Wo, y_ld, kh, kw, sh, sw, pt, pl, xns, yns, mode);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kUpsampleNearest:
    case kCopyChannels: {
      const int N = d.i[0], H = d.i[1], W = d.i[2], C = d.i[3], x_ld = d.i[4], y_ld = d.i[5];
      const int fh = kind == kCopyChannels ? 1 : static_cast<int>(d.i[6]);
      const int fw = kind == kCopyChannels ? 1 : static_cast<int>(d.i[7]);
      const long long xns = d.i[8] > 0 ? d.i[8] : static_cast<long long>(H) * W * x_ld;
      const long long yns = d.i[9] > 0 ? d.i[9] : static_cast<long long>(H) * fh * W * fw * y_ld;
      if (C % 8 || x_ld % 8 || y_ld % 8) { set_error("upsample/copy: C/ld must be multiples of 8"); delete op; return nullptr; }
      const long long total = static_cast<long long>(N) * H * fh * W * fw * (C / 8);
      op->fn = [=](cudaStream_t s) {
        upsample_nearest_kernel<<<grid_for(total, 256), 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, H, W, C / 8, x_ld, y_ld, fh, fw, xns, yns);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kDflDecode: {
      const int N = d.i[0], A = d.i[1], bins = d.i[2], rdt = d.i[3];
      DflLevels lv;
      lv.n = static_cast<int>(d.i[4]);
      if (lv.n < 1 || lv.n > 5) { set_error("dfl_decode: 1..5 levels"); delete op; return nullptr; }
      for (int k = 0; k < lv.n; ++k) {
        lv.start[k] = static_cast<int>(d.i[5 + 3 * k]);
        lv.w[k] = static_cast<int>(d.i[6 + 3 * k]);
        lv.stride[k] = static_cast<int>(d.i[7 + 3 * k]);
      }
      const float off = d.f[0];
      const int reg_ld = d.i[20] > 0 ? static_cast<int>(d.i[20]) : 4 * bins;
      op->fn = [=](cudaStream_t s) {
        const int total = N * A * 4;
        const int grid = (total + 255) / 256;
        if (rdt == kF32) dfl_decode_kernel<float><<<grid, 256, 0, s>>>((const float*)d.p[0], (float*)d.p[1], (const float*)d.p[2], N, A, bins, lv, off, reg_ld);
        else if (rdt == kBF16) dfl_decode_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)d.p[0], (float*)d.p[1], (const float*)d.p[2], N, A, bins, lv, off, reg_ld);
        else dfl_decode_kernel<__half><<<grid, 256, 0, s>>>((const __half*)d.p[0], (float*)d.p[1], (const float*)d.p[2], N, A, bins, lv, off, reg_ld);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kBinary: {
      const long long rows = d.i[0];
      const int C = d.i[1], a_ld = d.i[2], b_ld = d.i[3], y_ld = d.i[4];
      const bool bf = d.i[5] != 0;
      const int bop = d.i[6], act = d.i[7], b_mode = d.i[8];
      const float al = d.f[0], be = d.f[1];
      if (C % 8 || a_ld % 8 || b_ld % 8 || y_ld % 8) { set_error("binary: C/ld must be multiples of 8"); delete op; return nullptr; }
      const long long total = rows * (C / 8);
      op->fn = [=](cudaStream_t s) {
        const int grid = grid_for(total, 256);
        if (bf) binary_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const uint8_t*)d.p[1], (uint8_t*)d.p[2], total, C / 8, a_ld, b_ld, y_ld, bop, act, b_mode, al, be);
        else binary_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const uint8_t*)d.p[1], (uint8_t*)d.p[2], total, C / 8, a_ld, b_ld, y_ld, bop, act, b_mode, al, be);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kDepthwiseConv: {
      const int N = d.i[0], H = d.i[1], W = d.i[2], C = d.i[3], x_ld = d.i[4], Ho = d.i[5], Wo = d.i[6], y_ld = d.i[7];
      const int KH = d.i[8], KW = d.i[9], sh = d.i[10], sw = d.i[11], pt = d.i[12], pl = d.i[13];
      const bool bf = d.i[14] != 0;
      const long long xns = d.i[15] > 0 ? d.i[15] : static_cast<long long>(H) * W * x_ld;
      const long long yns = d.i[16] > 0 ? d.i[16] : static_cast<long long>(Ho) * Wo * y_ld;
      const int act = d.i[17];
      const float al = d.f[0], be = d.f[1];
      if (C % 8 || x_ld % 8 || y_ld % 8) { set_error("depthwise_conv: C/ld must be multiples of 8"); delete op; return nullptr; }
      const long long total = static_cast<long long>(N) * Ho * Wo * (C / 8);
      const bool tiled = KH == KW && (KH == 3 || KH == 5) && (sw == 1 || sw == 2) &&
                         reinterpret_cast<uintptr_t>(d.p[0]) % 16 == 0 && reinterpret_cast<uintptr_t>(d.p[1]) % 16 == 0;
      const long long total_tiled = static_cast<long long>(N) * Ho * ((Wo + 3) / 4) * (C / 8);
      op->fn = [=](cudaStream_t s) {
        if (tiled) {
          const int tgrid = grid_for(total_tiled, 256);
#define FDB_DW_LAUNCH(BF, K, SW)                                                                                      \
  depthwise_conv_tiled_kernel<BF, K, SW><<<tgrid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1],          \
      (const float*)d.p[2], (uint8_t*)d.p[3], total_tiled, H, W, C / 8, x_ld, Ho, Wo, y_ld, sh, pt, pl, xns, yns, act, al, be)
          if (bf) {
            if (KH == 3 && sw == 1) FDB_DW_LAUNCH(true, 3, 1); else if (KH == 3) FDB_DW_LAUNCH(true, 3, 2);
            else if (sw == 1) FDB_DW_LAUNCH(true, 5, 1); else FDB_DW_LAUNCH(true, 5, 2);
          } else {
            if (KH == 3 && sw == 1) FDB_DW_LAUNCH(false, 3, 1); else if (KH == 3) FDB_DW_LAUNCH(false, 3, 2);
            else if (sw == 1) FDB_DW_LAUNCH(false, 5, 1); else FDB_DW_LAUNCH(false, 5, 2);
          }
#undef FDB_DW_LAUNCH
          FDB_LAUNCH_CHECK();
        }
        const int grid = grid_for(total, 256);
        if (bf) depthwise_conv_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1], (const float*)d.p[2],
                                                                 (uint8_t*)d.p[3], total, H, W, C / 8, x_ld, Ho, Wo, y_ld, KH, KW, sh,
                                                                 sw, pt, pl, xns, yns, act, al, be);
        else depthwise_conv_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (const float*)d.p[1], (const float*)d.p[2],
                                                                (uint8_t*)d.p[3], total, H, W, C / 8, x_ld, Ho, Wo, y_ld, KH, KW, sh,
                                                                sw, pt, pl, xns, yns, act, al, be);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kUnary: {
      const long long rows = d.i[0];
      const int C = d.i[1], x_ld = d.i[2], y_ld = d.i[3];
      const bool bf = d.i[4] != 0;
      const int act = d.i[5];
      const float al = d.f[0], be = d.f[1];
      if (C % 8 || x_ld % 8 || y_ld % 8) { set_error("unary: C/ld must be multiples of 8"); delete op; return nullptr; }
      const long long total = rows * (C / 8);
      op->fn = [=](cudaStream_t s) {
        const int grid = grid_for(total, 256);
        if (bf) unary_kernel<true><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, C / 8, x_ld, y_ld, act, al, be);
        else unary_kernel<false><<<grid, 256, 0, s>>>((const uint8_t*)d.p[0], (uint8_t*)d.p[1], total, C / 8, x_ld, y_ld, act, al, be);
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    case kCast: {
      const long long n = d.i[0];
      const int sdt = d.i[1], ddt = d.i[2];
      op->fn = [=](cudaStream_t s) {
        const int grid = grid_for(n, 256);
#define FDB_CAST(S, D) cast_kernel<S, D><<<grid, 256, 0, s>>>((const S*)d.p[0], (D*)d.p[1], n)
        if (sdt == kF32 && ddt == kF16) FDB_CAST(float, __half);
        else if (sdt == kF32 && ddt == kBF16) FDB_CAST(float, __nv_bfloat16);
        else if (sdt == kF16 && ddt == kF32) FDB_CAST(__half, float);
        else if (sdt == kBF16 && ddt == kF32) FDB_CAST(__nv_bfloat16, float);
        else if (sdt == kI64 && ddt == kI32) FDB_CAST(long long, int);
        else if (sdt == kI32 && ddt == kI64) FDB_CAST(int, long long);
        else if (sdt == kI64 && ddt == kF32) FDB_CAST(long long, float);
        else if (sdt == kI32 && ddt == kF32) FDB_CAST(int, float);
        else if (sdt == kU8 && ddt == kF32) FDB_CAST(unsigned char, float);
        else { set_error("cast: unsupported dtype pair"); return -1; }
#undef FDB_CAST
        FDB_LAUNCH_CHECK();
      };
      break;
    }
    default:
      set_error("fdb_simple_create: unknown kind");
      delete op;
      return nullptr;
  }
  return op;
}
