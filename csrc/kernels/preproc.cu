// Fused image pre-processing: uint8 HWC source images (decode buffers) ->
// resize {nearest, bilinear, bicubic} -> optional placement inside a padded canvas
// (letterbox / pad-to-size / pad-to-stride / batch-max) -> optional R/B swap ->
// per-channel affine normalisation -> NHWC (channel-padded) or NCHW -> fp16/bf16/fp32.
// One launch per batch, one thread per destination pixel.
//
// It stands in for the reference's whole processor chain on GPU:
// Resize + Pad + Normalize + HWC2CHW + Cast through CV-CUDA and its own kernels
// (fastdeploy/vision/common/processors/normalize_and_permute.cu:21-40,
//  fastdeploy/vision/utils/yolo_preprocess.cu:37-113). Interpolation follows the
// OpenCV conventions (half-pixel centres, replicated border, cubic a = -0.75) and the
// resized value is rounded to uint8 before normalisation, as the reference's
// Resize-then-Normalize sequence does.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fdb_common.h"

namespace fdb {

// Per-image geometry, uploaded by the host for every batch (48 bytes).
struct PreprocImage {
  long long src_offset;  // bytes from the source base pointer
  int src_h, src_w, src_stride;  // stride in bytes between source rows
  int dst_top, dst_left;         // where the resized image sits in the canvas
  int rh, rw;                    // resized size
  float sx, sy;                  // src_w / rw, src_h / rh
  int pad0;
};

struct PreprocDesc {
  const uint8_t* src;
  const PreprocImage* meta;
  void* dst;
  int N, Ho, Wo;
  int c_out;        // channels written per pixel for NHWC (>= 3; extra channels are zero)
  int interp;       // 0 nearest, 1 bilinear, 2 bicubic
  int layout;       // 0 NHWC, 1 NCHW
  int out_dtype;    // kF16 | kBF16 | kF32
  int swap_rb;
  int round_u8;     // round the interpolated value to uint8 first (reference semantics)
  float alpha[3], beta[3];  // out = v * alpha[c] + beta[c], indexed by OUTPUT channel
  float pad[3];             // canvas value outside the resized image (output domain)
};

__device__ __forceinline__ float cubic_w(float x) {
  const float A = -0.75f;
  x = fabsf(x);
  if (x <= 1.f) return ((A + 2.f) * x - (A + 3.f)) * x * x + 1.f;
  if (x < 2.f) return ((A * x - 5.f * A) * x + 8.f * A) * x - 4.f * A;
  return 0.f;
}

__global__ void preproc_kernel(const PreprocDesc d) {
  const long long total = static_cast<long long>(d.N) * d.Ho * d.Wo;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ox = static_cast<int>(idx % d.Wo);
    const long long t = idx / d.Wo;
    const int oy = static_cast<int>(t % d.Ho);
    const int n = static_cast<int>(t / d.Ho);
    const PreprocImage m = d.meta[n];
    float v[3];
    const int rx = ox - m.dst_left, ry = oy - m.dst_top;
    if (rx < 0 || ry < 0 || rx >= m.rw || ry >= m.rh) {
      v[0] = d.pad[0]; v[1] = d.pad[1]; v[2] = d.pad[2];
    } else {
      const uint8_t* src = d.src + m.src_offset;
      float s[3];
      if (d.interp == 0) {
        const int sxi = min(static_cast<int>(floorf(rx * m.sx)), m.src_w - 1);
        const int syi = min(static_cast<int>(floorf(ry * m.sy)), m.src_h - 1);
        const uint8_t* p = src + static_cast<size_t>(syi) * m.src_stride + sxi * 3;
        s[0] = p[0]; s[1] = p[1]; s[2] = p[2];
      } else if (d.interp == 1) {
        float fx = (rx + 0.5f) * m.sx - 0.5f, fy = (ry + 0.5f) * m.sy - 0.5f;
        int x0 = static_cast<int>(floorf(fx)), y0 = static_cast<int>(floorf(fy));
        fx -= x0; fy -= y0;
        if (x0 < 0) { x0 = 0; fx = 0.f; }
        if (x0 >= m.src_w - 1) { x0 = m.src_w - 1; fx = 0.f; }
        if (y0 < 0) { y0 = 0; fy = 0.f; }
        if (y0 >= m.src_h - 1) { y0 = m.src_h - 1; fy = 0.f; }
        const int x1 = min(x0 + 1, m.src_w - 1), y1 = min(y0 + 1, m.src_h - 1);
        const uint8_t* r0 = src + static_cast<size_t>(y0) * m.src_stride;
        const uint8_t* r1 = src + static_cast<size_t>(y1) * m.src_stride;
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          const float top = r0[x0 * 3 + c] * (1.f - fx) + r0[x1 * 3 + c] * fx;
          const float bot = r1[x0 * 3 + c] * (1.f - fx) + r1[x1 * 3 + c] * fx;
          s[c] = top * (1.f - fy) + bot * fy;
        }
      } else {
        float fx = (rx + 0.5f) * m.sx - 0.5f, fy = (ry + 0.5f) * m.sy - 0.5f;
        const int x0 = static_cast<int>(floorf(fx)), y0 = static_cast<int>(floorf(fy));
        fx -= x0; fy -= y0;
        float wx[4], wy[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          wx[k] = cubic_w(fx - (k - 1));
          wy[k] = cubic_w(fy - (k - 1));
        }
        s[0] = s[1] = s[2] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int yy = min(max(y0 - 1 + j, 0), m.src_h - 1);
          const uint8_t* row = src + static_cast<size_t>(yy) * m.src_stride;
          float acc[3] = {0.f, 0.f, 0.f};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int xx = min(max(x0 - 1 + k, 0), m.src_w - 1);
            acc[0] += wx[k] * row[xx * 3 + 0];
            acc[1] += wx[k] * row[xx * 3 + 1];
            acc[2] += wx[k] * row[xx * 3 + 2];
          }
          s[0] += wy[j] * acc[0]; s[1] += wy[j] * acc[1]; s[2] += wy[j] * acc[2];
        }
      }
      if (d.round_u8) {
#pragma unroll
        for (int c = 0; c < 3; ++c) s[c] = fminf(fmaxf(rintf(s[c]), 0.f), 255.f);
      }
      if (d.swap_rb) { const float tmp = s[0]; s[0] = s[2]; s[2] = tmp; }
#pragma unroll
      for (int c = 0; c < 3; ++c) v[c] = s[c] * d.alpha[c] + d.beta[c];
    }
    if (d.layout == 0) {
      const size_t o = static_cast<size_t>(idx) * d.c_out;
      if (d.out_dtype == kF32) {
        float* y = reinterpret_cast<float*>(d.dst) + o;
        y[0] = v[0]; y[1] = v[1]; y[2] = v[2];
        for (int c = 3; c < d.c_out; ++c) y[c] = 0.f;
      } else if (d.c_out == 8) {
        uint32_t w0, w1;
        if (d.out_dtype == kBF16) {
          __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
          __nv_bfloat162 b = __floats2bfloat162_rn(v[2], 0.f);
          w0 = *reinterpret_cast<uint32_t*>(&a); w1 = *reinterpret_cast<uint32_t*>(&b);
        } else {
          __half2 a = __floats2half2_rn(v[0], v[1]);
          __half2 b = __floats2half2_rn(v[2], 0.f);
          w0 = *reinterpret_cast<uint32_t*>(&a); w1 = *reinterpret_cast<uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(d.dst) + o * 2) = make_uint4(w0, w1, 0u, 0u);
      } else {
        for (int c = 0; c < d.c_out; ++c) {
          const float val = c < 3 ? v[c] : 0.f;
          if (d.out_dtype == kBF16) reinterpret_cast<__nv_bfloat16*>(d.dst)[o + c] = __float2bfloat16_rn(val);
          else reinterpret_cast<__half*>(d.dst)[o + c] = __float2half_rn(val);
        }
      }
    } else {
      const size_t plane = static_cast<size_t>(d.Ho) * d.Wo;
      const size_t o = static_cast<size_t>(n) * 3 * plane + static_cast<size_t>(oy) * d.Wo + ox;
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        if (d.out_dtype == kF32) reinterpret_cast<float*>(d.dst)[o + c * plane] = v[c];
        else if (d.out_dtype == kBF16) reinterpret_cast<__nv_bfloat16*>(d.dst)[o + c * plane] = __float2bfloat16_rn(v[c]);
        else reinterpret_cast<__half*>(d.dst)[o + c * plane] = __float2half_rn(v[c]);
      }
    }
  }
}

struct PreprocOp : Op {
  PreprocDesc d;
  int launch(cudaStream_t s) override {
    const long long total = static_cast<long long>(d.N) * d.Ho * d.Wo;
    long long g = (total + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 32;
    if (g > cap) g = cap;
    preproc_kernel<<<static_cast<int>(g < 1 ? 1 : g), 256, 0, s>>>(d);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

}  // namespace fdb

FDB_API void* fdb_preproc_create(const fdb::PreprocDesc* d) {
  if (d->c_out < 3) { fdb::set_error("preproc: c_out must be >= 3"); return nullptr; }
  auto* op = new fdb::PreprocOp();
  op->d = *d;
  return op;
}

FDB_API int fdb_preproc_image_size() { return (int)sizeof(fdb::PreprocImage); }
