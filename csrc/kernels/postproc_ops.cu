// Device-side post-processing and geometric warps that the reference runs on the host:
//
//   row_topk            k largest entries of every row with their indices, ties to the lower index
//                       (classification top-k, OCR angle-classifier argmax, per-step CTC argmax;
//                       fastdeploy/vision/classification/ppcls/postprocessor.cc,
//                       fastdeploy/vision/ocr/ppocr/cls_postprocessor.cc)
//   ctc_collapse        greedy CTC: keep a step when its class is not blank (0) and differs from the
//                       previous step's; score = mean of the kept maxima
//                       (fastdeploy/vision/ocr/ppocr/rec_postprocessor.cc:46-83)
//   warp_batch          N perspective / affine warps of one uint8 HWC frame into an [N, OH, OW, C]
//                       canvas, bilinear, replicated or constant border: OCR text crops, face
//                       alignment, key-point crops (cv::warpPerspective / cv::warpAffine in
//                       fastdeploy/vision/ocr/ppocr/utils/get_rotate_crop_image.cc:21-81)
//   warp_normalize      N perspective crops of one frame resized, normalised and right-padded straight into the
//                       16-bit NHWC input of the OCR classifier / recogniser, optional 180-degree turn per crop
//                       (get_rotate_crop_image.cc + cls_preprocessor.cc / rec_preprocessor.cc in one pass)
//   hard_voxelize       points -> voxels in order of first appearance, at most max_points per voxel
//                       (fastdeploy/vision/perception/paddle3d/centerpoint ops, voxelize_op.cu)
#include "fdb_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fdb {

template <typename T> __device__ __forceinline__ float pp_to_f(T v);
template <> __device__ __forceinline__ float pp_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float pp_to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float pp_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

struct ValIdx {
  float v;
  int i;
};

// a is better than b: larger value, or equal value at a lower index; NaN never wins
__device__ __forceinline__ bool better(const ValIdx& a, const ValIdx& b) {
  return a.v > b.v || (a.v == b.v && a.i < b.i);
}

// One CTA per row; k rounds of a block-wide arg-max over the entries not yet taken. k is small
// (top-5 of 1000 classes, arg-max of 6625 characters), so the row stays in L1/L2 between rounds.
template <typename T>
__global__ void __launch_bounds__(256) row_topk_kernel(const T* x, long long ld, int cols, int k, int* out_idx,
                                                       float* out_val) {
  __shared__ ValIdx warp_best[8];
  __shared__ int taken[16];
  const T* row = x + static_cast<long long>(blockIdx.x) * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = 0; r < k; ++r) {
    ValIdx best{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      bool skip = false;
      for (int j = 0; j < r; ++j) skip |= (taken[j] == c);
      if (skip) continue;
      const ValIdx cand{pp_to_f<T>(row[c]), c};
      if (better(cand, best)) best = cand;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      ValIdx o{__shfl_down_sync(0xffffffffu, best.v, off), __shfl_down_sync(0xffffffffu, best.i, off)};
      if (better(o, best)) best = o;
    }
    if (lane == 0) warp_best[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      ValIdx b = warp_best[0];
      for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w)
        if (better(warp_best[w], b)) b = warp_best[w];
      if (b.i == 0x7fffffff) { b.i = -1; }   // fewer than k finite entries
      taken[r] = b.i;
      out_idx[static_cast<long long>(blockIdx.x) * k + r] = b.i;
      out_val[static_cast<long long>(blockIdx.x) * k + r] = b.v;
    }
    __syncthreads();
  }
}

// One warp per sequence. idx / val are the per-step arg-max [B, T]; writes the kept class ids packed
// to the front of out_ids[b] (the rest -1), their count and the mean of the kept maxima.
__global__ void ctc_collapse_kernel(const int* idx, const float* val, int B, int T, int* out_ids, int* out_len,
                                    float* out_score) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const int* id = idx + static_cast<long long>(b) * T;
  const float* vv = val + static_cast<long long>(b) * T;
  int* out = out_ids + static_cast<long long>(b) * T;
  int count = 0;
  float sum = 0.f;
  for (int t0 = 0; t0 < T; t0 += 32) {
    const int t = t0 + lane;
    int cur = 0;
    bool keep = false;
    if (t < T) {
      cur = id[t];
      const int prev = t > 0 ? id[t - 1] : -1;
      keep = cur > 0 && !(t > 0 && cur == prev);
    }
    const unsigned m = __ballot_sync(0xffffffffu, keep);
    const int pos = count + __popc(m & ((1u << lane) - 1u));
    if (keep) out[pos] = cur;
    float s = keep ? vv[t] : 0.f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    sum += s;
    count += __popc(m);
  }
  for (int t = count + lane; t < T; t += 32) out[t] = -1;
  if (lane == 0) {
    out_len[b] = count;
    out_score[b] = count > 0 ? sum / count : 0.f;
  }
}

}  // namespace fdb

using namespace fdb;

static int pp_check(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error(std::string(what) + ": " + cudaGetErrorString(e)); return -1; }
  return 0;
}

// x [rows, cols] with row pitch ld (elements) of dtype f16 / bf16 / f32 -> out_idx [rows, k] int32,
// out_val [rows, k] fp32, sorted by descending value. 1 <= k <= 16.
FDB_API int fdb_row_topk(const void* x, int dtype, long long rows, int cols, long long ld, int k, int* out_idx,
                         float* out_val, void* stream) {
  if (k < 1 || k > 16 || cols < 1 || rows < 0) { set_error("row_topk: k must be 1..16"); return -1; }
  if (rows == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  if (dtype == kF32) row_topk_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ld, cols, k, out_idx, out_val);
  else if (dtype == kF16) row_topk_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), ld, cols, k, out_idx, out_val);
  else if (dtype == kBF16) row_topk_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ld, cols, k, out_idx, out_val);
  else { set_error("row_topk: dtype must be fp16, bf16 or fp32"); return -1; }
  return pp_check("row_topk");
}

FDB_API int fdb_ctc_collapse(const int* idx, const float* val, int B, int T, int* out_ids, int* out_len,
                             float* out_score, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  ctc_collapse_kernel<<<(B + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(idx, val, B, T, out_ids, out_len, out_score);
  return pp_check("ctc_collapse");
}

// ------------------------------------------------------------------ batched perspective / affine warp
namespace fdb {

// out[n, y, x, :] = bilinear sample of src at M_n * (x, y, 1) (dst -> src homography, row-major 3x3).
// sizes[n] = (w, h) of the valid part of canvas n (null: the whole canvas); pixels outside it take `fill`.
// border 1: taps are clamped to the frame (replicate); border 0: taps outside the frame read `fill`.
__global__ void warp_batch_kernel(const uint8_t* src, int H, int W, int C, const float* mats, const int* sizes,
                                  uint8_t* out, int N, int OH, int OW, int border, int fill) {
  const int n = blockIdx.z;
  const int x = blockIdx.x * blockDim.x + threadIdx.x;
  const int y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= OW || y >= OH) return;
  uint8_t* o = out + ((static_cast<size_t>(n) * OH + y) * OW + x) * C;
  const int vw = sizes != nullptr ? sizes[2 * n] : OW, vh = sizes != nullptr ? sizes[2 * n + 1] : OH;
  if (x >= vw || y >= vh) {
    for (int c = 0; c < C; ++c) o[c] = static_cast<uint8_t>(fill);
    return;
  }
  const float* m = mats + 9 * n;
  const float fx = static_cast<float>(x), fy = static_cast<float>(y);
  float wz = m[6] * fx + m[7] * fy + m[8];
  wz = wz != 0.f ? 1.f / wz : 0.f;
  const float sx = (m[0] * fx + m[1] * fy + m[2]) * wz;
  const float sy = (m[3] * fx + m[4] * fy + m[5]) * wz;
  // keep the coordinates in a range where the int conversion is exact
  const float cx = fminf(fmaxf(sx, -2.f), static_cast<float>(W) + 1.f);
  const float cy = fminf(fmaxf(sy, -2.f), static_cast<float>(H) + 1.f);
  const int x0 = static_cast<int>(floorf(cx)), y0 = static_cast<int>(floorf(cy));
  const float ax = cx - x0, ay = cy - y0;
  int xs[2] = {x0, x0 + 1}, ys[2] = {y0, y0 + 1};
  bool in_x[2], in_y[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    in_x[k] = xs[k] >= 0 && xs[k] < W;
    in_y[k] = ys[k] >= 0 && ys[k] < H;
    xs[k] = min(max(xs[k], 0), W - 1);
    ys[k] = min(max(ys[k], 0), H - 1);
  }
  const float w00 = (1.f - ax) * (1.f - ay), w01 = ax * (1.f - ay), w10 = (1.f - ax) * ay, w11 = ax * ay;
  for (int c = 0; c < C; ++c) {
    float t[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int yi = k >> 1, xi = k & 1;
      const bool inside = in_x[xi] && in_y[yi];
      t[k] = (inside || border == 1) ? static_cast<float>(src[(static_cast<size_t>(ys[yi]) * W + xs[xi]) * C + c])
                                     : static_cast<float>(fill);
    }
    const float v = t[0] * w00 + t[1] * w01 + t[2] * w10 + t[3] * w11;
    o[c] = static_cast<uint8_t>(min(max(__float2int_rn(v), 0), 255));
  }
}

}  // namespace fdb

FDB_API int fdb_warp_batch(const void* src, int H, int W, int C, const float* mats, const int* sizes, void* out, int N,
                           int OH, int OW, int border, int fill, void* stream) {
  if (N <= 0) return 0;
  if (H < 1 || W < 1 || C < 1 || C > 4 || OH < 1 || OW < 1 || N > 65535) { set_error("warp_batch: bad shape"); return -1; }
  const dim3 block(32, 8), grid((OW + 31) / 32, (OH + 7) / 8, N);
  warp_batch_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), H, W, C, mats, sizes, static_cast<uint8_t*>(out), N, OH, OW, border, fill);
  return pp_check("warp_batch");
}

// ------------------------------------------------------------------ warp + resize + normalise into network inputs
namespace fdb {

// out[n, y, x, 0..2] = alpha[c] * bilinear(src at M_n * (x', y', 1)) + beta[c] for x < valid_w[n], else 0; channels
// 3..CP-1 are 0. (x', y') = (x, y), or (valid_w - 1 - x, OH - 1 - y) when flip[n] != 0 (the crop turned by 180 degrees).
// One pass from the source frame to the 16-bit NHWC input of the classifier / recogniser: perspective rectification,
// resize to the input height, normalisation and right padding in a single read of the source pixels.
template <typename T>
__global__ void warp_normalize_kernel(const uint8_t* src_all, int H, int W, const int* page, long long page_stride,
                                      const float* mats, const int* valid_w, const int* flip, T* out, int OH, int OW,
                                      int CP, float a0, float a1, float a2, float b0, float b1, float b2) {
  const int n = blockIdx.z;
  const int x = blockIdx.x * blockDim.x + threadIdx.x;
  const int y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= OW || y >= OH) return;
  T* o = out + ((static_cast<size_t>(n) * OH + y) * OW + x) * CP;
  const int vw = min(valid_w[n], OW);
  const uint8_t* src = src_all + (page != nullptr ? page[n] * page_stride : 0);
  float v[3] = {0.f, 0.f, 0.f};
  if (x < vw) {
    const bool fl = flip != nullptr && flip[n] != 0;
    const float fx = static_cast<float>(fl ? vw - 1 - x : x), fy = static_cast<float>(fl ? OH - 1 - y : y);
    const float* m = mats + 9 * n;
    float wz = m[6] * fx + m[7] * fy + m[8];
    wz = wz != 0.f ? 1.f / wz : 0.f;
    const float sx = fminf(fmaxf((m[0] * fx + m[1] * fy + m[2]) * wz, -2.f), static_cast<float>(W) + 1.f);
    const float sy = fminf(fmaxf((m[3] * fx + m[4] * fy + m[5]) * wz, -2.f), static_cast<float>(H) + 1.f);
    const int x0 = static_cast<int>(floorf(sx)), y0 = static_cast<int>(floorf(sy));
    const float ax = sx - x0, ay = sy - y0;
    const int xa = min(max(x0, 0), W - 1), xb = min(max(x0 + 1, 0), W - 1);       // replicated border
    const int ya = min(max(y0, 0), H - 1), yb = min(max(y0 + 1, 0), H - 1);
    const uint8_t* r0 = src + static_cast<size_t>(ya) * W * 3;
    const uint8_t* r1 = src + static_cast<size_t>(yb) * W * 3;
    const float al[3] = {a0, a1, a2}, be[3] = {b0, b1, b2};
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const float t = (r0[xa * 3 + c] * (1.f - ax) + r0[xb * 3 + c] * ax) * (1.f - ay) +
                      (r1[xa * 3 + c] * (1.f - ax) + r1[xb * 3 + c] * ax) * ay;
      v[c] = al[c] * t + be[c];
    }
  }
  for (int c = 0; c < CP; ++c) o[c] = static_cast<T>(c < 3 ? v[c] : 0.f);
}

// flip[n] = 1 when the arg-max class of row n is odd (180 degrees) and its probability exceeds thresh
// (fastdeploy/vision/ocr/ppocr/ppocr_v2.cc:150-160)
template <typename T>
__global__ void cls_flip_kernel(const T* probs, long long ld, int n, int ncls, float thresh, int* flip, int* label,
                                float* score) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int best = 0;
  float bv = -INFINITY;
  for (int c = 0; c < ncls; ++c) {
    const float v = pp_to_f<T>(probs[i * ld + c]);
    if (v > bv) { bv = v; best = c; }
  }
  flip[i] = ((best & 1) == 1 && bv > thresh) ? 1 : 0;
  if (label != nullptr) label[i] = best;
  if (score != nullptr) score[i] = bv;
}

}  // namespace fdb

// src: uint8 frames of [H, W, 3] on the device, frame k at byte offset k * page_stride; page: device int32 [N] = frame
// of each crop (null: all from frame 0); mats: device fp32 [N, 9] (output pixel -> source pixel); valid_w, flip: device
// int32 [N] (flip may be null); out: [N, OH, OW, CP] fp16 / bf16 / fp32 (out_dtype code).
FDB_API int fdb_warp_normalize_batch(const void* src, int H, int W, const int* page, long long page_stride, const float* mats,
                                     const int* valid_w, const int* flip, void* out, int out_dtype, int N, int OH, int OW,
                                     int CP, const float* alpha, const float* beta, void* stream) {
  if (N <= 0) return 0;
  if (H < 1 || W < 1 || OH < 1 || OW < 1 || CP < 3 || CP > 16 || N > 65535) { set_error("warp_normalize_batch: bad shape"); return -1; }
  const dim3 block(32, 8), grid((OW + 31) / 32, (OH + 7) / 8, N);
  auto st = static_cast<cudaStream_t>(stream);
  const uint8_t* s8 = static_cast<const uint8_t*>(src);
  switch (out_dtype) {
    case kF16:
      warp_normalize_kernel<__half><<<grid, block, 0, st>>>(s8, H, W, page, page_stride, mats, valid_w, flip, static_cast<__half*>(out), OH, OW,
                                                            CP, alpha[0], alpha[1], alpha[2], beta[0], beta[1], beta[2]);
      break;
    case kBF16:
      warp_normalize_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(s8, H, W, page, page_stride, mats, valid_w, flip,
                                                                   static_cast<__nv_bfloat16*>(out), OH, OW, CP, alpha[0],
                                                                   alpha[1], alpha[2], beta[0], beta[1], beta[2]);
      break;
    case kF32:
      warp_normalize_kernel<float><<<grid, block, 0, st>>>(s8, H, W, page, page_stride, mats, valid_w, flip, static_cast<float*>(out), OH, OW,
                                                           CP, alpha[0], alpha[1], alpha[2], beta[0], beta[1], beta[2]);
      break;
    default:
      set_error("warp_normalize_batch: fp16 / bf16 / fp32 output");
      return -1;
  }
  return pp_check("warp_normalize_batch");
}

FDB_API int fdb_cls_flip(const void* probs, int dtype, long long ld, int n, int ncls, float thresh, int* flip, int* label,
                         float* score, void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = (n + 127) / 128;
  switch (dtype) {
    case kF32: cls_flip_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float*>(probs), ld, n, ncls, thresh, flip, label, score); break;
    case kF16: cls_flip_kernel<__half><<<grid, 128, 0, st>>>(static_cast<const __half*>(probs), ld, n, ncls, thresh, flip, label, score); break;
    case kBF16: cls_flip_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(probs), ld, n, ncls, thresh, flip, label, score); break;
    default: set_error("cls_flip: fp32 / fp16 / bf16 probabilities"); return -1;
  }
  return pp_check("cls_flip");
}

// ------------------------------------------------------------------ hard voxelisation
#include <cub/cub.cuh>

namespace fdb {

struct VoxelGrid {
  float vx, vy, vz, x0, y0, z0;
  int gx, gy, gz;
};

__global__ void voxel_keys_kernel(const float* pts, int n, int c, VoxelGrid g, int* keys, int* vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* p = pts + static_cast<size_t>(i) * c;
  const int ix = static_cast<int>(floorf((p[0] - g.x0) / g.vx));
  const int iy = static_cast<int>(floorf((p[1] - g.y0) / g.vy));
  const int iz = static_cast<int>(floorf((p[2] - g.z0) / g.vz));
  const bool ok = ix >= 0 && ix < g.gx && iy >= 0 && iy < g.gy && iz >= 0 && iz < g.gz;
  keys[i] = ok ? (iz * g.gy + iy) * g.gx + ix : 0x7fffffff;   // points outside the range sort last
  vals[i] = i;
}

// After the stable sort by cell, every cell is a run of ascending point indices. start[p] = p at the
// head of a run, else 0 (an inclusive max-scan then gives every position its run's head);
// creator[i] = 1 for the first point of every cell.
__global__ void voxel_heads_kernel(const int* keys, const int* vals, int n, int* start, int* creator) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  const bool head = keys[p] != 0x7fffffff && (p == 0 || keys[p] != keys[p - 1]);
  start[p] = head ? p : 0;
  if (head) creator[vals[p]] = 1;
}

__global__ void voxel_fill_kernel(const float* pts, int n, int c, VoxelGrid g, const int* keys, const int* vals,
                                  const int* start, const int* creator_scan, int max_points, int max_voxels,
                                  float* voxels, int* coords, int* num) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  const int key = keys[p];
  if (key == 0x7fffffff) return;
  const int head = start[p];
  const int vid = creator_scan[vals[head]];     // cells are numbered by the index of their first point
  if (vid >= max_voxels) return;
  const int rank = p - head;
  if (rank < max_points) {
    const float* src = pts + static_cast<size_t>(vals[p]) * c;
    float* dst = voxels + (static_cast<size_t>(vid) * max_points + rank) * c;
    for (int k = 0; k < c; ++k) dst[k] = src[k];
  }
  if (rank == 0) {
    const int ix = key % g.gx, iy = (key / g.gx) % g.gy, iz = key / (g.gx * g.gy);
    coords[3 * vid] = iz; coords[3 * vid + 1] = iy; coords[3 * vid + 2] = ix;
  }
  if (p + 1 == n || keys[p + 1] != key) num[vid] = min(rank + 1, max_points);
}

__global__ void voxel_count_kernel(const int* creator_scan, const int* creator, int n, int max_voxels, int* count) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *count = min(creator_scan[n - 1] + creator[n - 1], max_voxels);
}

static size_t voxel_cub_bytes(int n) {
  size_t a = 0, b = 0, c = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr, n);
  cub::DeviceScan::InclusiveScan(nullptr, b, (const int*)nullptr, (int*)nullptr, cub::Max(), n);
  cub::DeviceScan::ExclusiveSum(nullptr, c, (const int*)nullptr, (int*)nullptr, n);
  return std::max(a, std::max(b, c));
}

}  // namespace fdb

// Bytes of scratch fdb_hard_voxelize needs for n points (seven int arrays of n plus the sort / scan space).
FDB_API long long fdb_hard_voxelize_workspace(int n) {
  const size_t arr = (static_cast<size_t>(n) * 4 + 255) / 256 * 256;
  return static_cast<long long>(7 * arr + (voxel_cub_bytes(n) + 255) / 256 * 256);
}

// points [n, c] fp32 (x, y, z first) -> voxels [max_voxels, max_points, c] (zero filled), coords [max_voxels, 3]
// as (z, y, x), num [max_voxels], count [1]. grid9 = voxel size (3), range minimum (3), grid cells (3, as floats).
// Deterministic: voxel v is the v-th distinct cell in order of its first point; points keep their input order.
FDB_API int fdb_hard_voxelize(const float* pts, int n, int c, const float* grid9, int max_points, int max_voxels,
                              float* voxels, int* coords, int* num, int* count, void* workspace, long long ws_bytes,
                              void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n <= 0 || c < 3 || max_points < 1 || max_voxels < 1) { set_error("hard_voxelize: bad shape"); return -1; }
  if (ws_bytes < fdb_hard_voxelize_workspace(n)) { set_error("hard_voxelize: workspace too small"); return -1; }
  VoxelGrid g{grid9[0], grid9[1], grid9[2], grid9[3], grid9[4], grid9[5], (int)grid9[6], (int)grid9[7], (int)grid9[8]};
  if (static_cast<long long>(g.gx) * g.gy * g.gz >= 0x7fffffffLL) { set_error("hard_voxelize: grid too large"); return -1; }
  const size_t arr = (static_cast<size_t>(n) * 4 + 255) / 256 * 256;
  char* w = static_cast<char*>(workspace);
  int* keys = reinterpret_cast<int*>(w);            int* vals = reinterpret_cast<int*>(w + arr);
  int* keys_s = reinterpret_cast<int*>(w + 2 * arr); int* vals_s = reinterpret_cast<int*>(w + 3 * arr);
  int* start = reinterpret_cast<int*>(w + 4 * arr);  int* creator = reinterpret_cast<int*>(w + 5 * arr);
  int* scan = reinterpret_cast<int*>(w + 6 * arr);
  void* tmp = w + 7 * arr;
  size_t tmp_bytes = static_cast<size_t>(ws_bytes) - 7 * arr;
  const int blocks = (n + 255) / 256;
  FDB_CUDA_OK(cudaMemsetAsync(voxels, 0, static_cast<size_t>(max_voxels) * max_points * c * 4, st));
  FDB_CUDA_OK(cudaMemsetAsync(coords, 0, static_cast<size_t>(max_voxels) * 3 * 4, st));
  FDB_CUDA_OK(cudaMemsetAsync(num, 0, static_cast<size_t>(max_voxels) * 4, st));
  FDB_CUDA_OK(cudaMemsetAsync(creator, 0, static_cast<size_t>(n) * 4, st));
  voxel_keys_kernel<<<blocks, 256, 0, st>>>(pts, n, c, g, keys, vals);
  FDB_CUDA_OK(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, keys, keys_s, vals, vals_s, n, 0, 32, st));
  voxel_heads_kernel<<<blocks, 256, 0, st>>>(keys_s, vals_s, n, start, creator);
  FDB_CUDA_OK(cub::DeviceScan::InclusiveScan(tmp, tmp_bytes, start, start, cub::Max(), n, st));
  FDB_CUDA_OK(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, creator, scan, n, st));
  voxel_fill_kernel<<<blocks, 256, 0, st>>>(pts, n, c, g, keys_s, vals_s, start, scan, max_points, max_voxels, voxels,
                                           coords, num);
  voxel_count_kernel<<<1, 32, 0, st>>>(scan, creator, n, max_voxels, count);
  return pp_check("hard_voxelize");
}
