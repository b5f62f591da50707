// Rasterisers for result visualisation and for matting / segmentation compositing, on interleaved
// uint8 BGR frames that already live on the device (headless: the output is a device buffer).
//
//   draw_boxes        rectangle outlines of a given thickness, one colour per box (boxes are drawn
//                     concurrently: where outlines of different boxes cross, either colour may win)
//   blend_label_map   per-pixel class map -> colour table, alpha-blended over the frame
//   blend_masks       per-instance binary masks alpha-blended with the instance colour
//   draw_points       filled discs (key points, landmarks)
//   draw_segments     thick line segments (skeleton limbs, polygon edges)
//   box_blur_h / _v   separable box blur (background blur of the portrait mode)
//   composite         out = alpha * foreground + (1 - alpha) * background with alpha taken from a
//                     float matte, a thresholded matte or a label map; background is an image, a
//                     blurred copy of the frame or a constant colour
//
// Reference behaviour: fastdeploy/vision/visualize/{detection,segmentation,matting,swap_background,
// keypoint,face_detection}.cc draw with OpenCV on the host; the compositing modes follow
// swap_background.cc:25-130 and the browser demo examples/application/js/.../humanseg (blur radius,
// mask threshold).
#include "fdb_common.h"

namespace fdb {

__global__ void draw_boxes_kernel(uint8_t* img, int H, int W, const float* boxes, const uint8_t* colors, int n, int thick) {
  const int b = blockIdx.y;
  if (b >= n) return;
  // edges that fall outside the frame are not drawn (the box is clipped, not clamped), but coordinates
  // are limited to one frame size around it so that absurd boxes cannot make the loops long
  const int x1 = max(-W, __float2int_rn(boxes[4 * b])), y1 = max(-H, __float2int_rn(boxes[4 * b + 1]));
  const int x2 = min(2 * W, __float2int_rn(boxes[4 * b + 2])), y2 = min(2 * H, __float2int_rn(boxes[4 * b + 3]));
  if (x2 < x1 || y2 < y1) return;
  const int bw = x2 - x1 + 1, bh = y2 - y1 + 1;
  const int t = min(thick, min(bw, bh));
  // perimeter pixels: two horizontal bands of bw x t and two vertical bands of t x (bh - 2t)
  const int band_h = bw * t, band_v = t * max(bh - 2 * t, 0);
  const int total = 2 * band_h + 2 * band_v;
  const uint8_t c0 = colors[3 * b], c1 = colors[3 * b + 1], c2 = colors[3 * b + 2];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    int x, y;
    if (i < band_h) { y = y1 + i / bw; x = x1 + i % bw; }
    else if (i < 2 * band_h) { const int j = i - band_h; y = y2 - j / bw; x = x1 + j % bw; }
    else if (i < 2 * band_h + band_v) { const int j = i - 2 * band_h; y = y1 + t + j / t; x = x1 + j % t; }
    else { const int j = i - 2 * band_h - band_v; y = y1 + t + j / t; x = x2 - j % t; }
    if (x < 0 || y < 0 || x >= W || y >= H) continue;
    uint8_t* p = img + (static_cast<size_t>(y) * W + x) * 3;
    p[0] = c0; p[1] = c1; p[2] = c2;
  }
}

__global__ void blend_label_map_kernel(uint8_t* img, const int* labels, const uint8_t* table, int n_colors, int npix,
                                       float weight, int skip_label) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < npix; i += gridDim.x * blockDim.x) {
    const int l = labels[i];
    if (l == skip_label || l < 0) continue;
    const uint8_t* c = table + 3 * (l % n_colors);
    uint8_t* p = img + static_cast<size_t>(i) * 3;
#pragma unroll
    for (int k = 0; k < 3; ++k) p[k] = static_cast<uint8_t>(__float2int_rn(p[k] * (1.f - weight) + c[k] * weight));
  }
}

// masks: [n][bh_max][bw_max] is awkward for ragged boxes, so each mask is full-frame uint8 [n][H][W]
__global__ void blend_masks_kernel(uint8_t* img, const uint8_t* masks, const uint8_t* colors, int n, int npix, float weight) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < npix; i += gridDim.x * blockDim.x) {
    uint8_t* p = img + static_cast<size_t>(i) * 3;
    for (int m = 0; m < n; ++m) {
      if (masks[static_cast<size_t>(m) * npix + i] == 0) continue;
      const uint8_t* c = colors + 3 * m;
#pragma unroll
      for (int k = 0; k < 3; ++k) p[k] = static_cast<uint8_t>(__float2int_rn(p[k] * (1.f - weight) + c[k] * weight));
    }
  }
}

__global__ void draw_points_kernel(uint8_t* img, int H, int W, const float* pts, const uint8_t* colors, int n, int radius) {
  const int k = blockIdx.y;
  if (k >= n) return;
  const int cx = __float2int_rn(pts[2 * k]), cy = __float2int_rn(pts[2 * k + 1]);
  const int side = 2 * radius + 1;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < side * side; i += gridDim.x * blockDim.x) {
    const int dx = i % side - radius, dy = i / side - radius;
    if (dx * dx + dy * dy > radius * radius) continue;
    const int x = cx + dx, y = cy + dy;
    if (x < 0 || y < 0 || x >= W || y >= H) continue;
    uint8_t* p = img + (static_cast<size_t>(y) * W + x) * 3;
    p[0] = colors[3 * k]; p[1] = colors[3 * k + 1]; p[2] = colors[3 * k + 2];
  }
}

__global__ void draw_segments_kernel(uint8_t* img, int H, int W, const float* segs, const uint8_t* colors, int n, int thick) {
  const int k = blockIdx.y;
  if (k >= n) return;
  const float x0 = segs[4 * k], y0 = segs[4 * k + 1], x1 = segs[4 * k + 2], y1 = segs[4 * k + 3];
  const float r = 0.5f * thick;
  const int bx0 = max(0, static_cast<int>(floorf(fminf(x0, x1) - r))), bx1 = min(W - 1, static_cast<int>(ceilf(fmaxf(x0, x1) + r)));
  const int by0 = max(0, static_cast<int>(floorf(fminf(y0, y1) - r))), by1 = min(H - 1, static_cast<int>(ceilf(fmaxf(y0, y1) + r)));
  if (bx1 < bx0 || by1 < by0) return;
  const int bw = bx1 - bx0 + 1, bh = by1 - by0 + 1;
  const float dx = x1 - x0, dy = y1 - y0, len2 = fmaxf(dx * dx + dy * dy, 1e-6f);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < bw * bh; i += gridDim.x * blockDim.x) {
    const int x = bx0 + i % bw, y = by0 + i / bw;
    const float t = fminf(fmaxf(((x - x0) * dx + (y - y0) * dy) / len2, 0.f), 1.f);
    const float ex = x - (x0 + t * dx), ey = y - (y0 + t * dy);
    if (ex * ex + ey * ey > r * r + 0.25f) continue;
    uint8_t* p = img + (static_cast<size_t>(y) * W + x) * 3;
    p[0] = colors[3 * k]; p[1] = colors[3 * k + 1]; p[2] = colors[3 * k + 2];
  }
}

// one thread per output pixel and channel; running sums would be faster for huge radii, the radii used
// for portrait blur (<= 32) keep this bandwidth bound through L1
__global__ void box_blur_kernel(const uint8_t* src, uint8_t* dst, int H, int W, int radius, int vertical) {
  const int n = H * W * 3;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int c = i % 3, x = (i / 3) % W, y = i / (3 * W);
    int acc = 0, cnt = 0;
    for (int d = -radius; d <= radius; ++d) {
      const int xx = vertical ? x : x + d, yy = vertical ? y + d : y;
      if (xx < 0 || yy < 0 || xx >= W || yy >= H) continue;
      acc += src[(static_cast<size_t>(yy) * W + xx) * 3 + c];
      ++cnt;
    }
    dst[i] = static_cast<uint8_t>((acc + cnt / 2) / cnt);
  }
}

// alpha_mode 0: float matte in [0,1]; 1: matte thresholded at `threshold`; 2: int label map, foreground = label `fg_label`
// bg_mode 0: background image; 1: constant colour
__global__ void composite_kernel(const uint8_t* fg, const void* alpha, const uint8_t* bg, uint8_t* out, int npix, int alpha_mode,
                                 float threshold, int fg_label, int bg_mode, uint8_t b0, uint8_t b1, uint8_t b2) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < npix; i += gridDim.x * blockDim.x) {
    float a;
    if (alpha_mode == 2) a = static_cast<const int*>(alpha)[i] == fg_label ? 1.f : 0.f;
    else {
      a = static_cast<const float*>(alpha)[i];
      if (alpha_mode == 1) a = a > threshold ? 1.f : 0.f;
      a = fminf(fmaxf(a, 0.f), 1.f);
    }
    const uint8_t* f = fg + static_cast<size_t>(i) * 3;
    uint8_t bgc[3] = {b0, b1, b2};
    const uint8_t* b = bg_mode == 0 ? bg + static_cast<size_t>(i) * 3 : bgc;
    uint8_t* o = out + static_cast<size_t>(i) * 3;
#pragma unroll
    for (int k = 0; k < 3; ++k) o[k] = static_cast<uint8_t>(__float2int_rn(a * f[k] + (1.f - a) * b[k]));
  }
}

static int vis_done() {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
  return 0;
}
static int vis_grid(long long work) { return static_cast<int>(std::max<long long>(1, std::min<long long>((work + 255) / 256, 8 * sm_count()))); }

}  // namespace fdb

using namespace fdb;

FDB_API int fdb_vis_draw_boxes(void* img, int H, int W, const float* boxes, const uint8_t* colors, int n, int thick, void* stream) {
  if (n <= 0) return 0;
  draw_boxes_kernel<<<dim3(8, n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(img), H, W, boxes, colors, n, thick);
  return vis_done();
}
FDB_API int fdb_vis_blend_label_map(void* img, const int* labels, const uint8_t* table, int n_colors, int H, int W, float weight,
                                    int skip_label, void* stream) {
  blend_label_map_kernel<<<vis_grid(1LL * H * W), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(img), labels, table,
                                                                                              n_colors, H * W, weight, skip_label);
  return vis_done();
}
FDB_API int fdb_vis_blend_masks(void* img, const uint8_t* masks, const uint8_t* colors, int n, int H, int W, float weight, void* stream) {
  if (n <= 0) return 0;
  blend_masks_kernel<<<vis_grid(1LL * H * W), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(img), masks, colors, n,
                                                                                          H * W, weight);
  return vis_done();
}
FDB_API int fdb_vis_draw_points(void* img, int H, int W, const float* pts, const uint8_t* colors, int n, int radius, void* stream) {
  if (n <= 0) return 0;
  draw_points_kernel<<<dim3(1, n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(img), H, W, pts, colors, n, radius);
  return vis_done();
}
FDB_API int fdb_vis_draw_segments(void* img, int H, int W, const float* segs, const uint8_t* colors, int n, int thick, void* stream) {
  if (n <= 0) return 0;
  draw_segments_kernel<<<dim3(4, n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(img), H, W, segs, colors, n, thick);
  return vis_done();
}
FDB_API int fdb_vis_box_blur(const void* src, void* tmp, void* dst, int H, int W, int radius, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  box_blur_kernel<<<vis_grid(3LL * H * W), 256, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(tmp), H, W, radius, 0);
  box_blur_kernel<<<vis_grid(3LL * H * W), 256, 0, s>>>(static_cast<const uint8_t*>(tmp), static_cast<uint8_t*>(dst), H, W, radius, 1);
  return vis_done();
}
FDB_API int fdb_vis_composite(const void* fg, const void* alpha, const void* bg, void* out, int H, int W, int alpha_mode, float threshold,
                              int fg_label, int bg_mode, int b0, int b1, int b2, void* stream) {
  composite_kernel<<<vis_grid(1LL * H * W), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(fg), alpha, static_cast<const uint8_t*>(bg), static_cast<uint8_t*>(out), H * W, alpha_mode, threshold,
      fg_label, bg_mode, static_cast<uint8_t>(b0), static_cast<uint8_t>(b1), static_cast<uint8_t>(b2));
  return vis_done();
}
