// DB (differentiable binarisation) text-detection post-processing on the device: probability map ->
// quadrilateral boxes, with no pixel leaving the GPU.
//
//   1. threshold (optionally the 2x2 dilation of the binary map);
//   2. connected components, 8-connectivity, by union-find with atomicMin links;
//   3. per component: bounding box, pixel count, probability sum;
//   4. per component and image column: the top-most and bottom-most pixel - the convex hull of a component
//      is the hull of these column extremes, so no contour tracing is needed;
//   5. one warp per component: monotone-chain hull, minimum-area rectangle over the hull's edge directions
//      (the optimum has a side collinear with a hull edge), score, "unclip" (grow by area * ratio / perimeter),
//      clockwise corner order, scaling to the source image, size filters.
//
// The reference does this on the host with OpenCV and Clipper: findContours -> minAreaRect -> polygon score
// -> Clipper offset -> minAreaRect -> order / clip (fastdeploy/vision/ocr/ppocr/utils/ocr_postprocess_op.cc:23-350,
// fastdeploy/vision/ocr/ppocr/det_postprocessor.cc:27-70). Offsetting a rectangle and taking the minimum-area
// rectangle of the result is the same rectangle grown by the offset on every side, which is what step 5 computes.
#include "fdb_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

namespace fdb {

struct DbParams {
  const void* prob;        // [N] images of H x W probabilities
  int dtype;               // kF32 / kF16 / kBF16
  long long px_stride, row_stride, img_stride;   // in elements
  int N, H, W;
  const int* info;         // [N, 4] = source width, source height, valid width, valid height of the map
  float thresh, box_thresh, unclip_ratio;
  int dilate, score_fast, max_candidates;
  // scratch, per image
  int* label;              // [N, H*W]
  int* cid;                // [N, H*W] component index at root pixels
  int* ncomp;              // [N]
  int* stats;              // [N, max_candidates, 8] = x0, x1, y0, y1, count, col offset, hull size, unused
  unsigned long long* psum; // [N, max_candidates] probability sums in 2^-20 fixed point
  int* colmin;             // [N, H*W]
  int* colmax;             // [N, H*W]
  int* hull;               // [N, 2*H*W + 8*max_candidates] packed (x << 16 | y)
  // results
  int* out_boxes;          // [N, max_candidates, 8]
  float* out_scores;       // [N, max_candidates]
  int* out_count;          // [N]
};

__device__ __forceinline__ float db_prob(const DbParams& p, int n, int y, int x) {
  const long long off = n * p.img_stride + y * p.row_stride + x * p.px_stride;
  switch (p.dtype) {
    case kF16: return __half2float(static_cast<const __half*>(p.prob)[off]);
    case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p.prob)[off]);
    default: return static_cast<const float*>(p.prob)[off];
  }
}

__device__ __forceinline__ bool db_fg(const DbParams& p, int n, int y, int x, int rw, int rh) {
  if (x < 0 || y < 0 || x >= rw || y >= rh) return false;
  if (!p.dilate) return db_prob(p, n, y, x) > p.thresh;
  // 2x2 structuring element anchored at its lower-right cell: a pixel is set when any of (x-1..x, y-1..y) is
  for (int dy = -1; dy <= 0; ++dy)
    for (int dx = -1; dx <= 0; ++dx) {
      const int xx = x + dx, yy = y + dy;
      if (xx >= 0 && yy >= 0 && db_prob(p, n, yy, xx) > p.thresh) return true;
    }
  return false;
}

__device__ __forceinline__ int db_find(const int* label, int i) {
  int r = i;
  // bounded walk: a chain is never longer than the pixel count; the bound only guards against corrupted links
  for (int it = 0; it < (1 << 22); ++it) {
    const int q = label[r];
    if (q == r) break;
    r = q;
  }
  return r;
}

__device__ __forceinline__ void db_union(int* label, int a, int b) {
  for (int it = 0; it < (1 << 22); ++it) {
    a = db_find(label, a);
    b = db_find(label, b);
    if (a == b) return;
    if (a < b) { const int t = a; a = b; b = t; }       // link the larger root under the smaller
    const int old = atomicMin(&label[a], b);
    if (old == a) return;
    a = old;
  }
}

// Labels start as "first pixel of my horizontal run inside this warp's 32-pixel segment": runs are merged without a
// single atomic, and only run heads and run-to-run contacts are left for the union step.
__global__ void db_init_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  const int rw = p.info[n * 4 + 2], rh = p.info[n * 4 + 3];
  const int lane = threadIdx.x & 31;
  const int hw32 = (hw + 31) & ~31;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hw32; i += gridDim.x * blockDim.x) {
    const int y = i / p.W, x = i - y * p.W;
    const bool fg = i < hw && db_fg(p, n, y, x, rw, rh);
    // a run may not continue across a row boundary that falls inside the segment
    const unsigned fgm = __ballot_sync(0xffffffffu, fg);
    const unsigned row_start = __ballot_sync(0xffffffffu, x == 0);
    if (i < hw) {
      int lab = -1;
      if (fg) {
        const unsigned below = (lane == 0) ? 0u : (0xffffffffu >> (32 - lane));      // lanes < mine
        const unsigned breaks = (~fgm | (row_start & ~1u)) & below;                   // background, or a row start
        // a row start at lane k ends the previous run at k - 1: the run containing me begins at the highest break
        // that is background (+1) or at the highest row start
        int start = 0;
        if (breaks != 0u) {
          const int hb = 31 - __clz(breaks);
          start = ((fgm >> hb) & 1u) ? hb : hb + 1;       // hb is fg only when it is a row start
        }
        if ((row_start >> lane) & 1u) start = lane;
        lab = i - lane + start;
      }
      p.label[static_cast<long long>(n) * hw + i] = lab;
      p.cid[static_cast<long long>(n) * hw + i] = -1;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) { p.ncomp[n] = 0; p.out_count[n] = 0; }
}

// Unions only where they can connect something new: the first pixel of a segment with the pixel to its left (a run
// that crosses the segment boundary), and contacts with the row above that the neighbour to the left has not already made.
__global__ void db_merge_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  int* label = p.label + static_cast<long long>(n) * hw;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hw; i += gridDim.x * blockDim.x) {
    if (label[i] < 0) continue;
    const int y = i / p.W, x = i - y * p.W;
    const bool w_fg = x > 0 && label[i - 1] >= 0;
    if (w_fg && (i & 31) == 0) db_union(label, i, i - 1);     // the run continues across the segment boundary
    if (y > 0) {
      const bool n_fg = label[i - p.W] >= 0;
      const bool nw_fg = x > 0 && label[i - p.W - 1] >= 0;
      const bool ne_fg = x + 1 < p.W && label[i - p.W + 1] >= 0;
      // N: unless W and NW are both set (then W is already tied to NW, which shares N's run)
      if (n_fg && !(w_fg && nw_fg)) db_union(label, i, i - p.W);
      // NW: only when neither N (same run as NW) nor W (directly below NW) makes the link
      if (nw_fg && !n_fg && !w_fg) db_union(label, i, i - p.W - 1);
      // NE: only when N is background (otherwise NE shares N's run)
      if (ne_fg && !n_fg) db_union(label, i, i - p.W + 1);
    }
  }
}

// path compression: every pixel points at its root, so that the later passes read one link
__global__ void db_flatten_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  int* label = p.label + static_cast<long long>(n) * hw;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hw; i += gridDim.x * blockDim.x) {
    if (label[i] < 0) continue;
    label[i] = db_find(label, i);
  }
}

__global__ void db_roots_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  int* label = p.label + static_cast<long long>(n) * hw;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hw; i += gridDim.x * blockDim.x) {
    if (label[i] != i) continue;
    const int c = atomicAdd(&p.ncomp[n], 1);
    if (c < p.max_candidates) {
      p.cid[static_cast<long long>(n) * hw + i] = c;
      int* st = p.stats + (static_cast<long long>(n) * p.max_candidates + c) * 8;
      st[0] = 0x7fffffff; st[1] = -1; st[2] = 0x7fffffff; st[3] = -1; st[4] = 0; st[5] = 0; st[6] = 0; st[7] = 0;
      p.psum[static_cast<long long>(n) * p.max_candidates + c] = 0ull;
    }
  }
}

// Lanes of a warp that sit in the same component (the common case: 32 neighbouring pixels of a text line) combine
// their contribution with masked warp reductions, so a component receives one set of atomics per warp, not per pixel.
// The probability sum is kept in 2^-20 fixed point: exact, and independent of the order of the additions.
__global__ void db_stats_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  const int* label = p.label + static_cast<long long>(n) * hw;
  const int lane = threadIdx.x & 31;
  const int hw32 = (hw + 31) & ~31;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hw32; i += gridDim.x * blockDim.x) {
    int c = -1, x = 0, y = 0;
    if (i < hw && label[i] >= 0) {
      c = p.cid[static_cast<long long>(n) * hw + label[i]];
      y = i / p.W;
      x = i - y * p.W;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, c);
    if (c < 0) continue;
    const int xmin = __reduce_min_sync(peers, x), xmax = __reduce_max_sync(peers, x);
    const int ymin = __reduce_min_sync(peers, y), ymax = __reduce_max_sync(peers, y);
    const unsigned fx = static_cast<unsigned>(fminf(fmaxf(db_prob(p, n, y, x), 0.f), 1.f) * 1048576.f + 0.5f);
    const unsigned fsum = __reduce_add_sync(peers, fx);
    if (lane == __ffs(peers) - 1) {
      int* st = p.stats + (static_cast<long long>(n) * p.max_candidates + c) * 8;
      atomicMin(&st[0], xmin); atomicMax(&st[1], xmax); atomicMin(&st[2], ymin); atomicMax(&st[3], ymax);
      atomicAdd(&st[4], __popc(peers));
      atomicAdd(&p.psum[static_cast<long long>(n) * p.max_candidates + c], static_cast<unsigned long long>(fsum));
    }
  }
}

// one block per image: exclusive scan of the bounding-box widths -> column offsets; clears the column extremes
__global__ void __launch_bounds__(1024) db_offsets_kernel(DbParams p) {
  const int n = blockIdx.x;
  const int nc = min(p.ncomp[n], p.max_candidates);
  int* st = p.stats + static_cast<long long>(n) * p.max_candidates * 8;
  __shared__ int carry;
  __shared__ int warp_sums[32];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < nc; base += blockDim.x) {
    const int c = base + threadIdx.x;
    const int wv = c < nc ? st[c * 8 + 1] - st[c * 8 + 0] + 1 : 0;
    int v = wv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int s = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += t;
      }
      warp_sums[lane] = s;
    }
    __syncthreads();
    const int incl = v + (warp > 0 ? warp_sums[warp - 1] : 0);
    if (c < nc) st[c * 8 + 5] = carry + incl - wv;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry += incl;
    __syncthreads();
  }
}

__global__ void db_cols_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  const int* label = p.label + static_cast<long long>(n) * hw;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hw; i += gridDim.x * blockDim.x) {
    if (label[i] < 0) continue;
    const int c = p.cid[static_cast<long long>(n) * hw + label[i]];
    if (c < 0) continue;
    const int y = i / p.W, x = i - y * p.W;
    const int* st = p.stats + (static_cast<long long>(n) * p.max_candidates + c) * 8;
    const long long col = static_cast<long long>(n) * hw + st[5] + (x - st[0]);
    atomicMin(&p.colmin[col], y);
    atomicMax(&p.colmax[col], y);
  }
}

struct P2 { float x, y; };
__device__ __forceinline__ P2 unpack_pt(int v) { return P2{static_cast<float>(v >> 16), static_cast<float>(v & 0xffff)}; }
__device__ __forceinline__ long long cross_i(int o, int a, int b) {
  const long long ox = o >> 16, oy = o & 0xffff, ax = a >> 16, ay = a & 0xffff, bx = b >> 16, by = b & 0xffff;
  return (ax - ox) * (by - oy) - (ay - oy) * (bx - ox);
}

// corners of the rectangle with axis u (unit), normal v, extents [p0, p1] x [q0, q1]
__device__ __forceinline__ void rect_corners(float ux, float uy, float p0, float p1, float q0, float q1, P2 out[4]) {
  const float vx = -uy, vy = ux;
  out[0] = P2{ux * p0 + vx * q0, uy * p0 + vy * q0};
  out[1] = P2{ux * p1 + vx * q0, uy * p1 + vy * q0};
  out[2] = P2{ux * p1 + vx * q1, uy * p1 + vy * q1};
  out[3] = P2{ux * p0 + vx * q1, uy * p0 + vy * q1};
}

// mini-box order: sort by x (stable), the left pair by y, the right pair by y -> left-top, right-top, right-bottom,
// left-bottom
__device__ __forceinline__ void order_clockwise(P2 pts[4]) {
  for (int i = 1; i < 4; ++i) {          // insertion sort by x keeps equal keys in order
    const P2 k = pts[i];
    int j = i - 1;
    while (j >= 0 && pts[j].x > k.x) { pts[j + 1] = pts[j]; --j; }
    pts[j + 1] = k;
  }
  if (pts[0].y > pts[1].y) { const P2 t = pts[0]; pts[0] = pts[1]; pts[1] = t; }
  if (pts[2].y > pts[3].y) { const P2 t = pts[2]; pts[2] = pts[3]; pts[3] = t; }
  const P2 l0 = pts[0], l1 = pts[1], r0 = pts[2], r1 = pts[3];
  pts[0] = l0; pts[1] = r0; pts[2] = r1; pts[3] = l1;
}

__device__ __forceinline__ bool inside_quad(const P2 q[4], float x, float y) {
  // convex quad in either orientation: all edge cross products share a sign (zero counts as inside)
  bool pos = false, neg = false;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const P2 a = q[k], b = q[(k + 1) & 3];
    const float c = (b.x - a.x) * (y - a.y) - (b.y - a.y) * (x - a.x);
    pos |= c > 0.f;
    neg |= c < 0.f;
  }
  return !(pos && neg);
}

__global__ void __launch_bounds__(128) db_boxes_kernel(DbParams p) {
  const int n = blockIdx.y, hw = p.H * p.W;
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int nc = min(p.ncomp[n], p.max_candidates);
  if (c >= nc) return;
  int* st = p.stats + (static_cast<long long>(n) * p.max_candidates + c) * 8;
  const int x0 = st[0], x1 = st[1], count = st[4], off = st[5];
  const int wcols = x1 - x0 + 1;
  const int* cmin = p.colmin + static_cast<long long>(n) * hw + off;
  const int* cmax = p.colmax + static_cast<long long>(n) * hw + off;
  // every component owns 2 * (its column count) + 8 hull slots: a strictly convex x-monotone chain has at most one
  // point per column plus a vertical edge at either end, and the lower and upper chains share the array
  int* hull = p.hull + static_cast<long long>(n) * (2LL * hw + 8LL * p.max_candidates) + 2LL * off + 8LL * c;
  int h = 0;
  if (lane == 0) {
    // Andrew's monotone chain over the column extremes, which are already sorted by x
    for (int k = 0; k < wcols; ++k) {                     // chain with non-negative turns (lower in image = larger y)
      const int a = ((x0 + k) << 16) | cmin[k];
      while (h >= 2 && cross_i(hull[h - 2], hull[h - 1], a) <= 0) --h;
      hull[h++] = a;
      const int b = ((x0 + k) << 16) | cmax[k];
      if (b != a) {
        while (h >= 2 && cross_i(hull[h - 2], hull[h - 1], b) <= 0) --h;
        hull[h++] = b;
      }
    }
    const int lower = h + 1;
    for (int k = wcols - 1; k >= 0; --k) {
      const int b = ((x0 + k) << 16) | cmax[k];
      if (!(k == wcols - 1 && hull[h - 1] == b)) {
        while (h >= lower && cross_i(hull[h - 2], hull[h - 1], b) <= 0) --h;
        hull[h++] = b;
      }
      const int a = ((x0 + k) << 16) | cmin[k];
      if (a != b) {
        while (h >= lower && cross_i(hull[h - 2], hull[h - 1], a) <= 0) --h;
        hull[h++] = a;
      }
    }
    if (h > 1 && hull[h - 1] == hull[0]) --h;           // the chain closes on its first point
    st[6] = h;
  }
  h = __shfl_sync(0xffffffffu, h, 0);
  __syncwarp();
  if (count <= 2 || h < 3) return;                        // a contour of one or two points, or a straight line
  // minimum-area rectangle: one candidate per hull edge
  float best_area = INFINITY;
  int best_e = -1;
  for (int e = lane; e < h; e += 32) {
    const P2 a = unpack_pt(hull[e]), b = unpack_pt(hull[(e + 1) % h]);
    float ux = b.x - a.x, uy = b.y - a.y;
    const float len = sqrtf(ux * ux + uy * uy);
    if (len < 1e-6f) continue;
    ux /= len; uy /= len;
    float p0 = INFINITY, p1 = -INFINITY, q0 = INFINITY, q1 = -INFINITY;
    for (int k = 0; k < h; ++k) {
      const P2 t = unpack_pt(hull[k]);
      const float pp = t.x * ux + t.y * uy, qq = -t.x * uy + t.y * ux;
      p0 = fminf(p0, pp); p1 = fmaxf(p1, pp); q0 = fminf(q0, qq); q1 = fmaxf(q1, qq);
    }
    const float area = (p1 - p0) * (q1 - q0);
    if (area < best_area) { best_area = area; best_e = e; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, best_area, o);
    const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
    if (oe >= 0 && (best_e < 0 || oa < best_area || (oa == best_area && oe < best_e))) { best_area = oa; best_e = oe; }
  }
  if (best_e < 0) return;
  // every lane recomputes the winning rectangle (cheap) so that the score loop below can be shared
  const P2 ea = unpack_pt(hull[best_e]), eb = unpack_pt(hull[(best_e + 1) % h]);
  float ux = eb.x - ea.x, uy = eb.y - ea.y;
  const float len = sqrtf(ux * ux + uy * uy);
  ux /= len; uy /= len;
  float p0 = INFINITY, p1 = -INFINITY, q0 = INFINITY, q1 = -INFINITY;
  for (int k = 0; k < h; ++k) {
    const P2 t = unpack_pt(hull[k]);
    const float pp = t.x * ux + t.y * uy, qq = -t.x * uy + t.y * ux;
    p0 = fminf(p0, pp); p1 = fmaxf(p1, pp); q0 = fminf(q0, qq); q1 = fmaxf(q1, qq);
  }
  const float rw_ = p1 - p0, rh_ = q1 - q0;
  if (fminf(rw_, rh_) < 3.f) return;
  float score;
  if (p.score_fast) {
    // mean probability over the pixels of the (integer-cast) box polygon
    P2 box[4];
    rect_corners(ux, uy, p0, p1, q0, q1, box);
    order_clockwise(box);
    float bx0 = INFINITY, bx1 = -INFINITY, by0 = INFINITY, by1 = -INFINITY;
    for (int k = 0; k < 4; ++k) {
      bx0 = fminf(bx0, box[k].x); bx1 = fmaxf(bx1, box[k].x); by0 = fminf(by0, box[k].y); by1 = fmaxf(by1, box[k].y);
    }
    const int vw = p.info[n * 4 + 2], vh = p.info[n * 4 + 3];
    const int xa = min(max(static_cast<int>(floorf(bx0)), 0), vw - 1), xb = min(max(static_cast<int>(ceilf(bx1)), 0), vw - 1);
    const int ya = min(max(static_cast<int>(floorf(by0)), 0), vh - 1), yb = min(max(static_cast<int>(ceilf(by1)), 0), vh - 1);
    P2 ib[4];
    for (int k = 0; k < 4; ++k) ib[k] = P2{truncf(box[k].x), truncf(box[k].y)};
    float s = 0.f;
    int cnt = 0;
    const int bw = xb - xa + 1, tot = bw * (yb - ya + 1);
    for (int i = lane; i < tot; i += 32) {
      const int yy = ya + i / bw, xx = xa + i % bw;
      if (inside_quad(ib, static_cast<float>(xx), static_cast<float>(yy))) { s += db_prob(p, n, yy, xx); ++cnt; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    }
    score = cnt > 0 ? s / cnt : 0.f;
  } else {
    // mean over the component's pixels
    score = static_cast<float>(static_cast<double>(p.psum[static_cast<long long>(n) * p.max_candidates + c]) / 1048576.0 / count);
  }
  if (lane != 0 || score < p.box_thresh) return;
  // grow by area * ratio / perimeter on every side
  const float peri = 2.f * (rw_ + rh_);
  if (peri < 1e-6f) return;
  const float d = rw_ * rh_ * p.unclip_ratio / peri;
  if (fminf(rw_ + 2.f * d, rh_ + 2.f * d) < 5.f) return;
  P2 g[4];
  rect_corners(ux, uy, p0 - d, p1 + d, q0 - d, q1 + d, g);
  order_clockwise(g);
  const int src_w = p.info[n * 4 + 0], src_h = p.info[n * 4 + 1], mw = p.info[n * 4 + 2], mh = p.info[n * 4 + 3];
  int q[8];
  for (int k = 0; k < 4; ++k) {
    q[2 * k] = min(max(static_cast<int>(rintf(g[k].x / mw * src_w)), 0), src_w - 1);
    q[2 * k + 1] = min(max(static_cast<int>(rintf(g[k].y / mh * src_h)), 0), src_h - 1);
  }
  const int bw = static_cast<int>(hypotf(static_cast<float>(q[0] - q[2]), static_cast<float>(q[1] - q[3])));
  const int bh = static_cast<int>(hypotf(static_cast<float>(q[0] - q[6]), static_cast<float>(q[1] - q[7])));
  if (bw <= 4 || bh <= 4) return;
  const int slot = atomicAdd(&p.out_count[n], 1);
  int* ob = p.out_boxes + (static_cast<long long>(n) * p.max_candidates + slot) * 8;
  for (int k = 0; k < 8; ++k) ob[k] = q[k];
  p.out_scores[static_cast<long long>(n) * p.max_candidates + slot] = score;
}

}  // namespace fdb

using namespace fdb;

// Scratch bytes for N maps of H x W with at most max_candidates components each.
FDB_API long long fdb_db_postprocess_workspace(int N, int H, int W, int max_candidates) {
  const long long hw = static_cast<long long>(H) * W;
  const long long ints = N * (hw * 4 + (2 * hw + 8LL * max_candidates) + max_candidates * 8LL + 1) + 64;
  const long long sums = static_cast<long long>(N) * max_candidates;
  return ints * 4 + sums * 8 + 1024;
}

// prob: N maps (dtype code, element strides); info: device int32 [N, 4] = source w, source h, valid map w, valid map h.
// out_boxes int32 [N, max_candidates, 8] (x0 y0 .. x3 y3 clockwise from the top-left corner, source pixels),
// out_scores fp32 [N, max_candidates], out_count int32 [N]. Boxes of an image come in no particular order.
FDB_API int fdb_db_postprocess(const void* prob, int dtype, long long px_stride, long long row_stride, long long img_stride,
                               int N, int H, int W, const int* info, float thresh, float box_thresh, float unclip_ratio,
                               int dilate, int score_fast, int max_candidates, void* workspace, long long workspace_bytes,
                               int* out_boxes, float* out_scores, int* out_count, cudaStream_t stream) {
  if (N < 1 || H < 1 || W < 1 || H > 32767 || W > 32767 || static_cast<long long>(H) * W > (1LL << 30)) {
    set_error("db_postprocess: bad map size");
    return -1;
  }
  if (max_candidates < 1 || max_candidates > 65536) { set_error("db_postprocess: max_candidates out of range"); return -1; }
  if (dtype != kF32 && dtype != kF16 && dtype != kBF16) { set_error("db_postprocess: fp32 / fp16 / bf16 maps"); return -1; }
  if (workspace_bytes < fdb_db_postprocess_workspace(N, H, W, max_candidates)) {
    set_error("db_postprocess: workspace too small");
    return -1;
  }
  const long long hw = static_cast<long long>(H) * W;
  DbParams p{};
  p.prob = prob; p.dtype = dtype; p.px_stride = px_stride; p.row_stride = row_stride; p.img_stride = img_stride;
  p.N = N; p.H = H; p.W = W; p.info = info;
  p.thresh = thresh; p.box_thresh = box_thresh; p.unclip_ratio = unclip_ratio;
  p.dilate = dilate; p.score_fast = score_fast; p.max_candidates = max_candidates;
  int* w = static_cast<int*>(workspace);
  p.label = w; w += N * hw;
  p.cid = w; w += N * hw;
  p.colmin = w; w += N * hw;
  p.colmax = w; w += N * hw;
  p.hull = w; w += N * (2 * hw + 8LL * max_candidates);
  p.stats = w; w += static_cast<long long>(N) * max_candidates * 8;
  p.ncomp = w; w += N;
  w += (4 - (N & 3)) & 3;
  p.psum = reinterpret_cast<unsigned long long*>(w);
  p.out_boxes = out_boxes; p.out_scores = out_scores; p.out_count = out_count;
  FDB_CUDA_OK(cudaMemsetAsync(p.colmin, 0x7f, N * hw * sizeof(int), stream));
  FDB_CUDA_OK(cudaMemsetAsync(p.colmax, 0xff, N * hw * sizeof(int), stream));
  const int bx = static_cast<int>(std::min<long long>((hw + 255) / 256, 148 * 8));
  const dim3 grid(bx, N);
  db_init_kernel<<<grid, 256, 0, stream>>>(p);
  db_merge_kernel<<<grid, 256, 0, stream>>>(p);
  db_flatten_kernel<<<grid, 256, 0, stream>>>(p);
  db_roots_kernel<<<grid, 256, 0, stream>>>(p);
  db_stats_kernel<<<grid, 256, 0, stream>>>(p);
  db_offsets_kernel<<<N, 1024, 0, stream>>>(p);
  db_cols_kernel<<<grid, 256, 0, stream>>>(p);
  db_boxes_kernel<<<dim3((max_candidates + 3) / 4, N), 128, 0, stream>>>(p);
  FDB_CUDA_OK(cudaGetLastError());
  return 0;
}
