// Rotated-box and 3-D perception kernels:
//
//   rotated IoU          exact intersection of two convex quadrilaterals by polygon clipping (device function)
//   rotated_nms          greedy NMS over score-sorted quadrilaterals: 64 x 64 tiles of a suppression bit matrix,
//                        then one block walks the rows in order; optional class ids restrict suppression to boxes of
//                        the same class. Serves the rotated multiclass NMS of PP-YOLOE-R
//                        (fastdeploy/vision/detection/ppdet/multiclass_nms_rotated.cc:59-477) and the bird's-eye-view
//                        NMS of CenterPoint (fastdeploy/runtime/backends/paddle/ops/iou3d_nms_kernel.cu:294-382)
//   multiclass_rotated   score filter -> (class, score) sort -> per-class top-k -> rotated_nms -> keep_top_k
//   centerpoint_decode   per heat-map cell: class arg-max, sigmoid score, box from the regression heads, range and
//                        score mask (fastdeploy/runtime/backends/paddle/ops/centerpoint_postprocess_op.cu:43-91)
//   grid_sample_3d       tri-linear / nearest sampling of a 5-D tensor at normalised grid positions, zeros / border /
//                        reflection padding (fastdeploy/runtime/backends/paddle/ops/grid_sample_3d.cu:96-250)
#include "fdb_common.h"

#include <cub/cub.cuh>
#include <cuda_fp16.h>

namespace fdb {

struct Pt { float x, y; };

__device__ __forceinline__ float cross2(Pt a, Pt b, Pt c) { return (b.x - a.x) * (c.y - a.y) - (b.y - a.y) * (c.x - a.x); }

__device__ __forceinline__ float poly_area(const Pt* p, int n) {
  float s = 0.f;
  for (int i = 0; i < n; ++i) {
    const Pt a = p[i], b = p[(i + 1) % n];
    s += a.x * b.y - a.y * b.x;
  }
  return 0.5f * s;
}

// Area of the intersection of two convex quadrilaterals (Sutherland-Hodgman: clip a by every edge of b).
__device__ float quad_intersection(const float* qa, const float* qb) {
  Pt poly[16], tmp[16];
  int n = 4;
  for (int i = 0; i < 4; ++i) poly[i] = Pt{qa[2 * i], qa[2 * i + 1]};
  Pt clip[4];
  for (int i = 0; i < 4; ++i) clip[i] = Pt{qb[2 * i], qb[2 * i + 1]};
  const float orient = poly_area(clip, 4) >= 0.f ? 1.f : -1.f;      // the inside test follows the clip polygon's winding
  for (int e = 0; e < 4 && n > 0; ++e) {
    const Pt a = clip[e], b = clip[(e + 1) & 3];
    int m = 0;
    Pt s = poly[n - 1];
    float ds = orient * cross2(a, b, s);
    for (int i = 0; i < n; ++i) {
      const Pt p = poly[i];
      const float dp = orient * cross2(a, b, p);
      if (dp >= 0.f) {
        if (ds < 0.f) { const float t = ds / (ds - dp); tmp[m++] = Pt{s.x + t * (p.x - s.x), s.y + t * (p.y - s.y)}; }
        tmp[m++] = p;
      } else if (ds >= 0.f) {
        const float t = ds / (ds - dp);
        tmp[m++] = Pt{s.x + t * (p.x - s.x), s.y + t * (p.y - s.y)};
      }
      s = p;
      ds = dp;
    }
    n = m;
    for (int i = 0; i < n; ++i) poly[i] = tmp[i];
  }
  return n >= 3 ? fabsf(poly_area(poly, n)) : 0.f;
}

__device__ __forceinline__ float quad_area(const float* q) {
  Pt p[4];
  for (int i = 0; i < 4; ++i) p[i] = Pt{q[2 * i], q[2 * i + 1]};
  return fabsf(poly_area(p, 4));
}

__device__ __forceinline__ float quad_iou(const float* a, const float* b) {
  const float inter = quad_intersection(a, b);
  const float uni = quad_area(a) + quad_area(b) - inter;
  return uni > 1e-9f ? inter / uni : 0.f;
}

// ---- pairwise IoU (tests, evaluation) ---------------------------------------------------------------------
__global__ void quad_iou_kernel(const float* a, const float* b, int na, int nb, float* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= na * nb) return;
  out[i] = quad_iou(a + 8 * (i / nb), b + 8 * (i % nb));
}

// ---- suppression bit matrix: mask[i][w] bit j set when box (64 w + j) > i is suppressed by box i ------------
__global__ void __launch_bounds__(64) rotated_mask_kernel(const float* __restrict__ quads, const int* __restrict__ cls,
                                                          const unsigned char* __restrict__ valid, int K, float thresh,
                                                          unsigned long long* __restrict__ mask) {
  const int row_tile = blockIdx.y, col_tile = blockIdx.x;
  if (col_tile < row_tile) return;                         // only j > i matters
  const int words = (K + 63) / 64;
  __shared__ float cq[64 * 8];
  __shared__ int ccls[64];
  __shared__ unsigned char cval[64];
  const int cj = col_tile * 64 + threadIdx.x;
  if (cj < K) {
    for (int k = 0; k < 8; ++k) cq[threadIdx.x * 8 + k] = quads[cj * 8 + k];
    ccls[threadIdx.x] = cls != nullptr ? cls[cj] : 0;
    cval[threadIdx.x] = valid != nullptr ? valid[cj] : 1;
  } else {
    cval[threadIdx.x] = 0;
  }
  __syncthreads();
  const int i = row_tile * 64 + threadIdx.x;
  if (i >= K) return;
  unsigned long long bits = 0ull;
  if (valid == nullptr || valid[i]) {
    float q[8];
    for (int k = 0; k < 8; ++k) q[k] = quads[i * 8 + k];
    const int ci = cls != nullptr ? cls[i] : 0;
    const int start = row_tile == col_tile ? threadIdx.x + 1 : 0;
    for (int j = start; j < 64; ++j) {
      if (!cval[j] || ccls[j] != ci) continue;
      if (quad_iou(q, cq + 8 * j) > thresh) bits |= 1ull << j;
    }
  }
  mask[static_cast<size_t>(i) * words + col_tile] = bits;
}

// one block: walks the boxes in order; a box survives when no earlier survivor has suppressed it
__global__ void __launch_bounds__(256) rotated_scan_kernel(const unsigned long long* __restrict__ mask,
                                                           const unsigned char* __restrict__ valid, int K, int max_keep,
                                                           const int* __restrict__ n_used, unsigned char* __restrict__ keep,
                                                           int* __restrict__ n_keep) {
  extern __shared__ unsigned long long removed[];
  const int words = (K + 63) / 64;
  const int used = n_used != nullptr ? min(*n_used, K) : K;      // entries past this are padding
  for (int i = used + threadIdx.x; i < K; i += blockDim.x) keep[i] = 0;
  for (int w = threadIdx.x; w < words; w += blockDim.x) removed[w] = 0ull;
  __shared__ int kept, alive;
  if (threadIdx.x == 0) kept = 0;
  __syncthreads();
  for (int i = 0; i < used; ++i) {
    if (threadIdx.x == 0) {
      alive = (valid == nullptr || valid[i]) && !((removed[i >> 6] >> (i & 63)) & 1ull) && (max_keep <= 0 || kept < max_keep);
      keep[i] = static_cast<unsigned char>(alive);
      if (alive) ++kept;
    }
    __syncthreads();
    if (alive) {
      const unsigned long long* row = mask + static_cast<size_t>(i) * words;
      for (int w = (i >> 6) + threadIdx.x; w < words; w += blockDim.x) removed[w] |= row[w];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_keep = kept;
}

// ---- multiclass rotated NMS helpers ---------------------------------------------------------------------
// scores [C, M] (class-major) of one image; candidates above the threshold get key = class << 32 | ~score bits
__global__ void rot_candidates_kernel(const float* __restrict__ scores, int C, int M, float thresh, int background,
                                      unsigned long long* __restrict__ keys, int* __restrict__ vals, int cap,
                                      int* __restrict__ count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= C * M) return;
  const int c = i / M;
  const float s = scores[i];
  if (c == background || !(s > thresh)) return;
  const int slot = atomicAdd(count, 1);
  if (slot >= cap) return;
  keys[slot] = (static_cast<unsigned long long>(c) << 32) | (0xffffffffu - __float_as_uint(s));   // scores are positive
  vals[slot] = i;
}

__global__ void rot_fill_tail_kernel(unsigned long long* keys, int* vals, const int* count, int cap) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= cap) return;
  const int n = min(*count, cap);
  if (i >= n) { keys[i] = ~0ull; vals[i] = -1; }
}

// after the sort: class heads, rank within the class, gather of the quads
__global__ void rot_class_heads_kernel(const unsigned long long* keys, const int* count, int cap, int* class_start) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = min(*count, cap);
  if (p >= n) return;
  const int c = static_cast<int>(keys[p] >> 32);
  if (p == 0 || static_cast<int>(keys[p - 1] >> 32) != c) class_start[c] = p;
}

__global__ void rot_gather_kernel(const unsigned long long* keys, const int* vals, const int* count, int cap,
                                  const int* class_start, int top_k, const float* boxes, int M, float* quads, int* cls,
                                  float* score, unsigned char* valid) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= cap) return;
  const int n = min(*count, cap);
  if (p >= n) { valid[p] = 0; cls[p] = -1; score[p] = 0.f; return; }
  const int c = static_cast<int>(keys[p] >> 32);
  const int m = vals[p] % M;
  cls[p] = c;
  score[p] = __uint_as_float(0xffffffffu - static_cast<unsigned>(keys[p] & 0xffffffffu));
  valid[p] = (top_k <= 0 || p - class_start[c] < top_k) ? 1 : 0;
  for (int k = 0; k < 8; ++k) quads[p * 8 + k] = boxes[m * 8 + k];
}

// keep_top_k over all classes: a survivor stays when fewer than keep_top_k survivors have a better score (ties: the
// earlier position wins); rows come out in (class ascending, score descending) order = position order
__global__ void __launch_bounds__(256) rot_finalize_kernel(const unsigned char* keep, const float* score, const int* cls,
                                                           const float* quads, const int* vals, int M, int K, int keep_top_k,
                                                           float* out, int* out_index, int* out_count) {
  __shared__ int total;
  if (threadIdx.x == 0) total = 0;
  __syncthreads();
  // rank of every survivor
  extern __shared__ unsigned char final_keep[];
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    unsigned char f = 0;
    if (keep[i]) {
      int better = 0;
      if (keep_top_k > 0) {
        const float s = score[i];
        for (int j = 0; j < K; ++j) better += keep[j] && (score[j] > s || (score[j] == s && j < i));
      }
      f = (keep_top_k <= 0 || better < keep_top_k) ? 1 : 0;
    }
    final_keep[i] = f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {                      // compaction in position order (a few thousand entries at most)
    int n = 0;
    for (int i = 0; i < K; ++i) {
      if (!final_keep[i]) continue;
      float* row = out + n * 10;
      row[0] = static_cast<float>(cls[i]);
      row[1] = score[i];
      for (int k = 0; k < 8; ++k) row[2 + k] = quads[i * 8 + k];
      if (out_index != nullptr) out_index[n] = vals[i] % M;
      ++n;
    }
    *out_count = n;
  }
}

// ---- CenterPoint decode ---------------------------------------------------------------------------------
struct CenterPointParams {
  const float *hm, *reg, *height, *dim, *vel, *rot;
  int C, H, W, with_velocity;
  float voxel_x, voxel_y, range_x, range_y, down_ratio, score_thresh;
  float post_range[6];
  int use_post_range;
  float* boxes;       // [H*W, 9 or 7]
  float* scores;      // [H*W], -1 where masked out
  int* labels;        // [H*W]
  float* bev_quads;   // [H*W, 8] corners of (x, y, w, l, yaw) for the NMS
};

__global__ void centerpoint_decode_kernel(CenterPointParams p) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int hw = p.H * p.W;
  if (i >= hw) return;
  int label = 0;
  float best = -INFINITY;
  for (int c = 0; c < p.C; ++c) {
    const float v = p.hm[c * hw + i];
    if (v > best) { best = v; label = c; }
  }
  const float score = 1.f / (1.f + __expf(-best));
  const int ys = i / p.W, xs = i - ys * p.W;
  const float x = (xs + p.reg[i]) * p.down_ratio * p.voxel_x + p.range_x;
  const float y = (ys + p.reg[hw + i]) * p.down_ratio * p.voxel_y + p.range_y;
  const float z = p.height[i];
  const float w = __expf(p.dim[i]), l = __expf(p.dim[hw + i]), h = __expf(p.dim[2 * hw + i]);
  const float yaw = atan2f(p.rot[i], p.rot[hw + i]);
  const int nb = p.with_velocity ? 9 : 7;
  float* b = p.boxes + static_cast<size_t>(i) * nb;
  b[0] = x; b[1] = y; b[2] = z; b[3] = w; b[4] = l; b[5] = h;
  if (p.with_velocity) { b[6] = p.vel[i]; b[7] = p.vel[hw + i]; }
  b[nb - 1] = yaw;
  bool ok = score > p.score_thresh;
  if (p.use_post_range)
    ok = ok && x >= p.post_range[0] && y >= p.post_range[1] && z >= p.post_range[2] && x <= p.post_range[3] &&
         y <= p.post_range[4] && z <= p.post_range[5];
  p.scores[i] = ok ? score : -1.f;
  p.labels[i] = label;
  // corners of the bird's-eye-view rectangle, rotated by yaw about (x, y)
  const float c = cosf(yaw), s = sinf(yaw);
  const float dx[4] = {-w / 2, w / 2, w / 2, -w / 2}, dy[4] = {-l / 2, -l / 2, l / 2, l / 2};
  float* q = p.bev_quads + static_cast<size_t>(i) * 8;
  for (int k = 0; k < 4; ++k) {
    q[2 * k] = dx[k] * c - dy[k] * s + x;
    q[2 * k + 1] = dx[k] * s + dy[k] * c + y;
  }
}

// sort helper: keys = ~score bits (descending), vals = cell index; masked cells sort last
__global__ void score_keys_kernel(const float* scores, int n, unsigned* keys, int* vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float s = scores[i];
  keys[i] = s > 0.f ? 0xffffffffu - __float_as_uint(s) : 0xffffffffu;
  vals[i] = i;
}

__global__ void gather_sorted_quads_kernel(const unsigned* keys, const int* vals, int K, const float* quads_all,
                                           float* quads, unsigned char* valid) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= K) return;
  valid[p] = keys[p] != 0xffffffffu;
  const int src = vals[p];
  for (int k = 0; k < 8; ++k) quads[p * 8 + k] = quads_all[static_cast<size_t>(src) * 8 + k];
}

// ---- grid_sample_3d --------------------------------------------------------------------------------------
__device__ __forceinline__ float gs_unnormalize(float c, int size, bool align) {
  return align ? (c + 1.f) * 0.5f * (size - 1) : ((c + 1.f) * size - 1.f) * 0.5f;
}
__device__ __forceinline__ float gs_reflect(float x, float lo2, float hi2) {       // bounds in half-pixel units
  if (lo2 == hi2) return 0.f;
  const float mn = lo2 * 0.5f, span = (hi2 - lo2) * 0.5f;
  x = fabsf(x - mn);
  const float extra = fmodf(x, span);
  const int flips = static_cast<int>(floorf(x / span));
  return (flips & 1) ? span - extra + mn : extra + mn;
}
__device__ __forceinline__ float gs_coord(float c, int size, bool align, int padding) {
  float x = gs_unnormalize(c, size, align);
  if (padding == 1) x = fminf(fmaxf(x, 0.f), static_cast<float>(size - 1));
  else if (padding == 2) {
    x = align ? gs_reflect(x, 0.f, 2.f * (size - 1)) : gs_reflect(x, -1.f, 2.f * size - 1.f);
    x = fminf(fmaxf(x, 0.f), static_cast<float>(size - 1));
  }
  return x;
}

// x [N, C, D, H, W], grid [N, Do, Ho, Wo, 3] (x, y, z in [-1, 1]) -> out [N, C, Do, Ho, Wo]; mode 0 tri-linear, 1 nearest;
// padding 0 zeros, 1 border, 2 reflection
__global__ void grid_sample_3d_kernel(const float* __restrict__ x, const float* __restrict__ grid, float* __restrict__ out,
                                      int N, int C, int D, int H, int W, int Do, int Ho, int Wo, int mode, int padding,
                                      int align) {
  const long long total = static_cast<long long>(N) * Do * Ho * Wo;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const long long vol_o = static_cast<long long>(Do) * Ho * Wo, vol_i = static_cast<long long>(D) * H * W;
  const int n = static_cast<int>(idx / vol_o);
  const long long sp = idx - n * vol_o;
  const float gx = grid[idx * 3], gy = grid[idx * 3 + 1], gz = grid[idx * 3 + 2];
  const float fx = gs_coord(gx, W, align != 0, padding), fy = gs_coord(gy, H, align != 0, padding),
              fz = gs_coord(gz, D, align != 0, padding);
  const float* xin = x + static_cast<long long>(n) * C * vol_i;
  float* o = out + static_cast<long long>(n) * C * vol_o + sp;
  if (mode == 1) {
    const int ix = static_cast<int>(nearbyintf(fx)), iy = static_cast<int>(nearbyintf(fy)), iz = static_cast<int>(nearbyintf(fz));
    const bool in = ix >= 0 && ix < W && iy >= 0 && iy < H && iz >= 0 && iz < D;
    for (int c = 0; c < C; ++c) o[c * vol_o] = in ? xin[c * vol_i + (static_cast<long long>(iz) * H + iy) * W + ix] : 0.f;
    return;
  }
  const int x0 = static_cast<int>(floorf(fx)), y0 = static_cast<int>(floorf(fy)), z0 = static_cast<int>(floorf(fz));
  const float ax = fx - x0, ay = fy - y0, az = fz - z0;
  float wgt[8];
  long long off[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int dx = k & 1, dy = (k >> 1) & 1, dz = k >> 2;
    const int xi = x0 + dx, yi = y0 + dy, zi = z0 + dz;
    const bool in = xi >= 0 && xi < W && yi >= 0 && yi < H && zi >= 0 && zi < D;
    wgt[k] = in ? (dx ? ax : 1.f - ax) * (dy ? ay : 1.f - ay) * (dz ? az : 1.f - az) : 0.f;
    off[k] = in ? (static_cast<long long>(zi) * H + yi) * W + xi : 0;
  }
  for (int c = 0; c < C; ++c) {
    const float* xc = xin + c * vol_i;
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) v += wgt[k] * xc[off[k]];
    o[c * vol_o] = v;
  }
}

static int pc_check(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error(std::string(what) + ": " + cudaGetErrorString(e)); return -1; }
  return 0;
}

}  // namespace fdb

using namespace fdb;

FDB_API int fdb_quad_iou(const float* a, const float* b, int na, int nb, float* out, void* stream) {
  if (na <= 0 || nb <= 0) return 0;
  quad_iou_kernel<<<(na * nb + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(a, b, na, nb, out);
  return pc_check("quad_iou");
}

// Workspace of rotated_nms for K boxes: the K x ceil(K / 64) bit matrix.
FDB_API long long fdb_rotated_nms_workspace(int K) { return static_cast<long long>(K) * ((K + 63) / 64) * 8 + 256; }

// quads [K, 8] in decreasing score order; cls [K] or null (class-agnostic); valid [K] or null; n_used (device, or null)
// = how many leading entries are real. keep [K] gets 1 for survivors, n_keep their count (at most max_keep when positive).
FDB_API int fdb_rotated_nms(const float* quads, const int* cls, const unsigned char* valid, int K, float thresh, int max_keep,
                            const int* n_used, void* workspace, long long workspace_bytes, unsigned char* keep, int* n_keep,
                            void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (K <= 0) { cudaMemsetAsync(n_keep, 0, sizeof(int), st); return 0; }
  if (K > 32768) { set_error("rotated_nms: at most 32768 boxes"); return -1; }
  if (workspace_bytes < fdb_rotated_nms_workspace(K)) { set_error("rotated_nms: workspace too small"); return -1; }
  const int tiles = (K + 63) / 64;
  auto* mask = static_cast<unsigned long long*>(workspace);
  FDB_CUDA_OK(cudaMemsetAsync(mask, 0, static_cast<size_t>(K) * tiles * 8, st));
  rotated_mask_kernel<<<dim3(tiles, tiles), 64, 0, st>>>(quads, cls, valid, K, thresh, mask);
  rotated_scan_kernel<<<1, 256, tiles * 8, st>>>(mask, valid, K, max_keep, n_used, keep, n_keep);
  return pc_check("rotated_nms");
}

// Bytes of scratch for multiclass_rotated with `cap` candidates.
FDB_API long long fdb_multiclass_rotated_workspace(int cap, int C) {
  size_t sort_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, static_cast<unsigned long long*>(nullptr),
                                  static_cast<unsigned long long*>(nullptr), static_cast<int*>(nullptr),
                                  static_cast<int*>(nullptr), cap);
  long long b = 0;
  b += 2LL * cap * 8 + 2LL * cap * 4;                  // keys in / out, vals in / out
  b += static_cast<long long>(cap) * (8 * 4 + 4 + 4 + 1 + 1) + 64;     // quads, cls, score, valid, keep
  b += (C + 2) * 4LL + 16;                             // class_start, count, n_keep
  b += fdb_rotated_nms_workspace(cap) + static_cast<long long>(sort_bytes) + 16 * 256 + 1024;   // every piece is 256-byte aligned
  return b;
}

// One image: boxes [M, 8] quadrilaterals, scores [C, M]. out [keep cap, 10] = label, score, x1 y1 .. x4 y4 in
// (class ascending, score descending) order, out_index [keep cap] box ids, out_count [1]; overflow [1] is set to the
// number of candidates when it exceeded `cap` (the result is then incomplete and the caller falls back).
FDB_API int fdb_multiclass_nms_rotated(const float* boxes, const float* scores, int C, int M, float score_thresh,
                                       float nms_thresh, int nms_top_k, int keep_top_k, int background, int cap,
                                       void* workspace, long long workspace_bytes, float* out, int* out_index,
                                       int* out_count, int* overflow, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (C < 1 || M < 1 || cap < 64 || cap > 32768) { set_error("multiclass_nms_rotated: bad sizes"); return -1; }
  if (workspace_bytes < fdb_multiclass_rotated_workspace(cap, C)) { set_error("multiclass_nms_rotated: workspace too small"); return -1; }
  char* w = static_cast<char*>(workspace);
  auto take = [&](size_t bytes) { char* p = w; w += (bytes + 255) / 256 * 256; return p; };
  auto* keys_in = reinterpret_cast<unsigned long long*>(take(cap * 8ull));
  auto* keys = reinterpret_cast<unsigned long long*>(take(cap * 8ull));
  auto* vals_in = reinterpret_cast<int*>(take(cap * 4ull));
  auto* vals = reinterpret_cast<int*>(take(cap * 4ull));
  auto* quads = reinterpret_cast<float*>(take(cap * 32ull));
  auto* cls = reinterpret_cast<int*>(take(cap * 4ull));
  auto* score = reinterpret_cast<float*>(take(cap * 4ull));
  auto* valid = reinterpret_cast<unsigned char*>(take(cap));
  auto* keep = reinterpret_cast<unsigned char*>(take(cap));
  auto* class_start = reinterpret_cast<int*>(take((C + 1) * 4ull));
  auto* count = reinterpret_cast<int*>(take(8));
  auto* n_keep = count + 1;
  size_t sort_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, keys_in, keys, vals_in, vals, cap);
  void* sort_ws = take(sort_bytes);
  void* nms_ws = take(static_cast<size_t>(fdb_rotated_nms_workspace(cap)));
  if (w - static_cast<char*>(workspace) > workspace_bytes) { set_error("multiclass_nms_rotated: workspace too small"); return -1; }
  FDB_CUDA_OK(cudaMemsetAsync(count, 0, 8, st));
  FDB_CUDA_OK(cudaMemsetAsync(class_start, 0, (C + 1) * 4ull, st));
  rot_candidates_kernel<<<(C * M + 255) / 256, 256, 0, st>>>(scores, C, M, score_thresh, background, keys_in, vals_in, cap, count);
  rot_fill_tail_kernel<<<(cap + 255) / 256, 256, 0, st>>>(keys_in, vals_in, count, cap);
  FDB_CUDA_OK(cub::DeviceRadixSort::SortPairs(sort_ws, sort_bytes, keys_in, keys, vals_in, vals, cap, 0, 64, st));
  rot_class_heads_kernel<<<(cap + 255) / 256, 256, 0, st>>>(keys, count, cap, class_start);
  rot_gather_kernel<<<(cap + 255) / 256, 256, 0, st>>>(keys, vals, count, cap, class_start, nms_top_k, boxes, M, quads, cls,
                                                       score, valid);
  if (fdb_rotated_nms(quads, cls, valid, cap, nms_thresh, 0, count, nms_ws, fdb_rotated_nms_workspace(cap), keep, n_keep, stream) != 0)
    return -1;
  rot_finalize_kernel<<<1, 256, cap, st>>>(keep, score, cls, quads, vals, M, cap, keep_top_k, out, out_index, out_count);
  FDB_CUDA_OK(cudaMemcpyAsync(overflow, count, sizeof(int), cudaMemcpyDeviceToDevice, st));
  return pc_check("multiclass_nms_rotated");
}

struct CenterPointDesc {
  const float *hm, *reg, *height, *dim, *vel, *rot;
  int C, H, W, with_velocity;
  float voxel_x, voxel_y, range_x, range_y, down_ratio, score_thresh, nms_thresh;
  float post_range[6];
  int use_post_range, pre_max, post_max;
};

FDB_API long long fdb_centerpoint_workspace(int H, int W, int pre_max) {
  const long long hw = static_cast<long long>(H) * W;
  size_t sort_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, static_cast<unsigned*>(nullptr), static_cast<unsigned*>(nullptr),
                                  static_cast<int*>(nullptr), static_cast<int*>(nullptr), static_cast<int>(hw));
  return hw * (8 * 4 + 4 * 4) + pre_max * (8 * 4 + 2LL) + fdb_rotated_nms_workspace(pre_max) +
         static_cast<long long>(sort_bytes) + 16 * 256 + 4096;     // every piece is 256-byte aligned
}

// One CenterPoint task head. boxes [H*W, 9|7], scores [H*W], labels [H*W] receive the per-cell decode; order [pre_max]
// the cell index of the i-th best candidate, keep [pre_max] whether it survived the bird's-eye-view NMS, n_keep their
// count (at most post_max).
FDB_API int fdb_centerpoint_decode(const CenterPointDesc* d, void* workspace, long long workspace_bytes, float* boxes,
                                   float* scores, int* labels, int* order, unsigned char* keep, int* n_keep, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  const int hw = d->H * d->W;
  const int K = d->pre_max < hw ? d->pre_max : hw;
  if (hw < 1 || d->C < 1 || K < 1 || K > 32768) { set_error("centerpoint_decode: bad sizes"); return -1; }
  if (workspace_bytes < fdb_centerpoint_workspace(d->H, d->W, d->pre_max)) { set_error("centerpoint_decode: workspace too small"); return -1; }
  char* w = static_cast<char*>(workspace);
  auto take = [&](size_t bytes) { char* p = w; w += (bytes + 255) / 256 * 256; return p; };
  auto* quads_all = reinterpret_cast<float*>(take(hw * 32ull));
  auto* keys_in = reinterpret_cast<unsigned*>(take(hw * 4ull));
  auto* keys = reinterpret_cast<unsigned*>(take(hw * 4ull));
  auto* vals_in = reinterpret_cast<int*>(take(hw * 4ull));
  auto* vals = reinterpret_cast<int*>(take(hw * 4ull));
  auto* quads = reinterpret_cast<float*>(take(K * 32ull));
  auto* valid = reinterpret_cast<unsigned char*>(take(K));
  size_t sort_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, keys_in, keys, vals_in, vals, hw);
  void* sort_ws = take(sort_bytes);
  void* nms_ws = take(static_cast<size_t>(fdb_rotated_nms_workspace(K)));
  CenterPointParams p{};
  p.hm = d->hm; p.reg = d->reg; p.height = d->height; p.dim = d->dim; p.vel = d->vel; p.rot = d->rot;
  p.C = d->C; p.H = d->H; p.W = d->W; p.with_velocity = d->with_velocity;
  p.voxel_x = d->voxel_x; p.voxel_y = d->voxel_y; p.range_x = d->range_x; p.range_y = d->range_y;
  p.down_ratio = d->down_ratio; p.score_thresh = d->score_thresh;
  for (int k = 0; k < 6; ++k) p.post_range[k] = d->post_range[k];
  p.use_post_range = d->use_post_range;
  p.boxes = boxes; p.scores = scores; p.labels = labels; p.bev_quads = quads_all;
  centerpoint_decode_kernel<<<(hw + 255) / 256, 256, 0, st>>>(p);
  score_keys_kernel<<<(hw + 255) / 256, 256, 0, st>>>(scores, hw, keys_in, vals_in);
  FDB_CUDA_OK(cub::DeviceRadixSort::SortPairs(sort_ws, sort_bytes, keys_in, keys, vals_in, vals, hw, 0, 32, st));
  gather_sorted_quads_kernel<<<(K + 255) / 256, 256, 0, st>>>(keys, vals, K, quads_all, quads, valid);
  FDB_CUDA_OK(cudaMemcpyAsync(order, vals, K * sizeof(int), cudaMemcpyDeviceToDevice, st));
  return fdb_rotated_nms(quads, nullptr, valid, K, d->nms_thresh, d->post_max, nullptr, nms_ws, fdb_rotated_nms_workspace(K),
                         keep, n_keep, stream);
}

FDB_API int fdb_grid_sample_3d(const float* x, const float* grid, float* out, int N, int C, int D, int H, int W, int Do, int Ho,
                               int Wo, int mode, int padding, int align_corners, void* stream) {
  const long long total = static_cast<long long>(N) * Do * Ho * Wo;
  if (total <= 0) return 0;
  if (C < 1 || D < 1 || H < 1 || W < 1 || mode < 0 || mode > 1 || padding < 0 || padding > 2) {
    set_error("grid_sample_3d: bad arguments");
    return -1;
  }
  grid_sample_3d_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, grid, out, N, C, D, H, W, Do, Ho, Wo, mode, padding, align_corners);
  return pc_check("grid_sample_3d");
}
