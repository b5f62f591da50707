// Multiclass NMS on the GPU with the reference's CPU semantics
// (fastdeploy/vision/detection/ppdet/multiclass_nms.cc:29-171): per class keep
// scores > score_threshold, stable sort descending, truncate to nms_top_k, greedy
// suppression with Jaccard overlap > nms_threshold, then a global stable sort by
// score and truncation to keep_top_k, output grouped by class ascending.
//
// Kernel 1 (grid = classes x images): radix-select the top nms_top_k keys in
// shared memory, bitonic-sort them on (score desc, index asc), then one warp
// sweeps the sorted candidates 32 at a time against the boxes kept so far. A
// class can contribute at most keep_top_k boxes to the final result, so the
// sweep stops there - exact, and it bounds the work for dense score maps.
// Kernel 2 (grid = images): merges the per-class lists, selects keep_top_k by
// (score desc, class asc, rank asc) and writes rows [label, score, x1, y1, x2, y2].
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fdb_common.h"

namespace fdb {

constexpr int kNmsMaxTopK = 1024;
constexpr int kNmsThreads = 256;
constexpr int kMergeMax = 8192;

struct NmsDesc {
  const float* boxes;   // [N][M][4]
  const void* scores;   // element (n, c, m) at n*s_n + c*s_c + m*s_m
  int score_dtype;      // kF32 | kF16 | kBF16
  long long s_n, s_c, s_m;
  int N, M, C;
  float score_threshold, nms_threshold;
  int nms_top_k, keep_top_k, normalized, background_label;
  // scratch (device): per (n, c) kept lists
  int* cls_count;       // [N][C]
  float* cls_score;     // [N][C][max_keep]
  int* cls_index;       // [N][C][max_keep]
  int max_keep;
  // outputs
  float* out;           // [N][out_cap][6]
  int* out_index;       // [N][out_cap]   (anchor index within the image)
  int* out_num;         // [N]
  int out_cap;
};

__device__ __forceinline__ float load_score(const void* base, int dt, long long off) {
  if (dt == kF32) return reinterpret_cast<const float*>(base)[off];
  if (dt == kBF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
  return __half2float(reinterpret_cast<const __half*>(base)[off]);
}

__device__ __forceinline__ float box_area(const float4& b, bool normalized) {
  if (b.z < b.x || b.w < b.y) return 0.f;
  const float w = __fsub_rn(b.z, b.x), h = __fsub_rn(b.w, b.y);
  return normalized ? __fmul_rn(w, h) : __fmul_rn(__fadd_rn(w, 1.f), __fadd_rn(h, 1.f));
}

__device__ __forceinline__ float jaccard(const float4& a, const float4& b, bool normalized) {
  if (b.x > a.z || b.z < a.x || b.y > a.w || b.w < a.y) return 0.f;
  const float ix0 = fmaxf(a.x, b.x), iy0 = fmaxf(a.y, b.y), ix1 = fminf(a.z, b.z), iy1 = fminf(a.w, b.w);
  const float norm = normalized ? 0.f : 1.f;
  const float iw = __fadd_rn(__fsub_rn(ix1, ix0), norm), ih = __fadd_rn(__fsub_rn(iy1, iy0), norm);
  const float inter = __fmul_rn(iw, ih);
  return __fdiv_rn(inter, __fsub_rn(__fadd_rn(box_area(a, normalized), box_area(b, normalized)), inter));
}

// Block-wide exclusive scan of one int per thread (kNmsThreads threads).
__device__ __forceinline__ int block_excl_scan(int v, int* smem_warp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) smem_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (kNmsThreads / 32) ? smem_warp[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    if (lane < kNmsThreads / 32) smem_warp[lane] = wi - w;
    if (lane == kNmsThreads / 32 - 1) smem_warp[kNmsThreads / 32] = wi;
  }
  __syncthreads();
  const int res = smem_warp[warp] + incl - v;
  *total = smem_warp[kNmsThreads / 32];
  __syncthreads();
  return res;
}

__global__ void __launch_bounds__(kNmsThreads) nms_class_kernel(const NmsDesc d) {
  const int c = blockIdx.x, n = blockIdx.y;
  int* count_out = d.cls_count + n * d.C + c;
  if (c == d.background_label) {
    if (threadIdx.x == 0) *count_out = 0;
    return;
  }
  extern __shared__ __align__(16) uint8_t nms_smem[];
  uint32_t* keys = reinterpret_cast<uint32_t*>(nms_smem);                       // [M]
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(keys + ((d.M + 3) & ~3));  // [1024]
  float4* cbox = reinterpret_cast<float4*>(cand + kNmsMaxTopK);                 // [1024]
  float4* kbox = cbox + kNmsMaxTopK;                                            // [max_keep<=1024]
  __shared__ int hist[256];
  __shared__ int warp_tmp[kNmsThreads / 32 + 1];
  __shared__ uint32_t sel_prefix;
  __shared__ int sel_remaining;
  __shared__ int s_nkept;

  const int tid = threadIdx.x;
  const int K = min(d.nms_top_k < 0 ? kNmsMaxTopK : d.nms_top_k, kNmsMaxTopK);
  const long long base = static_cast<long long>(n) * d.s_n + static_cast<long long>(c) * d.s_c;

  // 1. keys: positive scores compare like their bit patterns
  int local = 0;
  for (int m = tid; m < d.M; m += kNmsThreads) {
    const float s = load_score(d.scores, d.score_dtype, base + m * d.s_m);
    const uint32_t k = (s > d.score_threshold && s > 0.f) ? __float_as_uint(s) : 0u;
    keys[m] = k;
    local += k != 0u;
  }
  int total_pos;
  block_excl_scan(local, warp_tmp, &total_pos);

  // 2. radix select of the K-th largest key when there are more than K candidates
  uint32_t thr_key = 1u;   // admit keys >= thr_key ...
  int eq_budget = 1 << 30; // ... but only this many equal to thr_key (lowest indices first)
  if (total_pos > K) {
    if (tid == 0) { sel_prefix = 0u; sel_remaining = K; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      hist[tid] = 0;  // kNmsThreads == 256 bins
      __syncthreads();
      const uint32_t prefix = sel_prefix;
      const uint32_t mask_hi = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      // Score maps of a freshly initialised or confident head put most keys into one bin, so the
      // histogram is warp-aggregated: lanes with equal bins elect one lane that adds their count.
      for (int base_m = 0; base_m < d.M; base_m += kNmsThreads) {
        const int m = base_m + tid;
        int bin = -1;
        if (m < d.M) {
          const uint32_t k = keys[m];
          if (k != 0u && (k & mask_hi) == (prefix & mask_hi)) bin = static_cast<int>((k >> shift) & 0xFF);
        }
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        if (bin >= 0 && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
      }
      __syncthreads();
      if (tid == 0) {
        int rem = sel_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if (hist[b] >= rem) break;
          rem -= hist[b];
        }
        sel_prefix = prefix | (static_cast<uint32_t>(b) << shift);
        sel_remaining = rem;
      }
      __syncthreads();
    }
    thr_key = sel_prefix;
    eq_budget = sel_remaining;
    __syncthreads();
  }

  // 3. ordered compaction (index order decides between equal keys)
  const int per = (d.M + kNmsThreads - 1) / kNmsThreads;
  const int m_begin = min(tid * per, d.M), m_end = min(m_begin + per, d.M);
  int n_gt = 0, n_eq = 0;
  for (int m = m_begin; m < m_end; ++m) {
    const uint32_t k = keys[m];
    n_gt += (k != 0u && k > thr_key);
    n_eq += (k != 0u && k == thr_key);
  }
  int tot_gt, tot_eq;
  const int off_gt = block_excl_scan(n_gt, warp_tmp, &tot_gt);
  int off_eq = block_excl_scan(n_eq, warp_tmp, &tot_eq);
  const int eq_taken = min(tot_eq, eq_budget);
  const int ncand = min(tot_gt + eq_taken, kNmsMaxTopK);
  for (int i = tid; i < kNmsMaxTopK; i += kNmsThreads) cand[i] = 0ull;
  __syncthreads();
  {
    int pg = off_gt, pe = off_eq;
    for (int m = m_begin; m < m_end; ++m) {
      const uint32_t k = keys[m];
      if (k == 0u) continue;
      const unsigned long long v = (static_cast<unsigned long long>(k) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(m));
      if (k > thr_key) {
        if (pg < kNmsMaxTopK) cand[pg] = v;
        ++pg;
      } else if (k == thr_key) {
        if (pe < eq_taken && tot_gt + pe < kNmsMaxTopK) cand[tot_gt + pe] = v;
        ++pe;
      }
    }
  }
  __syncthreads();

  // 4. bitonic sort, descending, over the smallest power of two >= ncand
  int sort_n = 32;
  while (sort_n < ncand) sort_n <<= 1;
  for (int k = 2; k <= sort_n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < sort_n; i += kNmsThreads) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned long long a = cand[i], b = cand[ixj];
          const bool desc = (i & k) == 0;
          if (desc ? (a < b) : (a > b)) { cand[i] = b; cand[ixj] = a; }
        }
      }
      __syncthreads();
    }
  }

  // 5. boxes of the sorted candidates
  const float4* boxes = reinterpret_cast<const float4*>(d.boxes) + static_cast<size_t>(n) * d.M;
  for (int i = tid; i < ncand; i += kNmsThreads) {
    const uint32_t m = 0xFFFFFFFFu - static_cast<uint32_t>(cand[i] & 0xFFFFFFFFull);
    cbox[i] = boxes[m];
  }
  if (tid == 0) s_nkept = 0;
  __syncthreads();

  // 6. greedy sweep by one warp, 32 candidates per step
  const bool normalized = d.normalized != 0;
  const int max_keep = d.max_keep;
  if (tid < 32) {
    const int lane = tid;
    int nkept = 0;
    float* o_score = d.cls_score + (static_cast<size_t>(n) * d.C + c) * max_keep;
    int* o_index = d.cls_index + (static_cast<size_t>(n) * d.C + c) * max_keep;
    for (int b0 = 0; b0 < ncand && nkept < max_keep; b0 += 32) {
      const int j = b0 + lane;
      bool alive = j < ncand;
      float4 mine = alive ? cbox[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < nkept && alive; ++k) {
        if (jaccard(mine, kbox[k], normalized) > d.nms_threshold) alive = false;
      }
      // overlaps with earlier candidates of the same step
      uint32_t mask = 0u;
      for (int l = 0; l < 31; ++l) {
        float4 o;
        o.x = __shfl_sync(0xffffffffu, mine.x, l);
        o.y = __shfl_sync(0xffffffffu, mine.y, l);
        o.z = __shfl_sync(0xffffffffu, mine.z, l);
        o.w = __shfl_sync(0xffffffffu, mine.w, l);
        if (l < lane && alive && jaccard(mine, o, normalized) > d.nms_threshold) mask |= 1u << l;
      }
      uint32_t keptmask = 0u;
      for (int l = 0; l < 32; ++l) {
        const int a = __shfl_sync(0xffffffffu, alive ? 1 : 0, l);
        const uint32_t mk = __shfl_sync(0xffffffffu, mask, l);
        if (a && (mk & keptmask) == 0u) keptmask |= 1u << l;
      }
      const bool kept = (keptmask >> lane) & 1u;
      const int pos = nkept + __popc(keptmask & ((1u << lane) - 1u));
      if (kept && pos < max_keep) {
        kbox[pos] = mine;
        o_score[pos] = __uint_as_float(static_cast<uint32_t>(cand[j] >> 32));
        o_index[pos] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(cand[j] & 0xFFFFFFFFull));
      }
      nkept = min(nkept + __popc(keptmask), max_keep);
      __syncwarp();
    }
    if (lane == 0) *count_out = nkept;
  }
}

// One block per image. Selects keep_top_k of the per-class survivors.
__global__ void __launch_bounds__(1024) nms_merge_kernel(const NmsDesc d) {
  const int n = blockIdx.x;
  const int tid = threadIdx.x;
  extern __shared__ __align__(16) uint8_t merge_smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(merge_smem);  // [sort_n]
  __shared__ int s_total;
  __shared__ int cls_off[1025];
  const int C = d.C, mk = d.max_keep;
  const int* counts = d.cls_count + n * C;
  // exclusive offsets of the class lists (C <= 1024)
  if (tid == 0) {
    int acc = 0;
    for (int c = 0; c < C; ++c) { cls_off[c] = acc; acc += counts[c]; }
    cls_off[C] = acc;
    s_total = acc;
  }
  __syncthreads();
  const int total = s_total;
  float* out = d.out + static_cast<size_t>(n) * d.out_cap * 6;
  int* out_idx = d.out_index + static_cast<size_t>(n) * d.out_cap;
  const float4* boxes = reinterpret_cast<const float4*>(d.boxes) + static_cast<size_t>(n) * d.M;
  const bool select = d.keep_top_k > -1 && total > d.keep_top_k;
  const int n_out = min(select ? d.keep_top_k : total, d.out_cap);

  unsigned long long cut = 0ull;  // entries with key >= cut are selected
  if (select) {
    int sort_n = 32;
    while (sort_n < total) sort_n <<= 1;
    for (int i = tid; i < sort_n; i += blockDim.x) keys[i] = 0ull;
    __syncthreads();
    for (int e = tid; e < C * mk; e += blockDim.x) {
      const int c = e / mk, r = e - c * mk;
      if (r < counts[c]) {
        const uint32_t sb = __float_as_uint(d.cls_score[(static_cast<size_t>(n) * C + c) * mk + r]);
        keys[cls_off[c] + r] = (static_cast<unsigned long long>(sb) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(e));
      }
    }
    __syncthreads();
    for (int k = 2; k <= sort_n; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < sort_n; i += blockDim.x) {
          const int ixj = i ^ j;
          if (ixj > i) {
            const unsigned long long a = keys[i], b = keys[ixj];
            const bool desc = (i & k) == 0;
            if (desc ? (a < b) : (a > b)) { keys[i] = b; keys[ixj] = a; }
          }
        }
        __syncthreads();
      }
    }
    cut = keys[d.keep_top_k - 1];
    __syncthreads();
  }

  // Ordered output: class ascending, rank ascending. Each thread owns whole classes
  // in turn; positions come from a serial prefix over per-class selected counts.
  __shared__ int sel_off[1025];
  for (int c = tid; c < C; c += blockDim.x) {
    int cnt = 0;
    for (int r = 0; r < counts[c]; ++r) {
      const uint32_t sb = __float_as_uint(d.cls_score[(static_cast<size_t>(n) * C + c) * mk + r]);
      const unsigned long long key = (static_cast<unsigned long long>(sb) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(c * mk + r));
      cnt += (!select || key >= cut);
    }
    sel_off[c + 1] = cnt;
  }
  __syncthreads();
  if (tid == 0) {
    sel_off[0] = 0;
    for (int c = 0; c < C; ++c) sel_off[c + 1] += sel_off[c];
  }
  __syncthreads();
  for (int c = tid; c < C; c += blockDim.x) {
    int pos = sel_off[c];
    for (int r = 0; r < counts[c]; ++r) {
      const float sc = d.cls_score[(static_cast<size_t>(n) * C + c) * mk + r];
      const unsigned long long key = (static_cast<unsigned long long>(__float_as_uint(sc)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(c * mk + r));
      if (select && key < cut) continue;
      if (pos < n_out) {
        const int m = d.cls_index[(static_cast<size_t>(n) * C + c) * mk + r];
        const float4 b = boxes[m];
        float* o = out + static_cast<size_t>(pos) * 6;
        o[0] = static_cast<float>(c); o[1] = sc; o[2] = b.x; o[3] = b.y; o[4] = b.z; o[5] = b.w;
        out_idx[pos] = m;
      }
      ++pos;
    }
  }
  if (tid == 0) d.out_num[n] = n_out;
}

struct NmsOp : Op {
  NmsDesc d;
  size_t smem1 = 0, smem2 = 0;
  int launch(cudaStream_t s) override {
    dim3 grid(d.C, d.N);
    nms_class_kernel<<<grid, kNmsThreads, smem1, s>>>(d);
    nms_merge_kernel<<<d.N, 1024, smem2, s>>>(d);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

}  // namespace fdb

using namespace fdb;

// Scratch requirement in bytes for the per-class lists: counts, scores, indices.
FDB_API long long fdb_nms_scratch_bytes(int N, int C, int max_keep) {
  return static_cast<long long>(N) * C * (4 + 8ll * max_keep);
}

FDB_API void* fdb_nms_create(const NmsDesc* dp) {
  NmsDesc d = *dp;
  if (d.C > 1024) { set_error("nms: at most 1024 classes"); return nullptr; }
  if (d.nms_top_k > kNmsMaxTopK || d.nms_top_k < 0) {
    set_error("nms: nms_top_k must be in [0, 1024] for the device path"); return nullptr;
  }
  if (d.keep_top_k == 0) { set_error("nms: keep_top_k must be -1 or positive"); return nullptr; }
  if (d.max_keep < 1 || d.max_keep > kNmsMaxTopK) { set_error("nms: max_keep must be in [1, 1024]"); return nullptr; }
  if (d.keep_top_k > -1 && static_cast<long long>(d.C) * d.max_keep > kMergeMax && d.keep_top_k < d.C * d.max_keep) {
    set_error("nms: classes * max_keep exceeds the merge capacity (8192)"); return nullptr;
  }
  auto* op = new NmsOp();
  op->d = d;
  op->smem1 = static_cast<size_t>((d.M + 3) & ~3) * 4 + kNmsMaxTopK * 8 + 2 * kNmsMaxTopK * 16;
  int sort_n = 32;
  while (sort_n < d.C * d.max_keep && sort_n < kMergeMax) sort_n <<= 1;
  op->smem2 = d.keep_top_k > -1 ? static_cast<size_t>(sort_n) * 8 : 16;
  if (op->smem1 > 200 * 1024) { set_error("nms: too many boxes per image for shared memory"); delete op; return nullptr; }
  // The opt-in limit is per function: only ever raise it, other ops may need more.
  static size_t max1 = 0, max2 = 0;
  cudaError_t e = cudaSuccess;
  if (op->smem1 > max1) {
    e = cudaFuncSetAttribute(nms_class_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)op->smem1);
    if (e == cudaSuccess) max1 = op->smem1;
  }
  if (e == cudaSuccess && op->smem2 > max2) {
    e = cudaFuncSetAttribute(nms_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)op->smem2);
    if (e == cudaSuccess) max2 = op->smem2;
  }
  if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); delete op; return nullptr; }
  return op;
}
