// Multiclass NMS on the GPU with the reference's CPU semantics
// (fastdeploy/vision/detection/ppdet/multiclass_nms.cc:29-171): per class keep
// scores > score_threshold, stable sort descending, truncate to nms_top_k, greedy
// suppression with Jaccard overlap > nms_threshold, then a global stable sort by
// score and truncation to keep_top_k, output grouped by class ascending.
//
// Kernel 1 (grid = classes x images): radix-select the top nms_top_k keys in
// shared memory, bitonic-sort them on (score desc, index asc), then the block
// sweeps the sorted candidates 256 at a time against the boxes kept so far
// (the warps resolve their 32 candidates in turn). A
// class can contribute at most keep_top_k boxes to the final result, so the
// sweep stops there - exact, and it bounds the work for dense score maps.
// Kernel 2 (grid = images): merges the per-class lists, selects keep_top_k by
// (score desc, class asc, rank asc) and writes rows [label, score, x1, y1, x2, y2].
#include <algorithm>

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
  // optional scratch [N][C][M] in the score dtype: anchor-major scores are transposed into it
  // first so that every class reads its M scores contiguously
  void* scores_t;
  // optional pre-pass scratch: lead[N][C][kLead] scores of each class's leading kept boxes and tau[N], the
  // per-image score below which no box can reach the final keep_top_k rows (null = no pre-pass)
  float* lead;
  float* tau;
};

// Optional phase timing of the class kernel (compile with -DFDB_NMS_PROFILE): thread 0 of every
// block adds the cycles it spent in each phase.
#ifdef FDB_NMS_PROFILE
__device__ unsigned long long g_nms_phase[8];
#define NMS_PHASE(i) do { if (threadIdx.x == 0) { const long long t_ = clock64(); atomicAdd(&g_nms_phase[i], (unsigned long long)(t_ - t_phase)); t_phase = t_; } } while (0)
#define NMS_PHASE_BEGIN long long t_phase = clock64()
#else
#define NMS_PHASE(i) do { } while (0)
#define NMS_PHASE_BEGIN do { } while (0)
#endif

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

__device__ __forceinline__ float score_to_float(float v) { return v; }
__device__ __forceinline__ float score_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float score_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

// Fills keys[m] with the bit pattern of score m when it passes the threshold, else 0. Eight loads
// are in flight per thread before any is consumed. Returns this thread's count of passing scores.
template <typename T>
__device__ __forceinline__ int load_keys(const NmsDesc& d, uint32_t* keys, long long base, float floor_score) {
  const T* src = reinterpret_cast<const T*>(d.scores) + base;
  int local = 0;
  for (int m0 = threadIdx.x; m0 < d.M; m0 += 8 * kNmsThreads) {
    T v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int m = m0 + u * kNmsThreads;
      v[u] = src[static_cast<long long>(min(m, d.M - 1)) * d.s_m];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int m = m0 + u * kNmsThreads;
      if (m < d.M) {
        const float s = score_to_float(v[u]);
        const uint32_t k = (s > d.score_threshold && s > 0.f && s >= floor_score) ? __float_as_uint(s) : 0u;
        keys[m] = k;
        local += k != 0u;
      }
    }
  }
  return local;
}

// jaccard(a, b) > thr with the areas given. The quotient is only formed when the comparison is
// within rounding distance of the threshold, so the verdict equals the divided form exactly.
__device__ __forceinline__ bool overlaps(const float4& a, float area_a, const float4& b, float area_b, bool normalized,
                                         float thr) {
  const bool disjoint = b.x > a.z || b.z < a.x || b.y > a.w || b.w < a.y;
  const float ix0 = fmaxf(a.x, b.x), iy0 = fmaxf(a.y, b.y), ix1 = fminf(a.z, b.z), iy1 = fminf(a.w, b.w);
  const float norm = normalized ? 0.f : 1.f;
  const float iw = __fadd_rn(__fsub_rn(ix1, ix0), norm), ih = __fadd_rn(__fsub_rn(iy1, iy0), norm);
  const float inter = __fmul_rn(iw, ih);
  const float uni = __fsub_rn(__fadd_rn(area_a, area_b), inter);
  const float t = __fmul_rn(thr, uni);
  bool res = inter > __fmul_rn(t, 1.000002f);
  const bool sure = (res || inter < __fmul_rn(t, 0.999998f)) && uni > 0.f && thr > 0.f;
  if (!sure && !disjoint) res = __fdiv_rn(inter, uni) > thr;   // rare: within rounding distance of the threshold
  return disjoint ? (0.f > thr) : res;
}

// Does box a overlap any of the kept boxes [k0, k1)? Four independent tests per step hide the
// shared-memory latency; the arrays are padded so that reading up to three entries past k1 is safe.
__device__ __forceinline__ bool hits_kept(const float4& a, float area_a, const float4* kbox, const float* karea, int k0,
                                          int k1, bool normalized, float thr) {
  for (int k = k0; k < k1; k += 4) {
    bool hit = false;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      hit |= (k + u < k1) && overlaps(a, area_a, kbox[k + u], karea[k + u], normalized, thr);
    }
    if (hit) return true;
  }
  return false;
}

// Block-wide exclusive scan of one int per thread (NT threads; smem_warp holds NT/32 + 1 ints).
template <int NT = kNmsThreads>
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
    int w = lane < (NT / 32) ? smem_warp[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    if (lane < NT / 32) smem_warp[lane] = wi - w;
    if (lane == NT / 32 - 1) smem_warp[NT / 32] = wi;
  }
  __syncthreads();
  const int res = smem_warp[warp] + incl - v;
  *total = smem_warp[NT / 32];
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
  const int key_words = max((d.M + 3) & ~3, kNmsThreads * (kNmsThreads / 32));
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(keys + key_words);          // [1024]
  float4* cbox = reinterpret_cast<float4*>(cand + kNmsMaxTopK);                 // [1024]
  float4* kbox = cbox + kNmsMaxTopK;                                            // [max_keep + 4]
  float* carea = reinterpret_cast<float*>(kbox + d.max_keep + 4);               // [1024]
  float* karea = carea + kNmsMaxTopK;                                           // [max_keep + 4]
  __shared__ int hist[256];
  __shared__ int warp_tmp[kNmsThreads / 32 + 1];
  __shared__ uint32_t sel_prefix;
  __shared__ int sel_remaining;

  const int tid = threadIdx.x;
  // Candidates are taken in passes of at most 1024 (what the shared-memory arrays hold), best first: a pass selects
  // the best remaining keys, sweeps them against everything kept so far and among themselves, and removes them from
  // the key array. The passes stop when the class has produced max_keep boxes, when nms_top_k candidates have been
  // considered, or when no candidate is left - so any nms_top_k is exact, and the common case is one pass.
  int budget = d.nms_top_k < 0 ? d.M : d.nms_top_k;
  const long long base = static_cast<long long>(n) * d.s_n + static_cast<long long>(c) * d.s_c;

  NMS_PHASE_BEGIN;
  // 1. keys: positive scores compare like their bit patterns
  int local = 0;
  const float floor_score = d.tau != nullptr ? d.tau[n] : 0.f;
  switch (d.score_dtype) {
    case kF32: local = load_keys<float>(d, keys, base, floor_score); break;
    case kBF16: local = load_keys<__nv_bfloat16>(d, keys, base, floor_score); break;
    default: local = load_keys<__half>(d, keys, base, floor_score); break;
  }
  int total_pos;
  block_excl_scan(local, warp_tmp, &total_pos);

  NMS_PHASE(0);
  const bool normalized = d.normalized != 0;
  const int max_keep = d.max_keep;
  const float thr = d.nms_threshold;
  __shared__ int s_nk[2];
  float* o_score = d.cls_score + (static_cast<size_t>(n) * d.C + c) * max_keep;
  int* o_index = d.cls_index + (static_cast<size_t>(n) * d.C + c) * max_keep;
  const int lane = tid & 31, warp = tid >> 5;
  const uint32_t lower = (1u << lane) - 1u;
  int nkept = 0;
  while (total_pos > 0 && budget > 0 && nkept < max_keep) {
  const int K = min(budget, kNmsMaxTopK);
  // 2. radix select of the K-th largest key when there are more than K candidates
  uint32_t thr_key = 1u;   // admit keys >= thr_key ...
  int eq_budget = 1 << 30; // ... but only this many equal to thr_key (lowest indices first)
  if (total_pos > K) {
    if (tid == 0) { sel_prefix = 0u; sel_remaining = K; }
    __syncthreads();
    // fp16 scores widened to fp32 have 13 zero low bits, bf16 scores 16: their last passes are void
    const int min_shift = d.score_dtype == kF32 ? 0 : (d.score_dtype == kF16 ? 8 : 16);
    for (int shift = 24; shift >= min_shift; shift -= 8) {
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
      // thread t owns bin 255 - t; the bin whose suffix count first reaches the remainder is selected
      const int rem = sel_remaining;
      const int mybin = 255 - tid;
      const int hv = hist[mybin];
      int all_bins;
      const int above = block_excl_scan(hv, warp_tmp, &all_bins);
      if ((above < rem && above + hv >= rem) || (mybin == 0 && all_bins < rem)) {
        sel_prefix = prefix | (static_cast<uint32_t>(mybin) << shift);
        sel_remaining = rem - above;
      }
      __syncthreads();
    }
    thr_key = sel_prefix;
    eq_budget = sel_remaining;
    __syncthreads();
  }

  NMS_PHASE(1);
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
        if (pg < kNmsMaxTopK) { cand[pg] = v; keys[m] = 0u; }          // taken: out of the later passes
        ++pg;
      } else if (k == thr_key) {
        if (pe < eq_taken && tot_gt + pe < kNmsMaxTopK) { cand[tot_gt + pe] = v; keys[m] = 0u; }
        ++pe;
      }
    }
  }
  __syncthreads();

  NMS_PHASE(2);
  // 4. bitonic sort, descending, over the smallest power of two >= ncand
  int sort_n = 32;
  while (sort_n < ncand) sort_n <<= 1;
  for (int k = 2; k <= sort_n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int p = tid; p < (sort_n >> 1); p += kNmsThreads) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1)), ixj = i | j;
        const unsigned long long a = cand[i], b = cand[ixj];
        const bool desc = (i & k) == 0;
        if (desc ? (a < b) : (a > b)) { cand[i] = b; cand[ixj] = a; }
      }
      __syncthreads();
    }
  }

  NMS_PHASE(3);
  // 5. boxes of the sorted candidates
  const float4* boxes = reinterpret_cast<const float4*>(d.boxes) + static_cast<size_t>(n) * d.M;
  for (int i = tid; i < ncand; i += kNmsThreads) {
    const uint32_t m = 0xFFFFFFFFu - static_cast<uint32_t>(cand[i] & 0xFFFFFFFFull);
    const float4 b = boxes[m];
    cbox[i] = b;
    carea[i] = box_area(b, d.normalized != 0);
  }
  __syncthreads();

  NMS_PHASE(4);
  // 6. greedy sweep, 256 candidates per step, one per thread. Every thread first tests its
  // candidate against the boxes kept so far. Then the eight warps take turns: warp g resolves its
  // 32 candidates among themselves and appends the kept ones, and the later warps test their
  // candidates against just those new boxes. A candidate is therefore only ever compared with kept
  // boxes and with the members of its own group. Boxes past max_keep are dropped, which is exact
  // because a class contributes at most keep_top_k rows to the result.
  for (int b0 = 0; b0 < ncand && nkept < max_keep; b0 += kNmsThreads) {
    const int j = b0 + tid;
    bool alive = j < ncand;
    const float4 mine = alive ? cbox[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float my_area = alive ? carea[j] : 0.f;
    alive = alive && !hits_kept(mine, my_area, kbox, karea, 0, nkept, normalized, thr);
    // overlaps inside each group of 32, from the geometry alone: bit l of geo says that member l
    // (l < lane) overlaps this candidate. Computed by all warps at once, off the serial chain.
    uint32_t geo = 0u;
    if (__ballot_sync(0xffffffffu, alive)) {
#pragma unroll 4
      for (int l = 0; l < 31; ++l) {
        const int o = b0 + warp * 32 + l;   // always inside the 1024-entry arrays
        if (overlaps(mine, my_area, cbox[o], carea[o], normalized, thr)) geo |= 1u << l;
      }
      geo &= lower;
    }
    NMS_PHASE(5);
    for (int g = 0; g < kNmsThreads / 32 && nkept < max_keep && b0 + g * 32 < ncand; ++g) {
      if (warp == g) {
        const uint32_t am = __ballot_sync(0xffffffffu, alive);
        const uint32_t m = geo & am;   // earlier live members of the group that overlap this candidate
        bool a = alive;
        uint32_t pending = am, kept = 0u;
        while (pending) {
          const int l = __ffs(pending) - 1;   // the lowest live candidate is kept ...
          kept |= 1u << l;
          if ((m >> l) & 1u) a = false;        // ... and suppresses the later ones that overlap it
          pending = __ballot_sync(0xffffffffu, a) & ~((2u << l) - 1u);
        }
        const int pos = nkept + __popc(kept & lower);
        if (((kept >> lane) & 1u) && pos < max_keep) {
          kbox[pos] = mine;
          karea[pos] = my_area;
          o_score[pos] = __uint_as_float(static_cast<uint32_t>(cand[j] >> 32));
          o_index[pos] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(cand[j] & 0xFFFFFFFFull));
        }
        if (lane == 0) s_nk[g & 1] = min(nkept + __popc(kept), max_keep);
      }
      __syncthreads();
      const int newk = s_nk[g & 1];
      if (warp > g && alive) alive = !hits_kept(mine, my_area, kbox, karea, nkept, newk, normalized, thr);
#ifdef FDB_NMS_PROFILE
      if (threadIdx.x == 0) atomicAdd(&g_nms_phase[7], 1ull);
#endif
      nkept = newk;
    }
    __syncthreads();
    NMS_PHASE(6);
  }
  total_pos -= ncand;
  budget -= ncand;
  if (ncand == 0) break;
  __syncthreads();
  }  // passes
  if (tid == 0) *count_out = nkept;
}

// ------------------------------------------------------------------ pre-pass: a floor for the scores that can matter
// The result keeps at most keep_top_k rows per image, the best-scoring kept boxes over all classes. The
// kLead best candidates of a class, swept among themselves in score order, get exactly the verdict the
// full sweep gives them (a box is only ever suppressed by better-scoring boxes of its class). So these
// kept "leaders" are a subset of all kept boxes, and once an image has keep_top_k of them, the
// keep_top_k-th best leader score tau is a floor: a box scoring below tau is outranked by keep_top_k kept
// boxes and cannot reach the output, nor can it suppress a box scoring tau or more. The class kernel then
// drops everything below tau when it loads the scores, which is exact for every input and turns the dense
// score maps of an untrained or badly calibrated head (thousands of candidates per class, all swept for
// nothing) into a few candidates per class.
constexpr int kLead = 4;
constexpr int kTauMax = 4096;   // classes * kLead entries sorted per image

__device__ __forceinline__ void lead_insert(unsigned long long (&top)[kLead], unsigned long long v) {
#pragma unroll
  for (int i = 0; i < kLead; ++i) {
    if (v > top[i]) { const unsigned long long t = top[i]; top[i] = v; v = t; }
  }
}
// top kLead of the union of two descending lists, descending
__device__ __forceinline__ void lead_merge(unsigned long long (&a)[kLead], const unsigned long long (&b)[kLead]) {
  unsigned long long m[kLead];
#pragma unroll
  for (int i = 0; i < kLead; ++i) m[i] = a[i] > b[kLead - 1 - i] ? a[i] : b[kLead - 1 - i];   // bitonic, holds the top kLead
  // bitonic merge network for 4 elements, descending
  if (m[0] < m[2]) { const unsigned long long t = m[0]; m[0] = m[2]; m[2] = t; }
  if (m[1] < m[3]) { const unsigned long long t = m[1]; m[1] = m[3]; m[3] = t; }
  if (m[0] < m[1]) { const unsigned long long t = m[0]; m[0] = m[1]; m[1] = t; }
  if (m[2] < m[3]) { const unsigned long long t = m[2]; m[2] = m[3]; m[3] = t; }
#pragma unroll
  for (int i = 0; i < kLead; ++i) a[i] = m[i];
}
static_assert(kLead == 4, "lead_merge is written for four entries");

template <typename T>
__device__ __forceinline__ void lead_scan(const NmsDesc& d, long long base, unsigned long long (&top)[kLead]) {
  const T* src = reinterpret_cast<const T*>(d.scores) + base;
  for (int m0 = threadIdx.x; m0 < d.M; m0 += 4 * kNmsThreads) {
    T v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = src[static_cast<long long>(min(m0 + u * kNmsThreads, d.M - 1)) * d.s_m];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int m = m0 + u * kNmsThreads;
      const float sc = score_to_float(v[u]);
      if (m < d.M && sc > d.score_threshold && sc > 0.f)
        lead_insert(top, (static_cast<unsigned long long>(__float_as_uint(sc)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(m)));
    }
  }
}

__global__ void __launch_bounds__(kNmsThreads) nms_lead_kernel(const NmsDesc d) {
  const int c = blockIdx.x, n = blockIdx.y;
  float* out = d.lead + (static_cast<size_t>(n) * d.C + c) * kLead;
  if (c == d.background_label) {
    if (threadIdx.x < kLead) out[threadIdx.x] = 0.f;
    return;
  }
  const long long base = static_cast<long long>(n) * d.s_n + static_cast<long long>(c) * d.s_c;
  unsigned long long top[kLead] = {0ull, 0ull, 0ull, 0ull};
  switch (d.score_dtype) {
    case kF32: lead_scan<float>(d, base, top); break;
    case kBF16: lead_scan<__nv_bfloat16>(d, base, top); break;
    default: lead_scan<__half>(d, base, top); break;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other[kLead];
#pragma unroll
    for (int i = 0; i < kLead; ++i) other[i] = __shfl_xor_sync(0xffffffffu, top[i], o);
    lead_merge(top, other);
  }
  __shared__ unsigned long long wtop[kNmsThreads / 32][kLead];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kLead; ++i) wtop[warp][i] = top[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kNmsThreads / 32; ++w) {
      unsigned long long other[kLead];
#pragma unroll
      for (int i = 0; i < kLead; ++i) other[i] = wtop[w][i];
      lead_merge(top, other);
    }
    // greedy sweep of the leaders among themselves
    const float4* boxes = reinterpret_cast<const float4*>(d.boxes) + static_cast<size_t>(n) * d.M;
    const bool normalized = d.normalized != 0;
    float4 kb[kLead];
    float ka[kLead];
    int nk = 0;
    const int considered = min(kLead, d.nms_top_k < 0 ? kLead : d.nms_top_k);   // candidates past nms_top_k are never swept
    const int limit = min(considered, d.max_keep);
#pragma unroll
    for (int i = 0; i < kLead; ++i) {
      float sc = 0.f;
      if (top[i] != 0ull && i < considered && nk < limit) {
        const uint32_t m = 0xFFFFFFFFu - static_cast<uint32_t>(top[i] & 0xFFFFFFFFull);
        const float4 b = boxes[m];
        const float ar = box_area(b, normalized);
        bool hit = false;
        for (int k = 0; k < nk; ++k) hit |= overlaps(b, ar, kb[k], ka[k], normalized, d.nms_threshold);
        if (!hit) {
          kb[nk] = b; ka[nk] = ar; ++nk;
          sc = __uint_as_float(static_cast<uint32_t>(top[i] >> 32));
        }
      }
      out[i] = sc;
    }
  }
}

// tau[n] = keep_top_k-th best leader score of image n, or 0 when the image has fewer leaders.
__global__ void __launch_bounds__(1024) nms_tau_kernel(const NmsDesc d) {
  __shared__ uint32_t keys[kTauMax];
  const int n = blockIdx.x, tid = threadIdx.x;
  const int E = d.C * kLead;
  int sort_n = 32;
  while (sort_n < E) sort_n <<= 1;
  const float* lead = d.lead + static_cast<size_t>(n) * E;
  for (int i = tid; i < sort_n; i += 1024) keys[i] = i < E ? __float_as_uint(lead[i]) : 0u;
  __syncthreads();
  for (int k = 2; k <= sort_n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < sort_n; i += 1024) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const uint32_t a = keys[i], b = keys[ixj];
          const bool desc = (i & k) == 0;
          if (desc ? (a < b) : (a > b)) { keys[i] = b; keys[ixj] = a; }
        }
      }
      __syncthreads();
    }
  }
  if (tid == 0) d.tau[n] = d.keep_top_k <= sort_n ? __uint_as_float(keys[d.keep_top_k - 1]) : 0.f;
}

// Anchor-major scores [N][M][C] (unit class stride) -> class-major [N][C][M], 32 x 32 tiles.
template <typename T>
__global__ void __launch_bounds__(256) nms_transpose_kernel(const T* __restrict__ in, T* __restrict__ out, long long s_n,
                                                            long long s_m, int M, int C) {
  __shared__ T tile[32][33];
  const int n = blockIdx.z, m0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const T* src = in + n * s_n;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int m = m0 + ty + 8 * k, c = c0 + tx;
    if (m < M && c < C) tile[ty + 8 * k][tx] = src[m * s_m + c];
  }
  __syncthreads();
  T* dst = out + static_cast<size_t>(n) * C * M;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = c0 + ty + 8 * k, m = m0 + tx;
    if (m < M && c < C) dst[static_cast<size_t>(c) * M + m] = tile[tx][ty + 8 * k];
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

  // Ordered output: class ascending, rank ascending. Threads own consecutive runs of the
  // [class][rank] grid; positions come from a block scan over the selected counts.
  __shared__ int scan_tmp[1024 / 32 + 1];
  const int E = C * mk;
  const int per = (E + 1023) / 1024;
  const int e_begin = min(tid * per, E), e_end = min(e_begin + per, E);
  int cnt = 0;
  for (int e = e_begin; e < e_end; ++e) {
    const int c = e / mk, r = e - c * mk;
    if (r >= counts[c]) continue;
    const uint32_t sb = __float_as_uint(d.cls_score[static_cast<size_t>(n) * E + e]);
    const unsigned long long key = (static_cast<unsigned long long>(sb) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(e));
    cnt += (!select || key >= cut);
  }
  int sel_total;
  int pos = block_excl_scan<1024>(cnt, scan_tmp, &sel_total);
  for (int e = e_begin; e < e_end; ++e) {
    const int c = e / mk, r = e - c * mk;
    if (r >= counts[c]) continue;
    const float sc = d.cls_score[static_cast<size_t>(n) * E + e];
    const unsigned long long key = (static_cast<unsigned long long>(__float_as_uint(sc)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(e));
    if (select && key < cut) continue;
    if (pos < n_out) {
      const int m = d.cls_index[static_cast<size_t>(n) * E + e];
      const float4 b = boxes[m];
      float* o = out + static_cast<size_t>(pos) * 6;
      o[0] = static_cast<float>(c); o[1] = sc; o[2] = b.x; o[3] = b.y; o[4] = b.z; o[5] = b.w;
      out_idx[pos] = m;
    }
    ++pos;
  }
  if (tid == 0) d.out_num[n] = n_out;
}

struct NmsOp : Op {
  NmsDesc d;
  size_t smem1 = 0, smem2 = 0;
  int launch(cudaStream_t s) override {
    dim3 grid(d.C, d.N);
    if (d.scores_t != nullptr) {
      dim3 tgrid((d.M + 31) / 32, (d.C + 31) / 32, d.N);
      if (d.score_dtype == kF32) {
        nms_transpose_kernel<float><<<tgrid, 256, 0, s>>>(static_cast<const float*>(d.scores),
                                                          static_cast<float*>(d.scores_t), d.s_n, d.s_m, d.M, d.C);
      } else {
        nms_transpose_kernel<uint16_t><<<tgrid, 256, 0, s>>>(static_cast<const uint16_t*>(d.scores),
                                                             static_cast<uint16_t*>(d.scores_t), d.s_n, d.s_m, d.M, d.C);
      }
      NmsDesc t = d;
      t.scores = d.scores_t;
      t.s_n = static_cast<long long>(d.C) * d.M; t.s_c = d.M; t.s_m = 1;
      if (d.tau != nullptr) {
        nms_lead_kernel<<<grid, kNmsThreads, 0, s>>>(t);
        nms_tau_kernel<<<d.N, 1024, 0, s>>>(t);
      }
      nms_class_kernel<<<grid, kNmsThreads, smem1, s>>>(t);
    } else {
      if (d.tau != nullptr) {
        nms_lead_kernel<<<grid, kNmsThreads, 0, s>>>(d);
        nms_tau_kernel<<<d.N, 1024, 0, s>>>(d);
      }
      nms_class_kernel<<<grid, kNmsThreads, smem1, s>>>(d);
    }
    nms_merge_kernel<<<d.N, 1024, smem2, s>>>(d);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

}  // namespace fdb

using namespace fdb;

#ifdef FDB_NMS_PROFILE
FDB_API int fdb_nms_phase_read(unsigned long long* host8, int reset) {
  if (cudaMemcpyFromSymbol(host8, g_nms_phase, sizeof(g_nms_phase)) != cudaSuccess) return -1;
  if (reset) { unsigned long long z[8] = {}; cudaMemcpyToSymbol(g_nms_phase, z, sizeof(z)); }
  return 0;
}
#endif

// Scratch requirement in bytes for the per-class lists: counts, scores, indices.
// Leaders kept per class by the score-floor pre-pass (size of the `lead` scratch: N * C * this many floats).
FDB_API int fdb_nms_lead_per_class() { return kLead; }

FDB_API long long fdb_nms_scratch_bytes(int N, int C, int max_keep) {
  return static_cast<long long>(N) * C * (4 + 8ll * max_keep);
}

FDB_API void* fdb_nms_create(const NmsDesc* dp) {
  NmsDesc d = *dp;
  if (d.C > 1024) { set_error("nms: at most 1024 classes"); return nullptr; }
  if (d.scores_t != nullptr && d.s_c != 1) { set_error("nms: the transposing path needs unit class stride"); return nullptr; }
  if (d.N > 65535) { set_error("nms: at most 65535 images per launch"); return nullptr; }
  if (d.nms_top_k < -1 || d.nms_top_k == 0) {
    set_error("nms: nms_top_k must be -1 (no limit) or positive"); return nullptr;
  }
  if (d.keep_top_k == 0) { set_error("nms: keep_top_k must be -1 or positive"); return nullptr; }
  if (d.max_keep < 1 || d.max_keep > kNmsMaxTopK) { set_error("nms: max_keep must be in [1, 1024]"); return nullptr; }
  if (d.keep_top_k > -1 && static_cast<long long>(d.C) * d.max_keep > kMergeMax && d.keep_top_k < d.C * d.max_keep) {
    set_error("nms: classes * max_keep exceeds the merge capacity (8192)"); return nullptr;
  }
  if ((d.lead == nullptr) != (d.tau == nullptr)) { set_error("nms: lead and tau scratch come together"); return nullptr; }
  if (d.tau != nullptr && (d.keep_top_k < 1 || d.C * kLead > kTauMax || d.C * kLead < d.keep_top_k)) {
    set_error("nms: the score-floor pre-pass needs keep_top_k <= 4 * classes <= 4096"); return nullptr;
  }
  auto* op = new NmsOp();
  op->d = d;
  const int key_words = std::max((d.M + 3) & ~3, kNmsThreads * (kNmsThreads / 32));
  op->smem1 = static_cast<size_t>(key_words) * 4 + kNmsMaxTopK * 8 + kNmsMaxTopK * 20 + static_cast<size_t>(d.max_keep + 4) * 20;
  int sort_n = 32;
  while (sort_n < d.C * d.max_keep && sort_n < kMergeMax) sort_n <<= 1;
  op->smem2 = d.keep_top_k > -1 ? static_cast<size_t>(sort_n) * 8 : 16;
  if (op->smem1 > 200 * 1024) { set_error("nms: too many boxes per image for shared memory"); delete op; return nullptr; }
  // The opt-in limit is per function AND per device (one process may drive several GPUs): only ever raise it, other
  // ops on the same device may need more.
  static size_t max_dev[64][2] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("nms: no current device"); delete op; return nullptr; }
  size_t& max1 = max_dev[dev][0];
  size_t& max2 = max_dev[dev][1];
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
