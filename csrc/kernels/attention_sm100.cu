// Fused multi-head attention for short sequences (keys <= 512, head dim <= 128) on tcgen05 / TMEM.
//
// One CTA per (batch, head). K [Sk x D] and V^T [D x Sk] of that head are brought into shared memory
// once by TMA and stay there; the CTA then walks the query tiles of 128 rows:
//
//   S = Q K^T            tcgen05.mma, fp32 accumulator in tensor memory (one row per TMEM lane)
//   p = exp(scale * S + mask - rowmax)   two threads own each row (they split its 32-column blocks and
//                        exchange one maximum and one sum through shared memory); the whole row of
//                        scores is in TMEM, so the softmax is exact in one go (no running rescale)
//   O = P V              P is written as bf16 / fp16 into a 128B-swizzled K-major tile in shared memory,
//                        at most 256 keys at a time, and multiplied by the resident V^T; O's accumulator
//                        reuses the TMEM columns of S, which are dead by then
//   out = O / rowsum     straight from TMEM to the [B, S, H * D] output
//
// The score matrix never exists in global memory. The reference gets attention from its vendor
// back ends (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:347); there is no source to mirror.
//
// Every wait is bounded and reports through the status word; on a timeout the CTA frees its TMEM
// and returns.
#include "fdb_common.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <functional>

namespace fdb {

struct AttnDesc {
  const void* q; const void* k; const void* vt; void* out; const float* mask; int* status;
  const int* seq_len;        // device, one per batch item: keys (and, when S == Sk, queries) that are real; may be null
  const int* seq_start;      // device, one per batch item: first row of the item in q / k / out and first column
                             // in vt (multiples of 8); null = items are S (Sk) rows apart
  int dtype;                 // kF16 or kBF16
  int B, H, S, Sk, D;
  int q_ld, k_ld, o_ld;      // row pitches in elements; rows of one batch item are S (Sk) consecutive rows
  int skp;                   // row pitch of vt [B][H][D][skp]; with seq_start: vt is [H][D][skp] over all rows
  int total_rows;            // with seq_start: rows of q / k / out (all items together)
  long long m_b, m_s;        // mask element (b, s, k) at b * m_b + s * m_s + k; mask may be null
  float scale;
};

struct AttnParams {
  const float* mask; uint8_t* out; int* status;
  const int* seq_len; const int* seq_start;
  const int* key_len;        // per item, derived from the mask by mask_prefix_kernel: >= 1 when the mask row is "that
                             // many zeros, then only entries <= -1000" (a key-padding mask), else -1
  int total_rows;
  int H, S, Sk, D, o_ld;
  int sk_pad;                // keys rounded up: multiple of 16 (<= 256) or of 32 (> 256)
  int d_chunks;              // ceil(D / 64)
  int k_chunks;              // ceil(sk_pad / 64)
  int k_box, k_loads;        // rows per K TMA box and boxes per D chunk
  int q_tiles;
  int tmem_cols;
  long long m_b, m_s;
  float scale;
  uint32_t smem_k, smem_vt, smem_q, smem_p;   // byte offsets from the 1024-aligned base
};

constexpr int kAttnThreads = 256;   // two warps per TMEM lane quarter: they split the score columns

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (BF16) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One warp per batch item: key_len[b] = n when mask row b is n zeros followed only by entries <= -1000 (n >= 1),
// else -1. Such a row is a key-padding mask, and the attention kernel then works from the count alone.
__global__ void mask_prefix_kernel(const float* __restrict__ mask, long long m_b, int B, int Sk, int* __restrict__ key_len) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= B) return;
  const float* row = mask + b * m_b;
  int first_masked = Sk;          // first index whose entry is not zero
  bool ok = true;
  for (int c = lane; c < Sk; c += 32) {
    const float v = __ldg(row + c);
    if (v != 0.f) first_masked = min(first_masked, c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) first_masked = min(first_masked, __shfl_xor_sync(0xffffffffu, first_masked, o));
  for (int c = lane; c < Sk; c += 32) {
    const float v = __ldg(row + c);
    if (c >= first_masked && !(v <= -1000.f)) ok = false;
  }
  ok = __all_sync(0xffffffffu, ok);
  if (lane == 0) key_len[b] = (ok && first_masked >= 1) ? first_masked : -1;
}

template <bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_vt, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[4];      // 0 K/V landed, 1 Q landed, 2 S ready, 3 PV group done
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  __shared__ float red_max[2][128], red_sum[2][128];
  volatile int* abort_flag = &abort_word;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base + p.smem_k, sVT = base + p.smem_vt, sQ = base + p.smem_q, sP = base + p.smem_p;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127;          // row of the query tile this thread owns (lane of tensor memory)
  const int half = warp >> 2;       // which half of the 32-column blocks (and of the output columns) it handles
  const int b = blockIdx.x / p.H, h = blockIdx.x - b * p.H;
  const uint32_t bar_kv = smem_u32(&bars[0]), bar_q = smem_u32(&bars[1]), bar_s = smem_u32(&bars[2]),
                 bar_o = smem_u32(&bars[3]);

  if (tid == 0) {
    abort_word = 0;
    mbar_init(bar_kv, 1); mbar_init(bar_q, 1); mbar_init(bar_s, 1); mbar_init(bar_o, 1);
    fence_mbar_init();
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_vt);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  const uint32_t q_chunk_bytes = 128u * 128u;                         // 128 rows x 128 B
  const uint32_t k_chunk_bytes = static_cast<uint32_t>(p.sk_pad) * 128u;
  const uint32_t vt_chunk_bytes = static_cast<uint32_t>((p.D + 7) / 8 * 8) * 128u;
  const int col0 = h * p.D;

  // Per-item lengths. Everything below sizes its loops by `len`; the loads keep the planned box sizes (rows past
  // the item are other items' rows or the zero fill, and never reach a result: their probabilities are written
  // as zero and their scores are never read).
  int len = p.Sk, q_row0 = b * p.S, k_row0 = b * p.Sk, vt_x0 = 0, vt_y0 = (b * p.H + h) * p.D;
  bool valid = true;
  if (p.seq_len != nullptr) len = max(0, min(__ldg(p.seq_len + b), p.Sk));
  // A key-padding mask is the same as a key count: masked keys get weight exp(-1000 or less) = 0 exactly in fp32,
  // so they are left out (no mask loads, shorter loops); every query row is still computed.
  bool mask_as_len = false;
  if (p.key_len != nullptr) {
    const int kl = __ldg(p.key_len + b);
    if (kl >= 1) { len = min(kl, p.Sk); mask_as_len = true; }
  }
  if (p.seq_start != nullptr) {
    const int st = __ldg(p.seq_start + b);
    valid = st >= 0 && (st & 7) == 0 && st + len <= p.total_rows;
    q_row0 = k_row0 = vt_x0 = st;
    vt_y0 = h * p.D;
  }
  const int S_b = (p.seq_len != nullptr && p.S == p.Sk) ? len : p.S;
  const int sk_pad = len <= 256 ? (len + 15) / 16 * 16 : (len + 31) / 32 * 32;
  const int k_chunks = (sk_pad + 63) / 64;
  const int q_tiles = (S_b + 127) / 128;
  if (!valid && tid == 0) abort_word = kStatusBadShape;
  const bool run = valid && len > 0;

  if (run && tid == 0) {
    // K: d_chunks x k_loads boxes of [k_box rows x 64 cols]; V^T: k_chunks boxes of [D rows x 64 cols]. Only the
    // boxes that hold keys of this item are fetched.
    const int k_loads = sk_pad > p.k_box ? p.k_loads : 1;
    const uint32_t bytes = static_cast<uint32_t>(p.d_chunks * k_loads) * static_cast<uint32_t>(p.k_box) * 128u +
                           static_cast<uint32_t>(k_chunks) * static_cast<uint32_t>(p.D) * 128u;
    mbar_arrive_expect_tx(bar_kv, bytes);
    for (int c = 0; c < p.d_chunks; ++c)
      for (int l = 0; l < k_loads; ++l)
        tma_load_2d(sK + c * k_chunk_bytes + static_cast<uint32_t>(l * p.k_box) * 128u, &tm_k, bar_kv, col0 + c * 64,
                    k_row0 + l * p.k_box);
    for (int j = 0; j < k_chunks; ++j)
      tma_load_2d(sVT + j * vt_chunk_bytes, &tm_vt, bar_kv, vt_x0 + j * 64, vt_y0);
    mbar_arrive_expect_tx(bar_q, static_cast<uint32_t>(p.d_chunks) * q_chunk_bytes);
    for (int c = 0; c < p.d_chunks; ++c) tma_load_2d(sQ + c * q_chunk_bytes, &tm_q, bar_q, col0 + c * 64, q_row0);
  }

  const uint32_t fmt = BF16 ? 1u : 0u;
  const int n_first = sk_pad > 256 ? 256 : sk_pad;
  const int n_second = sk_pad - n_first;
  const int d_steps_last = ((p.D - (p.d_chunks - 1) * 64) + 15) / 16;
  const float sl2 = p.scale * 1.4426950408889634f;
  uint32_t o_phase = 0;
  bool ok = run && mbar_wait(bar_kv, 0, abort_flag, kStatusTimeoutProducer);

  for (int qt = 0; ok && qt < q_tiles; ++qt) {
    ok = mbar_wait(bar_q, qt & 1, abort_flag, kStatusTimeoutProducer);
    if (!ok) break;
    // ---------------------------------------------------------------- S = Q K^T
    if (tid == 0) {
      tc_fence_after();
      for (int part = 0; part < (n_second > 0 ? 2 : 1); ++part) {
        const int n = part == 0 ? n_first : n_second;
        const uint32_t idesc = make_idesc(fmt, 128, static_cast<uint32_t>(n));
        for (int c = 0; c < p.d_chunks; ++c) {
          const uint64_t ad = make_kmajor_desc(sQ + c * q_chunk_bytes, 128);
          const uint64_t bd = make_kmajor_desc(sK + c * k_chunk_bytes + static_cast<uint32_t>(part * 256) * 128u, 128);
          umma_f16_ksteps(tmem + static_cast<uint32_t>(part * 256), ad, bd, idesc, c != 0 ? 1u : 0u,
                          c + 1 == p.d_chunks ? static_cast<uint32_t>(d_steps_last) : 4u);
        }
      }
      umma_commit(bar_s);
    }
    ok = mbar_wait(bar_s, qt & 1, abort_flag, kStatusTimeoutMma);
    if (!ok) break;
    tc_fence_after();
    const int row = qt * 128 + r;
    const float* mrow = p.mask != nullptr ? p.mask + b * p.m_b + static_cast<long long>(row < S_b ? row : 0) * p.m_s : nullptr;
    // Warps whose 32 rows all lie beyond the last query take part in the barriers only.
    const bool warp_active = qt * 128 + (warp & 3) * 32 < S_b;
    const bool masked = mrow != nullptr && !mask_as_len;
    const int nblk = (sk_pad + 31) / 32;
    constexpr float kLog2e = 1.4426950408889634f;
    uint32_t va[32], vb[32];
    // ---------------------------------------------------------------- pass 1: row maximum
    // Without a mask the maximum is taken over the raw scores and scaled once (scale > 0); with a mask
    // it is taken over scale * s + mask in log2 units. Four partial maxima keep the chain short, and the
    // next 32 columns are already on their way out of tensor memory while these are compared.
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    auto max_block = [&](const uint32_t (&v)[32], int c0) {
      if (!masked && c0 + 32 <= len) {
#pragma unroll
        for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], __uint_as_float(v[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c0 + j;
          if (col < len) {
            float sv = __uint_as_float(v[j]);
            if (masked) sv = fmaf(sv, sl2, __ldg(mrow + col) * kLog2e);
            m4[j & 3] = fmaxf(m4[j & 3], sv);
          }
        }
      }
    };
    float mx = 0.f;
    if (warp_active) {
      int blk = half;
      if (blk < nblk) tmem_ld_32x32(lane_base + static_cast<uint32_t>(blk * 32), va);
      for (; blk < nblk; blk += 4) {
        tmem_ld_wait_dep(va);
        if (blk + 2 < nblk) tmem_ld_32x32(lane_base + static_cast<uint32_t>((blk + 2) * 32), vb);
        max_block(va, blk * 32);
        if (blk + 2 < nblk) {
          tmem_ld_wait_dep(vb);
          if (blk + 4 < nblk) tmem_ld_32x32(lane_base + static_cast<uint32_t>((blk + 4) * 32), va);
          max_block(vb, (blk + 2) * 32);
        }
      }
      float part = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      if (!masked) part *= sl2;
      red_max[half][r] = part;
    }
    __syncthreads();                 // the two warps of a row exchange their partial maxima
    if (warp_active) {
      mx = fmaxf(red_max[0][r], red_max[1][r]);
      if (mx == -INFINITY) mx = 0.f;
    }
    // ---------------------------------------------------------------- pass 2: P and O = P V, 4 key chunks at a time
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
    const int groups = (k_chunks + 3) / 4;
    const uint32_t prow = sP + static_cast<uint32_t>(r) * 128u;
    const uint32_t r7 = static_cast<uint32_t>(r & 7);
    const float neg_mx = -mx;
    // 32 probabilities -> 16 packed words -> four 16-byte stores into the swizzled row of chunk `lc`
    auto prob_block = [&](const uint32_t (&v)[32], int c0, int lc, int half) {
      uint32_t w[16];
      if (!masked && c0 + 32 <= len) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(v[2 * j]), sl2, neg_mx));
          const float e1 = ex2_approx(fmaf(__uint_as_float(v[2 * j + 1]), sl2, neg_mx));
          s4[j & 3] += e0 + e1;
          w[j] = pack2<BF16>(e0, e1);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float e[2];
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int col = c0 + 2 * j + t;
            float off = neg_mx;
            if (masked && col < len) off = fmaf(__ldg(mrow + col), kLog2e, neg_mx);
            e[t] = col < len ? ex2_approx(fmaf(__uint_as_float(v[2 * j + t]), sl2, off)) : 0.f;
          }
          s4[j & 3] += e[0] + e[1];
          w[j] = pack2<BF16>(e[0], e[1]);
        }
      }
      const uint32_t cbase = prow + static_cast<uint32_t>(lc) * q_chunk_bytes;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t addr = cbase + ((static_cast<uint32_t>(half * 4 + u) ^ r7) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * u]), "r"(w[4 * u + 1]),
                     "r"(w[4 * u + 2]), "r"(w[4 * u + 3]) : "memory");
      }
    };
    for (int g = 0; ok && g < groups; ++g) {
      const int ch0 = g * 4, ch1 = min(k_chunks, ch0 + 4);
      if (warp_active) {
        // 32-column blocks b0 .. b1-1 of this group; this warp takes every other one (blk & 1 == half), so
        // it always writes the same half of a 64-key chunk; blocks >= nblk are padding and written as zero
        const int b0 = ch0 * 2, b1 = ch1 * 2;
        auto zero_block = [&](int lc) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(
                prow + static_cast<uint32_t>(lc) * q_chunk_bytes + ((static_cast<uint32_t>(half * 4 + u) ^ r7) << 4)), "r"(0u) : "memory");
        };
        int blk = b0 + half;
        if (blk < nblk) tmem_ld_32x32(lane_base + static_cast<uint32_t>(blk * 32), va);
        for (; blk < b1; blk += 4) {
          if (blk < nblk) {
            tmem_ld_wait_dep(va);
            if (blk + 2 < b1 && blk + 2 < nblk) tmem_ld_32x32(lane_base + static_cast<uint32_t>((blk + 2) * 32), vb);
            prob_block(va, blk * 32, (blk >> 1) - ch0, half);
          } else {
            zero_block((blk >> 1) - ch0);
          }
          if (blk + 2 < b1) {
            if (blk + 2 < nblk) {
              tmem_ld_wait_dep(vb);
              if (blk + 4 < b1 && blk + 4 < nblk) tmem_ld_32x32(lane_base + static_cast<uint32_t>((blk + 4) * 32), va);
              prob_block(vb, (blk + 2) * 32, ((blk + 2) >> 1) - ch0, half);
            } else {
              zero_block(((blk + 2) >> 1) - ch0);
            }
          }
        }
        if (g + 1 == groups) red_sum[half][r] = (s4[0] + s4[1]) + (s4[2] + s4[3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        const uint32_t idesc = make_idesc(fmt, 128, static_cast<uint32_t>((p.D + 15) / 16 * 16));
        for (int ch = ch0; ch < ch1; ++ch) {
          const int keys = min(64, sk_pad - ch * 64);
          const uint64_t ad = make_kmajor_desc(sP + static_cast<uint32_t>(ch - ch0) * q_chunk_bytes, 128);
          const uint64_t bd = make_kmajor_desc(sVT + static_cast<uint32_t>(ch) * vt_chunk_bytes, 128);
          umma_f16_ksteps(tmem, ad, bd, idesc, ch != 0 ? 1u : 0u, static_cast<uint32_t>((keys + 15) / 16));
        }
        umma_commit(bar_o);
        // Q is free since S was committed, and every thread is past its wait on this tile's Q barrier
        // (they all met at the barrier above): fetch the next tile's Q behind the rest of this one.
        if (g == 0 && qt + 1 < q_tiles) {
          mbar_arrive_expect_tx(bar_q, static_cast<uint32_t>(p.d_chunks) * q_chunk_bytes);
          for (int c = 0; c < p.d_chunks; ++c)
            tma_load_2d(sQ + c * q_chunk_bytes, &tm_q, bar_q, col0 + c * 64, q_row0 + (qt + 1) * 128);
        }
      }
      ok = mbar_wait(bar_o, o_phase, abort_flag, kStatusTimeoutMma);
      o_phase ^= 1u;
      tc_fence_after();
    }
    if (!ok) break;
    // ---------------------------------------------------------------- out = O / sum
    const float sum = warp_active ? red_sum[0][r] + red_sum[1][r] : 0.f;
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    uint8_t* orow = p.out + ((static_cast<long long>(q_row0) + row) * p.o_ld + col0) * 2;
    for (int c0 = half * 32; warp_active && c0 < p.D; c0 += 64) {
      uint32_t v[32];
      tmem_ld_32x32(lane_base + static_cast<uint32_t>(c0), v);
      tmem_ld_wait_dep(v);
      if (row < S_b) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c0 + u * 8 < p.D) {
            uint4 o;
            o.x = pack2<BF16>(__uint_as_float(v[8 * u]) * inv, __uint_as_float(v[8 * u + 1]) * inv);
            o.y = pack2<BF16>(__uint_as_float(v[8 * u + 2]) * inv, __uint_as_float(v[8 * u + 3]) * inv);
            o.z = pack2<BF16>(__uint_as_float(v[8 * u + 4]) * inv, __uint_as_float(v[8 * u + 5]) * inv);
            o.w = pack2<BF16>(__uint_as_float(v[8 * u + 6]) * inv, __uint_as_float(v[8 * u + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + (c0 + u * 8) * 2) = o;
          }
        }
      }
    }
    // the next tile's S overwrites the TMEM columns that were just read
    tc_fence_before();
    __syncthreads();
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, abort_word);
  if (warp == 0) tmem_dealloc(tmem, static_cast<uint32_t>(p.tmem_cols));
}

}  // namespace fdb

using namespace fdb;

namespace {

struct AttnOp : Op {
  CUtensorMap tq, tk, tvt;
  AttnParams prm;
  int grid = 0, smem = 0;
  bool bf16 = true;
  int* key_len = nullptr;     // owned: filled from the mask before every launch (the mask is an input of the step)
  int batch = 0;
  ~AttnOp() override { if (key_len != nullptr) cudaFree(key_len); }
  int launch(cudaStream_t s) override {
    if (key_len != nullptr)
      mask_prefix_kernel<<<(batch + 7) / 8, 256, 0, s>>>(prm.mask, prm.m_b, batch, prm.Sk, key_len);
    if (bf16) attention_kernel<true><<<grid, kAttnThreads, smem, s>>>(tq, tk, tvt, prm);
    else attention_kernel<false><<<grid, kAttnThreads, smem, s>>>(tq, tk, tvt, prm);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error(std::string("attention: ") + cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

bool encode_2d(CUtensorMap* m, CUtensorMapDataType dt, const void* base, unsigned long long inner,
               unsigned long long rows, unsigned long long row_bytes, unsigned box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

FDB_API int fdb_attention_desc_size() { return static_cast<int>(sizeof(AttnDesc)); }

// Plans one fused attention launch over fixed buffers. q [B*S rows, q_ld], k [B*Sk rows, k_ld] (head h in
// columns h*D .. h*D+D-1), vt [B][H][D][skp] (V transposed per head, zero beyond Sk), out [B*S rows, o_ld].
// seq_len (device) gives each item's real length; with seq_start (device, multiples of 8) the items are packed
// back to back: q / k / out hold total_rows rows, vt is [H][D][skp] over all rows, S = Sk is the longest item
// the plan admits, and B is the largest number of items (an item of length 0 costs an empty CTA).
FDB_API void* fdb_attention_create(const AttnDesc* d) {
  if (d->dtype != kF16 && d->dtype != kBF16) { set_error("attention: dtype must be fp16 or bf16"); return nullptr; }
  if (!(d->scale > 0.f)) { set_error("attention: the score scale must be positive"); return nullptr; }
  if (d->D % 16 != 0 || d->D < 16 || d->D > 128 || d->Sk < 1 || d->Sk > 512 || d->S < 1 || d->B < 1 || d->H < 1) {
    set_error("attention: needs head dim in 16..128 (multiple of 16) and 1..512 keys"); return nullptr;
  }
  auto al16 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
  if (!al16(d->q) || !al16(d->k) || !al16(d->vt) || !al16(d->out) || d->q_ld % 8 || d->k_ld % 8 || d->o_ld % 8 ||
      d->skp % 8 || (d->seq_start == nullptr && d->skp < d->Sk)) {
    set_error("attention: pointers must be 16-byte aligned and row pitches multiples of 8 elements"); return nullptr;
  }
  const bool packed = d->seq_start != nullptr;
  if (packed && (d->seq_len == nullptr || d->S != d->Sk || d->total_rows < 1 || d->mask != nullptr)) {
    set_error("attention: packed batches need seq_len, S == Sk, total_rows and no mask"); return nullptr;
  }
  auto* op = new AttnOp();
  AttnParams& p = op->prm;
  p.seq_len = d->seq_len; p.seq_start = d->seq_start; p.total_rows = packed ? d->total_rows : d->B * d->S;
  p.mask = d->mask; p.out = static_cast<uint8_t*>(d->out); p.status = d->status;
  p.H = d->H; p.S = d->S; p.Sk = d->Sk; p.D = d->D; p.o_ld = d->o_ld;
  p.sk_pad = d->Sk <= 256 ? (d->Sk + 15) / 16 * 16 : (d->Sk + 31) / 32 * 32;
  p.d_chunks = (d->D + 63) / 64;
  p.k_chunks = (p.sk_pad + 63) / 64;
  p.k_loads = p.sk_pad > 256 ? 2 : 1;
  p.k_box = p.sk_pad / p.k_loads;
  p.q_tiles = (d->S + 127) / 128;
  int cols = 32;
  while (cols < std::max((p.sk_pad + 31) / 32 * 32, (d->D + 31) / 32 * 32)) cols *= 2;
  p.tmem_cols = cols;
  p.m_b = d->m_b; p.m_s = d->m_s; p.scale = d->scale;
  p.key_len = nullptr;
  op->batch = d->B;
  if (d->mask != nullptr && d->m_s == 0 && d->seq_len == nullptr) {
    // one mask row per item: worth a look whether it is a key-padding mask
    if (cudaMalloc(&op->key_len, sizeof(int) * static_cast<size_t>(d->B)) != cudaSuccess) {
      cudaGetLastError();
      op->key_len = nullptr;
    }
    p.key_len = op->key_len;
  }
  const uint32_t k_bytes = static_cast<uint32_t>(p.d_chunks) * p.sk_pad * 128u;
  const uint32_t vt_bytes = static_cast<uint32_t>(p.k_chunks) * d->D * 128u;
  const uint32_t q_bytes = static_cast<uint32_t>(p.d_chunks) * 16384u;
  const uint32_t p_bytes = static_cast<uint32_t>(std::min(p.k_chunks, 4)) * 16384u;
  p.smem_k = 0; p.smem_vt = k_bytes; p.smem_q = k_bytes + vt_bytes; p.smem_p = k_bytes + vt_bytes + q_bytes;
  op->smem = static_cast<int>(k_bytes + vt_bytes + q_bytes + p_bytes + 1024u);
  if (op->smem + 4096 > 227 * 1024) {      // 4 KB: the kernel's static shared memory (barriers, row exchange)
    set_error("attention: K, V and the probability tile do not fit in shared memory (" + std::to_string(op->smem) + " bytes)");
    delete op; return nullptr;
  }
  op->bf16 = d->dtype == kBF16;
  op->grid = d->B * d->H;
  const CUtensorMapDataType dt = op->bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const unsigned long long width = static_cast<unsigned long long>(d->H) * d->D;
  const unsigned long long q_rows = packed ? d->total_rows : static_cast<unsigned long long>(d->B) * d->S;
  const unsigned long long k_rows = packed ? d->total_rows : static_cast<unsigned long long>(d->B) * d->Sk;
  const unsigned long long vt_rows = static_cast<unsigned long long>(packed ? 1 : d->B) * d->H * d->D;
  if (!encode_2d(&op->tq, dt, d->q, width, q_rows, d->q_ld * 2ull, 128) ||
      !encode_2d(&op->tk, dt, d->k, width, k_rows, d->k_ld * 2ull, p.k_box) ||
      !encode_2d(&op->tvt, dt, d->vt, d->skp, vt_rows, d->skp * 2ull, d->D)) {
    set_error("attention: tensor map encoding failed"); delete op; return nullptr;
  }
  const void* fn = op->bf16 ? reinterpret_cast<const void*>(&attention_kernel<true>)
                            : reinterpret_cast<const void*>(&attention_kernel<false>);
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, op->smem) != cudaSuccess) {
    cudaGetLastError();
    set_error("attention: cannot raise the dynamic shared memory limit"); delete op; return nullptr;
  }
  return op;
}
