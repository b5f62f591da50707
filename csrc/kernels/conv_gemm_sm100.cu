// Implicit-GEMM convolution / GEMM on the 5th-generation tensor cores (sm_100a).
//
// One persistent, warp-specialised kernel serves conv2d (any KHxKW, stride 1/2,
// zero padding), 1x1 convolutions and plain row-major GEMMs (a GEMM is a 1x1
// convolution over a 1 x M "image"):
//
//   warp 0   TMA producer : for every (tap, 64-channel slab) one 4-D tiled
//            cp.async.bulk.tensor load of a  tile_h x tile_w x 64ch  activation
//            patch (NHWC) - the tap offset is a coordinate offset and the
//            zero padding is TMA's out-of-bounds fill, so no im2col buffer
//            exists - plus one 2-D load of the BN x 64 weight slab.
//   warp 1   MMA issuer   : tcgen05.mma kind::f16, 128 x BN x 16 per instruction,
//            accumulators double-buffered in TMEM (2 x BN fp32 columns).
//   warps 2-9 epilogue    : tcgen05.ld TMEM -> registers, + bias, (+ residual),
//            activation, cast, 16-byte stores straight into the (possibly
//            channel-offset, i.e. concat-fused) NHWC output.
//
// Replaces what the reference delegates to TensorRT / cuDNN / cuBLAS
// (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:347 enqueueV2).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <vector>

#include "fdb_common.h"
#include "sm100_ptx.cuh"

namespace fdb {

constexpr int kBM = 128;       // tile rows = TMEM lanes
constexpr int kBK = 64;        // K elements per pipeline stage (128-byte rows)
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;  // producer + MMA + 8 epilogue warps

// C ABI descriptor (mirrored by ctypes in fastdeploy_b200/ops/conv_gemm.py).
struct ConvGemmDesc {
  const void* x;         // NHWC input, already offset to the first used channel
  const void* w;         // packed weights [Cout][KH*KW][cin_pad], K-major
  const float* bias;     // [Cout] fp32 or null
  const void* residual;  // same dtype as x, NHWC with res_ld, or null
  void* y;               // NHWC output, already offset to the first written channel
  int* status;           // device int, receives a KernelStatus on failure
  int dtype;             // kF16 | kBF16 : x, w, residual
  int out_dtype;         // kF16 | kBF16 | kF32
  int N, H, W, Cin, x_ld;
  int Ho, Wo, Cout, y_ld;
  int KH, KW, stride, pad_h, pad_w;
  int res_ld, res_mode;  // 0 none, 1 add before activation, 2 add after activation
  int act;
  float act_alpha, act_beta;
  int tile_w, tile_h;    // 0 = choose
  int block_n;           // 0 = choose (32/64/128/256)
  int max_ctas;          // 0 = one per SM
  long long x_n_stride;  // elements between images (0 = H*W*x_ld)
  long long y_n_stride;  // elements between images (0 = Ho*Wo*y_ld)
  long long res_n_stride;
  int halo_mode;         // 3x3 stride-1 halo kernel: -1 choose, 0 never, 1 force
  // Batched "weights" (attention products): one [Cout][K] matrix per (image row h, image n),
  // row stride w_ld, matrix strides w_h_stride / w_n_stride (elements). Needs tile_h = 1.
  int w_batched;
  int w_ld;
  long long w_h_stride, w_n_stride;
  // elements between image rows (0 = W * ld): lets heads of a [B, S, H*D] tensor act as image rows
  long long x_h_stride, y_h_stride, res_h_stride;
  int y_tma_mode;        // -1/1: TMA tensor stores for 16-bit outputs when possible, 0: direct stores
  long long* trace;      // optional device buffer of 2*32*12 int64 for the timeline probe (null = off)
  // Tensor parallelism over peer memory (plain GEMMs only: 1x1, one image row of W = M rows).
  //   peer_mode 1, all-gather -> GEMM: the M rows of A live in peer_world equal shards of peer_rows
  //     rows; shard r is read straight from peer_ptrs[r] (this rank's own shard included) by TMA.
  //   peer_mode 2, GEMM -> reduce-scatter: the 128-row output block whose rows belong to rank o is
  //     stored by TMA into slot peer_rank of o's slot buffer peer_ptrs[o] ([world][peer_rows][y_ld])
  //     and o's counter for that block (peer_counters[o][block]) is bumped once per store.
  int peer_mode, peer_rows, peer_rank, peer_world;
  void* peer_ptrs[8];
  unsigned int* peer_counters[8];
  // peer_mode 1 only: x is this rank's gathered buffer [M][x_ld] (same heap offset on every rank, rank r's
  // shard valid at rows r * peer_rows of its own buffer, peer_ptrs[r] = base of rank r's buffer);
  // peer_ready = M / 128 flags in local memory; peer_copiers = CTAs set aside to pull the remote shards.
  unsigned int* peer_ready;
  int peer_copiers;
  // fp8 operands (dtype = kF8E4M3, generic kernel only): fp32 scales applied to the fp32 accumulator in
  // the epilogue, scale_a per output row (pixel / token), scale_b per output channel; either may be null.
  const float* scale_a;
  const float* scale_b;
  // CTA pairs (cta_group::2): -1 choose, 0 never, 1 force. A pair computes two 128-row tiles of the same
  // column tile with one M = 256 MMA; each CTA stages half of the weight tile.
  int pair_mode;
  // out_dtype = kF8E4M3: the result (after bias, activation and residual) is multiplied by out_scale - the
  // reciprocal of the consumer's activation scale - and stored as e4m3, so the next GEMM reads fp8 directly
  float out_scale;
};

// Device-resident table of the peers' tensor maps and counters (host-written before any launch).
struct PeerTable {
  alignas(64) CUtensorMap maps[8];
  unsigned int* counters[8];
};

struct ConvGemmParams {
  const float* bias;
  const void* residual;
  void* y;
  int* status;
  int Ho, Wo, Cout, y_ld, res_ld, res_mode, out_dtype, in_bf16;
  int KH, KW, stride, pad_h, pad_w;
  int tw, th, tiles_w, tiles_h, n_tiles, total_tiles;
  unsigned long long mul_n, mul_w, mul_h;   // ceil(2^40 / divisor) for n_tiles, tiles_w, tiles_h
  int kb_per_tap, k_iters;
  int last_ksteps;   // K = 16 steps that carry data in the last 64-wide slab of each tap (1..4)
  int act;
  float act_alpha, act_beta;
  uint32_t a_bytes;
  uint32_t idesc;
  int y_vec, res_vec;
  long long y_n_stride, res_n_stride;
  long long y_h_stride, res_h_stride;
  int b_batched;
  int y_tma;   // 16-bit output leaves through shared-memory staging + TMA tensor stores
  const PeerTable* peer;   // null unless peer_mode != 0
  int peer_mode, peer_rows, peer_rank;
  int kblk;                // K elements per pipeline stage: 64 (16-bit operands) or 128 (fp8), always 128 bytes
  int fp8;                 // operands are e4m3
  const float* scale_a;    // fp8: per-row and per-column dequantisation scales (null = 1)
  const float* scale_b;
  int gemm_ctas;           // CTAs that run the GEMM roles; the rest of the grid (peer_mode 1) are copiers
  int peer_world, peer_rot;       // all-gather mode: ranks, and the tile-row rotation that puts local rows first
  unsigned peer_epoch;            // value the ready flags take in this launch
  unsigned* ready;                // [tiles_w] flags of the gathered buffer, written by the copier CTAs
  uint8_t* gather_dst;            // this rank's gathered A buffer ([M][x_ld] 16-bit)
  const uint8_t* peer_src[8];     // every rank's gathered buffer (rank r's shard is valid in its own)
  long long gather_row_bytes;     // bytes per row of A
  long long* trace;  // optional: CTA 0 records clock64() at pipeline events of its first tiles
  int pair;          // launched as clusters of two CTAs that share every MMA
  int n_images;      // N: tiles decoded to an image index past it are padding of an odd tile count (pairs)
  int epi_teams;     // TMA-store epilogue: 1 = the two warp halves drain alternate tiles, 0 = both drain every tile
  float out_scale;   // applied before an e4m3 store
};

// Tile index -> (column tile, tile column, tile row, image). Integer division by the three runtime
// divisors is replaced by a multiply with ceil(2^40 / d) and a shift, exact while index * d < 2^40
// (the host refuses larger problems): every role decodes once per tile, and the hardware division
// sequence is long enough to show in the per-tile cost of small layers.
struct TileCoord { int n_tile, twi, thi, img; };
__device__ __forceinline__ uint32_t fast_div(uint32_t n, unsigned long long mul) {
  return static_cast<uint32_t>((static_cast<unsigned long long>(n) * mul) >> 40);
}
__device__ __forceinline__ TileCoord decode_tile(const ConvGemmParams& p, int tile) {
  const uint32_t t = static_cast<uint32_t>(tile);
  const uint32_t m = fast_div(t, p.mul_n);
  const uint32_t r = fast_div(m, p.mul_w);
  const uint32_t img = fast_div(r, p.mul_h);
  TileCoord c;
  c.n_tile = static_cast<int>(t - m * static_cast<uint32_t>(p.n_tiles));
  c.twi = static_cast<int>(m - r * static_cast<uint32_t>(p.tiles_w));
  c.thi = static_cast<int>(r - img * static_cast<uint32_t>(p.tiles_h));
  c.img = static_cast<int>(img);
  return c;
}

// Work item -> tile index. Without pairs they are the same. A CTA pair takes item v as the two
// consecutive pixel tiles 2m, 2m + 1 of column tile v % n_tiles (m = v / n_tiles), one per CTA; with an
// odd number of pixel tiles the last item's second tile decodes to an image index past the batch: its
// loads read zero fill and its stores are skipped.
__device__ __forceinline__ int work_first(const ConvGemmParams& p) {
  return p.pair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
}
__device__ __forceinline__ int work_tile(const ConvGemmParams& p, int v, uint32_t rank) {
  if (!p.pair) return v;
  const uint32_t m = fast_div(static_cast<uint32_t>(v), p.mul_n);
  const uint32_t nt = static_cast<uint32_t>(v) - m * static_cast<uint32_t>(p.n_tiles);
  return static_cast<int>((2u * m + rank) * static_cast<uint32_t>(p.n_tiles) + nt);
}

// Timeline probe for tuning (32 tiles of CTA 0): slot layout [tile][12]: 0 producer issue, 1 MMA got accumulator,
// 2 MMA first operands ready, 3 MMA committed, 4 epilogue saw accumulator, 5 epilogue TMEM read done,
// 6 epilogue released accumulator, 7 epilogue store issued, 8 epilogue warps met, 9 TMEM data
// arrived, 10 staging complete.
constexpr int kTraceTiles = 32;
constexpr int kTraceSlots = 12;
__device__ __forceinline__ void trace_mark(const ConvGemmParams& p, int local_tile, int slot) {
  // CTAs 0 and 1 (the two halves of the first pair) each fill their own kTraceTiles x kTraceSlots block
  if (p.trace != nullptr && blockIdx.x < 2 && local_tile < kTraceTiles)
    p.trace[(blockIdx.x * kTraceTiles + local_tile) * kTraceSlots + slot] = clock64();
}

// erf-form GELU, 0.5 x (1 + erf(x / sqrt 2)), with erf from the five-term rational-exponential fit
// 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z) (absolute error below 2e-7, far inside a 16-bit
// output's rounding). The negative side uses 1 + erf(z) = poly * exp(-z^2) directly, so the tail does not
// cancel. About a third of the instructions of erff(), which made GELU epilogues outlast their main loops.
__device__ __forceinline__ float gelu_erf_fast(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  const float t = __fdividef(1.f, fmaf(0.3275911f, z, 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float y = poly * t * __expf(-z * z);
  return 0.5f * x * (x < 0.f ? y : 2.f - y);
}

// Generic activation (runtime code); the hot ones have dedicated template paths.
__device__ __forceinline__ void apply_act8(float (&x)[8], int act, float alpha, float beta) {
  switch (act) {
    case kActRelu:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = fmaxf(x[j], 0.f);
      break;
    case kActSilu:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = __fdividef(x[j], 1.f + __expf(-x[j]));
      break;
    case kActHardSwish:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = x[j] * fminf(fmaxf(x[j] + 3.f, 0.f), 6.f) * (1.f / 6.f);
      break;
    case kActHardSigmoid:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = fminf(fmaxf(alpha * x[j] + beta, 0.f), 1.f);
      break;
    case kActSigmoid:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = __fdividef(1.f, 1.f + __expf(-x[j]));
      break;
    case kActGelu:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = gelu_erf_fast(x[j]);
      break;
    case kActRelu6:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = fminf(fmaxf(x[j], 0.f), 6.f);
      break;
    case kActLeakyRelu:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = x[j] > 0.f ? x[j] : alpha * x[j];
      break;
    case kActTanh:
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = tanhf(x[j]);
      break;
    default:
      break;
  }
}

// x * sigmoid(x) = h * tanh(h) + h with h = x/2 : one MUFU op per two elements.
__device__ __forceinline__ uint32_t silu_f16x2(uint32_t x) {
  uint32_t h, t, y;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(h) : "r"(x), "r"(0x38003800u));
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(h));
  asm("fma.rn.f16x2 %0, %1, %2, %1;" : "=r"(y) : "r"(h), "r"(t));
  return y;
}
__device__ __forceinline__ uint32_t silu_bf16x2(uint32_t x) {
  uint32_t h, t, y;
  asm("mul.bf16x2 %0, %1, %2;" : "=r"(h) : "r"(x), "r"(0x3F003F00u));
  asm("tanh.approx.bf16x2 %0, %1;" : "=r"(t) : "r"(h));
  asm("fma.rn.bf16x2 %0, %1, %2, %1;" : "=r"(y) : "r"(h), "r"(t));
  return y;
}
__device__ __forceinline__ float silu_f32(float x) {
  float h = 0.5f * x, t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, bool bf16) {
  if (bf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b, bool bf16) {
  if (bf16) {
    __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t relu2(uint32_t a, bool bf16) {
  uint32_t y;
  if (bf16) asm("max.bf16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(0u));
  else asm("max.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(0u));
  return y;
}

__device__ __forceinline__ void load8_as_float(const void* ptr, bool bf16, bool vec, int nvalid,
                                               float (&r)[8]) {
  if (vec && nvalid == 8) {
    uint4 u = *reinterpret_cast<const uint4*>(ptr);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (bf16) {
        float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
        r[2 * j] = f.x; r[2 * j + 1] = f.y;
      } else {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        r[2 * j] = f.x; r[2 * j + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < nvalid) {
        r[j] = bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ptr)[j])
                    : __half2float(reinterpret_cast<const __half*>(ptr)[j]);
      } else {
        r[j] = 0.f;
      }
    }
  }
}

// Slow, fully general store of up to 8 values (tails, misaligned rows, fp32 output).
__device__ __noinline__ void store8_general(void* ptr, int out_dtype, bool vec, int nvalid,
                                            const float* x) {
  if (out_dtype == kF32) {
    float* o = reinterpret_cast<float*>(ptr);
    if (vec && nvalid == 8) {
      reinterpret_cast<float4*>(o)[0] = make_float4(x[0], x[1], x[2], x[3]);
      reinterpret_cast<float4*>(o)[1] = make_float4(x[4], x[5], x[6], x[7]);
    } else {
      for (int j = 0; j < nvalid; ++j) o[j] = x[j];
    }
    return;
  }
  if (out_dtype == kF8E4M3) {
    if (nvalid == 8 && (reinterpret_cast<uintptr_t>(ptr) & 7) == 0) {
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * h], x[4 * h + 1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * h + 2], x[4 * h + 3]), __NV_SATFINITE, __NV_E4M3);
        w[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2*>(ptr) = make_uint2(w[0], w[1]);
    } else {
      for (int j = 0; j < nvalid; ++j)
        reinterpret_cast<uint8_t*>(ptr)[j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x[j], __NV_SATFINITE, __NV_E4M3));
    }
    return;
  }
  for (int j = 0; j < nvalid; ++j) {
    if (out_dtype == kBF16) reinterpret_cast<__nv_bfloat16*>(ptr)[j] = __float2bfloat16_rn(x[j]);
    else reinterpret_cast<__half*>(ptr)[j] = __float2half_rn(x[j]);
  }
}

// Template activation codes: the three hot ones are compiled in, the rest go
// through the runtime switch of the generic instantiation.
constexpr int kTplGeneric = -1;

// One group of 8 consecutive output channels of one output pixel.
template <int ACT>
__device__ __forceinline__ void epilogue8(const uint32_t* v, const ConvGemmParams& p, int co,
                                          int col_limit, uint8_t* yrow, const uint8_t* rrow,
                                          bool in_bf16, int out_es, uint32_t stage_addr = 0,
                                          const float* bias_s = nullptr, bool has_pre = false,
                                          uint4 res_pre = make_uint4(0, 0, 0, 0), float row_scale = 1.f) {
  const int nvalid = min(8, col_limit - co);
  if (nvalid <= 0) return;
  float x[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[j]);
  if (p.fp8) {   // dequantise: accumulator * scale of the row * scale of the column
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sb = (p.scale_b != nullptr && j < nvalid) ? __ldg(p.scale_b + co + j) : 1.f;
      x[j] *= row_scale * sb;
    }
  }
  if (bias_s != nullptr) {   // shared-memory copy (zeros where there is no bias), padded to the tile width
    const float4 b0 = *reinterpret_cast<const float4*>(bias_s);
    const float4 b1 = *reinterpret_cast<const float4*>(bias_s + 4);
    x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w;
    x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
  } else if (p.bias != nullptr) {
    if (nvalid == 8) {
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + co));
      const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + co) + 1);
      x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w;
      x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < nvalid) x[j] += __ldg(p.bias + co + j);
      }
    }
  }
  // staged rows go out through a TMA store that clips channel tails, so tails may take this path too
  const bool fast16 = (p.out_dtype == kF16 || p.out_dtype == kBF16) && (stage_addr != 0 || (p.y_vec != 0 && nvalid == 8));
  if (fast16) {
    const bool out_bf16 = p.out_dtype == kBF16;
    uint32_t w[4];
    uint4 rv = make_uint4(0, 0, 0, 0);
    const bool res_fast = p.res_mode != 0 && p.res_vec != 0 && in_bf16 == out_bf16 && nvalid == 8;
    if (p.res_mode != 0) {
      if (res_fast && p.res_mode == 2) {
        rv = has_pre ? res_pre : *reinterpret_cast<const uint4*>(rrow + co * 2);
      } else {
        float r[8];
        load8_as_float(rrow + co * 2, in_bf16, p.res_vec != 0, nvalid, r);
        if (p.res_mode == 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] += r[j];
        } else {
          // after-activation add with mismatching dtypes: stash as packed output type
          rv = make_uint4(pack2(r[0], r[1], out_bf16), pack2(r[2], r[3], out_bf16),
                          pack2(r[4], r[5], out_bf16), pack2(r[6], r[7], out_bf16));
        }
      }
    }
    if (ACT == kTplGeneric) apply_act8(x, p.act, p.act_alpha, p.act_beta);
    if (ACT == kActGelu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = gelu_erf_fast(x[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t h = pack2(x[2 * j], x[2 * j + 1], out_bf16);
      if (ACT == kActSilu) h = out_bf16 ? silu_bf16x2(h) : silu_f16x2(h);
      if (ACT == kActRelu) h = relu2(h, out_bf16);
      w[j] = h;
    }
    if (p.res_mode == 2) {
      w[0] = add2(w[0], rv.x, out_bf16); w[1] = add2(w[1], rv.y, out_bf16);
      w[2] = add2(w[2], rv.z, out_bf16); w[3] = add2(w[3], rv.w, out_bf16);
    }
    if (stage_addr != 0) {
      // no memory clobber: the next group's loads may move above this store; volatile keeps it
      // ordered against the barriers
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_addr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                   "r"(w[3]));
    } else {
      *reinterpret_cast<uint4*>(yrow + static_cast<size_t>(co) * 2) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return;
  }
  // general path: fp32 output, channel tails, unaligned rows
  float r[8];
  if (p.res_mode != 0) load8_as_float(rrow + co * 2, in_bf16, p.res_vec != 0, nvalid, r);
  if (p.res_mode == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += r[j];
  }
  if (ACT == kTplGeneric) apply_act8(x, p.act, p.act_alpha, p.act_beta);
  if (ACT == kActGelu) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = gelu_erf_fast(x[j]);
  }
  if (ACT == kActSilu) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = silu_f32(x[j]);
  }
  if (ACT == kActRelu) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = fmaxf(x[j], 0.f);
  }
  if (p.res_mode == 2) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += r[j];
  }
  // The out-of-line store takes an address, which would pin its argument in local memory for the
  // whole function, fast paths included: hand it a copy so that x itself stays in registers.
  float xs[8];
  const float os = p.out_dtype == kF8E4M3 ? p.out_scale : 1.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) xs[j] = x[j] * os;
  store8_general(yrow + static_cast<size_t>(co) * out_es, p.out_dtype, p.y_vec != 0, nvalid, xs);
}

// Straight-line epilogue of one 32-column chunk into the staging row: bias from shared memory,
// activation, optional after-activation residual already in registers, four 16-byte stores. All
// data-type and residual decisions are template parameters: with two or three warps per scheduler
// nothing hides branch latency, and a dozen uniform branches per 8 columns used to cost more than
// the arithmetic. Columns past Cout carry padding that the TMA store clips.
// bias (+ dequantisation scale) of one group of eight columns
template <bool SCALE>
__device__ __forceinline__ void chunk_affine(const uint32_t* v8, const float* bias8, const float* scale8, float (&x)[8]) {
  const float4 b0 = *reinterpret_cast<const float4*>(bias8);
  const float4 b1 = *reinterpret_cast<const float4*>(bias8 + 4);
  if (SCALE) {   // fp8 operands: accumulator * (activation scale * weight scale of the column) + bias
    const float4 s0 = *reinterpret_cast<const float4*>(scale8);
    const float4 s1 = *reinterpret_cast<const float4*>(scale8 + 4);
    x[0] = fmaf(__uint_as_float(v8[0]), s0.x, b0.x); x[1] = fmaf(__uint_as_float(v8[1]), s0.y, b0.y);
    x[2] = fmaf(__uint_as_float(v8[2]), s0.z, b0.z); x[3] = fmaf(__uint_as_float(v8[3]), s0.w, b0.w);
    x[4] = fmaf(__uint_as_float(v8[4]), s1.x, b1.x); x[5] = fmaf(__uint_as_float(v8[5]), s1.y, b1.y);
    x[6] = fmaf(__uint_as_float(v8[6]), s1.z, b1.z); x[7] = fmaf(__uint_as_float(v8[7]), s1.w, b1.w);
  } else {
    x[0] = __uint_as_float(v8[0]) + b0.x; x[1] = __uint_as_float(v8[1]) + b0.y;
    x[2] = __uint_as_float(v8[2]) + b0.z; x[3] = __uint_as_float(v8[3]) + b0.w;
    x[4] = __uint_as_float(v8[4]) + b1.x; x[5] = __uint_as_float(v8[5]) + b1.y;
    x[6] = __uint_as_float(v8[6]) + b1.z; x[7] = __uint_as_float(v8[7]) + b1.w;
  }
}

// e4m3 output: one 32-column chunk becomes 32 bytes of the staging row (32-byte rows, 32-byte swizzle).
template <int ACT, bool SCALE>
__device__ __forceinline__ void staged_chunk_e4m3(const uint32_t (&v)[32], const float* bias_s, const float* scale_s,
                                                  uint32_t srow, uint32_t row_sw1, const ConvGemmParams& p) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t w[4];
#pragma unroll
    for (int gg = 0; gg < 2; ++gg) {
      const int g = 2 * h + gg;
      float x[8];
      chunk_affine<SCALE>(v + g * 8, bias_s + g * 8, scale_s + g * 8, x);
      if (ACT == kTplGeneric) apply_act8(x, p.act, p.act_alpha, p.act_beta);
      if (ACT == kActGelu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = gelu_erf_fast(x[j]);
      }
      if (ACT == kActSilu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = silu_f32(x[j]);
      }
      if (ACT == kActRelu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = fmaxf(x[j], 0.f);
      }
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * q2] * p.out_scale, x[4 * q2 + 1] * p.out_scale),
                                                     __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * q2 + 2] * p.out_scale, x[4 * q2 + 3] * p.out_scale),
                                                     __NV_SATFINITE, __NV_E4M3);
        w[2 * gg + q2] = lo | (hi << 16);
      }
    }
    const uint32_t addr = srow + ((static_cast<uint32_t>(h) ^ row_sw1) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]));
  }
}

template <int ACT, bool BF16, bool RES, bool SCALE>
__device__ __forceinline__ void staged_chunk(const uint32_t (&v)[32], const float* bias_s, const float* scale_s,
                                             const uint4 (&rpre)[4], uint32_t srow, uint32_t row_sw,
                                             const ConvGemmParams& p) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float x[8];
    chunk_affine<SCALE>(v + g * 8, bias_s + g * 8, scale_s + g * 8, x);
    if (ACT == kTplGeneric) apply_act8(x, p.act, p.act_alpha, p.act_beta);
    if (ACT == kActGelu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = gelu_erf_fast(x[j]);
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t h = pack2(x[2 * j], x[2 * j + 1], BF16);
      if (ACT == kActSilu) h = BF16 ? silu_bf16x2(h) : silu_f16x2(h);
      if (ACT == kActRelu) h = relu2(h, BF16);
      w[j] = h;
    }
    if (RES) {
      w[0] = add2(w[0], rpre[g].x, BF16); w[1] = add2(w[1], rpre[g].y, BF16);
      w[2] = add2(w[2], rpre[g].z, BF16); w[3] = add2(w[3], rpre[g].w, BF16);
    }
    const uint32_t addr = srow + ((static_cast<uint32_t>(g) ^ row_sw) << 4);   // 64-byte rows, 64-byte swizzle
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]));
  }
}

// Epilogue role shared by the convolution kernels: drains the double-buffered TMEM
// accumulators tile by tile. `tfull0` / `tempty0` are the shared-memory addresses of
// tmem_full[0] and tmem_empty[0]; index 1 of each follows 8 bytes later.
constexpr int kTeamWarps = 4;                         // warps of one half of the epilogue
constexpr int kChunkCols = 32;                        // output columns per staged chunk (one tcgen05.ld)
constexpr int kChunkBytes = kBM * kChunkCols * 2;     // 128 rows x 32 channels (16-bit) = 8 KB
constexpr int kStagingBytes = 4 * kChunkBytes;        // two chunk buffers for each half of the epilogue warps

// Output path for 16-bit results, in two forms chosen per layer. Wide column tiles (more than 64
// columns): all eight epilogue warps drain ONE tile together, so an accumulator goes back to the MMA
// issuer after half the time a four-warp team would hold it (the accumulator cycle - MMA, then drain - is
// what bounds such layers); warps w and w + 4 read the same TMEM lane quarter and take alternate
// 32-column chunks. Narrow tiles (p.epi_teams): one or two chunks cannot be split usefully, so the two
// halves drain alternate tiles, each half its own accumulator. Each thread owns one accumulator row. A chunk
// is assembled in one of the half's two staging buffers (64-byte rows, 64-byte swizzle) and handed to a
// TMA tensor store by the half's leader, which writes whole lines and clips ragged tile edges and channel
// tails; with two buffers the next chunk is staged while the previous store still reads shared memory.
// Named barrier 1 + half (128 threads) keeps a half in step.
template <int BN, int ACT>
__device__ __forceinline__ void epilogue_loop_tma(const ConvGemmParams& p, const CUtensorMap* tmY, uint32_t stage0,
                                                  uint32_t tmem_base, uint32_t tfull0, uint32_t tempty0,
                                                  volatile int* abort_flag, float* s_bias, int warp, int lane) {
  const int q = warp & 3;                       // TMEM lane quarter this warp may read
  const int half = (warp - 2) >> 2;
  const bool leader_warp = ((warp - 2) & 3) == 0;
  const bool issuer = leader_warp && lane == 0;
  const bool in_bf16 = p.in_bf16 != 0;
  const int tt = static_cast<int>(threadIdx.x) - 64 - half * 128;   // index within the half
  const int row = q * 32 + lane;
  const int rh = row / p.tw, rw = row - rh * p.tw;
  const bool out_bf16 = p.out_dtype == kBF16;
  // after-activation residual rows can be fetched while the accumulator is still being produced
  const bool res_pre = p.res_mode == 2 && p.res_vec != 0 && in_bf16 == out_bf16;
  // fp8 operands with a per-column scale only (static activation scale folded in) ride the straight-line path too
  const bool col_scale = p.fp8 != 0 && p.scale_a == nullptr && p.scale_b != nullptr;
  const bool simple = (p.res_mode == 0 || res_pre) && (!p.fp8 || col_scale);   // else: general per-group path
  const bool out8 = p.out_dtype == kF8E4M3;
  const int row_bytes = out8 ? 32 : 64;                       // staging row of one chunk
  const uint32_t row_sw1 = static_cast<uint32_t>((row >> 2) & 1);
  const uint32_t buf0 = stage0 + half * (2 * kChunkBytes);
  const uint32_t row_sw = static_cast<uint32_t>((row >> 1) & 3);
  volatile int* abort_sample = abort_flag + 1 + half;
  bool aborted = false;
  uint32_t par = 0;                             // staging buffer of this half's next chunk
  float* bias_s = s_bias + half * 256;          // each half keeps the bias slice of the current column tile
  float* scale_s = s_bias + 512 + half * 256;   // ... and, for fp8 operands, the dequantisation scale slice
  if (p.n_tiles == 1) {
    for (int i = tt; i < BN; i += 128) {
      bias_s[i] = (p.bias != nullptr && i < p.Cout) ? __ldg(p.bias + i) : 0.f;
      scale_s[i] = (col_scale && i < p.Cout) ? __ldg(p.scale_b + i) : 1.f;
    }
    asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
  }
  unsigned int* pending_counter = nullptr;   // issuer only: stores of the previous tile not yet signalled
  unsigned pending_stores = 0;
  auto flush_signal = [&]() {
    if (pending_counter != nullptr) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(pending_counter), "r"(pending_stores) : "memory");
      pending_counter = nullptr;
      pending_stores = 0;
    }
  };
  const uint32_t pair_rank = p.pair ? cluster_ctarank() : 0u;
  const bool teams = p.epi_teams != 0;
  const int c_first = teams ? 0 : half, c_step = teams ? 1 : 2;
  for (int it = teams ? half : 0; !aborted; it += teams ? 2 : 1) {
    const long long tile_ll = static_cast<long long>(work_first(p)) + static_cast<long long>(it) * p.gemm_ctas;
    if (tile_ll >= p.total_tiles) break;
    if (issuer) flush_signal();
    const int acc = it & 1;
    const uint32_t acc_ph = static_cast<uint32_t>(it >> 1) & 1u;
    const uint32_t tfull = tfull0 + 8u * acc, tempty = tempty0 + 8u * acc;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
    const int tile = work_tile(p, static_cast<int>(tile_ll), pair_rank);
    const TileCoord tc = decode_tile(p, tile);
    const int n_tile = tc.n_tile, thi = tc.thi, img = tc.img;
    int twi = tc.twi;
    if (p.peer_mode == 1) {   // same rotation as the producer: local rows first
      twi += p.peer_rot;
      if (twi >= p.tiles_w) twi -= p.tiles_w;
    }
    const int oh = thi * p.th + rh, ow = twi * p.tw + rw;
    const bool real_tile = img < p.n_images;
    const bool valid = rh < p.th && oh < p.Ho && ow < p.Wo && real_tile;
    const uint8_t* rrow = reinterpret_cast<const uint8_t*>(p.residual) +
                          (static_cast<size_t>(img) * p.res_n_stride + static_cast<size_t>(oh) * p.res_h_stride +
                           static_cast<size_t>(ow) * p.res_ld) * 2;
    const int colbase = n_tile * BN;
    const int col_limit = min(p.Cout, colbase + BN);
    const int nchunks = (col_limit - colbase + kChunkCols - 1) / kChunkCols;
    const float row_scale = (p.fp8 && p.scale_a != nullptr && valid)
                                ? __ldg(p.scale_a + (static_cast<long long>(img) * p.Ho + oh) * p.Wo + ow) : 1.f;
    if (p.n_tiles > 1) {
      // the previous tile's chunks of this half were all staged before its last barrier, so the slice is free
      for (int i = tt; i < BN; i += 128) {
        bias_s[i] = (p.bias != nullptr && colbase + i < p.Cout) ? __ldg(p.bias + colbase + i) : 0.f;
        scale_s[i] = (col_scale && colbase + i < p.Cout) ? __ldg(p.scale_b + colbase + i) : 1.f;
      }
    }
    // The leader warp waits for the accumulator; the other warps sleep at the named barrier, which wakes
    // them faster than separate polls would. Every half waits here, also one without a chunk in this tile:
    // it may only hand the accumulator back once the tile exists, or its arrivals would run ahead into the
    // accumulator's next phase.
    if (leader_warp) {
      mbar_wait(tfull, acc_ph, abort_flag, kStatusTimeoutEpilogue);
      if (issuer) trace_mark(p, it, 4);
      if (lane == 0) *abort_sample = *abort_flag;
    }
    asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
    if (*abort_sample != 0) { aborted = true; break; }
    tc_fence_after();
    for (int c = c_first; c < nchunks; c += c_step) {
      const int co0 = colbase + c * kChunkCols;
      uint4 rpre[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) rpre[g] = make_uint4(0, 0, 0, 0);
      if (res_pre && valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          // a ragged last group still reads 16 bytes: the row pitch is a multiple of 8 elements and
          // columns past Cout are clipped by the store
          if (co0 + g * 8 < col_limit) rpre[g] = *reinterpret_cast<const uint4*>(rrow + (co0 + g * 8) * 2);
        }
      }
      uint32_t v[32];
      tmem_ld_32x32(t_row + c * kChunkCols, v);
      tmem_ld_wait_dep(v);
      const bool last = c + c_step >= nchunks;
      if (issuer && last) trace_mark(p, it, 9);
      if (last) {        // this half's last TMEM read of the accumulator
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (pair_rank != 0) mbar_arrive_remote(tempty, 0);   // the MMA issuer lives in the even CTA
          else mbar_arrive(tempty);
        }
        if (issuer) trace_mark(p, it, 6);
      }
      // buffer `par` is free: the store that last read it was waited for before the previous chunk's barrier
      const uint32_t buf = buf0 + par * kChunkBytes;
      const uint32_t srow = buf + row * row_bytes;
      if (valid) {
        const float* bs = bias_s + c * kChunkCols;
        const float* ss = scale_s + c * kChunkCols;
        if (out8) {          // host side: only planned with simple == true and no residual
          if (col_scale) staged_chunk_e4m3<ACT, true>(v, bs, ss, srow, row_sw1, p);
          else staged_chunk_e4m3<ACT, false>(v, bs, ss, srow, row_sw1, p);
        } else if (simple && col_scale) {
          if (out_bf16) staged_chunk<ACT, true, false, true>(v, bs, ss, rpre, srow, row_sw, p);
          else staged_chunk<ACT, false, false, true>(v, bs, ss, rpre, srow, row_sw, p);
        } else if (simple) {
          if (out_bf16) {
            if (res_pre) staged_chunk<ACT, true, true, false>(v, bs, ss, rpre, srow, row_sw, p);
            else staged_chunk<ACT, true, false, false>(v, bs, ss, rpre, srow, row_sw, p);
          } else {
            if (res_pre) staged_chunk<ACT, false, true, false>(v, bs, ss, rpre, srow, row_sw, p);
            else staged_chunk<ACT, false, false, false>(v, bs, ss, rpre, srow, row_sw, p);
          }
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            epilogue8<ACT>(v + g * 8, p, co0 + g * 8, col_limit, nullptr, rrow, in_bf16, 2,
                           srow + ((static_cast<uint32_t>(g) ^ row_sw) << 4), bs + g * 8, false, make_uint4(0, 0, 0, 0), row_scale);
          }
        }
      }
      if (issuer && last) trace_mark(p, it, 5);
      fence_proxy_async_smem();
      // One barrier per chunk: behind it the chunk is complete in shared memory, and - because the issuer
      // first waits for every earlier store to have read its buffer - the other buffer is free for the
      // next chunk.
      if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
      if (issuer && real_tile) {
        if (last) trace_mark(p, it, 10);
        if (p.peer_mode == 2) {
          // reduce-scatter: the chunk goes to the rank that owns these rows, into this rank's slot
          const int grow = twi * p.tw;
          const int owner = grow / p.peer_rows;
          const int local = grow - owner * p.peer_rows;
          asm volatile(
              "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                  reinterpret_cast<uint64_t>(&p.peer->maps[owner])),
              "r"(buf), "r"(co0), "r"(p.peer_rank * p.peer_rows + local), "r"(0), "r"(0)
              : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          // The signal may only follow the data, and waiting for a remote store to complete takes
          // microseconds: the wait is deferred to the start of the next tile (or the end of the kernel),
          // where it overlaps the tensor-core work of the tiles in between.
          pending_counter = p.peer->counters[owner] + local / kBM;
          ++pending_stores;
        } else {
          asm volatile(
              "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                  reinterpret_cast<uint64_t>(tmY)),
              "r"(buf), "r"(co0), "r"(twi * p.tw), "r"(thi * p.th), "r"(img)
              : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          if (p.peer_mode == 3) {
            // pull form of the reduce-scatter: the partial block stays in this rank's memory; only the arrival
            // count goes to the rank that owns the rows, which then reads the block over NVLink itself
            const int grow = twi * p.tw;
            const int owner = grow / p.peer_rows;
            pending_counter = p.peer->counters[owner] + (grow - owner * p.peer_rows) / kBM;
            ++pending_stores;
          }
        }
        if (last) trace_mark(p, it, 7);
      }
      par ^= 1;
    }
    if (!teams && half >= nchunks) {   // nothing to drain in this tile: hand the accumulator back at once
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (pair_rank != 0) mbar_arrive_remote(tempty, 0);
        else mbar_arrive(tempty);
      }
    }
  }
  if (issuer) {
    flush_signal();
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
}

template <int BN, int ACT>
__device__ __forceinline__ void epilogue_loop(const ConvGemmParams& p, uint32_t tmem_base, uint32_t tfull0,
                                              uint32_t tempty0, volatile int* abort_flag, int warp, int lane) {
  auto tfull_bar = [&](int a) { return tfull0 + 8u * a; };
  auto tempty_bar = [&](int a) { return tempty0 + 8u * a; };
  // Two warps share each TMEM lane quarter and split the tile's columns.
  const int q = warp & 3;
  const int half = (warp - 2) >> 2;
  constexpr int kChunks = (BN + 31) / 32;
  constexpr int kChunksHalf0 = (kChunks + 1) / 2;
  const int c_begin = half == 0 ? 0 : kChunksHalf0;
  const int c_end = half == 0 ? kChunksHalf0 : kChunks;
  const bool in_bf16 = p.in_bf16 != 0;
  const int out_es = p.out_dtype == kF32 ? 4 : (p.out_dtype == kF8E4M3 ? 1 : 2);
  int acc = 0;
  uint32_t acc_ph = 0;
  const uint32_t pair_rank = p.pair ? cluster_ctarank() : 0u;
  for (int v = work_first(p); v < p.total_tiles; v += p.gemm_ctas) {
    const int tile = work_tile(p, v, pair_rank);
    const TileCoord tc = decode_tile(p, tile);
    const int n_tile = tc.n_tile, thi = tc.thi, img = tc.img;
    int twi = tc.twi;
    if (p.peer_mode == 1) {   // same rotation as the producer: local rows first
      twi += p.peer_rot;
      if (twi >= p.tiles_w) twi -= p.tiles_w;
    }
    if (!mbar_wait(tfull_bar(acc), acc_ph, abort_flag, kStatusTimeoutEpilogue)) break;
    tc_fence_after();
    const int row = q * 32 + lane;
    const int rh = row / p.tw, rw = row - rh * p.tw;
    const int oh = thi * p.th + rh, ow = twi * p.tw + rw;
    const bool valid = rh < p.th && oh < p.Ho && ow < p.Wo && img < p.n_images;
    uint8_t* yrow = reinterpret_cast<uint8_t*>(p.y) +
                    (static_cast<size_t>(img) * p.y_n_stride + static_cast<size_t>(oh) * p.y_h_stride +
                     static_cast<size_t>(ow) * p.y_ld) * out_es;
    const uint8_t* rrow = reinterpret_cast<const uint8_t*>(p.residual) +
                          (static_cast<size_t>(img) * p.res_n_stride + static_cast<size_t>(oh) * p.res_h_stride +
                           static_cast<size_t>(ow) * p.res_ld) * 2;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
    const int colbase = n_tile * BN;
    const int col_limit = min(p.Cout, colbase + BN);
    const float row_scale = (p.fp8 && p.scale_a != nullptr && valid)
                                ? __ldg(p.scale_a + (static_cast<long long>(img) * p.Ho + oh) * p.Wo + ow) : 1.f;
    uint32_t va[32], vb[32];
    int c = c_begin;
    bool have = c < c_end && colbase + c * 32 < col_limit;
    if (have) tmem_ld_32x32(t_row + c * 32, va);
    while (have) {
      tmem_ld_wait_dep(va);
      bool next = (c + 1 < c_end) && (colbase + (c + 1) * 32 < col_limit);
      if (next) tmem_ld_32x32(t_row + (c + 1) * 32, vb);
      if (valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
          epilogue8<ACT>(va + g * 8, p, colbase + c * 32 + g * 8, col_limit, yrow, rrow, in_bf16, out_es, 0, nullptr, false,
                         make_uint4(0, 0, 0, 0), row_scale);
      }
      if (!next) break;
      ++c;
      tmem_ld_wait_dep(vb);
      next = (c + 1 < c_end) && (colbase + (c + 1) * 32 < col_limit);
      if (next) tmem_ld_32x32(t_row + (c + 1) * 32, va);
      if (valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
          epilogue8<ACT>(vb + g * 8, p, colbase + c * 32 + g * 8, col_limit, yrow, rrow, in_bf16, out_es, 0, nullptr, false,
                         make_uint4(0, 0, 0, 0), row_scale);
      }
      ++c;
      have = next;
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (pair_rank != 0) mbar_arrive_remote(tempty_bar(acc), 0);
      else mbar_arrive(tempty_bar(acc));
    }
    acc ^= 1;
    if (acc == 0) acc_ph ^= 1;
  }
}

constexpr int kMaxSmem = 232448 - 5120;  // 227 KB opt-in limit per CTA less the static shared memory
constexpr int kBiasFloats = 1024;     // shared memory: per epilogue half a bias slice and a column-scale slice of up to 256 columns
constexpr int kBarBytes = 256;

constexpr int next_pow2_cols(int c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : c <= 256 ? 256 : 512; }

template <int BN, bool PAIR = false>
struct KernelCfg {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N must be a multiple of 16 up to 256");
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;      // weight rows staged by this CTA
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagesFit = (kMaxSmem - kBarBytes - 1024 - kStagingBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kTmemCols = next_pow2_cols(2 * BN);
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarBytes + 1024;  // +1024: alignment slack
};

template <int BN, int ACT, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
conv_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmY, const ConvGemmParams p) {
  using Cfg = KernelCfg<BN, PAIR>;
  const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(16) float s_bias[kBiasFloats];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes + kStagingBytes);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * S + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 + a); };
  const uint32_t tile0 = smem_u32(smem);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      // a pair's accumulator is handed back by the epilogue warps of both CTAs
      mbar_init(tempty_bar(a), ((p.y_tma && p.epi_teams) ? kTeamWarps : kEpiWarps) * (PAIR ? 2 : 1));
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int first_copier = PAIR ? 2 * p.gemm_ctas : p.gemm_ctas;   // GEMM CTAs come first, in pairs when PAIR
  if (static_cast<int>(blockIdx.x) >= first_copier) {
    // ------------------------------------------------------------ copier CTA (all-gather -> GEMM)
    // Pulls the remote shards of A over NVLink into this rank's gathered buffer, one 128-row block
    // at a time in the order the GEMM CTAs will want them, and publishes a flag per block. Each
    // remote row crosses NVLink exactly once however many column tiles later read it from HBM / L2.
    const int copiers = static_cast<int>(gridDim.x) - first_copier;
    const int c = static_cast<int>(blockIdx.x) - first_copier;
    const int per_shard = p.peer_rows / p.tw;
    // One thread drives a ring of bulk copies: peer memory -> shared memory -> this rank's buffer, 16 KB per
    // stage. The copy engine keeps every stage in flight at once (a CTA holds well over 100 KB in transit, which
    // is what it takes to fill an NVLink round trip), where ordinary loads are limited by the registers that can
    // wait for them.
    if (threadIdx.x == 0) {
      constexpr int kCopyStage = 16384;
      constexpr int kLag = 2;          // a stage is refilled this many chunks after its store was issued
      const int ring_max = (S * Cfg::kStageBytes + kStagingBytes) / kCopyStage;
      const int NS = min(min(2 * S, ring_max), 12);       // the operand ring's 2 * S mbarriers serve as stage barriers
      const long long blk_bytes = static_cast<long long>(p.tw) * p.gather_row_bytes;
      const int n_chunks = static_cast<int>((blk_bytes + kCopyStage - 1) / kCopyStage);
      uint32_t phase_bits = 0;         // parity per stage
      bool ok = true;
      for (int j = per_shard + c; ok && j < p.tiles_w; j += copiers) {      // rotated order, remote blocks only
        int b = j + p.peer_rot;
        if (b >= p.tiles_w) b -= p.tiles_w;
        const int owner = b / per_shard;
        const long long off = static_cast<long long>(b) * p.tw * p.gather_row_bytes;
        const uint8_t* from = p.peer_src[owner] + off;
        uint8_t* to = p.gather_dst + off;
        auto chunk_bytes = [&](int i) {
          return static_cast<uint32_t>(min(static_cast<long long>(kCopyStage), blk_bytes - static_cast<long long>(i) * kCopyStage));
        };
        auto issue_load = [&](int i) {
          const int st = i % NS;
          const uint32_t bar = bar0 + 8u * st;
          mbar_arrive_expect_tx(bar, chunk_bytes(i));
          bulk_load(tile0 + st * kCopyStage, from + static_cast<long long>(i) * kCopyStage, chunk_bytes(i), bar);
        };
        const int ahead = NS - kLag;
        for (int i = 0; i < min(ahead, n_chunks); ++i) issue_load(i);
        for (int i = 0; i < n_chunks; ++i) {
          const int st = i % NS;
          if (!mbar_wait(bar0 + 8u * st, (phase_bits >> st) & 1u, abort_flag, kStatusTimeoutPeer)) { ok = false; break; }
          phase_bits ^= 1u << st;
          bulk_store(to + static_cast<long long>(i) * kCopyStage, tile0 + st * kCopyStage, chunk_bytes(i));
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          if (i + ahead < n_chunks) {
            // the stage of chunk i + ahead last held chunk i - kLag: all but the newest kLag stores have read theirs
            asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kLag) : "memory");
            issue_load(i + ahead);
          }
        }
        // every byte of the block is in this rank's memory before the flag says so
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (!ok) {
          // aborting: give the loads still in flight a bounded chance to land before this CTA's shared memory
          // is handed on
          for (int st = 0; st < NS; ++st)
            for (int spin = 0; spin < (1 << 14); ++spin)
              if (mbar_try_wait(bar0 + 8u * st, (phase_bits >> st) & 1u)) break;
          break;
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        st_release_gpu(p.ready + b, p.peer_epoch);
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint32_t armed = 0, armed_parity = 0;
      bool ok = true;
      int item = 0;
      for (int v = work_first(p); ok && v < p.total_tiles; v += p.gemm_ctas, ++item) {
        const int tile = work_tile(p, v, pair_rank);
        const TileCoord tc = decode_tile(p, tile);
        const int n_tile = tc.n_tile, thi = tc.thi, img = tc.img;
        int twi = tc.twi;
        if (p.peer_mode == 1) {
          // local rows first, then the shards in the order the copier CTAs bring them in
          twi += p.peer_rot;
          if (twi >= p.tiles_w) twi -= p.tiles_w;
          const int owner = (twi * p.tw) / p.peer_rows;
          if (owner != p.peer_rank) {
            const long long t0 = clock64();
            while (static_cast<int>(ld_acquire_gpu(p.ready + twi) - p.peer_epoch) < 0) {
              // an error already recorded by an earlier kernel of this forward ends the wait at once
              const bool dead = p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0;
              if (*abort_flag || dead || clock64() - t0 > kWaitClockLimit) {
                *abort_flag = kStatusTimeoutPeer;
                ok = false;
                break;
              }
            }
            if (!ok) break;
            // acquire (generic proxy) -> TMA reads of the gathered rows (async proxy)
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        const int x0 = twi * p.tw * p.stride - p.pad_w;
        const int y0 = thi * p.th * p.stride - p.pad_h;
        trace_mark(p, item, 0);
        int kcol = 0;
        for (int kh = 0; ok && kh < p.KH; ++kh) {
          for (int kw = 0; ok && kw < p.KW; ++kw) {
            for (int kb = 0; kb < p.kb_per_tap; ++kb, kcol += p.kblk) {
              if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, kStatusTimeoutProducer)) {
                ok = false;
                break;
              }
              const uint32_t a_dst = tile0 + s * Cfg::kStageBytes;
              if (PAIR) {
                // Both CTAs' bytes complete on the even CTA's barrier, which alone is armed (for both).
                if (pair_rank == 0) {
                  mbar_arrive_expect_tx(full_bar(s), 2u * (p.a_bytes + Cfg::kBBytes));
                  armed |= 1u << s;
                  armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                }
                tma_load_4d_pair(a_dst, &tmA, full_bar(s), kb * p.kblk, x0 + kw, y0 + kh, img);
                tma_load_2d_pair(a_dst + Cfg::kABytes, &tmB, full_bar(s), kcol,
                                 n_tile * BN + static_cast<int>(pair_rank) * Cfg::kBRows);
              } else {
                mbar_arrive_expect_tx(full_bar(s), p.a_bytes + Cfg::kBBytes);
                armed |= 1u << s;
                armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
                tma_load_4d(a_dst, &tmA, full_bar(s), kb * p.kblk, x0 + kw, y0 + kh, img);
                if (p.b_batched)   // 1: one matrix per (image row, image); 2: one matrix per image
                  tma_load_4d(a_dst + Cfg::kABytes, &tmB, full_bar(s), kcol, n_tile * BN, p.b_batched == 2 ? 0 : thi * p.th, img);
                else
                  tma_load_2d(a_dst + Cfg::kABytes, &tmB, full_bar(s), kcol, n_tile * BN);
              }
              if (++s == S) { s = 0; ph ^= 1; }
            }
          }
        }
      }
      if (!ok) {
        // Aborting: give the copies already issued a bounded chance to land
        // before the CTA exits and its shared memory is handed to another CTA.
        for (int i = 0; i < S; ++i) {
          if (!(armed & (1u << i))) continue;
          const uint32_t par = (armed_parity >> i) & 1u;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(full_bar(i), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // One elected thread runs the whole loop. tcgen05.mma issue is nearly synchronous for narrow
    // tiles (the thread cannot run far ahead of the tensor pipe), so every vote, fence or poll
    // between two MMAs adds its full latency to the tile: the loop holds nothing but the waits that
    // are needed. No tcgen05 fence follows them: operands arrive through the async proxy (TMA
    // complete_tx), and an accumulator is only handed back after the epilogue's tcgen05.wait::ld,
    // so its reads have finished before the arrive that this thread observes.
    if (pair_rank == 0 && elect_one()) {   // in a pair only the even CTA issues; its MMAs drive both tensor cores
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      const uint64_t desc_hi = make_kmajor_desc(0, 128);
      int it = 0;
      for (int v = work_first(p); ok && v < p.total_tiles; v += p.gemm_ctas, ++it) {
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, kStatusTimeoutMma)) break;
        trace_mark(p, it, 1);
        const uint32_t d_tmem = tmem_base + acc * BN;
        int kb = 0;
        for (int k = 0; k < p.k_iters; ++k) {
          const uint32_t ksteps = kb == p.kb_per_tap - 1 ? static_cast<uint32_t>(p.last_ksteps) : 4u;
          if (++kb == p.kb_per_tap) kb = 0;
          if (!mbar_wait(full_bar(s), ph, abort_flag, kStatusTimeoutMma)) {
            ok = false;
            break;
          }
          if (k == 0) trace_mark(p, it, 2);
          const uint32_t a_addr = tile0 + s * Cfg::kStageBytes;
          const uint64_t adesc = desc_hi | ((a_addr & 0x3FFFF) >> 4);
          const uint64_t bdesc = desc_hi | (((a_addr + Cfg::kABytes) & 0x3FFFF) >> 4);
          if (PAIR) {
            if (p.fp8) umma_f8_ksteps_pair(d_tmem, adesc, bdesc, p.idesc, k != 0 ? 1u : 0u, ksteps);
            else umma_f16_ksteps_pair(d_tmem, adesc, bdesc, p.idesc, k != 0 ? 1u : 0u, ksteps);
            umma_commit_pair(empty_bar(s));      // frees the stage in both CTAs
          } else {
            if (p.fp8) umma_f8_ksteps(d_tmem, adesc, bdesc, p.idesc, k != 0 ? 1u : 0u, ksteps);
            else umma_f16_ksteps(d_tmem, adesc, bdesc, p.idesc, k != 0 ? 1u : 0u, ksteps);
            umma_commit(empty_bar(s));
          }
          if (++s == S) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        if (PAIR) umma_commit_pair(tfull_bar(acc));
        else umma_commit(tfull_bar(acc));
        trace_mark(p, it, 3);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
    __syncwarp();
  } else if (p.y_tma) {
    epilogue_loop_tma<BN, ACT>(p, &tmY, tile0 + S * Cfg::kStageBytes, tmem_base, tfull_bar(0), tempty_bar(0),
                               abort_flag, s_bias, warp, lane);
  } else {
    epilogue_loop<BN, ACT>(p, tmem_base, tfull_bar(0), tempty_bar(0), abort_flag, warp, lane);
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  // A pair leaves together: the even CTA's MMAs read the odd CTA's shared memory and signal its barriers
  // until the last tile has been drained on both sides.
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, *abort_flag);
}


// ------------------------------------------------------------------ 3x3 stride-1 "halo" variant
// The generic kernel re-fetches the activation tile once per filter tap (9x for a 3x3
// filter), which makes small-channel layers L2-bound. Here an output tile is 8 pixels wide and
// 16 high; per 64-channel slab ONE (16+2) x (8+2) halo patch is loaded and all 9 taps read it
// through shifted shared-memory descriptors: tap (kh, kw) starts (kh*10 + kw) pixel rows into
// the patch and consecutive 8-row groups are 10 pixel rows (1280 bytes) apart, so the 8 pixels
// of an output row stay one contiguous swizzled group. Weights stream through their own ring;
// when the whole filter fits (`b_resident`) it is loaded once per CTA and kept.
constexpr int kHaloTw = 8, kHaloTh = 16;
constexpr int kHaloCols = kHaloTw + 2, kHaloRows = kHaloTh + 2;
constexpr int kHaloABytes = ((kHaloCols * kHaloRows * 128) + 1023) / 1024 * 1024;   // 23552
constexpr int kHaloMaxB = 18;   // weight stages (barrier slots)
constexpr int kHaloMaxA = 8;    // activation patch stages
constexpr int kHaloBarBytes = 512;

struct HaloParams {
  int a_stages, b_stages, b_resident;
};

template <int BN, int ACT, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_halo_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmY, const ConvGemmParams p, const HaloParams hp) {
  constexpr int kBRows = PAIR ? BN / 2 : BN;      // weight rows staged by this CTA (a pair splits the column tile)
  constexpr int kBBytes = kBRows * kBK * 2;
  constexpr int kTmemCols = next_pow2_cols(2 * BN);
  const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(16) float s_bias[kBiasFloats];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int SA = hp.a_stages, SB = hp.b_stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SA * kHaloABytes + SB * 3 * kBBytes + kStagingBytes);
  // bars: a_full[SA] a_empty[SA] b_full[SB] b_empty[SB] tfull[2] tempty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SA + 2 * SB + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto a_full = [&](int s) { return bar0 + 8u * s; };
  auto a_empty = [&](int s) { return bar0 + 8u * (SA + s); };
  auto b_full = [&](int s) { return bar0 + 8u * (2 * SA + s); };
  auto b_empty = [&](int s) { return bar0 + 8u * (2 * SA + SB + s); };
  const uint32_t tfull0 = bar0 + 8u * (2 * SA + 2 * SB);
  const uint32_t tempty0 = tfull0 + 16u;
  const uint32_t a0 = smem_u32(smem);
  const uint32_t b0 = a0 + SA * kHaloABytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < SB; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8u * a, 1);
      mbar_init(tempty0 + 8u * a, ((p.y_tma && p.epi_teams) ? kTeamWarps : kEpiWarps) * (PAIR ? 2 : 1));
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(tmem_slot), kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int slabs = p.kb_per_tap;
  const uint32_t halo_bytes = kHaloCols * kHaloRows * 128;

  if (warp == 0) {
    if (lane == 0) {
      int sa = 0, sb = 0;
      uint32_t pa = 0, pb = 0;
      bool ok = true, first = true;
      int item = 0;
      for (int v = work_first(p); ok && v < p.total_tiles; v += p.gemm_ctas, ++item) {
        const int tile = work_tile(p, v, pair_rank);
        const TileCoord tc = decode_tile(p, tile);
        const int n_tile = tc.n_tile, twi = tc.twi, thi = tc.thi, img = tc.img;
        for (int kb = 0; ok && kb < slabs; ++kb) {
          if (!mbar_wait(a_empty(sa), pa ^ 1, abort_flag, kStatusTimeoutProducer)) { ok = false; break; }
          // in a pair both CTAs' bytes complete on the even CTA's barriers, which it arms for both
          if (!PAIR) mbar_arrive_expect_tx(a_full(sa), halo_bytes);
          else if (pair_rank == 0) mbar_arrive_expect_tx(a_full(sa), 2u * halo_bytes);
          if (kb == 0) trace_mark(p, item, 0);
          if (PAIR) tma_load_4d_pair(a0 + sa * kHaloABytes, &tmA, a_full(sa), kb * kBK, twi * kHaloTw - 1, thi * kHaloTh - 1, img);
          else tma_load_4d(a0 + sa * kHaloABytes, &tmA, a_full(sa), kb * kBK, twi * kHaloTw - 1, thi * kHaloTh - 1, img);
          if (++sa == SA) { sa = 0; pa ^= 1; }
          if (hp.b_resident && !first) continue;
          // weights travel one filter row (3 taps) per stage
          for (int kh = 0; kh < 3; ++kh) {
            if (!hp.b_resident) {
              if (!mbar_wait(b_empty(sb), pb ^ 1, abort_flag, kStatusTimeoutProducer)) { ok = false; break; }
            }
            if (!PAIR) mbar_arrive_expect_tx(b_full(sb), 3 * kBBytes);
            else if (pair_rank == 0) mbar_arrive_expect_tx(b_full(sb), 2u * 3u * kBBytes);
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
              if (PAIR)
                tma_load_2d_pair(b0 + sb * (3 * kBBytes) + kw * kBBytes, &tmB, b_full(sb),
                                 ((kh * 3 + kw) * slabs + kb) * kBK, n_tile * BN + static_cast<int>(pair_rank) * kBRows);
              else
                tma_load_2d(b0 + sb * (3 * kBBytes) + kw * kBBytes, &tmB, b_full(sb),
                            ((kh * 3 + kw) * slabs + kb) * kBK, n_tile * BN);
            }
            if (++sb == SB) { sb = 0; pb ^= 1; }
          }
        }
        first = false;
      }
      if (!ok) {
        for (int i = 0; i < SA; ++i)
          for (int it = 0; it < (1 << 14); ++it)
            if (mbar_try_wait(a_full(i), 0) || mbar_try_wait(a_full(i), 1)) break;
      }
    }
  } else if (warp == 1) {
    // One elected thread issues everything; see the note in conv_gemm_kernel on why the loop holds
    // no votes and no tcgen05 fences.
    if (pair_rank == 0 && elect_one()) {
      int sa = 0, sb = 0, acc = 0;
      uint32_t pa = 0, pb = 0, acc_ph = 0;
      bool ok = true, weights_ready = false;
      const uint64_t bdesc_hi = make_kmajor_desc(0, 128);
      // shifted views of the halo patch: 8-row groups are 10 pixel rows (1280 bytes) apart
      const uint64_t adesc_hi = (bdesc_hi & ~(0x3FFFull << 32)) | (static_cast<uint64_t>((kHaloCols * 128) >> 4) << 32);
      auto mma = [&](uint32_t d, uint64_t ad, uint64_t bd, uint32_t accum, uint32_t nsteps) {
        if (PAIR) umma_f16_ksteps_pair(d, ad, bd, p.idesc, accum, nsteps);
        else umma_f16_ksteps(d, ad, bd, p.idesc, accum, nsteps);
      };
      auto commit = [&](uint32_t bar) {
        if (PAIR) umma_commit_pair(bar);
        else umma_commit(bar);
      };
      int it = 0;
      for (int v = work_first(p); ok && v < p.total_tiles; v += p.gemm_ctas, ++it) {
        if (!mbar_wait(tempty0 + 8u * acc, acc_ph ^ 1, abort_flag, kStatusTimeoutMma)) break;
        trace_mark(p, it, 1);
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; ok && kb < slabs; ++kb) {
          if (!mbar_wait(a_full(sa), pa, abort_flag, kStatusTimeoutMma)) { ok = false; break; }
          if (kb == 0) trace_mark(p, it, 2);
          const uint32_t a_base = a0 + sa * kHaloABytes;
          const uint32_t ksteps = kb == slabs - 1 ? static_cast<uint32_t>(p.last_ksteps) : 4u;
          if (hp.b_resident && weights_ready) {
            // Steady state with all weights resident: nine taps, straight-line. Nothing but the
            // descriptor additions sits between the MMAs, because whatever does is paid in full.
            const uint64_t ad = adesc_hi | ((a_base & 0x3FFFF) >> 4);
            const uint64_t bd = bdesc_hi | (((b0 + kb * 9 * kBBytes) & 0x3FFFF) >> 4);
#pragma unroll
            for (int t = 0; t < 9; ++t) {
              const int kh = t / 3, kw = t - 3 * kh;
              mma(d_tmem, ad + (((kh * kHaloCols + kw) * 128) >> 4), bd + ((t * kBBytes) >> 4), (kb | t) != 0 ? 1u : 0u,
                  ksteps);
            }
            commit(a_empty(sa));
            if (++sa == SA) { sa = 0; pa ^= 1; }
            continue;
          }
#pragma unroll 1
          for (int kh = 0; kh < 3; ++kh) {
            if (hp.b_resident) sb = kb * 3 + kh;
            if (!(hp.b_resident && weights_ready)) {
              if (!mbar_wait(b_full(sb), hp.b_resident ? 0u : pb, abort_flag, kStatusTimeoutMma)) { ok = false; break; }
            }
            // tap (kh, kw) starts (kh*10 + kw) pixel rows into the patch
            const uint32_t a_row = a_base + kh * kHaloCols * 128;
            const uint32_t b_row = b0 + sb * (3 * kBBytes);
            const uint64_t ad0 = adesc_hi | ((a_row & 0x3FFFF) >> 4);
            const uint64_t bd0 = bdesc_hi | ((b_row & 0x3FFFF) >> 4);
            mma(d_tmem, ad0, bd0, (kb | kh) != 0 ? 1u : 0u, ksteps);
            mma(d_tmem, ad0 + (128 >> 4), bd0 + (kBBytes >> 4), 1u, ksteps);
            mma(d_tmem, ad0 + (256 >> 4), bd0 + (2 * kBBytes >> 4), 1u, ksteps);
            if (!hp.b_resident) {
              commit(b_empty(sb));
              if (++sb == SB) { sb = 0; pb ^= 1; }
            }
          }
          if (!ok) break;
          commit(a_empty(sa));
          if (++sa == SA) { sa = 0; pa ^= 1; }
        }
        if (!ok) break;
        commit(tfull0 + 8u * acc);
        weights_ready = true;
        trace_mark(p, it, 3);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
    __syncwarp();
  } else if (p.y_tma) {
    epilogue_loop_tma<BN, ACT>(p, &tmY, b0 + SB * 3 * kBBytes, tmem_base, tfull0, tempty0, abort_flag, s_bias, warp,
                               lane);
  } else {
    epilogue_loop<BN, ACT>(p, tmem_base, tfull0, tempty0, abort_flag, warp, lane);
  }

  tc_fence_before();
  if (PAIR) cluster_sync_all();    // see conv_gemm_kernel: a pair leaves together
  else __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, *abort_flag);
}

// ------------------------------------------------------------------ host side
struct ConvGemmOp : Op {
  alignas(64) CUtensorMap tmA;
  alignas(64) CUtensorMap tmB;
  alignas(64) CUtensorMap tmY;
  ConvGemmParams prm;
  int block_n = 0;
  int grid = 0;
  int pair = 0;          // 1: clusters of two CTAs sharing every MMA (cta_group::2)
  int halo = 0;          // 1: conv3x3_halo_kernel
  HaloParams hp{};
  int halo_smem = 0;
  PeerTable* peer_dev = nullptr;
  int launch(cudaStream_t stream) override;
  ~ConvGemmOp() override {
    if (peer_dev != nullptr) cudaFree(peer_dev);
  }
};

template <int BN, int ACT>
static int launch_inst(ConvGemmOp* op, cudaStream_t stream) {
  using Cfg = KernelCfg<BN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  FDB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    FDB_CUDA_OK(cudaFuncSetAttribute(conv_gemm_kernel<BN, ACT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::kSmemBytes));
    attr_set[dev] = true;
  }
  if (op->prm.peer_mode == 1) ++op->prm.peer_epoch;   // the ready flags of this launch
  conv_gemm_kernel<BN, ACT, false><<<op->grid, kThreads, Cfg::kSmemBytes, stream>>>(op->tmA, op->tmB, op->tmY, op->prm);
  FDB_CUDA_OK(cudaGetLastError());
  return 0;
}

// CTA-pair form: the grid is launched as clusters of two CTAs.
template <int BN, int ACT>
static int launch_pair_inst(ConvGemmOp* op, cudaStream_t stream) {
  using Cfg = KernelCfg<BN, true>;
  static bool attr_set[64] = {false};
  int dev = 0;
  FDB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    FDB_CUDA_OK(cudaFuncSetAttribute(conv_gemm_kernel<BN, ACT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::kSmemBytes));
    attr_set[dev] = true;
  }
  if (op->prm.peer_mode == 1) ++op->prm.peer_epoch;   // the ready flags of this launch
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(op->grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FDB_CUDA_OK(cudaLaunchKernelEx(&cfg, conv_gemm_kernel<BN, ACT, true>, op->tmA, op->tmB, op->tmY, op->prm));
  return 0;
}

template <int BN, int ACT>
static int launch_halo_inst(ConvGemmOp* op, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  FDB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    FDB_CUDA_OK(cudaFuncSetAttribute(conv3x3_halo_kernel<BN, ACT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kMaxSmem));
    attr_set[dev] = true;
  }
  conv3x3_halo_kernel<BN, ACT, false><<<op->grid, kThreads, op->halo_smem, stream>>>(op->tmA, op->tmB, op->tmY, op->prm, op->hp);
  FDB_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int BN, int ACT>
static int launch_halo_pair_inst(ConvGemmOp* op, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  FDB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    FDB_CUDA_OK(cudaFuncSetAttribute(conv3x3_halo_kernel<BN, ACT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kMaxSmem));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(op->grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = op->halo_smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FDB_CUDA_OK(cudaLaunchKernelEx(&cfg, conv3x3_halo_kernel<BN, ACT, true>, op->tmA, op->tmB, op->tmY, op->prm, op->hp));
  return 0;
}

template <int BN>
static int launch_bn(ConvGemmOp* op, cudaStream_t stream) {
  if (op->halo && op->pair) {
    if constexpr (BN >= 64) {
      switch (op->prm.act) {
        case kActNone: return launch_halo_pair_inst<BN, kActNone>(op, stream);
        case kActRelu: return launch_halo_pair_inst<BN, kActRelu>(op, stream);
        case kActSilu: return launch_halo_pair_inst<BN, kActSilu>(op, stream);
        default: return launch_halo_pair_inst<BN, kTplGeneric>(op, stream);
      }
    } else {
      set_error("conv_gemm: CTA pairs need block_n >= 64");
      return -1;
    }
  }
  if (op->halo) {
    switch (op->prm.act) {
      case kActNone: return launch_halo_inst<BN, kActNone>(op, stream);
      case kActRelu: return launch_halo_inst<BN, kActRelu>(op, stream);
      case kActSilu: return launch_halo_inst<BN, kActSilu>(op, stream);
      default: return launch_halo_inst<BN, kTplGeneric>(op, stream);
    }
  }
  if (op->pair) {
    if constexpr (BN >= 64) {      // pairs are only planned for wide column tiles
      switch (op->prm.act) {
        case kActNone: return launch_pair_inst<BN, kActNone>(op, stream);
        case kActRelu: return launch_pair_inst<BN, kActRelu>(op, stream);
        case kActSilu: return launch_pair_inst<BN, kActSilu>(op, stream);
        case kActGelu: return launch_pair_inst<BN, kActGelu>(op, stream);
        default: return launch_pair_inst<BN, kTplGeneric>(op, stream);
      }
    } else {
      set_error("conv_gemm: CTA pairs need block_n >= 64");
      return -1;
    }
  }
  switch (op->prm.act) {
    case kActNone: return launch_inst<BN, kActNone>(op, stream);
    case kActRelu: return launch_inst<BN, kActRelu>(op, stream);
    case kActSilu: return launch_inst<BN, kActSilu>(op, stream);
    case kActGelu: return launch_inst<BN, kActGelu>(op, stream);
    default: return launch_inst<BN, kTplGeneric>(op, stream);
  }
}

int ConvGemmOp::launch(cudaStream_t stream) {
  switch (block_n) {
    case 32: return launch_bn<32>(this, stream);
    case 48: return launch_bn<48>(this, stream);
    case 64: return launch_bn<64>(this, stream);
    case 80: return launch_bn<80>(this, stream);
    case 96: return launch_bn<96>(this, stream);
    case 128: return launch_bn<128>(this, stream);
    case 160: return launch_bn<160>(this, stream);
    case 192: return launch_bn<192>(this, stream);
    case 256: return launch_bn<256>(this, stream);
  }
  set_error("conv_gemm: bad block_n");
  return -1;
}

// Picks the output-pixel tile (tile_w x tile_h <= 128) that wastes the fewest MMA rows.
static void choose_tile(int Ho, int Wo, int stride, int* tw_out, int* th_out) {
  double best = -1.0;
  int btw = 1, bth = 1;
  for (int tw = 1; tw <= std::min(Wo, kBM); ++tw) {
    if (tw * stride > 256) break;
    int th = std::min(kBM / tw, Ho);
    if (th * stride > 256) th = 256 / stride;
    if (th < 1) continue;
    const long tiles = static_cast<long>((Wo + tw - 1) / tw) * ((Ho + th - 1) / th);
    const double util = static_cast<double>(Ho) * Wo / (static_cast<double>(tiles) * kBM);
    if (util > best + 1e-9 || (util > best - 1e-9 && tw > btw)) {
      best = util;
      btw = tw;
      bth = th;
    }
  }
  *tw_out = btw;
  *th_out = bth;
}

static const int kBlockNs[9] = {256, 192, 160, 128, 96, 80, 64, 48, 32};

static bool valid_block_n(int bn) {
  for (int i = 0; i < 9; ++i)
    if (kBlockNs[i] == bn) return true;
  return false;
}

// Smallest padded width wins (fewest wasted MMA columns); among equals the widest tile,
// because the activation tile is fetched once per column tile.
static int choose_block_n(int Cout, long m_tiles, int sms) {
  (void)m_tiles; (void)sms;
  int pick = 256;
  long best = -1;
  for (int i = 0; i < 9; ++i) {
    const int bn = kBlockNs[i];
    const long padded = static_cast<long>((Cout + bn - 1) / bn) * bn;
    if (best < 0 || padded < best) {
      best = padded;
      pick = bn;
    }
  }
  return pick;
}

}  // namespace fdb

using namespace fdb;

FDB_API void* fdb_conv_gemm_create(const ConvGemmDesc* d) {
  const bool fp8 = d->dtype == kF8E4M3;
  if (d->dtype != kF16 && d->dtype != kBF16 && !fp8) { set_error("conv_gemm: dtype must be fp16, bf16 or fp8 e4m3"); return nullptr; }
  if (fp8 && (d->residual != nullptr || d->w_batched || d->halo_mode == 1)) {
    set_error("conv_gemm: fp8 operands take the plain kernel without residual or batched weights"); return nullptr;
  }
  if (d->out_dtype == kF8E4M3 && (d->peer_mode >= 2 || d->residual != nullptr)) {
    set_error("conv_gemm: an e4m3 output cannot be combined with a residual or the reduce-scatter mode"); return nullptr;
  }
  const int es = fp8 ? 1 : 2;                 // operand element size
  const int kblk = fp8 ? 2 * kBK : kBK;       // K elements per 128-byte stage row
  if (d->Cin % 8 != 0 || d->x_ld % 8 != 0) { set_error("conv_gemm: Cin and x_ld must be multiples of 8"); return nullptr; }
  if (fp8 && (d->Cin % 16 != 0 || d->x_ld % 16 != 0)) { set_error("conv_gemm: fp8 rows must be multiples of 16 elements"); return nullptr; }
  if ((reinterpret_cast<uintptr_t>(d->x) & 15) || (reinterpret_cast<uintptr_t>(d->w) & 15)) {
    set_error("conv_gemm: x and w must be 16-byte aligned"); return nullptr;
  }
  if (d->stride < 1 || d->stride > 8) { set_error("conv_gemm: stride must be in [1,8]"); return nullptr; }
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) { set_error("conv_gemm: cuTensorMapEncodeTiled unavailable"); return nullptr; }

  auto* op = new ConvGemmOp();
  ConvGemmParams& p = op->prm;
  int tw = d->tile_w, th = d->tile_h;
  if (tw <= 0 || th <= 0) choose_tile(d->Ho, d->Wo, d->stride, &tw, &th);
  if (d->w_batched) {
    if (d->KH != 1 || d->KW != 1 || d->stride != 1 || d->w_ld % 8 != 0 || (d->w_batched != 1 && d->w_batched != 2)) {
      set_error("conv_gemm: batched weights need a 1x1 stride-1 product and w_ld % 8 == 0"); delete op; return nullptr;
    }
    if (d->w_batched == 2 && (d->w_n_stride % 8 != 0 || d->w_n_stride < static_cast<long long>(d->Cout) * d->w_ld)) {
      set_error("conv_gemm: per-image weights need w_n_stride % 8 == 0 covering Cout rows"); delete op; return nullptr;
    }
    if (d->w_batched == 1) {   // one matrix per image row: a tile may not span rows
      th = 1;
      tw = std::min(d->Wo, kBM);
    }
  }
  if (tw * th > kBM || tw * d->stride > 256 || th * d->stride > 256) {
    set_error("conv_gemm: tile too large"); delete op; return nullptr;
  }
  // 3x3 / stride 1 / pad 1: prefer the halo kernel unless its fixed 8x16 tile wastes too many rows
  const bool halo_ok = !d->w_batched && d->KH == 3 && d->KW == 3 && d->stride == 1 && d->pad_h == 1 && d->pad_w == 1;
  if (d->halo_mode == 1 && !halo_ok) { set_error("conv_gemm: halo kernel needs 3x3, stride 1, pad 1"); delete op; return nullptr; }
  if (halo_ok && d->halo_mode != 0 && !fp8) {
    const double util_gen = static_cast<double>(d->Ho) * d->Wo /
        (static_cast<double>((d->Wo + tw - 1) / tw) * ((d->Ho + th - 1) / th) * kBM);
    const double util_halo = static_cast<double>(d->Ho) * d->Wo /
        (static_cast<double>((d->Wo + kHaloTw - 1) / kHaloTw) * ((d->Ho + kHaloTh - 1) / kHaloTh) * kBM);
    if (d->halo_mode == 1 || util_halo >= 0.75 * util_gen) {
      op->halo = 1;
      tw = kHaloTw;
      th = kHaloTh;
    }
  }
  p.tw = tw; p.th = th;
  p.tiles_w = (d->Wo + tw - 1) / tw;
  p.tiles_h = (d->Ho + th - 1) / th;
  const long m_tiles = static_cast<long>(p.tiles_w) * p.tiles_h * d->N;
  const int sms = sm_count();
  int bn = d->block_n > 0 ? d->block_n : choose_block_n(d->Cout, m_tiles, sms);
  if (!valid_block_n(bn)) { set_error("conv_gemm: block_n must be one of 32,48,64,80,96,128,160,192,256"); delete op; return nullptr; }
  op->block_n = bn;
  p.n_tiles = (d->Cout + bn - 1) / bn;
  const long total = m_tiles * p.n_tiles;
  if (total > 0x7fffffffL) { set_error("conv_gemm: too many tiles"); delete op; return nullptr; }
  p.total_tiles = static_cast<int>(total);
  p.kb_per_tap = (d->Cin + kblk - 1) / kblk;
  p.k_iters = d->KH * d->KW * p.kb_per_tap;
  p.last_ksteps = (d->Cin - (p.kb_per_tap - 1) * kblk + kblk / 4 - 1) / (kblk / 4);
  p.kblk = kblk; p.fp8 = fp8 ? 1 : 0; p.scale_a = d->scale_a; p.scale_b = d->scale_b;
  p.bias = d->bias; p.residual = d->residual; p.y = d->y; p.status = d->status;
  p.Ho = d->Ho; p.Wo = d->Wo; p.Cout = d->Cout; p.y_ld = d->y_ld;
  p.res_ld = d->res_ld; p.res_mode = d->residual ? d->res_mode : 0;
  p.out_dtype = d->out_dtype; p.in_bf16 = d->dtype == kBF16;
  p.out_scale = d->out_scale != 0.f ? d->out_scale : 1.f;
  p.KH = d->KH; p.KW = d->KW; p.stride = d->stride; p.pad_h = d->pad_h; p.pad_w = d->pad_w;
  p.act = d->act; p.act_alpha = d->act_alpha; p.act_beta = d->act_beta;
  p.b_batched = d->w_batched;
  p.trace = d->trace;
  p.y_h_stride = d->y_h_stride > 0 ? d->y_h_stride : static_cast<long long>(d->Wo) * d->y_ld;
  p.res_h_stride = d->res_h_stride > 0 ? d->res_h_stride : static_cast<long long>(d->Wo) * d->res_ld;
  p.y_n_stride = d->y_n_stride > 0 ? d->y_n_stride : static_cast<long long>(d->Ho) * d->Wo * d->y_ld;
  p.res_n_stride = d->res_n_stride > 0 ? d->res_n_stride : static_cast<long long>(d->Ho) * d->Wo * d->res_ld;
  p.a_bytes = static_cast<uint32_t>(tw * th * kBK * 2);
  p.idesc = make_idesc(d->dtype == kBF16 ? 1u : 0u, kBM, bn);   // format 0 = F16 (kind::f16) or E4M3 (kind::f8f6f4)
  const int out_es = d->out_dtype == kF32 ? 4 : (d->out_dtype == kF8E4M3 ? 1 : 2);
  p.y_vec = (reinterpret_cast<uintptr_t>(d->y) % 16 == 0) && ((d->y_ld * out_es) % 16 == 0) &&
            (d->bias == nullptr || reinterpret_cast<uintptr_t>(d->bias) % 16 == 0);
  p.res_vec = d->residual && (reinterpret_cast<uintptr_t>(d->residual) % 16 == 0) && (d->res_ld % 8 == 0);
  // The bias fast path reads float4 pairs; fall back to scalars when misaligned.
  if (d->bias != nullptr && reinterpret_cast<uintptr_t>(d->bias) % 16 != 0) {
    set_error("conv_gemm: bias must be 16-byte aligned"); delete op; return nullptr;
  }
  int grid = static_cast<int>(std::min<long>(total, d->max_ctas > 0 ? d->max_ctas : sms));
  op->grid = std::max(grid, 1);
  p.pair = 0;
  p.n_images = d->N;
  if (op->halo) {
    const int budget = kMaxSmem - 1024 - kHaloBarBytes - kStagingBytes;
    // CTA pairs: each CTA stages half of the filter, so twice the channels stay resident and streamed
    // weights cost half the L2 traffic per SM
    const long items_pair = ((m_tiles + 1) / 2) * p.n_tiles;
    const bool pair_can = d->pair_mode != 0 && bn >= 64 && m_tiles >= 2 && d->peer_mode == 0 && d->max_ctas != 1;
    if (d->pair_mode == 1 && !pair_can) {
      set_error("conv_gemm: CTA pairs need block_n >= 64, no peer mode and 2+ tiles"); delete op; return nullptr;
    }
    bool use_pair = pair_can && (d->pair_mode == 1 || (bn >= 96 && items_pair >= sms / 2));
    const int all_b = 3 * p.kb_per_tap;
    HaloParams hp{};
    auto plan_rings = [&](bool pair_now) {
      const int b_bytes = 3 * (pair_now ? bn / 2 : bn) * kBK * 2;   // one filter row (3 taps) per weight stage
      hp = HaloParams{};
      // Activation patches come from DRAM, weights from L2: bytes in flight matter for the patches,
      // so they get the deeper ring.
      if (p.n_tiles == 1 && all_b <= kHaloMaxB && 3 * kHaloABytes + all_b * b_bytes <= budget) {
        hp.b_resident = 1;
        hp.b_stages = all_b;
        hp.a_stages = std::min(kHaloMaxA, (budget - all_b * b_bytes) / kHaloABytes);
      } else {
        hp.b_resident = 0;
        // three patch stages first, the rest of the budget to the weight ring (at least two stages)
        hp.b_stages = std::max(2, std::min(kHaloMaxB, (budget - 3 * kHaloABytes) / b_bytes));
        hp.a_stages = std::min(kHaloMaxA, (budget - hp.b_stages * b_bytes) / kHaloABytes);
        if (hp.a_stages < 2) { hp.a_stages = 2; hp.b_stages = (budget - 2 * kHaloABytes) / b_bytes; }
      }
    };
    plan_rings(use_pair);
    if (hp.b_stages < 2 && !use_pair && pair_can) {
      // a wide filter row that one CTA cannot double-buffer fits when a CTA pair splits it
      use_pair = true;
      plan_rings(true);
    }
    if (use_pair && hp.b_stages >= 2) {
      op->pair = p.pair = 1;
      p.total_tiles = static_cast<int>(items_pair);
      const int max_pairs = std::max(1, (d->max_ctas > 0 ? d->max_ctas : sms) / 2);
      op->grid = 2 * static_cast<int>(std::min<long>(items_pair, max_pairs));
    }
    if (hp.b_stages < 2) {
      if (d->halo_mode == 1) { set_error("conv_gemm: halo kernel does not fit shared memory"); delete op; return nullptr; }
      op->halo = 0;   // fall back to the generic kernel with its own tile choice
      op->pair = p.pair = 0;
      choose_tile(d->Ho, d->Wo, d->stride, &tw, &th);
      p.tw = tw; p.th = th;
      p.tiles_w = (d->Wo + tw - 1) / tw;
      p.tiles_h = (d->Ho + th - 1) / th;
      const long mt = static_cast<long>(p.tiles_w) * p.tiles_h * d->N;
      p.total_tiles = static_cast<int>(mt * p.n_tiles);
      p.a_bytes = static_cast<uint32_t>(tw * th * kBK * 2);
      op->grid = std::max(1, static_cast<int>(std::min<long>(p.total_tiles, d->max_ctas > 0 ? d->max_ctas : sms)));
    } else {
      op->hp = hp;
      const int b_bytes = 3 * (use_pair ? bn / 2 : bn) * kBK * 2;
      op->halo_smem = hp.a_stages * kHaloABytes + hp.b_stages * b_bytes + kStagingBytes + kHaloBarBytes + 1024;
    }
  }

  // ---- CTA pairs: two pixel tiles of one column tile per MMA, half of the weight tile staged per CTA
  if (!op->halo && d->pair_mode != 0) {
    const long mt = static_cast<long>(p.tiles_w) * p.tiles_h * d->N;
    const bool can = !d->w_batched && bn >= 64 && mt >= 2 && d->max_ctas != 1;
    if (d->pair_mode == 1 && !can) {
      set_error("conv_gemm: CTA pairs need shared weights, block_n >= 64, 2+ tiles");
      delete op; return nullptr;
    }
    // worthwhile when the weight tile is a large share of the operand traffic and there is work for every pair
    const long items = ((mt + 1) / 2) * p.n_tiles;
    if (can && (d->pair_mode == 1 || (bn >= 128 && items >= sms / 2))) {
      op->pair = p.pair = 1;
      p.total_tiles = static_cast<int>(items);
      const int max_pairs = std::max(1, (d->max_ctas > 0 ? d->max_ctas : sms) / 2);
      const int pairs = static_cast<int>(std::min<long>(items, max_pairs));
      op->grid = 2 * pairs;
    }
  }

  const CUtensorMapDataType tdt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
      : d->dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  {
    cuuint64_t dims[4] = {(cuuint64_t)d->Cin, (cuuint64_t)d->W, (cuuint64_t)d->H, (cuuint64_t)d->N};
    cuuint64_t strides[3] = {(cuuint64_t)d->x_ld * es,
                             (cuuint64_t)(d->x_h_stride > 0 ? d->x_h_stride : (long long)d->W * d->x_ld) * es,
                             (cuuint64_t)(d->x_n_stride > 0 ? d->x_n_stride : (long long)d->H * d->W * d->x_ld) * es};
    cuuint32_t box[4] = {(cuuint32_t)kblk, (cuuint32_t)(tw * d->stride), (cuuint32_t)(th * d->stride), 1};
    if (op->halo) { box[1] = kHaloCols; box[2] = kHaloRows; }
    cuuint32_t estr[4] = {1, (cuuint32_t)d->stride, (cuuint32_t)d->stride, 1};
    CUresult r = enc(&op->tmA, tdt, 4, const_cast<void*>(d->x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("conv_gemm: encode activation tensor map failed, CUresult " + std::to_string((int)r));
      delete op; return nullptr;
    }
  }
  if (d->w_batched) {
    const bool per_image = d->w_batched == 2;
    cuuint64_t dims[4] = {(cuuint64_t)d->Cin, (cuuint64_t)d->Cout, (cuuint64_t)(per_image ? 1 : d->H), (cuuint64_t)d->N};
    cuuint64_t strides[3] = {(cuuint64_t)d->w_ld * 2, (cuuint64_t)(per_image ? d->w_n_stride : d->w_h_stride) * 2,
                             (cuuint64_t)d->w_n_stride * 2};
    cuuint32_t box[4] = {(cuuint32_t)kBK, (cuuint32_t)bn, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&op->tmB, tdt, 4, const_cast<void*>(d->w), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("conv_gemm: encode batched weight tensor map failed, CUresult " + std::to_string((int)r));
      delete op; return nullptr;
    }
  } else {
    const cuuint64_t ktot = (cuuint64_t)d->KH * d->KW * p.kb_per_tap * kblk;
    cuuint64_t dims[2] = {ktot, (cuuint64_t)d->Cout};
    cuuint64_t strides[1] = {ktot * es};
    cuuint32_t box[2] = {(cuuint32_t)kblk, (cuuint32_t)(op->pair ? bn / 2 : bn)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&op->tmB, tdt, 2, const_cast<void*>(d->w), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("conv_gemm: encode weight tensor map failed, CUresult " + std::to_string((int)r));
      delete op; return nullptr;
    }
  }
  // 16-bit outputs leave through TMA tensor stores when the layout allows it
  p.y_tma = 0;
  {
    const bool out16 = d->out_dtype == kF16 || d->out_dtype == kBF16;
    // e4m3 results take the same staged path (32-byte rows) when nothing but bias, column scale and activation
    // sits between the accumulator and the store
    const bool out8 = d->out_dtype == kF8E4M3 && d->residual == nullptr && (!fp8 || d->scale_a == nullptr);
    const int yes = out8 ? 1 : 2;
    const bool aligned = reinterpret_cast<uintptr_t>(d->y) % 16 == 0 && (d->y_ld * yes) % 16 == 0 &&
                         (p.y_h_stride * yes) % 16 == 0 && (p.y_n_stride * yes) % 16 == 0;
    const bool cols_ok = p.n_tiles == 1 || bn % kChunkCols == 0;
    if ((out16 || out8) && aligned && cols_ok && d->y_tma_mode != 0) {
      const CUtensorMapDataType ydt = out8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
          : d->out_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      cuuint64_t dims[4] = {(cuuint64_t)d->Cout, (cuuint64_t)d->Wo, (cuuint64_t)d->Ho, (cuuint64_t)d->N};
      cuuint64_t strides[3] = {(cuuint64_t)d->y_ld * yes, (cuuint64_t)p.y_h_stride * yes, (cuuint64_t)p.y_n_stride * yes};
      cuuint32_t box[4] = {kChunkCols, (cuuint32_t)p.tw, (cuuint32_t)p.th, 1};
      cuuint32_t estr[4] = {1, 1, 1, 1};
      CUresult r = enc(&op->tmY, ydt, 4, d->y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       out8 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r == CUDA_SUCCESS) p.y_tma = 1;
    }
    if (!p.y_tma) op->tmY = op->tmA;   // a valid map is still passed; the kernel does not touch it
    p.epi_teams = bn <= 64 ? 1 : 0;
  }
  p.peer = nullptr;
  p.peer_mode = 0; p.peer_rows = 0; p.peer_rank = 0;
  p.peer_world = 1; p.peer_rot = 0; p.peer_epoch = 0; p.ready = nullptr; p.gather_dst = nullptr; p.gather_row_bytes = 0;
  for (int r = 0; r < 8; ++r) p.peer_src[r] = nullptr;
  if (d->peer_mode != 0) {
    const bool gemm_shape = d->KH == 1 && d->KW == 1 && d->stride == 1 && d->H == 1 && d->N == 1 && d->Ho == 1 &&
                            d->pad_h == 0 && d->pad_w == 0 && !op->halo && !d->w_batched && p.tw == kBM && p.th == 1;
    if (!gemm_shape || d->peer_world < 1 || d->peer_world > 8 || d->peer_rows % kBM != 0 ||
        d->W != d->peer_rows * d->peer_world || d->peer_rank < 0 || d->peer_rank >= d->peer_world ||
        (d->peer_mode != 1 && d->peer_mode != 2 && d->peer_mode != 3)) {
      set_error("conv_gemm: peer modes take a plain GEMM whose M is world * peer_rows, peer_rows a multiple of 128");
      delete op; return nullptr;
    }
    if (d->peer_mode >= 2 && !p.y_tma) {
      set_error("conv_gemm: reduce-scatter mode needs the TMA store path (16-bit output, aligned rows)");
      delete op; return nullptr;
    }
    PeerTable host{};
    for (int r = 0; r < d->peer_world; ++r) {
      if ((d->peer_mode != 3 && d->peer_ptrs[r] == nullptr) || (d->peer_mode >= 2 && d->peer_counters[r] == nullptr)) {
        set_error("conv_gemm: missing peer pointer"); delete op; return nullptr;
      }
      CUresult res = CUDA_SUCCESS;
      if (d->peer_mode == 1) {
        p.peer_src[r] = static_cast<const uint8_t*>(d->peer_ptrs[r]);
      } else if (d->peer_mode == 3) {
        host.counters[r] = d->peer_counters[r];      // the result goes through the ordinary local store
      } else {
        const CUtensorMapDataType ydt =
            d->out_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const cuuint64_t rows = (cuuint64_t)d->peer_rows * d->peer_world;
        cuuint64_t dims[4] = {(cuuint64_t)d->Cout, rows, 1, 1};
        cuuint64_t strides[3] = {(cuuint64_t)d->y_ld * 2, rows * d->y_ld * 2, rows * d->y_ld * 2};
        cuuint32_t box[4] = {kChunkCols, (cuuint32_t)p.tw, 1, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        res = enc(&host.maps[r], ydt, 4, d->peer_ptrs[r], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        host.counters[r] = d->peer_counters[r];
      }
      if (res != CUDA_SUCCESS) {
        set_error("conv_gemm: encode peer tensor map failed, CUresult " + std::to_string((int)res));
        delete op; return nullptr;
      }
    }
    if (cudaMalloc(reinterpret_cast<void**>(&op->peer_dev), sizeof(PeerTable)) != cudaSuccess ||
        cudaMemcpy(op->peer_dev, &host, sizeof(PeerTable), cudaMemcpyHostToDevice) != cudaSuccess) {
      set_error("conv_gemm: peer table allocation failed"); delete op; return nullptr;
    }
    p.peer = op->peer_dev;
    p.peer_mode = d->peer_mode; p.peer_rows = d->peer_rows; p.peer_rank = d->peer_rank;
    p.peer_world = d->peer_world;
    if (d->peer_mode == 1) {
      if (d->peer_ready == nullptr || (static_cast<long long>(d->x_ld) * es) % 16 != 0) {
        set_error("conv_gemm: all-gather mode needs ready flags and 16-byte rows"); delete op; return nullptr;
      }
      const int remote_blocks = p.tiles_w - d->peer_rows / p.tw;
      int copiers = d->peer_copiers > 0 ? d->peer_copiers : 12;
      copiers = std::min(copiers, std::min(remote_blocks, op->grid / 2));
      if (op->pair) {
        // clusters of two throughout: an even number of copier CTAs behind the GEMM pairs
        copiers = (std::max(copiers, 0) + 1) / 2 * 2;
        const int total = std::max(op->grid, copiers + 2);
        op->grid = (total - copiers) / 2 * 2 + copiers;
        p.gemm_ctas = (op->grid - copiers) / 2;
      } else {
        op->grid = std::max(op->grid, copiers + 1);
        p.gemm_ctas = op->grid - std::max(copiers, 0);
      }
      // the copier CTAs and the GEMM CTAs wait on one another inside this launch: all of them must be resident
      if (op->grid > sms) {
        set_error("conv_gemm: the all-gather GEMM needs every CTA resident at once (grid <= SM count)");
        delete op; return nullptr;
      }
      p.peer_rot = d->peer_rank * (d->peer_rows / p.tw);
      p.peer_epoch = 0;
      p.ready = d->peer_ready;
      p.gather_dst = static_cast<uint8_t*>(const_cast<void*>(d->x));
      p.gather_row_bytes = static_cast<long long>(d->x_ld) * es;
    }
  }
  if (p.peer_mode != 1) p.gemm_ctas = op->pair ? op->grid / 2 : op->grid;
  if (op->pair) p.idesc = make_idesc(d->dtype == kBF16 ? 1u : 0u, 2 * kBM, bn);   // M = 256 over the two CTAs
  {
    const unsigned long long one = 1ull << 40;
    const long long dmax = std::max(p.n_tiles, std::max(p.tiles_w, p.tiles_h));
    if ((static_cast<long long>(p.total_tiles) * (op->pair ? 2 : 1) + p.n_tiles) * dmax >= static_cast<long long>(one)) {
      set_error("conv_gemm: too many tiles for the tile decoder"); delete op; return nullptr;
    }
    p.mul_n = (one + p.n_tiles - 1) / p.n_tiles;
    p.mul_w = (one + p.tiles_w - 1) / p.tiles_w;
    p.mul_h = (one + p.tiles_h - 1) / p.tiles_h;
  }
  return op;
}

// Size of the descriptor as this library was compiled: the Python mirror checks it at load time.
FDB_API int fdb_conv_gemm_desc_size() { return static_cast<int>(sizeof(ConvGemmDesc)); }

// Introspection for tests and the autotuner: tile_w, tile_h, block_n, grid, total tiles.
FDB_API void fdb_conv_gemm_info(void* handle, int* out5) {
  auto* op = static_cast<ConvGemmOp*>(handle);
  out5[0] = op->prm.tw; out5[1] = op->prm.th; out5[2] = op->block_n; out5[3] = op->grid;
  out5[4] = op->prm.total_tiles;
}

// 0 generic kernel, 1 halo kernel with streamed weights, 2 halo kernel with resident weights,
// 3 generic kernel on CTA pairs, 4 / 5 halo kernel on CTA pairs with streamed / resident weights
FDB_API int fdb_conv_gemm_variant(void* handle) {
  auto* op = static_cast<ConvGemmOp*>(handle);
  if (op->halo) return op->pair ? (op->hp.b_resident ? 5 : 4) : (op->hp.b_resident ? 2 : 1);
  return op->pair ? 3 : 0;
}
