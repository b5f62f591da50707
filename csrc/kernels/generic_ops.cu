// Shape-plumbing kernels of the executor: whatever is left of a graph once the tensor-core ops and the
// fused NHWC helpers have taken their share - layout changes, type casts, small integer / boolean
// arithmetic (masks, position ids), soft-max over the last axis, gathers and reductions - also runs as
// native launches, so that a plan never leaves the stream for a framework operator.
//
//  * strided_copy : dst[idx] = cast(src[idx]) over up to six dimensions with independent element
//                   strides on both sides (transpose, NCHW <-> NHWC, slices of concatenation buffers,
//                   broadcast expansion through zero strides);
//  * elementwise  : unary / binary arithmetic, comparisons and logic with broadcasting, computed in
//                   double (exact for the int64 ids and fp32 values that reach it), any of the
//                   executor's element types in and out;
//  * softmax_last : numerically stable soft-max (or log-soft-max) over the innermost axis, one warp per row;
//  * reduce_last  : sum / mean / max / min / arg-max over the innermost axis;
//  * gather_rows  : out[i, :] = table[index[i], :] for int64 / int32 indices;
//  * where        : out = cond ? a : b with broadcasting.
//
// In the reference these are TensorRT / Paddle Inference layers (trt_backend.cc:347 enqueueV2).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <functional>

#include "fdb_common.h"

namespace fdb {

struct GenericDesc {
  void* p[4];
  long long i[48];
  float f[4];
};

struct GenericOp : Op {
  std::function<int(cudaStream_t)> fn;
  int launch(cudaStream_t s) override { return fn(s); }
};

#define FDB_GEN_CHECK()                                 \
  do {                                                  \
    cudaError_t e_ = cudaGetLastError();                \
    if (e_ != cudaSuccess) {                            \
      set_error(cudaGetErrorString(e_));                \
      return -1;                                        \
    }                                                   \
    return 0;                                           \
  } while (0)

constexpr int kMaxDims = 6;
constexpr int kBool = 8;   // one byte per element, 0 / 1 (the executor's extra type code next to fdb_common.h's)

struct Strides {
  long long shape[kMaxDims];
  long long a[kMaxDims];
  long long b[kMaxDims];
  long long c[kMaxDims];
  long long o[kMaxDims];
  int nd;
};

__device__ __forceinline__ double load_as_double(const void* p, int dt, long long off) {
  switch (dt) {
    case kF32: return static_cast<const float*>(p)[off];
    case kF16: return __half2float(static_cast<const __half*>(p)[off]);
    case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]);
    case kI64: return static_cast<double>(static_cast<const long long*>(p)[off]);
    case kI32: return static_cast<const int*>(p)[off];
    case kU8: case kBool: return static_cast<const unsigned char*>(p)[off];
    case kI8: return static_cast<const signed char*>(p)[off];
    default: return 0.0;
  }
}
__device__ __forceinline__ void store_from_double(void* p, int dt, long long off, double v) {
  switch (dt) {
    case kF32: static_cast<float*>(p)[off] = static_cast<float>(v); break;
    case kF16: static_cast<__half*>(p)[off] = __float2half_rn(static_cast<float>(v)); break;
    case kBF16: static_cast<__nv_bfloat16*>(p)[off] = __float2bfloat16_rn(static_cast<float>(v)); break;
    case kI64: static_cast<long long*>(p)[off] = static_cast<long long>(v); break;
    case kI32: static_cast<int*>(p)[off] = static_cast<int>(v); break;
    case kU8: static_cast<unsigned char*>(p)[off] = static_cast<unsigned char>(v); break;
    case kBool: static_cast<unsigned char*>(p)[off] = v != 0.0 ? 1 : 0; break;
    case kI8: static_cast<signed char*>(p)[off] = static_cast<signed char>(v); break;
    default: break;
  }
}

// ---- copy / cast over strided views ---------------------------------------------------------------
__global__ void strided_copy_kernel(const void* __restrict__ src, void* __restrict__ dst, Strides st, long long total,
                                    int sdt, int ddt) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = idx, so = 0, dof = 0;
#pragma unroll
    for (int d = kMaxDims - 1; d >= 0; --d) {
      if (d < st.nd) {
        const long long k = r % st.shape[d];
        r /= st.shape[d];
        so += k * st.a[d];
        dof += k * st.o[d];
      }
    }
    if (sdt == ddt && (sdt == kF16 || sdt == kBF16)) {      // same 16-bit type: move the bits
      static_cast<unsigned short*>(dst)[dof] = static_cast<const unsigned short*>(src)[so];
    } else if (sdt == ddt && sdt == kF32) {
      static_cast<float*>(dst)[dof] = static_cast<const float*>(src)[so];
    } else if (sdt == ddt && sdt == kI64) {
      static_cast<long long*>(dst)[dof] = static_cast<const long long*>(src)[so];
    } else {
      store_from_double(dst, ddt, dof, load_as_double(src, sdt, so));
    }
  }
}

// ---- elementwise with broadcasting ------------------------------------------------------------------
enum EwOp : int {
  kEwAdd = 0, kEwSub, kEwMul, kEwDiv, kEwMax, kEwMin, kEwPow, kEwEq, kEwNe, kEwLt, kEwLe, kEwGt, kEwGe, kEwAnd, kEwOr,
  kEwXor, kEwFloorDiv, kEwMod,
  kEwNot = 32, kEwNeg, kEwAbs, kEwSqrt, kEwRsqrt, kEwExp, kEwLog, kEwTanh, kEwSigmoid, kEwRelu, kEwErf, kEwFloor, kEwCeil,
  kEwRound, kEwSign, kEwReciprocal, kEwAffine /* x * f0 + f1 */, kEwClip /* f0..f1 */, kEwIdentity, kEwSin, kEwCos,
  kEwHardSigmoid /* clip(f0 x + f1, 0, 1) */, kEwHardSwish, kEwSilu, kEwGelu, kEwLeakyRelu /* f0 */, kEwSoftplus,
};

__device__ __forceinline__ double ew_apply(int op, double a, double b, float f0, float f1) {
  switch (op) {
    case kEwAdd: return a + b;
    case kEwSub: return a - b;
    case kEwMul: return a * b;
    case kEwDiv: return a / b;
    case kEwMax: return fmax(a, b);
    case kEwMin: return fmin(a, b);
    case kEwPow: return pow(a, b);
    case kEwEq: return a == b;
    case kEwNe: return a != b;
    case kEwLt: return a < b;
    case kEwLe: return a <= b;
    case kEwGt: return a > b;
    case kEwGe: return a >= b;
    case kEwAnd: return (a != 0.0) && (b != 0.0);
    case kEwOr: return (a != 0.0) || (b != 0.0);
    case kEwXor: return (a != 0.0) != (b != 0.0);
    case kEwFloorDiv: return floor(a / b);
    case kEwMod: return a - floor(a / b) * b;
    case kEwNot: return a == 0.0;
    case kEwNeg: return -a;
    case kEwAbs: return fabs(a);
    case kEwSqrt: return sqrt(a);
    case kEwRsqrt: return 1.0 / sqrt(a);
    case kEwExp: return exp(a);
    case kEwLog: return log(a);
    case kEwTanh: return tanh(a);
    case kEwSigmoid: return 1.0 / (1.0 + exp(-a));
    case kEwRelu: return fmax(a, 0.0);
    case kEwErf: return erf(a);
    case kEwFloor: return floor(a);
    case kEwCeil: return ceil(a);
    case kEwRound: return rint(a);
    case kEwSign: return (a > 0.0) - (a < 0.0);
    case kEwReciprocal: return 1.0 / a;
    case kEwAffine: return a * static_cast<double>(f0) + static_cast<double>(f1);
    case kEwClip: return fmin(fmax(a, static_cast<double>(f0)), static_cast<double>(f1));
    case kEwSin: return sin(a);
    case kEwCos: return cos(a);
    case kEwHardSigmoid: return fmin(fmax(static_cast<double>(f0) * a + static_cast<double>(f1), 0.0), 1.0);
    case kEwHardSwish: return a * fmin(fmax(a + 3.0, 0.0), 6.0) / 6.0;
    case kEwSilu: return a / (1.0 + exp(-a));
    case kEwGelu: return 0.5 * a * (1.0 + erf(a * 0.70710678118654752));
    case kEwLeakyRelu: return a > 0.0 ? a : static_cast<double>(f0) * a;
    case kEwSoftplus: return log1p(exp(a));
    default: return a;
  }
}

__global__ void elementwise_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                                   Strides st, long long total, int op, int adt, int bdt, int odt, float f0, float f1) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = idx, ao = 0, bo = 0, oo = 0;
#pragma unroll
    for (int d = kMaxDims - 1; d >= 0; --d) {
      if (d < st.nd) {
        const long long k = r % st.shape[d];
        r /= st.shape[d];
        ao += k * st.a[d];
        bo += k * st.b[d];
        oo += k * st.o[d];
      }
    }
    const double x = load_as_double(a, adt, ao);
    const double y = b != nullptr ? load_as_double(b, bdt, bo) : 0.0;
    store_from_double(out, odt, oo, ew_apply(op, x, y, f0, f1));
  }
}

// ---- out = cond ? a : b with broadcasting ---------------------------------------------------------------
__global__ void where_kernel(const void* __restrict__ cond, const void* __restrict__ a, const void* __restrict__ b,
                             void* __restrict__ out, Strides st, long long total, int cdt, int adt, int bdt, int odt) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = idx, ao = 0, bo = 0, co = 0, oo = 0;
#pragma unroll
    for (int d = kMaxDims - 1; d >= 0; --d) {
      if (d < st.nd) {
        const long long k = r % st.shape[d];
        r /= st.shape[d];
        ao += k * st.a[d];
        bo += k * st.b[d];
        co += k * st.c[d];
        oo += k * st.o[d];
      }
    }
    const bool pick = load_as_double(cond, cdt, co) != 0.0;
    store_from_double(out, odt, oo, pick ? load_as_double(a, adt, ao) : load_as_double(b, bdt, bo));
  }
}

// ---- soft-max over the last axis: one warp per row -------------------------------------------------
__global__ void __launch_bounds__(256) softmax_last_kernel(const void* __restrict__ x, void* __restrict__ y, long long rows,
                                                           int C, long long x_ld, long long y_ld, int xdt, int ydt,
                                                           int log_form) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long xo = row * x_ld, yo = row * y_ld;
  float m = -INFINITY;
  for (int c = lane; c < C; c += 32) m = fmaxf(m, static_cast<float>(load_as_double(x, xdt, xo + c)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += __expf(static_cast<float>(load_as_double(x, xdt, xo + c)) - m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float inv = 1.f / s, ls = __logf(s);
  for (int c = lane; c < C; c += 32) {
    const float v = static_cast<float>(load_as_double(x, xdt, xo + c)) - m;
    store_from_double(y, ydt, yo + c, log_form ? v - ls : __expf(v) * inv);
  }
}

// Typed soft-max for floating inputs and outputs: TPR threads per row (a warp for short rows, a 256-thread block for
// long ones such as a 6625-class recogniser head), one online pass for maximum and sum, one pass to write.
template <typename T> __device__ __forceinline__ float sm_load(const T* p, long long i);
template <> __device__ __forceinline__ float sm_load<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float sm_load<__half>(const __half* p, long long i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float sm_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void sm_store(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void sm_store(__half* p, long long i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void sm_store(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ void sm_combine(float& m, float& s, float om, float os) {
  const float nm = fmaxf(m, om);
  if (nm == -INFINITY) { s = 0.f; return; }
  s = s * __expf(m - nm) + os * __expf(om - nm);
  m = nm;
}

template <typename Tin, typename Tout, int TPR>
__global__ void __launch_bounds__(256) softmax_last_fast_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, long long rows,
                                                                int C, long long x_ld, long long y_ld, int log_form) {
  __shared__ float red_m[8], red_s[8];
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) / TPR;
  const int t = threadIdx.x % TPR, lane = threadIdx.x & 31;
  const bool live = row < rows;                     // TPR == 256: the whole block shares one row
  const Tin* xr = x + (live ? row : 0) * x_ld;
  float m = -INFINITY, s = 0.f;
  if (live) {
    for (int c = t; c < C; c += TPR) {
      const float v = sm_load<Tin>(xr, c);
      if (v > m) { s = s * __expf(m - v) + 1.f; m = v; }
      else if (m > -INFINITY) s += __expf(v - m);      // (both -inf: a masked entry before any finite one adds nothing)
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sm_combine(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  if (TPR > 32) {
    if (lane == 0) { red_m[threadIdx.x >> 5] = m; red_s[threadIdx.x >> 5] = s; }
    __syncthreads();
    m = red_m[0]; s = red_s[0];
#pragma unroll
    for (int w = 1; w < TPR / 32; ++w) sm_combine(m, s, red_m[w], red_s[w]);
  }
  if (!live) return;
  const float inv = 1.f / s, ls = __logf(s);
  Tout* yr = y + row * y_ld;
  for (int c = t; c < C; c += TPR) {
    const float v = sm_load<Tin>(xr, c) - m;
    sm_store(yr, c, log_form ? v - ls : __expf(v) * inv);
  }
}

template <typename Tin, typename Tout>
static void launch_softmax_fast(const void* x, void* y, long long rows, int C, long long x_ld, long long y_ld, int lf,
                                cudaStream_t s) {
  if (C >= 2048)
    softmax_last_fast_kernel<Tin, Tout, 256><<<static_cast<unsigned>(rows), 256, 0, s>>>(
        static_cast<const Tin*>(x), static_cast<Tout*>(y), rows, C, x_ld, y_ld, lf);
  else
    softmax_last_fast_kernel<Tin, Tout, 32><<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, s>>>(
        static_cast<const Tin*>(x), static_cast<Tout*>(y), rows, C, x_ld, y_ld, lf);
}

// false when the dtype pair has no typed kernel (the generic one then runs)
static bool softmax_fast(const void* x, void* y, long long rows, int C, long long x_ld, long long y_ld, int xdt, int ydt,
                         int lf, cudaStream_t s) {
  if (rows > 0x7fffffffLL) return false;
#define FDB_SM_CASE(XD, XT, YD, YT) \
  if (xdt == XD && ydt == YD) { launch_softmax_fast<XT, YT>(x, y, rows, C, x_ld, y_ld, lf, s); return true; }
  FDB_SM_CASE(kF16, __half, kF16, __half) FDB_SM_CASE(kF16, __half, kF32, float)
  FDB_SM_CASE(kBF16, __nv_bfloat16, kBF16, __nv_bfloat16) FDB_SM_CASE(kBF16, __nv_bfloat16, kF32, float)
  FDB_SM_CASE(kF32, float, kF32, float) FDB_SM_CASE(kF32, float, kF16, __half) FDB_SM_CASE(kF32, float, kBF16, __nv_bfloat16)
#undef FDB_SM_CASE
  return false;
}

// ---- reductions over the last axis: one warp per row -------------------------------------------------
// mode 0 sum, 1 mean, 2 max, 3 min, 4 arg-max (first maximum), 5 arg-min, 6 product
__global__ void __launch_bounds__(256) reduce_last_kernel(const void* __restrict__ x, void* __restrict__ y, long long rows,
                                                          int C, long long x_ld, int xdt, int ydt, int mode) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long xo = row * x_ld;
  const bool want_max = mode == 2 || mode == 4;
  double acc = mode == 6 ? 1.0 : (mode <= 1 ? 0.0 : (want_max ? -INFINITY : INFINITY));
  int arg = 0x7fffffff;
  for (int c = lane; c < C; c += 32) {
    const double v = load_as_double(x, xdt, xo + c);
    if (mode <= 1) acc += v;
    else if (mode == 6) acc *= v;
    else if (want_max ? (v > acc) : (v < acc)) { acc = v; arg = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const double ov = __shfl_xor_sync(0xffffffffu, acc, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (mode <= 1) acc += ov;
    else if (mode == 6) acc *= ov;
    else if ((want_max ? (ov > acc) : (ov < acc)) || (ov == acc && oa < arg)) { acc = ov; arg = oa; }
  }
  if (lane == 0) {
    if (mode == 1) acc /= C;
    store_from_double(y, ydt, row, mode >= 4 && mode <= 5 ? static_cast<double>(arg) : acc);
  }
}

// ---- row gather: out[i, :] = table[index[i], :] -------------------------------------------------------
__global__ void gather_rows_kernel(const void* __restrict__ table, const void* __restrict__ index, void* __restrict__ out,
                                   long long n_idx, long long row_elems, long long table_rows, int tdt, int idt, int odt) {
  const long long total = n_idx * row_elems;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = idx / row_elems, c = idx - i * row_elems;
    long long r = idt == kI64 ? static_cast<const long long*>(index)[i] : static_cast<const int*>(index)[i];
    if (r < 0) r += table_rows;
    if (c == 0) FDB_NOTE_OOB(1, r, table_rows);
    r = r < 0 ? 0 : (r >= table_rows ? table_rows - 1 : r);      // clamp: an out-of-range id never reads outside
    store_from_double(out, odt, idx, load_as_double(table, tdt, r * row_elems + c));
  }
}

}  // namespace fdb
FDB_BOUNDS_TU("generic_ops")
namespace fdb {

static int grid_of(long long total) {
  long long g = (total + 255) / 256;
  return static_cast<int>(g < 1 ? 1 : (g > 148LL * 32 ? 148LL * 32 : g));
}

}  // namespace fdb

using namespace fdb;

// kind 0 strided_copy : p0 src, p1 dst; i0 nd, i1 src dtype, i2 dst dtype, i3.. shape[6], i9.. src strides[6], i15.. dst strides[6]
// kind 1 elementwise  : p0 a, p1 b (null for unary), p2 out; i0 nd, i1 op, i2 a dtype, i3 b dtype, i4 out dtype,
//                       i5.. shape[6], i11.. a strides, i17.. b strides, i23.. out strides; f0, f1 parameters
// kind 2 softmax_last : p0 x, p1 y; i0 rows, i1 C, i2 x_ld, i3 y_ld, i4 x dtype, i5 y dtype, i6 log form
// kind 3 reduce_last  : p0 x, p1 y; i0 rows, i1 C, i2 x_ld, i3 x dtype, i4 y dtype, i5 mode
// kind 5 where        : p0 cond, p1 a, p2 b, p3 out; i0 nd, i1 cond dtype, i2 a dtype, i3 b dtype, i4 out dtype,
//                       i5.. shape[6], i11.. cond strides, i17.. a strides, i23.. b strides, i29.. out strides
// kind 4 gather_rows  : p0 table, p1 index, p2 out; i0 n_idx, i1 row_elems, i2 table_rows, i3 table dtype, i4 index dtype, i5 out dtype
FDB_API void* fdb_generic_create(int kind, const GenericDesc* dp) {
  const GenericDesc d = *dp;
  auto* op = new GenericOp();
  switch (kind) {
    case 0: {
      Strides st{};
      st.nd = static_cast<int>(d.i[0]);
      const int sdt = d.i[1], ddt = d.i[2];
      if (st.nd < 1 || st.nd > kMaxDims) { set_error("strided_copy: 1..6 dimensions"); delete op; return nullptr; }
      long long total = 1;
      for (int k = 0; k < st.nd; ++k) {
        st.shape[k] = d.i[3 + k]; st.a[k] = d.i[9 + k]; st.o[k] = d.i[15 + k];
        if (st.shape[k] < 0) { set_error("strided_copy: negative extent"); delete op; return nullptr; }
        total *= st.shape[k];
      }
      op->fn = [=](cudaStream_t s) {
        if (total == 0) return 0;
        strided_copy_kernel<<<grid_of(total), 256, 0, s>>>(d.p[0], d.p[1], st, total, sdt, ddt);
        FDB_GEN_CHECK();
      };
      break;
    }
    case 1: {
      Strides st{};
      st.nd = static_cast<int>(d.i[0]);
      const int eop = d.i[1], adt = d.i[2], bdt = d.i[3], odt = d.i[4];
      const float f0 = d.f[0], f1 = d.f[1];
      if (st.nd < 1 || st.nd > kMaxDims) { set_error("elementwise: 1..6 dimensions"); delete op; return nullptr; }
      long long total = 1;
      for (int k = 0; k < st.nd; ++k) {
        st.shape[k] = d.i[5 + k]; st.a[k] = d.i[11 + k]; st.b[k] = d.i[17 + k]; st.o[k] = d.i[23 + k];
        total *= st.shape[k];
      }
      if (eop < kEwNot && d.p[1] == nullptr) { set_error("elementwise: binary op without a second operand"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        if (total == 0) return 0;
        elementwise_kernel<<<grid_of(total), 256, 0, s>>>(d.p[0], d.p[1], d.p[2], st, total, eop, adt, bdt, odt, f0, f1);
        FDB_GEN_CHECK();
      };
      break;
    }
    case 2: {
      const long long rows = d.i[0], x_ld = d.i[2], y_ld = d.i[3];
      const int C = d.i[1], xdt = d.i[4], ydt = d.i[5], lf = d.i[6];
      if (C < 1) { set_error("softmax: empty axis"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        if (rows == 0) return 0;
        if (!softmax_fast(d.p[0], d.p[1], rows, C, x_ld, y_ld, xdt, ydt, lf, s))
          softmax_last_kernel<<<static_cast<int>((rows * 32 + 255) / 256), 256, 0, s>>>(d.p[0], d.p[1], rows, C, x_ld, y_ld, xdt, ydt, lf);
        FDB_GEN_CHECK();
      };
      break;
    }
    case 3: {
      const long long rows = d.i[0], x_ld = d.i[2];
      const int C = d.i[1], xdt = d.i[3], ydt = d.i[4], mode = d.i[5];
      if (C < 1 || mode < 0 || mode > 6) { set_error("reduce: empty axis or unknown mode"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        if (rows == 0) return 0;
        reduce_last_kernel<<<static_cast<int>((rows * 32 + 255) / 256), 256, 0, s>>>(d.p[0], d.p[1], rows, C, x_ld, xdt, ydt, mode);
        FDB_GEN_CHECK();
      };
      break;
    }
    case 4: {
      const long long n_idx = d.i[0], row_elems = d.i[1], table_rows = d.i[2];
      const int tdt = d.i[3], idt = d.i[4], odt = d.i[5];
      if (idt != kI64 && idt != kI32) { set_error("gather_rows: int32 or int64 indices"); delete op; return nullptr; }
      op->fn = [=](cudaStream_t s) {
        if (n_idx * row_elems == 0) return 0;
        gather_rows_kernel<<<grid_of(n_idx * row_elems), 256, 0, s>>>(d.p[0], d.p[1], d.p[2], n_idx, row_elems, table_rows, tdt, idt, odt);
        FDB_GEN_CHECK();
      };
      break;
    }
    case 5: {
      Strides st{};
      st.nd = static_cast<int>(d.i[0]);
      const int cdt = d.i[1], adt = d.i[2], bdt = d.i[3], odt = d.i[4];
      if (st.nd < 1 || st.nd > kMaxDims) { set_error("where: 1..6 dimensions"); delete op; return nullptr; }
      long long total = 1;
      for (int k = 0; k < st.nd; ++k) {
        st.shape[k] = d.i[5 + k]; st.c[k] = d.i[11 + k]; st.a[k] = d.i[17 + k]; st.b[k] = d.i[23 + k]; st.o[k] = d.i[29 + k];
        total *= st.shape[k];
      }
      op->fn = [=](cudaStream_t s) {
        if (total == 0) return 0;
        where_kernel<<<grid_of(total), 256, 0, s>>>(d.p[0], d.p[1], d.p[2], d.p[3], st, total, cdt, adt, bdt, odt);
        FDB_GEN_CHECK();
      };
      break;
    }
    default:
      set_error("fdb_generic_create: unknown kind");
      delete op;
      return nullptr;
  }
  return op;
}
