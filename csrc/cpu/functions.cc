// Host tensor math of the function library (fastdeploy/function/functions.h:17-37 and the files it includes:
// cast, clip, concat, cumprod, elementwise, reduce, argmax/argmin, softmax, sort, tile, transpose, pad, slice,
// gather/scatter along an axis, quantile, isfinite, math) on strided n-d views, plain C ABI.
//
// Every entry point takes FnTensor views: a base pointer, a dtype code, up to 8 dimensions and element strides
// (0 = broadcast, any sign of layout: transposes, slices and tiles are strided copies). Arithmetic runs in double
// for the floating types and in int64 for the integer types, and is rounded once on the way out; integer division
// truncates toward zero (C++ semantics, as the reference's Eigen functors do). Sorting is stable, arg-max / arg-min
// return the first extreme, quantile interpolates linearly between the two nearest order statistics.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <numeric>
#include <string>
#include <vector>

#include "fdb_cpu.h"

namespace {

enum DType : int { kBool = 0, kU8 = 1, kI8 = 2, kI32 = 3, kI64 = 4, kF32 = 5, kF64 = 6 };
constexpr int kMaxDims = 8;

struct FnTensor {
  void* data;
  int dtype;
  int ndim;
  long long shape[kMaxDims];
  long long strides[kMaxDims];   // in elements
};

inline bool is_float(int dt) { return dt == kF32 || dt == kF64; }

inline double load_f(const void* p, int dt, long long i) {
  switch (dt) {
    case kBool: case kU8: return static_cast<const uint8_t*>(p)[i];
    case kI8: return static_cast<const int8_t*>(p)[i];
    case kI32: return static_cast<const int32_t*>(p)[i];
    case kI64: return static_cast<double>(static_cast<const int64_t*>(p)[i]);
    case kF32: return static_cast<const float*>(p)[i];
    default: return static_cast<const double*>(p)[i];
  }
}

inline long long to_int64_fwd(double v) {
  if (v != v) return 0;
  if (v >= 9.2233720368547748e18) return std::numeric_limits<long long>::max();
  if (v <= -9.2233720368547758e18) return std::numeric_limits<long long>::min();
  return static_cast<long long>(v);
}

inline long long load_i(const void* p, int dt, long long i) {
  switch (dt) {
    case kBool: case kU8: return static_cast<const uint8_t*>(p)[i];
    case kI8: return static_cast<const int8_t*>(p)[i];
    case kI32: return static_cast<const int32_t*>(p)[i];
    case kI64: return static_cast<const int64_t*>(p)[i];
    case kF32: return static_cast<long long>(static_cast<const float*>(p)[i]);
    default: return static_cast<long long>(static_cast<const double*>(p)[i]);
  }
}

// A floating value on its way into an integer type: NaN becomes 0 and the value is clamped to what int64 holds
// before the conversion (converting an out-of-range double is undefined); narrowing from int64 then wraps.
inline long long to_int64(double v) {
  if (v != v) return 0;
  if (v >= 9.2233720368547748e18) return std::numeric_limits<long long>::max();
  if (v <= -9.2233720368547758e18) return std::numeric_limits<long long>::min();
  return static_cast<long long>(v);
}

inline void store_f(void* p, int dt, long long i, double v) {
  switch (dt) {
    case kBool: static_cast<uint8_t*>(p)[i] = v != 0.0 ? 1 : 0; break;
    case kU8: static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(static_cast<unsigned long long>(to_int64(v))); break;
    case kI8: static_cast<int8_t*>(p)[i] = static_cast<int8_t>(static_cast<uint8_t>(static_cast<unsigned long long>(to_int64(v)))); break;
    case kI32: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(static_cast<uint32_t>(static_cast<unsigned long long>(to_int64(v)))); break;
    case kI64: static_cast<int64_t*>(p)[i] = to_int64(v); break;
    case kF32: static_cast<float*>(p)[i] = static_cast<float>(v); break;
    default: static_cast<double*>(p)[i] = v; break;
  }
}

inline void store_i(void* p, int dt, long long i, long long v) {
  switch (dt) {
    case kBool: static_cast<uint8_t*>(p)[i] = v != 0 ? 1 : 0; break;
    case kU8: static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(v); break;
    case kI8: static_cast<int8_t*>(p)[i] = static_cast<int8_t>(v); break;
    case kI32: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
    case kI64: static_cast<int64_t*>(p)[i] = v; break;
    case kF32: static_cast<float*>(p)[i] = static_cast<float>(v); break;
    default: static_cast<double*>(p)[i] = static_cast<double>(v); break;
  }
}

long long numel(const FnTensor& t) {
  long long n = 1;
  for (int d = 0; d < t.ndim; ++d) n *= t.shape[d];
  return n;
}

bool valid(const FnTensor* t, const char* what) {
  if (t == nullptr || t->ndim < 0 || t->ndim > kMaxDims || t->dtype < kBool || t->dtype > kF64 ||
      (t->data == nullptr && numel(*t) != 0)) {
    fdbcpu::set_error((std::string(what) + ": bad tensor view").c_str());
    return false;
  }
  return true;
}

// Walks the index space of `shape`; offs[k] is the element offset into operand k.
template <int N, typename Fn>
void for_each(int ndim, const long long* shape, const long long* const (&strides)[N], Fn&& fn) {
  long long total = 1;
  for (int d = 0; d < ndim; ++d) total *= shape[d];
  if (total == 0) return;
  long long idx[kMaxDims] = {0};
  long long offs[N] = {0};
  for (long long it = 0; it < total; ++it) {
    fn(offs);
    for (int d = ndim - 1; d >= 0; --d) {
      ++idx[d];
      for (int k = 0; k < N; ++k) offs[k] += strides[k][d];
      if (idx[d] < shape[d]) break;
      for (int k = 0; k < N; ++k) offs[k] -= strides[k][d] * shape[d];
      idx[d] = 0;
    }
  }
}

bool same_shape(const FnTensor& a, const FnTensor& b) {
  if (a.ndim != b.ndim) return false;
  for (int d = 0; d < a.ndim; ++d) if (a.shape[d] != b.shape[d]) return false;
  return true;
}

}  // namespace

FDB_CPU_API int fdf_tensor_size() { return static_cast<int>(sizeof(FnTensor)); }

// out[...] = in[...] converted to out's dtype (float -> integer truncates toward zero, anything -> bool is != 0).
// The views may differ in layout: this is also transpose, slice, tile (stride 0) and the body of concat and pad.
FDB_CPU_API int fdf_copy(const FnTensor* in, const FnTensor* out) {
  if (!valid(in, "copy") || !valid(out, "copy")) return -1;
  if (!same_shape(*in, *out)) { fdbcpu::set_error("copy: shapes differ"); return -1; }
  const long long* const st[2] = {in->strides, out->strides};
  const bool via_int = !is_float(in->dtype) && !is_float(out->dtype);
  for_each<2>(in->ndim, in->shape, st, [&](const long long* o) {
    if (via_int) store_i(out->data, out->dtype, o[1], load_i(in->data, in->dtype, o[0]));
    else if (out->dtype == kBool) store_i(out->data, out->dtype, o[1], load_f(in->data, in->dtype, o[0]) != 0.0 ? 1 : 0);
    else if (!is_float(out->dtype)) store_i(out->data, out->dtype, o[1], to_int64(std::trunc(load_f(in->data, in->dtype, o[0]))));
    else store_f(out->data, out->dtype, o[1], load_f(in->data, in->dtype, o[0]));
  });
  return 0;
}

FDB_CPU_API int fdf_fill(const FnTensor* out, double value) {
  if (!valid(out, "fill")) return -1;
  const long long* const st[1] = {out->strides};
  for_each<1>(out->ndim, out->shape, st, [&](const long long* o) { store_f(out->data, out->dtype, o[0], value); });
  return 0;
}

// op: 0 clip(a, b)  1 sqrt  2 log  3 round (half away from zero is NOT used: ties go to even, as std::nearbyint)
//     4 exp  5 abs  6 ceil  7 floor  8 isnan  9 isinf  10 isfinite
FDB_CPU_API int fdf_unary(int op, const FnTensor* in, const FnTensor* out, double a, double b) {
  if (!valid(in, "unary") || !valid(out, "unary")) return -1;
  if (!same_shape(*in, *out)) { fdbcpu::set_error("unary: shapes differ"); return -1; }
  const long long* const st[2] = {in->strides, out->strides};
  const bool ints = !is_float(in->dtype);
  for_each<2>(in->ndim, in->shape, st, [&](const long long* o) {
    if (ints && (op == 0 || op == 5)) {
      long long v = load_i(in->data, in->dtype, o[0]);
      if (op == 0) v = std::min(std::max(v, static_cast<long long>(a)), static_cast<long long>(b));
      else v = v < 0 ? -v : v;
      store_i(out->data, out->dtype, o[1], v);
      return;
    }
    const double x = load_f(in->data, in->dtype, o[0]);
    double y = x;
    switch (op) {
      case 0: y = std::isnan(x) ? x : std::min(std::max(x, a), b); break;
      case 1: y = std::sqrt(x); break;
      case 2: y = std::log(x); break;
      case 3: y = std::nearbyint(x); break;
      case 4: y = std::exp(x); break;
      case 5: y = std::fabs(x); break;
      case 6: y = std::ceil(x); break;
      case 7: y = std::floor(x); break;
      case 8: y = std::isnan(x) ? 1.0 : 0.0; break;
      case 9: y = std::isinf(x) ? 1.0 : 0.0; break;
      case 10: y = std::isfinite(x) ? 1.0 : 0.0; break;
      default: break;
    }
    store_f(out->data, out->dtype, o[1], y);
  });
  return 0;
}

// op: 0 add  1 subtract  2 multiply  3 divide  4 maximum  5 minimum; a and b are given with out's shape
// (broadcast dimensions carry stride 0). Integer operands: int64 arithmetic, division truncates toward zero and a
// zero divisor is an error (the reference would trap).
FDB_CPU_API int fdf_binary(int op, const FnTensor* a, const FnTensor* b, const FnTensor* out) {
  if (!valid(a, "binary") || !valid(b, "binary") || !valid(out, "binary")) return -1;
  if (!same_shape(*a, *out) || !same_shape(*b, *out)) { fdbcpu::set_error("binary: operands must be expanded to the output shape"); return -1; }
  const long long* const st[3] = {a->strides, b->strides, out->strides};
  const bool ints = !is_float(a->dtype) && !is_float(b->dtype);
  bool div_zero = false;
  for_each<3>(out->ndim, out->shape, st, [&](const long long* o) {
    if (ints) {
      const long long x = load_i(a->data, a->dtype, o[0]), y = load_i(b->data, b->dtype, o[1]);
      long long r = 0;
      switch (op) {
        case 0: r = x + y; break;
        case 1: r = x - y; break;
        case 2: r = x * y; break;
        case 3: if (y == 0) { div_zero = true; r = 0; } else r = x / y; break;
        case 4: r = std::max(x, y); break;
        default: r = std::min(x, y); break;
      }
      if (is_float(out->dtype)) store_f(out->data, out->dtype, o[2], static_cast<double>(r));
      else store_i(out->data, out->dtype, o[2], r);
      return;
    }
    const double x = load_f(a->data, a->dtype, o[0]), y = load_f(b->data, b->dtype, o[1]);
    double r = 0;
    switch (op) {
      case 0: r = x + y; break;
      case 1: r = x - y; break;
      case 2: r = x * y; break;
      case 3: r = x / y; break;
      case 4: r = (std::isnan(x) || std::isnan(y)) ? std::numeric_limits<double>::quiet_NaN() : std::max(x, y); break;
      default: r = (std::isnan(x) || std::isnan(y)) ? std::numeric_limits<double>::quiet_NaN() : std::min(x, y); break;
    }
    store_f(out->data, out->dtype, o[2], r);
  });
  if (div_zero) { fdbcpu::set_error("divide: integer division by zero"); return -1; }
  return 0;
}

// Reduction over the axes whose bit is set in axis_mask; `out` has the input's rank with extent 1 on the reduced
// axes. op: 0 sum  1 mean  2 max  3 min  4 prod  5 all  6 any. Integer sums and products stay in int64.
FDB_CPU_API int fdf_reduce(int op, const FnTensor* in, const FnTensor* out, unsigned axis_mask) {
  if (!valid(in, "reduce") || !valid(out, "reduce")) return -1;
  if (in->ndim != out->ndim) { fdbcpu::set_error("reduce: output must keep the rank"); return -1; }
  long long kept_shape[kMaxDims], red_shape[kMaxDims], in_keep[kMaxDims], in_red[kMaxDims], out_keep[kMaxDims];
  long long count = 1;
  for (int d = 0; d < in->ndim; ++d) {
    const bool r = (axis_mask >> d) & 1u;
    if (out->shape[d] != (r ? 1 : in->shape[d])) { fdbcpu::set_error("reduce: output shape"); return -1; }
    kept_shape[d] = r ? 1 : in->shape[d];
    red_shape[d] = r ? in->shape[d] : 1;
    in_keep[d] = r ? 0 : in->strides[d];
    in_red[d] = r ? in->strides[d] : 0;
    out_keep[d] = r ? 0 : out->strides[d];
    if (r) count *= in->shape[d];
  }
  if (count == 0 && (op == 2 || op == 3)) { fdbcpu::set_error("reduce: max / min of an empty range"); return -1; }
  const bool ints = !is_float(in->dtype);
  const long long* const outer[2] = {in_keep, out_keep};
  const long long* const inner[1] = {in_red};
  for_each<2>(in->ndim, kept_shape, outer, [&](const long long* o) {
    double facc = (op == 4) ? 1.0 : 0.0;
    long long iacc = (op == 4) ? 1 : 0;
    bool first = true, flag = (op == 5);
    for_each<1>(in->ndim, red_shape, inner, [&](const long long* q) {
      const long long at = o[0] + q[0];
      if (op == 5 || op == 6) {
        const bool nz = ints ? load_i(in->data, in->dtype, at) != 0 : load_f(in->data, in->dtype, at) != 0.0;
        flag = op == 5 ? (flag && nz) : (flag || nz);
      } else if (ints) {
        const long long v = load_i(in->data, in->dtype, at);
        if (op <= 1) iacc += v;
        else if (op == 4) iacc *= v;
        else if (first || (op == 2 ? v > iacc : v < iacc)) iacc = v;
      } else {
        const double v = load_f(in->data, in->dtype, at);
        if (op <= 1) facc += v;
        else if (op == 4) facc *= v;
        else if (first || std::isnan(v) || (!std::isnan(facc) && (op == 2 ? v > facc : v < facc))) facc = v;
      }
      first = false;
    });
    if (op == 5 || op == 6) store_i(out->data, out->dtype, o[1], flag ? 1 : 0);
    else if (op == 1) store_f(out->data, out->dtype, o[1], (ints ? static_cast<double>(iacc) : facc) / static_cast<double>(count));
    else if (ints && !is_float(out->dtype)) store_i(out->data, out->dtype, o[1], iacc);
    else store_f(out->data, out->dtype, o[1], ints ? static_cast<double>(iacc) : facc);
  });
  return 0;
}

// Index of the first maximum (want_max) or minimum along `axis`; `out` (integer) has extent 1 there. NaN counts
// as the extreme, as in the reference's comparison-based scan a NaN never loses its place once taken.
FDB_CPU_API int fdf_arg_extreme(int want_max, const FnTensor* in, const FnTensor* out, int axis) {
  if (!valid(in, "arg") || !valid(out, "arg")) return -1;
  if (axis < 0 || axis >= in->ndim || in->ndim != out->ndim || in->shape[axis] < 1) { fdbcpu::set_error("arg: bad axis"); return -1; }
  long long kept[kMaxDims], in_keep[kMaxDims], out_keep[kMaxDims];
  for (int d = 0; d < in->ndim; ++d) {
    kept[d] = d == axis ? 1 : in->shape[d];
    in_keep[d] = d == axis ? 0 : in->strides[d];
    out_keep[d] = d == axis ? 0 : out->strides[d];
  }
  const long long n = in->shape[axis], step = in->strides[axis];
  const long long* const st[2] = {in_keep, out_keep};
  for_each<2>(in->ndim, kept, st, [&](const long long* o) {
    long long best = 0;
    double bv = load_f(in->data, in->dtype, o[0]);
    for (long long k = 1; k < n && !std::isnan(bv); ++k) {
      const double v = load_f(in->data, in->dtype, o[0] + k * step);
      if (std::isnan(v) || (want_max ? v > bv : v < bv)) { bv = v; best = k; }
    }
    store_i(out->data, out->dtype, o[1], best);
  });
  return 0;
}

// mode 0: soft-max along `axis` (max-subtracted, accumulated in double); mode 1: cumulative product along `axis`.
FDB_CPU_API int fdf_scan(int mode, const FnTensor* in, const FnTensor* out, int axis) {
  if (!valid(in, "scan") || !valid(out, "scan")) return -1;
  if (!same_shape(*in, *out) || axis < 0 || axis >= in->ndim) { fdbcpu::set_error("scan: shapes / axis"); return -1; }
  long long kept[kMaxDims], in_keep[kMaxDims], out_keep[kMaxDims];
  for (int d = 0; d < in->ndim; ++d) {
    kept[d] = d == axis ? 1 : in->shape[d];
    in_keep[d] = d == axis ? 0 : in->strides[d];
    out_keep[d] = d == axis ? 0 : out->strides[d];
  }
  const long long n = in->shape[axis], si = in->strides[axis], so = out->strides[axis];
  const bool ints = !is_float(in->dtype);
  const long long* const st[2] = {in_keep, out_keep};
  for_each<2>(in->ndim, kept, st, [&](const long long* o) {
    if (mode == 1) {
      double facc = 1.0;
      long long iacc = 1;
      for (long long k = 0; k < n; ++k) {
        if (ints) { iacc *= load_i(in->data, in->dtype, o[0] + k * si); store_i(out->data, out->dtype, o[1] + k * so, iacc); }
        else { facc *= load_f(in->data, in->dtype, o[0] + k * si); store_f(out->data, out->dtype, o[1] + k * so, facc); }
      }
      return;
    }
    double mx = -std::numeric_limits<double>::infinity(), sum = 0.0;
    for (long long k = 0; k < n; ++k) mx = std::max(mx, load_f(in->data, in->dtype, o[0] + k * si));
    if (std::isinf(mx) && mx < 0) mx = 0.0;
    for (long long k = 0; k < n; ++k) sum += std::exp(load_f(in->data, in->dtype, o[0] + k * si) - mx);
    for (long long k = 0; k < n; ++k)
      store_f(out->data, out->dtype, o[1] + k * so, std::exp(load_f(in->data, in->dtype, o[0] + k * si) - mx) / sum);
  });
  return 0;
}

// Stable sort along `axis`: values into `values` (may be null) and source positions into `indices` (may be null).
// NaNs go last in ascending order and first in descending order (they compare as the largest value).
FDB_CPU_API int fdf_sort(const FnTensor* in, const FnTensor* values, const FnTensor* indices, int axis, int descending) {
  if (!valid(in, "sort")) return -1;
  if (axis < 0 || axis >= in->ndim) { fdbcpu::set_error("sort: bad axis"); return -1; }
  if ((values && (!valid(values, "sort") || !same_shape(*in, *values))) ||
      (indices && (!valid(indices, "sort") || !same_shape(*in, *indices)))) { fdbcpu::set_error("sort: output shapes"); return -1; }
  long long kept[kMaxDims], in_keep[kMaxDims], v_keep[kMaxDims], i_keep[kMaxDims];
  for (int d = 0; d < in->ndim; ++d) {
    kept[d] = d == axis ? 1 : in->shape[d];
    in_keep[d] = d == axis ? 0 : in->strides[d];
    v_keep[d] = (values && d != axis) ? values->strides[d] : 0;
    i_keep[d] = (indices && d != axis) ? indices->strides[d] : 0;
  }
  const long long n = in->shape[axis], si = in->strides[axis];
  const bool ints = !is_float(in->dtype);
  const long long* const st[3] = {in_keep, v_keep, i_keep};
  std::vector<long long> order(static_cast<size_t>(n));
  std::vector<double> fv(static_cast<size_t>(ints ? 0 : n));
  std::vector<long long> iv(static_cast<size_t>(ints ? n : 0));
  for_each<3>(in->ndim, kept, st, [&](const long long* o) {
    for (long long k = 0; k < n; ++k) {
      order[k] = k;
      if (ints) iv[k] = load_i(in->data, in->dtype, o[0] + k * si);
      else fv[k] = load_f(in->data, in->dtype, o[0] + k * si);
    }
    auto less_f = [&](long long a, long long b) {            // NaN is the largest value
      const double x = fv[a], y = fv[b];
      if (std::isnan(x)) return false;
      if (std::isnan(y)) return true;
      return x < y;
    };
    if (ints) {
      if (descending) std::stable_sort(order.begin(), order.end(), [&](long long a, long long b) { return iv[a] > iv[b]; });
      else std::stable_sort(order.begin(), order.end(), [&](long long a, long long b) { return iv[a] < iv[b]; });
    } else {
      if (descending) std::stable_sort(order.begin(), order.end(), [&](long long a, long long b) { return less_f(b, a); });
      else std::stable_sort(order.begin(), order.end(), less_f);
    }
    for (long long k = 0; k < n; ++k) {
      if (values) {
        if (ints) store_i(values->data, values->dtype, o[1] + k * values->strides[axis], iv[order[k]]);
        else store_f(values->data, values->dtype, o[1] + k * values->strides[axis], fv[order[k]]);
      }
      if (indices) store_i(indices->data, indices->dtype, o[2] + k * indices->strides[axis], order[k]);
    }
  });
  return 0;
}

// out[..., i, ...] = in[..., index[..., i, ...], ...] along `axis` (gather, scatter = 0) or
// out[..., index[..., i, ...], ...] = src[..., i, ...] (scatter = 1; `out` already holds the base values).
// Negative indices count from the end; anything still outside the axis is an error, nothing is written for it.
FDB_CPU_API int fdf_along_axis(int scatter, const FnTensor* data, const FnTensor* index, const FnTensor* other, int axis) {
  if (!valid(data, "along_axis") || !valid(index, "along_axis") || !valid(other, "along_axis")) return -1;
  if (axis < 0 || axis >= data->ndim || index->ndim != data->ndim || !same_shape(*index, *other) || is_float(index->dtype)) {
    fdbcpu::set_error("along_axis: ranks, index dtype or shapes"); return -1;
  }
  long long data_no_axis[kMaxDims];
  for (int d = 0; d < data->ndim; ++d) data_no_axis[d] = d == axis ? 0 : data->strides[d];
  const long long extent = data->shape[axis], step = data->strides[axis];
  const long long* const st[3] = {index->strides, other->strides, data_no_axis};
  bool bad = false;
  for_each<3>(index->ndim, index->shape, st, [&](const long long* o) {
    long long k = load_i(index->data, index->dtype, o[0]);
    if (k < 0) k += extent;
    if (k < 0 || k >= extent) { bad = true; return; }
    const long long at = o[2] + k * step;
    if (scatter) store_f(data->data, data->dtype, at, load_f(other->data, other->dtype, o[1]));
    else if (is_float(data->dtype)) store_f(other->data, other->dtype, o[1], load_f(data->data, data->dtype, at));
    else store_i(other->data, other->dtype, o[1], load_i(data->data, data->dtype, at));
  });
  if (bad) { fdbcpu::set_error("along_axis: index out of range"); return -1; }
  return 0;
}

// Quantiles q[0..nq) along `axis` with linear interpolation between the order statistics at floor and ceil of
// q * (n - 1); `out` has the input's shape with extent nq on `axis`. A lane that holds a NaN gives NaN.
FDB_CPU_API int fdf_quantile(const FnTensor* in, const FnTensor* out, int axis, const double* q, int nq) {
  if (!valid(in, "quantile") || !valid(out, "quantile")) return -1;
  if (axis < 0 || axis >= in->ndim || in->ndim != out->ndim || out->shape[axis] != nq || in->shape[axis] < 1) {
    fdbcpu::set_error("quantile: axis / output shape"); return -1;
  }
  for (int k = 0; k < nq; ++k) if (!(q[k] >= 0.0 && q[k] <= 1.0)) { fdbcpu::set_error("quantile: q outside [0, 1]"); return -1; }
  long long kept[kMaxDims], in_keep[kMaxDims], out_keep[kMaxDims];
  for (int d = 0; d < in->ndim; ++d) {
    if (d != axis && in->shape[d] != out->shape[d]) { fdbcpu::set_error("quantile: output shape"); return -1; }
    kept[d] = d == axis ? 1 : in->shape[d];
    in_keep[d] = d == axis ? 0 : in->strides[d];
    out_keep[d] = d == axis ? 0 : out->strides[d];
  }
  const long long n = in->shape[axis], si = in->strides[axis], so = out->strides[axis];
  std::vector<double> lane(static_cast<size_t>(n));
  const long long* const st[2] = {in_keep, out_keep};
  for_each<2>(in->ndim, kept, st, [&](const long long* o) {
    bool has_nan = false;
    for (long long k = 0; k < n; ++k) { lane[k] = load_f(in->data, in->dtype, o[0] + k * si); has_nan = has_nan || std::isnan(lane[k]); }
    std::sort(lane.begin(), lane.end());
    for (int k = 0; k < nq; ++k) {
      double r = std::numeric_limits<double>::quiet_NaN();
      if (!has_nan) {
        const double pos = q[k] * static_cast<double>(n - 1);
        const long long lo = static_cast<long long>(std::floor(pos)), hi = static_cast<long long>(std::ceil(pos));
        r = lane[lo] + (lane[hi] - lane[lo]) * (pos - static_cast<double>(lo));
      }
      store_f(out->data, out->dtype, o[1] + k * so, r);
    }
  });
  return 0;
}
