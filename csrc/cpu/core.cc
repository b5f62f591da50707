// Small value types of the core: a tagged scalar, the ue8m0 block-scale format and a wall-clock interval timer.
// Counterparts in the reference: fastdeploy/core/fd_scalar.h:25-115 (Scalar), fastdeploy/utils/perf.h:22-48 (TimeCounter).
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <string>

#include "fdb_cpu.h"

namespace {

// type codes are FDDataType values (BOOL 0, INT16 1, INT32 2, INT64 3, FP16 4, FP32 5, FP64 6, UINT8 20, INT8 21)
struct Scalar {
  int dtype;
  union {
    double f64; float f32; int64_t i64; int32_t i32; int16_t i16; int8_t i8; uint8_t u8; bool b; uint16_t f16;
  } v;
};

float half_to_float(uint16_t h) {
  const uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
  float out;
  if (exp == 0) out = std::ldexp(static_cast<float>(man), -24);
  else if (exp == 31) out = man ? std::numeric_limits<float>::quiet_NaN() : std::numeric_limits<float>::infinity();
  else out = std::ldexp(static_cast<float>(man | 0x400u), static_cast<int>(exp) - 25);
  return sign ? -out : out;
}

double as_double(const Scalar& s) {
  switch (s.dtype) {
    case 0: return s.v.b ? 1.0 : 0.0;
    case 1: return s.v.i16;
    case 2: return s.v.i32;
    case 3: return static_cast<double>(s.v.i64);
    case 4: return half_to_float(s.v.f16);
    case 5: return s.v.f32;
    case 6: return s.v.f64;
    case 20: return s.v.u8;
    case 21: return s.v.i8;
    default: return 0.0;
  }
}

struct Timer {
  std::chrono::steady_clock::time_point begin, end;
};

}  // namespace

// ---- Scalar: 16 bytes, passed by pointer -------------------------------------------------------------
FDB_CPU_API int fdb_scalar_size() { return static_cast<int>(sizeof(Scalar)); }

FDB_CPU_API void fdb_scalar_from_double(void* out, double v, int dtype) {
  Scalar s{};
  s.dtype = dtype;
  switch (dtype) {
    case 0: s.v.b = v != 0.0; break;
    case 1: s.v.i16 = static_cast<int16_t>(v); break;
    case 2: s.v.i32 = static_cast<int32_t>(v); break;
    case 3: s.v.i64 = static_cast<int64_t>(v); break;
    case 5: s.v.f32 = static_cast<float>(v); break;
    case 20: s.v.u8 = static_cast<uint8_t>(v); break;
    case 21: s.v.i8 = static_cast<int8_t>(v); break;
    default: s.dtype = 6; s.v.f64 = v; break;
  }
  std::memcpy(out, &s, sizeof(s));
}

FDB_CPU_API void fdb_scalar_from_int64(void* out, int64_t v) {
  Scalar s{};
  s.dtype = 3;
  s.v.i64 = v;
  std::memcpy(out, &s, sizeof(s));
}

// "inf", "-inf", "nan" or a decimal number -> FP64 scalar (the string form the operator attributes use)
FDB_CPU_API int fdb_scalar_from_string(void* out, const char* text) {
  Scalar s{};
  s.dtype = 6;
  const std::string t(text ? text : "");
  if (t == "inf") s.v.f64 = std::numeric_limits<double>::infinity();
  else if (t == "-inf") s.v.f64 = -std::numeric_limits<double>::infinity();
  else if (t == "nan") s.v.f64 = std::numeric_limits<double>::quiet_NaN();
  else {
    char* end = nullptr;
    s.v.f64 = std::strtod(t.c_str(), &end);
    if (t.empty() || end == t.c_str() || *end != '\0') { fdbcpu::set_error("scalar: not a number"); return -1; }
  }
  std::memcpy(out, &s, sizeof(s));
  return 0;
}

FDB_CPU_API int fdb_scalar_dtype(const void* p) { return static_cast<const Scalar*>(p)->dtype; }
FDB_CPU_API double fdb_scalar_to_double(const void* p) { return as_double(*static_cast<const Scalar*>(p)); }
FDB_CPU_API int64_t fdb_scalar_to_int64(const void* p) {
  const Scalar& s = *static_cast<const Scalar*>(p);
  return s.dtype == 3 ? s.v.i64 : static_cast<int64_t>(as_double(s));
}

// ---- ue8m0: an 8-bit power-of-two scale, value 2^(e - 127); 255 is NaN (the block-scale type of the MX formats) ----
FDB_CPU_API uint8_t fdb_ue8m0_from_float(float v) {
  if (!(v > 0.f) || std::isinf(v)) return std::isnan(v) || std::isinf(v) ? 255 : 0;
  int e;
  const float m = std::frexp(v, &e);          // v = m * 2^e, m in [0.5, 1)
  int exp = e - 1 + (m > 0.5f ? 1 : 0);       // round up to the next power of two: the scaled block never overflows
  exp += 127;
  return static_cast<uint8_t>(exp < 0 ? 0 : (exp > 254 ? 254 : exp));
}
FDB_CPU_API float fdb_ue8m0_to_float(uint8_t e) {
  return e == 255 ? std::numeric_limits<float>::quiet_NaN() : std::ldexp(1.0f, static_cast<int>(e) - 127);
}

// ---- TimeCounter ----------------------------------------------------------------------------------------
FDB_CPU_API void* fdb_timer_create() { return new Timer(); }
FDB_CPU_API void fdb_timer_destroy(void* t) { delete static_cast<Timer*>(t); }
FDB_CPU_API void fdb_timer_start(void* t) { static_cast<Timer*>(t)->begin = std::chrono::steady_clock::now(); }
FDB_CPU_API void fdb_timer_end(void* t) { static_cast<Timer*>(t)->end = std::chrono::steady_clock::now(); }
FDB_CPU_API double fdb_timer_duration(void* t) {
  auto* tm = static_cast<Timer*>(t);
  return std::chrono::duration<double>(tm->end - tm->begin).count();
}
