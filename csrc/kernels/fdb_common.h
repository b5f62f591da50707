// Host-side plumbing shared by every kernel family of the native backend.
//
// A kernel family exposes `fdb_<family>_create(const Desc*) -> FdbOp*`; the
// returned object owns everything a launch needs (tensor maps, grid, kernel
// parameters) so that a launch is a single virtual call with no host work,
// which keeps the executor's replay loop and CUDA-graph capture cheap.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#define FDB_API extern "C" __attribute__((visibility("default")))

namespace fdb {

// Element types understood by the kernels (values are part of the C ABI).
enum DType : int {
  kF16 = 0,
  kBF16 = 1,
  kF32 = 2,
  kU8 = 3,
  kI32 = 4,
  kI64 = 5,
  kF8E4M3 = 6,
  kI8 = 7,
};

inline int dtype_size(int dt) {
  switch (dt) {
    case kF16: case kBF16: return 2;
    case kF32: case kI32: return 4;
    case kI64: return 8;
    default: return 1;
  }
}

// Activation codes applied in fused epilogues (values are part of the C ABI).
enum Act : int {
  kActNone = 0,
  kActRelu = 1,
  kActSilu = 2,
  kActHardSwish = 3,
  kActHardSigmoid = 4,   // clip(alpha*x + beta, 0, 1)
  kActSigmoid = 5,
  kActGelu = 6,          // exact erf form
  kActRelu6 = 7,
  kActLeakyRelu = 8,     // alpha = negative slope
  kActTanh = 9,
};

struct Op {
  virtual ~Op() {}
  virtual int launch(cudaStream_t stream) = 0;
};

// Last error message of this thread, readable from Python.
void set_error(const std::string& msg);
const char* get_error();

// cuTensorMapEncodeTiled resolved at run time (no link-time libcuda dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace fdb

// Checked build (-DFDB_BOUNDS_CHECK): a data-dependent index (a token id, a gather index) that the release
// build silently clamps into range is also counted, and the first offender kept, in a record per .cu file;
// fdb_bounds_report() sums the records and names the first site. A .cu file that uses FDB_NOTE_OOB puts
// FDB_BOUNDS_TU("its name") once at namespace scope.
namespace fdb {
struct OobRecord { unsigned long long count; long long index; long long extent; int site; int pad; };
typedef int (*OobReader)(OobRecord* out, int reset);
void register_oob_reader(const char* unit, OobReader fn);
}  // namespace fdb
#ifdef FDB_BOUNDS_CHECK
namespace fdb {
static __device__ OobRecord g_oob_record;
static __device__ __forceinline__ void note_oob(int site, long long i, long long n) {
  if (atomicAdd(&g_oob_record.count, 1ull) == 0ull) { g_oob_record.index = i; g_oob_record.extent = n; g_oob_record.site = site; }
}
}  // namespace fdb
#define FDB_NOTE_OOB(site, i, n) do { if ((i) < 0 || (i) >= (n)) fdb::note_oob((site), (i), (n)); } while (0)
#define FDB_BOUNDS_TU(unit)                                                                      \
  namespace {                                                                                    \
  int fdb_read_oob_record(fdb::OobRecord* out, int reset) {                                      \
    if (cudaMemcpyFromSymbol(out, fdb::g_oob_record, sizeof(fdb::OobRecord)) != cudaSuccess) return -1; \
    if (reset) {                                                                                 \
      fdb::OobRecord zero = {};                                                                  \
      if (cudaMemcpyToSymbol(fdb::g_oob_record, &zero, sizeof(zero)) != cudaSuccess) return -1;  \
    }                                                                                            \
    return 0;                                                                                    \
  }                                                                                              \
  struct FdbOobRegistrar { FdbOobRegistrar() { fdb::register_oob_reader(unit, &fdb_read_oob_record); } } fdb_oob_registrar; \
  }
#else
#define FDB_NOTE_OOB(site, i, n) do { } while (0)
#define FDB_BOUNDS_TU(unit)
#endif

#define FDB_CUDA_OK(expr)                                                          \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess) {                                                       \
      fdb::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e));          \
      return -1;                                                                   \
    }                                                                              \
  } while (0)
