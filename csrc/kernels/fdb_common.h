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

#define FDB_CUDA_OK(expr)                                                          \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess) {                                                       \
      fdb::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e));          \
      return -1;                                                                   \
    }                                                                              \
  } while (0)
