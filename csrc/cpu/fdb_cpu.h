// Host-side native library: plain C ABI, loaded with ctypes.
#pragma once
#include <cstdint>

#if defined(_WIN32)
#define FDB_CPU_API extern "C" __declspec(dllexport)
#else
#define FDB_CPU_API extern "C" __attribute__((visibility("default")))
#endif

// Last error message of the calling thread (empty string when none).
FDB_CPU_API const char* fdb_cpu_last_error();

namespace fdbcpu {
void set_error(const char* msg);
}
