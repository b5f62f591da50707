#include <string>

#include "fdb_cpu.h"

namespace fdbcpu {
static thread_local std::string g_error;
void set_error(const char* msg) { g_error = msg ? msg : ""; }
}  // namespace fdbcpu

FDB_CPU_API const char* fdb_cpu_last_error() { return fdbcpu::g_error.c_str(); }
