// Error slot, driver entry point lookup, launch-list ("plan") executor.
#include "fdb_common.h"

#include <mutex>
#include <vector>

namespace fdb {

static thread_local std::string g_err;
void set_error(const std::string& msg) { g_err = msg; }
const char* get_error() { return g_err.c_str(); }

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  });
  return fn;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

struct OobUnit { const char* unit; OobReader fn; };
static std::vector<OobUnit>& oob_units() { static std::vector<OobUnit> v; return v; }
void register_oob_reader(const char* unit, OobReader fn) { oob_units().push_back({unit, fn}); }

// A plan is an ordered launch list. The executor builds it once per
// (model, shape bucket); replay is one native call that issues every kernel on
// the given stream, so it can be captured into a CUDA graph as a whole.
struct Plan {
  std::vector<Op*> ops;
  std::vector<bool> owned;
  unsigned long long launches = 0;
};

}  // namespace fdb

FDB_API const char* fdb_last_error() { return fdb::get_error(); }

// 1 when the library was compiled with -DFDB_BOUNDS_CHECK.
FDB_API int fdb_bounds_checked() {
#ifdef FDB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

// Synchronises the device and writes "count=<n>" (plus " unit=<file> site=<id> index=<i> extent=<n>" of the first
// offender) into buf; returns the count of out-of-range indices seen since the last reset, -1 on a CUDA error.
FDB_API long long fdb_bounds_report(char* buf, int buf_len, int reset) {
  if (cudaDeviceSynchronize() != cudaSuccess) { fdb::set_error("fdb_bounds_report: device synchronise failed"); return -1; }
  unsigned long long total = 0;
  std::string first;
  for (const fdb::OobUnit& u : fdb::oob_units()) {
    fdb::OobRecord r = {};
    if (u.fn(&r, reset) != 0) { fdb::set_error("fdb_bounds_report: cannot read a record"); return -1; }
    if (r.count != 0 && first.empty())
      first = std::string(" unit=") + u.unit + " site=" + std::to_string(r.site) + " index=" + std::to_string(r.index) +
              " extent=" + std::to_string(r.extent);
    total += r.count;
  }
  const std::string msg = "count=" + std::to_string(total) + first;
  if (buf != nullptr && buf_len > 0) snprintf(buf, static_cast<size_t>(buf_len), "%s", msg.c_str());
  return static_cast<long long>(total);
}

FDB_API void* fdb_plan_create() { return new fdb::Plan(); }

FDB_API void fdb_plan_add(void* plan, void* op, int take_ownership) {
  auto* p = static_cast<fdb::Plan*>(plan);
  p->ops.push_back(static_cast<fdb::Op*>(op));
  p->owned.push_back(take_ownership != 0);
}

FDB_API int fdb_plan_size(void* plan) { return (int)static_cast<fdb::Plan*>(plan)->ops.size(); }

FDB_API unsigned long long fdb_plan_launch_count(void* plan) {
  return static_cast<fdb::Plan*>(plan)->launches;
}

FDB_API int fdb_plan_run(void* plan, void* stream) {
  auto* p = static_cast<fdb::Plan*>(plan);
  for (size_t i = 0; i < p->ops.size(); ++i) {
    int rc = p->ops[i]->launch((cudaStream_t)stream);
    if (rc != 0) {
      fdb::set_error("plan op " + std::to_string(i) + " failed: " + fdb::get_error());
      return rc;
    }
  }
  p->launches += p->ops.size();
  return 0;
}

// Runs ops [begin, end) only; used by the per-layer profiler.
FDB_API int fdb_plan_run_range(void* plan, int begin, int end, void* stream) {
  auto* p = static_cast<fdb::Plan*>(plan);
  if (begin < 0) begin = 0;
  if (end > (int)p->ops.size()) end = (int)p->ops.size();
  for (int i = begin; i < end; ++i) {
    int rc = p->ops[i]->launch((cudaStream_t)stream);
    if (rc != 0) return rc;
  }
  p->launches += (end > begin) ? (end - begin) : 0;
  return 0;
}

FDB_API void fdb_plan_destroy(void* plan) {
  auto* p = static_cast<fdb::Plan*>(plan);
  for (size_t i = 0; i < p->ops.size(); ++i)
    if (p->owned[i]) delete p->ops[i];
  delete p;
}

FDB_API int fdb_op_launch(void* op, void* stream) {
  return static_cast<fdb::Op*>(op)->launch((cudaStream_t)stream);
}

FDB_API void fdb_op_destroy(void* op) { delete static_cast<fdb::Op*>(op); }

FDB_API int fdb_sm_count() { return fdb::sm_count(); }

// Blocking copy of device memory to the host by raw address (plan export reads allocator blocks that no tensor
// object covers as a whole).
FDB_API int fdb_copy_to_host(void* dst, const void* src, unsigned long long bytes) {
  if (cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
    fdb::set_error(std::string("fdb_copy_to_host: ") + cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  return 0;
}
