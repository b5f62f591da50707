// Stand-in for the kernel library in the host-only test of the plan runner: the entry points the runner resolves
// (plan list, op launch, generic strided copy) plus two toy ops, all on host memory. It mirrors the calling
// conventions of csrc/kernels (create(kind?, descriptor) -> op, launch(op, stream)), nothing else.
#include <stdint.h>
#include <string.h>

#include <functional>
#include <string>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {
struct Op { std::function<int()> fn; };
struct Plan { std::vector<Op*> ops; };
std::string g_err;
struct GenericDesc { void* p[4]; long long i[48]; float f[4]; };
struct ScaleDesc { const float* x; float* y; long long n; float a; float b; };
struct TableSumDesc { const float* const* table; int count; float* out; long long n; };
}  // namespace

API const char* fdb_last_error() { return g_err.c_str(); }
API void* fdb_plan_create() { return new Plan(); }
API void fdb_plan_add(void* plan, void* op, int) { static_cast<Plan*>(plan)->ops.push_back(static_cast<Op*>(op)); }
API int fdb_plan_run(void* plan, void*) {
  for (Op* op : static_cast<Plan*>(plan)->ops) if (op->fn() != 0) return -1;
  return 0;
}
API void fdb_plan_destroy(void* plan) { delete static_cast<Plan*>(plan); }
API int fdb_op_launch(void* op, void*) { return static_cast<Op*>(op)->fn(); }
API void fdb_op_destroy(void* op) { delete static_cast<Op*>(op); }

// kind 0: strided copy of fp32 (dtype code 2) elements; i0 nd, i3.. shape, i9.. src strides, i15.. dst strides
API void* fdb_generic_create(int kind, const GenericDesc* dp) {
  if (kind != 0 || dp->i[1] != 2 || dp->i[2] != 2) { g_err = "fake generic op: fp32 strided copy only"; return nullptr; }
  const GenericDesc d = *dp;
  auto* op = new Op();
  op->fn = [d]() {
    const int nd = static_cast<int>(d.i[0]);
    long long total = 1;
    for (int k = 0; k < nd; ++k) total *= d.i[3 + k];
    const float* src = static_cast<const float*>(d.p[0]);
    float* dst = static_cast<float*>(d.p[1]);
    for (long long it = 0; it < total; ++it) {
      long long rem = it, so = 0, dof = 0;
      for (int k = nd - 1; k >= 0; --k) {
        const long long idx = rem % d.i[3 + k];
        rem /= d.i[3 + k];
        so += idx * d.i[9 + k];
        dof += idx * d.i[15 + k];
      }
      dst[dof] = src[so];
    }
    return 0;
  };
  return op;
}

// y = a * x + b over n floats
API void* fdb_fake_scale_create(const ScaleDesc* dp) {
  const ScaleDesc d = *dp;
  if (d.x == nullptr || d.y == nullptr) { g_err = "fake scale: null operand"; return nullptr; }
  auto* op = new Op();
  op->fn = [d]() { for (long long k = 0; k < d.n; ++k) d.y[k] = d.a * d.x[k] + d.b; return 0; };
  return op;
}

// out = sum of the `count` arrays whose addresses sit in a table in "device" memory (read at launch time)
API void* fdb_fake_table_sum_create(int kind, const TableSumDesc* dp) {
  const TableSumDesc d = *dp;
  if (kind != 7) { g_err = "fake table sum: kind must be 7"; return nullptr; }
  auto* op = new Op();
  op->fn = [d]() {
    for (long long k = 0; k < d.n; ++k) {
      float acc = 0.f;
      for (int t = 0; t < d.count; ++t) if (d.table[t] != nullptr) acc += d.table[t][k];
      d.out[k] = acc;
    }
    return 0;
  };
  return op;
}
