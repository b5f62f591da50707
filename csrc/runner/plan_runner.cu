// Replays a serialised launch plan (fastdeploy_b200/runtime/plan_file.py) without Python: allocates the plan's
// device buffers, uploads the constants, patches the device addresses into the op descriptors, re-creates every
// op through the kernel library's own fdb_*_create functions (resolved with dlsym) and launches the list, captured
// into one CUDA graph after the first run. Plain C ABI (fdplan_*), plus a command-line tool when compiled with
// -DFDPLAN_MAIN. The reference's counterpart is its C++ runtime loading a serialised engine
// (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:61-114).
#ifdef FDPLAN_HOST_ONLY
// Test build without a GPU: device memory is host memory, streams and graphs are immediate. It exists so that the
// file reader, the address relocation, the pointer tables and the input / output staging can be exercised against a
// stand-in kernel library on a machine that has no device (tests/test_plan_runner_host_cpu.py).
#include <stdlib.h>
#include <string.h>
typedef int cudaError_t;
typedef void* cudaStream_t;
typedef void* cudaGraph_t;
typedef void* cudaGraphExec_t;
typedef void* cudaEvent_t;
enum { cudaSuccess = 0, cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2, cudaStreamNonBlocking = 1,
       cudaStreamCaptureModeThreadLocal = 1 };
static cudaError_t cudaMalloc(void** p, size_t n) { *p = malloc(n ? n : 1); return *p ? 0 : 2; }
static cudaError_t cudaFree(void* p) { free(p); return 0; }
static cudaError_t cudaMemcpy(void* d, const void* s, size_t n, int) { memcpy(d, s, n); return 0; }
static cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, int, cudaStream_t) { memcpy(d, s, n); return 0; }
static cudaError_t cudaMemset(void* d, int v, size_t n) { memset(d, v, n); return 0; }
static cudaError_t cudaStreamCreateWithFlags(cudaStream_t* s, unsigned) { *s = nullptr; return 0; }
static cudaError_t cudaStreamDestroy(cudaStream_t) { return 0; }
static cudaError_t cudaStreamSynchronize(cudaStream_t) { return 0; }
static cudaError_t cudaDeviceSynchronize() { return 0; }
static cudaError_t cudaGetLastError() { return 0; }
static const char* cudaGetErrorString(cudaError_t) { return "host-only build"; }
// no capture on the host: the "graph" stays null and every run walks the launch list
static cudaError_t cudaStreamBeginCapture(cudaStream_t, int) { return 1; }
static cudaError_t cudaStreamEndCapture(cudaStream_t, cudaGraph_t* g) { *g = nullptr; return 1; }
static cudaError_t cudaGraphInstantiate(cudaGraphExec_t*, cudaGraph_t, unsigned long long) { return 1; }
static cudaError_t cudaGraphDestroy(cudaGraph_t) { return 0; }
static cudaError_t cudaGraphExecDestroy(cudaGraphExec_t) { return 0; }
static cudaError_t cudaGraphLaunch(cudaGraphExec_t, cudaStream_t) { return 1; }
static cudaError_t cudaEventCreate(cudaEvent_t*) { return 0; }
static cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t) { return 0; }
static cudaError_t cudaEventSynchronize(cudaEvent_t) { return 0; }
static cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t, cudaEvent_t) { *ms = 0.f; return 0; }
static cudaError_t cudaEventDestroy(cudaEvent_t) { return 0; }
#else
#include <cuda_runtime.h>
#endif
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#define FDPLAN_API extern "C" __attribute__((visibility("default")))

namespace {

#ifdef FDPLAN_HOST_ONLY
constexpr bool kHostOnly = true;
#else
constexpr bool kHostOnly = false;
#endif

thread_local std::string g_error;
void fail(const std::string& m) { g_error = m; }

// descriptor of the kernel library's generic ops (csrc/kernels/generic_ops.cu); kind 0 = strided copy
struct GenericDesc { void* p[4]; long long i[48]; float f[4]; };

int dtype_bytes(int dt) {
  switch (dt) {
    case 0: case 1: return 2;      // fp16, bf16
    case 2: case 4: return 4;      // fp32, int32
    case 5: return 8;              // int64
    default: return 1;             // uint8, e4m3, int8, bool
  }
}

struct IoTensor {
  std::string name;
  uint32_t buffer = 0;
  uint64_t offset = 0;
  int dtype = 0;
  std::vector<long long> dims, strides;
  void* staging = nullptr;         // contiguous device copy in dims order
  void* copy_op = nullptr;         // strided copy between staging and the plan's own tensor
  long long numel() const { long long n = 1; for (long long d : dims) n *= d; return n; }
  unsigned long long bytes() const { return static_cast<unsigned long long>(numel()) * dtype_bytes(dtype); }
};

struct Reader {
  FILE* f = nullptr;
  bool ok = true;
  bool read(void* dst, size_t n) { if (ok && fread(dst, 1, n, f) != n) ok = false; return ok; }
  template <typename T> T get() { T v{}; read(&v, sizeof(T)); return v; }
  std::string str() { uint16_t n = get<uint16_t>(); std::string s(n, '\0'); if (n) read(&s[0], n); return s; }
};

struct LoadedPlan {
  void* lib = nullptr;
  std::vector<void*> buffers;
  std::vector<uint64_t> sizes;
  std::vector<void*> ops;
  void* plan = nullptr;
  std::vector<IoTensor> inputs, outputs;
  cudaStream_t stream = nullptr;
  cudaGraphExec_t graph = nullptr;
  bool ran_once = false;
  // kernel library entry points
  void* (*plan_create)() = nullptr;
  void (*plan_add)(void*, void*, int) = nullptr;
  int (*plan_run)(void*, void*) = nullptr;
  void (*plan_destroy)(void*) = nullptr;
  int (*op_launch)(void*, void*) = nullptr;
  void (*op_destroy)(void*) = nullptr;
  const char* (*last_error)() = nullptr;
  void* (*generic_create)(int, const void*) = nullptr;

  ~LoadedPlan() {
    if (graph) cudaGraphExecDestroy(graph);
    if (plan && plan_destroy) plan_destroy(plan);
    for (void* op : ops) if (op && op_destroy) op_destroy(op);
    for (IoTensor& t : inputs) { if (t.copy_op) op_destroy(t.copy_op); if (t.staging) cudaFree(t.staging); }
    for (IoTensor& t : outputs) { if (t.copy_op) op_destroy(t.copy_op); if (t.staging) cudaFree(t.staging); }
    for (void* b : buffers) if (b) cudaFree(b);
    if (stream) cudaStreamDestroy(stream);
    if (lib) dlclose(lib);
  }
};

template <typename Fn> bool sym(void* lib, const char* name, Fn* out) {
  *out = reinterpret_cast<Fn>(dlsym(lib, name));
  if (*out == nullptr) { fail(std::string("kernel library has no symbol ") + name); return false; }
  return true;
}

bool make_io(LoadedPlan* p, IoTensor* t, bool is_output) {
  if (t->dims.size() > 6) { fail("plan input / output " + t->name + " has more than 6 dimensions"); return false; }
  if (cudaMalloc(&t->staging, t->bytes() ? t->bytes() : 1) != cudaSuccess) { fail("cudaMalloc of a staging buffer failed"); return false; }
  GenericDesc d;
  memset(&d, 0, sizeof(d));
  void* own = static_cast<char*>(p->buffers[t->buffer]) + t->offset;
  d.p[0] = is_output ? own : t->staging;
  d.p[1] = is_output ? t->staging : own;
  const int nd = static_cast<int>(t->dims.size());
  d.i[0] = nd; d.i[1] = t->dtype; d.i[2] = t->dtype;
  long long dense = 1;
  std::vector<long long> cont(nd);
  for (int k = nd - 1; k >= 0; --k) { cont[k] = dense; dense *= t->dims[k]; }
  for (int k = 0; k < nd; ++k) {
    d.i[3 + k] = t->dims[k];
    d.i[9 + k] = is_output ? t->strides[k] : cont[k];
    d.i[15 + k] = is_output ? cont[k] : t->strides[k];
  }
  t->copy_op = p->generic_create(0, &d);
  if (t->copy_op == nullptr) { fail("strided copy for " + t->name + ": " + p->last_error()); return false; }
  return true;
}

}  // namespace

FDPLAN_API const char* fdplan_last_error() { return g_error.c_str(); }

FDPLAN_API void fdplan_destroy(void* h) { delete static_cast<LoadedPlan*>(h); }

FDPLAN_API void* fdplan_load(const char* plan_path, const char* kernels_lib_path) {
  auto* p = new LoadedPlan();
  auto bail = [&](const std::string& m) -> void* { fail(m); delete p; return nullptr; };
  p->lib = dlopen(kernels_lib_path, RTLD_NOW | RTLD_LOCAL);
  if (p->lib == nullptr) return bail(std::string("cannot load the kernel library: ") + dlerror());
  if (!sym(p->lib, "fdb_plan_create", &p->plan_create) || !sym(p->lib, "fdb_plan_add", &p->plan_add) ||
      !sym(p->lib, "fdb_plan_run", &p->plan_run) || !sym(p->lib, "fdb_plan_destroy", &p->plan_destroy) ||
      !sym(p->lib, "fdb_op_launch", &p->op_launch) || !sym(p->lib, "fdb_op_destroy", &p->op_destroy) ||
      !sym(p->lib, "fdb_last_error", &p->last_error) || !sym(p->lib, "fdb_generic_create", &p->generic_create)) {
    delete p; return nullptr;
  }
  Reader r;
  r.f = fopen(plan_path, "rb");
  if (r.f == nullptr) return bail(std::string("cannot open ") + plan_path);
  struct Closer { FILE* f; ~Closer() { fclose(f); } } closer{r.f};
  char magic[8];
  if (!r.read(magic, 8) || memcmp(magic, "FDPLAN1\0", 8) != 0) return bail("not a plan file");
  if (cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) != cudaSuccess) return bail("cannot create a stream");
  // ---- buffers
  const uint32_t nbuf = r.get<uint32_t>();
  std::vector<uint8_t> host;
  for (uint32_t b = 0; r.ok && b < nbuf; ++b) {
    const uint64_t size = r.get<uint64_t>();
    const uint8_t has_data = r.get<uint8_t>();
    void* dev = nullptr;
    if (cudaMalloc(&dev, size ? size : 1) != cudaSuccess) return bail("cudaMalloc of a plan buffer failed (" + std::to_string(size) + " bytes)");
    p->buffers.push_back(dev);
    p->sizes.push_back(size);
    if (has_data) {
      const size_t chunk = 64u << 20;
      host.resize(size < chunk ? size : chunk);
      for (uint64_t off = 0; r.ok && off < size; off += chunk) {
        const size_t n = static_cast<size_t>(size - off < chunk ? size - off : chunk);
        if (!r.read(host.data(), n)) break;
        if (cudaMemcpy(static_cast<char*>(dev) + off, host.data(), n, cudaMemcpyHostToDevice) != cudaSuccess) return bail("upload of a constant failed");
      }
    } else if (cudaMemset(dev, 0, size) != cudaSuccess) {
      return bail("cudaMemset of a plan buffer failed");
    }
  }
  auto address = [&](uint32_t buffer, uint64_t offset, void** out) {
    if (buffer >= p->buffers.size() || offset >= (p->sizes[buffer] ? p->sizes[buffer] : 1)) return false;
    *out = static_cast<char*>(p->buffers[buffer]) + offset;
    return true;
  };
  // ---- pointer tables are patched before the ops that read them are created (creation may launch nothing, but
  // the order costs nothing); they are read after the ops section in the file, so keep the ops' records first
  struct OpRec { std::string fn; int kind; std::vector<uint8_t> desc; };
  std::vector<OpRec> recs;
  const uint32_t nops = r.get<uint32_t>();
  for (uint32_t k = 0; r.ok && k < nops; ++k) {
    OpRec rec;
    rec.fn = r.str();
    rec.kind = r.get<int32_t>();
    const uint32_t dsz = r.get<uint32_t>();
    if (!r.ok || dsz > (1u << 20)) return bail("corrupt plan file (descriptor size)");
    rec.desc.resize(dsz);
    r.read(rec.desc.data(), dsz);
    const uint32_t nrel = r.get<uint32_t>();
    for (uint32_t j = 0; r.ok && j < nrel; ++j) {
      const uint32_t off = r.get<uint32_t>();
      const uint32_t buf = r.get<uint32_t>();
      const uint64_t boff = r.get<uint64_t>();
      void* ptr = nullptr;
      if (!r.ok || off + sizeof(void*) > dsz || !address(buf, boff, &ptr)) return bail("corrupt plan file (relocation)");
      memcpy(rec.desc.data() + off, &ptr, sizeof(void*));
    }
    recs.push_back(std::move(rec));
  }
  const uint32_t ntab = r.get<uint32_t>();
  for (uint32_t k = 0; r.ok && k < ntab; ++k) {
    const uint32_t buf = r.get<uint32_t>();
    const uint64_t off = r.get<uint64_t>();
    const uint32_t count = r.get<uint32_t>();
    std::vector<void*> elems(count, nullptr);
    for (uint32_t j = 0; r.ok && j < count; ++j) {
      const int32_t eb = r.get<int32_t>();
      const uint64_t eo = r.get<uint64_t>();
      if (eb >= 0 && !address(static_cast<uint32_t>(eb), eo, &elems[j])) return bail("corrupt plan file (pointer table)");
    }
    void* dst = nullptr;
    if (!r.ok || !address(buf, off, &dst)) return bail("corrupt plan file (pointer table address)");
    if (cudaMemcpy(dst, elems.data(), count * sizeof(void*), cudaMemcpyHostToDevice) != cudaSuccess) return bail("upload of a pointer table failed");
  }
  const uint32_t nio = r.get<uint32_t>();
  for (uint32_t k = 0; r.ok && k < nio; ++k) {
    IoTensor t;
    const uint8_t is_out = r.get<uint8_t>();
    t.name = r.str();
    t.buffer = r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    t.dtype = r.get<uint8_t>();
    const uint8_t nd = r.get<uint8_t>();
    t.dims.resize(nd); t.strides.resize(nd);
    for (int j = 0; j < nd; ++j) t.dims[j] = r.get<int64_t>();
    for (int j = 0; j < nd; ++j) t.strides[j] = r.get<int64_t>();
    void* ptr = nullptr;
    if (!r.ok || !address(t.buffer, t.offset, &ptr)) return bail("corrupt plan file (input / output)");
    (is_out ? p->outputs : p->inputs).push_back(t);
  }
  if (!r.ok) return bail("plan file is truncated");
  // ---- ops
  p->plan = p->plan_create();
  for (OpRec& rec : recs) {
    void* fn = dlsym(p->lib, rec.fn.c_str());
    if (fn == nullptr) return bail("kernel library has no creation function " + rec.fn);
    void* op = rec.kind >= 0 ? reinterpret_cast<void* (*)(int, const void*)>(fn)(rec.kind, rec.desc.data())
                             : reinterpret_cast<void* (*)(const void*)>(fn)(rec.desc.data());
    if (op == nullptr) return bail(rec.fn + " failed: " + p->last_error());
    p->ops.push_back(op);
    p->plan_add(p->plan, op, 0);
  }
  for (IoTensor& t : p->inputs) if (!make_io(p, &t, false)) { delete p; return nullptr; }
  for (IoTensor& t : p->outputs) if (!make_io(p, &t, true)) { delete p; return nullptr; }
  if (cudaDeviceSynchronize() != cudaSuccess) return bail("device error while loading the plan");
  return p;
}

FDPLAN_API int fdplan_num_ops(void* h) { return static_cast<int>(static_cast<LoadedPlan*>(h)->ops.size()); }
FDPLAN_API int fdplan_num_inputs(void* h) { return static_cast<int>(static_cast<LoadedPlan*>(h)->inputs.size()); }
FDPLAN_API int fdplan_num_outputs(void* h) { return static_cast<int>(static_cast<LoadedPlan*>(h)->outputs.size()); }

static IoTensor* io_of(void* h, int is_output, int idx) {
  auto* p = static_cast<LoadedPlan*>(h);
  std::vector<IoTensor>& v = is_output ? p->outputs : p->inputs;
  if (idx < 0 || idx >= static_cast<int>(v.size())) { fail("input / output index out of range"); return nullptr; }
  return &v[idx];
}

FDPLAN_API const char* fdplan_io_name(void* h, int is_output, int idx) {
  IoTensor* t = io_of(h, is_output, idx);
  return t ? t->name.c_str() : "";
}

// dims must have room for 8 entries; returns the number of dimensions, -1 on a bad index
FDPLAN_API int fdplan_io_desc(void* h, int is_output, int idx, int* dtype, long long* dims) {
  IoTensor* t = io_of(h, is_output, idx);
  if (t == nullptr) return -1;
  *dtype = t->dtype;
  for (size_t k = 0; k < t->dims.size(); ++k) dims[k] = t->dims[k];
  return static_cast<int>(t->dims.size());
}

FDPLAN_API unsigned long long fdplan_io_bytes(void* h, int is_output, int idx) {
  IoTensor* t = io_of(h, is_output, idx);
  return t ? t->bytes() : 0;
}

// host data in the tensor's own dimension order (channel-innermost for image inputs), densely packed
FDPLAN_API int fdplan_set_input(void* h, int idx, const void* host, unsigned long long bytes) {
  auto* p = static_cast<LoadedPlan*>(h);
  IoTensor* t = io_of(h, 0, idx);
  if (t == nullptr) return -1;
  if (bytes != t->bytes()) { fail("input " + t->name + " takes " + std::to_string(t->bytes()) + " bytes"); return -1; }
  if (cudaMemcpyAsync(t->staging, host, bytes, cudaMemcpyHostToDevice, p->stream) != cudaSuccess) { fail("input copy failed"); return -1; }
  if (p->op_launch(t->copy_op, p->stream) != 0) { fail(p->last_error()); return -1; }
  return 0;
}

// Launches the plan (eagerly the first time, as one CUDA graph from then on) and waits for it.
FDPLAN_API int fdplan_run(void* h) {
  auto* p = static_cast<LoadedPlan*>(h);
  if (p->graph != nullptr) {
    if (cudaGraphLaunch(p->graph, p->stream) != cudaSuccess) { fail("graph launch failed"); return -1; }
  } else if (!p->ran_once || kHostOnly) {
    if (p->plan_run(p->plan, p->stream) != 0) { fail(p->last_error()); return -1; }
    p->ran_once = true;
  } else {
    cudaGraph_t g = nullptr;
    if (cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { fail("cannot begin capture"); return -1; }
    const int rc = p->plan_run(p->plan, p->stream);
    const cudaError_t e = cudaStreamEndCapture(p->stream, &g);
    if (rc != 0 || e != cudaSuccess || g == nullptr) { fail(rc != 0 ? p->last_error() : "capture failed"); if (g) cudaGraphDestroy(g); return -1; }
    const cudaError_t ie = cudaGraphInstantiate(&p->graph, g, 0);
    cudaGraphDestroy(g);
    if (ie != cudaSuccess) { p->graph = nullptr; fail("graph instantiation failed"); return -1; }
    if (cudaGraphLaunch(p->graph, p->stream) != cudaSuccess) { fail("graph launch failed"); return -1; }
  }
  if (cudaStreamSynchronize(p->stream) != cudaSuccess) { fail(std::string("plan run: ") + cudaGetErrorString(cudaGetLastError())); return -1; }
  return 0;
}

FDPLAN_API int fdplan_get_output(void* h, int idx, void* host, unsigned long long bytes) {
  auto* p = static_cast<LoadedPlan*>(h);
  IoTensor* t = io_of(h, 1, idx);
  if (t == nullptr) return -1;
  if (bytes != t->bytes()) { fail("output " + t->name + " holds " + std::to_string(t->bytes()) + " bytes"); return -1; }
  if (p->op_launch(t->copy_op, p->stream) != 0) { fail(p->last_error()); return -1; }
  if (cudaMemcpyAsync(host, t->staging, bytes, cudaMemcpyDeviceToHost, p->stream) != cudaSuccess ||
      cudaStreamSynchronize(p->stream) != cudaSuccess) { fail("output copy failed"); return -1; }
  return 0;
}

// Milliseconds per run over `iters` graph launches (CUDA events on the plan's stream), -1 on error.
FDPLAN_API double fdplan_time(void* h, int iters) {
  auto* p = static_cast<LoadedPlan*>(h);
  for (int k = 0; k < 3; ++k) if (fdplan_run(h) != 0) return -1.0;       // eager, capture, first replay
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0, p->stream);
  for (int k = 0; k < iters; ++k) {
    if (p->graph != nullptr) cudaGraphLaunch(p->graph, p->stream);
    else if (p->plan_run(p->plan, p->stream) != 0) break;
  }
  cudaEventRecord(e1, p->stream);
  float ms = -1.f;
  if (cudaEventSynchronize(e1) == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  return iters > 0 && ms >= 0.f ? ms / iters : -1.0;
}

#ifdef FDPLAN_MAIN
// fdplan_run <plan> <kernel library> [--in <index> <file>]... [--out <index> <file>]... [--iters N]
int main(int argc, char** argv) {
  if (argc < 3) { fprintf(stderr, "usage: %s <plan file> <libfdb200_kernels.so> [--in i file] [--out i file] [--iters n]\n", argv[0]); return 2; }
  void* h = fdplan_load(argv[1], argv[2]);
  if (h == nullptr) { fprintf(stderr, "load failed: %s\n", fdplan_last_error()); return 1; }
  printf("plan: %d ops, %d inputs, %d outputs\n", fdplan_num_ops(h), fdplan_num_inputs(h), fdplan_num_outputs(h));
  int iters = 0;
  std::vector<std::pair<int, std::string>> outs;
  for (int a = 3; a < argc; ++a) {
    const std::string flag = argv[a];
    if (flag == "--iters" && a + 1 < argc) { iters = atoi(argv[++a]); continue; }
    if ((flag == "--in" || flag == "--out") && a + 2 < argc) {
      const int idx = atoi(argv[a + 1]);
      const std::string path = argv[a + 2];
      a += 2;
      if (flag == "--out") { outs.push_back({idx, path}); continue; }
      const unsigned long long n = fdplan_io_bytes(h, 0, idx);
      std::vector<char> buf(n);
      FILE* f = fopen(path.c_str(), "rb");
      if (f == nullptr || fread(buf.data(), 1, n, f) != n) { fprintf(stderr, "cannot read %llu bytes from %s\n", n, path.c_str()); return 1; }
      fclose(f);
      if (fdplan_set_input(h, idx, buf.data(), n) != 0) { fprintf(stderr, "%s\n", fdplan_last_error()); return 1; }
      continue;
    }
    fprintf(stderr, "unknown argument %s\n", argv[a]); return 2;
  }
  if (fdplan_run(h) != 0) { fprintf(stderr, "run failed: %s\n", fdplan_last_error()); return 1; }
  if (iters > 0) printf("ms_per_run %.4f\n", fdplan_time(h, iters));
  for (auto& o : outs) {
    const unsigned long long n = fdplan_io_bytes(h, 1, o.first);
    std::vector<char> buf(n);
    if (fdplan_get_output(h, o.first, buf.data(), n) != 0) { fprintf(stderr, "%s\n", fdplan_last_error()); return 1; }
    FILE* f = fopen(o.second.c_str(), "wb");
    if (f == nullptr || fwrite(buf.data(), 1, n, f) != n) { fprintf(stderr, "cannot write %s\n", o.second.c_str()); return 1; }
    fclose(f);
    printf("output %d (%s): %llu bytes -> %s\n", o.first, fdplan_io_name(h, 1, o.first), n, o.second.c_str());
  }
  fdplan_destroy(h);
  return 0;
}
#endif
