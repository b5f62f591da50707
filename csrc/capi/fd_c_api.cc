// C API over an embedded interpreter (see fd_c_api.h). Every entry point takes the GIL, forwards to the
// Python package and converts results into malloc'ed C arrays. Errors never cross the boundary as
// exceptions: calls return NULL / false and FD_C_GetLastError() holds the text.
#include "fd_c_api.h"

#include <Python.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace {

thread_local std::string g_err;
std::once_flag g_init;
PyObject* g_pkg = nullptr;      // fastdeploy_b200
PyObject* g_np = nullptr;       // numpy
bool g_owns_interpreter = false;

void set_err(const std::string& s) { g_err = s; }

void fetch_py_error(const char* what) {
  PyObject *t = nullptr, *v = nullptr, *tb = nullptr;
  PyErr_Fetch(&t, &v, &tb);
  PyErr_NormalizeException(&t, &v, &tb);
  std::string msg = what;
  if (v != nullptr) {
    PyObject* s = PyObject_Str(v);
    if (s != nullptr) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c != nullptr) msg += std::string(": ") + c;
      Py_DECREF(s);
    }
  }
  Py_XDECREF(t); Py_XDECREF(v); Py_XDECREF(tb);
  set_err(msg);
}

void ensure_python() {
  std::call_once(g_init, [] {
    if (!Py_IsInitialized()) {
      Py_InitializeEx(0);
      g_owns_interpreter = true;
      PyEval_SaveThread();      // release the GIL acquired by initialisation; every call re-takes it
    }
    PyGILState_STATE st = PyGILState_Ensure();
    g_pkg = PyImport_ImportModule("fastdeploy_b200");
    if (g_pkg == nullptr) fetch_py_error("import fastdeploy_b200");
    g_np = PyImport_ImportModule("numpy");
    if (g_np == nullptr) fetch_py_error("import numpy");
    PyGILState_Release(st);
  });
}

struct Gil {
  PyGILState_STATE st;
  Gil() { ensure_python(); st = PyGILState_Ensure(); }
  ~Gil() { PyGILState_Release(st); }
};

PyObject* call_method(PyObject* obj, const char* name, const char* fmt = nullptr, ...) {
  PyObject* m = PyObject_GetAttrString(obj, name);
  if (m == nullptr) { fetch_py_error(name); return nullptr; }
  PyObject* args = nullptr;
  if (fmt != nullptr) {
    va_list va;
    va_start(va, fmt);
    args = Py_VaBuildValue(fmt, va);
    va_end(va);
    if (args != nullptr && !PyTuple_Check(args)) {
      PyObject* t = PyTuple_Pack(1, args);
      Py_DECREF(args);
      args = t;
    }
  } else {
    args = PyTuple_New(0);
  }
  PyObject* r = args != nullptr ? PyObject_CallObject(m, args) : nullptr;
  Py_XDECREF(args);
  Py_DECREF(m);
  if (r == nullptr) fetch_py_error(name);
  return r;
}

// numpy array viewing (copying) a C buffer
PyObject* np_from_buffer(const void* data, size_t nbytes, const char* dtype, const int64_t* shape, size_t ndim) {
  PyObject* bytes = PyBytes_FromStringAndSize(static_cast<const char*>(data), static_cast<Py_ssize_t>(nbytes));
  PyObject* arr = PyObject_CallMethod(g_np, "frombuffer", "Os", bytes, dtype);
  Py_DECREF(bytes);
  if (arr == nullptr) { fetch_py_error("numpy.frombuffer"); return nullptr; }
  PyObject* shp = PyTuple_New(static_cast<Py_ssize_t>(ndim));
  for (size_t i = 0; i < ndim; ++i) PyTuple_SET_ITEM(shp, i, PyLong_FromLongLong(shape[i]));
  PyObject* out = PyObject_CallMethod(arr, "reshape", "O", shp);
  Py_DECREF(shp);
  Py_DECREF(arr);
  if (out == nullptr) fetch_py_error("reshape");
  return out;
}

PyObject* mat_to_numpy(const FD_C_Mat& m) {
  const int64_t shape[3] = {m.height, m.width, m.channels};
  return np_from_buffer(m.data, static_cast<size_t>(m.height) * m.width * m.channels, "uint8", shape, 3);
}

bool floats_from_seq(PyObject* seq, FD_C_OneDimArrayFloat* out) {
  PyObject* fast = PySequence_Fast(seq, "sequence expected");
  if (fast == nullptr) { fetch_py_error("result"); return false; }
  const Py_ssize_t n = PySequence_Fast_GET_SIZE(fast);
  out->size = static_cast<size_t>(n);
  out->data = static_cast<float*>(std::malloc(sizeof(float) * (n > 0 ? n : 1)));
  for (Py_ssize_t i = 0; i < n; ++i) out->data[i] = static_cast<float>(PyFloat_AsDouble(PySequence_Fast_GET_ITEM(fast, i)));
  Py_DECREF(fast);
  return true;
}
bool ints_from_seq(PyObject* seq, FD_C_OneDimArrayInt32* out) {
  PyObject* fast = PySequence_Fast(seq, "sequence expected");
  if (fast == nullptr) { fetch_py_error("result"); return false; }
  const Py_ssize_t n = PySequence_Fast_GET_SIZE(fast);
  out->size = static_cast<size_t>(n);
  out->data = static_cast<int32_t*>(std::malloc(sizeof(int32_t) * (n > 0 ? n : 1)));
  for (Py_ssize_t i = 0; i < n; ++i) out->data[i] = static_cast<int32_t>(PyLong_AsLong(PySequence_Fast_GET_ITEM(fast, i)));
  Py_DECREF(fast);
  return true;
}

PyObject* get_class(const char* dotted) {      // e.g. "vision.detection.PPYOLOE"
  PyObject* cur = g_pkg;
  Py_XINCREF(cur);
  std::string path = dotted;
  size_t pos = 0;
  while (cur != nullptr && pos <= path.size()) {
    const size_t dot = path.find('.', pos);
    const std::string part = path.substr(pos, dot == std::string::npos ? std::string::npos : dot - pos);
    PyObject* nxt = PyObject_GetAttrString(cur, part.c_str());
    Py_DECREF(cur);
    cur = nxt;
    if (dot == std::string::npos) break;
    pos = dot + 1;
  }
  if (cur == nullptr) fetch_py_error(dotted);
  return cur;
}

}  // namespace

struct FD_C_RuntimeOptionWrapper { PyObject* obj; };
struct FD_C_RuntimeWrapper { PyObject* obj; };
struct FD_C_ModelWrapper { PyObject* obj; };

extern "C" {

const char* FD_C_GetLastError(void) { return g_err.c_str(); }

FD_C_RuntimeOptionWrapper* FD_C_CreateRuntimeOptionWrapper(void) {
  Gil g;
  if (g_pkg == nullptr) return nullptr;
  PyObject* o = PyObject_CallMethod(g_pkg, "RuntimeOption", nullptr);
  if (o == nullptr) { fetch_py_error("RuntimeOption"); return nullptr; }
  return new FD_C_RuntimeOptionWrapper{o};
}
void FD_C_DestroyRuntimeOptionWrapper(FD_C_RuntimeOptionWrapper* w) {
  if (w == nullptr) return;
  Gil g;
  Py_XDECREF(w->obj);
  delete w;
}
#define FD_OPT_CALL0(cname, pyname)                                    \
  void cname(FD_C_RuntimeOptionWrapper* w) {                           \
    Gil g;                                                             \
    PyObject* r = call_method(w->obj, pyname);                         \
    Py_XDECREF(r);                                                     \
  }
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseCpu, "use_cpu")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUsePaddleBackend, "use_paddle_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUsePaddleInferBackend, "use_paddle_infer_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseOrtBackend, "use_ort_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseTrtBackend, "use_trt_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseOpenVINOBackend, "use_openvino_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnableTrtFP16, "enable_trt_fp16")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperDisableTrtFP16, "disable_trt_fp16")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnablePinnedMemory, "enable_pinned_memory")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperDisablePinnedMemory, "disable_pinned_memory")

void FD_C_RuntimeOptionWrapperSetModelPath(FD_C_RuntimeOptionWrapper* w, const char* model_path, const char* params_path,
                                           FD_C_ModelFormat format) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_model_path", "(ssi)", model_path, params_path ? params_path : "", static_cast<int>(format));
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperUseGpu(FD_C_RuntimeOptionWrapper* w, int gpu_id) {
  Gil g;
  PyObject* r = call_method(w->obj, "use_gpu", "(i)", gpu_id);
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperSetCpuThreadNum(FD_C_RuntimeOptionWrapper* w, int n) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_cpu_thread_num", "(i)", n);
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperSetTrtCacheFile(FD_C_RuntimeOptionWrapper* w, const char* path) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_trt_cache_file", "(s)", path);
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperSetEncryptionKey(FD_C_RuntimeOptionWrapper* w, const char* key) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_encryption_key", "(s)", key);
  Py_XDECREF(r);
}

// ---------------------------------------------------------------- runtime
FD_C_RuntimeWrapper* FD_C_CreateRuntimeWrapper(FD_C_RuntimeOptionWrapper* option) {
  Gil g;
  if (g_pkg == nullptr || option == nullptr) return nullptr;
  PyObject* o = PyObject_CallMethod(g_pkg, "Runtime", "O", option->obj);
  if (o == nullptr) { fetch_py_error("Runtime"); return nullptr; }
  return new FD_C_RuntimeWrapper{o};
}
void FD_C_DestroyRuntimeWrapper(FD_C_RuntimeWrapper* w) {
  if (w == nullptr) return;
  Gil g;
  Py_XDECREF(w->obj);
  delete w;
}
static int int_call(PyObject* o, const char* name) {
  PyObject* r = call_method(o, name);
  if (r == nullptr) return -1;
  const int v = static_cast<int>(PyLong_AsLong(r));
  Py_DECREF(r);
  return v;
}
int FD_C_RuntimeWrapperNumInputs(FD_C_RuntimeWrapper* w) { Gil g; return int_call(w->obj, "num_inputs"); }
int FD_C_RuntimeWrapperNumOutputs(FD_C_RuntimeWrapper* w) { Gil g; return int_call(w->obj, "num_outputs"); }

FD_C_Bool FD_C_RuntimeWrapperInfer(FD_C_RuntimeWrapper* w, const FD_C_Tensor* inputs, int n_inputs, FD_C_Tensor* outputs,
                                   int max_outputs, int* n_outputs) {
  Gil g;
  static const char* kDtypes[] = {"float32", "int64", "int32", "uint8"};
  PyObject* feeds = PyDict_New();
  for (int i = 0; i < n_inputs; ++i) {
    const FD_C_Tensor& t = inputs[i];
    if (t.dtype < 0 || t.dtype > 3) { set_err("unsupported tensor dtype"); Py_DECREF(feeds); return 0; }
    PyObject* arr = np_from_buffer(t.data, t.nbytes, kDtypes[t.dtype], t.shape.data, t.shape.size);
    if (arr == nullptr) { Py_DECREF(feeds); return 0; }
    PyDict_SetItemString(feeds, t.name, arr);
    Py_DECREF(arr);
  }
  PyObject* outs = call_method(w->obj, "infer", "(O)", feeds);
  Py_DECREF(feeds);
  if (outs == nullptr) return 0;
  const Py_ssize_t n = PySequence_Size(outs);
  *n_outputs = static_cast<int>(n);
  for (Py_ssize_t i = 0; i < n && i < max_outputs; ++i) {
    PyObject* o = PySequence_GetItem(outs, i);
    PyObject* c = PyObject_CallMethod(g_np, "ascontiguousarray", "Os", o, "float32");
    Py_DECREF(o);
    if (c == nullptr) { fetch_py_error("ascontiguousarray"); Py_DECREF(outs); return 0; }
    PyObject* shp = PyObject_GetAttrString(c, "shape");
    const Py_ssize_t nd = PyTuple_Size(shp);
    FD_C_Tensor& t = outputs[i];
    t.name = nullptr;
    t.dtype = 0;
    t.shape.size = static_cast<size_t>(nd);
    t.shape.data = static_cast<int64_t*>(std::malloc(sizeof(int64_t) * (nd > 0 ? nd : 1)));
    for (Py_ssize_t k = 0; k < nd; ++k) t.shape.data[k] = PyLong_AsLongLong(PyTuple_GET_ITEM(shp, k));
    Py_DECREF(shp);
    PyObject* b = PyObject_CallMethod(c, "tobytes", nullptr);
    Py_DECREF(c);
    char* buf = nullptr;
    Py_ssize_t len = 0;
    PyBytes_AsStringAndSize(b, &buf, &len);
    t.nbytes = static_cast<size_t>(len);
    t.data = std::malloc(len > 0 ? len : 1);
    std::memcpy(t.data, buf, len);
    Py_DECREF(b);
  }
  Py_DECREF(outs);
  return 1;
}
void FD_C_DestroyTensors(FD_C_Tensor* tensors, int n) {
  for (int i = 0; i < n; ++i) {
    std::free(tensors[i].data);
    std::free(tensors[i].shape.data);
    tensors[i].data = nullptr;
    tensors[i].shape.data = nullptr;
  }
}

// ---------------------------------------------------------------- models
static FD_C_ModelWrapper* create_model(const char* dotted, const char* model_file, const char* params_file, const char* config_file,
                                       FD_C_RuntimeOptionWrapper* option, FD_C_ModelFormat format) {
  Gil g;
  if (g_pkg == nullptr) return nullptr;
  PyObject* cls = get_class(dotted);
  if (cls == nullptr) return nullptr;
  PyObject* kwargs = PyDict_New();
  if (option != nullptr) PyDict_SetItemString(kwargs, "runtime_option", option->obj);
  PyObject* fmt = PyLong_FromLong(static_cast<long>(format));
  PyDict_SetItemString(kwargs, "model_format", fmt);
  Py_DECREF(fmt);
  PyObject* args = config_file != nullptr && config_file[0] != 0
                       ? Py_BuildValue("(sss)", model_file, params_file ? params_file : "", config_file)
                       : Py_BuildValue("(ss)", model_file, params_file ? params_file : "");
  PyObject* o = PyObject_Call(cls, args, kwargs);
  Py_DECREF(args); Py_DECREF(kwargs); Py_DECREF(cls);
  if (o == nullptr) { fetch_py_error(dotted); return nullptr; }
  return new FD_C_ModelWrapper{o};
}
void FD_C_DestroyModelWrapper(FD_C_ModelWrapper* w) {
  if (w == nullptr) return;
  Gil g;
  Py_XDECREF(w->obj);
  delete w;
}
static FD_C_Bool predict_detection(FD_C_ModelWrapper* w, FD_C_Mat img, FD_C_DetectionResult* out) {
  Gil g;
  PyObject* arr = mat_to_numpy(img);
  if (arr == nullptr) return 0;
  PyObject* r = call_method(w->obj, "predict", "(O)", arr);
  Py_DECREF(arr);
  if (r == nullptr) return 0;
  PyObject *boxes = PyObject_GetAttrString(r, "boxes"), *scores = PyObject_GetAttrString(r, "scores"),
           *labels = PyObject_GetAttrString(r, "label_ids");
  bool ok = boxes && scores && labels && floats_from_seq(scores, &out->scores) && ints_from_seq(labels, &out->label_ids);
  if (ok) {
    const Py_ssize_t n = PySequence_Size(boxes);
    out->boxes.size = static_cast<size_t>(n);
    out->boxes.data = static_cast<FD_C_OneDimArrayFloat*>(std::calloc(n > 0 ? n : 1, sizeof(FD_C_OneDimArrayFloat)));
    for (Py_ssize_t i = 0; i < n && ok; ++i) {
      PyObject* b = PySequence_GetItem(boxes, i);
      ok = floats_from_seq(b, &out->boxes.data[i]);
      Py_DECREF(b);
    }
  } else if (PyErr_Occurred()) {
    fetch_py_error("DetectionResult");
  }
  Py_XDECREF(boxes); Py_XDECREF(scores); Py_XDECREF(labels); Py_DECREF(r);
  return ok ? 1 : 0;
}

FD_C_PPYOLOEWrapper* FD_C_CreatePPYOLOEWrapper(const char* m, const char* p, const char* c, FD_C_RuntimeOptionWrapper* o,
                                               FD_C_ModelFormat f) {
  return create_model("vision.detection.PPYOLOE", m, p, c, o, f);
}
void FD_C_DestroyPPYOLOEWrapper(FD_C_PPYOLOEWrapper* w) { FD_C_DestroyModelWrapper(w); }
FD_C_Bool FD_C_PPYOLOEWrapperPredict(FD_C_PPYOLOEWrapper* w, FD_C_Mat img, FD_C_DetectionResult* r) { return predict_detection(w, img, r); }
FD_C_Bool FD_C_PPYOLOEWrapperInitialized(FD_C_PPYOLOEWrapper* w) {
  Gil g;
  PyObject* r = call_method(w->obj, "initialized");
  const FD_C_Bool v = r != nullptr && PyObject_IsTrue(r) ? 1 : 0;
  Py_XDECREF(r);
  return v;
}
FD_C_ModelWrapper* FD_C_CreateDetectionModelWrapper(const char* class_name, const char* m, const char* p, const char* c,
                                                    FD_C_RuntimeOptionWrapper* o, FD_C_ModelFormat f) {
  return create_model((std::string("vision.detection.") + class_name).c_str(), m, p, c, o, f);
}
FD_C_Bool FD_C_DetectionModelWrapperPredict(FD_C_ModelWrapper* w, FD_C_Mat img, FD_C_DetectionResult* r) {
  return predict_detection(w, img, r);
}

FD_C_PaddleClasModelWrapper* FD_C_CreatePaddleClasModelWrapper(const char* m, const char* p, const char* c,
                                                               FD_C_RuntimeOptionWrapper* o, FD_C_ModelFormat f) {
  return create_model("vision.classification.PaddleClasModel", m, p, c, o, f);
}
void FD_C_DestroyPaddleClasModelWrapper(FD_C_PaddleClasModelWrapper* w) { FD_C_DestroyModelWrapper(w); }
FD_C_Bool FD_C_PaddleClasModelWrapperPredict(FD_C_PaddleClasModelWrapper* w, FD_C_Mat img, FD_C_ClassifyResult* out) {
  Gil g;
  PyObject* arr = mat_to_numpy(img);
  if (arr == nullptr) return 0;
  PyObject* r = call_method(w->obj, "predict", "(O)", arr);
  Py_DECREF(arr);
  if (r == nullptr) return 0;
  PyObject *ids = PyObject_GetAttrString(r, "label_ids"), *scores = PyObject_GetAttrString(r, "scores");
  const bool ok = ids && scores && ints_from_seq(ids, &out->label_ids) && floats_from_seq(scores, &out->scores);
  Py_XDECREF(ids); Py_XDECREF(scores); Py_DECREF(r);
  return ok ? 1 : 0;
}

// ---------------------------------------------------------------- batch predict, segmentation, OCR, visualisation
static bool detection_from_py(PyObject* r, FD_C_DetectionResult* out) {
  PyObject *boxes = PyObject_GetAttrString(r, "boxes"), *scores = PyObject_GetAttrString(r, "scores"),
           *labels = PyObject_GetAttrString(r, "label_ids");
  bool ok = boxes && scores && labels && floats_from_seq(scores, &out->scores) && ints_from_seq(labels, &out->label_ids);
  if (ok) {
    const Py_ssize_t n = PySequence_Size(boxes);
    out->boxes.size = static_cast<size_t>(n);
    out->boxes.data = static_cast<FD_C_OneDimArrayFloat*>(std::calloc(n > 0 ? n : 1, sizeof(FD_C_OneDimArrayFloat)));
    for (Py_ssize_t i = 0; i < n && ok; ++i) {
      PyObject* b = PySequence_GetItem(boxes, i);
      ok = floats_from_seq(b, &out->boxes.data[i]);
      Py_DECREF(b);
    }
  } else if (PyErr_Occurred()) {
    fetch_py_error("DetectionResult");
  }
  Py_XDECREF(boxes); Py_XDECREF(scores); Py_XDECREF(labels);
  return ok;
}

FD_C_Bool FD_C_DetectionModelWrapperBatchPredict(FD_C_ModelWrapper* w, const FD_C_Mat* imgs, int n_imgs,
                                                 FD_C_DetectionResult* results) {
  Gil g;
  PyObject* list = PyList_New(n_imgs);
  for (int i = 0; i < n_imgs; ++i) {
    PyObject* arr = mat_to_numpy(imgs[i]);
    if (arr == nullptr) { Py_DECREF(list); return 0; }
    PyList_SET_ITEM(list, i, arr);
  }
  PyObject* r = call_method(w->obj, "batch_predict", "(O)", list);
  Py_DECREF(list);
  if (r == nullptr) return 0;
  bool ok = PySequence_Check(r) && PySequence_Size(r) == n_imgs;
  for (int i = 0; i < n_imgs && ok; ++i) {
    PyObject* item = PySequence_GetItem(r, i);
    ok = item != nullptr && detection_from_py(item, &results[i]);
    Py_XDECREF(item);
  }
  if (!ok && g_err.empty()) set_err("batch_predict: unexpected result");
  Py_DECREF(r);
  return ok ? 1 : 0;
}

FD_C_PaddleSegModelWrapper* FD_C_CreatePaddleSegModelWrapper(const char* m, const char* p, const char* c,
                                                             FD_C_RuntimeOptionWrapper* o, FD_C_ModelFormat f) {
  return create_model("vision.segmentation.PaddleSegModel", m, p, c, o, f);
}
static bool seg_from_py(PyObject* r, FD_C_SegmentationResult* out) {
  std::memset(out, 0, sizeof(*out));
  PyObject *lm = PyObject_GetAttrString(r, "label_map"), *sm = PyObject_GetAttrString(r, "score_map"),
           *shape = PyObject_GetAttrString(r, "shape"), *has = PyObject_GetAttrString(r, "contain_score_map");
  bool ok = lm && sm && shape && ints_from_seq(lm, &out->label_map) && floats_from_seq(sm, &out->score_map) &&
            PySequence_Check(shape) && PySequence_Size(shape) >= 2;
  if (ok) {
    PyObject *h = PySequence_GetItem(shape, 0), *wd = PySequence_GetItem(shape, 1);
    out->height = static_cast<int>(PyLong_AsLong(h));
    out->width = static_cast<int>(PyLong_AsLong(wd));
    Py_XDECREF(h); Py_XDECREF(wd);
    out->contain_score_map = has != nullptr && PyObject_IsTrue(has) ? 1 : 0;
  } else if (PyErr_Occurred()) {
    fetch_py_error("SegmentationResult");
  }
  Py_XDECREF(lm); Py_XDECREF(sm); Py_XDECREF(shape); Py_XDECREF(has);
  return ok;
}
FD_C_Bool FD_C_PaddleSegModelWrapperPredict(FD_C_PaddleSegModelWrapper* w, FD_C_Mat img, FD_C_SegmentationResult* out) {
  Gil g;
  PyObject* arr = mat_to_numpy(img);
  if (arr == nullptr) return 0;
  PyObject* r = call_method(w->obj, "predict", "(O)", arr);
  Py_DECREF(arr);
  if (r == nullptr) return 0;
  const bool ok = seg_from_py(r, out);
  Py_DECREF(r);
  return ok ? 1 : 0;
}
void FD_C_DestroySegmentationResult(FD_C_SegmentationResult* r) {
  if (r == nullptr) return;
  std::free(r->label_map.data); std::free(r->score_map.data);
  r->label_map.data = nullptr; r->score_map.data = nullptr;
}

static FD_C_ModelWrapper* create_ocr_pipeline(const char* pipeline, const char* det_m, const char* det_p, const char* cls_m,
                                              const char* cls_p, const char* rec_m, const char* rec_p, const char* rec_label,
                                              FD_C_RuntimeOptionWrapper* option) {
  Gil g;
  if (g_pkg == nullptr) return nullptr;
  auto make = [&](const char* dotted, PyObject* args) -> PyObject* {
    PyObject* cls = get_class(dotted);
    if (cls == nullptr) { Py_DECREF(args); return nullptr; }
    PyObject* kwargs = PyDict_New();
    if (option != nullptr) PyDict_SetItemString(kwargs, "runtime_option", option->obj);
    PyObject* o = PyObject_Call(cls, args, kwargs);
    Py_DECREF(args); Py_DECREF(kwargs); Py_DECREF(cls);
    if (o == nullptr) fetch_py_error(dotted);
    return o;
  };
  PyObject* det = make("vision.ocr.DBDetector", Py_BuildValue("(ss)", det_m, det_p ? det_p : ""));
  if (det == nullptr) return nullptr;
  PyObject* cls = nullptr;
  if (cls_m != nullptr && cls_m[0] != 0) {
    cls = make("vision.ocr.Classifier", Py_BuildValue("(ss)", cls_m, cls_p ? cls_p : ""));
    if (cls == nullptr) { Py_DECREF(det); return nullptr; }
  }
  PyObject* rec = make("vision.ocr.Recognizer", Py_BuildValue("(sss)", rec_m, rec_p ? rec_p : "", rec_label ? rec_label : ""));
  if (rec == nullptr) { Py_DECREF(det); Py_XDECREF(cls); return nullptr; }
  PyObject* pipe_cls = get_class(pipeline);
  PyObject* pipe = pipe_cls != nullptr ? PyObject_CallFunctionObjArgs(pipe_cls, det, cls != nullptr ? cls : Py_None, rec, nullptr)
                                       : nullptr;
  Py_XDECREF(pipe_cls); Py_DECREF(det); Py_XDECREF(cls); Py_DECREF(rec);
  if (pipe == nullptr) { fetch_py_error(pipeline); return nullptr; }
  return new FD_C_ModelWrapper{pipe};
}
FD_C_PPOCRv3Wrapper* FD_C_CreatePPOCRv3Wrapper(const char* det_m, const char* det_p, const char* cls_m, const char* cls_p,
                                               const char* rec_m, const char* rec_p, const char* rec_label,
                                               FD_C_RuntimeOptionWrapper* option) {
  return create_ocr_pipeline("vision.ocr.PPOCRv3", det_m, det_p, cls_m, cls_p, rec_m, rec_p, rec_label, option);
}
FD_C_PPOCRv2Wrapper* FD_C_CreatePPOCRv2Wrapper(const char* det_m, const char* det_p, const char* cls_m, const char* cls_p,
                                               const char* rec_m, const char* rec_p, const char* rec_label,
                                               FD_C_RuntimeOptionWrapper* option) {
  return create_ocr_pipeline("vision.ocr.PPOCRv2", det_m, det_p, cls_m, cls_p, rec_m, rec_p, rec_label, option);
}
static bool ocr_from_py(PyObject* r, FD_C_OCRResult* out) {
  std::memset(out, 0, sizeof(*out));
  PyObject *boxes = PyObject_GetAttrString(r, "boxes"), *text = PyObject_GetAttrString(r, "text"),
           *rs = PyObject_GetAttrString(r, "rec_scores"), *cs = PyObject_GetAttrString(r, "cls_scores"),
           *cl = PyObject_GetAttrString(r, "cls_labels");
  bool ok = boxes && text && rs && cs && cl && floats_from_seq(rs, &out->rec_scores) && floats_from_seq(cs, &out->cls_scores) &&
            ints_from_seq(cl, &out->cls_labels);
  if (ok) {
    const Py_ssize_t n = PySequence_Size(boxes);
    out->boxes.size = static_cast<size_t>(n);
    out->boxes.data = static_cast<FD_C_OneDimArrayFloat*>(std::calloc(n > 0 ? n : 1, sizeof(FD_C_OneDimArrayFloat)));
    for (Py_ssize_t i = 0; i < n && ok; ++i) {
      PyObject* b = PySequence_GetItem(boxes, i);
      ok = floats_from_seq(b, &out->boxes.data[i]);
      Py_DECREF(b);
    }
    const Py_ssize_t nt = PySequence_Size(text);
    out->n_text = static_cast<size_t>(nt);
    out->text = static_cast<char**>(std::calloc(nt > 0 ? nt : 1, sizeof(char*)));
    for (Py_ssize_t i = 0; i < nt && ok; ++i) {
      PyObject* t = PySequence_GetItem(text, i);
      const char* c = t != nullptr ? PyUnicode_AsUTF8(t) : nullptr;
      out->text[i] = strdup(c != nullptr ? c : "");
      Py_XDECREF(t);
    }
  } else if (PyErr_Occurred()) {
    fetch_py_error("OCRResult");
  }
  Py_XDECREF(boxes); Py_XDECREF(text); Py_XDECREF(rs); Py_XDECREF(cs); Py_XDECREF(cl);
  return ok;
}
FD_C_Bool FD_C_PPOCRv3WrapperPredict(FD_C_PPOCRv3Wrapper* w, FD_C_Mat img, FD_C_OCRResult* out) {
  Gil g;
  std::memset(out, 0, sizeof(*out));
  PyObject* arr = mat_to_numpy(img);
  if (arr == nullptr) return 0;
  PyObject* r = call_method(w->obj, "predict", "(O)", arr);
  Py_DECREF(arr);
  if (r == nullptr) return 0;
  const bool ok = ocr_from_py(r, out);
  Py_DECREF(r);
  return ok ? 1 : 0;
}
void FD_C_DestroyOCRResult(FD_C_OCRResult* r) {
  if (r == nullptr) return;
  for (size_t i = 0; i < r->boxes.size; ++i) std::free(r->boxes.data[i].data);
  std::free(r->boxes.data);
  for (size_t i = 0; i < r->n_text; ++i) std::free(r->text[i]);
  std::free(r->text);
  std::free(r->rec_scores.data); std::free(r->cls_scores.data); std::free(r->cls_labels.data);
  std::memset(r, 0, sizeof(*r));
}

static bool copy_image_back(PyObject* arr, FD_C_Mat* out) {
  PyObject* bytes = call_method(arr, "tobytes");
  if (bytes == nullptr) return false;
  char* buf = nullptr;
  Py_ssize_t n = 0;
  const bool ok = PyBytes_AsStringAndSize(bytes, &buf, &n) == 0 &&
                  n == static_cast<Py_ssize_t>(out->height) * out->width * out->channels;
  if (ok) std::memcpy(out->data, buf, static_cast<size_t>(n));
  else set_err("visualisation: the result image does not fit the output buffer");
  Py_DECREF(bytes);
  return ok;
}

static PyObject* py_list_of_floats(const float* v, size_t n) {
  PyObject* l = PyList_New(static_cast<Py_ssize_t>(n));
  for (size_t i = 0; i < n; ++i) PyList_SET_ITEM(l, i, PyFloat_FromDouble(v[i]));
  return l;
}

FD_C_Bool FD_C_VisDetection(FD_C_Mat img, const FD_C_DetectionResult* result, float score_threshold, int line_size,
                            float font_size, FD_C_Mat* out) {
  Gil g;
  PyObject* res_cls = get_class("vision.DetectionResult");
  PyObject* vis = get_class("vision.vis_detection");
  if (res_cls == nullptr || vis == nullptr) { Py_XDECREF(res_cls); Py_XDECREF(vis); return 0; }
  PyObject* res = PyObject_CallObject(res_cls, nullptr);
  Py_DECREF(res_cls);
  if (res == nullptr) { fetch_py_error("DetectionResult"); Py_DECREF(vis); return 0; }
  PyObject* boxes = PyList_New(static_cast<Py_ssize_t>(result->boxes.size));
  for (size_t i = 0; i < result->boxes.size; ++i)
    PyList_SET_ITEM(boxes, i, py_list_of_floats(result->boxes.data[i].data, result->boxes.data[i].size));
  PyObject* scores = py_list_of_floats(result->scores.data, result->scores.size);
  PyObject* labels = PyList_New(static_cast<Py_ssize_t>(result->label_ids.size));
  for (size_t i = 0; i < result->label_ids.size; ++i) PyList_SET_ITEM(labels, i, PyLong_FromLong(result->label_ids.data[i]));
  PyObject_SetAttrString(res, "boxes", boxes);
  PyObject_SetAttrString(res, "scores", scores);
  PyObject_SetAttrString(res, "label_ids", labels);
  Py_DECREF(boxes); Py_DECREF(scores); Py_DECREF(labels);
  PyObject* arr = mat_to_numpy(img);
  PyObject* drawn = arr != nullptr ? PyObject_CallFunction(vis, "OOfif", arr, res, score_threshold, line_size, font_size) : nullptr;
  Py_XDECREF(arr); Py_DECREF(res); Py_DECREF(vis);
  if (drawn == nullptr) { fetch_py_error("vis_detection"); return 0; }
  const bool ok = copy_image_back(drawn, out);
  Py_DECREF(drawn);
  return ok ? 1 : 0;
}

FD_C_Bool FD_C_VisSegmentation(FD_C_Mat img, const FD_C_SegmentationResult* result, float weight, FD_C_Mat* out) {
  Gil g;
  PyObject* res_cls = get_class("vision.SegmentationResult");
  PyObject* vis = get_class("vision.vis_segmentation");
  if (res_cls == nullptr || vis == nullptr) { Py_XDECREF(res_cls); Py_XDECREF(vis); return 0; }
  PyObject* res = PyObject_CallObject(res_cls, nullptr);
  Py_DECREF(res_cls);
  if (res == nullptr) { fetch_py_error("SegmentationResult"); Py_DECREF(vis); return 0; }
  PyObject* lm = PyList_New(static_cast<Py_ssize_t>(result->label_map.size));
  for (size_t i = 0; i < result->label_map.size; ++i) PyList_SET_ITEM(lm, i, PyLong_FromLong(result->label_map.data[i]));
  PyObject* shape = Py_BuildValue("[ii]", result->height, result->width);
  PyObject_SetAttrString(res, "label_map", lm);
  PyObject_SetAttrString(res, "shape", shape);
  Py_DECREF(lm); Py_DECREF(shape);
  PyObject* arr = mat_to_numpy(img);
  PyObject* drawn = arr != nullptr ? PyObject_CallFunction(vis, "OOf", arr, res, weight) : nullptr;
  Py_XDECREF(arr); Py_DECREF(res); Py_DECREF(vis);
  if (drawn == nullptr) { fetch_py_error("vis_segmentation"); return 0; }
  const bool ok = copy_image_back(drawn, out);
  Py_DECREF(drawn);
  return ok ? 1 : 0;
}

void FD_C_DestroyClassifyResult(FD_C_ClassifyResult* r) {
  if (r == nullptr) return;
  std::free(r->label_ids.data); std::free(r->scores.data);
  r->label_ids.data = nullptr; r->scores.data = nullptr;
}
void FD_C_DestroyDetectionResult(FD_C_DetectionResult* r) {
  if (r == nullptr) return;
  for (size_t i = 0; i < r->boxes.size; ++i) std::free(r->boxes.data[i].data);
  std::free(r->boxes.data); std::free(r->scores.data); std::free(r->label_ids.data);
  r->boxes.data = nullptr; r->scores.data = nullptr; r->label_ids.data = nullptr;
}


// ---------------------------------------------------------------- the remaining option entry points
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseTimVX, "use_timvx")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseAscend, "use_ascend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseSophgo, "use_sophgo")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseSophgoBackend, "use_sophgo_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUsePorosBackend, "use_poros_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUseLiteBackend, "use_lite_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperUsePaddleLiteBackend, "use_paddle_lite_backend")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnablePaddleToTrt, "enable_paddle_to_trt")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnablePaddleLogInfo, "enable_paddle_log_info")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperDisablePaddleLogInfo, "disable_paddle_log_info")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnableLiteFP16, "enable_lite_fp16")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperDisableLiteFP16, "disable_lite_fp16")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnableLiteInt8, "enable_lite_int8")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperDisableLiteInt8, "disable_lite_int8")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperEnablePaddleTrtCollectShape, "enable_paddle_trt_collect_shape")
FD_OPT_CALL0(FD_C_RuntimeOptionWrapperDisablePaddleTrtCollectShape, "disable_paddle_trt_collect_shape")
#define FD_OPT_CALL_INT(cname, pyname)                                 \
  void cname(FD_C_RuntimeOptionWrapper* w, int v) {                    \
    Gil g;                                                             \
    PyObject* r = call_method(w->obj, pyname, "(i)", v);               \
    Py_XDECREF(r);                                                     \
  }
#define FD_OPT_CALL_STR(cname, pyname)                                 \
  void cname(FD_C_RuntimeOptionWrapper* w, const char* v) {            \
    Gil g;                                                             \
    PyObject* r = call_method(w->obj, pyname, "(s)", v ? v : "");      \
    Py_XDECREF(r);                                                     \
  }
FD_OPT_CALL_INT(FD_C_RuntimeOptionWrapperSetOrtGraphOptLevel, "set_ort_graph_opt_level")
FD_OPT_CALL_INT(FD_C_RuntimeOptionWrapperSetPaddleMKLDNNCacheSize, "set_paddle_mkldnn_cache_size")
FD_OPT_CALL_INT(FD_C_RuntimeOptionWrapperSetOpenVINOStreams, "set_openvino_streams")
FD_OPT_CALL_INT(FD_C_RuntimeOptionWrapperSetLitePowerMode, "set_lite_power_mode")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperDeletePaddleBackendPass, "delete_paddle_backend_pass")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetOpenVINODevice, "set_openvino_device")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetLiteOptimizedModelDir, "set_lite_optimized_model_dir")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetLiteSubgraphPartitionPath, "set_lite_subgraph_partition_path")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetLiteSubgraphPartitionConfigBuffer, "set_lite_subgraph_partition_config_buffer")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetLiteContextProperties, "set_lite_context_properties")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetLiteModelCacheDir, "set_lite_model_cache_dir")
FD_OPT_CALL_STR(FD_C_RuntimeOptionWrapperSetLiteMixedPrecisionQuantizationConfigPath,
                "set_lite_mixed_precision_quantization_config_path")
void FD_C_RuntimeOptionWrapperSetPaddleMKLDNN(FD_C_RuntimeOptionWrapper* w, FD_C_Bool on) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_paddle_mkldnn", "(O)", on ? Py_True : Py_False);
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperSetExternalStream(FD_C_RuntimeOptionWrapper* w, void* stream) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_external_raw_stream", "(K)", static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(stream)));
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperSetModelBuffer(FD_C_RuntimeOptionWrapper* w, const char* model, size_t model_size, const char* params,
                                             size_t params_size, FD_C_ModelFormat format) {
  Gil g;
  PyObject* r = call_method(w->obj, "set_model_buffer", "(y#y#i)", model, static_cast<Py_ssize_t>(model_size), params ? params : "",
                            static_cast<Py_ssize_t>(params ? params_size : 0), static_cast<int>(format));
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperUseKunlunXin(FD_C_RuntimeOptionWrapper* w, int id, int l3, FD_C_Bool locked, FD_C_Bool autotune,
                                           const char* autotune_file, const char* precision, FD_C_Bool adaptive_seqlen,
                                           FD_C_Bool multi_stream, int64_t gm_default_size) {
  Gil g;
  PyObject* r = call_method(w->obj, "use_kunlunxin", "(iiiissiiL)", id, l3, static_cast<int>(locked), static_cast<int>(autotune),
                            autotune_file ? autotune_file : "", precision ? precision : "", static_cast<int>(adaptive_seqlen),
                            static_cast<int>(multi_stream), static_cast<long long>(gm_default_size));
  Py_XDECREF(r);
}
void FD_C_RuntimeOptionWrapperUseIpu(FD_C_RuntimeOptionWrapper* w, int device_num, int micro_batch_size, FD_C_Bool pipelining,
                                     int batches_per_step) {
  Gil g;
  PyObject* r = call_method(w->obj, "use_ipu", "(iiii)", device_num, micro_batch_size, static_cast<int>(pipelining), batches_per_step);
  Py_XDECREF(r);
}

// ---------------------------------------------------------------- detection classes by name
static FD_C_Bool model_initialized(FD_C_ModelWrapper* w) {
  Gil g;
  PyObject* r = call_method(w->obj, "initialized");
  const FD_C_Bool v = r != nullptr && PyObject_IsTrue(r) ? 1 : 0;
  Py_XDECREF(r);
  return v;
}
#define FD_C_IMPLEMENT_DETECTION_COMMON(T)                                                                                   \
  void FD_C_Destroy##T##Wrapper(FD_C_##T##Wrapper* w) { FD_C_DestroyModelWrapper(w); }                                       \
  FD_C_Bool FD_C_##T##WrapperPredict(FD_C_##T##Wrapper* w, FD_C_Mat img, FD_C_DetectionResult* r) {                          \
    return predict_detection(w, img, r);                                                                                     \
  }                                                                                                                          \
  FD_C_Bool FD_C_##T##WrapperInitialized(FD_C_##T##Wrapper* w) { return model_initialized(w); }                              \
  FD_C_Bool FD_C_##T##WrapperBatchPredict(FD_C_##T##Wrapper* w, const FD_C_Mat* imgs, int n, FD_C_DetectionResult* r) {      \
    return FD_C_DetectionModelWrapperBatchPredict(w, imgs, n, r);                                                            \
  }
#define FD_C_IMPLEMENT_PPDET(T)                                                                                              \
  FD_C_IMPLEMENT_DETECTION_COMMON(T)                                                                                         \
  FD_C_##T##Wrapper* FD_C_Create##T##Wrapper(const char* m, const char* p, const char* c, FD_C_RuntimeOptionWrapper* o,      \
                                             FD_C_ModelFormat f) {                                                           \
    return create_model("vision.detection." #T, m, p, c, o, f);                                                              \
  }
#define FD_C_IMPLEMENT_YOLO(T)                                                                                               \
  FD_C_IMPLEMENT_DETECTION_COMMON(T)                                                                                         \
  FD_C_##T##Wrapper* FD_C_Create##T##Wrapper(const char* m, const char* p, FD_C_RuntimeOptionWrapper* o, FD_C_ModelFormat f) { \
    return create_model("vision.detection." #T, m, p, nullptr, o, f);                                                        \
  }
FD_C_PPDET_MODELS(FD_C_IMPLEMENT_PPDET)
FD_C_YOLO_MODELS(FD_C_IMPLEMENT_YOLO)
FD_C_Bool FD_C_PPYOLOEWrapperBatchPredict(FD_C_PPYOLOEWrapper* w, const FD_C_Mat* imgs, int n, FD_C_DetectionResult* r) {
  return FD_C_DetectionModelWrapperBatchPredict(w, imgs, n, r);
}

// ---------------------------------------------------------------- batches of the other model kinds
// Runs `batch_predict` on the images and hands each item of the returned list to `convert(item, index)`.
}  // extern "C"
template <typename Convert>
static FD_C_Bool batch_predict_generic(FD_C_ModelWrapper* w, const FD_C_Mat* imgs, int n_imgs, Convert convert) {
  Gil g;
  PyObject* list = PyList_New(n_imgs);
  for (int i = 0; i < n_imgs; ++i) {
    PyObject* arr = mat_to_numpy(imgs[i]);
    if (arr == nullptr) { Py_DECREF(list); return 0; }
    PyList_SET_ITEM(list, i, arr);
  }
  PyObject* r = call_method(w->obj, "batch_predict", "(O)", list);
  Py_DECREF(list);
  if (r == nullptr) return 0;
  bool ok = PySequence_Check(r) && PySequence_Size(r) == n_imgs;
  for (int i = 0; i < n_imgs && ok; ++i) {
    PyObject* item = PySequence_GetItem(r, i);
    ok = item != nullptr && convert(item, i);
    Py_XDECREF(item);
  }
  if (!ok && g_err.empty()) set_err("batch_predict: unexpected result");
  Py_DECREF(r);
  return ok ? 1 : 0;
}
extern "C" {
static bool classify_from_py(PyObject* r, FD_C_ClassifyResult* out) {
  PyObject *ids = PyObject_GetAttrString(r, "label_ids"), *scores = PyObject_GetAttrString(r, "scores");
  const bool ok = ids && scores && ints_from_seq(ids, &out->label_ids) && floats_from_seq(scores, &out->scores);
  Py_XDECREF(ids); Py_XDECREF(scores);
  return ok;
}
FD_C_Bool FD_C_PaddleClasModelWrapperInitialized(FD_C_PaddleClasModelWrapper* w) { return model_initialized(w); }
FD_C_Bool FD_C_PaddleClasModelWrapperBatchPredict(FD_C_PaddleClasModelWrapper* w, const FD_C_Mat* imgs, int n, FD_C_ClassifyResult* out) {
  return batch_predict_generic(w, imgs, n, [&](PyObject* item, int i) { return classify_from_py(item, &out[i]); });
}
void FD_C_DestroyPaddleSegModelWrapper(FD_C_PaddleSegModelWrapper* w) { FD_C_DestroyModelWrapper(w); }
FD_C_Bool FD_C_PaddleSegModelWrapperInitialized(FD_C_PaddleSegModelWrapper* w) { return model_initialized(w); }
FD_C_Bool FD_C_PaddleSegModelWrapperBatchPredict(FD_C_PaddleSegModelWrapper* w, const FD_C_Mat* imgs, int n, FD_C_SegmentationResult* out) {
  return batch_predict_generic(w, imgs, n, [&](PyObject* item, int i) { return seg_from_py(item, &out[i]); });
}
FD_C_Bool FD_C_PPOCRv2WrapperPredict(FD_C_PPOCRv2Wrapper* w, FD_C_Mat img, FD_C_OCRResult* out) {
  return FD_C_PPOCRv3WrapperPredict(w, img, out);
}
FD_C_Bool FD_C_PPOCRv3WrapperBatchPredict(FD_C_PPOCRv3Wrapper* w, const FD_C_Mat* imgs, int n, FD_C_OCRResult* out) {
  return batch_predict_generic(w, imgs, n, [&](PyObject* item, int i) { return ocr_from_py(item, &out[i]); });
}
FD_C_Bool FD_C_PPOCRv2WrapperBatchPredict(FD_C_PPOCRv2Wrapper* w, const FD_C_Mat* imgs, int n, FD_C_OCRResult* out) {
  return FD_C_PPOCRv3WrapperBatchPredict(w, imgs, n, out);
}
void FD_C_DestroyPPOCRv2Wrapper(FD_C_PPOCRv2Wrapper* w) { FD_C_DestroyModelWrapper(w); }
void FD_C_DestroyPPOCRv3Wrapper(FD_C_PPOCRv3Wrapper* w) { FD_C_DestroyModelWrapper(w); }

// ---------------------------------------------------------------- images
FD_C_Mat FD_C_Imread(const char* path) {
  FD_C_Mat m{nullptr, 0, 0, 0};
  Gil g;
  PyObject* cv2 = PyImport_ImportModule("cv2");
  if (cv2 == nullptr) { fetch_py_error("import cv2"); return m; }
  PyObject* img = PyObject_CallMethod(cv2, "imread", "s", path);
  Py_DECREF(cv2);
  if (img == nullptr) { fetch_py_error("imread"); return m; }
  if (img == Py_None) { Py_DECREF(img); set_err(std::string("imread: cannot read ") + path); return m; }
  PyObject* shp = PyObject_GetAttrString(img, "shape");
  PyObject* bytes = call_method(img, "tobytes");
  if (shp != nullptr && bytes != nullptr && PyTuple_Size(shp) == 3) {
    m.height = static_cast<int>(PyLong_AsLong(PyTuple_GET_ITEM(shp, 0)));
    m.width = static_cast<int>(PyLong_AsLong(PyTuple_GET_ITEM(shp, 1)));
    m.channels = static_cast<int>(PyLong_AsLong(PyTuple_GET_ITEM(shp, 2)));
    char* buf = nullptr;
    Py_ssize_t n = 0;
    PyBytes_AsStringAndSize(bytes, &buf, &n);
    m.data = static_cast<uint8_t*>(std::malloc(n > 0 ? n : 1));
    std::memcpy(m.data, buf, static_cast<size_t>(n));
  } else {
    set_err("imread: unexpected image layout");
  }
  Py_XDECREF(shp); Py_XDECREF(bytes); Py_DECREF(img);
  return m;
}
FD_C_Bool FD_C_Imwrite(const char* path, FD_C_Mat img) {
  Gil g;
  PyObject* cv2 = PyImport_ImportModule("cv2");
  if (cv2 == nullptr) { fetch_py_error("import cv2"); return 0; }
  PyObject* arr = mat_to_numpy(img);
  PyObject* r = arr != nullptr ? PyObject_CallMethod(cv2, "imwrite", "sO", path, arr) : nullptr;
  Py_DECREF(cv2); Py_XDECREF(arr);
  if (r == nullptr) { if (PyErr_Occurred()) fetch_py_error("imwrite"); return 0; }
  const FD_C_Bool ok = PyObject_IsTrue(r) ? 1 : 0;
  if (!ok) set_err(std::string("imwrite: cannot write ") + path);
  Py_DECREF(r);
  return ok;
}
void FD_C_DestroyMat(FD_C_Mat img) { std::free(img.data); }

// ---------------------------------------------------------------- result text
static PyObject* py_detection_result(const FD_C_DetectionResult* result) {
  PyObject* res_cls = get_class("vision.DetectionResult");
  if (res_cls == nullptr) return nullptr;
  PyObject* res = PyObject_CallObject(res_cls, nullptr);
  Py_DECREF(res_cls);
  if (res == nullptr) { fetch_py_error("DetectionResult"); return nullptr; }
  PyObject* boxes = PyList_New(static_cast<Py_ssize_t>(result->boxes.size));
  for (size_t i = 0; i < result->boxes.size; ++i)
    PyList_SET_ITEM(boxes, i, py_list_of_floats(result->boxes.data[i].data, result->boxes.data[i].size));
  PyObject* scores = py_list_of_floats(result->scores.data, result->scores.size);
  PyObject* labels = PyList_New(static_cast<Py_ssize_t>(result->label_ids.size));
  for (size_t i = 0; i < result->label_ids.size; ++i) PyList_SET_ITEM(labels, i, PyLong_FromLong(result->label_ids.data[i]));
  PyObject_SetAttrString(res, "boxes", boxes);
  PyObject_SetAttrString(res, "scores", scores);
  PyObject_SetAttrString(res, "label_ids", labels);
  Py_DECREF(boxes); Py_DECREF(scores); Py_DECREF(labels);
  return res;
}
static PyObject* py_ocr_result(const FD_C_OCRResult* result) {
  PyObject* res_cls = get_class("vision.OCRResult");
  if (res_cls == nullptr) return nullptr;
  PyObject* res = PyObject_CallObject(res_cls, nullptr);
  Py_DECREF(res_cls);
  if (res == nullptr) { fetch_py_error("OCRResult"); return nullptr; }
  PyObject* boxes = PyList_New(static_cast<Py_ssize_t>(result->boxes.size));
  for (size_t i = 0; i < result->boxes.size; ++i) {
    PyObject* b = PyList_New(static_cast<Py_ssize_t>(result->boxes.data[i].size));
    for (size_t k = 0; k < result->boxes.data[i].size; ++k)
      PyList_SET_ITEM(b, k, PyLong_FromLong(static_cast<long>(result->boxes.data[i].data[k])));
    PyList_SET_ITEM(boxes, i, b);
  }
  PyObject* text = PyList_New(static_cast<Py_ssize_t>(result->n_text));
  for (size_t i = 0; i < result->n_text; ++i) PyList_SET_ITEM(text, i, PyUnicode_FromString(result->text[i] ? result->text[i] : ""));
  PyObject* rs = py_list_of_floats(result->rec_scores.data, result->rec_scores.size);
  PyObject* cs = py_list_of_floats(result->cls_scores.data, result->cls_scores.size);
  PyObject* cl = PyList_New(static_cast<Py_ssize_t>(result->cls_labels.size));
  for (size_t i = 0; i < result->cls_labels.size; ++i) PyList_SET_ITEM(cl, i, PyLong_FromLong(result->cls_labels.data[i]));
  PyObject_SetAttrString(res, "boxes", boxes); PyObject_SetAttrString(res, "text", text);
  PyObject_SetAttrString(res, "rec_scores", rs); PyObject_SetAttrString(res, "cls_scores", cs);
  PyObject_SetAttrString(res, "cls_labels", cl);
  Py_DECREF(boxes); Py_DECREF(text); Py_DECREF(rs); Py_DECREF(cs); Py_DECREF(cl);
  return res;
}
// str(obj) into the caller's buffer; steals the reference
static size_t str_into(PyObject* obj, char* buffer, size_t capacity) {
  if (obj == nullptr) return 0;
  PyObject* s = PyObject_Str(obj);
  Py_DECREF(obj);
  if (s == nullptr) { fetch_py_error("str"); return 0; }
  Py_ssize_t n = 0;
  const char* c = PyUnicode_AsUTF8AndSize(s, &n);
  if (c != nullptr && buffer != nullptr && capacity > 0) {
    const size_t k = static_cast<size_t>(n) < capacity - 1 ? static_cast<size_t>(n) : capacity - 1;
    std::memcpy(buffer, c, k);
    buffer[k] = 0;
  }
  Py_DECREF(s);
  return static_cast<size_t>(n) + 1;
}
size_t FD_C_DetectionResultStr(const FD_C_DetectionResult* r, char* buffer, size_t capacity) {
  Gil g;
  return str_into(py_detection_result(r), buffer, capacity);
}
size_t FD_C_OCRResultStr(const FD_C_OCRResult* r, char* buffer, size_t capacity) {
  Gil g;
  return str_into(py_ocr_result(r), buffer, capacity);
}
size_t FD_C_ClassifyResultStr(const FD_C_ClassifyResult* r, char* buffer, size_t capacity) {
  Gil g;
  PyObject* res_cls = get_class("vision.ClassifyResult");
  if (res_cls == nullptr) return 0;
  PyObject* res = PyObject_CallObject(res_cls, nullptr);
  Py_DECREF(res_cls);
  if (res == nullptr) { fetch_py_error("ClassifyResult"); return 0; }
  PyObject* ids = PyList_New(static_cast<Py_ssize_t>(r->label_ids.size));
  for (size_t i = 0; i < r->label_ids.size; ++i) PyList_SET_ITEM(ids, i, PyLong_FromLong(r->label_ids.data[i]));
  PyObject* sc = py_list_of_floats(r->scores.data, r->scores.size);
  PyObject_SetAttrString(res, "label_ids", ids); PyObject_SetAttrString(res, "scores", sc);
  Py_DECREF(ids); Py_DECREF(sc);
  return str_into(res, buffer, capacity);
}
size_t FD_C_SegmentationResultStr(const FD_C_SegmentationResult* r, char* buffer, size_t capacity) {
  Gil g;
  PyObject* res_cls = get_class("vision.SegmentationResult");
  if (res_cls == nullptr) return 0;
  PyObject* res = PyObject_CallObject(res_cls, nullptr);
  Py_DECREF(res_cls);
  if (res == nullptr) { fetch_py_error("SegmentationResult"); return 0; }
  PyObject* lm = PyList_New(static_cast<Py_ssize_t>(r->label_map.size));
  for (size_t i = 0; i < r->label_map.size; ++i) PyList_SET_ITEM(lm, i, PyLong_FromLong(r->label_map.data[i]));
  PyObject* sm = py_list_of_floats(r->score_map.data, r->score_map.size);
  PyObject* shape = Py_BuildValue("[ii]", r->height, r->width);
  PyObject_SetAttrString(res, "label_map", lm); PyObject_SetAttrString(res, "score_map", sm);
  PyObject_SetAttrString(res, "shape", shape);
  PyObject_SetAttrString(res, "contain_score_map", r->contain_score_map ? Py_True : Py_False);
  Py_DECREF(lm); Py_DECREF(sm); Py_DECREF(shape);
  return str_into(res, buffer, capacity);
}

// ---------------------------------------------------------------- more visualisers
FD_C_Bool FD_C_VisDetectionWithLabel(FD_C_Mat img, const FD_C_DetectionResult* result, const char* const* labels, int n_labels,
                                     float score_threshold, int line_size, float font_size, FD_C_Mat* out) {
  Gil g;
  PyObject* vis = get_class("vision.vis_detection");
  PyObject* res = vis != nullptr ? py_detection_result(result) : nullptr;
  if (res == nullptr) { Py_XDECREF(vis); return 0; }
  PyObject* names = PyList_New(n_labels);
  for (int i = 0; i < n_labels; ++i) PyList_SET_ITEM(names, i, PyUnicode_FromString(labels[i] ? labels[i] : ""));
  PyObject* arr = mat_to_numpy(img);
  PyObject* drawn = arr != nullptr ? PyObject_CallFunction(vis, "OOOfif", arr, res, names, score_threshold, line_size, font_size) : nullptr;
  Py_XDECREF(arr); Py_DECREF(res); Py_DECREF(names); Py_DECREF(vis);
  if (drawn == nullptr) { fetch_py_error("vis_detection"); return 0; }
  const bool ok = copy_image_back(drawn, out);
  Py_DECREF(drawn);
  return ok ? 1 : 0;
}
FD_C_Bool FD_C_VisOcr(FD_C_Mat img, const FD_C_OCRResult* result, FD_C_Mat* out) {
  Gil g;
  PyObject* vis = get_class("vision.vis_ppocr");
  PyObject* res = vis != nullptr ? py_ocr_result(result) : nullptr;
  if (res == nullptr) { Py_XDECREF(vis); return 0; }
  PyObject* arr = mat_to_numpy(img);
  PyObject* drawn = arr != nullptr ? PyObject_CallFunction(vis, "OO", arr, res) : nullptr;
  Py_XDECREF(arr); Py_DECREF(res); Py_DECREF(vis);
  if (drawn == nullptr) { fetch_py_error("vis_ppocr"); return 0; }
  const bool ok = copy_image_back(drawn, out);
  Py_DECREF(drawn);
  return ok ? 1 : 0;
}


// ---------------------------------------------------------------- OCR stages on their own
FD_C_DBDetectorWrapper* FD_C_CreateDBDetectorWrapper(const char* m, const char* p, FD_C_RuntimeOptionWrapper* o, FD_C_ModelFormat f) {
  return create_model("vision.ocr.DBDetector", m, p, nullptr, o, f);
}
FD_C_ClassifierWrapper* FD_C_CreateClassifierWrapper(const char* m, const char* p, FD_C_RuntimeOptionWrapper* o, FD_C_ModelFormat f) {
  return create_model("vision.ocr.Classifier", m, p, nullptr, o, f);
}
FD_C_RecognizerWrapper* FD_C_CreateRecognizerWrapper(const char* m, const char* p, const char* label_path, FD_C_RuntimeOptionWrapper* o,
                                                     FD_C_ModelFormat f) {
  Gil g;
  if (g_pkg == nullptr) return nullptr;
  PyObject* cls = get_class("vision.ocr.Recognizer");
  if (cls == nullptr) return nullptr;
  PyObject* kwargs = PyDict_New();
  if (o != nullptr) PyDict_SetItemString(kwargs, "runtime_option", o->obj);
  PyObject* fmt = PyLong_FromLong(static_cast<long>(f));
  PyDict_SetItemString(kwargs, "model_format", fmt);
  Py_DECREF(fmt);
  PyObject* args = Py_BuildValue("(sss)", m, p ? p : "", label_path ? label_path : "");     // the label file may be empty
  PyObject* obj = PyObject_Call(cls, args, kwargs);
  Py_DECREF(args); Py_DECREF(kwargs); Py_DECREF(cls);
  if (obj == nullptr) { fetch_py_error("vision.ocr.Recognizer"); return nullptr; }
  return new FD_C_ModelWrapper{obj};
}
void FD_C_DestroyDBDetectorWrapper(FD_C_DBDetectorWrapper* w) { FD_C_DestroyModelWrapper(w); }
void FD_C_DestroyClassifierWrapper(FD_C_ClassifierWrapper* w) { FD_C_DestroyModelWrapper(w); }
void FD_C_DestroyRecognizerWrapper(FD_C_RecognizerWrapper* w) { FD_C_DestroyModelWrapper(w); }
FD_C_Bool FD_C_DBDetectorWrapperInitialized(FD_C_DBDetectorWrapper* w) { return model_initialized(w); }
FD_C_Bool FD_C_ClassifierWrapperInitialized(FD_C_ClassifierWrapper* w) { return model_initialized(w); }
FD_C_Bool FD_C_RecognizerWrapperInitialized(FD_C_RecognizerWrapper* w) { return model_initialized(w); }

static PyObject* predict_on_image(FD_C_ModelWrapper* w, FD_C_Mat img) {
  PyObject* arr = mat_to_numpy(img);
  if (arr == nullptr) return nullptr;
  PyObject* r = call_method(w->obj, "predict", "(O)", arr);
  Py_DECREF(arr);
  return r;
}
FD_C_Bool FD_C_DBDetectorWrapperPredict(FD_C_DBDetectorWrapper* w, FD_C_Mat img, FD_C_TwoDimArrayInt32* boxes) {
  Gil g;
  boxes->size = 0; boxes->data = nullptr;
  PyObject* r = predict_on_image(w, img);
  if (r == nullptr) return 0;
  const Py_ssize_t n = PySequence_Size(r);
  bool ok = n >= 0;
  if (ok) {
    boxes->size = static_cast<size_t>(n);
    boxes->data = static_cast<FD_C_OneDimArrayInt32*>(std::calloc(n > 0 ? n : 1, sizeof(FD_C_OneDimArrayInt32)));
    for (Py_ssize_t i = 0; i < n && ok; ++i) {
      PyObject* b = PySequence_GetItem(r, i);
      ok = b != nullptr && ints_from_seq(b, &boxes->data[i]);
      Py_XDECREF(b);
    }
  } else {
    fetch_py_error("DBDetector.predict");
  }
  Py_DECREF(r);
  return ok ? 1 : 0;
}
FD_C_Bool FD_C_ClassifierWrapperPredict(FD_C_ClassifierWrapper* w, FD_C_Mat img, int32_t* cls_label, float* cls_score) {
  Gil g;
  PyObject* r = predict_on_image(w, img);
  if (r == nullptr) return 0;
  int label = 0;
  float score = 0.0f;
  const bool ok = PyArg_ParseTuple(r, "if", &label, &score) != 0;
  if (!ok) fetch_py_error("Classifier.predict");
  Py_DECREF(r);
  if (ok) { *cls_label = label; *cls_score = score; }
  return ok ? 1 : 0;
}
FD_C_Bool FD_C_RecognizerWrapperPredict(FD_C_RecognizerWrapper* w, FD_C_Mat img, char** text, float* rec_score) {
  Gil g;
  *text = nullptr;
  PyObject* r = predict_on_image(w, img);
  if (r == nullptr) return 0;
  const char* t = nullptr;
  float score = 0.0f;
  const bool ok = PyArg_ParseTuple(r, "sf", &t, &score) != 0;
  if (ok) { *text = strdup(t); *rec_score = score; }
  else fetch_py_error("Recognizer.predict");
  Py_DECREF(r);
  return ok ? 1 : 0;
}
void FD_C_DestroyTwoDimArrayInt32(FD_C_TwoDimArrayInt32* a) {
  if (a == nullptr) return;
  for (size_t i = 0; i < a->size; ++i) std::free(a->data[i].data);
  std::free(a->data);
  a->data = nullptr; a->size = 0;
}
void FD_C_DestroyCstr(char* text) { std::free(text); }

}  // extern "C"
