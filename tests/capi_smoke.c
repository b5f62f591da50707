/* C caller of the library: loads an ONNX model through FD_C_RuntimeWrapper, runs it, prints the output
 * checksum; then exercises error reporting with a missing file. Built and run by tests/test_capi_cpu.py. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fd_c_api.h"

int main(int argc, char** argv) {
  if (argc < 6) { fprintf(stderr, "usage: capi_smoke model.onnx input_name n c hw\n"); return 2; }
  const char* model = argv[1];
  const char* input_name = argv[2];
  long n = atol(argv[3]), c = atol(argv[4]), hw = atol(argv[5]);

  FD_C_RuntimeOptionWrapper* opt = FD_C_CreateRuntimeOptionWrapper();
  if (!opt) { fprintf(stderr, "option: %s\n", FD_C_GetLastError()); return 1; }
  FD_C_RuntimeOptionWrapperSetModelPath(opt, model, "", FD_C_ModelFormat_ONNX);
  FD_C_RuntimeOptionWrapperUseCpu(opt);
  FD_C_RuntimeWrapper* rt = FD_C_CreateRuntimeWrapper(opt);
  if (!rt) { fprintf(stderr, "runtime: %s\n", FD_C_GetLastError()); return 1; }
  printf("inputs=%d outputs=%d\n", FD_C_RuntimeWrapperNumInputs(rt), FD_C_RuntimeWrapperNumOutputs(rt));

  size_t count = (size_t)(n * c * hw * hw);
  float* x = (float*)malloc(sizeof(float) * count);
  for (size_t i = 0; i < count; ++i) x[i] = (float)((i * 2654435761u) % 1000) / 1000.0f - 0.5f;
  int64_t shape[4] = {n, c, hw, hw};
  FD_C_Tensor in;
  in.name = input_name; in.dtype = 0; in.shape.size = 4; in.shape.data = shape; in.data = x; in.nbytes = sizeof(float) * count;
  FD_C_Tensor outs[4];
  int n_out = 0;
  if (!FD_C_RuntimeWrapperInfer(rt, &in, 1, outs, 4, &n_out)) { fprintf(stderr, "infer: %s\n", FD_C_GetLastError()); return 1; }
  double sum = 0;
  size_t elems = outs[0].nbytes / sizeof(float);
  for (size_t i = 0; i < elems; ++i) sum += ((float*)outs[0].data)[i];
  printf("n_out=%d ndim=%zu elems=%zu checksum=%.6f\n", n_out, outs[0].shape.size, elems, sum);
  FD_C_DestroyTensors(outs, n_out < 4 ? n_out : 4);
  FD_C_DestroyRuntimeWrapper(rt);

  FD_C_RuntimeOptionWrapperSetModelPath(opt, "/nonexistent/model.onnx", "", FD_C_ModelFormat_ONNX);
  FD_C_RuntimeWrapper* bad = FD_C_CreateRuntimeWrapper(opt);
  printf("bad=%s err=%s\n", bad ? "non-null" : "null", strlen(FD_C_GetLastError()) > 0 ? "set" : "empty");
  FD_C_DestroyRuntimeOptionWrapper(opt);
  free(x);
  return 0;
}
