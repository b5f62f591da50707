/* C caller of the model-level entry points: option setters, a detection class created by name, batches, result text,
 * image files and the label visualiser. Built and run by tests/test_capi_cpu.py.
 *   capi_models det.pdmodel det.pdiparams det.yml cls.pdmodel cls.pdiparams cls.yaml out.png */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fd_c_api.h"

static FD_C_Mat make_image(int h, int w, unsigned seed) {
  FD_C_Mat m;
  m.height = h; m.width = w; m.channels = 3;
  m.data = (uint8_t*)malloc((size_t)h * w * 3);
  for (int i = 0; i < h * w * 3; ++i) { seed = seed * 1664525u + 1013904223u; m.data[i] = (uint8_t)(seed >> 24); }
  return m;
}

int main(int argc, char** argv) {
  if (argc < 8) { fprintf(stderr, "usage\n"); return 2; }
  FD_C_RuntimeOptionWrapper* opt = FD_C_CreateRuntimeOptionWrapper();
  if (!opt) { fprintf(stderr, "option: %s\n", FD_C_GetLastError()); return 1; }
  /* settings for other vendors' back ends are accepted and change nothing */
  FD_C_RuntimeOptionWrapperUseAscend(opt);
  FD_C_RuntimeOptionWrapperUseKunlunXin(opt, 0, 1 << 20, 0, 1, "", "int16", 0, 0, 0);
  FD_C_RuntimeOptionWrapperUseIpu(opt, 1, 1, 0, 1);
  FD_C_RuntimeOptionWrapperUsePaddleLiteBackend(opt);
  FD_C_RuntimeOptionWrapperSetLitePowerMode(opt, 3);
  FD_C_RuntimeOptionWrapperSetLiteModelCacheDir(opt, "/tmp/none");
  FD_C_RuntimeOptionWrapperEnableLiteInt8(opt);
  FD_C_RuntimeOptionWrapperSetOpenVINODevice(opt, "CPU");
  FD_C_RuntimeOptionWrapperSetOpenVINOStreams(opt, 2);
  FD_C_RuntimeOptionWrapperSetOrtGraphOptLevel(opt, 99);
  FD_C_RuntimeOptionWrapperSetPaddleMKLDNN(opt, 1);
  FD_C_RuntimeOptionWrapperDeletePaddleBackendPass(opt, "fc_fuse_pass");
  FD_C_RuntimeOptionWrapperDisablePaddleLogInfo(opt);
  FD_C_RuntimeOptionWrapperSetExternalStream(opt, NULL);
  FD_C_RuntimeOptionWrapperUseCpu(opt);
  printf("options=%s\n", strlen(FD_C_GetLastError()) == 0 ? "ok" : FD_C_GetLastError());

  /* a detection class by its own name */
  FD_C_PicoDetWrapper* det = FD_C_CreatePicoDetWrapper(argv[1], argv[2], argv[3], opt, FD_C_ModelFormat_PADDLE);
  if (!det) { fprintf(stderr, "PicoDet: %s\n", FD_C_GetLastError()); return 1; }
  printf("initialized=%d\n", (int)FD_C_PicoDetWrapperInitialized(det));
  FD_C_Mat imgs[2] = {make_image(60, 120, 1u), make_image(70, 120, 2u)};
  FD_C_DetectionResult batch[2], single;
  memset(batch, 0, sizeof(batch)); memset(&single, 0, sizeof(single));
  if (!FD_C_PicoDetWrapperBatchPredict(det, imgs, 2, batch)) { fprintf(stderr, "batch: %s\n", FD_C_GetLastError()); return 1; }
  if (!FD_C_PicoDetWrapperPredict(det, imgs[1], &single)) { fprintf(stderr, "predict: %s\n", FD_C_GetLastError()); return 1; }
  int same = batch[1].scores.size == single.scores.size;
  for (size_t i = 0; same && i < single.scores.size; ++i) {
    float d = batch[1].scores.data[i] - single.scores.data[i];
    same = d < 1e-5f && d > -1e-5f && batch[1].label_ids.data[i] == single.label_ids.data[i];
  }
  printf("boxes=%zu,%zu batch_equals_single=%d\n", batch[0].scores.size, batch[1].scores.size, same);
  char text[256];
  size_t need = FD_C_DetectionResultStr(&batch[0], text, sizeof(text));
  printf("str_need=%zu head=%.40s\n", need, text);
  char tiny[8];
  FD_C_DetectionResultStr(&batch[0], tiny, sizeof(tiny));
  printf("tiny=%s\n", tiny);

  /* drawing with class names, then a round trip through an image file */
  const char* labels[6] = {"a", "b", "c", "d", "e", "f"};
  FD_C_Mat drawn = make_image(60, 120, 0u);
  if (!FD_C_VisDetectionWithLabel(imgs[0], &batch[0], labels, 6, 0.0f, 1, 0.4f, &drawn)) {
    fprintf(stderr, "vis: %s\n", FD_C_GetLastError()); return 1;
  }
  if (!FD_C_Imwrite(argv[7], drawn)) { fprintf(stderr, "imwrite: %s\n", FD_C_GetLastError()); return 1; }
  FD_C_Mat back = FD_C_Imread(argv[7]);
  int identical = back.data != NULL && back.height == 60 && back.width == 120 && back.channels == 3 &&
                  memcmp(back.data, drawn.data, 60 * 120 * 3) == 0;
  printf("png_roundtrip=%d\n", identical);
  FD_C_DestroyMat(back);
  FD_C_Mat missing = FD_C_Imread("/nonexistent/image.png");
  printf("missing=%s err=%s\n", missing.data ? "non-null" : "null", strlen(FD_C_GetLastError()) > 0 ? "set" : "empty");
  FD_C_DestroyDetectionResult(&batch[0]); FD_C_DestroyDetectionResult(&batch[1]); FD_C_DestroyDetectionResult(&single);
  FD_C_DestroyPicoDetWrapper(det);

  /* a YOLO-family class takes no config file; a missing model is an error, not a crash */
  FD_C_YOLOv5Wrapper* y = FD_C_CreateYOLOv5Wrapper("/nonexistent/yolov5.onnx", "", opt, FD_C_ModelFormat_ONNX);
  printf("yolov5=%s\n", y ? "non-null" : "null");

  /* classifier: batch against single, and the result text */
  FD_C_PaddleClasModelWrapper* cls = FD_C_CreatePaddleClasModelWrapper(argv[4], argv[5], argv[6], opt, FD_C_ModelFormat_PADDLE);
  if (!cls) { fprintf(stderr, "cls: %s\n", FD_C_GetLastError()); return 1; }
  FD_C_ClassifyResult cb[2], cs;
  memset(cb, 0, sizeof(cb)); memset(&cs, 0, sizeof(cs));
  if (!FD_C_PaddleClasModelWrapperBatchPredict(cls, imgs, 2, cb)) { fprintf(stderr, "cls batch: %s\n", FD_C_GetLastError()); return 1; }
  if (!FD_C_PaddleClasModelWrapperPredict(cls, imgs[0], &cs)) { fprintf(stderr, "cls predict: %s\n", FD_C_GetLastError()); return 1; }
  printf("cls_initialized=%d labels=%d,%d single=%d\n", (int)FD_C_PaddleClasModelWrapperInitialized(cls), cb[0].label_ids.data[0],
         cb[1].label_ids.data[0], cs.label_ids.data[0]);
  FD_C_ClassifyResultStr(&cb[0], text, sizeof(text));
  printf("cls_str=%.15s\n", text);
  FD_C_DestroyClassifyResult(&cb[0]); FD_C_DestroyClassifyResult(&cb[1]); FD_C_DestroyClassifyResult(&cs);
  FD_C_DestroyPaddleClasModelWrapper(cls);

  FD_C_OCRResult ocr;
  memset(&ocr, 0, sizeof(ocr));
  FD_C_OCRResultStr(&ocr, text, sizeof(text));
  printf("empty_ocr_str_len=%zu\n", strlen(text));
  free(imgs[0].data); free(imgs[1].data); free(drawn.data);
  FD_C_DestroyRuntimeOptionWrapper(opt);
  return 0;
}
