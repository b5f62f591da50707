/* C caller of the OCR stage wrappers: detector boxes, direction classifier, recogniser text on one synthetic page.
 *   capi_ocr_stages det.pdmodel det.pdiparams cls.pdmodel cls.pdiparams rec.pdmodel rec.pdiparams dict.txt */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fd_c_api.h"

int main(int argc, char** argv) {
  if (argc < 8) { fprintf(stderr, "usage\n"); return 2; }
  FD_C_RuntimeOptionWrapper* opt = FD_C_CreateRuntimeOptionWrapper();
  FD_C_RuntimeOptionWrapperUseCpu(opt);
  FD_C_DBDetectorWrapper* det = FD_C_CreateDBDetectorWrapper(argv[1], argv[2], opt, FD_C_ModelFormat_PADDLE);
  FD_C_ClassifierWrapper* cls = FD_C_CreateClassifierWrapper(argv[3], argv[4], opt, FD_C_ModelFormat_PADDLE);
  FD_C_RecognizerWrapper* rec = FD_C_CreateRecognizerWrapper(argv[5], argv[6], argv[7], opt, FD_C_ModelFormat_PADDLE);
  if (!det || !cls || !rec) { fprintf(stderr, "create: %s\n", FD_C_GetLastError()); return 1; }
  printf("initialized=%d%d%d\n", (int)FD_C_DBDetectorWrapperInitialized(det), (int)FD_C_ClassifierWrapperInitialized(cls),
         (int)FD_C_RecognizerWrapperInitialized(rec));
  FD_C_Mat page;
  page.height = 64; page.width = 160; page.channels = 3;
  page.data = (uint8_t*)malloc(64 * 160 * 3);
  unsigned seed = 7u;
  for (int i = 0; i < 64 * 160 * 3; ++i) { seed = seed * 1664525u + 1013904223u; page.data[i] = (uint8_t)(seed >> 24); }
  FD_C_TwoDimArrayInt32 boxes;
  if (!FD_C_DBDetectorWrapperPredict(det, page, &boxes)) { fprintf(stderr, "det: %s\n", FD_C_GetLastError()); return 1; }
  int eights = 1;
  for (size_t i = 0; i < boxes.size; ++i) eights = eights && boxes.data[i].size == 8;
  printf("boxes=%zu all_have_8=%d\n", boxes.size, eights);
  FD_C_DestroyTwoDimArrayInt32(&boxes);
  int32_t label = -1;
  float score = -1.0f;
  if (!FD_C_ClassifierWrapperPredict(cls, page, &label, &score)) { fprintf(stderr, "cls: %s\n", FD_C_GetLastError()); return 1; }
  printf("cls=%d %.6f\n", label, score);
  char* text = NULL;
  float rec_score = -1.0f;
  if (!FD_C_RecognizerWrapperPredict(rec, page, &text, &rec_score)) { fprintf(stderr, "rec: %s\n", FD_C_GetLastError()); return 1; }
  printf("rec_bytes=%zu %.6f\n", strlen(text), rec_score);
  printf("rec_text=%s\n", text);
  FD_C_DestroyCstr(text);
  FD_C_DestroyDBDetectorWrapper(det); FD_C_DestroyClassifierWrapper(cls); FD_C_DestroyRecognizerWrapper(rec);
  FD_C_DBDetectorWrapper* bad = FD_C_CreateDBDetectorWrapper("/nonexistent/det.pdmodel", "", opt, FD_C_ModelFormat_PADDLE);
  printf("bad=%s\n", bad ? "non-null" : "null");
  free(page.data);
  FD_C_DestroyRuntimeOptionWrapper(opt);
  return 0;
}
