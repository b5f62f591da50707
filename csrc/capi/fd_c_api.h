/* C API of the deployment library: opaque wrappers with FD_C_Create / Destroy / Predict entry points,
 * named after the reference's c_api/fastdeploy_capi (core/fd_type.h, runtime/runtime_option.h,
 * vision/result.h, vision/detection/ppdet/model.h, vision/classification/ppcls/model.h). The
 * implementation drives the Python package through an embedded interpreter, so one shared library
 * serves C, C# (P/Invoke) and Java (JNI) callers; images are plain interleaved BGR buffers. */
#ifndef FASTDEPLOY_B200_C_API_H_
#define FASTDEPLOY_B200_C_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FD_C_EXPORT __attribute__((visibility("default")))

typedef int8_t FD_C_Bool;

typedef enum { FD_C_ModelFormat_AUTOREC = 0, FD_C_ModelFormat_PADDLE = 1, FD_C_ModelFormat_ONNX = 2 } FD_C_ModelFormat;

typedef struct FD_C_OneDimArrayInt32 { size_t size; int32_t* data; } FD_C_OneDimArrayInt32;
typedef struct FD_C_OneDimArrayInt64 { size_t size; int64_t* data; } FD_C_OneDimArrayInt64;
typedef struct FD_C_OneDimArrayFloat { size_t size; float* data; } FD_C_OneDimArrayFloat;
typedef struct FD_C_TwoDimArrayFloat { size_t size; FD_C_OneDimArrayFloat* data; } FD_C_TwoDimArrayFloat;

/* interleaved uint8 image, BGR channel order (what cv::Mat holds in the reference) */
typedef struct FD_C_Mat { uint8_t* data; int height; int width; int channels; } FD_C_Mat;

typedef struct FD_C_ClassifyResult {
  FD_C_OneDimArrayInt32 label_ids;
  FD_C_OneDimArrayFloat scores;
} FD_C_ClassifyResult;

typedef struct FD_C_DetectionResult {
  FD_C_TwoDimArrayFloat boxes;        /* n x 4 */
  FD_C_OneDimArrayFloat scores;
  FD_C_OneDimArrayInt32 label_ids;
} FD_C_DetectionResult;

typedef struct FD_C_Tensor {
  const char* name;
  int dtype;                          /* 0 float32, 1 int64, 2 int32, 3 uint8 */
  FD_C_OneDimArrayInt64 shape;
  void* data;
  size_t nbytes;
} FD_C_Tensor;

typedef struct FD_C_RuntimeOptionWrapper FD_C_RuntimeOptionWrapper;
typedef struct FD_C_RuntimeWrapper FD_C_RuntimeWrapper;
typedef struct FD_C_ModelWrapper FD_C_ModelWrapper;
typedef FD_C_ModelWrapper FD_C_PPYOLOEWrapper;
typedef FD_C_ModelWrapper FD_C_PaddleClasModelWrapper;

/* last error text of the calling thread ("" when none) */
FD_C_EXPORT const char* FD_C_GetLastError(void);

/* ---- RuntimeOption */
FD_C_EXPORT FD_C_RuntimeOptionWrapper* FD_C_CreateRuntimeOptionWrapper(void);
FD_C_EXPORT void FD_C_DestroyRuntimeOptionWrapper(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetModelPath(FD_C_RuntimeOptionWrapper* w, const char* model_path,
                                                       const char* params_path, FD_C_ModelFormat format);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseCpu(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseGpu(FD_C_RuntimeOptionWrapper* w, int gpu_id);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetCpuThreadNum(FD_C_RuntimeOptionWrapper* w, int thread_num);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUsePaddleBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUsePaddleInferBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseOrtBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseTrtBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseOpenVINOBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnableTrtFP16(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDisableTrtFP16(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetTrtCacheFile(FD_C_RuntimeOptionWrapper* w, const char* path);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnablePinnedMemory(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDisablePinnedMemory(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetEncryptionKey(FD_C_RuntimeOptionWrapper* w, const char* key);

/* the rest of the reference's option entry points (c_api/fastdeploy_capi/runtime/runtime_option.h:40-500). Options that
 * name another vendor's device or library are recorded on the option object and change nothing about execution. */
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetModelBuffer(FD_C_RuntimeOptionWrapper* w, const char* model_buffer, size_t model_size,
                                                         const char* params_buffer, size_t params_size, FD_C_ModelFormat format);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseTimVX(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseAscend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseSophgo(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseKunlunXin(FD_C_RuntimeOptionWrapper* w, int kunlunxin_id, int l3_workspace_size,
                                                       FD_C_Bool locked, FD_C_Bool autotune, const char* autotune_file,
                                                       const char* precision, FD_C_Bool adaptive_seqlen,
                                                       FD_C_Bool enable_multi_stream, int64_t gm_default_size);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseIpu(FD_C_RuntimeOptionWrapper* w, int device_num, int micro_batch_size,
                                                 FD_C_Bool enable_pipelining, int batches_per_step);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetExternalStream(FD_C_RuntimeOptionWrapper* w, void* external_stream);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetOrtGraphOptLevel(FD_C_RuntimeOptionWrapper* w, int level);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseSophgoBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUsePorosBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUseLiteBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperUsePaddleLiteBackend(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetPaddleMKLDNN(FD_C_RuntimeOptionWrapper* w, FD_C_Bool pd_mkldnn);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnablePaddleToTrt(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDeletePaddleBackendPass(FD_C_RuntimeOptionWrapper* w, const char* delete_pass_name);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnablePaddleLogInfo(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDisablePaddleLogInfo(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetPaddleMKLDNNCacheSize(FD_C_RuntimeOptionWrapper* w, int size);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetOpenVINODevice(FD_C_RuntimeOptionWrapper* w, const char* name);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetOpenVINOStreams(FD_C_RuntimeOptionWrapper* w, int num_streams);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLiteOptimizedModelDir(FD_C_RuntimeOptionWrapper* w, const char* dir);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLiteSubgraphPartitionPath(FD_C_RuntimeOptionWrapper* w, const char* path);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLiteSubgraphPartitionConfigBuffer(FD_C_RuntimeOptionWrapper* w, const char* buffer);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLiteContextProperties(FD_C_RuntimeOptionWrapper* w, const char* properties);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLiteModelCacheDir(FD_C_RuntimeOptionWrapper* w, const char* dir);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLiteMixedPrecisionQuantizationConfigPath(FD_C_RuntimeOptionWrapper* w, const char* path);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnableLiteFP16(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDisableLiteFP16(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnableLiteInt8(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDisableLiteInt8(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperSetLitePowerMode(FD_C_RuntimeOptionWrapper* w, int mode);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperEnablePaddleTrtCollectShape(FD_C_RuntimeOptionWrapper* w);
FD_C_EXPORT void FD_C_RuntimeOptionWrapperDisablePaddleTrtCollectShape(FD_C_RuntimeOptionWrapper* w);

/* ---- Runtime (generic tensors in, tensors out) */
FD_C_EXPORT FD_C_RuntimeWrapper* FD_C_CreateRuntimeWrapper(FD_C_RuntimeOptionWrapper* option);
FD_C_EXPORT void FD_C_DestroyRuntimeWrapper(FD_C_RuntimeWrapper* w);
FD_C_EXPORT int FD_C_RuntimeWrapperNumInputs(FD_C_RuntimeWrapper* w);
FD_C_EXPORT int FD_C_RuntimeWrapperNumOutputs(FD_C_RuntimeWrapper* w);
/* outputs[i].data / shape.data are allocated by the library: release with FD_C_DestroyTensors */
FD_C_EXPORT FD_C_Bool FD_C_RuntimeWrapperInfer(FD_C_RuntimeWrapper* w, const FD_C_Tensor* inputs, int n_inputs,
                                               FD_C_Tensor* outputs, int max_outputs, int* n_outputs);
FD_C_EXPORT void FD_C_DestroyTensors(FD_C_Tensor* tensors, int n);

/* ---- vision models */
FD_C_EXPORT FD_C_PPYOLOEWrapper* FD_C_CreatePPYOLOEWrapper(const char* model_file, const char* params_file,
                                                           const char* config_file, FD_C_RuntimeOptionWrapper* option,
                                                           FD_C_ModelFormat format);
FD_C_EXPORT void FD_C_DestroyPPYOLOEWrapper(FD_C_PPYOLOEWrapper* w);
FD_C_EXPORT FD_C_Bool FD_C_PPYOLOEWrapperPredict(FD_C_PPYOLOEWrapper* w, FD_C_Mat img, FD_C_DetectionResult* result);
FD_C_EXPORT FD_C_Bool FD_C_PPYOLOEWrapperInitialized(FD_C_PPYOLOEWrapper* w);

FD_C_EXPORT FD_C_PaddleClasModelWrapper* FD_C_CreatePaddleClasModelWrapper(const char* model_file, const char* params_file,
                                                                           const char* config_file,
                                                                           FD_C_RuntimeOptionWrapper* option,
                                                                           FD_C_ModelFormat format);
FD_C_EXPORT void FD_C_DestroyPaddleClasModelWrapper(FD_C_PaddleClasModelWrapper* w);
FD_C_EXPORT FD_C_Bool FD_C_PaddleClasModelWrapperPredict(FD_C_PaddleClasModelWrapper* w, FD_C_Mat img,
                                                         FD_C_ClassifyResult* result);

/* any detection class of the Python package by name ("PicoDet", "YOLOv5", ...) */
FD_C_EXPORT FD_C_ModelWrapper* FD_C_CreateDetectionModelWrapper(const char* class_name, const char* model_file,
                                                                const char* params_file, const char* config_file,
                                                                FD_C_RuntimeOptionWrapper* option, FD_C_ModelFormat format);
FD_C_EXPORT FD_C_Bool FD_C_DetectionModelWrapperPredict(FD_C_ModelWrapper* w, FD_C_Mat img, FD_C_DetectionResult* result);
FD_C_EXPORT void FD_C_DestroyModelWrapper(FD_C_ModelWrapper* w);

/* a batch of images through any detection model (c_api/fastdeploy_capi/vision/detection/ppdet/base_define.h:73-115):
 * results[i] is filled for every image; release each with FD_C_DestroyDetectionResult */
FD_C_EXPORT FD_C_Bool FD_C_DetectionModelWrapperBatchPredict(FD_C_ModelWrapper* w, const FD_C_Mat* imgs, int n_imgs,
                                                             FD_C_DetectionResult* results);

/* ---- segmentation (c_api/fastdeploy_capi/vision/segmentation/ppseg/model.h) */
typedef struct FD_C_SegmentationResult {
  FD_C_OneDimArrayInt32 label_map;    /* height * width class ids */
  FD_C_OneDimArrayFloat score_map;    /* empty unless the model returns scores */
  int height, width;
  FD_C_Bool contain_score_map;
} FD_C_SegmentationResult;
typedef FD_C_ModelWrapper FD_C_PaddleSegModelWrapper;
FD_C_EXPORT FD_C_PaddleSegModelWrapper* FD_C_CreatePaddleSegModelWrapper(const char* model_file, const char* params_file,
                                                                         const char* config_file,
                                                                         FD_C_RuntimeOptionWrapper* option,
                                                                         FD_C_ModelFormat format);
FD_C_EXPORT FD_C_Bool FD_C_PaddleSegModelWrapperPredict(FD_C_PaddleSegModelWrapper* w, FD_C_Mat img,
                                                        FD_C_SegmentationResult* result);
FD_C_EXPORT void FD_C_DestroySegmentationResult(FD_C_SegmentationResult* r);

/* ---- OCR (c_api/fastdeploy_capi/vision/ocr/ppocr/model.h): detector + optional classifier + recogniser */
typedef struct FD_C_OCRResult {
  FD_C_TwoDimArrayFloat boxes;        /* n x 8 corner coordinates */
  size_t n_text;
  char** text;                        /* n_text UTF-8 strings */
  FD_C_OneDimArrayFloat rec_scores;
  FD_C_OneDimArrayFloat cls_scores;
  FD_C_OneDimArrayInt32 cls_labels;
} FD_C_OCRResult;
typedef FD_C_ModelWrapper FD_C_PPOCRv3Wrapper;
/* cls_model_file may be NULL or "" for a pipeline without the angle classifier */
FD_C_EXPORT FD_C_PPOCRv3Wrapper* FD_C_CreatePPOCRv3Wrapper(const char* det_model_file, const char* det_params_file,
                                                           const char* cls_model_file, const char* cls_params_file,
                                                           const char* rec_model_file, const char* rec_params_file,
                                                           const char* rec_label_file, FD_C_RuntimeOptionWrapper* option);
FD_C_EXPORT FD_C_Bool FD_C_PPOCRv3WrapperPredict(FD_C_PPOCRv3Wrapper* w, FD_C_Mat img, FD_C_OCRResult* result);
FD_C_EXPORT void FD_C_DestroyOCRResult(FD_C_OCRResult* r);

/* ---- visualisation (c_api/fastdeploy_capi/vision/visualize.h): draws into `out`, an image of the input's size that
 * the caller owns (out->data must hold height * width * channels bytes) */
FD_C_EXPORT FD_C_Bool FD_C_VisDetection(FD_C_Mat img, const FD_C_DetectionResult* result, float score_threshold,
                                        int line_size, float font_size, FD_C_Mat* out);
FD_C_EXPORT FD_C_Bool FD_C_VisSegmentation(FD_C_Mat img, const FD_C_SegmentationResult* result, float weight, FD_C_Mat* out);

/* ---- the detection classes by name (c_api/fastdeploy_capi/vision/detection/ppdet/model.h,
 * vision/detection/contrib/yolo/model.h): FD_C_Create<T>Wrapper, FD_C_Destroy<T>Wrapper, FD_C_<T>WrapperPredict,
 * FD_C_<T>WrapperInitialized, FD_C_<T>WrapperBatchPredict for every T below. The PaddleDetection exports take a config
 * file; the YOLO family (ONNX exports) does not. */
#define FD_C_PPDET_MODELS(X)                                                                                              \
  X(PicoDet) X(PPYOLO) X(YOLOv3) X(PaddleYOLOX) X(FasterRCNN) X(MaskRCNN) X(SSD) X(PaddleYOLOv5) X(PaddleYOLOv6)          \
  X(PaddleYOLOv7) X(PaddleYOLOv8) X(RTMDet) X(CascadeRCNN) X(PSSDet) X(RetinaNet) X(FCOS) X(TTFNet) X(TOOD) X(GFL)
#define FD_C_YOLO_MODELS(X) X(YOLOv5) X(YOLOv7) X(YOLOv8) X(YOLOv6) X(YOLOR) X(YOLOX)

#define FD_C_DECLARE_DETECTION_COMMON(T)                                                                                  \
  typedef FD_C_ModelWrapper FD_C_##T##Wrapper;                                                                            \
  FD_C_EXPORT void FD_C_Destroy##T##Wrapper(FD_C_##T##Wrapper* w);                                                        \
  FD_C_EXPORT FD_C_Bool FD_C_##T##WrapperPredict(FD_C_##T##Wrapper* w, FD_C_Mat img, FD_C_DetectionResult* result);       \
  FD_C_EXPORT FD_C_Bool FD_C_##T##WrapperInitialized(FD_C_##T##Wrapper* w);                                               \
  FD_C_EXPORT FD_C_Bool FD_C_##T##WrapperBatchPredict(FD_C_##T##Wrapper* w, const FD_C_Mat* imgs, int n_imgs,             \
                                                      FD_C_DetectionResult* results);
#define FD_C_DECLARE_PPDET(T)                                                                                             \
  FD_C_DECLARE_DETECTION_COMMON(T)                                                                                        \
  FD_C_EXPORT FD_C_##T##Wrapper* FD_C_Create##T##Wrapper(const char* model_file, const char* params_file,                 \
                                                         const char* config_file, FD_C_RuntimeOptionWrapper* option,      \
                                                         FD_C_ModelFormat format);
#define FD_C_DECLARE_YOLO(T)                                                                                              \
  FD_C_DECLARE_DETECTION_COMMON(T)                                                                                        \
  FD_C_EXPORT FD_C_##T##Wrapper* FD_C_Create##T##Wrapper(const char* model_file, const char* params_file,                 \
                                                         FD_C_RuntimeOptionWrapper* option, FD_C_ModelFormat format);
FD_C_PPDET_MODELS(FD_C_DECLARE_PPDET)
FD_C_YOLO_MODELS(FD_C_DECLARE_YOLO)
FD_C_EXPORT FD_C_Bool FD_C_PPYOLOEWrapperBatchPredict(FD_C_PPYOLOEWrapper* w, const FD_C_Mat* imgs, int n_imgs,
                                                      FD_C_DetectionResult* results);

/* ---- classification and segmentation: batches and the initialised flag */
FD_C_EXPORT FD_C_Bool FD_C_PaddleClasModelWrapperInitialized(FD_C_PaddleClasModelWrapper* w);
FD_C_EXPORT FD_C_Bool FD_C_PaddleClasModelWrapperBatchPredict(FD_C_PaddleClasModelWrapper* w, const FD_C_Mat* imgs, int n_imgs,
                                                              FD_C_ClassifyResult* results);
FD_C_EXPORT void FD_C_DestroyPaddleSegModelWrapper(FD_C_PaddleSegModelWrapper* w);
FD_C_EXPORT FD_C_Bool FD_C_PaddleSegModelWrapperInitialized(FD_C_PaddleSegModelWrapper* w);
FD_C_EXPORT FD_C_Bool FD_C_PaddleSegModelWrapperBatchPredict(FD_C_PaddleSegModelWrapper* w, const FD_C_Mat* imgs, int n_imgs,
                                                             FD_C_SegmentationResult* results);

/* ---- OCR: the pipeline of the previous generation and batches (c_api/fastdeploy_capi/vision/ocr/ppocr/model.h:330-460) */
typedef FD_C_ModelWrapper FD_C_PPOCRv2Wrapper;
FD_C_EXPORT FD_C_PPOCRv2Wrapper* FD_C_CreatePPOCRv2Wrapper(const char* det_model_file, const char* det_params_file,
                                                           const char* cls_model_file, const char* cls_params_file,
                                                           const char* rec_model_file, const char* rec_params_file,
                                                           const char* rec_label_file, FD_C_RuntimeOptionWrapper* option);
FD_C_EXPORT FD_C_Bool FD_C_PPOCRv2WrapperPredict(FD_C_PPOCRv2Wrapper* w, FD_C_Mat img, FD_C_OCRResult* result);
FD_C_EXPORT FD_C_Bool FD_C_PPOCRv2WrapperBatchPredict(FD_C_PPOCRv2Wrapper* w, const FD_C_Mat* imgs, int n_imgs, FD_C_OCRResult* results);
FD_C_EXPORT FD_C_Bool FD_C_PPOCRv3WrapperBatchPredict(FD_C_PPOCRv3Wrapper* w, const FD_C_Mat* imgs, int n_imgs, FD_C_OCRResult* results);
FD_C_EXPORT void FD_C_DestroyPPOCRv2Wrapper(FD_C_PPOCRv2Wrapper* w);
FD_C_EXPORT void FD_C_DestroyPPOCRv3Wrapper(FD_C_PPOCRv3Wrapper* w);

/* ---- the three OCR stages on their own (c_api/fastdeploy_capi/vision/ocr/ppocr/model.h:30-330) */
typedef struct FD_C_TwoDimArrayInt32 { size_t size; FD_C_OneDimArrayInt32* data; } FD_C_TwoDimArrayInt32;
typedef FD_C_ModelWrapper FD_C_DBDetectorWrapper;
typedef FD_C_ModelWrapper FD_C_ClassifierWrapper;
typedef FD_C_ModelWrapper FD_C_RecognizerWrapper;
FD_C_EXPORT FD_C_DBDetectorWrapper* FD_C_CreateDBDetectorWrapper(const char* model_file, const char* params_file,
                                                                 FD_C_RuntimeOptionWrapper* option, FD_C_ModelFormat format);
/* boxes->data[i] holds the 8 corner coordinates of text box i; release with FD_C_DestroyTwoDimArrayInt32 */
FD_C_EXPORT FD_C_Bool FD_C_DBDetectorWrapperPredict(FD_C_DBDetectorWrapper* w, FD_C_Mat img, FD_C_TwoDimArrayInt32* boxes);
FD_C_EXPORT FD_C_Bool FD_C_DBDetectorWrapperInitialized(FD_C_DBDetectorWrapper* w);
FD_C_EXPORT void FD_C_DestroyDBDetectorWrapper(FD_C_DBDetectorWrapper* w);
FD_C_EXPORT FD_C_ClassifierWrapper* FD_C_CreateClassifierWrapper(const char* model_file, const char* params_file,
                                                                 FD_C_RuntimeOptionWrapper* option, FD_C_ModelFormat format);
FD_C_EXPORT FD_C_Bool FD_C_ClassifierWrapperPredict(FD_C_ClassifierWrapper* w, FD_C_Mat img, int32_t* cls_label, float* cls_score);
FD_C_EXPORT FD_C_Bool FD_C_ClassifierWrapperInitialized(FD_C_ClassifierWrapper* w);
FD_C_EXPORT void FD_C_DestroyClassifierWrapper(FD_C_ClassifierWrapper* w);
FD_C_EXPORT FD_C_RecognizerWrapper* FD_C_CreateRecognizerWrapper(const char* model_file, const char* params_file,
                                                                 const char* label_path, FD_C_RuntimeOptionWrapper* option,
                                                                 FD_C_ModelFormat format);
/* *text is a UTF-8 string the library allocates; release with FD_C_DestroyCstr */
FD_C_EXPORT FD_C_Bool FD_C_RecognizerWrapperPredict(FD_C_RecognizerWrapper* w, FD_C_Mat img, char** text, float* rec_score);
FD_C_EXPORT FD_C_Bool FD_C_RecognizerWrapperInitialized(FD_C_RecognizerWrapper* w);
FD_C_EXPORT void FD_C_DestroyRecognizerWrapper(FD_C_RecognizerWrapper* w);
FD_C_EXPORT void FD_C_DestroyTwoDimArrayInt32(FD_C_TwoDimArrayInt32* a);
FD_C_EXPORT void FD_C_DestroyCstr(char* text);

/* ---- images (c_api/fastdeploy_capi/core/fd_type.h:150-165). FD_C_Imread returns a BGR image whose pixels the library
 * owns (data is NULL on failure); release it with FD_C_DestroyMat. */
FD_C_EXPORT FD_C_Mat FD_C_Imread(const char* path);
FD_C_EXPORT FD_C_Bool FD_C_Imwrite(const char* path, FD_C_Mat img);
FD_C_EXPORT void FD_C_DestroyMat(FD_C_Mat img);

/* ---- result text, the reference's Str(): writes at most `capacity` bytes including the terminator and returns the
 * length the whole text needs (c_api/fastdeploy_capi/vision/result.h: FD_C_*ResultStr) */
FD_C_EXPORT size_t FD_C_ClassifyResultStr(const FD_C_ClassifyResult* r, char* buffer, size_t capacity);
FD_C_EXPORT size_t FD_C_DetectionResultStr(const FD_C_DetectionResult* r, char* buffer, size_t capacity);
FD_C_EXPORT size_t FD_C_OCRResultStr(const FD_C_OCRResult* r, char* buffer, size_t capacity);
FD_C_EXPORT size_t FD_C_SegmentationResultStr(const FD_C_SegmentationResult* r, char* buffer, size_t capacity);

/* ---- more visualisers (c_api/fastdeploy_capi/vision/visualize.h:40-100) */
FD_C_EXPORT FD_C_Bool FD_C_VisDetectionWithLabel(FD_C_Mat img, const FD_C_DetectionResult* result, const char* const* labels,
                                                 int n_labels, float score_threshold, int line_size, float font_size, FD_C_Mat* out);
FD_C_EXPORT FD_C_Bool FD_C_VisOcr(FD_C_Mat img, const FD_C_OCRResult* result, FD_C_Mat* out);

/* ---- results */
FD_C_EXPORT void FD_C_DestroyClassifyResult(FD_C_ClassifyResult* r);
FD_C_EXPORT void FD_C_DestroyDetectionResult(FD_C_DetectionResult* r);

#ifdef __cplusplus
}
#endif
#endif
