// JPEG decode on the GPU straight into a caller-provided device buffer (the pre-processing kernel's input), through
// nvJPEG resolved at run time: the library stays loadable on machines without libnvjpeg, where the decoder reports
// "unavailable" and the caller uses the host decoder.
//
// Counterpart: fastdeploy/vision/common/image_decoder/nvjpeg_decoder.cc:195-270 (decode into an FDMat on the device).
#include "fdb_common.h"

#include <dlfcn.h>
#include <nvjpeg.h>

#include <mutex>

namespace fdb {

struct NvJpegApi {
  void* lib = nullptr;
  nvjpegStatus_t (*CreateSimple)(nvjpegHandle_t*) = nullptr;
  nvjpegStatus_t (*Destroy)(nvjpegHandle_t) = nullptr;
  nvjpegStatus_t (*StateCreate)(nvjpegHandle_t, nvjpegJpegState_t*) = nullptr;
  nvjpegStatus_t (*StateDestroy)(nvjpegJpegState_t) = nullptr;
  nvjpegStatus_t (*GetImageInfo)(nvjpegHandle_t, const unsigned char*, size_t, int*, nvjpegChromaSubsampling_t*, int*,
                                 int*) = nullptr;
  nvjpegStatus_t (*Decode)(nvjpegHandle_t, nvjpegJpegState_t, const unsigned char*, size_t, nvjpegOutputFormat_t,
                           nvjpegImage_t*, cudaStream_t) = nullptr;
  bool ok = false;
};

static NvJpegApi& api() {
  static NvJpegApi a;
  static std::once_flag once;
  std::call_once(once, []() {
    for (const char* name : {"libnvjpeg.so.12", "libnvjpeg.so", "/usr/local/cuda/lib64/libnvjpeg.so.12"}) {
      a.lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (a.lib != nullptr) break;
    }
    if (a.lib == nullptr) return;
    a.CreateSimple = reinterpret_cast<decltype(a.CreateSimple)>(dlsym(a.lib, "nvjpegCreateSimple"));
    a.Destroy = reinterpret_cast<decltype(a.Destroy)>(dlsym(a.lib, "nvjpegDestroy"));
    a.StateCreate = reinterpret_cast<decltype(a.StateCreate)>(dlsym(a.lib, "nvjpegJpegStateCreate"));
    a.StateDestroy = reinterpret_cast<decltype(a.StateDestroy)>(dlsym(a.lib, "nvjpegJpegStateDestroy"));
    a.GetImageInfo = reinterpret_cast<decltype(a.GetImageInfo)>(dlsym(a.lib, "nvjpegGetImageInfo"));
    a.Decode = reinterpret_cast<decltype(a.Decode)>(dlsym(a.lib, "nvjpegDecode"));
    a.ok = a.CreateSimple && a.Destroy && a.StateCreate && a.StateDestroy && a.GetImageInfo && a.Decode;
  });
  return a;
}

// one handle and one decode state per host thread: nvJPEG states are not re-entrant
struct ThreadDecoder {
  nvjpegHandle_t handle = nullptr;
  nvjpegJpegState_t state = nullptr;
  ~ThreadDecoder() {
    NvJpegApi& a = api();
    if (state != nullptr && a.ok) a.StateDestroy(state);
    if (handle != nullptr && a.ok) a.Destroy(handle);
  }
};

static ThreadDecoder* decoder() {
  static thread_local ThreadDecoder d;
  NvJpegApi& a = api();
  if (!a.ok) return nullptr;
  if (d.handle == nullptr) {
    if (a.CreateSimple(&d.handle) != NVJPEG_STATUS_SUCCESS) { d.handle = nullptr; return nullptr; }
    if (a.StateCreate(d.handle, &d.state) != NVJPEG_STATUS_SUCCESS) { d.state = nullptr; return nullptr; }
  }
  return d.state != nullptr ? &d : nullptr;
}

}  // namespace fdb

using namespace fdb;

FDB_API int fdb_jpeg_available() { return api().ok ? 1 : 0; }

// Width, height and component count of an encoded image. Returns 0 on success.
FDB_API int fdb_jpeg_info(const unsigned char* data, long long len, int* width, int* height, int* components) {
  ThreadDecoder* d = decoder();
  if (d == nullptr) { set_error("jpeg: nvJPEG is not available"); return -1; }
  int comps = 0, widths[NVJPEG_MAX_COMPONENT] = {0}, heights[NVJPEG_MAX_COMPONENT] = {0};
  nvjpegChromaSubsampling_t sub;
  const nvjpegStatus_t st = api().GetImageInfo(d->handle, data, static_cast<size_t>(len), &comps, &sub, widths, heights);
  if (st != NVJPEG_STATUS_SUCCESS) { set_error("jpeg: not a decodable JPEG stream (status " + std::to_string(st) + ")"); return -1; }
  *width = widths[0];
  *height = heights[0];
  *components = comps;
  return 0;
}

// Decodes into dst (device memory, interleaved 3 x uint8 per pixel, row pitch in bytes >= 3 * width); bgr != 0 gives
// the channel order of cv::imread. The decode is queued on `stream`; dst must stay alive until it has run.
FDB_API int fdb_jpeg_decode(const unsigned char* data, long long len, void* dst, long long pitch, int bgr, void* stream) {
  ThreadDecoder* d = decoder();
  if (d == nullptr) { set_error("jpeg: nvJPEG is not available"); return -1; }
  int w = 0, h = 0, c = 0;
  if (fdb_jpeg_info(data, len, &w, &h, &c) != 0) return -1;
  if (pitch < 3LL * w) { set_error("jpeg: destination pitch is smaller than a row"); return -1; }
  nvjpegImage_t img{};
  img.channel[0] = static_cast<unsigned char*>(dst);
  img.pitch[0] = static_cast<size_t>(pitch);
  const nvjpegStatus_t st = api().Decode(d->handle, d->state, data, static_cast<size_t>(len),
                                         bgr ? NVJPEG_OUTPUT_BGRI : NVJPEG_OUTPUT_RGBI, &img, static_cast<cudaStream_t>(stream));
  if (st != NVJPEG_STATUS_SUCCESS) { set_error("jpeg: decode failed (status " + std::to_string(st) + ")"); return -1; }
  return 0;
}
