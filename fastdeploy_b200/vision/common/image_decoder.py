"""Image decoding: nvJPEG on the GPU (csrc/kernels/jpeg_decode.cu) straight into a device buffer - for example the
staging buffer the fused pre-processing kernel reads - or OpenCV on the host.

Counterpart of ``ImageDecoder`` with ``ImageDecoderLib.OPENCV / NVJPEG``
(fastdeploy/vision/common/image_decoder/image_decoder.h:24-49, nvjpeg_decoder.cc:195-270)."""
from __future__ import annotations

import ctypes
import enum
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np

from ... import _native


class ImageDecoderLib(enum.IntEnum):
    OPENCV = 0
    NVJPEG = 1


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_jpeg_ready", False):
        lib.fdb_jpeg_info.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.POINTER(ctypes.c_int),
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        lib.fdb_jpeg_decode.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                        ctypes.c_void_p]
        lib._jpeg_ready = True
    return lib


def nvjpeg_available() -> bool:
    import torch
    return _native.kernels_available() and torch.cuda.is_available() and bool(_lib().fdb_jpeg_available())


def jpeg_info(data: bytes) -> Tuple[int, int, int]:
    """(height, width, components) of an encoded JPEG."""
    w, h, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    if _lib().fdb_jpeg_info(data, len(data), ctypes.byref(w), ctypes.byref(h), ctypes.byref(c)) != 0:
        raise ValueError(_native.last_error())
    return h.value, w.value, c.value


class ImageDecoder:
    """``decode(data)`` / ``batch_decode(list)``: encoded bytes (or a file name) -> image. With ``NVJPEG`` the result is
    a ``uint8 [H, W, 3]`` torch tensor on the GPU in BGR order (what ``cv2.imread`` yields), and ``decode_into`` writes
    into memory the caller owns; with ``OPENCV`` it is a numpy array on the host."""

    def __init__(self, lib: ImageDecoderLib = ImageDecoderLib.OPENCV, device: int = 0):
        self.lib = ImageDecoderLib(lib)
        self.device = device
        if self.lib == ImageDecoderLib.NVJPEG and not nvjpeg_available():
            raise RuntimeError("ImageDecoderLib.NVJPEG: nvJPEG or a CUDA device is not available")

    @staticmethod
    def _bytes(data: Union[bytes, bytearray, str, np.ndarray]) -> bytes:
        if isinstance(data, str):
            with open(data, "rb") as f:
                return f.read()
        if isinstance(data, np.ndarray):
            return data.tobytes()
        return bytes(data)

    def decode_into(self, data, dst, bgr: bool = True) -> Tuple[int, int]:
        """Decodes into ``dst`` (a device uint8 tensor whose leading bytes take the ``H x W x 3`` image, e.g. a slice of a
        batch staging buffer) on the current stream; returns ``(H, W)``."""
        import torch
        from ...ops.base import current_stream_ptr
        raw = self._bytes(data)
        h, w, _ = jpeg_info(raw)
        assert dst.is_cuda and dst.dtype == torch.uint8 and dst.is_contiguous() and dst.numel() >= h * w * 3
        if _lib().fdb_jpeg_decode(raw, len(raw), ctypes.c_void_p(dst.data_ptr()), 3 * w, int(bgr),
                                  ctypes.c_void_p(current_stream_ptr(dst.device))) != 0:
            raise ValueError(_native.last_error())
        return h, w

    def decode(self, data, bgr: bool = True):
        raw = self._bytes(data)
        if self.lib == ImageDecoderLib.OPENCV:
            import cv2
            im = cv2.imdecode(np.frombuffer(raw, np.uint8), cv2.IMREAD_COLOR)
            if im is None:
                raise ValueError("image could not be decoded")
            return im if bgr else im[:, :, ::-1].copy()
        import torch
        h, w, _ = jpeg_info(raw)
        with torch.cuda.device(self.device):
            out = torch.empty(h, w, 3, dtype=torch.uint8, device=f"cuda:{self.device}")
            self.decode_into(raw, out, bgr)
        return out

    def batch_decode(self, items: Sequence, bgr: bool = True) -> List:
        return [self.decode(d, bgr) for d in items]
