"""The processor framework: ``FDMat``, the 17 image processors, ``FuseTransforms`` and
``ProcessorManager`` (fastdeploy/vision/common/processors/{base,mat,manager,transform}.*).

Each processor keeps the reference's constructor signature and OpenCV semantics. Two
implementations exist per processor chain instead of the reference's four libraries: the CPU
path below (cv2 / numpy, also the oracle of the tests) and the fused CUDA path
(:func:`run_chain_gpu`), which compiles a whole chain of geometric + photometric processors into
ONE launch of the pre-processing kernel (csrc/kernels/preproc.cu)."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np


class FDMat:
    """HWC image with layout / device bookkeeping (fastdeploy/vision/common/processors/mat.h:34-169)."""

    def __init__(self, mat: Optional[np.ndarray] = None, layout: str = "HWC"):
        self.mat = mat
        self.layout = layout

    def from_numpy(self, image: np.ndarray) -> "FDMat":
        """Takes an HWC image (the array is shared, not copied)."""
        self.mat, self.layout = np.asarray(image), "HWC"
        return self

    def numpy(self) -> np.ndarray:
        return self.mat

    def print_info(self, flag: str = "") -> str:
        """One line with type, channels, size and the per-channel mean (fastdeploy/vision/common/processors/mat.cc:149-188)."""
        chans = self.channels()
        means = (self.mat.reshape(self.height(), self.width(), -1).mean((0, 1)) if self.layout == "HWC" or self.mat.ndim < 3
                 else self.mat.reshape(chans, -1).mean(1))
        msg = (f"{flag}: DataType={self.mat.dtype}, Channel={chans}, Height={self.height()}, Width={self.width()}, Mean="
               + " ".join(f"{float(m):g}" for m in means))
        print(msg)
        return msg

    def height(self) -> int:
        return self.mat.shape[0] if self.layout == "HWC" else self.mat.shape[1]

    def width(self) -> int:
        return self.mat.shape[1] if self.layout == "HWC" else self.mat.shape[2]

    def channels(self) -> int:
        return (self.mat.shape[2] if self.mat.ndim == 3 else 1) if self.layout == "HWC" else self.mat.shape[0]

    Height, Width, Channels = height, width, channels


class FDMatBatch:
    """A list of images that the processors treat as one batch
    (fastdeploy/vision/common/processors/mat_batch.h:27-110). ``tensor()`` stacks them once every image has the same
    shape."""

    def __init__(self, mats: Optional[Sequence[FDMat]] = None):
        self.mats: List[FDMat] = list(mats) if mats is not None else []
        self.input_cache = None
        self.output_cache = None

    def from_mats(self, mats: Sequence) -> "FDMatBatch":
        self.mats = [m if isinstance(m, FDMat) else FDMat(np.asarray(m)) for m in mats]
        return self

    def __len__(self) -> int:
        return len(self.mats)

    @property
    def layout(self) -> str:
        return "N" + (self.mats[0].layout if self.mats else "HWC")

    def tensor(self) -> np.ndarray:
        shapes = {m.mat.shape for m in self.mats}
        if len(shapes) != 1:
            raise ValueError(f"the images of the batch differ in shape: {sorted(shapes)}")
        return np.stack([m.mat for m in self.mats])


class Processor:
    def name(self) -> str:
        return type(self).__name__

    Name = name

    def __call__(self, mat) -> bool:
        if isinstance(mat, FDMatBatch):         # image by image, as base.cc:24-60 does without a batched kernel
            ok = True
            for m in mat.mats:
                ok = self.impl(m) and ok
            return ok
        return self.impl(mat)

    def impl(self, mat: FDMat) -> bool:
        raise NotImplementedError


def _cv2():
    import cv2
    return cv2


class Resize(Processor):
    def __init__(self, width: int, height: int, scale_w: float = -1.0, scale_h: float = -1.0, interp: int = 1,
                 use_scale: bool = False):
        self.width, self.height, self.scale_w, self.scale_h, self.interp, self.use_scale = \
            width, height, scale_w, scale_h, interp, use_scale

    def target(self, h: int, w: int) -> Tuple[int, int]:
        if self.use_scale and self.scale_w > 0 and self.scale_h > 0:
            return int(round(h * self.scale_h)), int(round(w * self.scale_w))
        if self.width > 0 and self.height > 0:
            return self.height, self.width
        return h, w

    def set_width_and_height(self, width: int, height: int):
        self.width, self.height = width, height

    def impl(self, mat):
        th, tw = self.target(mat.height(), mat.width())
        if (th, tw) != (mat.height(), mat.width()):
            mat.mat = _cv2().resize(mat.mat, (tw, th), interpolation=self.interp)
        return True


class ResizeByShort(Processor):
    def __init__(self, target_size: int, interp: int = 1, use_scale: bool = True, max_hw: Sequence[int] = ()):
        self.target_size, self.interp, self.use_scale, self.max_hw = target_size, interp, use_scale, list(max_hw)

    def scale(self, h: int, w: int) -> float:
        """GenerateScale of the reference (resize_by_short.cc:156-180)."""
        s = self.target_size / min(h, w)
        if self.max_hw:
            if round(s * h) > self.max_hw[0]:
                s = self.max_hw[0] / h
            if round(s * w) > self.max_hw[1]:
                s = self.max_hw[1] / w
        return s

    def target(self, h: int, w: int) -> Tuple[int, int]:
        s = self.scale(h, w)
        return int(round(h * s)), int(round(w * s))

    def impl(self, mat):
        th, tw = self.target(mat.height(), mat.width())
        if (th, tw) != (mat.height(), mat.width()):
            mat.mat = _cv2().resize(mat.mat, (tw, th), interpolation=self.interp)
        return True


class CenterCrop(Processor):
    def __init__(self, width: int, height: int):
        self.width, self.height = width, height

    def impl(self, mat):
        h, w = mat.height(), mat.width()
        if h < self.height or w < self.width:
            raise ValueError("[CenterCrop] Image size less than crop size")
        x, y = (w - self.width) // 2, (h - self.height) // 2
        mat.mat = np.ascontiguousarray(mat.mat[y:y + self.height, x:x + self.width])
        return True


class Crop(Processor):
    def __init__(self, offset_w: int, offset_h: int, width: int, height: int):
        self.ow, self.oh, self.width, self.height = offset_w, offset_h, width, height

    def impl(self, mat):
        if self.oh + self.height > mat.height() or self.ow + self.width > mat.width():
            raise ValueError("[Crop] crop window exceeds the image")
        mat.mat = np.ascontiguousarray(mat.mat[self.oh:self.oh + self.height, self.ow:self.ow + self.width])
        return True


class Pad(Processor):
    def __init__(self, top: int, bottom: int, left: int, right: int, value: Sequence[float]):
        self.t, self.b, self.l, self.r, self.value = top, bottom, left, right, list(value)

    def impl(self, mat):
        c = mat.channels()
        if len(self.value) not in (1, c):
            raise ValueError("[Pad] value size must equal the channel count")
        val = self.value if len(self.value) == c else self.value * c
        mat.mat = _cv2().copyMakeBorder(mat.mat, self.t, self.b, self.l, self.r, _cv2().BORDER_CONSTANT, value=val)
        return True


class PadToSize(Processor):
    def __init__(self, width: int, height: int, value: Sequence[float] = (0, 0, 0)):
        self.width, self.height, self.value = width, height, list(value)

    def set_width_height(self, width: int, height: int):
        self.width, self.height = width, height

    SetWidthHeight = set_width_height

    def impl(self, mat):
        h, w = mat.height(), mat.width()
        if w > self.width or h > self.height:
            raise ValueError("[PadToSize] image is larger than the target size")
        if (h, w) == (self.height, self.width):
            return True
        return Pad(0, self.height - h, 0, self.width - w, self.value).impl(mat)


class StridePad(Processor):
    def __init__(self, stride: int, value: Sequence[float] = (0, 0, 0)):
        self.stride, self.value = stride, list(value)

    def impl(self, mat):
        h, w = mat.height(), mat.width()
        ph = (self.stride - h % self.stride) % self.stride
        pw = (self.stride - w % self.stride) % self.stride
        if ph == 0 and pw == 0:
            return True
        return Pad(0, ph, 0, pw, self.value).impl(mat)


class LimitByStride(Processor):
    def __init__(self, stride: int = 32, interp: int = 1):
        self.stride, self.interp = stride, interp

    def impl(self, mat):
        h, w = mat.height(), mat.width()
        nh, nw = max(h // self.stride * self.stride, self.stride), max(w // self.stride * self.stride, self.stride)
        if (nh, nw) != (h, w):
            mat.mat = _cv2().resize(mat.mat, (nw, nh), interpolation=self.interp)
        return True


class LimitShort(Processor):
    def __init__(self, max_short: int = -1, min_short: int = -1, interp: int = 1):
        self.max_short, self.min_short, self.interp = max_short, min_short, interp

    def impl(self, mat):
        h, w = mat.height(), mat.width()
        short = min(h, w)
        target = short
        if self.max_short > 0 and short > self.max_short:
            target = self.max_short
        elif self.min_short > 0 and short < self.min_short:
            target = self.min_short
        if target != short:
            s = target / short
            mat.mat = _cv2().resize(mat.mat, None, fx=s, fy=s, interpolation=self.interp)
        return True


class Normalize(Processor):
    """alpha = 1 / ((max - min) * std) (when is_scale), beta = -(mean + min * alpha0) / std
    (fastdeploy/vision/common/processors/normalize.cc:23-55)."""

    def __init__(self, mean: Sequence[float], std: Sequence[float], is_scale: bool = True,
                 min: Sequence[float] = (), max: Sequence[float] = (), swap_rb: bool = False):   # noqa: A002
        from ...ops.preproc import normalize_coeffs
        n = len(mean)
        lo = list(min) if len(min) else [0.0] * n
        hi = list(max) if len(max) else [255.0] * n
        self.alpha, self.beta = normalize_coeffs(list(mean), list(std), is_scale, lo, hi)
        self.swap_rb = swap_rb

    def impl(self, mat):
        x = mat.mat.astype(np.float32)
        if self.swap_rb:
            x = x[..., ::-1]
        mat.mat = x * np.asarray(self.alpha, np.float32) + np.asarray(self.beta, np.float32)
        return True


class HWC2CHW(Processor):
    def impl(self, mat):
        if mat.layout != "HWC":
            raise ValueError("HWC2CHW: The input data is not Layout::HWC format!")
        mat.mat = np.ascontiguousarray(mat.mat.transpose(2, 0, 1))
        mat.layout = "CHW"
        return True


class NormalizeAndPermute(Normalize):
    def impl(self, mat):
        super().impl(mat)
        return HWC2CHW().impl(mat)


class Cast(Processor):
    def __init__(self, dtype: str = "float"):
        self.dtype = dtype

    def impl(self, mat):
        mat.mat = mat.mat.astype({"float": np.float32, "double": np.float64, "uint8": np.uint8}.get(self.dtype, np.float32))
        return True


class Convert(Processor):
    def __init__(self, alpha: Sequence[float], beta: Sequence[float]):
        self.alpha, self.beta = list(alpha), list(beta)

    def impl(self, mat):
        mat.mat = mat.mat.astype(np.float32) * np.asarray(self.alpha, np.float32) + np.asarray(self.beta, np.float32)
        return True


class ConvertAndPermute(Convert):
    def __init__(self, alpha, beta, swap_rb: bool = False):
        super().__init__(alpha, beta)
        self.swap_rb = swap_rb

    def impl(self, mat):
        if self.swap_rb:
            mat.mat = mat.mat[..., ::-1]
        super().impl(mat)
        return HWC2CHW().impl(mat)


class _Color(Processor):
    code = None

    def impl(self, mat):
        mat.mat = _cv2().cvtColor(mat.mat, getattr(_cv2(), self.code))
        return True


class BGR2RGB(_Color): code = "COLOR_BGR2RGB"
class RGB2BGR(_Color): code = "COLOR_RGB2BGR"
class BGR2GRAY(_Color): code = "COLOR_BGR2GRAY"
class RGB2GRAY(_Color): code = "COLOR_RGB2GRAY"


class WarpAffine(Processor):
    def __init__(self, trans_matrix: np.ndarray, width: int, height: int, interp: int = 1, border_mode: int = 0,
                 border_value=(0, 0, 0)):
        self.m, self.width, self.height, self.interp, self.border_mode, self.border_value = \
            np.asarray(trans_matrix, np.float64), width, height, interp, border_mode, border_value

    def impl(self, mat):
        mat.mat = _cv2().warpAffine(mat.mat, self.m, (self.width, self.height), flags=self.interp,
                                    borderMode=self.border_mode, borderValue=self.border_value)
        return True


class LetterBoxResize(Processor):
    """Keep-ratio resize then centre pad (fastdeploy/vision/tracking/pptracking/letter_box_resize.cc)."""

    def __init__(self, target_size: Sequence[int], color: Sequence[float] = (127.5, 127.5, 127.5)):
        self.target_size, self.color = list(target_size), list(color)

    def impl(self, mat):
        h, w = mat.height(), mat.width()
        th, tw = self.target_size
        r = min(th / h, tw / w)
        nh, nw = int(round(h * r)), int(round(w * r))
        mat.mat = _cv2().resize(mat.mat, (nw, nh), interpolation=_cv2().INTER_AREA)
        top, left = int(round((th - nh) / 2 - 0.1)), int(round((tw - nw) / 2 - 0.1))
        return Pad(top, th - nh - top, left, tw - nw - left, self.color).impl(mat)


def fuse_transforms(processors: List[Processor]) -> List[Processor]:
    """Normalize+Cast -> Normalize; Normalize+HWC2CHW -> NormalizeAndPermute; a BGR2RGB / RGB2BGR anywhere
    before the Normalize folds into its ``swap_rb`` (fastdeploy/vision/common/processors/transform.cc:19-171)."""
    procs = list(processors)
    norm_idx = next((i for i, p in enumerate(procs) if type(p) in (Normalize, NormalizeAndPermute)), None)
    if norm_idx is not None:
        for i in range(norm_idx):
            if type(procs[i]) in (BGR2RGB, RGB2BGR):
                import copy
                procs[norm_idx] = copy.copy(procs[norm_idx])      # the caller's processor stays untouched
                procs[norm_idx].swap_rb = not procs[norm_idx].swap_rb
                procs.pop(i)
                norm_idx -= 1
                break
    out: List[Processor] = []
    i = 0
    while i < len(procs):
        p = procs[i]
        nxt = procs[i + 1] if i + 1 < len(procs) else None
        if type(p) is Normalize and isinstance(nxt, Cast) and nxt.dtype == "float":
            out.append(p)
            i += 2
        elif type(p) is Normalize and isinstance(nxt, HWC2CHW):
            q = NormalizeAndPermute.__new__(NormalizeAndPermute)
            q.alpha, q.beta, q.swap_rb = p.alpha, p.beta, p.swap_rb
            out.append(q)
            i += 2
        else:
            out.append(p)
            i += 1
    return out


FuseTransforms = fuse_transforms


def chain_geometry(processors: Sequence[Processor], h: int, w: int) -> Optional[Dict[str, Any]]:
    """Folds a processor chain into the parameters of the fused kernel; ``None`` when the chain contains
    something the kernel cannot express (crop windows, gray conversion, affine warps)."""
    rh, rw = h, w
    interp = 1
    pad_value = [0.0, 0.0, 0.0]
    ch = cw = None
    alpha, beta, swap = [1.0] * 3, [0.0] * 3, False
    chw = False
    normalized = False
    for p in processors:
        t = type(p)
        if t in (Resize, ResizeByShort):
            if normalized:
                return None
            rh, rw = p.target(rh, rw)
            interp = p.interp
        elif t is LimitByStride:
            rh, rw = max(rh // p.stride * p.stride, p.stride), max(rw // p.stride * p.stride, p.stride)
            interp = p.interp
        elif t is PadToSize:
            ch, cw, pad_value = p.height, p.width, list(p.value)
        elif t is StridePad:
            bh, bw = ch or rh, cw or rw
            ch, cw = math.ceil(bh / p.stride) * p.stride, math.ceil(bw / p.stride) * p.stride
            pad_value = list(p.value)
        elif t in (Normalize, NormalizeAndPermute, Convert, ConvertAndPermute):
            alpha, beta = list(p.alpha), list(p.beta)
            swap = swap != bool(getattr(p, "swap_rb", False))
            normalized = True
            if t in (NormalizeAndPermute, ConvertAndPermute):
                chw = True
        elif t in (BGR2RGB, RGB2BGR):
            swap = not swap
        elif t is HWC2CHW:
            chw = True
        elif t is Cast:
            continue
        else:
            return None
    if interp not in (0, 1, 2):
        return None
    return {"rh": rh, "rw": rw, "ch": ch or rh, "cw": cw or rw, "interp": interp, "alpha": alpha, "beta": beta,
            "swap_rb": swap, "pad_value": pad_value, "chw": chw, "pad_before_norm": not normalized}


class ProcessorManager:
    """Owns the processor list of a model's pre-processing and picks the CPU or the fused CUDA path
    (fastdeploy/vision/common/processors/manager.cc:25-98)."""

    def __init__(self):
        self.processors: List[Processor] = []
        self._use_cuda = False
        self._gpu_id = -1

    def use_cuda(self, enable_cv_cuda: bool = False, gpu_id: int = -1) -> None:
        self._use_cuda = True
        self._gpu_id = gpu_id

    UseCuda = use_cuda

    def cuda_used(self) -> bool:
        return self._use_cuda

    def run_cpu(self, image: np.ndarray) -> FDMat:
        mat = FDMat(np.asarray(image))
        for p in self.processors:
            if not p(mat):
                raise RuntimeError(f"Failed to process image in {p.name()}.")
        return mat

    def run(self, images: Sequence[np.ndarray]) -> List[np.ndarray]:
        """Batch of images -> one stacked tensor (padding to the batch maximum, bottom/right)."""
        if len(images) == 0:
            raise ValueError("The size of input images should be greater than 0.")
        if self._use_cuda:
            out = run_chain_gpu(self.processors, images, self._gpu_id)
            if out is not None:
                return [out]
        mats = [self.run_cpu(im).mat for im in images]
        chw = mats[0].ndim == 3 and self.processors and any(type(p) in (HWC2CHW, NormalizeAndPermute, ConvertAndPermute)
                                                            for p in self.processors)
        hs = [m.shape[1] if chw else m.shape[0] for m in mats]
        ws = [m.shape[2] if chw else m.shape[1] for m in mats]
        mh, mw = max(hs), max(ws)
        padded = []
        for m, h, w in zip(mats, hs, ws):
            if (h, w) != (mh, mw):
                pw = ((0, 0), (0, mh - h), (0, mw - w)) if chw else ((0, mh - h), (0, mw - w), (0, 0))
                m = np.pad(m, pw)
            padded.append(m)
        return [np.stack(padded)]


def run_chain_gpu(processors: Sequence[Processor], images: Sequence[np.ndarray], gpu_id: int = -1,
                  out_dtype=None):
    """Whole chain in one kernel launch; returns a CUDA tensor ``[N,3,H,W]`` (or ``[N,H,W,3]``) or ``None``
    when the chain cannot be fused."""
    import torch
    from ...ops import preproc as P
    if not torch.cuda.is_available():
        return None
    geos = []
    for im in images:
        g = chain_geometry(processors, im.shape[0], im.shape[1])
        if g is None or im.ndim != 3 or im.shape[2] != 3 or im.dtype != np.uint8:
            return None
        geos.append(g)
    dev = torch.device("cuda", gpu_id if gpu_id >= 0 else torch.cuda.current_device())
    n = len(images)
    ch, cw = max(g["ch"] for g in geos), max(g["cw"] for g in geos)
    meta = np.zeros(n, dtype=P.IMAGE_META)
    blobs, off = [], 0
    for i, (im, g) in enumerate(zip(images, geos)):
        a = np.ascontiguousarray(im).reshape(-1)
        P.fill_meta(meta, i, src_offset=off, src_hw=im.shape[:2], src_stride=im.shape[1] * 3,
                    resized_hw=(g["rh"], g["rw"]))
        blobs.append(a)
        off += a.size
    g0 = geos[0]
    src = torch.from_numpy(np.concatenate(blobs)).to(dev)
    meta_d = torch.from_numpy(meta.view(np.uint8)).to(dev)
    chw = g0["chw"]
    dst = torch.empty((n, 3, ch, cw) if chw else (n, ch, cw, 3), dtype=out_dtype or torch.float32, device=dev)
    pad = g0["pad_value"]
    if g0["pad_before_norm"]:
        pad_out = [pad[c] * g0["alpha"][c] + g0["beta"][c] for c in range(3)]
    else:
        pad_out = pad
    with torch.cuda.device(dev):
        P.Preprocess(src, meta_d, dst, n=n, out_hw=(ch, cw), layout="nchw" if chw else "nhwc", c_out=3,
                     interp=g0["interp"], swap_rb=g0["swap_rb"], alpha=g0["alpha"], beta=g0["beta"],
                     pad_value=pad_out).launch()
    return dst
