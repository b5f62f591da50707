"""PaddleDetection model family: ``PaddleDetPreprocessor``, ``PaddleDetPostprocessor``,
``PPDetBase`` and its subclasses (PPYOLOE, PicoDet, YOLOv3, ...), following
fastdeploy/vision/detection/ppdet/{preprocessor,postprocessor,base}.cc and model.h:24-492.

On a GPU runtime the whole chain stays on the device: raw uint8 frames are copied once
(async, from pinned memory when the caller provides it), one fused kernel does
BGR->RGB + resize + normalise + layout + cast straight into the plan's input buffer, the
plan runs the network, DFL decode and multiclass NMS, and only ``keep_top_k x 6`` floats
per image come back. The CPU path restates the reference's OpenCV pipeline with cv2 /
numpy and doubles as the oracle in the tests.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import yaml

from ...core.types import ModelFormat
from ...ops.nms import multiclass_nms_reference
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ...utils import log
from ..result import DetectionResult, Mask


class NMSOption:
    """Defaults of fastdeploy/vision/detection/ppdet/multiclass_nms.h:32-41."""

    def __init__(self):
        self.background_label = -1
        self.keep_top_k = 100
        self.nms_eta = 1.0
        self.nms_threshold = 0.5
        self.nms_top_k = 1000
        self.normalized = True
        self.score_threshold = 0.3


class NMSRotatedOption:
    """Defaults of fastdeploy/vision/detection/ppdet/multiclass_nms_rotated.h:32-41 (PP-YOLOE-R)."""

    def __init__(self):
        self.background_label = -1
        self.keep_top_k = -1
        self.nms_eta = 1.0
        self.nms_threshold = 0.1
        self.nms_top_k = 2000
        self.normalized = False
        self.score_threshold = 0.1


class PaddleDetPreprocessor:
    def __init__(self, config_file: str):
        self.config_file = config_file
        self.disable_normalize_ = False
        self.disable_permute_ = False
        self.use_cuda_ = False
        self.gpu_id = -1
        self._build()

    # ------------------------------------------------------------------ config
    def _build(self) -> None:
        with open(self.config_file) as f:
            cfg = yaml.safe_load(f)
        if "arch" not in cfg:
            raise ValueError("Please set model arch, support value : SOLOv2, YOLO, SSD, RetinaNet, RCNN, Face.")
        self.arch = cfg["arch"]
        self.ops: List[Dict[str, Any]] = []
        self.has_permute = False
        for op in cfg.get("Preprocess", []):
            t = op["type"]
            if t == "NormalizeImage":
                if self.disable_normalize_:
                    continue
                mean, std = list(op["mean"]), list(op["std"])
                if op.get("norm_type", "mean_std") != "mean_std":
                    mean, std = [0.0] * 3, [1.0] * 3
                self.ops.append({"type": "Normalize", "mean": mean, "std": std, "is_scale": op.get("is_scale", True)})
            elif t == "Resize":
                ts = op["target_size"]
                assert len(ts) == 2, f"Require size of target_size be 2, but now it's {len(ts)}."
                self.ops.append({"type": "Resize", "keep_ratio": bool(op["keep_ratio"]), "target_size": list(ts),
                                 "interp": int(op["interp"])})
            elif t == "Permute":
                self.has_permute = True
            elif t == "Pad":
                self.ops.append({"type": "PadToSize", "size": list(op["size"]), "value": list(op["fill_value"])})
            elif t == "PadStride":
                self.ops.append({"type": "StridePad", "stride": int(op["stride"])})
            else:
                raise ValueError(f"Unexcepted preprocess operator: {t}.")
        self.label_list = cfg.get("label_list", [])

    def disable_normalize(self):
        self.disable_normalize_ = True
        self._build()

    def disable_permute(self):
        self.disable_permute_ = True

    def use_cuda(self, enable_cv_cuda: bool = False, gpu_id: int = -1):
        self.use_cuda_ = True
        self.gpu_id = gpu_id

    # ------------------------------------------------------------------ geometry shared by both paths
    def plan_image(self, h: int, w: int) -> Dict[str, Any]:
        """Resolves the op list for one source size: resized size, canvas size, scale factor."""
        rh, rw = h, w
        interp = 1
        resized = False
        pad_to = None
        stride = 0
        for op in self.ops:
            if op["type"] == "Resize":
                interp = op["interp"]
                if not op["keep_ratio"]:
                    rh, rw = op["target_size"][0], op["target_size"][1]
                else:
                    tmin, tmax = min(op["target_size"]), max(op["target_size"])
                    scale = tmin / min(rh, rw)
                    if tmax > 0 and round(scale * max(rh, rw)) > tmax:
                        scale = tmax / max(rh, rw)
                    rh, rw = int(round(rh * scale)), int(round(rw * scale))
                resized = True
            elif op["type"] == "PadToSize":
                pad_to = (op["size"][0], op["size"][1], op["value"])
            elif op["type"] == "StridePad":
                stride = op["stride"]
        ch, cw = rh, rw
        if pad_to is not None:
            ch, cw = max(ch, pad_to[0]), max(cw, pad_to[1])
        if stride > 0:
            ch, cw = math.ceil(ch / stride) * stride, math.ceil(cw / stride) * stride
        sf = (rh / h, rw / w) if resized else (1.0, 1.0)
        return {"rh": rh, "rw": rw, "ch": ch, "cw": cw, "interp": interp, "scale_factor": sf,
                "pad_value": pad_to[2] if pad_to is not None else [0.0, 0.0, 0.0]}

    def norm_coeffs(self) -> Tuple[List[float], List[float]]:
        from ...ops.preproc import normalize_coeffs
        for op in self.ops:
            if op["type"] == "Normalize":
                return normalize_coeffs(op["mean"], op["std"], op["is_scale"])
        return [1.0] * 3, [0.0] * 3

    # ------------------------------------------------------------------ CPU path
    def run(self, images: Sequence[np.ndarray]) -> List[np.ndarray]:
        """Returns ``[image NCHW fp32, scale_factor [N,2], im_shape [N,2]]``."""
        import cv2
        if len(images) == 0:
            raise ValueError("The size of input images should be greater than 0.")
        alpha, beta = self.norm_coeffs()
        alpha, beta = np.asarray(alpha, np.float32), np.asarray(beta, np.float32)
        plans = [self.plan_image(im.shape[0], im.shape[1]) for im in images]
        max_h = max(p["ch"] for p in plans)
        max_w = max(p["cw"] for p in plans)
        n = len(images)
        out = np.zeros((n, max_h, max_w, 3), np.float32)
        sf = np.zeros((n, 2), np.float32)
        im_shape = np.zeros((n, 2), np.float32)
        for i, (im, p) in enumerate(zip(images, plans)):
            x = im[..., ::-1]                                    # BGR2RGB
            if (p["rh"], p["rw"]) != im.shape[:2]:
                x = cv2.resize(np.ascontiguousarray(x), (p["rw"], p["rh"]), interpolation=p["interp"])
            x = x.astype(np.float32) * alpha + beta
            out[i, :p["rh"], :p["rw"]] = x
            if p["ch"] > p["rh"] or p["cw"] > p["rw"]:
                pv = np.asarray(p["pad_value"], np.float32)
                out[i, p["rh"]:p["ch"], :p["cw"]] = pv
                out[i, :p["rh"], p["rw"]:p["cw"]] = pv
            sf[i] = p["scale_factor"]
            im_shape[i] = (max_h, max_w)
        if self.has_permute and not self.disable_permute_:
            out = np.ascontiguousarray(out.transpose(0, 3, 1, 2))
        return [out, sf, im_shape]


class PaddleDetPostprocessor:
    def __init__(self, arch: str = "YOLO"):
        self.arch = arch
        self.with_nms_ = True
        self.nms_option = NMSOption()
        self.decode_and_nms = None

    def apply_nms(self):
        """The exported model has no NMS: run it here (reference: ApplyNMS / ProcessWithoutNMS)."""
        self.with_nms_ = False

    ApplyNMS = apply_nms

    def set_nms_option(self, option: NMSOption):
        self.nms_option = option

    def set_nms_rotated_option(self, option):
        self.nms_rotated_option = option

    def set_scale_factor(self, scale_factor) -> None:
        """(scale_h, scale_w) the pre-processor resized the image by; rotated boxes are divided by it."""
        self.scale_factor = [float(scale_factor[0]), float(scale_factor[1])]

    def run(self, tensors: Sequence[np.ndarray]) -> List[DetectionResult]:
        """Dispatch of the reference (fastdeploy/vision/detection/ppdet/postprocessor.cc:318-357): SOLOv2 (boxes from
        masks), PP-YOLOE-R (8-value boxes -> rotated multiclass NMS), boxes with or without NMS in the graph, and the
        mask output of Mask R-CNN cropped to each box."""
        if self.arch == "SOLOv2":
            return self._solov2(tensors)
        first = tensors[0]
        if getattr(first, "ndim", 0) == 3 and first.shape[2] == 8:
            return self._rotated(first, tensors[1])
        if self.with_nms_:
            results = self._with_nms(np.asarray(tensors[0]), np.asarray(tensors[1]))
        else:
            results = self._without_nms(np.asarray(tensors[0]), np.asarray(tensors[1]))
        if len(tensors) > 2:
            masks = np.asarray(tensors[2])
            if masks.shape[0] != np.asarray(tensors[0]).reshape(-1, 6).shape[0]:
                raise ValueError(f"mask output has {masks.shape[0]} entries for "
                                 f"{np.asarray(tensors[0]).reshape(-1, 6).shape[0]} boxes")
            self._process_mask(masks, results)
        return results

    @staticmethod
    def _process_mask(masks: np.ndarray, results: List[DetectionResult]) -> None:
        """Every box keeps the part of its full-image mask that lies inside the (rounded) box (postprocessor.cc:24-59)."""
        masks = np.asarray(masks).astype(np.uint8)
        index = 0
        for res in results:
            res.contain_masks = True
            res.masks = []
            for box in res.boxes:
                x1, y1, x2, y2 = (int(round(float(v))) for v in box)
                h, w = max(y2 - y1, 0), max(x2 - x1, 0)
                crop = masks[index, max(y1, 0):max(y1, 0) + h, max(x1, 0):max(x1, 0) + w]
                full = np.zeros((h, w), np.uint8)
                full[:crop.shape[0], :crop.shape[1]] = crop
                res.masks.append(Mask(data=full.reshape(-1).tolist(), shape=[h, w]))
                index += 1

    def _solov2(self, tensors: Sequence[np.ndarray]) -> List[DetectionResult]:
        """SOLOv2 exports (count, labels, scores, full-image masks) for one image; a box is the extent of its mask
        (postprocessor.cc:180-262)."""
        if len(tensors) != 4:
            raise ValueError("SOLOv2 post-processing needs 4 output tensors")
        count = int(np.asarray(tensors[0]).reshape(-1)[0])
        labels, scores = np.asarray(tensors[1]).reshape(-1), np.asarray(tensors[2]).reshape(-1)
        masks = np.asarray(tensors[3]).astype(np.uint8)
        res = DetectionResult()
        res.contain_masks = True
        kept = []
        for i in range(count):
            if scores[i] < self.nms_option.score_threshold:
                continue
            rows = np.nonzero(masks[i].sum(1) > 0.5)[0]
            cols = np.nonzero(masks[i].sum(0) > 0.5)[0]
            y1, y2 = (float(rows[0]), float(rows[-1] + 1)) if len(rows) else (float(masks.shape[1]), 0.0)
            x1, x2 = (float(cols[0]), float(cols[-1] + 1)) if len(cols) else (float(masks.shape[2]), 0.0)
            res.label_ids.append(int(labels[i]))
            res.scores.append(float(scores[i]))
            res.boxes.append([x1, y1, x2, y2])
            kept.append(i)
        self._process_mask(masks[kept] if kept else masks[:0], [res])
        return [res]

    def _rotated(self, boxes, scores) -> List[DetectionResult]:
        """PP-YOLOE-R: ``boxes [N, M, 8]`` quadrilaterals and ``scores [N, C, M]`` through the rotated multiclass NMS
        (on the GPU when the tensors live there), then divided by the resize factors (postprocessor.cc:264-316; the
        x coordinates are divided by the width factor and the y coordinates by the height factor)."""
        from ...ops import perception as PR
        opt = getattr(self, "nms_rotated_option", None) or self.nms_option
        on_gpu = hasattr(boxes, "is_cuda") and boxes.is_cuda
        n = boxes.shape[0]
        results = []
        for i in range(n):
            if on_gpu:
                key = (int(scores.shape[1]), int(boxes.shape[1]), str(boxes.device))
                if getattr(self, "_rot_key", None) != key:
                    self._rot_nms = PR.MulticlassNMSRotated(key[0], key[1], boxes.device, score_threshold=opt.score_threshold,
                                                            nms_threshold=opt.nms_threshold, nms_top_k=opt.nms_top_k,
                                                            keep_top_k=opt.keep_top_k, background_label=opt.background_label)
                    self._rot_key = key
                try:
                    rows, _ = self._rot_nms.run(boxes[i], scores[i])
                except OverflowError:
                    rows, _ = PR.multiclass_nms_rotated_numpy(boxes[i].float().cpu().numpy(), scores[i].float().cpu().numpy(),
                                                              opt.score_threshold, opt.nms_threshold, opt.nms_top_k,
                                                              opt.keep_top_k, opt.background_label)
            else:
                rows, _ = PR.multiclass_nms_rotated_numpy(np.asarray(boxes[i], np.float32), np.asarray(scores[i], np.float32),
                                                          opt.score_threshold, opt.nms_threshold, opt.nms_top_k,
                                                          opt.keep_top_k, opt.background_label)
            res = DetectionResult()
            sf = getattr(self, "scale_factor", None)
            for r in rows:
                quad = [float(v) for v in r[2:10]]
                if sf and sf[0] != 0:
                    quad = [v / (sf[1] if j % 2 == 0 else sf[0]) for j, v in enumerate(quad)]
                res.label_ids.append(int(round(float(r[0]))))
                res.scores.append(float(r[1]))
                res.rotated_boxes.append(quad)
            results.append(res)
        return results

    @staticmethod
    def _rows_to_results(rows: np.ndarray, counts: np.ndarray) -> List[DetectionResult]:
        # one conversion per column for the whole batch, then list slices per image: a batch of 32 images costs three
        # array-to-list calls instead of ninety-six
        rows = np.asarray(rows)
        labels = rows[:, 0].astype(np.int32).tolist() if len(rows) else []
        scores = rows[:, 1].astype(np.float32).tolist() if len(rows) else []
        boxes = rows[:, 2:6].astype(np.float32).tolist() if len(rows) else []
        results = []
        pos = 0
        for c in counts:
            c = int(c)
            res = DetectionResult()
            if c:
                res.label_ids = labels[pos:pos + c]
                res.scores = scores[pos:pos + c]
                res.boxes = boxes[pos:pos + c]
            pos += c
            results.append(res)
        return results

    def _with_nms(self, out: np.ndarray, num: np.ndarray) -> List[DetectionResult]:
        return self._rows_to_results(out.reshape(-1, out.shape[-1]), num.reshape(-1))

    def _without_nms(self, boxes: np.ndarray, scores: np.ndarray) -> List[DetectionResult]:
        o = self.nms_option
        out, _, num = multiclass_nms_reference(boxes, scores, o.score_threshold, o.nms_threshold, o.nms_top_k,
                                               o.keep_top_k, o.normalized, o.background_label, o.nms_eta)
        return self._rows_to_results(out, num)


class _GpuSlot:
    """Staging buffers of one in-flight batch."""

    def __init__(self, device, raw_bytes: int, n: int, out_rows: int):
        from ...core.allocator import pinned_tensor
        from ...ops.preproc import IMAGE_META
        self.raw = torch.empty(raw_bytes, dtype=torch.uint8, device=device)
        # page-locked staging from the caching pool: a new slot (a new batch shape) costs no cudaHostAlloc after the
        # pool has warmed up
        self.meta_host = pinned_tensor([n * IMAGE_META.itemsize], torch.uint8)
        self.meta_dev = torch.empty(n * IMAGE_META.itemsize, dtype=torch.uint8, device=device)
        self.sf_host = pinned_tensor([n, 2], torch.float32)
        self.out_host = pinned_tensor([n, out_rows, 6], torch.float32)
        self.num_host = pinned_tensor([n], torch.int32)
        self.status_host = pinned_tensor([1], torch.int32).zero_()
        self.copied = torch.cuda.Event()
        self.done = torch.cuda.Event()
        self.pre = None
        self.layout_sig = None      # (frame size, count, packed) whose placement records the device copy holds
        self.h2d_bytes = 0
        self.d2h_bytes = 0


class PendingDetection:
    """Handle of a batch submitted with :meth:`PPDetBase.predict_async`."""

    def __init__(self, slot: _GpuSlot, n: int, status):
        self.slot, self.n, self.status = slot, n, status

    def result(self) -> List[DetectionResult]:
        self.slot.done.synchronize()
        self.status.check_snapshot(self.slot.status_host, "detection")
        num = self.slot.num_host[:self.n].numpy()
        out = self.slot.out_host[:self.n].numpy()
        rows = np.concatenate([out[i, :num[i]] for i in range(self.n)], 0) if self.n else np.zeros((0, 6), np.float32)
        return PaddleDetPostprocessor._rows_to_results(rows, num)


class PPDetBase(FastDeployModel):
    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = PaddleDetPreprocessor(config_file)
        self.postprocessor = PaddleDetPostprocessor(self.preprocessor.arch)
        self.init_runtime()
        out_names = [vi.name for vi in self.runtime.graph.outputs]
        self._nms_in_graph = any(n.op in ("MultiClassNMS", "PPYOLOEPost") for n in self.runtime.graph.nodes)
        if not self._nms_in_graph:
            self.postprocessor.apply_nms()
        self._slots: Dict[Tuple, List[_GpuSlot]] = {}
        self._slot_rr = 0
        self._geo_cache: Dict[Tuple[int, int], Dict[str, Any]] = {}
        self.slots_in_flight = 3        # batches whose copies / compute / read-back may overlap
        self._copy_stream = None
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0

    def get_preprocessor(self):
        return self.preprocessor

    def get_postprocessor(self):
        return self.postprocessor

    # ------------------------------------------------------------------ public API
    def predict(self, im: np.ndarray) -> DetectionResult:
        return self.batch_predict([im])[0]

    def batch_predict(self, images: Sequence[Any]) -> List[DetectionResult]:
        if self.runtime.on_gpu and self._nms_in_graph:
            return self.predict_async(images).result()
        tensors = self.preprocessor.run([np.asarray(im) for im in images])
        feeds = self._name_inputs(tensors)
        outs = self.infer(feeds)
        names = [vi.name for vi in self.runtime.graph.outputs]
        self.postprocessor.set_scale_factor(np.asarray(tensors[1], np.float32).reshape(-1, 2)[0])
        first = outs[names[0]]
        if hasattr(first, "is_cuda") and first.is_cuda and first.dim() == 3 and first.shape[2] == 8:
            # rotated boxes stay on the device for the rotated NMS
            return self.postprocessor.run([outs[n] for n in names])
        arrs = [self.runtime._to_numpy(outs[n]) for n in names]
        return self.postprocessor.run(arrs)

    def _name_inputs(self, tensors: List[np.ndarray]) -> Dict[str, np.ndarray]:
        pool = {"image": tensors[0], "scale_factor": tensors[1], "im_shape": tensors[2]}
        return {vi.name: pool[vi.name] for vi in self.runtime.graph.inputs}

    # ------------------------------------------------------------------ device pipeline
    def predict_async(self, images: Sequence[Any]) -> PendingDetection:
        """Enqueues copy + pre-processing + network + NMS for one batch and returns at once.
        Up to two batches are in flight: the next batch's host->device copy overlaps the
        current batch's compute."""
        from ...ops import preproc as P
        rt = self.runtime
        dev = rt.device
        if not isinstance(images, (list, tuple)) and getattr(images, "ndim", 0) == 4:
            images = [images[i] for i in range(images.shape[0])]      # one [N,H,W,3] batch buffer
        n = len(images)
        # frames of one size (the common case: a camera, a video) share their geometry; it is planned once
        hw0 = (int(images[0].shape[0]), int(images[0].shape[1])) if n else (0, 0)
        uniform = all(int(im.shape[0]) == hw0[0] and int(im.shape[1]) == hw0[1] for im in images)
        if uniform and n:
            g0 = self._geo_cache.get(hw0)
            if g0 is None:
                g0 = self._geo_cache[hw0] = self.preprocessor.plan_image(*hw0)
            geo = [g0] * n
        else:
            geo = [self.preprocessor.plan_image(int(im.shape[0]), int(im.shape[1])) for im in images]
        ch, cw = max(g["ch"] for g in geo), max(g["cw"] for g in geo)
        shapes = {}
        for vi in rt.graph.inputs:
            shapes[vi.name] = [n, 3, ch, cw] if vi.name == "image" else [n, 2]
        with torch.cuda.device(dev):
            plan = rt.plan_for_shapes(shapes)
            sizes = [int(im.shape[0]) * int(im.shape[1]) * 3 for im in images]
            raw_bytes = sum((s + 255) // 256 * 256 for s in sizes)
            nms = plan.extra["nms"][0]
            key = (tuple(sorted((k, tuple(v)) for k, v in shapes.items())), raw_bytes)
            if key not in self._slots:
                self._slots[key] = [_GpuSlot(dev, raw_bytes, n, nms.out.shape[1]) for _ in range(self.slots_in_flight)]
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(dev)
            self._slot_rr = (self._slot_rr + 1) % len(self._slots[key])
            slot = self._slots[key][self._slot_rr]
            slot.done.synchronize()                 # the slot's previous batch has been read back
            compute = torch.cuda.current_stream(dev)
            # ---- host->device copies on the copy stream
            meta = np.frombuffer(slot.meta_host.numpy(), dtype=P.IMAGE_META)
            off = 0
            h2d = 0
            with torch.cuda.stream(self._copy_stream):
                tens = [im if isinstance(im, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(im))
                        for im in images]
                # Frames that sit back to back in one host (or device) buffer - a batch staged in one pinned
                # allocation - travel as ONE copy: a copy per frame costs a launch each and keeps the link
                # from streaming.
                t0 = tens[0] if n else None
                step = t0.numel() if n else 0
                base_ptr = t0.data_ptr() if n else 0
                packed = n > 0 and uniform and all(
                    t.dtype == torch.uint8 and t.device == t0.device and t.data_ptr() == base_ptr + i * step and
                    t.is_contiguous() for i, t in enumerate(tens))
                if packed:
                    total = step * n
                    try:
                        whole = torch.as_strided(tens[0].reshape(-1), (total,), (1,)) if n > 1 else tens[0].reshape(-1)
                    except RuntimeError:      # the frames are separate storages that merely happen to be adjacent
                        packed = False
                if packed:
                    slot.raw[:total].copy_(whole, non_blocking=True)
                    if whole.device.type == "cpu":
                        h2d += total
                # per-frame placement records: identical for every batch of packed same-size frames, so a slot that
                # has seen this layout before keeps what it already holds on the device
                sig = (hw0, n, packed) if (packed and uniform) else None
                if sig is None or slot.layout_sig != sig:
                    for i, (t, g) in enumerate(zip(tens, geo)):
                        flat = t.reshape(-1)
                        if not packed:
                            slot.raw[off:off + flat.numel()].copy_(flat, non_blocking=True)
                            if flat.device.type == "cpu":
                                h2d += flat.numel()
                        P.fill_meta(meta, i, src_offset=off, src_hw=(int(t.shape[0]), int(t.shape[1])),
                                    src_stride=int(t.shape[1]) * 3, resized_hw=(g["rh"], g["rw"]))
                        slot.sf_host[i, 0], slot.sf_host[i, 1] = g["scale_factor"]
                        off += flat.numel() if packed else (flat.numel() + 255) // 256 * 256
                    slot.meta_dev.copy_(slot.meta_host, non_blocking=True)
                    h2d += slot.meta_host.numel()
                    slot.layout_sig = sig
                slot.copied.record(self._copy_stream)
            # ---- compute stream: pre-process, network, NMS, read-back
            compute.wait_event(slot.copied)
            if "scale_factor" in plan.inputs:
                # the plan's input buffer is shared by both slots: write it in compute-stream order
                plan.inputs["scale_factor"].t.copy_(slot.sf_host[:n], non_blocking=True)
                h2d += n * 8
            if slot.pre is None:
                alpha, beta = self.preprocessor.norm_coeffs()
                img_val = plan.inputs["image"]
                base = img_val.t
                c_phys = base.stride(2)
                dst = torch.as_strided(base, (n, ch, cw, c_phys), base.stride())
                slot.pre = P.Preprocess(slot.raw, slot.meta_dev, dst, n=n, out_hw=(ch, cw), layout="nhwc",
                                        c_out=c_phys, interp=geo[0]["interp"], swap_rb=True, alpha=alpha, beta=beta,
                                        pad_value=[0.0, 0.0, 0.0])
            slot.pre.launch()
            plan.run()
            slot.out_host[:n].copy_(nms.out, non_blocking=True)
            slot.num_host[:n].copy_(nms.out_num, non_blocking=True)
            plan.status.snapshot_async(slot.status_host)
            slot.done.record(compute)
            rt.gpu_launches += plan.native_kernel_launches + 1
            self.h2d_bytes_last = h2d
            self.d2h_bytes_last = n * nms.out.shape[1] * 6 * 4 + n * 4 + 4
        return PendingDetection(slot, n, plan.status)


def _subclass(name: str, doc: str):
    return type(name, (PPDetBase,), {"__doc__": doc})


PPYOLOE = _subclass("PPYOLOE", "PP-YOLOE / PP-YOLOE+ (fastdeploy/vision/detection/ppdet/model.h:52-74).")
PicoDet = _subclass("PicoDet", "PicoDet (model.h:24-50).")
PPYOLO = _subclass("PPYOLO", "PP-YOLO / PP-YOLOv2 (model.h:76-98).")
YOLOv3 = _subclass("YOLOv3", "YOLOv3 (model.h:100-122).")
PaddleYOLOX = _subclass("PaddleYOLOX", "YOLOX exported by PaddleDetection (model.h:124-146).")
FasterRCNN = _subclass("FasterRCNN", "Faster R-CNN (model.h:148-167).")
MaskRCNN = _subclass("MaskRCNN", "Mask R-CNN (model.h:169-188).")
SSD = _subclass("SSD", "SSD (model.h:190-210).")
PaddleYOLOv5 = _subclass("PaddleYOLOv5", "YOLOv5 exported by PaddleDetection (model.h:212-230).")
PaddleYOLOv6 = _subclass("PaddleYOLOv6", "YOLOv6 exported by PaddleDetection (model.h:232-250).")
PaddleYOLOv7 = _subclass("PaddleYOLOv7", "YOLOv7 exported by PaddleDetection (model.h:252-270).")
PaddleYOLOv8 = _subclass("PaddleYOLOv8", "YOLOv8 exported by PaddleDetection (model.h:272-292).")
RTMDet = _subclass("RTMDet", "RTMDet (model.h:294-312).")
CascadeRCNN = _subclass("CascadeRCNN", "Cascade R-CNN (model.h:314-332).")
PSSDet = _subclass("PSSDet", "PSS-Det (model.h:334-352).")
RetinaNet = _subclass("RetinaNet", "RetinaNet (model.h:354-372).")
PPYOLOESOD = _subclass("PPYOLOESOD", "PP-YOLOE-SOD (model.h:374-392).")
FCOS = _subclass("FCOS", "FCOS (model.h:394-412).")
TTFNet = _subclass("TTFNet", "TTFNet (model.h:414-432).")
TOOD = _subclass("TOOD", "TOOD (model.h:434-452).")
GFL = _subclass("GFL", "GFL (model.h:454-472).")


class SOLOv2(PPDetBase):
    """SOLOv2 instance segmentation (fastdeploy/vision/detection/ppdet/model.h:24-50 family): the graph's four outputs
    (count, labels, scores, full-image masks) become boxes from the mask extents plus per-box mask crops."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.postprocessor.arch = "SOLOv2"
PaddleDetectionModel = _subclass("PaddleDetectionModel", "Any PaddleDetection export (model.h:474-492).")
PPYOLOER = _subclass("PPYOLOER", "PP-YOLOE-R rotated detector.")
