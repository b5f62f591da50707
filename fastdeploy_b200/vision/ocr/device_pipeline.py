"""PP-OCR with every pixel staying on the GPU between the page and the text.

    pages (uint8, pinned host or device)
      -> fused resize + normalise into the detector's input            (ops.preproc.Preprocess)
      -> detector plan                                                  (CUDA graph)
      -> DB post-processing: components, min-area boxes, scores, unclip (ops.postproc.DBPostprocess)
      -> [host: box coordinates only - sort into reading order, choose batch / width buckets]
      -> perspective crop + resize + normalise into the classifier input, one launch for all crops of all pages
      -> classifier plan -> 180-degree flags on the device
      -> the same crops (turned where flagged) into width-bucketed recogniser inputs
      -> recogniser plans -> arg-max + CTC collapse on the device
      -> [host: character ids, lengths, scores]

The host sees two small read-backs per batch of pages (box corners; decoded ids), never a pixel or a probability
map. Shapes are bucketed - crops per classifier batch and per recogniser batch in powers of two, recogniser widths in
a fixed list - so that every launch replays a plan built at start-up; a batch is padded with empty crops.

The reference runs the same stages with OpenCV on the host between three engine calls
(fastdeploy/vision/ocr/ppocr/ppocr_v2.cc:108-175, utils/ocr_postprocess_op.cc, utils/get_rotate_crop_image.cc).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ...ops import postproc as PP
from ...ops import preproc as P
from ..result import OCRResult

REC_WIDTHS = (160, 240, 320, 480, 640, 960)
BATCHES = (8, 16, 32, 64)


def _bucket(v: int, buckets: Sequence[int]) -> int:
    for b in buckets:
        if v <= b:
            return b
    return buckets[-1]


class _Stage:
    """One network with its plans keyed by input shape; hands out the plan's input buffer as a dense NHWC tensor."""

    def __init__(self, model):
        self.model = model
        self.rt = model.runtime
        self.in_name = self.rt.graph.inputs[0].name
        self.out_name = self.rt.graph.outputs[0].name
        self.rt.option.native_option.max_plans = max(self.rt.option.native_option.max_plans, 64)

    def plan(self, n: int, h: int, w: int):
        return self.rt.plan_for_shapes({self.in_name: [n, 3, h, w]})

    def input_nhwc(self, plan) -> torch.Tensor:
        base = plan.inputs[self.in_name].t
        n, h, w, _ = base.shape
        return torch.as_strided(base, (n, h, w, base.stride(2)), base.stride())

    def output(self, plan) -> torch.Tensor:
        return plan.outputs[self.out_name].logical()


class DeviceOCR:
    """GPU-resident PP-OCR pipeline over a detector, an optional angle classifier and a recogniser that all run on the
    same GPU. ``predict_pages`` takes pages of one common size."""

    def __init__(self, det, cls, rec, *, rec_widths: Sequence[int] = REC_WIDTHS, batches: Sequence[int] = BATCHES):
        self.det, self.cls, self.rec = _Stage(det), (_Stage(cls) if cls is not None else None), _Stage(rec)
        self.det_model, self.cls_model, self.rec_model = det, cls, rec
        assert self.det.rt.on_gpu and self.rec.rt.on_gpu, "DeviceOCR needs the detector and the recogniser on a GPU"
        self.device = self.det.rt.device
        self.rec_widths, self.batches = tuple(rec_widths), tuple(batches)
        self.rec_h = rec.preprocessor.rec_image_shape[1]
        self.cls_h, self.cls_w = (cls.preprocessor.cls_image_shape[1:] if cls is not None else (48, 192))
        self._det_state: Dict[Tuple[int, int, int], dict] = {}
        self._crop_bufs: Dict[int, dict] = {}
        self.gpu_launches = 0
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.stage_counts: Dict[str, int] = {}
        self.rec_streams = 4
        self._side: List[torch.cuda.Stream] = []
        self._plan_stream: Dict[Tuple[int, int], int] = {}

    # ------------------------------------------------------------------ start-up
    def warm_up(self, page_hw: Tuple[int, int], pages: int) -> None:
        """Builds every plan a page batch of this size can ask for, so that no request pays for a plan build."""
        with torch.cuda.device(self.device):
            self._det_for(pages, *page_hw)
            for b in self.batches:
                if self.cls is not None:
                    self.cls.plan(b, self.cls_h, self.cls_w)
                for w in self.rec_widths:
                    self.rec.plan(b, self.rec_h, w)
            torch.cuda.synchronize(self.device)

    def _det_for(self, n: int, h: int, w: int) -> dict:
        key = (n, h, w)
        st = self._det_state.get(key)
        if st is None:
            pre = self.det_model.preprocessor
            rh, rw = pre.target_hw(h, w)
            plan = self.det.plan(n, rh, rw)
            alpha, beta = P.normalize_coeffs(pre.mean, pre.scale, pre.is_scale)
            raw = torch.empty(n, h, w, 3, dtype=torch.uint8, device=self.device)
            meta_host = np.zeros(n, dtype=P.IMAGE_META)
            for i in range(n):
                P.fill_meta(meta_host, i, src_offset=i * h * w * 3, src_hw=(h, w), src_stride=w * 3, resized_hw=(rh, rw))
            meta = torch.from_numpy(meta_host.view(np.uint8).copy()).to(self.device)
            dst = self.det.input_nhwc(plan)
            op = P.Preprocess(raw, meta, dst, n=n, out_hw=(rh, rw), layout="nhwc", c_out=dst.shape[3], interp="linear",
                              swap_rb=False, alpha=alpha, beta=beta)
            post = self.det_model.postprocessor
            db = PP.DBPostprocess(n, rh, rw, self.device, thresh=post.det_db_thresh, box_thresh=post.det_db_box_thresh,
                                  unclip_ratio=post.det_db_unclip_ratio, score_mode=post.det_db_score_mode,
                                  use_dilation=post.use_dilation, max_candidates=post.max_candidates)
            db.set_info([(w, h, rw, rh)] * n)
            st = dict(plan=plan, raw=raw, pre=op, db=db, meta=meta, rh=rh, rw=rw)
            self._det_state[key] = st
        return st

    def _crop_state(self, cap: int) -> dict:
        st = self._crop_bufs.get(cap)
        if st is None:
            dev = self.device
            full = cap + max(self.batches)      # a padded batch may start near the end: its tail reads stay in bounds
            st = dict(mats=torch.zeros(full, 9, dtype=torch.float32, device=dev),
                      vw=torch.zeros(full, dtype=torch.int32, device=dev),
                      page=torch.zeros(full, dtype=torch.int32, device=dev),
                      flip=torch.zeros(full, dtype=torch.int32, device=dev),
                      flip_sorted=torch.zeros(full, dtype=torch.int32, device=dev),
                      label=torch.zeros(full, dtype=torch.int32, device=dev),
                      score=torch.zeros(full, dtype=torch.float32, device=dev),
                      stage=torch.zeros(2, cap, 11, dtype=torch.float32, device=dev),
                      vw_pad=torch.zeros(self.rec_streams, max(self.batches), dtype=torch.int32, device=dev),
                      order=torch.zeros(cap, dtype=torch.int64, device=dev),
                      order_host=torch.zeros(cap, dtype=torch.int64).pin_memory(),
                      host=torch.zeros(2, cap, 11, dtype=torch.float32).pin_memory())
            self._crop_bufs[cap] = st
        return st

    # ------------------------------------------------------------------ stages
    def detect(self, pages) -> List[List[List[int]]]:
        """Detector + device DB post-processing; returns each page's boxes in reading order."""
        from . import sort_boxes
        if isinstance(pages, (list, tuple)):
            n, (h, w) = len(pages), pages[0].shape[:2]
        else:
            n, h, w = pages.shape[:3]
        st = self._det_for(n, int(h), int(w))
        if isinstance(pages, (list, tuple)):
            for i, pg in enumerate(pages):
                t = pg if isinstance(pg, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(pg))
                st["raw"][i].copy_(t, non_blocking=True)
                self.h2d_bytes_last += t.numel() if t.device.type == "cpu" else 0
        else:
            t = pages if isinstance(pages, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(pages))
            st["raw"].copy_(t, non_blocking=True)          # the whole batch in one copy
            self.h2d_bytes_last += t.numel() if t.device.type == "cpu" else 0
        st["pre"].launch()
        st["plan"].run()
        prob = self.det.output(st["plan"])[:, 0]          # [n, rh, rw] view of the probability map
        st["db"].run(prob)
        boxes, _ = st["db"].boxes()
        self.d2h_bytes_last += n * 4 + sum(len(b) for b in boxes) * 36
        self.gpu_launches += 1 + st["plan"].native_kernel_launches + st["db"].launches
        self._pages_dev = st["raw"]
        return [sort_boxes(b) for b in boxes]

    def recognize(self, pages_dev: torch.Tensor, boxes: Sequence[Sequence[Sequence[int]]]) -> List[OCRResult]:
        """Crops, classifies and reads all ``boxes`` (per page, reading order) of the pages already on the device."""
        flat = [(pi, b) for pi, bl in enumerate(boxes) for b in bl]
        results = [OCRResult() for _ in boxes]
        for pi, bl in enumerate(boxes):
            results[pi].boxes = [list(map(int, b)) for b in bl]
        total = len(flat)
        if total == 0:
            return results
        cap = max(64, 1 << (total - 1).bit_length())
        cs = self._crop_state(cap)
        all_boxes = [b for _, b in flat]
        page_idx = np.asarray([pi for pi, _ in flat], np.int32)
        rp = self.rec_model.preprocessor
        alpha_r, beta_r = P.normalize_coeffs(rp.mean, rp.scale, rp.is_scale)
        rec_mats, rec_vw, ratios = PP.crop_matrices(all_boxes, self.rec_h, self.rec_widths[-1])
        # ---- angle classifier: every crop at 48 x 192, batches in powers of two
        if self.cls is not None:
            cp = self.cls_model.preprocessor
            alpha_c, beta_c = P.normalize_coeffs(cp.mean, cp.scale, cp.is_scale)
            cls_mats, cls_vw, _ = PP.crop_matrices(all_boxes, self.cls_h, self.cls_w)
            self._upload(cs, cls_mats, cls_vw, page_idx, total)
            done = 0
            while done < total:
                b = _bucket(total - done, self.batches)
                k = min(b, total - done)
                plan = self.cls.plan(b, self.cls_h, self.cls_w)
                x = self.cls.input_nhwc(plan)
                if k < b:
                    cs["vw"][done + k:done + b].zero_()     # padding crops are empty
                PP.warp_normalize_batch(pages_dev, cs["mats"][done:], cs["vw"][done:], x, alpha_c, beta_c,
                                        page=cs["page"][done:])
                plan.run()
                probs = self.cls.output(plan)
                PP.cls_flip(probs[:k], self.cls_model.postprocessor.cls_thresh, cs["flip"][done:], cs["label"][done:],
                            cs["score"][done:])
                self.gpu_launches += 2 + plan.native_kernel_launches
                done += k
        else:
            cs["flip"].zero_()
        # ---- recogniser: crops sorted by aspect ratio, grouped by width bucket, batches in powers of two
        order = np.argsort(ratios, kind="stable")
        need_w = np.minimum(np.ceil(self.rec_h * ratios[order]).astype(np.int64), self.rec_widths[-1])
        groups: List[Tuple[int, np.ndarray]] = []
        start = 0
        while start < total:
            wb = _bucket(int(need_w[start]), self.rec_widths)
            end = start
            while end < total and _bucket(int(need_w[end]), self.rec_widths) == wb:
                end += 1
            groups.append((wb, order[start:end]))
            start = end
        # crops travel in sorted order, so each group's matrices are one contiguous slice
        sorted_vw = np.minimum(rec_vw[order], [_bucket(int(v), self.rec_widths) for v in need_w]).astype(np.int32)
        self._upload(cs, rec_mats[order], sorted_vw, page_idx[order], total, keep_flip_order=order)
        # The recogniser plans of different (batch, width) buckets own separate buffers, and each is a chain of
        # small launches that leaves most SMs idle: the buckets run side by side on a few streams. A plan always
        # runs on the same stream, so two chunks that share a plan stay ordered.
        pieces = []
        pos = 0
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        if not self._side:
            self._side = [torch.cuda.Stream(self.device) for _ in range(self.rec_streams)]
        used = {}
        for wb, idx in groups:
            done = 0
            while done < len(idx):
                b = _bucket(len(idx) - done, self.batches)
                k = min(b, len(idx) - done)
                plan = self.rec.plan(b, self.rec_h, wb)
                key = (b, wb)
                if key not in self._plan_stream:
                    self._plan_stream[key] = len(self._plan_stream) % len(self._side)
                si = self._plan_stream[key]
                side = self._side[si]
                if si not in used:
                    side.wait_event(ready)
                    used[si] = side
                x = self.rec.input_nhwc(plan)
                s = pos + done
                with torch.cuda.stream(side):
                    if k < b:
                        pad = cs["vw_pad"][si]
                        pad[:b].copy_(cs["vw"][s:s + b])
                        pad[k:b].zero_()
                        vw = pad
                    else:
                        vw = cs["vw"][s:]
                    PP.warp_normalize_batch(pages_dev, cs["mats"][s:], vw, x, alpha_r, beta_r, flip=cs["flip_sorted"][s:],
                                            page=cs["page"][s:])
                    plan.run()
                    probs = self.rec.output(plan)
                    ids, lens, scores = PP.ctc_greedy_decode_device(probs[:k].contiguous() if k < b else probs)
                pieces.append((idx[done:done + k], ids[:k], lens[:k], scores[:k]))
                self.gpu_launches += 3 + plan.native_kernel_launches
                self.stage_counts[f"rec_b{b}_w{wb}"] = self.stage_counts.get(f"rec_b{b}_w{wb}", 0) + 1
                done += k
            pos += len(idx)
        for side in used.values():
            ev = torch.cuda.Event()
            ev.record(side)
            main.wait_event(ev)
        # ---- one read-back of everything the host needs
        labels = self.rec_model.postprocessor.label_list
        texts, rscores = [""] * total, [0.0] * total
        for idx, ids, lens, scores in pieces:
            t, s = PP.ctc_texts(ids, lens, scores, labels)
            self.d2h_bytes_last += ids.numel() * 4 + lens.numel() * 8
            for j, i in enumerate(idx):
                texts[int(i)], rscores[int(i)] = t[j], s[j]
        if self.cls is not None:
            lab = cs["label"][:total].cpu().tolist()
            sc = cs["score"][:total].cpu().tolist()
            self.d2h_bytes_last += total * 8
        for k, (pi, _) in enumerate(flat):
            r = results[pi]
            r.text.append(texts[k])
            r.rec_scores.append(rscores[k])
            if self.cls is not None:
                r.cls_labels.append(int(lab[k]))
                r.cls_scores.append(float(sc[k]))
        return results

    def _upload(self, cs: dict, mats: np.ndarray, vw: np.ndarray, page: np.ndarray, total: int,
                keep_flip_order: Optional[np.ndarray] = None) -> None:
        """One pinned staging row per crop (9 matrix entries, valid width, page) -> one host->device copy. The
        classifier's and the recogniser's rows use separate staging halves: the first copy may still be in flight
        when the second set is written."""
        which = 0 if keep_flip_order is None else 1
        host = cs["host"][which]
        hv = host.numpy()
        hv[:total, :9] = mats
        hv[:total, 9] = vw
        hv[:total, 10] = page
        stage = cs["stage"][which]
        stage[:total].copy_(host[:total], non_blocking=True)
        self.h2d_bytes_last += total * 44
        cs["mats"][:total].copy_(stage[:total, :9])
        cs["vw"][:total].copy_(stage[:total, 9])
        cs["page"][:total].copy_(stage[:total, 10])
        self.gpu_launches += 3
        if keep_flip_order is not None:
            cs["order_host"][:total] = torch.from_numpy(np.ascontiguousarray(keep_flip_order, dtype=np.int64))
            cs["order"][:total].copy_(cs["order_host"][:total], non_blocking=True)
            from ...ops import generic as G
            G.gather_rows(cs["flip"], cs["order"][:total], cs["flip_sorted"][:total]).launch()
            self.h2d_bytes_last += total * 8
            self.gpu_launches += 1

    # ------------------------------------------------------------------ whole pipeline
    def predict_pages(self, pages, boxes: Optional[Sequence[Sequence[Sequence[int]]]] = None) -> List[OCRResult]:
        """``pages``: ``[N, H, W, 3]`` uint8 (numpy, pinned or device tensor) or a list of equal-size pages. ``boxes``
        replaces the detector's boxes for the later stages when given (the detector and its post-processing still run)."""
        self.h2d_bytes_last = self.d2h_bytes_last = 0
        with torch.cuda.device(self.device):
            found = self.detect(pages)
            use = [list(b) for b in boxes] if boxes is not None else found
            res = self.recognize(self._pages_dev, use)
        self.last_detected = found
        return res
