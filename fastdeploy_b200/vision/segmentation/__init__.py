"""``fastdeploy.vision.segmentation``: ``PaddleSegModel`` with ``deploy.yaml`` pre-processing and the three output
kinds of the post-processor (fastdeploy/vision/segmentation/ppseg/{preprocessor,postprocessor}.cc)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import yaml

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..common.processors import BGR2RGB, HWC2CHW, Normalize, ProcessorManager, Resize, fuse_transforms
from ..result import SegmentationResult


class PaddleSegPreprocessor(ProcessorManager):
    def __init__(self, config_file: str):
        super().__init__()
        self.config_file = config_file
        self.is_vertical_screen = False
        self.disable_normalize_ = False
        self.disable_permute_ = False
        self._build()

    def disable_normalize(self) -> None:
        """For a model that normalises inside its graph: the chain is rebuilt without Normalize
        (fastdeploy/vision/segmentation/ppseg/preprocessor.cc:150-170)."""
        self.disable_normalize_ = True
        self._build()

    def disable_permute(self) -> None:
        """Leaves the image HWC."""
        self.disable_permute_ = True
        self._build()

    def _build(self) -> None:
        with open(self.config_file) as f:
            cfg = yaml.safe_load(f)
        procs = [BGR2RGB()]
        self.is_contain_resize_op = False
        deploy = cfg.get("Deploy", {})
        for op in deploy.get("transforms", []) or []:
            t = op["type"]
            if t == "Normalize":
                if self.disable_normalize_:
                    continue
                procs.append(Normalize(list(op.get("mean", [0.5] * 3)), list(op.get("std", [0.5] * 3))))
            elif t == "Resize":
                self.is_contain_resize_op = True
                ts = op.get("target_size", [512, 512])
                procs.append(Resize(int(ts[0]), int(ts[1])))
        shape = deploy.get("input_shape")
        if shape and not self.is_contain_resize_op and all(int(d) > 0 for d in shape[2:]):
            procs.insert(1, Resize(int(shape[3]), int(shape[2])))
            self.is_contain_resize_op = True
        if not self.disable_permute_:
            procs.append(HWC2CHW())
        self.processors = fuse_transforms(procs)
        self.with_softmax = deploy.get("output_op", "") == "softmax"
        self.with_argmax = deploy.get("output_op", "argmax") == "argmax"


class PaddleSegPostprocessor:
    def __init__(self, with_argmax=True, with_softmax: bool = False):
        """``PaddleSegPostprocessor(config_file)`` reads ``Deploy.output_op`` of the model's ``deploy.yaml`` as the reference
        does (fastdeploy/vision/segmentation/ppseg/postprocessor.cc:22-50); the two flags can also be given directly."""
        if isinstance(with_argmax, str):
            with open(with_argmax) as f:
                deploy = (yaml.safe_load(f) or {}).get("Deploy", {})
            with_softmax = deploy.get("output_op", "") == "softmax"
            with_argmax = deploy.get("output_op", "argmax") == "argmax"
        self.is_with_argmax, self.is_with_softmax = bool(with_argmax), bool(with_softmax)
        self.apply_softmax = False
        self.store_score_map = False

    def run(self, infer: np.ndarray, im_infos: Sequence[Sequence[int]]) -> List[SegmentationResult]:
        """``infer``: [N,H,W] labels (argmax in graph) or [N,C,H,W] logits / probabilities. ``im_infos[i]`` =
        (source_h, source_w); results are resized back (nearest for labels, linear for scores)."""
        import cv2
        out = []
        x = np.asarray(infer)
        for i in range(x.shape[0]):
            h0, w0 = im_infos[i]
            res = SegmentationResult()
            if x.ndim == 3 or (x.ndim == 4 and x.shape[1] == 1 and np.issubdtype(x.dtype, np.integer)):
                lab = x[i] if x.ndim == 3 else x[i, 0]
                lab = lab.astype(np.uint8) if lab.max(initial=0) < 256 else lab.astype(np.int32)
                score = None
            else:
                logit = x[i].astype(np.float32)
                if self.apply_softmax and not self.is_with_softmax:
                    e = np.exp(logit - logit.max(0, keepdims=True))
                    logit = e / e.sum(0, keepdims=True)
                lab = logit.argmax(0).astype(np.uint8)
                score = logit.max(0)
            if lab.shape != (h0, w0):
                lab = cv2.resize(lab, (w0, h0), interpolation=cv2.INTER_NEAREST)
                if score is not None:
                    score = cv2.resize(score, (w0, h0), interpolation=cv2.INTER_LINEAR)
            res.label_map = lab.reshape(-1).astype(np.int32).tolist()
            res.shape = [h0, w0]
            if self.store_score_map and score is not None:
                res.contain_score_map = True
                res.score_map = score.reshape(-1).astype(np.float32).tolist()
            out.append(res)
        return out


class PaddleSegModel(FastDeployModel):
    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = PaddleSegPreprocessor(config_file)
        self.postprocessor = PaddleSegPostprocessor(self.preprocessor.with_argmax, self.preprocessor.with_softmax)
        self.init_runtime()

    def predict(self, im: np.ndarray) -> SegmentationResult:
        return self.batch_predict([im])[0]

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[SegmentationResult]:
        if self.runtime.on_gpu:
            self.preprocessor.use_cuda(gpu_id=self.runtime_option.device_id)
        x = self.preprocessor.run([np.asarray(im) for im in images])[0]
        outs = self.infer({self.runtime.graph.inputs[0].name: x})
        first = self.runtime._to_numpy(outs[self.runtime.graph.outputs[0].name])
        return self.postprocessor.run(first, [im.shape[:2] for im in images])

    def get_preprocessor(self): return self.preprocessor
    def get_postprocessor(self): return self.postprocessor
