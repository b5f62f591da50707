"""Processor managers with the reference's module path (python/fastdeploy/vision/common/manager.py:20-75)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Sequence

import numpy as np

from .processors import FDMat, FDMatBatch, ProcessorManager    # noqa: F401  (ProcessorManager is re-exported)


class PyProcessorManager(ABC):
    """Base class of a pre-processing chain written in Python: a subclass creates its processors in ``__init__`` and
    applies them to the batch in :meth:`apply`; calling the object with a list of images (``FDMat`` or arrays) wraps
    them into an :class:`FDMatBatch`, runs ``apply`` and returns what it returns.

    Processors called one by one run on the host. ``use_cuda`` is kept for source compatibility and recorded; the fused
    device pre-processing is what the model classes' own ``ProcessorManager.run`` uses, where the whole chain is known."""

    def __init__(self):
        self._manager = ProcessorManager()

    def use_cuda(self, enable_cv_cuda: bool = False, gpu_id: int = -1) -> None:
        self._manager.use_cuda(enable_cv_cuda, gpu_id)

    def cuda_used(self) -> bool:
        return self._manager.cuda_used()

    def __call__(self, images: Sequence) -> List:
        batch = FDMatBatch().from_mats(images)
        return self.apply(batch)

    @abstractmethod
    def apply(self, image_batch: FDMatBatch) -> List:
        raise NotImplementedError
