from .processors import (BGR2GRAY, BGR2RGB, RGB2BGR, RGB2GRAY, Cast, CenterCrop, Convert, ConvertAndPermute, Crop,
                         FDMat, FDMatBatch, FuseTransforms, HWC2CHW, LetterBoxResize, LimitByStride, LimitShort, Normalize,
                         NormalizeAndPermute, Pad, PadToSize, Processor, ProcessorManager, Resize, ResizeByShort,
                         StridePad, WarpAffine, chain_geometry, fuse_transforms, run_chain_gpu)
from .manager import PyProcessorManager
from . import manager, processors
