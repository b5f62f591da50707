"""``fastdeploy.vision.detection``."""
from .ppdet import (FCOS, GFL, PPYOLO, PPYOLOE, PPYOLOER, PPYOLOESOD, RTMDet, SOLOv2, SSD, TOOD, CascadeRCNN,
                    FasterRCNN, MaskRCNN, NMSOption, NMSRotatedOption, PaddleDetectionModel, PaddleDetPostprocessor,
                    PaddleDetPreprocessor, PaddleYOLOv5, PaddleYOLOv6, PaddleYOLOv7, PaddleYOLOv8, PaddleYOLOX,
                    PicoDet, PPDetBase, PSSDet, RetinaNet, TTFNet, YOLOv3)
from .contrib import (RKYOLOV5, RKYOLOV7, RKYOLOX, YOLOR, YOLOX, FastestDet, NanoDetPlus, ScaledYOLOv4,  # noqa: E402
                      YOLOPostprocessor, YOLOPreprocessor, YOLOv5, YOLOv5Lite, YOLOv5Seg, YOLOv6, YOLOv7,
                      YOLOv7End2EndORT, YOLOv7End2EndTRT, YOLOv8, letterbox,
                      FastestDetPostprocessor, FastestDetPreprocessor, RKYOLOPostprocessor, RKYOLOPreprocessor,
                      YOLOv5Postprocessor, YOLOv5Preprocessor, YOLOv5SegPostprocessor, YOLOv5SegPreprocessor,
                      YOLOv7Postprocessor, YOLOv7Preprocessor, YOLOv8Postprocessor, YOLOv8Preprocessor)
