"""``fastdeploy.vision.detection``."""
from .ppdet import (FCOS, GFL, PPYOLO, PPYOLOE, PPYOLOER, PPYOLOESOD, RTMDet, SOLOv2, SSD, TOOD, CascadeRCNN,
                    FasterRCNN, MaskRCNN, NMSOption, PaddleDetectionModel, PaddleDetPostprocessor,
                    PaddleDetPreprocessor, PaddleYOLOv5, PaddleYOLOv6, PaddleYOLOv7, PaddleYOLOv8, PaddleYOLOX,
                    PicoDet, PPDetBase, PSSDet, RetinaNet, TTFNet, YOLOv3)
