"""Vision models and box utilities (reference: vision/): ResNet-18/34/50, MobileNetV2 and ViT behind one
features / head interface with options for channels, small pictures, width and dropout; a CenterNet
``Detector`` over any ``Backbone`` with targets, loss and decoding; U-Net; box IoU, NMS, GIoU loss,
mean average precision and mean IoU."""
from .models import (Backbone, CenterNet, DetectionTargets, Detector, Head, MobileNetV2, PictureModel, ResNet, UNet, ViT,  # noqa: F401
                     centernet_decode, centernet_loss, resnet18, resnet34, resnet50, tiny_backbone, vit_b16, vit_tiny)
from .boxes import (Detection, average_precision, box_iou, giou_loss, iou, mean_average_precision, mean_iou, nms,  # noqa: F401
                    nms_detections)
