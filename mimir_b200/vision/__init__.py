"""Vision models and box utilities (reference: vision/): ResNet-18/34/50, MobileNetV2, ViT,
U-Net, CenterNet, IoU / NMS / average precision."""
from .models import (CenterNet, MobileNetV2, ResNet, UNet, ViT, centernet_decode, centernet_loss, resnet18,
                     resnet34, resnet50)
from .boxes import average_precision, box_iou, nms
