"""Box metrics (reference: vision/boxes.go): IoU matrix, greedy NMS, average precision."""
from __future__ import annotations

import torch


def box_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[n, 4] x [m, 4] (x1, y1, x2, y2) -> [n, m]."""
    area = lambda t: (t[:, 2] - t[:, 0]).clamp_min(0) * (t[:, 3] - t[:, 1]).clamp_min(0)
    lt = torch.maximum(a[:, None, :2], b[None, :, :2])
    rb = torch.minimum(a[:, None, 2:], b[None, :, 2:])
    inter = (rb - lt).clamp_min(0).prod(-1)
    return inter / (area(a)[:, None] + area(b)[None] - inter).clamp_min(1e-12)


def nms(boxes: torch.Tensor, scores: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    order = scores.argsort(descending=True)
    iou = box_iou(boxes[order], boxes[order])
    keep, dead = [], torch.zeros(len(order), dtype=torch.bool)
    for i in range(len(order)):
        if dead[i]:
            continue
        keep.append(int(order[i]))
        dead |= iou[i] > threshold
    return torch.tensor(keep, dtype=torch.long)


def average_precision(pred_boxes, pred_scores, true_boxes, iou_threshold: float = 0.5) -> float:
    """Area under the interpolated precision/recall curve for one class in one image set."""
    if len(true_boxes) == 0:
        return 0.0
    order = pred_scores.argsort(descending=True)
    iou = box_iou(pred_boxes[order], true_boxes) if len(order) else torch.zeros(0, len(true_boxes))
    used = torch.zeros(len(true_boxes), dtype=torch.bool)
    tp = torch.zeros(len(order))
    for i in range(len(order)):
        best = iou[i].clone()
        best[used] = -1
        j = int(best.argmax())
        if best[j] >= iou_threshold:
            used[j], tp[i] = True, 1
    ctp = tp.cumsum(0)
    recall = ctp / len(true_boxes)
    precision = ctp / torch.arange(1, len(order) + 1)
    for i in range(len(precision) - 2, -1, -1):
        precision[i] = torch.maximum(precision[i], precision[i + 1])
    prev, ap = 0.0, 0.0
    for r, p in zip(recall.tolist(), precision.tolist()):
        ap += (r - prev) * p
        prev = r
    return ap
