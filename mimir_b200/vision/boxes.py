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
    """The boxes kept by greedy suppression, best first.  On the host each box is compared with the boxes kept
    so far in native code (``mimir_cpu_nms``); elsewhere against a full table of overlaps."""
    order = scores.argsort(descending=True, stable=True)
    if boxes.device.type == "cpu" and scores.device.type == "cpu":
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_nms_bound", False):
            lib.mimir_cpu_nms.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p]
            lib.mimir_cpu_nms.restype = ctypes.c_longlong
            lib._nms_bound = True
        b = boxes.float().reshape(-1, 4).contiguous()
        order = order.contiguous()
        keep = torch.empty(b.shape[0], dtype=torch.long)
        count = lib.mimir_cpu_nms(b.data_ptr(), order.data_ptr(), b.shape[0], float(threshold), keep.data_ptr())
        if count < 0:
            raise ValueError("nms: boxes and scores do not match")
        return keep[:count].clone()
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


# ---------------------------------------------------------------------------------------------
# Things found, their losses and scores (reference: vision/boxes.go, vision/unet.go: MeanIoU)
# ---------------------------------------------------------------------------------------------
from dataclasses import dataclass  # noqa: E402


@dataclass
class Detection:
    cls: int
    score: float
    box: tuple                # (x1, y1, x2, y2)

    def area(self) -> float:
        return max(self.box[2] - self.box[0], 0.0) * max(self.box[3] - self.box[1], 0.0)


def iou(a, b) -> float:
    """Intersection over union of two ``(x1, y1, x2, y2)`` boxes."""
    return float(box_iou(torch.tensor([a], dtype=torch.float64), torch.tensor([b], dtype=torch.float64))[0, 0])


def nms_detections(dets, threshold: float = 0.5) -> list:
    """Greedy suppression within each class: a detection goes when a better one of its class overlaps it by
    more than ``threshold``."""
    out = []
    for c in sorted({d.cls for d in dets}):
        group = [d for d in dets if d.cls == c]
        keep = nms(torch.tensor([d.box for d in group], dtype=torch.float32), torch.tensor([d.score for d in group]), threshold)
        out += [group[i] for i in keep.tolist()]
    return sorted(out, key=lambda d: -d.score)


def giou_loss(pred, target):
    """``1 - GIoU`` of each pair of boxes ``[n, 4]`` in lazy tensor ops (so it trains a box regressor):
    IoU minus the share of the smallest enclosing box that neither covers."""
    from .. import tensor as T
    n = pred.shape[0]
    col = lambda t, j: T.reshape(T.shrink(t, ((0, n), (j, j + 1))), (n,))  # noqa: E731
    px1, py1, px2, py2 = (col(pred, j) for j in range(4))
    tx1, ty1, tx2, ty2 = (col(target, j) for j in range(4))
    area = lambda x1, y1, x2, y2: T.relu(x2 - x1) * T.relu(y2 - y1)  # noqa: E731
    inter = T.relu(T.minimum(px2, tx2) - T.maximum(px1, tx1)) * T.relu(T.minimum(py2, ty2) - T.maximum(py1, ty1))
    union = area(px1, py1, px2, py2) + area(tx1, ty1, tx2, ty2) - inter
    hull = T.relu(T.maximum(px2, tx2) - T.minimum(px1, tx1)) * T.relu(T.maximum(py2, ty2) - T.minimum(py1, ty1))
    g = inter / T.maximum(union, 1e-12) - (hull - union) / T.maximum(hull, 1e-12)
    return T.mean(1.0 - g)


def mean_average_precision(dets, truth, classes: int, iou_threshold: float = 0.5) -> float:
    """``dets[i]`` / ``truth[i]``: the detections found in, and the true things of, picture i (``Detection``s;
    a true thing's score is ignored).  Average precision per class over all pictures (a detection matches the
    unmatched true thing of its picture and class it overlaps most, at ``iou_threshold`` or more), averaged
    over the classes that have true things."""
    aps = []
    for c in range(classes):
        total = sum(1 for t in truth for d in t if d.cls == c)
        if total == 0:
            continue
        cand = sorted(((d.score, i, d) for i, ds in enumerate(dets) for d in ds if d.cls == c), key=lambda z: -z[0])
        used = {i: [False] * len([d for d in t if d.cls == c]) for i, t in enumerate(truth)}
        tp = []
        for _, i, d in cand:
            gts = [t for t in truth[i] if t.cls == c]
            best, at = 0.0, -1
            for j, gt in enumerate(gts):
                if not used[i][j]:
                    v = iou(d.box, gt.box)
                    if v > best:
                        best, at = v, j
            hit = at >= 0 and best >= iou_threshold
            if hit:
                used[i][at] = True
            tp.append(1.0 if hit else 0.0)
        if not tp:
            aps.append(0.0)
            continue
        ctp = torch.tensor(tp).cumsum(0)
        recall, precision = ctp / total, ctp / torch.arange(1, len(tp) + 1)
        precision = torch.flip(torch.cummax(torch.flip(precision, [0]), 0).values, [0])
        prev = torch.cat([torch.zeros(1), recall[:-1]])
        aps.append(float(((recall - prev) * precision).sum()))
    return sum(aps) / len(aps) if aps else 0.0


def mean_iou(pred, truth, classes: int) -> float:
    """Segmentation score: intersection over union of each class's pixels, averaged over the classes that
    appear in either."""
    p, t = torch.as_tensor(pred).reshape(-1).long(), torch.as_tensor(truth).reshape(-1).long()
    conf = torch.bincount(t * classes + p, minlength=classes * classes).reshape(classes, classes).double()
    inter = conf.diag()
    union = conf.sum(0) + conf.sum(1) - inter
    seen = union > 0
    return float((inter[seen] / union[seen]).mean()) if seen.any() else 0.0
