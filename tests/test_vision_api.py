"""Picture models behind one features / head interface, and detection as points (the categories of the
reference's vision tests: options change sizes as documented, a swapped head trains alone, a detector
learns to find squares, box scores)."""
import torch

import mimir_b200.tensor as T
from mimir_b200 import nn, optim, vision


def test_options_heads_and_transfer():
    small = vision.resnet18(10, small=True, width=16, in_channels=1, dropout=0.1).eval()
    x = T.tensor(torch.randn(2, 1, 32, 32))
    assert small.forward_features(x).shape == (2, 128, 4, 4) and small.features(x).shape == (2, 128) and small.width == 128
    assert small(x).shape == (2, 10)
    big = vision.resnet18(10, width=16).eval()
    assert big.forward_features(T.tensor(torch.randn(1, 3, 64, 64))).shape == (1, 128, 2, 2)
    before = {id(p) for p in small.parameters()}
    small.set_head(3)
    head = small.head_parameters()
    assert small(x).shape == (2, 3) and len(head) == 2 and all(id(p) not in before for p in head)
    # an optimizer given the head alone leaves the features as they were
    stem = small.stem.layers[0].weight.value().data().clone()
    opt = optim.SGD(head, lr=0.1)
    small.train()
    loss = nn.loss.cross_entropy(small(x), T.tensor(torch.tensor([0, 2])))
    loss.backward()
    opt.step()
    assert torch.equal(small.stem.layers[0].weight.value().data(), stem) and head[0].grad() is not None
    m = vision.MobileNetV2(4, width=0.25, small=True).eval()
    assert m(T.tensor(torch.randn(1, 3, 32, 32))).shape == (1, 4) and m.width == 320
    v = vision.ViT(image=32, patch=8, dim=32, depth=1, heads=2, mlp=64, classes=5).eval()
    assert v.features(T.tensor(torch.randn(2, 3, 32, 32))).shape == (2, 32) and v.width == 32
    v.set_head(2)
    assert v(T.tensor(torch.randn(2, 3, 32, 32))).shape == (2, 2)
    try:
        vision.ViT(image=30, patch=8)
        raise AssertionError("expected ValueError")
    except ValueError:
        pass


def _scene(gen, n=8, size=32):
    """Pictures with one bright square each, and where it is."""
    x = torch.zeros(n, 1, size, size)
    truth = []
    for i in range(n):
        s = int(torch.randint(8, 13, (1,), generator=gen))
        x0, y0 = (int(v) for v in torch.randint(0, size - s, (2,), generator=gen))
        x[i, 0, y0:y0 + s, x0:x0 + s] = 1.0
        truth.append([(0, float(x0), float(y0), float(x0 + s), float(y0 + s))])
    return x, truth


def test_detector_learns_to_find_squares():
    nn.manual_seed(0)
    gen = torch.Generator().manual_seed(0)
    det = vision.Detector(1, vision.tiny_backbone(1, 8), head_width=16)
    opt = optim.Adam(det.parameters(), lr=5e-3)
    first = last = None
    for step in range(80):
        x, truth = _scene(gen)
        out = det(T.tensor(x))
        assert out.shape == (8, 5, 8, 8)
        loss = det.loss(out, det.targets(truth, 32, 32))
        loss.backward()
        last = float(loss.item())
        first = last if first is None else first
        opt.step()
        opt.zero_grad()
    assert last < 0.5 * first
    det.eval()
    x, truth = _scene(gen, n=16)
    found = det.detect(det(T.tensor(x)), threshold=0.2, top=5)
    hits = sum(1 for f, t in zip(found, truth) if f and vision.iou(f[0].box, t[0][1:]) > 0.5)
    assert hits >= 12, hits
    dets = [[vision.Detection(0, d.score, d.box) for d in f] for f in found]
    gts = [[vision.Detection(0, 1.0, t[0][1:])] for t in truth]
    assert vision.mean_average_precision(dets, gts, 1) > 0.6
    t = det.targets([[(0, 8.0, 8.0, 20.0, 16.0)]], 32, 32)
    assert t.heat[0, 0, 3, 3] == 1.0 and t.mask.sum() == 1 and torch.allclose(t.size[0, :, 3, 3], torch.tensor([3.0, 2.0]))
    assert torch.allclose(t.offset[0, :, 3, 3], torch.tensor([0.5, 0.0])) and 0 < t.heat[0, 0, 3, 4] < 1
    coarse = vision.Detector(2, vision.resnet18(1, width=8).backbone(), head_width=8)
    assert coarse(T.tensor(torch.randn(1, 3, 64, 64))).shape == (1, 6, 16, 16)


def test_box_scores_and_losses():
    a, b = (0.0, 0.0, 2.0, 2.0), (1.0, 1.0, 3.0, 3.0)
    assert abs(vision.iou(a, b) - 1 / 7) < 1e-9 and vision.Detection(0, 1.0, a).area() == 4.0
    dets = [vision.Detection(0, 0.9, a), vision.Detection(0, 0.8, (0.1, 0.0, 2.0, 2.0)), vision.Detection(1, 0.7, a)]
    kept = vision.nms_detections(dets, 0.5)
    assert [(d.cls, d.score) for d in kept] == [(0, 0.9), (1, 0.7)]
    p = T.Param(torch.tensor([[0.0, 0.0, 2.0, 2.0], [5.0, 5.0, 6.0, 6.0]]))
    tgt = T.tensor(torch.tensor([[0.0, 0.0, 2.0, 2.0], [0.0, 0.0, 1.0, 1.0]]))
    loss = vision.giou_loss(p.value(), tgt)
    # identical boxes cost 0; disjoint ones cost 1 + the empty share of their hull (34 of 36)
    loss.backward()
    assert abs(float(loss.item()) - 0.5 * (1 + 34 / 36)) < 1e-6
    assert p.grad().data()[1].abs().sum() > 0 and p.grad().data()[0].abs().sum() < 1e-6
    pred, truth = torch.tensor([0, 0, 1, 1, 2, 2]), torch.tensor([0, 1, 1, 1, 2, 0])
    assert abs(vision.mean_iou(pred, truth, 4) - (1 / 3 + 2 / 3 + 1 / 2) / 3) < 1e-9


def test_native_suppression_keeps_the_boxes_of_the_overlap_table():
    """Greedy suppression on the host compares each box with the boxes kept so far; a full table of overlaps
    visited in the same order is its oracle, ties in score included."""
    import torch
    from mimir_b200.vision import boxes as VB
    g = torch.Generator().manual_seed(0)
    for n in (0, 1, 400):
        b = torch.rand(n, 4, generator=g) * 100
        b[:, 2:] = b[:, :2] + 10 + torch.rand(n, 2, generator=g) * 30
        s = (torch.rand(n, generator=g) * 20).round() / 20                     # repeated scores
        order = s.argsort(descending=True, stable=True)
        iou = VB.box_iou(b[order], b[order])
        keep, dead = [], torch.zeros(n, dtype=torch.bool)
        for i in range(n):
            if not dead[i]:
                keep.append(int(order[i]))
                dead |= iou[i] > 0.4
        assert VB.nms(b, s, 0.4).tolist() == keep
