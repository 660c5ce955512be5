"""Image models on the nn layer set (reference: vision/resnet.go, mobilenet.go, vit.go, unet.go,
centernet.go)."""
from __future__ import annotations

import math

import torch

from .. import nn
from .. import tensor as T


def _conv_bn(cin, cout, k, stride=1, padding=None, groups=1, act=True):
    padding = k // 2 if padding is None else padding
    layers = [nn.Conv2d(cin, cout, k, stride, padding, groups=groups, bias=False), nn.BatchNorm2d(cout)]
    if act:
        layers.append(nn.ReLU())
    return nn.Sequential(*layers)


class Head(nn.Module):
    """A classifier: dropout (while training), then a linear layer."""

    def __init__(self, width: int, classes: int, dropout: float = 0.0):
        self.drop = nn.Dropout(dropout) if dropout > 0 else None
        self.linear = nn.Linear(width, classes)

    def forward(self, x):
        return self.linear(self.drop(x) if self.drop is not None else x)


class PictureModel(nn.Module):
    """A picture network split into what it sees and what it says (vision/vision.go: Model):
    ``features`` reads a batch of pictures into one vector each and ``head`` turns that into logits.
    Transfer learning keeps the features and swaps the head: ``set_head`` starts a new one for other
    classes, and ``head_parameters`` alone are what an optimizer is given to fit only the head."""

    width = 0
    _nn_skip_dropout = 0.0

    def features(self, x):
        raise NotImplementedError

    def forward(self, x):
        return self.head(self.features(x))

    def set_head(self, classes: int) -> None:
        self.head = Head(self.width, classes, self._nn_skip_dropout)

    def head_parameters(self) -> list:
        return self.head.parameters()


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, cin, planes, stride):
        self.a = _conv_bn(cin, planes, 3, stride)
        self.b = _conv_bn(planes, planes, 3, act=False)
        self.down = _conv_bn(cin, planes, 1, stride, act=False) if stride != 1 or cin != planes else None

    def forward(self, x):
        y = self.b(self.a(x))
        return T.relu(y + (self.down(x) if self.down is not None else x))


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, planes, stride):
        self.a = _conv_bn(cin, planes, 1)
        self.b = _conv_bn(planes, planes, 3, stride)
        self.c = _conv_bn(planes, planes * 4, 1, act=False)
        self.down = _conv_bn(cin, planes * 4, 1, stride, act=False) if stride != 1 or cin != planes * 4 else None

    def forward(self, x):
        y = self.c(self.b(self.a(x)))
        return T.relu(y + (self.down(x) if self.down is not None else x))


class ResNet(PictureModel):
    """``small`` fits the model to 32 to 64 pixel pictures (CIFAR): the first layer keeps the size where
    it otherwise shrinks a 224-pixel photo fourfold.  ``width`` is the first stage's channels (64 times
    a multiplier, e.g. 32 for a model a quarter the size); ``dropout`` acts on the features before the head."""

    def __init__(self, block, depths, classes=1000, in_channels=3, width=64, small=False, dropout=0.0):
        width = max(8, int(round(width)))
        self.stem = _conv_bn(in_channels, width, 3, 1, 1) if small else _conv_bn(in_channels, width, 7, 2, 3)
        self.pool = None if small else nn.MaxPool2d(3, 2, 1)
        self._nn_skip_small, self._nn_skip_dropout = small, dropout
        blocks, cin = [], width
        for i, n in enumerate(depths):
            planes = width * 2 ** i
            for j in range(n):
                blocks.append(block(cin, planes, 2 if (j == 0 and i > 0) else 1))
                cin = planes * block.expansion
        self.blocks = blocks
        self.width = cin
        self.head = Head(cin, classes, dropout)

    def forward_features(self, x):
        """The last feature map, before the average and head: 32 times smaller than the picture (8 when small)."""
        x = self.stem(x)
        if self.pool is not None:
            x = self.pool(x)
        for b in self.blocks:
            x = b(x)
        return x

    def features(self, x):
        return T.mean(self.forward_features(x), dim=(2, 3))

    def backbone(self) -> "Backbone":
        """This network's feature maps as a detector's backbone; the weights are shared, so a ResNet taught to
        classify starts a detector that already sees."""
        return Backbone(self.forward_features, self.width, 8 if self._nn_skip_small else 32, self)


def resnet18(classes=1000, **kw): return ResNet(BasicBlock, (2, 2, 2, 2), classes, **kw)
def resnet34(classes=1000, **kw): return ResNet(BasicBlock, (3, 4, 6, 3), classes, **kw)
def resnet50(classes=1000, **kw): return ResNet(Bottleneck, (3, 4, 6, 3), classes, **kw)


class InvertedResidual(nn.Module):
    def __init__(self, cin, cout, stride, expand):
        hidden = cin * expand
        layers = []
        if expand != 1:
            layers.append(_conv_bn(cin, hidden, 1))
        layers += [_conv_bn(hidden, hidden, 3, stride, groups=hidden), _conv_bn(hidden, cout, 1, act=False)]
        self.body = nn.Sequential(*layers)
        self.skip = stride == 1 and cin == cout

    def forward(self, x):
        return x + self.body(x) if self.skip else self.body(x)


class MobileNetV2(PictureModel):
    CFG = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, classes=1000, width=1.0, in_channels=3, small=False, dropout=0.2):
        c = lambda v: max(8, int(v * width + 4) // 8 * 8)
        layers, cin = [_conv_bn(in_channels, c(32), 3, 1 if small else 2)], c(32)
        for k, (t, ch, n, s) in enumerate(self.CFG):
            if small and k == 1:
                s = 1                                           # small pictures keep their size one stage longer
            for i in range(n):
                layers.append(InvertedResidual(cin, c(ch), s if i == 0 else 1, t))
                cin = c(ch)
        layers.append(_conv_bn(cin, c(1280), 1))
        self.body = nn.Sequential(*layers)
        self.width, self._nn_skip_dropout = c(1280), dropout
        self.head = Head(self.width, classes, dropout)

    def features(self, x):
        return T.mean(self.body(x), dim=(2, 3))


class ViT(PictureModel):
    """Patch embedding by a strided convolution, class token, learned positions, transformer encoder layers."""

    def __init__(self, image=224, patch=16, dim=768, depth=12, heads=12, mlp=3072, classes=1000, in_channels=3, dropout=0.0):
        if image % patch or dim % heads:
            raise ValueError(f"ViT: pictures of {image} pixels in patches of {patch}, or {dim} features over {heads} heads")
        self.patch = nn.Conv2d(in_channels, dim, patch, patch)
        self.width, self._nn_skip_dropout = dim, dropout
        n = (image // patch) ** 2
        self.cls = T.Param(torch.zeros(1, 1, dim), "cls")
        self.pos = T.Param(nn.normal_init((1, n + 1, dim), 0.02), "pos")
        self.layers = [nn.TransformerEncoderLayer(dim, heads, mlp, eps=1e-12, activation="gelu", dropout=0.0) for _ in range(depth)]
        self.norm = nn.LayerNorm(dim)
        self.head = Head(dim, classes, dropout)

    def features(self, x):
        p = self.patch(x)                                       # [B, dim, h, w]
        B, dim = p.shape[0], p.shape[1]
        tok = T.transpose(T.reshape(p, (B, dim, -1)), 1, 2)     # [B, n, dim]
        tok = T.cat([T.expand(self.cls.value(), (B, 1, dim)), tok], 1) + self.pos.value()
        for l in self.layers:
            tok = l(tok)
        return self.norm(tok)[:, 0]


def vit_b16(classes=1000, **kw):
    """ViT-B/16: 224-pixel pictures in 16-pixel patches, 768 features, 12 layers of 12 heads."""
    return ViT(224, 16, 768, 12, 12, 3072, classes, **kw)


def vit_tiny(classes=1000, image=224, patch=16, **kw):
    """ViT-Ti: 192 features, 12 layers of 3 heads."""
    return ViT(image, patch, 192, 12, 3, 768, classes, **kw)


class UNet(nn.Module):
    def __init__(self, in_channels=3, classes=1, width=32, depth=4):
        def block(a, b):
            return nn.Sequential(_conv_bn(a, b, 3), _conv_bn(b, b, 3))
        self.down = [block(in_channels if i == 0 else width * 2 ** (i - 1), width * 2 ** i) for i in range(depth)]
        self.mid = block(width * 2 ** (depth - 1), width * 2 ** depth)
        self.up = [nn.ConvTranspose2d(width * 2 ** (i + 1), width * 2 ** i, 2, 2) for i in reversed(range(depth))]
        self.dec = [block(width * 2 ** (i + 1), width * 2 ** i) for i in reversed(range(depth))]
        self.pool = nn.MaxPool2d(2)
        self.head = nn.Conv2d(width, classes, 1)

    def forward(self, x):
        skips = []
        for d in self.down:
            x = d(x)
            skips.append(x)
            x = self.pool(x)
        x = self.mid(x)
        for u, d, s in zip(self.up, self.dec, reversed(skips)):
            x = d(T.cat([u(x), s], 1))
        return self.head(x)


class CenterNet(nn.Module):
    """Keypoint detector: a ResNet trunk, three transposed-convolution upsamplings, and heat-map /
    size / offset heads at stride 4."""

    def __init__(self, classes=80, backbone=None, head_width=64):
        self.backbone = backbone or resnet18()
        cin, ups = self.backbone.width, []
        for c in (256, 128, 64):
            ups += [nn.ConvTranspose2d(cin, c, 4, 2, 1, bias=False), nn.BatchNorm2d(c), nn.ReLU()]
            cin = c
        self.up = nn.Sequential(*ups)

        def head(n):
            return nn.Sequential(nn.Conv2d(64, head_width, 3, padding=1), nn.ReLU(), nn.Conv2d(head_width, n, 1))
        self.heat, self.size, self.offset = head(classes), head(2), head(2)
        self.heat.layers[-1].bias.set(torch.full((classes,), -2.19))

    def forward(self, x):
        f = self.up(self.backbone.forward_features(x))
        return self.heat(f), self.size(f), self.offset(f)


def centernet_loss(heat, size, offset, target_heat, target_size, target_offset, mask, alpha=2.0, beta=4.0):
    """Penalty-reduced focal loss on the heat map plus L1 on size / offset at object centres (``mask``)."""
    p = T.clamp(T.sigmoid(heat), 1e-4, 1 - 1e-4)
    pos = T.cast(T.equal(target_heat, T.ones_like(target_heat)) if hasattr(T, "ones_like") else (target_heat >= 1.0), p.dtype)
    neg = 1.0 - pos
    pos_loss = T.log(p) * T.pow_(1.0 - p, alpha) * pos
    neg_loss = T.log(1.0 - p) * T.pow_(p, alpha) * T.pow_(1.0 - target_heat, beta) * neg
    n = T.maximum(T.sum_(pos), T.tensor(1.0))
    focal = -(T.sum_(pos_loss) + T.sum_(neg_loss)) / n
    m = T.unsqueeze(mask, 1)
    l1 = (T.sum_(T.abs_(size - target_size) * m) * 0.1 + T.sum_(T.abs_(offset - target_offset) * m)) / n
    return focal + l1


def centernet_decode(heat: torch.Tensor, size: torch.Tensor, offset: torch.Tensor, k: int = 100, stride: int = 4):
    """Peaks of the heat map (3x3 max filter) -> ``boxes [B, k, 4]`` (x1, y1, x2, y2), ``scores``, ``classes``."""
    p = torch.sigmoid(heat)
    keep = (torch.nn.functional.max_pool2d(p, 3, 1, 1) == p).float() * p
    B, C, H, W = keep.shape
    scores, idx = keep.view(B, -1).topk(min(k, C * H * W))
    cls, pix = idx // (H * W), idx % (H * W)
    ys, xs = (pix // W).float(), (pix % W).float()
    gather = lambda t, c: t[:, c].reshape(B, -1).gather(1, pix)
    cx, cy = xs + gather(offset, 0), ys + gather(offset, 1)
    w, h = gather(size, 0), gather(size, 1)
    boxes = torch.stack([cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2], -1) * stride
    return boxes, scores, cls


# ---------------------------------------------------------------------------------------------
# Detection as points (reference: vision/detect.go)
# ---------------------------------------------------------------------------------------------
class Backbone(nn.Module):
    """Reads pictures into feature maps for a ``Detector``: ``[N, C, H, W] -> [N, channels, H/stride, W/stride]``."""

    def __init__(self, fn, channels: int, stride: int, owner=None):
        self._nn_skip_fn, self.channels, self.stride = fn, channels, stride
        self.owner = owner                      # the module whose weights ``fn`` runs (kept so they are saved and trained)

    def forward(self, x):
        return self._nn_skip_fn(x)


def tiny_backbone(in_channels: int, width: int) -> Backbone:
    """Four convolutions from ``in_channels`` to ``2 * width`` channels, four times smaller than the picture:
    a backbone that learns in seconds, for small pictures and few kinds of thing."""
    body = nn.Sequential(_conv_bn(in_channels, width, 3, 1), _conv_bn(width, width, 3, 2), _conv_bn(width, 2 * width, 3, 2),
                         _conv_bn(2 * width, 2 * width, 3, 1))
    return Backbone(body, 2 * width, 4, body)


DETECTOR_STRIDE = 4


class DetectionTargets:
    """What a detector should give for a batch of pictures, on its grid: ``heat [N, classes, h, w]`` (a
    Gaussian bump around every true centre, 1 at the centre), ``size`` and ``offset [N, 2, h, w]`` and
    ``mask [N, h, w]`` (1 at the centres)."""

    def __init__(self, heat, size, offset, mask):
        self.heat, self.size, self.offset, self.mask = heat, size, offset, mask


def _gaussian_radius(h: float, w: float, min_overlap: float = 0.7) -> float:
    """How far a corner may move with the box still overlapping the true one by ``min_overlap`` (CenterNet)."""
    a1, b1, c1 = 1.0, h + w, w * h * (1 - min_overlap) / (1 + min_overlap)
    r1 = (b1 - math.sqrt(max(b1 * b1 - 4 * a1 * c1, 0.0))) / 2
    a2, b2, c2 = 4.0, 2 * (h + w), (1 - min_overlap) * w * h
    r2 = (b2 - math.sqrt(max(b2 * b2 - 4 * a2 * c2, 0.0))) / (2 * a2)
    a3, b3, c3 = 4 * min_overlap, -2 * min_overlap * (h + w), (min_overlap - 1) * w * h
    r3 = (b3 + math.sqrt(max(b3 * b3 - 4 * a3 * c3, 0.0))) / (2 * a3)
    return max(0.0, min(r1, r2, r3))


class Detector(nn.Module):
    """Finds things in pictures as CenterNet does ("objects as points"): on a grid four times smaller than
    the picture it scores, for each kind of thing, how likely each cell holds a thing's centre, and says how
    wide and tall that thing is and where in the cell its centre lies.  The peaks of the scores are the
    things found, so it needs no anchors and no NMS.  ``forward`` maps ``[N, C, H, W]`` to
    ``[N, classes + 4, H/4, W/4]``: centre logits per class, then width, height, x and y offset in grid cells.
    A backbone coarser than the grid is grown to it by transposed convolutions."""

    def __init__(self, classes: int, backbone: Backbone, head_width: int = 64):
        if classes < 1 or backbone.stride < DETECTOR_STRIDE or backbone.stride & (backbone.stride - 1):
            raise ValueError(f"detector: {classes} classes on a backbone of stride {backbone.stride} (want a power of two, at least 4)")
        self.classes, self.backbone = classes, backbone
        cin, ups, stride, c = backbone.channels, [], backbone.stride, 256
        while stride > DETECTOR_STRIDE:
            ups += [nn.ConvTranspose2d(cin, c, 4, 2, 1, bias=False), nn.BatchNorm2d(c), nn.ReLU()]
            cin, c, stride = c, max(c // 2, 64), stride // 2
        self.up = nn.Sequential(*ups) if ups else None
        self.neck = nn.Sequential(nn.Conv2d(cin, head_width, 3, padding=1), nn.ReLU())
        self.out = nn.Conv2d(head_width, classes + 4, 1)
        bias = torch.zeros(classes + 4)
        bias[:classes] = -2.19                              # centres are rare: start the scores near 0.1
        self.out.bias.set(bias)

    def forward(self, x):
        f = self.backbone(x)
        if self.up is not None:
            f = self.up(f)
        return self.out(self.neck(f))

    def targets(self, truth, h: int, w: int) -> DetectionTargets:
        """``truth[i]``: the true things of picture i as ``(class, x1, y1, x2, y2)`` in pixels, for pictures of
        height ``h`` and width ``w``."""
        if h % DETECTOR_STRIDE or w % DETECTOR_STRIDE:
            raise ValueError(f"detector: pictures of {h} x {w}, want multiples of {DETECTOR_STRIDE}")
        gh, gw, n = h // DETECTOR_STRIDE, w // DETECTOR_STRIDE, len(truth)
        heat = torch.zeros(n, self.classes, gh, gw)
        size, offset, mask = torch.zeros(n, 2, gh, gw), torch.zeros(n, 2, gh, gw), torch.zeros(n, gh, gw)
        ys, xs = torch.arange(gh, dtype=torch.float32)[:, None], torch.arange(gw, dtype=torch.float32)[None]
        for i, things in enumerate(truth):
            for cls, x1, y1, x2, y2 in things:
                if not 0 <= int(cls) < self.classes:
                    raise ValueError(f"detector: class {cls} of {self.classes}")
                bw, bh = (x2 - x1) / DETECTOR_STRIDE, (y2 - y1) / DETECTOR_STRIDE
                if bw <= 0 or bh <= 0:
                    continue
                cx, cy = (x1 + x2) / 2 / DETECTOR_STRIDE, (y1 + y2) / 2 / DETECTOR_STRIDE
                ix, iy = min(max(int(cx), 0), gw - 1), min(max(int(cy), 0), gh - 1)
                sigma = (2 * int(_gaussian_radius(math.ceil(bh), math.ceil(bw))) + 1) / 6.0     # a bump of diameter 2 r + 1
                bump = torch.exp(-((xs - ix) ** 2 + (ys - iy) ** 2) / (2 * sigma * sigma))
                heat[i, int(cls)] = torch.maximum(heat[i, int(cls)], bump)
                size[i, :, iy, ix] = torch.tensor([bw, bh])
                offset[i, :, iy, ix] = torch.tensor([cx - ix, cy - iy])
                mask[i, iy, ix] = 1.0
        return DetectionTargets(heat, size, offset, mask)

    def _parts(self, out):
        n, _, gh, gw = out.shape
        c = self.classes
        cut = lambda lo, hi: T.shrink(out, ((0, n), (lo, hi), (0, gh), (0, gw)))  # noqa: E731
        return cut(0, c), cut(c, c + 2), cut(c + 2, c + 4)

    def loss(self, out, t: DetectionTargets):
        """The penalty-reduced focal loss of the centre scores, plus a tenth of the L1 error of the sizes and
        the L1 error of the offsets at the centres."""
        heat, size, offset = self._parts(out)
        dev = out.device
        return centernet_loss(heat, size, offset, T.tensor(t.heat, device=dev), T.tensor(t.size, device=dev),
                              T.tensor(t.offset, device=dev), T.tensor(t.mask, device=dev))

    def detect(self, out, threshold: float = 0.3, top: int = 100) -> list:
        """The things found in each picture: the peaks of the centre scores (cells whose 3x3 neighbourhood
        holds no higher score), up to ``top`` a picture scoring at least ``threshold``, best first, as
        ``Detection(cls, score, (x1, y1, x2, y2))`` with boxes in pixels."""
        from .boxes import Detection
        v = out.data().float().cpu()
        c = self.classes
        boxes, scores, cls = centernet_decode(v[:, :c], v[:, c:c + 2], v[:, c + 2:], k=top, stride=DETECTOR_STRIDE)
        found = []
        for b in range(v.shape[0]):
            keep = scores[b] >= threshold
            found.append([Detection(int(k), float(s), tuple(float(z) for z in bx))
                          for k, s, bx in zip(cls[b][keep], scores[b][keep], boxes[b][keep])])
        return found
