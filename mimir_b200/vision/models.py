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


class ResNet(nn.Module):
    def __init__(self, block, depths, classes=1000, in_channels=3, width=64):
        self.stem = _conv_bn(in_channels, width, 7, 2, 3)
        self.pool = nn.MaxPool2d(3, 2, 1)
        blocks, cin = [], width
        for i, n in enumerate(depths):
            planes = width * 2 ** i
            for j in range(n):
                blocks.append(block(cin, planes, 2 if (j == 0 and i > 0) else 1))
                cin = planes * block.expansion
        self.blocks = blocks
        self.head = nn.Linear(cin, classes)
        self.features = cin

    def forward_features(self, x):
        x = self.pool(self.stem(x))
        for b in self.blocks:
            x = b(x)
        return x

    def forward(self, x):
        return self.head(T.mean(self.forward_features(x), dim=(2, 3)))


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


class MobileNetV2(nn.Module):
    CFG = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, classes=1000, width=1.0, in_channels=3):
        c = lambda v: max(8, int(v * width + 4) // 8 * 8)
        layers, cin = [_conv_bn(in_channels, c(32), 3, 2)], c(32)
        for t, ch, n, s in self.CFG:
            for i in range(n):
                layers.append(InvertedResidual(cin, c(ch), s if i == 0 else 1, t))
                cin = c(ch)
        layers.append(_conv_bn(cin, c(1280), 1))
        self.body = nn.Sequential(*layers)
        self.head = nn.Linear(c(1280), classes)

    def forward(self, x):
        return self.head(T.mean(self.body(x), dim=(2, 3)))


class ViT(nn.Module):
    """Patch embedding by a strided convolution, class token, learned positions, transformer encoder layers."""

    def __init__(self, image=224, patch=16, dim=768, depth=12, heads=12, mlp=3072, classes=1000, in_channels=3):
        self.patch = nn.Conv2d(in_channels, dim, patch, patch)
        n = (image // patch) ** 2
        self.cls = T.Param(torch.zeros(1, 1, dim), "cls")
        self.pos = T.Param(nn.normal_init((1, n + 1, dim), 0.02), "pos")
        self.layers = [nn.TransformerEncoderLayer(dim, heads, mlp, eps=1e-12, activation="gelu", dropout=0.0) for _ in range(depth)]
        self.norm = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, classes)

    def forward(self, x):
        p = self.patch(x)                                       # [B, dim, h, w]
        B, dim = p.shape[0], p.shape[1]
        tok = T.transpose(T.reshape(p, (B, dim, -1)), 1, 2)     # [B, n, dim]
        tok = T.cat([T.expand(self.cls.value(), (B, 1, dim)), tok], 1) + self.pos.value()
        for l in self.layers:
            tok = l(tok)
        return self.head(self.norm(tok)[:, 0])


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
        cin, ups = self.backbone.features, []
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
