"""Operations the graph vocabulary has no word for, rewritten in operations it has.

The exporter translates a traced op into graph primitives and standard-library calls (``io/export.py``).
An op without a translation of its own is rebuilt here from public tensor ops that do have one; since the
trace is live while the rewrite runs, every op of the rewrite is reported and translated in turn, and the
exporter then lets the original result stand for the rewrite's.  So a rewrite is ordinary lazy-tensor code
and is checked the ordinary way: it must agree with the op it replaces (``tests/test_graph.py``).

Sizes that a rewrite bakes in as constants (an index range, a window count) must be fixed sizes: an axis
declared dynamic at export keeps working only where the rewrite does not need its length.
"""
from __future__ import annotations

import math

import torch

from ..tensor import core as C
from ..tensor import errors as E

T = C


def _const(v, like, dtype=None):
    return C.tensor(torch.as_tensor(v, dtype=dtype), device=like.device)


def _iota(n, like, shape=None, dtype=torch.int64):
    t = torch.arange(n, dtype=dtype)
    return C.tensor(t.reshape(shape) if shape is not None else t, device=like.device)


def clamp(x, lo=None, hi=None):
    y = x
    if lo is not None:
        y = T.maximum(y, lo)
    if hi is not None:
        y = T.minimum(y, hi)
    return y


def softplus(x):
    return T.relu(x) + T.log(T.exp(T.neg(T.abs_(x))) + 1.0)


def log1p(x):
    # the logarithm of 1 + x loses x below float32's spacing at 1: the first terms of the series stand in there
    small = T.less(T.abs_(x), 1e-4)
    return T.where(small, x * (1.0 - x * 0.5), T.log(x + 1.0))


def expm1(x):
    small = T.less(T.abs_(x), 1e-4)
    return T.where(small, x * (x * 0.5 + 1.0), T.exp(x) - 1.0)


def sign(x):
    return T.where(T.less(x, 0.0), x * 0.0 - 1.0, T.where(T.less(0.0, x), x * 0.0 + 1.0, x * 0.0))


def _trunc(x):
    return T.cast(T.cast(x, torch.int32), x.dtype)


def floor(x):
    t = _trunc(x)
    return T.where(T.less(x, t), t - 1.0, t)


def ceil(x):
    t = _trunc(x)
    return T.where(T.less(t, x), t + 1.0, t)


def var(x, dim=None, keepdim=False):
    """The sample variance (divisor n - 1), like the op."""
    shape = tuple(x.shape)
    axes = tuple(range(len(shape))) if dim is None else tuple(d % len(shape) for d in ((dim,) if isinstance(dim, int) else dim))
    n = math.prod(shape[a] for a in axes)
    d = x - T.mean(x, dim=axes, keepdim=True)
    s = T.sum_(d * d, axes, keepdim=True) * (1.0 / max(n - 1, 1))
    if keepdim and dim is not None:
        return s
    return T.reshape(s, tuple(shape[i] for i in range(len(shape)) if i not in axes))


def logsumexp(x, dim=None, keepdim=False):
    shape = tuple(x.shape)
    axes = tuple(range(len(shape))) if dim is None else tuple(d % len(shape) for d in ((dim,) if isinstance(dim, int) else dim))
    m = T.max_(x, axes, keepdim=True) if len(axes) == 1 else T.reshape(T.max_(x), (1,) * len(shape)) if dim is None else None
    if m is None:
        m = x
        for a in axes:
            m = T.max_(m, a, keepdim=True)
    s = T.log(T.sum_(T.exp(x - m), axes, keepdim=True)) + m
    if keepdim and dim is not None:
        return s
    return T.reshape(s, tuple(shape[i] for i in range(len(shape)) if i not in axes))


def flip(x, dims):
    """Rows taken in reverse order, one axis at a time (the axis moves to the front for the row gather)."""
    n = len(x.shape)
    for d in ((dims,) if isinstance(dims, int) else dims):
        d %= n
        perm = [d] + [i for i in range(n) if i != d]
        back = [perm.index(i) for i in range(n)]
        rev = C.tensor(torch.arange(x.shape[d] - 1, -1, -1, dtype=torch.int64), device=x.device)
        x = T.permute(T.gather_rows(T.permute(x, perm), rev), back)
    return x


def stack(xs, dim=0):
    n = len(xs[0].shape) + 1
    return T.cat([T.unsqueeze(t, dim % n) for t in xs], dim % n)


def split(x, sizes, dim=0):
    n = len(x.shape)
    dim %= n
    total = x.shape[dim]
    if isinstance(sizes, int):
        sizes = [sizes] * (total // sizes) + ([total % sizes] if total % sizes else [])
    out, at = [], 0
    for s in sizes:
        out.append(T.shrink(x, tuple((at, at + s) if i == dim else (0, x.shape[i]) for i in range(n))))
        at += s
    return tuple(out)


def one_hot(index, classes, dtype=torch.float32):
    hit = T.equal(T.unsqueeze(index, -1), _iota(classes, index, dtype=index.dtype))
    return T.cast(hit, dtype)


def argmax(x, dim=-1):
    """The first position of the maximum along ``dim``: positions that hold it keep their number, the others the
    axis' length, and the smallest wins."""
    n = len(x.shape)
    dim %= n
    size = x.shape[dim]
    shape = [1] * n
    shape[dim] = size
    pos = C.tensor(torch.arange(size, dtype=torch.float32).reshape(shape), device=x.device)
    best = T.max_(x, dim, keepdim=True)
    cand = T.where(T.equal(x, best), pos, pos * 0.0 + float(size))
    return T.cast(T.min_(cand, dim), torch.int64)


def gather(x, dim, index):
    """``out[..., j, ...] = x[..., index[..., j, ...], ...]`` along ``dim`` by comparing the index with the
    positions of the axis (cost: the axis' length times the result; meant for short axes such as classes)."""
    n = len(x.shape)
    dim %= n
    if len(index.shape) != n or any(index.shape[i] != x.shape[i] for i in range(n) if i != dim):
        raise E.ErrUnsupported("export: gather whose index does not cover the operand's other axes")
    perm = [i for i in range(n) if i != dim] + [dim]
    back = [perm.index(i) for i in range(n)]
    xs, idx = T.permute(x, perm), T.permute(index, perm)                   # [..., K] and [..., J]
    hit = T.equal(T.unsqueeze(idx, -1), _iota(x.shape[dim], x, dtype=index.dtype))       # [..., J, K]
    picked = T.sum_(T.where(hit, T.unsqueeze(xs, -2), 0.0 if x.dtype.is_floating_point else 0), -1)
    return T.permute(T.cast(picked, x.dtype) if picked.dtype != x.dtype else picked, back)


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _windows2d(x, kernel, stride, padding, fill):
    """The ``kh * kw`` strided views of a padded ``[N, C, H, W]``: view (i, j) holds, for every output place, the
    element at offset (i, j) of its window.  Every ``s``-th element of a slice is taken by reshaping the slice
    to ``[out, s]`` and keeping column 0."""
    (kh, kw), (sh, sw), (ph, pw) = _pair(kernel), _pair(stride if stride is not None else kernel), _pair(padding)
    n, c, h, w = x.shape
    ho, wo = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    need_h, need_w = (kh - 1) + sh * ho, (kw - 1) + sw * wo          # so that every slice of s * out exists
    p = T.pad(x, ((0, 0), (0, 0), (ph, max(need_h - h - ph, 0)), (pw, max(need_w - w - pw, 0))), fill)
    views = []
    for i in range(kh):
        rows = T.shrink(p, ((0, n), (0, c), (i, i + sh * ho), (0, p.shape[3])))
        rows = T.reshape(T.shrink(T.reshape(rows, (n, c, ho, sh, p.shape[3])), ((0, n), (0, c), (0, ho), (0, 1), (0, p.shape[3]))),
                         (n, c, ho, p.shape[3]))
        for j in range(kw):
            cols = T.shrink(rows, ((0, n), (0, c), (0, ho), (j, j + sw * wo)))
            cols = T.reshape(T.shrink(T.reshape(cols, (n, c, ho, wo, sw)), ((0, n), (0, c), (0, ho), (0, wo), (0, 1))), (n, c, ho, wo))
            views.append(cols)
    return views


def max_pool2d(x, kernel, stride=None, padding=0):
    views = _windows2d(x, kernel, stride, padding, -math.inf)
    out = views[0]
    for v in views[1:]:
        out = T.maximum(out, v)
    return out


def avg_pool2d(x, kernel, stride=None, padding=0):
    """Padding counts as zeros in the average, like the op."""
    views = _windows2d(x, kernel, stride, padding, 0.0)
    out = views[0]
    for v in views[1:]:
        out = out + v
    return out * (1.0 / len(views))


def upsample_nearest(x, scale):
    n, c, h, w = x.shape
    s = int(scale)
    y = T.expand(T.reshape(x, (n, c, h, 1, w, 1)), (n, c, h, s, w, s))
    return T.reshape(y, (n, c, h * s, w * s))


def conv1d(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
    y = T.conv2d(T.unsqueeze(x, 2), T.unsqueeze(w, 2), bias, (1, int(stride)), (0, int(padding)), (1, int(dilation)), groups)
    return T.squeeze(y, 2)


def conv_transpose2d(x, w, bias=None, stride=1, padding=0, output_padding=0):
    """A transposed convolution is the convolution, with the kernel turned round and its channel axes swapped,
    of the input with ``stride - 1`` zeros between its elements and ``kernel - 1 - padding`` zeros around."""
    (sh, sw), (ph, pw), (oh, ow) = _pair(stride), _pair(padding), _pair(output_padding)
    n, c, h, wd = x.shape
    kh, kw = w.shape[2], w.shape[3]
    if ph > kh - 1 or pw > kw - 1:
        raise E.ErrUnsupported("export: transposed convolution with padding beyond the kernel")
    up = T.reshape(T.pad(T.reshape(x, (n, c, h, 1, wd, 1)), ((0, 0), (0, 0), (0, 0), (0, sh - 1), (0, 0), (0, sw - 1)), 0.0),
                   (n, c, h * sh, wd * sw))
    up = T.shrink(up, ((0, n), (0, c), (0, (h - 1) * sh + 1), (0, (wd - 1) * sw + 1)))
    up = T.pad(up, ((0, 0), (0, 0), (kh - 1 - ph, kh - 1 - ph + oh), (kw - 1 - pw, kw - 1 - pw + ow)), 0.0)
    turned = T.permute(flip(w, (2, 3)), (1, 0, 2, 3))
    return T.conv2d(up, turned, bias, 1, 0, 1, 1)


def conv_transpose1d(x, w, bias=None, stride=1, padding=0, output_padding=0):
    y = conv_transpose2d(T.unsqueeze(x, 2), T.unsqueeze(w, 2), bias, (1, int(stride)), (0, int(padding)), (0, int(output_padding)))
    return T.squeeze(y, 2)


def windows(x, axis, size, step=1):
    """Overlapping windows along ``axis`` (the window's elements become a new last axis): a row gather with the
    table of positions ``start * step + offset``."""
    n = len(x.shape)
    axis %= n
    length = x.shape[axis]
    count = (length - size) // step + 1
    pos = C.tensor((torch.arange(count)[:, None] * step + torch.arange(size)[None]).to(torch.int64), device=x.device)
    perm = [axis] + [i for i in range(n) if i != axis]
    g = T.gather_rows(T.permute(x, perm), pos)                  # [count, size, the other axes]
    # count goes back to where the axis was, size to the end
    order = list(range(2, 2 + axis)) + [0] + list(range(2 + axis, n + 1)) + [1]
    return T.permute(g, order)


def arange(n, dtype=torch.int32, device=None):
    """A range of a fixed length is a constant of the graph."""
    return C.tensor(torch.arange(n, dtype=dtype), device=device)


def detach(x):
    """A graph has no gradients to cut."""
    return x


def with_effects(x, *effects):
    return x


def greater(a, b):
    return T.less(b, a)


REWRITES = {f.__name__: f for f in (clamp, softplus, log1p, expm1, sign, floor, ceil, var, logsumexp, flip, stack, split, one_hot,
                                    argmax, gather, max_pool2d, avg_pool2d, upsample_nearest, conv1d, conv_transpose2d,
                                    conv_transpose1d, with_effects, greater, windows, arange, detach)}
