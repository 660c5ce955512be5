"""Datasets and batching (reference: data/data.go:55-167, data/stream.go:58-167).

``Tensors`` is an in-memory dataset with a seeded shuffle that changes with
``set_epoch`` (so a resumed run sees the same order); ``Stream`` reads shards
from ``Source`` objects with a prefetch thread and a shuffle buffer, in flat
memory however many rows flow through.
"""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass

import torch

from .. import tensor as T


@dataclass
class Batch:
    x: T.Tensor
    y: T.Tensor | None


class Dataset:
    def all(self):
        raise NotImplementedError

    def __iter__(self):
        return iter(self.all())

    def set_epoch(self, epoch: int) -> None:
        pass


class Tensors(Dataset):
    def __init__(self, x, y=None, batch_size: int = 32, shuffle: bool = True, drop_last: bool = False,
                 seed: int = 0, class_targets: bool = False, normalize=None):
        self.x = x.data() if isinstance(x, T.Tensor) else torch.as_tensor(x)
        self.y = None if y is None else (y.data() if isinstance(y, T.Tensor) else torch.as_tensor(y))
        if class_targets and self.y is not None:
            self.y = self.y.to(torch.int32)
        if normalize is not None:
            mean, std = normalize
            self.x = (self.x - mean) / std
        self.batch_size, self.shuffle, self.drop_last, self.seed, self.epoch = batch_size, shuffle, drop_last, seed, 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __len__(self):
        n = self.x.shape[0]
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def rows(self) -> int:
        return self.x.shape[0]

    def all(self):
        n = self.x.shape[0]
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed * 1000003 + self.epoch)
            order = torch.randperm(n, generator=g)
        else:
            order = torch.arange(n)
        for i in range(0, n, self.batch_size):
            idx = order[i: i + self.batch_size]
            if self.drop_last and idx.numel() < self.batch_size:
                break
            yield Batch(T.from_torch(self.x[idx]), None if self.y is None else T.from_torch(self.y[idx]))


def _merge_moments(a, b):
    """Chan's pairwise update of (count, mean, sum of squared deviations)."""
    (na, ma, sa), (nb, mb, sb) = a, b
    if na == 0:
        return b
    if nb == 0:
        return a
    n = na + nb
    delta = mb - ma
    return n, ma + delta * (nb / n), sa + sb + delta * delta * (na * nb / n)


def statistics(x, workers: int = 4):
    """Per-feature mean and standard deviation (data.Statistics, README "Scale").  A tensor is
    reduced directly; a ``Stream`` (or a list of ``Source`` shards) is read ONCE, its shards in
    parallel, with the moments of the chunks merged pairwise, so a data set of any size needs the
    memory of a few chunks."""
    if isinstance(x, Stream) or (isinstance(x, (list, tuple)) and x and isinstance(x[0], Source)):
        import concurrent.futures
        sources = x.sources if isinstance(x, Stream) else list(x)

        def one(src):
            acc = (0, None, None)
            for cx, _ in src.read():
                c = cx.double().reshape(cx.shape[0], -1) if cx.dim() != 2 else cx.double()
                if not c.shape[0]:
                    continue
                m = c.mean(0)
                acc = _merge_moments(acc, (c.shape[0], m, ((c - m) ** 2).sum(0)))
            return acc
        with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
            parts = list(ex.map(one, sources))
        total = (0, None, None)
        for part in parts:                      # merged in shard order: the result does not depend on timing
            total = _merge_moments(total, part)
        n, mean, ss = total
        if not n:
            raise ValueError("statistics of an empty source")
        std = (ss / max(n - 1, 1)).sqrt().clamp_min(1e-8)
        return mean.float(), std.float()
    v = x.data() if isinstance(x, T.Tensor) else torch.as_tensor(x)
    v = v.float()
    dims = tuple(d for d in range(v.dim()) if d != 1) if v.dim() > 2 else (0,)
    return v.mean(dims, keepdim=True).squeeze(0), v.std(dims, keepdim=True).squeeze(0).clamp_min(1e-8)


class Source:
    """One shard of a streamed dataset: ``read()`` yields (x_rows, y_rows) chunks as torch tensors."""

    def read(self):
        raise NotImplementedError


class FunctionSource(Source):
    def __init__(self, fn):
        self.fn = fn

    def read(self):
        yield from self.fn()


class Stream(Dataset):
    """Batches from shards with a background prefetch thread and an optional shuffle buffer."""

    def __init__(self, sources, batch_size: int = 32, prefetch: int = 4, shuffle_buffer: int = 0, seed: int = 0,
                 in_order: bool = True, drop_last: bool = False, normalize=None, class_targets: bool = False):
        """``normalize``: ``(mean, std)`` per feature, as ``statistics`` returns them, applied to every
        chunk as it is read; ``class_targets``: labels become integer class indices (data.Normalize,
        data.ClassTargets)."""
        self.sources, self.batch_size, self.prefetch = list(sources), batch_size, prefetch
        self.shuffle_buffer, self.seed, self.epoch, self.drop_last = shuffle_buffer, seed, 0, drop_last
        self.normalize, self.class_targets = normalize, class_targets

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _chunks(self):
        for s in self.sources:
            for x, y in s.read():
                if self.normalize is not None:
                    mean, std = self.normalize
                    x = (x.float() - mean) / std
                if self.class_targets and y is not None:
                    y = y.long()
                yield x, y

    def _rows(self):
        g = torch.Generator().manual_seed(self.seed * 7919 + self.epoch)
        bx, by = [], []
        held = 0
        for x, y in self._chunks():
            bx.append(x)
            by.append(y)
            held += x.shape[0]
            while held >= max(self.shuffle_buffer, self.batch_size) + self.batch_size or (not self.shuffle_buffer and held >= self.batch_size):
                X, Y = torch.cat(bx), (torch.cat(by) if by[0] is not None else None)
                if self.shuffle_buffer:
                    perm = torch.randperm(X.shape[0], generator=g)
                    X, Y = X[perm], (Y[perm] if Y is not None else None)
                yield X[: self.batch_size], (None if Y is None else Y[: self.batch_size])
                bx, by = [X[self.batch_size:]], [None if Y is None else Y[self.batch_size:]]
                held = bx[0].shape[0]
        if held:
            X, Y = torch.cat(bx), (torch.cat(by) if by[0] is not None else None)
            for i in range(0, X.shape[0], self.batch_size):
                if self.drop_last and X.shape[0] - i < self.batch_size:
                    break
                yield X[i: i + self.batch_size], (None if Y is None else Y[i: i + self.batch_size])

    def all(self):
        q: queue.Queue = queue.Queue(maxsize=max(1, self.prefetch))
        stop = object()

        def worker():
            try:
                for item in self._rows():
                    q.put(item)
                q.put(stop)
            except BaseException as exc:  # noqa: BLE001 - surfaced to the consumer
                q.put(exc)
        th = threading.Thread(target=worker, daemon=True)
        th.start()
        while True:
            item = q.get()
            if item is stop:
                break
            if isinstance(item, BaseException):
                raise item
            x, y = item
            yield Batch(T.from_torch(x), None if y is None else T.from_torch(y))
