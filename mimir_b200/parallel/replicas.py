"""Replicated data-parallel training, one process per device (reference: nn/replicate.go:39-227
module copies and frozen inference views; train/parallel.go:78-286 ``Parallel``: broadcast of
changed parameters, batch split with share-weighted losses, gradient reduction, optimizer step
on the root or on every replica).

The reference keeps all replicas in one process and drives them from goroutines; here every
rank of the job holds one replica, so "replicate" is a broadcast of the root's parameters and
the reduction is the bucketed ``Group.all_reduce_grads`` / ``reduce_grads``.  The fused
peer-memory kernel path for the GPT-2 engine lives in ``parallel/dp.py``; this class is the
general path for any ``nn.Module`` and the baseline that kernel is measured against.
"""
from __future__ import annotations

import copy
import time

import torch

from .. import tensor as T
from ..tensor.group import Group


def replicate(module, device=None):
    """Deep copy of a module (parameters, buffers, configuration) on ``device``."""
    m = copy.deepcopy(module)
    return m.to(device) if device is not None else m


def inference(module):
    """A frozen view: shares the parameter storage of ``module``, never trains, eval mode."""
    m = copy.copy(module)
    m.__dict__ = dict(module.__dict__)
    view = copy.deepcopy(module)
    for (_, p), (_, q) in zip(module.named_params(), view.named_params()):
        q._data = p._data          # same storage: later updates of the original are visible
        q.freeze()
    return view.eval()


class Parallel:
    """``mode="all_reduce"``: every rank reduces to the same gradients and steps its own optimizer
    (bit-identical replicas); ``mode="reduce"``: gradients go to rank 0, which steps and broadcasts
    the parameters that changed."""

    def __init__(self, model, group: Group, mode: str = "all_reduce"):
        if mode not in ("all_reduce", "reduce"):
            raise ValueError(f"unknown mode {mode!r}")
        self.model, self.group, self.mode = model, group, mode
        self.params = model.parameters()
        group.broadcast_params([p for _, p in model.named_params()], root=0)

    def shard(self, x: torch.Tensor):
        """This rank's rows of a global batch and their share of it (axis 0, contiguous blocks)."""
        n, w, r = x.shape[0], self.group.size, self.group.rank
        per = (n + w - 1) // w
        lo, hi = min(n, r * per), min(n, (r + 1) * per)
        return lo, hi, (hi - lo) / max(n, 1)

    def backward(self, x, y, loss_fn) -> float:
        """Forward + backward of this rank's share; returns the global batch loss (same on every rank)."""
        xd = x.data() if isinstance(x, T.Tensor) else x
        yd = None if y is None else (y.data() if isinstance(y, T.Tensor) else y)
        lo, hi, share = self.shard(xd)
        value = 0.0
        if hi > lo:
            l = loss_fn(self.model(T.from_torch(xd[lo:hi])), None if yd is None else T.from_torch(yd[lo:hi])) * share
            l.backward()
            value = float(l.item())
        for p in self.params:              # a rank without rows still takes part in the reduction
            if p._grad is None:
                p._grad = torch.zeros_like(p._data)
        if self.mode == "all_reduce":
            self.group.all_reduce_grads(self.params, op="sum")
        else:
            self.group.reduce_grads(self.params, root=0, op="sum")
        total = self.group.all_reduce(T.tensor([value]), "sum")
        return float(total.data()[0])

    def step(self, opt) -> None:
        if self.mode == "all_reduce" or self.group.rank == 0:
            opt.step()
        if self.mode == "reduce":
            self.group.broadcast_params(self.params, root=0)
        opt.zero_grad()


def fit_data_parallel(model, opt, ds, loss, epochs, group, schedule=None, on_epoch=None, progress=None, mode="all_reduce"):
    """``train.fit`` over the ranks of ``group``: every rank iterates the same batches (same seed and
    epoch) and works on its block of each."""
    from ..train.fit import EpochReport
    from .dp import FusedFlatDataParallel, fused_flat_eligible
    if mode == "all_reduce" and fused_flat_eligible(opt, group):
        return _fit_fused(model, opt, ds, loss, epochs, group, schedule, on_epoch, progress)
    par = Parallel(model, group, mode)
    reports, steps = [], 0
    for epoch in range(epochs):
        t0 = time.perf_counter()
        model.train()
        if schedule is not None:
            opt.lr = float(schedule(epoch))
        ds.set_epoch(epoch)
        total, rows = 0.0, 0
        for batch in ds.all():
            value = par.backward(batch.x, batch.y, loss)
            par.step(opt)
            steps += 1
            total += value * batch.x.shape[0]
            rows += batch.x.shape[0]
        rep = EpochReport(epoch + 1, total / max(rows, 1), opt.lr, steps, time.perf_counter() - t0)
        reports.append(rep)
        if on_epoch:
            on_epoch(rep)
        if progress is not None and group.rank == 0:
            progress.write(f"epoch {rep.epoch}/{epochs} loss={rep.loss:.4f} lr={rep.lr:.3g} steps={rep.steps} {rep.duration:.1f}s\n")
    return reports


def _fit_fused(model, opt, ds, loss, epochs, group, schedule, on_epoch, progress):
    """``fit_data_parallel`` on the fused peer-memory kernel (``parallel/dp.py``): every rank runs its
    share of each batch through the lazy layer (native kernels), then one kernel per step reduces the
    gradients, applies AdamW to the owned slice and distributes the new parameters."""
    from ..train.fit import EpochReport
    from .dp import FusedFlatDataParallel
    fused = FusedFlatDataParallel(opt, group)
    helper = Parallel.__new__(Parallel)
    helper.group = group
    reports, steps = [], 0
    try:
        for epoch in range(epochs):
            t0 = time.perf_counter()
            model.train()
            if schedule is not None:
                opt.lr = float(schedule(epoch))
            ds.set_epoch(epoch)
            total, rows = 0.0, 0
            for batch in ds.all():
                xd = batch.x.data().to(fused.flat.param.device)
                yd = None if batch.y is None else batch.y.data().to(xd.device)
                lo, hi, share = helper.shard(xd)
                value = torch.zeros(1, device=xd.device)
                fused.begin()
                if hi > lo:
                    l = loss(model(T.from_torch(xd[lo:hi])), None if yd is None else T.from_torch(yd[lo:hi])) * share
                    l.backward()
                    value = l._val.reshape(1).float()
                fused.step()
                dist_value = group.all_reduce(T.from_torch(value), "sum")
                v = float(dist_value.data()[0])
                steps += 1
                total += v * xd.shape[0]
                rows += xd.shape[0]
            rep = EpochReport(epoch + 1, total / max(rows, 1), opt.lr, steps, time.perf_counter() - t0)
            reports.append(rep)
            if on_epoch:
                on_epoch(rep)
            if progress is not None and group.rank == 0:
                progress.write(f"epoch {rep.epoch}/{epochs} loss={rep.loss:.4f} lr={rep.lr:.3g} steps={rep.steps} {rep.duration:.1f}s\n")
    finally:
        fused.close()
    return reports
