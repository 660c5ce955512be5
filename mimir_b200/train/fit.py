"""``fit``: the training loop (reference: train/train.go:265-724, checkpoint.go:40-119).

Options mirror the reference: ``loss``, ``epochs``, ``eval`` (dataset + metrics),
``checkpoint`` (directory, atomic ``checkpoint.mim`` after every epoch, exact
resume), ``schedule`` (lr per epoch), ``early_stopping``, ``micro_batch``
(gradient accumulation equal to the full batch), ``memory_budget`` (split a batch
until the estimate fits), ``loss_scale`` / ``dynamic_loss_scale`` (start 65536,
halve on a non-finite gradient and skip the step, double after 2000 good steps,
floor 1: train.go:194-210,536-560), ``precise_batch_norm``, ``on_epoch`` /
``on_batch`` callbacks and ``progress``.  A step that fails leaves no gradients
behind (train.go:504-508).  On a GPU, steps whose structure repeats are captured
into a CUDA graph and replayed (``train/replay.py``).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field

import torch

from .. import tensor as T
from ..io import mim


@dataclass
class EpochReport:
    epoch: int
    loss: float
    lr: float
    steps: int
    duration: float
    metrics: dict = field(default_factory=dict)


@dataclass
class BatchReport:
    loss: float
    skipped: bool
    loss_scale: float


def evaluate(model, ds, loss_fn=None, metrics=()):
    """Mean loss and metric values over ``ds`` in eval mode (train.Evaluate)."""
    was = model.training
    model.eval()
    total, rows = 0.0, 0
    for m in metrics:
        m.reset()
    for b in ds.all():
        out = model(b.x)
        n = b.x.shape[0]
        if loss_fn is not None and b.y is not None:
            total += loss_fn(out, b.y).item() * n
        rows += n
        if b.y is not None:
            for m in metrics:
                m.update(out.data().float().cpu(), b.y.data().cpu())
    model.train(was)
    return (total / max(rows, 1)), {m.name: m.value() for m in metrics}


def save_checkpoint(directory, model, opt, epoch: int, steps: int, extras=None) -> str:
    """Writes ``<directory>/checkpoint.mim`` atomically: ``model.<path>`` tensors,
    ``optim.<i>.<state>`` tensors and a Training section (counters, lr)."""
    os.makedirs(directory, exist_ok=True)
    tensors = {f"model.{n}": p._data for n, p in model.named_params()}
    for k, v in opt.snapshot().items():
        tensors[f"optim.{k}"] = v
    training = {"epochs": int(epoch), "steps": int(steps), "lr": float(opt.lr), "optimizer": opt.name}
    for k, v in (extras or {}).items():
        training[f"extra.{k}"] = v
    path = os.path.join(directory, "checkpoint.mim")
    mim.write_tensors(path, tensors, training=training)
    return path


def load_checkpoint(directory, model, opt):
    """Restores model and optimizer; returns the Training section, or None when absent."""
    path = os.path.join(directory, "checkpoint.mim")
    if not os.path.exists(path):
        return None
    with mim.open(path) as m:
        tr = m.training() or {}
        sd = {n[len("model."):]: m.tensor(n).clone() for n in m.names() if n.startswith("model.")}
        model.load_state_dict(sd)
        snap = {n[len("optim."):]: m.tensor(n).clone() for n in m.names() if n.startswith("optim.")}
        opt.restore(snap, steps=int(tr.get("steps", 0)))
        if "lr" in tr:
            opt.lr = float(tr["lr"])
    return tr


def _split(batch, parts):
    n = batch.x.shape[0]
    size = (n + parts - 1) // parts
    out = []
    for i in range(0, n, size):
        x = T.from_torch(batch.x.data()[i: i + size])
        y = None if batch.y is None else T.from_torch(batch.y.data()[i: i + size])
        out.append((x, y, x.shape[0] / n))
    return out


def fit(model, opt, ds, loss=None, epochs: int = 1, eval=None, metrics=(), checkpoint=None, schedule=None,
        early_stopping: int = 0, micro_batch: int = 0, memory_budget: int | None = None, loss_scale: float = 1.0,
        dynamic_loss_scale: bool = False, precise_batch_norm=None, on_epoch=None, on_batch=None, progress=None,
        device=None, data_parallel=None, sharded=None):
    """Trains ``model`` on ``ds``; returns the list of ``EpochReport``."""
    if loss is None:
        raise ValueError("fit needs a loss function")
    if checkpoint and sharded is not None:
        raise ValueError("checkpoint and sharded training are mutually exclusive (train.go:279-280)")
    if data_parallel is not None:
        from ..parallel.replicas import fit_data_parallel
        return fit_data_parallel(model, opt, ds, loss, epochs, data_parallel, schedule=schedule, on_epoch=on_epoch,
                                 progress=progress)
    shard_mesh = None
    if sharded is not None:
        # the partitioner: parameters get layouts on the mesh, every batch is placed P("data"), and the
        # graphs built from them are analysed and lowered per rank (train/sharded.go:37-56)
        from ..parallel import spmd
        shard_mesh, rule = sharded
        if getattr(model, "_mesh", None) is not shard_mesh:
            spmd.shard_params(model, shard_mesh, rule)
    device = device or T.default_device()
    start_epoch, steps = 0, 0
    if checkpoint:
        tr = load_checkpoint(checkpoint, model, opt)
        if tr:
            start_epoch, steps = int(tr.get("epochs", 0)), int(tr.get("steps", 0))
    scale = 65536.0 if dynamic_loss_scale else float(loss_scale)
    good_steps = 0
    reports, best, since_best = [], float("inf"), 0
    if memory_budget is not None:
        T.set_memory_budget(device, memory_budget)
    from .replay import StepReplay
    replay = StepReplay(model, opt, loss, device)     # CUDA-graph replay of whole steps where it applies
    try:
        for epoch in range(start_epoch, epochs):
            t0 = time.perf_counter()
            model.train()
            if schedule is not None:
                opt.lr = float(schedule(epoch))
            ds.set_epoch(epoch)
            total, rows = 0.0, 0
            for batch in ds.all():
                if shard_mesh is not None:
                    from ..parallel import spmd
                    from ..parallel.mesh import P
                    spec = P("data") if "data" in shard_mesh.axes and shard_mesh.axis_size("data") > 1 else None
                    x = spmd.place(batch.x.to(device), shard_mesh, spec)
                    y = None if batch.y is None else spmd.place(batch.y.to(device), shard_mesh, spec)
                else:
                    x = batch.x.to(device)
                    y = None if batch.y is None else batch.y.to(device)
                parts = 1
                if micro_batch and x.shape[0] > micro_batch:
                    parts = (x.shape[0] + micro_batch - 1) // micro_batch
                skipped, value = False, 0.0
                if replay.enabled and shard_mesh is None and parts == 1 and memory_budget is None \
                        and not dynamic_loss_scale and scale == 1.0:
                    opt.grad_scale = 1.0
                    lt = replay.step(x.data(), None if y is None else y.data())
                    if lt is not None:
                        value = float(lt.item())
                        steps += 1
                        good_steps += 1
                        total += value * x.shape[0]
                        rows += x.shape[0]
                        if on_batch:
                            on_batch(BatchReport(value, False, scale))
                        continue
                while True:
                    try:
                        value = 0.0
                        for xs, ys, share in ([(x, y, 1.0)] if shard_mesh is not None else _split(Batch_(x, y), parts)):
                            l = loss(model(xs), ys) * (share * scale)
                            l.backward()
                            value += l.item() / scale
                        break
                    except T.ErrMemoryBudget:
                        opt.zero_grad()
                        if parts >= x.shape[0]:
                            raise
                        parts *= 2
                    except Exception:
                        opt.zero_grad()  # a failed step leaves no gradients behind
                        raise
                opt.grad_scale = scale
                if (dynamic_loss_scale or loss_scale != 1.0) and not opt.grads_finite():
                    skipped = True
                    if dynamic_loss_scale:
                        scale, good_steps = max(1.0, scale / 2), 0
                else:
                    opt.step()
                    steps += 1
                    good_steps += 1
                    if dynamic_loss_scale and good_steps >= 2000:
                        scale, good_steps = scale * 2, 0
                opt.zero_grad()
                total += value * x.shape[0]
                rows += x.shape[0]
                if on_batch:
                    on_batch(BatchReport(value, skipped, scale))
            if precise_batch_norm is not None:
                _recompute_batch_norm(model, precise_batch_norm, device)
            rep = EpochReport(epoch + 1, total / max(rows, 1), opt.lr, steps, time.perf_counter() - t0)
            if eval is not None:
                ev_loss, ev_metrics = evaluate(model, eval, loss, metrics)
                rep.metrics = dict(ev_metrics, eval_loss=ev_loss)
            reports.append(rep)
            if checkpoint:
                save_checkpoint(checkpoint, model, opt, epoch + 1, steps)
            if on_epoch:
                on_epoch(rep)
            if progress is not None:
                extra = " ".join(f"{k}={v:.4f}" for k, v in rep.metrics.items())
                progress.write(f"epoch {rep.epoch}/{epochs} loss={rep.loss:.4f} lr={rep.lr:.3g} "
                               f"steps={rep.steps} {rep.duration:.1f}s {extra}\n")
            if early_stopping:
                watched = rep.metrics.get("eval_loss", rep.loss)
                if watched < best - 1e-12:
                    best, since_best = watched, 0
                else:
                    since_best += 1
                    if since_best >= early_stopping:
                        break
    finally:
        if memory_budget is not None:
            T.set_memory_budget(device, None)
    return reports


class Batch_:
    def __init__(self, x, y):
        self.x, self.y = x, y


def _recompute_batch_norm(model, ds, device):
    """PreciseBatchNorm: re-estimates running statistics over ``ds`` with cumulative averaging."""
    bns = model.batch_norms()
    if not bns:
        return
    old = [(b.momentum) for b in bns]
    for b in bns:
        b.running_mean._data.zero_()
        b.running_var._data.fill_(1.0)
    model.train()
    for i, batch in enumerate(ds.all()):
        for b in bns:
            b.momentum = 1.0 / (i + 1)
        model(batch.x.to(device)).realize()
    for b, m in zip(bns, old):
        b.momentum = m
