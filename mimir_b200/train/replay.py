"""Step replay for ``fit``: forward + loss + backward + optimizer update captured once per batch
signature into a CUDA graph and replayed for every later batch of that signature.

The reference records the schedule of a training step and replays it without rebuilding or
re-planning the graph (tensor/record.go:70-184, tensor/replay.go:128-523,
internal/sched/replay.go:63-204), and submits the kernels of a schedule as one CUDA graph
whose constants are patched in place (backend/cuda/batch_linux.go:116-320).  Here both happen
at once: after two eager steps of a signature the third one is captured; from then on a step
is one copy of the batch into the graph's input buffers, one small copy of the step's
hyper-parameters (learning rate, bias corrections, gradient scale: device-side values, so any
schedule still works), and one graph launch.  No Python graph building, no planning, no
per-kernel launch cost.

What is captured is decided conservatively; anything else keeps running eagerly through the
cached schedules of ``tensor/plan.py``:

* the optimizer is on its fused flat path (``optim.FlatAdamW``): its update is one kernel
  reading device-side hyper-parameters,
* the model draws no random numbers in training mode (dropout seeds change per step) and has no
  batch-norm buffers (their lazy updates are host-driven),
* no loss scaling, micro-batching or memory budget is active for the step.

A capture that fails for any reason (a model that uploads a host tensor in ``forward``, an op that
synchronises) switches replay off for that signature and the step is redone eagerly; gradients
are cleared first, and the optimizer has not run, so nothing is applied twice.
``MIMIR_CUDA_GRAPHS=0`` disables the whole mechanism (backend/cuda/batch_linux.go:63).
"""
from __future__ import annotations

import os

import torch

from .. import tensor as T

_MAX_GRAPHS = 4
_WARM_STEPS = 2


class _Captured:
    __slots__ = ("graph", "x", "y", "loss")


class StepReplay:
    def __init__(self, model, opt, loss_fn, device):
        self.model, self.opt, self.loss_fn, self.device = model, opt, loss_fn, device
        self.enabled = (device.kind == "gpu" and os.environ.get("MIMIR_CUDA_GRAPHS", "1") != "0"
                        and self._model_is_static())
        self._seen: dict = {}        # signature -> eager steps so far, or _Captured, or False
        self.replays = 0
        self.captures = 0

    def _model_is_static(self) -> bool:
        from ..nn.module import Dropout, _BatchNorm
        for m in self.model.modules():
            if isinstance(m, _BatchNorm) or (isinstance(m, Dropout) and m.p > 0):
                return False
        return True

    def _signature(self, x: torch.Tensor, y):
        o = self.opt
        h = o.hyper
        return (tuple(x.shape), x.dtype, None if y is None else (tuple(y.shape), y.dtype), o.weight_decay,
                o.clip_norm, h.get("beta1"), h.get("beta2"), h.get("eps"), self.model.training)

    def _eager(self, x, y) -> torch.Tensor:
        """One step through the lazy layer; returns the loss as a device tensor."""
        l = self.loss_fn(self.model(T.from_torch(x)), None if y is None else T.from_torch(y))
        l.backward()
        return l._val

    def step(self, x: torch.Tensor, y):
        """Runs one optimizer step on the device batch ``(x, y)`` and returns the loss tensor, or
        returns None when this step has to go through the ordinary path."""
        opt = self.opt
        if not self.enabled or opt._flat is None or opt.grad_scale != 1.0:
            return None
        sig = self._signature(x, y)
        st = self._seen.get(sig, 0)
        if st is False:
            return None
        if isinstance(st, int):
            if st < _WARM_STEPS or sum(isinstance(v, _Captured) for v in self._seen.values()) >= _MAX_GRAPHS:
                self._seen[sig] = st + 1
                return None
            st = self._capture(sig, x, y)
            if st is None:
                return None
            return st.loss          # _capture has already replayed the new graph once for this batch
        st.x.copy_(x, non_blocking=True)
        if y is not None:
            st.y.copy_(y, non_blocking=True)
        opt.steps += 1
        opt._flat.stage(opt)
        st.graph.replay()
        opt._flat.bump()
        self.replays += 1
        return st.loss

    def _capture(self, sig, x, y):
        opt, flat = self.opt, self.opt._flat
        cap = _Captured()
        cap.x = x.clone()
        cap.y = None if y is None else y.clone()
        for p in flat.params:
            p._grad = None
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g):
                loss = self._eager(cap.x, cap.y)
                flat.gather_grads()
                flat.launch(opt)
                cap.loss = loss
        except Exception:  # noqa: BLE001 - any failure only means "this model is not capturable"
            torch.cuda.synchronize()
            for p in flat.params:
                p._grad = None
            self._seen[sig] = False
            return None
        for p in flat.params:
            p._grad = None
        cap.graph = g
        self._seen[sig] = cap
        self.captures += 1
        # capturing records the kernels without running them: run the step now
        opt.steps += 1
        flat.stage(opt)
        g.replay()
        flat.bump()
        self.replays += 1
        return cap
