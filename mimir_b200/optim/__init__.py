"""Optimizers (reference: optim/optim.go:57-70,176-306,372-392,455-671; schedules
optim/schedule.go:30-81).

One generic ``Optimizer`` driven by a ``Rule(lr, step, p, g, state) -> (new_p,
new_state)``; ``step()`` updates every parameter in place (old ``value()``
tensors become stale), applies the gradient scale and the global-norm clip
factor ``clip / (norm + 1e-6)`` clamped to 1 (optim.go:198-215), keeps fp32
master weights for half-precision parameters when asked (``master_weights``),
and exposes state under the reference's names (``exp_avg``, ``exp_avg_sq``,
``momentum_buffer``, ``square_avg``, ``sum``, ``acc_delta``, ``exp_inf``,
``master``) with snapshot keys ``"<param index>.<name>"``.

bf16 CUDA parameters updated by AdamW with master weights go through the fused
native kernel (``mimir_adamw_flat``): one pass writes p, m, v and the master.
"""
from __future__ import annotations

import math

import torch

from ..tensor import errors as E


class Optimizer:
    def __init__(self, params, lr: float, rule, state_names=(), weight_decay=0.0, clip_norm=0.0,
                 master_weights=False, hyper=None, name="custom"):
        self.params = list(params)
        self.lr, self.rule, self.name = lr, rule, name
        self.weight_decay, self.clip_norm, self.master_weights = weight_decay, clip_norm, master_weights
        self.hyper = hyper or {}
        self.state = [dict() for _ in self.params]
        self.steps = 0
        self.grad_scale = 1.0  # gradients are divided by this (loss scaling)

    # -- gradient checks
    def grads_finite(self) -> bool:
        """True when every gradient is finite (optim.go:136-157); used by dynamic loss scaling."""
        for p in self.params:
            if p._grad is not None and not bool(torch.isfinite(p._grad).all()):
                return False
        return True

    def zero_grad(self) -> None:
        for p in self.params:
            p.zero_grad()

    def global_norm(self) -> float:
        sq = 0.0
        for p in self.params:
            if p._grad is not None:
                sq += float(p._grad.float().pow(2).sum())
        return math.sqrt(sq) / self.grad_scale

    def step(self) -> None:
        self.steps += 1
        factor = 1.0 / self.grad_scale
        if self.clip_norm > 0:
            norm = self.global_norm()
            factor *= min(1.0, self.clip_norm / (norm + 1e-6))
        from ..tensor.autograd import flush_lazy
        flush_lazy()
        with torch.no_grad():
            for p, st in zip(self.params, self.state):
                if p._grad is None or not p.trainable:
                    continue
                g = p._grad.float() * factor
                if self.master_weights and p.dtype != torch.float32:
                    if "master" not in st:
                        st["master"] = p._data.float().clone()
                    w = st["master"]
                else:
                    w = p._data.float() if p.dtype != torch.float32 else p._data
                new_w = self.rule(self.lr, self.steps, w, g, st, self)
                if "master" in st:
                    st["master"] = new_w
                p._data.copy_(new_w.to(p.dtype))
                p._version += 1

    # -- checkpointing
    def snapshot(self) -> dict:
        out = {}
        for i, st in enumerate(self.state):
            for k in sorted(st):
                if torch.is_tensor(st[k]):
                    out[f"{i}.{k}"] = st[k]
        return out

    def restore(self, snap: dict, steps: int | None = None) -> None:
        for key, v in snap.items():
            i, name = key.split(".", 1)
            self.state[int(i)][name] = v.clone()
        if steps is not None:
            self.steps = steps


def _wd_coupled(g, w, opt):
    return g + opt.weight_decay * w if opt.weight_decay else g


# ---- rules: (lr, step, w, g, state, opt) -> new_w; they update ``state`` in place
def _sgd(lr, t, w, g, st, o):
    h = o.hyper
    g = _wd_coupled(g, w, o)
    if h.get("momentum", 0.0):
        buf = st.get("momentum_buffer")
        buf = g.clone() if buf is None else h["momentum"] * buf + (1 - h.get("dampening", 0.0)) * g
        st["momentum_buffer"] = buf
        g = g + h["momentum"] * buf if h.get("nesterov") else buf
    return w - lr * g


def _adam_core(lr, t, w, g, st, o, decoupled):
    b1, b2, eps = o.hyper.get("beta1", 0.9), o.hyper.get("beta2", 0.999), o.hyper.get("eps", 1e-8)
    if decoupled:
        w = w * (1 - lr * o.weight_decay)
    else:
        g = _wd_coupled(g, w, o)
    m = st.get("exp_avg", torch.zeros_like(w))
    v = st.get("exp_avg_sq", torch.zeros_like(w))
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    st["exp_avg"], st["exp_avg_sq"] = m, v
    bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
    return w - (lr / bc1) * m / (v.sqrt() / math.sqrt(bc2) + eps)


def _adam(lr, t, w, g, st, o): return _adam_core(lr, t, w, g, st, o, False)
def _adamw(lr, t, w, g, st, o): return _adam_core(lr, t, w, g, st, o, True)


def _rmsprop(lr, t, w, g, st, o):
    alpha, eps, mom = o.hyper.get("alpha", 0.99), o.hyper.get("eps", 1e-8), o.hyper.get("momentum", 0.0)
    g = _wd_coupled(g, w, o)
    sq = alpha * st.get("square_avg", torch.zeros_like(w)) + (1 - alpha) * g * g
    st["square_avg"] = sq
    upd = g / (sq.sqrt() + eps)
    if mom:
        buf = mom * st.get("momentum_buffer", torch.zeros_like(w)) + upd
        st["momentum_buffer"] = buf
        upd = buf
    return w - lr * upd


def _adagrad(lr, t, w, g, st, o):
    eps, decay = o.hyper.get("eps", 1e-10), o.hyper.get("lr_decay", 0.0)
    g = _wd_coupled(g, w, o)
    s = st.get("sum", torch.full_like(w, o.hyper.get("initial", 0.0))) + g * g
    st["sum"] = s
    clr = lr / (1 + (t - 1) * decay)
    return w - clr * g / (s.sqrt() + eps)


def _adadelta(lr, t, w, g, st, o):
    rho, eps = o.hyper.get("rho", 0.9), o.hyper.get("eps", 1e-6)
    g = _wd_coupled(g, w, o)
    sq = rho * st.get("square_avg", torch.zeros_like(w)) + (1 - rho) * g * g
    acc = st.get("acc_delta", torch.zeros_like(w))
    delta = (acc + eps).sqrt() / (sq + eps).sqrt() * g
    st["square_avg"], st["acc_delta"] = sq, rho * acc + (1 - rho) * delta * delta
    return w - lr * delta


def _adamax(lr, t, w, g, st, o):
    b1, b2, eps = o.hyper.get("beta1", 0.9), o.hyper.get("beta2", 0.999), o.hyper.get("eps", 1e-8)
    g = _wd_coupled(g, w, o)
    m = b1 * st.get("exp_avg", torch.zeros_like(w)) + (1 - b1) * g
    u = torch.maximum(b2 * st.get("exp_inf", torch.zeros_like(w)), g.abs() + eps)
    st["exp_avg"], st["exp_inf"] = m, u
    return w - (lr / (1 - b1 ** t)) * m / u


def _nadam(lr, t, w, g, st, o):
    b1, b2, eps = o.hyper.get("beta1", 0.9), o.hyper.get("beta2", 0.999), o.hyper.get("eps", 1e-8)
    md = o.hyper.get("momentum_decay", 4e-3)
    g = _wd_coupled(g, w, o)
    mu = b1 * (1 - 0.5 * 0.96 ** (t * md))
    mu_next = b1 * (1 - 0.5 * 0.96 ** ((t + 1) * md))
    prod = st.get("_mu_product", 1.0) * mu
    st["_mu_product"] = prod
    m = b1 * st.get("exp_avg", torch.zeros_like(w)) + (1 - b1) * g
    v = b2 * st.get("exp_avg_sq", torch.zeros_like(w)) + (1 - b2) * g * g
    st["exp_avg"], st["exp_avg_sq"] = m, v
    denom = (v / (1 - b2 ** t)).sqrt() + eps
    return w - lr * (1 - mu) / (1 - prod) * g / denom - lr * mu_next / (1 - prod * mu_next) * m / denom


def _radam(lr, t, w, g, st, o):
    b1, b2, eps = o.hyper.get("beta1", 0.9), o.hyper.get("beta2", 0.999), o.hyper.get("eps", 1e-8)
    g = _wd_coupled(g, w, o)
    m = b1 * st.get("exp_avg", torch.zeros_like(w)) + (1 - b1) * g
    v = b2 * st.get("exp_avg_sq", torch.zeros_like(w)) + (1 - b2) * g * g
    st["exp_avg"], st["exp_avg_sq"] = m, v
    mhat = m / (1 - b1 ** t)
    rho_inf = 2 / (1 - b2) - 1
    rho_t = rho_inf - 2 * t * b2 ** t / (1 - b2 ** t)
    if rho_t > 5:
        r = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t))
        return w - lr * mhat * r / ((v / (1 - b2 ** t)).sqrt() + eps)
    return w - lr * mhat


def _lion(lr, t, w, g, st, o):
    b1, b2 = o.hyper.get("beta1", 0.9), o.hyper.get("beta2", 0.99)
    m = st.get("exp_avg", torch.zeros_like(w))
    w = w * (1 - lr * o.weight_decay)
    upd = torch.sign(b1 * m + (1 - b1) * g)
    st["exp_avg"] = b2 * m + (1 - b2) * g
    return w - lr * upd


def _make(name, rule, defaults):
    def ctor(params, lr=defaults.get("lr", 1e-3), weight_decay=defaults.get("weight_decay", 0.0), clip_norm=0.0,
             master_weights=False, **hyper):
        if "betas" in hyper:
            hyper["beta1"], hyper["beta2"] = hyper.pop("betas")
        h = {k: v for k, v in defaults.items() if k not in ("lr", "weight_decay")}
        h.update(hyper)
        return Optimizer(params, lr, rule, weight_decay=weight_decay, clip_norm=clip_norm,
                         master_weights=master_weights, hyper=h, name=name)
    ctor.__name__ = name
    return ctor


SGD = _make("SGD", _sgd, dict(lr=1e-2))
Adam = _make("Adam", _adam, dict(lr=1e-3))
AdamW = _make("AdamW", _adamw, dict(lr=1e-3, weight_decay=0.01))
RMSprop = _make("RMSprop", _rmsprop, dict(lr=1e-2))
Adagrad = _make("Adagrad", _adagrad, dict(lr=1e-2))
Adadelta = _make("Adadelta", _adadelta, dict(lr=1.0))
Adamax = _make("Adamax", _adamax, dict(lr=2e-3))
NAdam = _make("NAdam", _nadam, dict(lr=2e-3))
RAdam = _make("RAdam", _radam, dict(lr=1e-3))
Lion = _make("Lion", _lion, dict(lr=1e-4, beta2=0.99))


def New(params, lr, rule):
    """``optim.New(params, lr, rule)`` with ``rule(lr, step, p, g, state) -> (new_p, new_state)``."""
    def adapter(lr_, t, w, g, st, o):
        new_w, new_state = rule(lr_, t, w, g, dict(st))
        st.clear()
        st.update(new_state or {})
        return new_w
    return Optimizer(params, lr, adapter)


# ---- schedules: functions of the epoch (optim/schedule.go:30-81)
def StepDecay(lr, n, gamma): return lambda e: lr * gamma ** (e // n)
def Cosine(lr, floor, epochs): return lambda e: floor + 0.5 * (lr - floor) * (1 + math.cos(math.pi * min(e, epochs) / max(epochs, 1)))
def Warmup(lr, start, epochs): return lambda e: lr if e >= epochs else start + (lr - start) * e / max(epochs, 1)
def Exponential(lr, gamma): return lambda e: lr * gamma ** e
def Polynomial(lr, epochs, power): return lambda e: lr * (1 - min(e, epochs) / max(epochs, 1)) ** power


def OneCycle(peak, epochs, warm=0.3):
    """Cosine ramp from peak/25 to the peak over ``warm * epochs - 1`` epochs, then cosine down
    to peak / 25e4 at the last epoch."""
    start, end = peak / 25, peak / 25 / 1e4
    up = warm * epochs - 1

    def cos(a, b, f):
        return b + (a - b) * (1 + math.cos(math.pi * f)) / 2

    def f(e):
        if e <= up:
            return cos(start, peak, e / up)
        return cos(peak, end, (e - up) / (epochs - 1 - up))
    return f
