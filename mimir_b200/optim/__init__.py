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
native kernel (``mimir_adamw_flat``): at the first step the optimizer moves the
parameters, their gradients, the fp32 masters and both moments into flat buffers
(``FlatAdamW``), after which a step is ONE launch that writes p, m, v and the master
(plus one sum-of-squares launch when a global-norm clip is set; the clip factor is
computed on the device, so the step never waits for the host).  Every other rule runs
as per-parameter PyTorch updates.
"""
from __future__ import annotations

import math

import torch

from ..tensor import errors as E


class FlatAdamW:
    """Flat storage of an AdamW-with-master-weights optimizer over bf16 CUDA parameters.

    ``param`` / ``grad`` are bf16, ``master`` / ``exp_avg`` / ``exp_avg_sq`` fp32; every parameter
    owns a slice that starts on a multiple of 8 elements (the kernels move 16 bytes at a time) and
    ``Param._data`` / ``Param._grad_buf`` are re-pointed at views of the slices, so the model, the
    checkpoint code and ``backward`` keep working on the same memory.  The learning rate, the bias
    corrections and the gradient scale reach the kernel through a 4-float device array, so a step
    captured in a CUDA graph replays with new values (internal/sched/key.go:28-44 keeps constants
    out of a schedule's key for the same reason)."""

    def __init__(self, opt, alloc=None, multiple: int = 8):
        """``alloc(numel, dtype)`` supplies the parameter and gradient buffers (peer-visible memory for
        data parallelism); ``multiple`` pads the total length (8 x ranks there)."""
        params = [p for p in opt.params if p.trainable]
        dev = params[0]._data.device
        offs, n = [], 0
        for p in params:
            offs.append(n)
            n += (p.numel() + 7) // 8 * 8
        n = (n + multiple - 1) // multiple * multiple
        self.n, self.params, self.offsets = n, params, offs
        alloc = alloc or (lambda numel, dtype: torch.zeros(numel, dtype=dtype, device=dev))
        self.param = alloc(n, torch.bfloat16)
        self.grad = alloc(n, torch.bfloat16)
        self.master = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.hyper = torch.zeros(4, dtype=torch.float32, device=dev)
        from ..ops._util import PinnedRing
        self._ring = PinnedRing(4)
        index = {id(p): i for i, p in enumerate(opt.params)}
        for p, o in zip(params, offs):
            k, st = p.numel(), opt.state[index[id(p)]]
            view = lambda buf: buf.narrow(0, o, k).view(p.shape)  # noqa: E731
            pv, mv = view(self.param), view(self.master)
            pv.copy_(p._data)
            mv.copy_(st["master"] if "master" in st else p._data.float())
            for name, buf in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                if name in st:
                    view(buf).copy_(st[name])
                st[name] = view(buf)
            st["master"] = mv
            gv = view(self.grad)
            if p._grad is not None:
                gv.copy_(p._grad)
                p._grad = gv
            p._data, p._grad_buf = pv, gv
            p._version += 1

    def step(self, opt) -> None:
        self.stage(opt)
        self.gather_grads()
        self.launch(opt)
        self.bump()

    def stage(self, opt) -> None:
        """Host side of a step: the learning rate, the bias corrections of step ``opt.steps`` and the
        gradient scale go to the device array the kernel reads (an asynchronous copy from pinned memory)."""
        h = opt.hyper
        b1, b2 = h.get("beta1", 0.9), h.get("beta2", 0.999)
        self._ring.stage((opt.lr, 1.0 - b1 ** opt.steps, math.sqrt(1.0 - b2 ** opt.steps), 1.0 / opt.grad_scale),
                         self.hyper)

    def gather_grads(self) -> None:
        """Makes the flat gradient buffer current: a parameter the loss did not reach gets zeros, a
        gradient that was produced outside its slice is copied in."""
        for p in self.params:
            if p._grad is None:
                p._grad_buf.zero_()
            elif p._grad is not p._grad_buf:
                p._grad_buf.copy_(p._grad)

    def bump(self) -> None:
        for p in self.params:
            p._version += 1

    def launch(self, opt) -> None:
        """The device work of one step (what a captured training step contains)."""
        from ..ops import kernels as K
        h = opt.hyper
        clip = float(opt.clip_norm or 0.0)
        if clip > 0:
            self.gnorm_sq.zero_()
            K.sumsq(self.grad, self.gnorm_sq)
        K.adamw_flat(self.master, self.param, self.grad, self.exp_avg, self.exp_avg_sq, decay_n=self.n, lr=0.0,
                     beta1=h.get("beta1", 0.9), beta2=h.get("beta2", 0.999), eps=h.get("eps", 1e-8),
                     wd=opt.weight_decay, step=1, gnorm_sq=self.gnorm_sq if clip > 0 else None, clip=clip,
                     hyper=self.hyper)


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
        self._flat = None      # FlatAdamW once the fused path has taken over

    def _flat_eligible(self) -> bool:
        from ..tensor import core as C
        if self.rule is not _adamw or not self.master_weights or not C._NATIVE:
            return False
        ps = [p for p in self.params if p.trainable]
        if not ps or type(self).step is not Optimizer.step:
            return False
        dev = ps[0]._data.device
        return dev.type == "cuda" and all(p._data.dtype == torch.bfloat16 and p._data.device == dev
                                          and getattr(p, "_gather", None) is None and p._sharding is None for p in ps)

    # -- gradient checks
    def grads_finite(self) -> bool:
        """True when every gradient is finite (optim.go:136-157); used by dynamic loss scaling."""
        gs = [p._grad for p in self.params if p._grad is not None]
        if not gs:
            return True
        if gs[0].is_cuda:       # one reduction and one host read for all gradients
            return bool(torch.stack([torch.isfinite(g).all() for g in gs]).all())
        return all(bool(torch.isfinite(g).all()) for g in gs)

    def zero_grad(self) -> None:
        for p in self.params:
            p.zero_grad()

    def global_norm(self) -> float:
        gs = [p._grad for p in self.params if p._grad is not None]
        if not gs:
            return 0.0
        sq = torch.stack([g.float().pow(2).sum() for g in gs]).sum()      # one host read in all
        return math.sqrt(float(sq)) / self.grad_scale

    def step(self) -> None:
        self.steps += 1
        from ..tensor.autograd import flush_lazy
        if self._flat is None and self._flat_eligible():
            flush_lazy()
            self._flat = FlatAdamW(self)
        if self._flat is not None:
            flush_lazy()
            self._flat.step(self)
            return
        factor = 1.0 / self.grad_scale
        if self.clip_norm > 0:
            norm = self.global_norm()
            factor *= min(1.0, self.clip_norm / (norm + 1e-6))
        from ..tensor.autograd import flush_lazy
        flush_lazy()
        if self.rule in (_adam, _adamw) and self._foreach_adam(factor):
            return
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

    def _foreach_adam(self, factor: float) -> bool:
        """Adam / AdamW over all float32 / float64 parameters at once, in place: the same update as
        the rule (optim.go:455-520), as seven multi-tensor operations instead of a dozen temporaries
        per parameter.  False when some parameter needs the general path (half precision, master
        weights, mixed devices)."""
        ws, gs, ms, vs, ps = [], [], [], [], []
        for p, st in zip(self.params, self.state):
            if p._grad is None or not p.trainable:
                continue
            w, g = p._data, p._grad
            if w.dtype not in (torch.float32, torch.float64) or g.dtype != w.dtype or g.device != w.device or "master" in st:
                return False
            ws.append(w)
            gs.append(g)
            ps.append((p, st))
        if not ws:
            return True
        for (p, st), w in zip(ps, ws):
            if "exp_avg" not in st:
                st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(w), torch.zeros_like(w)
            ms.append(st["exp_avg"])
            vs.append(st["exp_avg_sq"])
        h, t, lr = self.hyper, self.steps, self.lr
        b1, b2, eps = h.get("beta1", 0.9), h.get("beta2", 0.999), h.get("eps", 1e-8)
        with torch.no_grad():
            if factor != 1.0:
                gs = torch._foreach_mul(gs, factor)
            if self.rule is _adamw:
                if self.weight_decay:
                    torch._foreach_mul_(ws, 1 - lr * self.weight_decay)
            elif self.weight_decay:
                gs = torch._foreach_add(gs, ws, alpha=self.weight_decay)
            torch._foreach_mul_(ms, b1)
            torch._foreach_add_(ms, gs, alpha=1 - b1)
            torch._foreach_mul_(vs, b2)
            torch._foreach_addcmul_(vs, gs, gs, value=1 - b2)
            den = torch._foreach_sqrt(vs)
            torch._foreach_div_(den, math.sqrt(1 - b2 ** t))
            torch._foreach_add_(den, eps)
            torch._foreach_addcdiv_(ws, ms, den, value=-(lr / (1 - b1 ** t)))
        for p, _ in ps:
            p._version += 1
        return True

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
            st = self.state[int(i)]
            if self._flat is not None and name in st and torch.is_tensor(st[name]):
                st[name].copy_(v)       # views of the flat buffers: written in place
                if name == "master":
                    self.params[int(i)]._data.copy_(v)
            else:
                st[name] = v.clone().to(self.params[int(i)]._data.device)
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
    # the running product of the momentum factors is a function of the step number alone
    # (optim/optim.go:604-609), so nothing beyond the tensors has to be checkpointed
    cached = getattr(o, "_nadam_prod", None)      # (step, product): a cache, recomputable from t
    if cached is not None and cached[0] == t:
        prod = cached[1]
    else:
        start, prod = (cached[0], cached[1]) if cached is not None and cached[0] < t else (0, 1.0)
        for i in range(start + 1, t + 1):
            prod *= b1 * (1 - 0.5 * 0.96 ** (i * md))
        o._nadam_prod = (t, prod)
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
