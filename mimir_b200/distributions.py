"""Probability distributions over lazy tensors (reference: distributions/): Normal,
MultivariateNormal, Bernoulli, Categorical, Uniform, Exponential, Laplace, Gamma, Beta,
Dirichlet, Poisson, each with ``sample / rsample / log_prob / entropy / mean / variance``,
and ``kl(p, q)`` (``ErrNoKL`` when no closed form is registered)."""
from __future__ import annotations

import torch
import torch.distributions as D

from . import tensor as T


# shape inference runs the constructors on meta tensors, which cannot be value-checked
D.Distribution.set_default_validate_args(False)


class ErrNoKL(T.MimirError):
    pass


def _v(x):
    return x.data() if isinstance(x, T.Tensor) else torch.as_tensor(x, dtype=torch.float32)


class Distribution:
    _cls = None
    _reparam = True

    def __init__(self, *params, **kw):
        self._params = params
        self._kw = kw

    def _dist(self, vals=None):
        vals = [_v(p) for p in self._params] if vals is None else vals
        return self._cls(*vals, **self._kw)

    def _lazy(self, name, fn, *extra):
        ps = [p if isinstance(p, T.Tensor) else T.from_torch(_v(p)) for p in self._params]
        n = len(ps)
        return T.core._node(lambda *a: fn(self._cls(*a[:n], **self._kw), *a[n:]), (*ps, *extra), {}, name)

    def sample(self, shape=(), seed: int | None = None):
        g = None
        if seed is not None:
            torch.manual_seed(seed)
        with torch.no_grad():
            return T.from_torch(self._dist().sample(tuple(shape)))

    def rsample(self, shape=(), seed: int | None = None):
        """Reparameterised sample: gradients flow to the parameters."""
        if not self._reparam:
            raise T.ErrNotDifferentiable(f"{type(self).__name__} has no reparameterised sampler")
        if seed is not None:
            torch.manual_seed(seed)
        return self._lazy("rsample", lambda d: d.rsample(tuple(shape)))

    def log_prob(self, x):
        x = x if isinstance(x, T.Tensor) else T.from_torch(_v(x))
        return self._lazy("log_prob", lambda d, v: d.log_prob(v), x)

    def entropy(self):
        return self._lazy("entropy", lambda d: d.entropy())

    def mean(self):
        return self._lazy("mean", lambda d: d.mean)

    def variance(self):
        return self._lazy("variance", lambda d: d.variance)


def _make(name, cls, reparam=True):
    return type(name, (Distribution,), {"_cls": cls, "_reparam": reparam})


Normal = _make("Normal", D.Normal)
Uniform = _make("Uniform", D.Uniform)
Exponential = _make("Exponential", D.Exponential)
Laplace = _make("Laplace", D.Laplace)
Gamma = _make("Gamma", D.Gamma)
Beta = _make("Beta", D.Beta)
Dirichlet = _make("Dirichlet", D.Dirichlet)
Poisson = _make("Poisson", D.Poisson, False)


class Bernoulli(Distribution):
    _cls, _reparam = D.Bernoulli, False

    def __init__(self, probs=None, logits=None):
        super().__init__(probs if probs is not None else logits)
        self._cls = (lambda p: D.Bernoulli(probs=p)) if probs is not None else (lambda l: D.Bernoulli(logits=l))


class Categorical(Distribution):
    _reparam = False

    def __init__(self, probs=None, logits=None):
        super().__init__(probs if probs is not None else logits)
        self._cls = (lambda p: D.Categorical(probs=p)) if probs is not None else (lambda l: D.Categorical(logits=l))


class MultivariateNormal(Distribution):
    def __init__(self, loc, covariance=None, scale_tril=None):
        super().__init__(loc, covariance if covariance is not None else scale_tril)
        self._cls = (lambda m, c: D.MultivariateNormal(m, covariance_matrix=c)) if covariance is not None \
            else (lambda m, l: D.MultivariateNormal(m, scale_tril=l))


def kl(p: Distribution, q: Distribution):
    """KL(p || q) in closed form."""
    try:
        with torch.no_grad():
            D.kl_divergence(p._dist(), q._dist())
    except NotImplementedError as exc:
        raise ErrNoKL(f"no closed-form KL between {type(p).__name__} and {type(q).__name__}") from exc
    pp = [x if isinstance(x, T.Tensor) else T.from_torch(_v(x)) for x in p._params]
    qp = [x if isinstance(x, T.Tensor) else T.from_torch(_v(x)) for x in q._params]
    n = len(pp)
    return T.core._node(lambda *a: D.kl_divergence(p._cls(*a[:n], **p._kw), q._cls(*a[n:], **q._kw)), (*pp, *qp), {}, "kl")
