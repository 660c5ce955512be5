"""Probability distributions over lazy tensors (reference: distributions/).

Normal, MultivariateNormal, Bernoulli, Categorical, Uniform, Exponential, Laplace, Gamma, Beta,
Dirichlet and Poisson, each with ``sample / log_prob / entropy / mean / variance`` (and ``rsample``
where a draw can carry gradients to the parameters), and ``kl(p, q)`` in closed form between two
distributions of one family.  Every method is a composition of the tensor layer's own ops, so it
is part of the lazy graph: gradients of any order, ``vmap``, the fusion planner and the partitioner
see its parts.  Parameters broadcast to a *batch shape*; one value has the *event shape* (``()`` for
a scalar, ``(n,)`` for a vector).  Draws are shaped ``shape + batch + event`` and are reproducible
from ``seed`` on every device (Philox streams); without a seed each call takes the next one of a
process-wide counter.  A construction error (a shape that does not broadcast, an integer parameter)
is kept and comes back as a sticky error tensor from every method, never as an exception.
"""
from __future__ import annotations

import itertools
import math

import torch

from . import tensor as T
from .tensor import errors as E
from .tensor.random import splitmix64

_core = T.core

TINY = 2.0 ** -126          # the smallest normal float32
EPS = 2.0 ** -23            # float32's spacing at 1
HALF_LOG_2PI = 0.5 * math.log(2 * math.pi)
MIN_LOGIT = -3.4028234663852886e38


class ErrNoKL(T.MimirError):
    """No closed-form KL divergence for this pair of distributions."""


_SEEDS = itertools.count(0x5EED)


def _seed(seed):
    return splitmix64(next(_SEEDS)) if seed is None else int(seed)


def sub_seed(seed: int, k: int) -> int:
    """The k-th seed derived from ``seed``: independent streams for the draws of one sample."""
    return splitmix64((int(seed) + (k + 1) * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)


def _t(x):
    if isinstance(x, T.Tensor):
        return x
    v = torch.as_tensor(x)
    if isinstance(x, int) or v.dtype == torch.float64:      # a Python number is a float32 constant
        v = v.float()
    return T.from_torch(v)


def _broadcast(shapes):
    rank = max((len(s) for s in shapes), default=0)
    out = [1] * rank
    for s in shapes:
        for i, d in enumerate(s):
            j = rank - len(s) + i
            if d == out[j] or d == 1:
                continue
            if out[j] == 1:
                out[j] = d
            else:
                raise E.ErrShape(f"shapes {[tuple(x) for x in shapes]} do not broadcast")
    return tuple(out)


def _expand(t, shape):
    if t._err is not None:
        return t
    shape = tuple(shape)
    s = tuple(t.shape)
    if s == shape:
        return t
    if len(shape) > len(s):
        t = T.reshape(t, (1,) * (len(shape) - len(s)) + s)
    return T.expand(t, shape)


def _at_least_tiny(x):
    """``x`` raised to the smallest normal float32 where it is below, with the gradient of ``x``."""
    d = T.detach(x)
    return x + (T.maximum(d, TINY) - d)


def _xlogy(x, y):
    return T.where(T.equal(x, 0.0), x * 0.0, x * T.log(y))


def _softplus(x):
    return T.relu(x) + T.log1p(T.exp(T.neg(T.abs_(x))))


def _clamp_probs(p):
    return T.minimum(T.maximum(p, EPS), 1.0 - EPS)


class Distribution:
    """Base: the batch and event shapes, the construction error, and sampling shapes."""

    reparameterized = False

    def _init(self, family, params, dims, event=()):
        """``params`` with ``dims[i]`` trailing event dimensions each; their leading dimensions broadcast
        to the batch shape."""
        self._err, self.batch_shape, self.event_shape = None, (), tuple(event)
        shapes = []
        for i, (p, d) in enumerate(zip(params, dims)):
            if p._err is not None:
                self._err = p._err
                return
            s = tuple(p.shape)
            if len(s) < d:
                self._err = E.ErrShape(f"distributions: {family} parameter {i} of shape {s} has fewer than {d} dimensions")
                return
            if not p.dtype.is_floating_point:
                self._err = E.ErrDType(f"distributions: {family} parameter {i} of {p.dtype}, want a float type")
                return
            shapes.append(s[:len(s) - d])
        try:
            self.batch_shape = _broadcast(shapes)
        except E.ErrShape as exc:
            self._err = E.ErrShape(f"distributions: {family} parameters: {exc}")

    def _failed(self):
        return _core._error_tensor(self._err) if self._err is not None else None

    def _sample_shape(self, shape=()):
        return tuple(shape) + tuple(self.batch_shape) + tuple(self.event_shape)

    def _device(self):
        return self._params()[0].device

    def _params(self):
        raise NotImplementedError

    # -- the interface
    def sample(self, shape=(), seed: int | None = None):
        """Values without gradients, shaped ``shape + batch + event``."""
        return T.detach(self.rsample(shape, seed))

    def rsample(self, shape=(), seed: int | None = None):
        return _core._error_tensor(E.ErrNotDifferentiable(f"{type(self).__name__} has no reparameterised sampler"))

    def log_prob(self, value):
        raise NotImplementedError

    def entropy(self):
        raise NotImplementedError

    def mean(self):
        raise NotImplementedError

    def variance(self):
        raise NotImplementedError

    def stddev(self):
        return T.sqrt(self.variance())


def _guard(method):
    """Returns the construction error, or the first failed operand, instead of running the method."""
    def wrapped(self, *args, **kw):
        f = self._failed()
        if f is not None:
            return f
        if args and method.__name__ in ("log_prob", "cdf", "icdf"):
            args = (_t(args[0]),) + tuple(args[1:])
        for a in args:
            if isinstance(a, T.Tensor) and a._err is not None:
                return a
        return method(self, *args, **kw)
    wrapped.__name__, wrapped.__doc__ = method.__name__, method.__doc__
    return wrapped


# ------------------------------------------------------------------ normal
class Normal(Distribution):
    """Independent normals with means ``loc`` and standard deviations ``scale`` (distributions/normal.go)."""

    reparameterized = True

    def __init__(self, loc, scale):
        self.loc, self.scale = _t(loc), _t(scale)
        self._init("normal", (self.loc, self.scale), (0, 0))

    def _params(self):
        return self.loc, self.scale

    @_guard
    def rsample(self, shape=(), seed=None):
        """``loc + scale * e`` for standard normal ``e``."""
        e = T.randn(self._sample_shape(shape), _seed(seed), device=self._device())
        return self.loc + self.scale * e

    @_guard
    def log_prob(self, value):
        z = (value - self.loc) / self.scale
        return z * z * -0.5 - T.log(self.scale) - HALF_LOG_2PI

    @_guard
    def entropy(self):
        return _expand(T.log(self.scale) + (0.5 + HALF_LOG_2PI), self.batch_shape)

    @_guard
    def mean(self):
        return _expand(self.loc, self.batch_shape)

    @_guard
    def variance(self):
        return _expand(self.scale * self.scale, self.batch_shape)

    @_guard
    def cdf(self, value):
        return (T.erf((value - self.loc) / (self.scale * math.sqrt(2.0))) + 1.0) * 0.5

    @_guard
    def icdf(self, p):
        """The value whose CDF is ``p``."""
        return T.erfinv(p * 2.0 - 1.0) * math.sqrt(2.0) * self.scale + self.loc


def _tril(m):
    n, k = m.shape[-2], m.shape[-1]
    return m * T.tensor(torch.tril(torch.ones(n, k)).to(m.dtype), device=m.device)


def _diagonal(m):
    n = m.shape[-1]
    return T.sum_(m * T.tensor(torch.eye(n).to(m.dtype), device=m.device), -1)


class MultivariateNormal(Distribution):
    """Normal vectors with mean ``loc [..., n]`` and covariance ``L L^T`` for the lower-triangular
    ``scale_tril [..., n, n]`` (its upper triangle is ignored), or from a symmetric positive definite
    ``covariance`` by its Cholesky factor (distributions/normal.go:105-225)."""

    reparameterized = True

    def __init__(self, loc, covariance=None, scale_tril=None):
        self.loc = _t(loc)
        if (covariance is None) == (scale_tril is None):
            self._err, self.batch_shape, self.event_shape = E.ErrShape("distributions: multivariate normal wants one of covariance and scale_tril"), (), ()
            return
        L = T.cholesky(_t(covariance)) if covariance is not None else _t(scale_tril)
        self._init("multivariate normal", (self.loc, L), (1, 2))
        self.scale_tril = L
        if self._err is None:
            n = self.loc.shape[-1]
            if L.shape[-1] != n or L.shape[-2] != n:
                self._err = E.ErrShape(f"distributions: multivariate normal of mean {tuple(self.loc.shape)} and scale {tuple(L.shape)}")
            self.event_shape = (n,)
            self.scale_tril = _tril(L) if self._err is None else L

    def _params(self):
        return self.loc, self.scale_tril

    def _half_log_det(self):
        return T.sum_(T.log(_diagonal(self.scale_tril)), -1)

    def _mahalanobis(self, x):
        """``|L^-1 x|^2`` for vectors ``x`` whose leading dimensions broadcast against ``L``'s."""
        L, col = self.scale_tril, T.unsqueeze(x, -1)
        lead = _broadcast([tuple(L.shape[:-2]), tuple(col.shape[:-2])])
        y = T.triangular_solve(_expand(L, lead + tuple(L.shape[-2:])), _expand(col, lead + tuple(col.shape[-2:])), False)
        return T.sum_(T.sum_(y * y, -1), -1)

    @_guard
    def rsample(self, shape=(), seed=None):
        """``loc + L e`` for a vector ``e`` of standard normals."""
        s = self._sample_shape(shape)
        e = T.randn(s, _seed(seed), device=self._device())
        L = _expand(self.scale_tril, s + s[-1:])
        return T.squeeze(T.matmul(L, T.unsqueeze(e, -1)), -1) + self.loc

    @_guard
    def log_prob(self, value):
        n = self.event_shape[0]
        return self._mahalanobis(value - self.loc) * -0.5 - self._half_log_det() - n * HALF_LOG_2PI

    @_guard
    def entropy(self):
        n = self.event_shape[0]
        return _expand(self._half_log_det() + n * (0.5 + HALF_LOG_2PI), self.batch_shape)

    @_guard
    def mean(self):
        return _expand(self.loc, self._sample_shape())

    @_guard
    def variance(self):
        """The diagonal of the covariance: the squared norms of the rows of ``L``."""
        return _expand(T.sum_(self.scale_tril * self.scale_tril, -1), self._sample_shape())

    def covariance(self):
        f = self._failed()
        return f if f is not None else T.matmul(self.scale_tril, T.transpose(self.scale_tril, -1, -2))


# ------------------------------------------------------------------ uniform, exponential, laplace
class Uniform(Distribution):
    """Uniform on ``[low, high)`` (distributions/continuous.go:25-82)."""

    reparameterized = True

    def __init__(self, low, high):
        self.low, self.high = _t(low), _t(high)
        self._init("uniform", (self.low, self.high), (0, 0))

    def _params(self):
        return self.low, self.high

    @_guard
    def rsample(self, shape=(), seed=None):
        u = T.rand(self._sample_shape(shape), _seed(seed), device=self._device())
        return u * (self.high - self.low) + self.low

    @_guard
    def log_prob(self, value):
        """``-log(high - low)`` inside the support and -Inf outside."""
        inside = T.logical_and(T.logical_not(T.less(value, self.low)), T.less(value, self.high))
        dens = T.neg(T.log(self.high - self.low))
        return T.where(inside, dens + value * 0.0, value * 0.0 + dens * 0.0 - math.inf)

    @_guard
    def entropy(self):
        return _expand(T.log(self.high - self.low), self.batch_shape)

    @_guard
    def mean(self):
        return _expand((self.low + self.high) * 0.5, self.batch_shape)

    @_guard
    def variance(self):
        w = self.high - self.low
        return _expand(w * w * (1.0 / 12), self.batch_shape)


class Exponential(Distribution):
    """Exponential with rate ``rate`` (distributions/continuous.go:84-139)."""

    reparameterized = True

    def __init__(self, rate):
        self.rate = _t(rate)
        self._init("exponential", (self.rate,), (0,))

    def _params(self):
        return (self.rate,)

    @_guard
    def rsample(self, shape=(), seed=None):
        """``-log(1 - u) / rate``."""
        u = T.rand(self._sample_shape(shape), _seed(seed), device=self._device())
        return T.neg(T.log1p(T.neg(u))) / self.rate

    @_guard
    def log_prob(self, value):
        return T.log(self.rate) - self.rate * value

    @_guard
    def entropy(self):
        return _expand(1.0 - T.log(self.rate), self.batch_shape)

    @_guard
    def mean(self):
        return _expand(T.recip(self.rate), self.batch_shape)

    @_guard
    def variance(self):
        return _expand(T.recip(self.rate * self.rate), self.batch_shape)


class Laplace(Distribution):
    """Laplace with location ``loc`` and scale ``scale`` (distributions/continuous.go:141-200)."""

    reparameterized = True

    def __init__(self, loc, scale):
        self.loc, self.scale = _t(loc), _t(scale)
        self._init("laplace", (self.loc, self.scale), (0, 0))

    def _params(self):
        return self.loc, self.scale

    @_guard
    def rsample(self, shape=(), seed=None):
        """``loc - scale * sign(u) * log(1 - |u|)`` for ``u`` uniform on the open interval (-1, 1)."""
        u = T.rand(self._sample_shape(shape), _seed(seed), device=self._device()) * (2.0 - 2.0 * EPS) + (EPS - 1.0)
        return self.loc - self.scale * T.sign(u) * T.log1p(T.neg(T.abs_(u)))

    @_guard
    def log_prob(self, value):
        return T.neg(T.log(self.scale * 2.0)) - T.abs_(value - self.loc) / self.scale

    @_guard
    def entropy(self):
        return _expand(T.log(self.scale * 2.0) + 1.0, self.batch_shape)

    @_guard
    def mean(self):
        return _expand(self.loc, self.batch_shape)

    @_guard
    def variance(self):
        return _expand(self.scale * self.scale * 2.0, self.batch_shape)


# ------------------------------------------------------------------ gamma family
def _log_beta(a, b):
    return T.lgamma(a) + T.lgamma(b) - T.lgamma(a + b)


class Gamma(Distribution):
    """Gamma with shape ``concentration`` and ``rate`` (distributions/gamma.go:26-88)."""

    reparameterized = True

    def __init__(self, concentration, rate):
        self.concentration, self.rate = _t(concentration), _t(rate)
        self._init("gamma", (self.concentration, self.rate), (0, 0))

    def _params(self):
        return self.concentration, self.rate

    @_guard
    def rsample(self, shape=(), seed=None):
        """Gamma(concentration, 1) draws (implicit gradients in the concentration) divided by the rate;
        at least the smallest normal float32."""
        a = _expand(self.concentration, self._sample_shape(shape))
        return _at_least_tiny(T.rand_gamma(a, _seed(seed)) / self.rate)

    @_guard
    def log_prob(self, value):
        a, b = self.concentration, self.rate
        return _xlogy(a, b) + _xlogy(a - 1.0, value) - b * value - T.lgamma(a)

    @_guard
    def entropy(self):
        a = self.concentration
        return _expand(a - T.log(self.rate) + T.lgamma(a) + (1.0 - a) * T.digamma(a), self.batch_shape)

    @_guard
    def mean(self):
        return _expand(self.concentration / self.rate, self.batch_shape)

    @_guard
    def variance(self):
        return _expand(self.concentration / (self.rate * self.rate), self.batch_shape)


class Dirichlet(Distribution):
    """Dirichlet over the probability vectors of K categories, concentrations along the last axis
    (distributions/gamma.go:90-178)."""

    reparameterized = True

    def __init__(self, concentration):
        self.concentration = _t(concentration)
        self._init("dirichlet", (self.concentration,), (1,))
        if self._err is None:
            k = self.concentration.shape[-1]
            self.event_shape = (k,)
            if k == 0:
                self._err = E.ErrShape("distributions: dirichlet of no categories")

    def _params(self):
        return (self.concentration,)

    @_guard
    def rsample(self, shape=(), seed=None):
        """Gamma draws of the concentrations divided by their sum."""
        g = T.rand_gamma(_expand(self.concentration, self._sample_shape(shape)), _seed(seed))
        return _at_least_tiny(g / T.unsqueeze(T.sum_(g, -1), -1))

    @_guard
    def log_prob(self, value):
        a = self.concentration
        return T.sum_(_xlogy(a - 1.0, value), -1) + T.lgamma(T.sum_(a, -1)) - T.sum_(T.lgamma(a), -1)

    @_guard
    def entropy(self):
        a = self.concentration
        k, a0 = float(a.shape[-1]), T.sum_(a, -1)
        return T.sum_(T.lgamma(a), -1) - T.lgamma(a0) - (k - a0) * T.digamma(a0) - T.sum_((a - 1.0) * T.digamma(a), -1)

    @_guard
    def mean(self):
        a = self.concentration
        return _expand(a / T.unsqueeze(T.sum_(a, -1), -1), self._sample_shape())

    @_guard
    def variance(self):
        a = self.concentration
        a0 = T.unsqueeze(T.sum_(a, -1), -1)
        return _expand(a * (a0 - a) / (a0 * a0 * (a0 + 1.0)), self._sample_shape())


class Beta(Distribution):
    """Beta on [0, 1] with density ``x^(a-1) (1-x)^(b-1) / B(a, b)`` for ``concentration1`` a and
    ``concentration0`` b (distributions/gamma.go:180-250)."""

    reparameterized = True

    def __init__(self, concentration1, concentration0):
        self.concentration1, self.concentration0 = _t(concentration1), _t(concentration0)
        self._init("beta", (self.concentration1, self.concentration0), (0, 0))

    def _params(self):
        return self.concentration1, self.concentration0

    @_guard
    def rsample(self, shape=(), seed=None):
        """``X / (X + Y)`` for gamma draws X, Y of the two concentrations."""
        s, seed = self._sample_shape(shape), _seed(seed)
        x = T.rand_gamma(_expand(self.concentration1, s), sub_seed(seed, 0))
        y = T.rand_gamma(_expand(self.concentration0, s), sub_seed(seed, 1))
        return _at_least_tiny(x / (x + y))

    @_guard
    def log_prob(self, value):
        a, b = self.concentration1, self.concentration0
        return _xlogy(a - 1.0, value) + _xlogy(b - 1.0, 1.0 - value) - _log_beta(a, b)

    @_guard
    def entropy(self):
        a, b = self.concentration1, self.concentration0
        t = a + b
        return _expand(_log_beta(a, b) - (a - 1.0) * T.digamma(a) - (b - 1.0) * T.digamma(b) + (t - 2.0) * T.digamma(t),
                       self.batch_shape)

    @_guard
    def mean(self):
        a, b = self.concentration1, self.concentration0
        return _expand(a / (a + b), self.batch_shape)

    @_guard
    def variance(self):
        a, b = self.concentration1, self.concentration0
        t = a + b
        return _expand(a * b / (t * t * (t + 1.0)), self.batch_shape)


# ------------------------------------------------------------------ discrete
class Bernoulli(Distribution):
    """0 / 1 with probability ``probs`` of 1, or from its log-odds ``logits``; one is computed from the
    other.  Log-odds made from probabilities keep them within float32's spacing of 0 and 1
    (distributions/discrete.go:27-89)."""

    def __init__(self, probs=None, logits=None):
        if (probs is None) == (logits is None):
            self._err, self.batch_shape, self.event_shape = E.ErrShape("distributions: bernoulli wants one of probs and logits"), (), ()
            return
        if probs is not None:
            self.probs = _t(probs)
            self._init("bernoulli", (self.probs,), (0,))
            if self._err is None:
                p = _clamp_probs(self.probs)
                self.logits = T.log(p) - T.log1p(T.neg(p))
        else:
            self.logits = _t(logits)
            self._init("bernoulli", (self.logits,), (0,))
            if self._err is None:
                self.probs = T.sigmoid(self.logits)

    def _params(self):
        return (self.probs,)

    @_guard
    def sample(self, shape=(), seed=None):
        u = T.rand(self._sample_shape(shape), _seed(seed), device=self._device())
        return T.cast(T.less(u, T.detach(self.probs)), T.float32)

    @_guard
    def log_prob(self, value):
        """Minus the binary cross-entropy, from the log-odds."""
        return self.logits * value - _softplus(self.logits)

    @_guard
    def entropy(self):
        return _expand(_softplus(self.logits) - self.logits * self.probs, self.batch_shape)

    @_guard
    def mean(self):
        return _expand(self.probs, self.batch_shape)

    @_guard
    def variance(self):
        return _expand(self.probs * (1.0 - self.probs), self.batch_shape)


class Categorical(Distribution):
    """Categories 0..K-1 with probabilities ``probs [..., K]`` (normalised along the last axis: they need
    not sum to 1) or unnormalised log-probabilities ``logits`` (distributions/discrete.go:91-185)."""

    def __init__(self, probs=None, logits=None):
        if (probs is None) == (logits is None):
            self._err, self.batch_shape, self.event_shape = E.ErrShape("distributions: categorical wants one of probs and logits"), (), ()
            return
        raw = _t(probs if probs is not None else logits)
        self._init("categorical", (raw,), (1,))
        if self._err is None and raw.shape[-1] == 0:
            self._err = E.ErrShape("distributions: categorical of no categories")
        if self._err is not None:
            return
        if probs is not None:
            self.probs = raw / T.unsqueeze(T.sum_(raw, -1), -1)
            self.logits = T.log(_clamp_probs(self.probs))
        else:
            self.logits = T.log_softmax(raw, -1)
            self.probs = T.exp(self.logits)

    def _params(self):
        return (self.logits,)

    @property
    def categories(self) -> int:
        return self.logits.shape[-1]

    @_guard
    def sample(self, shape=(), seed=None):
        """The Gumbel-max trick: the position of the largest log-probability plus Gumbel noise."""
        u = T.rand(self._sample_shape(shape) + (self.categories,), _seed(seed), device=self._device())
        gumbel = T.neg(T.log(T.neg(T.log(u))))
        return T.argmax(T.detach(self.logits) + gumbel, -1)

    @_guard
    def log_prob(self, value):
        """The log-probabilities of the categories ``value`` (integers or floats), which broadcast against
        the batch shape."""
        if value.dtype.is_floating_point or value.dtype == torch.bool:
            value = T.cast(value, T.int32)
        try:
            shape = _broadcast([tuple(value.shape), self.batch_shape])
        except E.ErrShape as exc:
            return _core._error_tensor(E.ErrShape(f"distributions: categorical value of shape {tuple(value.shape)}: {exc}"))
        logits = _expand(self.logits, shape + (self.categories,))
        return T.squeeze(T.gather(logits, -1, T.unsqueeze(_expand(value, shape), -1)), -1)

    @_guard
    def entropy(self):
        """``-sum p log p``; a zero probability counts 0."""
        return T.neg(T.sum_(self.probs * T.maximum(self.logits, MIN_LOGIT), -1))

    @_guard
    def mean(self):
        """NaN: categories have no order."""
        return T.full(self.batch_shape, math.nan, device=self._device())

    def variance(self):
        return self.mean()


POISSON_TERMS, POISSON_SMALL = 96, 24.0


class Poisson(Distribution):
    """Counts with mean ``rate``; values are float counts (distributions/discrete.go:187-263)."""

    def __init__(self, rate):
        self.rate = _t(rate)
        self._init("poisson", (self.rate,), (0,))

    def _params(self):
        return (self.rate,)

    @_guard
    def sample(self, shape=(), seed=None):
        return T.rand_poisson(_expand(T.detach(self.rate), self._sample_shape(shape)), _seed(seed))

    @_guard
    def log_prob(self, value):
        """``k log(rate) - rate - log k!``."""
        return _xlogy(value, self.rate) - self.rate - T.lgamma(value + 1.0)

    @_guard
    def entropy(self):
        """``-sum p(k) log p(k)`` over the first 96 counts for rates below 24, and the asymptotic series
        ``0.5 log(2 pi e r) - 1/(12 r) - 1/(24 r^2) - 19/(360 r^3)`` above; what either leaves out is
        below float32's precision.  Each branch sees a rate in its own range, so the other's NaN or
        infinity never reaches the gradient."""
        rate = _expand(self.rate, self.batch_shape)
        small = T.less(rate, POISSON_SMALL)
        lo = T.unsqueeze(T.where(small, rate, rate * 0.0 + 1.0), -1)
        k = T.reshape(T.arange(POISSON_TERMS, dtype=T.float32, device=rate.device), (1,) * len(self.batch_shape) + (POISSON_TERMS,))
        lp = _xlogy(k, lo) - lo - T.lgamma(k + 1.0)
        summed = T.neg(T.sum_(T.exp(lp) * lp, -1))
        hi = T.where(small, rate * 0.0 + POISSON_SMALL, rate)
        r = T.recip(hi)
        series = T.log(hi * (2 * math.pi * math.e)) * 0.5 - r * (1.0 / 12 + r * (1.0 / 24 + r * (19.0 / 360)))
        return T.where(small, summed, series)

    @_guard
    def mean(self):
        return _expand(self.rate, self.batch_shape)

    def variance(self):
        return self.mean()


# ------------------------------------------------------------------ KL
def _kl_normal(p, q):
    r = p.scale / q.scale
    r = r * r
    t = (p.loc - q.loc) / q.scale
    return (r + t * t - 1.0 - T.log(r)) * 0.5


def _kl_mvn(p, q):
    n = p.event_shape[0]
    if n != q.event_shape[0]:
        return _core._error_tensor(E.ErrShape(f"distributions: KL of multivariate normals of {n} and {q.event_shape[0]} dimensions"))
    lead = _broadcast([tuple(q.scale_tril.shape[:-2]), tuple(p.scale_tril.shape[:-2])])
    m = T.triangular_solve(_expand(q.scale_tril, lead + (n, n)), _expand(p.scale_tril, lead + (n, n)), False)
    frob = T.sum_(T.sum_(m * m, -1), -1)
    return q._half_log_det() - p._half_log_det() + (frob + q._mahalanobis(q.loc - p.loc) - float(n)) * 0.5


def _kl_bernoulli(p, q):
    t1 = p.probs * (_softplus(T.neg(q.logits)) - _softplus(T.neg(p.logits)))
    t2 = (1.0 - p.probs) * (_softplus(q.logits) - _softplus(p.logits))
    return t1 + t2


def _kl_categorical(p, q):
    if p.categories != q.categories:
        return _core._error_tensor(E.ErrShape(f"distributions: KL of categoricals of {p.categories} and {q.categories} categories"))
    t = p.probs * (p.logits - q.logits)
    t = T.where(T.equal(q.probs, 0.0), t * 0.0 + math.inf, t)
    return T.sum_(T.where(T.equal(p.probs, 0.0), t * 0.0, t), -1)


def _kl_uniform(p, q):
    r = T.log((q.high - q.low) / (p.high - p.low))
    outside = T.logical_or(T.less(p.low, q.low), T.less(q.high, p.high))
    return T.where(outside, r * 0.0 + math.inf, r)


def _kl_exponential(p, q):
    r = q.rate / p.rate
    return r - T.log(r) - 1.0


def _kl_laplace(p, q):
    r = p.scale / q.scale
    d = T.abs_(p.loc - q.loc)
    return T.neg(T.log(r)) + d / q.scale + r * T.exp(T.neg(d / p.scale)) - 1.0


def _kl_gamma(p, q):
    ap, bp, aq, bq = p.concentration, p.rate, q.concentration, q.rate
    return aq * T.log(bp / bq) + T.lgamma(aq) - T.lgamma(ap) + (ap - aq) * T.digamma(ap) + (bq - bp) * (ap / bp)


def _kl_beta(p, q):
    ap, bp, aq, bq = p.concentration1, p.concentration0, q.concentration1, q.concentration0
    return (_log_beta(aq, bq) - _log_beta(ap, bp) + (ap - aq) * T.digamma(ap) + (bp - bq) * T.digamma(bp)
            + (aq - ap + bq - bp) * T.digamma(ap + bp))


def _kl_dirichlet(p, q):
    if p.event_shape != q.event_shape:
        return _core._error_tensor(E.ErrShape(f"distributions: KL of dirichlets of {p.event_shape[0]} and {q.event_shape[0]} categories"))
    ap, aq = p.concentration, q.concentration
    sp = T.sum_(ap, -1)
    return (T.lgamma(sp) - T.lgamma(T.sum_(aq, -1)) - T.sum_(T.lgamma(ap) - T.lgamma(aq), -1)
            + T.sum_((ap - aq) * (T.digamma(ap) - T.unsqueeze(T.digamma(sp), -1)), -1))


def _kl_poisson(p, q):
    return _xlogy(p.rate, p.rate) - _xlogy(p.rate, q.rate) - p.rate + q.rate


_KL = {Normal: _kl_normal, MultivariateNormal: _kl_mvn, Bernoulli: _kl_bernoulli, Categorical: _kl_categorical,
       Uniform: _kl_uniform, Exponential: _kl_exponential, Laplace: _kl_laplace, Gamma: _kl_gamma, Beta: _kl_beta,
       Dirichlet: _kl_dirichlet, Poisson: _kl_poisson}


def kl(p: Distribution, q: Distribution):
    """KL(p || q) of each pair of the two batches (which broadcast), in closed form between two
    distributions of one family; other pairs give a sticky ``ErrNoKL``.  Where p puts mass that q does
    not, the divergence is +Inf (distributions/kl.go:31-97)."""
    f = _KL.get(type(p))
    if f is None or type(q) is not type(p):
        return _core._error_tensor(ErrNoKL(f"distributions: KL of {type(p).__name__} and {type(q).__name__}"))
    for d in (p, q):
        if d._err is not None:
            return _core._error_tensor(d._err)
    return f(p, q)
