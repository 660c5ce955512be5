"""Distributions: sample moments against the closed-form mean and variance, category frequencies,
gradients through reparameterised draws against the derivative of the mean, sample shapes and seeds,
values outside a support, infinite divergences, and errors that stay sticky."""
import math

import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200 import distributions as D
from mimir_b200.tensor import errors as E
from mimir_b200.tensor.autograd import Param, backward

N = 40000


def vec(*v):
    return T.tensor(torch.tensor(v, dtype=torch.float32))


FAMILIES = {
    "normal": lambda: D.Normal(vec(-1, 2), vec(0.5, 3)),
    "multivariate normal": lambda: D.MultivariateNormal(vec(1, -2, 0.5), scale_tril=T.tensor(torch.tensor(
        [[1, 0, 0], [0.5, 2, 0], [-0.3, 0.2, 0.7]]))),
    "bernoulli": lambda: D.Bernoulli(probs=vec(0.1, 0.5, 0.97)),
    "uniform": lambda: D.Uniform(vec(-1, 5), vec(3, 5.5)),
    "exponential": lambda: D.Exponential(vec(0.5, 4)),
    "laplace": lambda: D.Laplace(vec(1, -2), vec(0.5, 2)),
    "gamma": lambda: D.Gamma(vec(0.3, 1, 7.5), vec(2, 1, 0.5)),
    "beta": lambda: D.Beta(vec(0.5, 2, 9), vec(0.5, 5, 1)),
    "dirichlet": lambda: D.Dirichlet(vec(0.4, 1, 3, 6)),
    "poisson": lambda: D.Poisson(vec(0.2, 4, 15, 120)),
}


@pytest.mark.parametrize("name", sorted(FAMILIES))
def test_samples_have_the_moments_the_distribution_reports(name):
    d = FAMILIES[name]()
    x = d.sample((N,), seed=11).data().double()
    assert tuple(x.shape) == (N,) + d.batch_shape + d.event_shape
    mean, var = d.mean().data().double(), d.variance().data().double()
    sd = var.sqrt()
    # the mean of N draws lies within six standard errors; the variance within 10 %
    assert bool(((x.mean(0) - mean).abs() <= 6 * sd / math.sqrt(N) + 1e-6).all()), (x.mean(0), mean)
    assert bool(((x.var(0) - var).abs() <= 0.1 * var + 1e-6).all()), (x.var(0), var)


def test_categorical_samples_follow_the_probabilities():
    p = [0.05, 0.6, 0.0, 0.35]
    d = D.Categorical(probs=vec(1, 12, 0, 7))
    x = d.sample((N,), seed=3).data()
    assert not x.dtype.is_floating_point and tuple(x.shape) == (N,)
    freq = torch.bincount(x.long(), minlength=4).double() / N
    for k in range(4):
        assert abs(float(freq[k]) - p[k]) <= 6 * math.sqrt(p[k] * (1 - p[k]) / N) + 1e-12, (k, float(freq[k]))
    assert torch.isnan(d.mean().data()).all()


RSAMPLE = [
    ("normal", [0.3, 1.5], lambda p: (lambda x: T.mean(x * x))(D.Normal(p[0], p[1]).rsample((N,), seed=1)),
     lambda p: [2 * p[0], 2 * p[1]]),                                                  # E x^2 = mu^2 + sigma^2
    ("gamma", [2.5, 1.5], lambda p: T.mean(D.Gamma(p[0], p[1]).rsample((N,), seed=2)),
     lambda p: [1 / p[1], -p[0] / p[1] ** 2]),
    ("gamma below 1", [0.4, 1.0], lambda p: T.mean(D.Gamma(p[0], p[1]).rsample((N,), seed=3)),
     lambda p: [1 / p[1], -p[0] / p[1] ** 2]),
    ("beta", [2.0, 3.0], lambda p: T.mean(D.Beta(p[0], p[1]).rsample((N,), seed=4)),
     lambda p: [p[1] / (p[0] + p[1]) ** 2, -p[0] / (p[0] + p[1]) ** 2]),
    ("dirichlet", [1.5, 0.7, 2.0],
     lambda p: T.mean(T.shrink(D.Dirichlet(T.stack(list(p), 0)).rsample((N,), seed=5), ((0, N), (0, 1)))),
     lambda p: [(sum(p) - p[0]) / sum(p) ** 2, -p[0] / sum(p) ** 2, -p[0] / sum(p) ** 2]),
    ("exponential", [2.0], lambda p: T.mean(D.Exponential(p[0]).rsample((N,), seed=6)), lambda p: [-1 / p[0] ** 2]),
    ("laplace", [0.5, 2.0], lambda p: (lambda x: T.mean(x * x))(D.Laplace(p[0], p[1]).rsample((N,), seed=7)),
     lambda p: [2 * p[0], 4 * p[1]]),                                                  # mu^2 + 2 b^2
    ("uniform", [-1.0, 3.0], lambda p: T.mean(D.Uniform(p[0], p[1]).rsample((N,), seed=8)), lambda p: [0.5, 0.5]),
    ("multivariate normal", [0.5, 2.0],
     lambda p: (lambda x: T.mean(T.sum_(x * x, -1)))(D.MultivariateNormal(
         vec(0, 0), scale_tril=T.reshape(T.stack([p[0], p[0] * 0.0, p[1], p[0] * 0.0 + 1.0], 0), (2, 2))).rsample((N,), seed=9)),
     lambda p: [2 * p[0], 2 * p[1]]),                                                  # E |x|^2 = p0^2 + p1^2 + 1
]


@pytest.mark.parametrize("name,params,draw,want", RSAMPLE, ids=[c[0] for c in RSAMPLE])
def test_gradients_flow_through_reparameterised_draws(name, params, draw, want):
    ps = [Param(torch.tensor(v)) for v in params]
    backward(draw([p.value() for p in ps]))
    for i, w in enumerate(want(params)):
        g = float(ps[i].grad().data())
        assert abs(g - w) <= 0.05 * max(1.0, abs(w)), (name, i, g, w)


def test_sample_shapes_seeds_and_gradients():
    loc = Param(torch.zeros(3, 1))
    d = D.Normal(loc.value(), vec(1, 2))
    assert d.batch_shape == (3, 2) and d.event_shape == ()
    x = d.sample((4, 2), seed=5)
    assert tuple(x.shape) == (4, 2, 3, 2)
    assert torch.equal(d.sample((4, 2), seed=5).data(), x.data())
    assert not torch.equal(d.sample((4, 2), seed=6).data(), x.data())
    assert not torch.equal(d.sample((4, 2)).data(), d.sample((4, 2)).data())        # unseeded calls take fresh seeds
    with pytest.raises(E.ErrNoGrad):
        backward(T.sum_(d.sample((2,), seed=1)))
    backward(T.sum_(d.rsample((2,), seed=1)))
    assert torch.equal(loc.grad().data(), torch.full((3, 1), 4.0))
    m = D.Dirichlet(T.tensor(torch.ones(2, 5)))
    s = m.sample((3,), seed=1)
    assert tuple(s.shape) == (3, 2, 5) and tuple(m.log_prob(s).shape) == (3, 2)
    assert isinstance(D.Poisson(vec(1.0)).rsample().err, E.ErrNotDifferentiable)
    c = D.Categorical(logits=T.tensor(torch.zeros(2, 3, 5)))
    assert tuple(c.sample((4,), seed=2).shape) == (4, 2, 3) and c.batch_shape == (2, 3)
    assert tuple(c.log_prob(T.tensor(torch.tensor([1, 0, 4], dtype=torch.int32))).shape) == (2, 3)


def test_support_and_limits():
    u = D.Uniform(vec(0), vec(2))
    got = u.log_prob(vec(-1, 0, 1, 2)).data()
    assert got[0] == -math.inf and got[3] == -math.inf and abs(float(got[1]) + math.log(2)) < 1e-6 and got[1] == got[2]
    assert float(D.kl(u, D.Uniform(vec(0.5), vec(3))).data()) == math.inf
    assert abs(float(D.kl(u, D.Uniform(vec(-1), vec(3))).data()) - math.log(2)) < 1e-6
    p, q, r = D.Categorical(probs=vec(0, 1, 1)), D.Categorical(probs=vec(1, 0, 1)), D.Categorical(probs=vec(1, 1, 1))
    assert float(D.kl(p, q).data()) == math.inf
    assert abs(float(D.kl(p, r).data()) - math.log(1.5)) < 1e-6
    assert abs(float(p.entropy().data()) - math.log(2)) < 1e-6
    assert float(D.Bernoulli(probs=vec(0, 1)).entropy().data().max()) < 1e-5
    big = D.Poisson(vec(30.0, 200.0)).entropy().data()
    want = torch.distributions.Normal(0.0, torch.tensor([30.0, 200.0]).sqrt()).entropy()     # the leading term
    assert torch.allclose(big, want, atol=5e-3)
    n = D.Normal(vec(1.0), vec(2.0))
    assert abs(float(n.icdf(n.cdf(vec(2.5))).data()) - 2.5) < 1e-5


def test_covariance_form_and_python_numbers():
    cov = torch.tensor([[2.0, 0.3], [0.3, 1.0]])
    a = D.MultivariateNormal(vec(0.5, -1), covariance=T.tensor(cov))
    want = torch.distributions.MultivariateNormal(torch.tensor([0.5, -1.0]), covariance_matrix=cov)
    x = torch.tensor([[0.1, 0.2], [1.0, -2.0]])
    assert torch.allclose(a.log_prob(T.tensor(x)).data(), want.log_prob(x), atol=1e-5)
    assert torch.allclose(a.covariance().data(), cov, atol=1e-6) and abs(float(a.entropy().data()) - float(want.entropy())) < 1e-5
    assert abs(float(D.Normal(0.0, 1.0).log_prob(0.0).data()) + 0.5 * math.log(2 * math.pi)) < 1e-6
    assert D.Normal(0, 1).batch_shape == ()


def test_errors_are_sticky_not_raised():
    cases = {
        "normal shapes": (D.Normal(vec(1, 2), vec(1, 2, 3)).sample(seed=1), E.ErrShape),
        "normal dtype": (D.Normal(T.tensor(torch.ones(2, dtype=torch.int32)), vec(1, 2)).entropy(), E.ErrDType),
        "mvn shapes": (D.MultivariateNormal(vec(1, 2), scale_tril=T.tensor(torch.ones(3, 3))).mean(), E.ErrShape),
        "mvn rank": (D.MultivariateNormal(vec(1, 2), scale_tril=vec(1, 2)).log_prob(vec(0, 0)), E.ErrShape),
        "categorical empty": (D.Categorical(probs=T.tensor(torch.ones(2, 0))).sample(seed=1), E.ErrShape),
        "categorical sizes": (D.kl(D.Categorical(probs=vec(1, 1)), D.Categorical(probs=vec(1, 1, 1))), E.ErrShape),
        "no KL": (D.kl(D.Normal(vec(0), vec(1)), D.Laplace(vec(0), vec(1))), D.ErrNoKL),
        "failed parameter": (D.Gamma(T.core._error_tensor(E.ErrIndex("x")), vec(1)).rsample(seed=1), E.ErrIndex),
        "failed value": (D.Normal(vec(0), vec(1)).log_prob(T.core._error_tensor(E.ErrIndex("x"))), E.ErrIndex),
        "both forms": (D.Bernoulli(probs=vec(0.5), logits=vec(0.0)).entropy(), E.ErrShape),
    }
    for name, (got, want) in cases.items():
        assert isinstance(got.err, want), (name, got.err)
