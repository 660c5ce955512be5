"""The 20 losses, built from the tensor layer's own ops, against ``torch.nn.functional`` in float64:
values and gradients (reference: nn/loss/loss_test.go, golden ``losses.mim``)."""
import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200.nn import loss as L
from mimir_b200.tensor.autograd import Param, backward

F = torch.nn.functional
torch.manual_seed(0)
N, C = 6, 5
logits = torch.randn(N, C, dtype=torch.float64)
cls = torch.randint(0, C, (N,))
prob = torch.rand(N, C, dtype=torch.float64) * 0.98 + 0.01
tgt01 = (torch.rand(N, C) > 0.5).double()
dist = torch.softmax(torch.randn(N, C, dtype=torch.float64), 1)
dist[0, 0] = 0.0                                         # an entry with zero probability
other = torch.randn(N, C, dtype=torch.float64)
third = torch.randn(N, C, dtype=torch.float64)
sign = torch.tensor([1.0, -1.0, 1.0, -1.0, -1.0, 1.0], dtype=torch.float64)
seg_logits = torch.randn(2, 3, 4, 4, dtype=torch.float64)
seg_cls = torch.randint(0, 3, (2, 4, 4))
seg01 = (torch.rand(2, 1, 4, 4) > 0.5).double()
var = torch.rand(N, C, dtype=torch.float64) + 0.1


def _dice(l, t, eps=1.0):
    p = torch.softmax(l, 1)
    oh = F.one_hot(t, l.shape[1]).movedim(-1, 1).double()
    dims = tuple(range(2, l.dim()))
    return (1 - (2 * (p * oh).sum(dims) + eps) / (p.sum(dims) + oh.sum(dims) + eps)).mean()


def _bdice(l, t, eps=1.0):
    p, t = torch.sigmoid(l).flatten(1), t.flatten(1)
    return (1 - (2 * (p * t).sum(1) + eps) / (p.sum(1) + t.sum(1) + eps)).mean()


def _focal(g):
    def f(l, t):
        lp = F.log_softmax(l, -1).gather(-1, t.unsqueeze(-1)).squeeze(-1)
        return (-(1 - lp.exp()) ** g * lp).mean()
    return f


def _bfocal(g, a):
    def f(l, t):
        p = torch.sigmoid(l)
        pt = p * t + (1 - p) * (1 - t)
        al = a * t + (1 - a) * (1 - t)
        return (al * (1 - pt) ** g * F.binary_cross_entropy_with_logits(l, t, reduction="none")).mean()
    return f


def _hinge(s, t):
    m = (1 + s - s.gather(-1, t.unsqueeze(-1))).clamp_min(0).scatter(-1, t.unsqueeze(-1), 0.0)
    return m.sum(-1).mean()


CASES = [
    ("cross_entropy", L.cross_entropy, F.cross_entropy, (logits,), (cls,)),
    ("nll", L.nll, F.nll_loss, (torch.log_softmax(logits, 1),), (cls,)),
    ("label_smoothing", L.label_smoothing(0.1), lambda l, t: F.cross_entropy(l, t, label_smoothing=0.1), (logits,), (cls,)),
    ("focal", L.focal(2.0), _focal(2.0), (logits,), (cls,)),
    ("hinge", L.hinge, _hinge, (logits,), (cls,)),
    ("dice", L.dice, _dice, (seg_logits,), (seg_cls,)),
    ("bce_with_logits", L.bce_with_logits, F.binary_cross_entropy_with_logits, (logits,), (tgt01,)),
    ("bce", L.bce, F.binary_cross_entropy, (prob,), (tgt01,)),
    ("mse", L.mse, F.mse_loss, (logits,), (other,)),
    ("l1", L.l1, F.l1_loss, (logits,), (other,)),
    ("huber", lambda p, t: L.huber(p, t, 0.7), lambda p, t: F.huber_loss(p, t, delta=0.7), (logits,), (other,)),
    ("smooth_l1", L.smooth_l1(0.5), lambda p, t: F.smooth_l1_loss(p, t, beta=0.5), (logits,), (other,)),
    ("kl_div", L.kl_div, lambda l, t: F.kl_div(l, t, reduction="batchmean"), (torch.log_softmax(logits, 1),), (dist,)),
    ("poisson_nll", L.poisson_nll, lambda l, t: F.poisson_nll_loss(l, t, log_input=True), (logits,), (tgt01 * 3,)),
    ("gaussian_nll", lambda m, v, t: L.gaussian_nll(m, v, t), lambda m, v, t: F.gaussian_nll_loss(m, t, v), (logits, var), (other,)),
    ("binary_focal", L.binary_focal(2.0, 0.25), _bfocal(2.0, 0.25), (logits,), (tgt01,)),
    ("binary_dice", L.binary_dice, _bdice, (seg_logits[:, :1],), (seg01,)),
    ("margin_ranking", L.margin_ranking(0.3), lambda a, b, y: F.margin_ranking_loss(a, b, y, margin=0.3), (logits[:, 0], other[:, 0]), (sign,)),
    ("triplet", L.triplet(1.0), lambda a, p, n: F.triplet_margin_loss(a, p, n, margin=1.0), (logits, other, third), ()),
    ("cosine_embedding", L.cosine_embedding(0.2), lambda a, b, y: F.cosine_embedding_loss(a, b, y, margin=0.2), (logits, other), (sign,)),
]


def test_all_twenty_are_covered():
    assert sorted(n for n, *_ in CASES) == sorted(L.ALL)


@pytest.mark.parametrize("name,ours,ref,diff_in,fixed_in", CASES, ids=[c[0] for c in CASES])
def test_value_and_gradients_match_float64_reference(name, ours, ref, diff_in, fixed_in):
    refs = [x.clone().requires_grad_(True) for x in diff_in]
    want = ref(*refs, *fixed_in)
    want.backward()
    params = [Param(x.float()) for x in diff_in]
    fixed = [T.tensor(x.float() if x.dtype.is_floating_point else x) for x in fixed_in]
    got = ours(*[p.value() for p in params], *fixed)
    assert got.err is None, got.err
    backward(got)
    assert got.shape == () and abs(got.item() - want.item()) < 2e-5 * max(1.0, abs(want.item())), (got.item(), want.item())
    for p, r in zip(params, refs):
        assert torch.allclose(p.grad().data().double(), r.grad, atol=2e-5, rtol=1e-4), name


def test_half_inputs_are_widened_and_misfits_are_sticky_errors():
    x = T.cast(T.tensor(logits.float()), T.bfloat16)
    y = T.tensor(other.float())
    out = L.mse(x, y)
    assert out.dtype == T.float32 and abs(out.item() - F.mse_loss(logits.float().bfloat16().float(), other.float()).item()) < 1e-5
    assert isinstance(L.mse(T.tensor(torch.zeros(3)), T.tensor(torch.zeros(4))).err, T.ErrShape)
    assert isinstance(L.nll(T.tensor(torch.zeros(3, 2)), T.tensor(torch.zeros(3))).err, T.ErrDType)
    assert isinstance(L.hinge(T.tensor(torch.zeros(3, 2)), T.tensor(torch.zeros(4, dtype=torch.int64))).err, T.ErrShape)
    bad = T.matmul(T.tensor(torch.ones(2, 3)), T.tensor(torch.ones(2, 3)))
    assert L.l1(bad, T.tensor(torch.zeros(2, 2))).err is bad.err          # errors pass through
