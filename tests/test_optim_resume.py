"""Every optimizer: save, restore into a fresh optimizer, take one more step; the result equals the
uninterrupted run exactly (exact-resume contract of train/train_test.go:101 for optim/optim.go:269-306)."""
import pytest
import torch

from mimir_b200 import optim
from mimir_b200.tensor.autograd import Param

NAMES = ["SGD", "Adam", "AdamW", "RMSprop", "Adagrad", "Adadelta", "Adamax", "NAdam", "RAdam", "Lion"]


def _run(name, steps, resume_at=None):
    torch.manual_seed(0)
    mk = lambda: [Param(torch.linspace(-1, 1, 12).reshape(3, 4)), Param(torch.linspace(0.5, 2, 5))]  # noqa: E731
    kw = dict(momentum=0.9) if name == "SGD" else {}
    ps = mk()
    opt = getattr(optim, name)(ps, **kw)
    g = torch.Generator().manual_seed(1)
    grads = [[torch.randn(p.shape, generator=g) for p in ps] for _ in range(steps)]
    for t in range(steps):
        if resume_at is not None and t == resume_at:
            snap = {k: v.clone() for k, v in opt.snapshot().items()}
            vals = [p._data.clone() for p in ps]
            ps = mk()
            for p, v in zip(ps, vals):
                p.set(v)
            fresh = getattr(optim, name)(ps, **kw)
            fresh.restore(snap, steps=opt.steps)
            opt = fresh
        for p, gr in zip(ps, grads[t]):
            p._grad = gr.clone()
        opt.step()
        opt.zero_grad()
    return [p._data.clone() for p in ps]


@pytest.mark.parametrize("name", NAMES)
def test_resume_is_exact(name):
    a = _run(name, 6)
    b = _run(name, 6, resume_at=3)
    for x, y in zip(a, b):
        assert torch.equal(x, y), name
