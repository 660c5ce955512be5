"""Effects carried by tensors (``with_effects``), lazy buffer values and batch normalisation built on
them (reference: tensor/autograd.go:753-777, nn/layers.go:196-243)."""
import pytest
import torch

from mimir_b200 import nn, optim
from mimir_b200 import tensor as T


def test_with_effects_keeps_value_and_gradient_and_backward_computes_the_effect():
    w = T.Param(torch.tensor([1.0, 2.0, 3.0]), "w")
    x = T.from_torch(torch.tensor([0.5, -1.0, 2.0]))
    side = T.sum_(w.value() * 10.0)
    y = T.with_effects(w.value() * x, side)
    assert side._val is None
    loss = T.sum_(y * y)
    T.backward(loss)
    torch.testing.assert_close(w.grad().data(), 2 * torch.tensor([1.0, 2.0, 3.0]) * torch.tensor([0.25, 1.0, 4.0]))
    assert side._val is not None and side.item() == 60.0       # computed by the backward pass itself
    assert T.with_effects(x) is x                               # no effects: the tensor itself
    torch.testing.assert_close(T.with_effects(x, side).data(), x.data())


def test_with_effects_propagates_errors():
    bad = T.from_torch(torch.ones(2)) + T.from_torch(torch.ones(3))
    assert T.with_effects(T.from_torch(torch.ones(2)), bad).err is not None


def test_buffer_takes_a_lazy_value_on_the_next_read():
    b = T.Buffer(torch.zeros(3), "state")
    src = T.Param(torch.ones(3), "src")
    b.set(src.value() * 4.0)
    assert b.__dict__["_lazy"] is not None
    torch.testing.assert_close(b.value().data(), torch.full((3,), 4.0))
    assert b.__dict__["_lazy"] is None
    with pytest.raises(T.ErrShape):
        b.set(T.from_torch(torch.ones(4)) * 2.0)


def test_batch_norm_matches_torch_in_training_and_evaluation():
    torch.manual_seed(0)
    nn.manual_seed(0)
    x = torch.randn(6, 3, 4, 4)
    m = nn.Sequential(nn.Conv2d(3, 3, 1), nn.BatchNorm2d(3))
    ref = torch.nn.Sequential(torch.nn.Conv2d(3, 3, 1), torch.nn.BatchNorm2d(3))
    ref[0].weight.data.copy_(m.layers[0].weight._data)
    ref[0].bias.data.copy_(m.layers[0].bias._data)
    scale = torch.arange(3.0).reshape(1, 3, 1, 1)
    for _ in range(2):
        out = m(T.from_torch(x))
        T.backward(T.sum_(out * out * T.from_torch(scale)))
        o = ref(x)
        (o * o * scale).sum().backward()
    bn = m.layers[1]
    lazy = bn.running_mean.__dict__["_lazy"]
    assert lazy is not None and lazy._val is not None            # the backward pass computed it
    torch.testing.assert_close(bn.running_mean._data, ref[1].running_mean)
    torch.testing.assert_close(bn.running_var._data, ref[1].running_var)
    torch.testing.assert_close(m.layers[0].weight.grad().data(), ref[0].weight.grad, rtol=1e-4, atol=1e-4)
    m.eval()
    ref.eval()
    torch.testing.assert_close(m(T.from_torch(x)).data(), ref(x), rtol=1e-5, atol=1e-5)


def test_running_statistics_survive_an_optimizer_step_without_backward():
    torch.manual_seed(1)
    nn.manual_seed(1)
    x = torch.randn(8, 4)
    m = nn.Sequential(nn.Linear(4, 4), nn.BatchNorm1d(4))
    ref = torch.nn.BatchNorm1d(4)
    h = m.layers[0](T.from_torch(x)).data()
    m(T.from_torch(x))                          # forward only: the buffers hold recipes
    for p in m.parameters():
        p._grad = torch.ones_like(p._data)
    optim.SGD(m.parameters(), lr=0.5).step()
    ref(h)
    torch.testing.assert_close(m.layers[1].running_mean._data, ref.running_mean)
    torch.testing.assert_close(m.layers[1].running_var._data, ref.running_var)


def test_batch_norm_needs_two_values_per_channel():
    bn = nn.BatchNorm1d(3)
    assert bn(T.from_torch(torch.ones(1, 3))).err is not None
