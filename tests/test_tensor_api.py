"""Behavioural contracts of the lazy tensor layer (tensor/tensor.go semantics)."""
import pytest
import torch


def test_lazy_until_realized_and_sticky_errors():
    import mimir_b200.tensor as T
    a = T.tensor([[1.0, 2.0], [3.0, 4.0]], device=T.CPU())
    c = (a @ a + 1.0) * 2
    assert c._val is None and c.shape == (2, 2)
    assert torch.equal(c.data(), (a.data() @ a.data() + 1) * 2)
    bad = a @ T.tensor([1.0, 2.0, 3.0], device=T.CPU())
    assert isinstance(bad.err, T.ErrShape)
    later = T.relu(bad + 1) * 3
    assert later.err is bad.err
    with pytest.raises(T.ErrShape):
        later.item()
    mixed = a + T.tensor([1, 2], device=T.CPU())
    assert isinstance(mixed.err, T.ErrDType)
    half = T.cast(a, torch.bfloat16) + a
    assert half.dtype == torch.float32  # half (+) float32 -> float32 is the one promotion
    assert T.sum_(T.cast(a, torch.float16)).dtype == torch.float32
    idx = T.gather_rows(a, T.tensor([0, 5], device=T.CPU()))
    with pytest.raises(T.ErrIndex):
        idx.data()
    with pytest.raises(T.ErrDivideByZero):
        (T.tensor([4, 2], device=T.CPU()) / T.tensor([2, 0], device=T.CPU())).data()


def test_param_backward_accumulates_and_staleness():
    import mimir_b200.tensor as T
    p = T.Param(torch.tensor([1.0, 2.0, 3.0]))
    x = p.value()
    T.sum_(x * x).backward()
    T.sum_(p.value() * 3.0).backward()
    assert torch.allclose(p.grad().data(), 2 * p._data + 3)
    p.set(torch.zeros(3))
    with pytest.raises(T.ErrOverwritten):
        (x + 1).data()
    frozen = T.Param(torch.ones(2)).freeze()
    with pytest.raises(T.ErrNoGrad):
        T.sum_(frozen.value() * 2).backward()


def test_transforms_scan_record_trace_budget():
    import mimir_b200.tensor as T
    cpu = T.CPU()
    x = T.tensor([1.0, 2.0, 3.0], device=cpu)
    assert torch.allclose(T.grad(lambda t: T.sum_(t * t * t))(x).data(), 3 * x.data() ** 2)
    out, pull = T.vjp(lambda t: t * t, x)
    assert torch.allclose(pull(T.tensor([1.0, 1.0, 1.0], device=cpu))[0].data(), 2 * x.data())
    _, tan = T.jvp(lambda t: T.sin(t), (x,), (T.ones((3,), device=cpu),))
    assert torch.allclose(tan.data(), x.data().cos())
    assert torch.allclose(T.hessian(lambda t: T.sum_(t * t * t), x).data(), torch.diag(6 * x.data()))
    assert torch.allclose(T.jacobian(lambda t: t * t, x).data(), torch.diag(2 * x.data()))
    per = T.vmap(lambda t: T.sum_(t * t))(T.tensor([[1.0, 2.0], [3.0, 4.0]], device=cpu))
    assert per.tolist() == [5.0, 25.0]
    carry, ys = T.scan(lambda c, v: (c + v, c * v), T.tensor(0.0, device=cpu), x)
    assert carry.item() == 6.0 and ys.tolist() == [0.0, 2.0, 9.0]
    rc, ys_r = T.scan(lambda c, v: (c + v, c), T.tensor(0.0, device=cpu), x, reverse=True)
    assert ys_r.tolist() == [5.0, 3.0, 0.0]
    rec = T.record(lambda t: T.relu(t) * 2, x)
    again, ok = rec.replay(T.tensor([-1.0, 5.0, 2.0], device=cpu))
    assert ok and again.tolist() == [0.0, 10.0, 4.0]
    _, ok = rec.replay(T.ones((4,), device=cpu))
    assert not ok
    assert T.trace(lambda t: T.relu(t) + 1, x).ops() == ["input", "relu", "const", "add"]
    T.set_memory_budget(cpu, 64)
    try:
        with pytest.raises(T.ErrMemoryBudget):
            (T.ones((1000,), device=cpu) * 2).data()
    finally:
        T.set_memory_budget(cpu, None)
    d = T.ones((2,), device=cpu).realize().donate()
    with pytest.raises(T.ErrDonated):
        (d + 1).data()


def test_custom_func_and_checkpoint_gradients():
    import mimir_b200.tensor as T
    sq = T.func(lambda v: v * v, lambda xs, out, g: (2 * xs[0] * g,))
    p = T.Param(torch.tensor([1.0, -2.0]))
    T.sum_(sq(p.value())).backward()
    assert torch.allclose(p.grad().data(), 2 * p._data)
    q = T.Param(torch.tensor([0.5, 1.5]))
    T.sum_(T.checkpoint(lambda t: T.exp(t) * t)(q.value())).backward()
    want = q._data.exp() * (1 + q._data)
    assert torch.allclose(q.grad().data(), want)
