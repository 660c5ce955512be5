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
    assert (d + 1).data().tolist() == [2.0, 2.0]          # the next schedule that reads it may
    with pytest.raises(T.ErrDonated):                     # from then on it is stale
        (d + 1).data()
    with pytest.raises(T.ErrDonated):
        d.data()


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


def test_bytes_round_trip_realize_into_and_record_into():
    import mimir_b200.tensor as T
    x = T.tensor([[1.0, 2.0], [3.0, 4.0]])
    raw = x.bytes()
    assert len(raw) == 16
    y = T.from_bytes(raw, (2, 2))
    assert y.data().tolist() == [[1.0, 2.0], [3.0, 4.0]]
    buf = bytearray(16)
    assert x.read_bytes(buf) == 16 and bytes(buf) == raw
    assert T.from_bytes(raw[:8], (2, 2)).err is not None                 # too few bytes: a sticky error, no exception
    z = T.from_bytes_func(lambda mv: mv.__setitem__(slice(0, 16), raw), (2, 2))
    assert z.data().tolist() == y.data().tolist()
    dst = T.tensor([[0.0, 0.0], [0.0, 0.0]])
    held = dst.data()
    view = T.from_torch(held[0])                                          # a view of the same memory, realized earlier
    built = dst + 1.0                                                     # built from the old value, not computed yet
    new = T.realize_into(dst, x * 2.0)
    assert held.tolist() == [[2.0, 4.0], [6.0, 8.0]]                      # same storage, new value
    assert new.data().data_ptr() == held.data_ptr() and new.data().tolist() == held.tolist()
    for stale in (dst, view, built):                                      # the destination, its views and what was built on it
        try:
            stale.data()
            raise AssertionError("a stale tensor was read")
        except T.ErrOverwritten:
            pass
    assert (new + 1.0).data().tolist() == [[3.0, 5.0], [7.0, 9.0]]
    out = T.tensor([0.0, 0.0])
    rec = T.record_into(out, lambda a: a + 1.0, T.tensor([1.0, 2.0]))
    assert out.data().tolist() == [2.0, 3.0]
    assert rec.replay_into(out, T.tensor([5.0, 6.0])) and out.data().tolist() == [6.0, 7.0]
    assert not rec.replay_into(out, T.tensor([5.0, 6.0, 7.0]))            # other shape: refused, nothing written
    assert out.data().tolist() == [6.0, 7.0]
    assert isinstance(T.gpus(), list)


def test_kv_cache_write_then_advance():
    import torch
    from mimir_b200 import nn
    c = nn.KVCache(1, 2, 4, 3)
    k = torch.ones(1, 2, 1, 3)
    c.write(k, 2 * k)
    assert c.len == 0 and c.k[0, 0, 0, 0] == 1 and c.v[0, 1, 0, 2] == 2
    c.advance()
    assert c.len == 1 and c.positions(1).tolist() == [1]


def test_apply_lora_to_a_module(tmp_path):
    import os
    import torch
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from mimir_b200.io import mim
    nn.manual_seed(0)
    net = nn.Sequential(nn.Linear(4, 6), nn.ReLU(), nn.Linear(6, 2))
    x = T.from_torch(torch.randn(3, 4))
    base = net(x).data().clone()
    a, b = torch.randn(2, 4) * 0.1, torch.randn(6, 2) * 0.1
    p = os.path.join(tmp_path, "ad.mim")
    mim.write_tensors(p, {"layers.0.lora_a": a, "layers.0.lora_b": b},
                      metadata={"adapter.type": "lora", "adapter.lora.rank": 2, "adapter.lora.alpha": 4.0, "adapter.base": "net"})
    ad = mim.open(p)
    assert mim.lora_info(ad) == {"rank": 2, "alpha": 4.0, "base": "net", "targets": ["layers.0"]}
    assert mim.apply_lora(net, ad) == 1
    w = net.layers[0].base.weight._data
    want = torch.relu(x.data() @ (w + 2.0 * b @ a).t() + net.layers[0].base.bias._data) @ net.layers[2].weight._data.t() + net.layers[2].bias._data
    assert torch.allclose(net(x).data(), want, atol=1e-5) and not torch.allclose(want, base)
