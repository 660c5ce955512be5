"""Storage versions, destinations of ``realize_into`` and the buffer pool (reference:
internal/sched/into.go:24-66, memory.go:144-190, internal/graph/graph.go:86-115; behaviour after
tensor/tensor.go:356-378)."""
import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200.tensor import memory, plan


def _stale(t):
    with pytest.raises(T.ErrOverwritten):
        t.data()


def test_elementwise_update_is_computed_straight_into_its_destination(unfused):
    p = T.tensor(torch.arange(6.0).reshape(2, 3))
    g = T.tensor(torch.ones(2, 3))
    mem = p.data()
    before = plan.stats()["into_direct"]
    new = T.realize_into(p, p - g * 0.5)                 # an optimizer's update: reads p elementwise, writes p
    assert plan.stats()["into_direct"] == before + 1     # no temporary, no copy
    assert new.data().data_ptr() == mem.data_ptr()
    assert mem.tolist() == [[-0.5, 0.5, 1.5], [2.5, 3.5, 4.5]]
    _stale(p)
    again = T.realize_into(new, new * 2.0)               # the live handle can be written over in turn
    assert again.data().data_ptr() == mem.data_ptr() and mem[0, 0] == -1.0
    _stale(new)


def test_a_destination_that_is_read_later_is_written_after_the_schedule(unfused):
    a = T.tensor(torch.tensor([1.0, 2.0, 3.0]))
    b = T.tensor(torch.tensor([10.0, 20.0, 30.0]))
    ma, mb = a.data(), b.data()
    before = plan.stats()["into_direct"]
    na, nb = T.realize_into([a, b], [b * 2.0, a * 3.0])    # each source reads the other's destination
    assert ma.tolist() == [20.0, 40.0, 60.0] and mb.tolist() == [3.0, 6.0, 9.0]     # old values on both sides
    # the second product runs last, so it alone may land straight in its destination
    assert plan.stats()["into_direct"] - before <= 1
    assert na.data().data_ptr() == ma.data_ptr() and nb.data().data_ptr() == mb.data_ptr()
    _stale(a)
    _stale(b)


def test_non_elementwise_sources_and_realized_sources_are_copied():
    w = T.tensor(torch.eye(3) * 2.0)
    x = T.tensor(torch.arange(9.0).reshape(3, 3))
    dst = T.tensor(torch.zeros(3, 3))
    mem = dst.data()
    out = T.realize_into(dst, T.matmul(x, w))
    assert torch.equal(mem, torch.arange(9.0).reshape(3, 3) * 2.0) and out.data().data_ptr() == mem.data_ptr()
    ready = (x + 1.0).realize()
    dst2 = T.tensor(torch.zeros(3, 3))
    out2 = T.realize_into(dst2, ready)
    assert out2 is ready and torch.equal(out2.data(), torch.arange(9.0).reshape(3, 3) + 1.0)
    assert T.realize_into([None], [x * 1.0])[0].data().tolist() == x.data().tolist()     # no destination: new memory


def test_views_of_overwritten_memory_are_stale_and_misfits_are_refused():
    base = torch.arange(8.0)
    whole = T.from_torch(base)
    half = T.from_torch(base[4:])                          # shares the memory
    other = T.tensor(torch.arange(8.0))                    # does not
    T.realize_into(whole, whole + 1.0)
    _stale(half)
    assert other.data()[1] == 1.0
    fresh = T.from_torch(base[4:])                         # realized after the write: current
    assert fresh.data().tolist() == [5.0, 6.0, 7.0, 8.0]
    with pytest.raises(T.ErrShape):
        T.realize_into(other, T.tensor([1.0, 2.0]) * 2.0)
    with pytest.raises(T.ErrShape):
        T.realize_into(other, T.cast(other, T.int32) * 2)
    both = T.from_torch(torch.zeros(4))
    with pytest.raises(T.ErrOverwritten):
        T.realize_into([both, T.from_torch(both.data())], [both * 2.0, both * 3.0])
    lazy = other + 1.0
    with pytest.raises(T.ErrNilTensor):
        T.realize_into(lazy, other * 1.0)
    bad = T.matmul(T.tensor(torch.ones(2, 3)), T.tensor(torch.ones(2, 3)))     # a sticky shape error
    keep = T.tensor(torch.zeros(2, 2))
    with pytest.raises(T.ErrShape):
        T.realize_into(keep, bad)
    assert keep.data().sum() == 0                          # nothing written, still current


@pytest.fixture
def unfused():
    """The pool tests watch the temporaries of single elementwise instructions, so the planner must not
    fold their chains into one program."""
    old = plan.set_elementwise_fusion(False)
    yield
    plan.set_elementwise_fusion(old)


def test_pool_serves_elementwise_temporaries_and_replays_over_the_same_buffers(unfused):
    memory.set_pool("cpu")
    pool = memory.pool()
    pool.trim()
    x = T.tensor(torch.randn(64, 64))
    y = T.tensor(torch.randn(64, 64))

    def f(a, b):
        return T.exp(T.tanh(a * b + a) - b).reshape((32, 128))

    want = torch.exp(torch.tanh(x.data() * y.data() + x.data()) - y.data()).reshape(32, 128)
    first = f(x, y).realize()
    st0 = pool.stats()
    assert torch.allclose(first.data(), want) and st0["takes"] >= 4
    second = f(x, y).realize()
    st1 = pool.stats()
    assert st1["reused"] - st0["reused"] >= 3              # the temporaries of the first run serve the second
    third = f(x, y).realize()
    st2 = pool.stats()
    assert st2["obtained_bytes"] - st1["obtained_bytes"] <= 64 * 64 * 4      # steady state: one result buffer per run leaves the pool
    # results left the pool with their buffers: later runs did not write over them
    assert torch.equal(first.data(), second.data()) and torch.equal(first.data(), third.data())
    assert len({first.data().data_ptr(), second.data().data_ptr(), third.data().data_ptr()}) == 3


def test_pooled_buffer_stays_out_while_a_view_of_it_is_read(unfused):
    memory.set_pool("cpu")
    a = T.tensor(torch.arange(12.0))
    s = (a + 1.0).reshape((3, 4))                          # a view of a pooled buffer ...
    t = T.permute(s, (1, 0))                               # ... and a view of that view
    u = t * 2.0 + T.sum_(s)                                # read after the buffer's own slot has been dropped
    want = (torch.arange(12.0) + 1).reshape(3, 4).t() * 2 + (torch.arange(12.0) + 1).sum()
    for _ in range(3):
        assert torch.equal((t * 2.0 + T.sum_(s)).data(), want)
    assert torch.equal(u.data(), want)
    parts = T.split(a * 3.0, [5, 7])                       # a tuple of views of one pooled buffer as results
    T.realize(*parts)
    (a * 5.0).realize()
    (a * 7.0).realize()
    assert parts[0].data().tolist() == [0.0, 3.0, 6.0, 9.0, 12.0] and parts[1].data()[-1] == 33.0


def test_pool_is_not_used_under_autograd_and_can_be_turned_off():
    from mimir_b200.tensor.autograd import Param, backward
    memory.set_pool("cpu")
    pool = memory.pool()
    p = Param(torch.randn(8, 8))
    takes = pool.stats()["takes"]
    loss = T.sum_(T.tanh(p.value() * 2.0) * T.tanh(p.value() * 2.0))
    backward(loss)
    assert pool.stats()["takes"] == takes and p.grad() is not None
    memory.set_pool("0")
    (T.tensor(torch.ones(4)) * 2.0 + 1.0).realize()
    assert pool.stats()["takes"] == takes and pool.stats()["buffers"] == 0
    memory.set_pool("cpu")


def test_a_view_made_before_the_write_and_read_after_it_keeps_the_old_values():
    d = T.tensor(torch.arange(6.0))
    mem = d.data()
    v = T.reshape(d, (2, 3))
    total, new, later = T.realize_into([None, d, None], [T.sum_(v), d * 2.0, v + 1.0])
    assert total.item() == 15.0
    assert later.data().tolist() == [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]      # computed from the old values
    assert mem.tolist() == [0.0, 2.0, 4.0, 6.0, 8.0, 10.0] and new.data().data_ptr() == mem.data_ptr()


def test_broadcast_operands_and_mixed_dtypes_take_the_pool_path_correctly(unfused):
    memory.set_pool("cpu")
    a = T.tensor(torch.randn(4, 1, 8))
    b = T.tensor(torch.randn(5, 1))
    h = T.cast(T.tensor(torch.randn(4, 5, 8)), T.bfloat16)
    want = (a.data() * b.data() + h.data().float()).abs().neg()
    for _ in range(3):
        got = T.neg(T.abs_(a * b + h)).data()
        assert got.dtype == torch.float32 and torch.equal(got, want)
    small = T.tensor(torch.randn(3)) + 1                    # a Python scalar operand
    assert small.data().shape == (3,)


def test_donated_batch_is_read_once_and_its_memory_serves_the_same_schedule(unfused):
    memory.set_pool("cpu")
    pool = memory.pool()
    pool.trim()
    w = T.tensor(torch.randn(64, 64))

    def step(batch):
        return T.sum_(T.tanh(batch * 2.0 + 1.0) * 3.0)

    want = float(torch.sum(torch.tanh(torch.ones(64, 64) * 2.0 + 1.0) * 3.0))
    kept = T.tensor(torch.ones(64, 64))
    assert abs(step(kept).item() - want) < 1e-3
    base = pool.stats()
    for _ in range(3):
        batch = T.tensor(torch.ones(64, 64)).donate()       # the tensor owns its memory: nobody else holds it
        out = step(batch)
        assert abs(out.item() - want) < 1e-3
        with pytest.raises(T.ErrDonated):
            (batch + 1.0).data()
    after = pool.stats()
    assert after["obtained_bytes"] == base["obtained_bytes"]        # the donated batches fed the pool: nothing new was asked for
    assert plan.stats()["cached"] >= 2                              # the donating step has a program of its own
    # memory somebody else can reach is never taken
    mine = torch.ones(64, 64)
    shared = T.from_torch(mine).donate()
    assert abs(step(shared).item() - want) < 1e-3
    for _ in range(4):
        step(T.tensor(torch.zeros(64, 64))).item()
    assert float(mine.sum()) == 64 * 64                               # still the caller's values
    with pytest.raises(T.ErrDonated):
        shared.data()
    # a tensor that is not computed yet is left alone; a refused schedule leaves its batch alone
    lazy = (w + 1.0).donate()
    assert lazy.data().shape == (64, 64) and lazy.data().shape == (64, 64)
    cpu = T.CPU()
    T.set_memory_budget(cpu, 1024)
    try:
        b = T.tensor(torch.ones(64, 64)).donate()
        with pytest.raises(T.ErrMemoryBudget):
            step(b).item()
    finally:
        T.set_memory_budget(cpu, None)
    assert abs(step(b).item() - want) < 1e-3                          # it was not consumed by the refused schedule


def test_unused_buffers_age_out_of_the_pool(unfused):
    memory.set_pool("cpu")
    pool = memory.pool()
    pool.trim()
    big = T.tensor(torch.randn(256, 256))
    (T.exp(big * 2.0) + 1.0).realize()
    assert pool.stats()["held_bytes"] >= 256 * 256 * 4          # a temporary of that size waits for reuse
    small = T.tensor(torch.randn(8))
    for _ in range(2 * pool.AGE_OUT + 1):
        (small * 2.0 + 1.0).realize()                           # schedules that never ask for it
    assert all(k[2] != 256 * 256 for k in pool.free)           # released
    assert pool.stats()["held_bytes"] < 256 * 256 * 4


def test_elementwise_chains_run_as_one_fused_program_on_the_cpu():
    """internal/sched/fuse.go:200-362: a chain of elementwise ops is one kernel; here one native program
    over cache-sized blocks, with the composed PyTorch ops as the path under autograd."""
    from mimir_b200.tensor.autograd import Param, backward
    plan.set_elementwise_fusion(True)
    torch.manual_seed(0)
    a, b = torch.randn(300, 77), torch.rand(300, 77) + 0.5
    x, y = T.tensor(a), T.tensor(b)
    before = plan.stats()["fused"]

    def f(p, q):
        u = T.tanh(p * q + 1.5) - T.sqrt(q)
        return T.maximum(T.exp(u) * 0.25, T.abs_(p)) / (T.softplus(q) + T.sigmoid(p)) + T.gelu(p) * T.silu(q)

    def ref(p, q):
        F = torch.nn.functional
        u = torch.tanh(p * q + 1.5) - torch.sqrt(q)
        return torch.maximum(torch.exp(u) * 0.25, torch.abs(p)) / (F.softplus(q) + torch.sigmoid(p)) + F.gelu(p, approximate="tanh") * F.silu(q)
    got = f(x, y).data()
    assert plan.stats()["fused"] - before == 1                       # the whole expression is one program
    assert torch.allclose(got, ref(a, b), rtol=2e-6, atol=2e-6)
    assert torch.equal(f(x, y).data(), got)                          # cached program, same result
    # NaNs and signed zeros go through like the single ops
    s = torch.tensor([float("nan"), -0.0, 0.0, -3.0, 2.0, float("inf")] * 100)
    st = T.tensor(s)
    out = (T.relu(st) + T.sign(st) * 2.0 + T.minimum(st, 1.0)).data()
    want = torch.relu(s) + torch.sign(s) * 2.0 + torch.minimum(s, torch.tensor(1.0))
    assert torch.equal(torch.isnan(out), torch.isnan(want)) and torch.equal(out[~torch.isnan(out)], want[~torch.isnan(want)])
    # under autograd the same program runs as composed ops and gives gradients
    p = Param(a.clone())
    loss = T.sum_(f(p.value(), y))
    backward(loss)
    ar = a.clone().requires_grad_(True)
    ref(ar, b).sum().backward()
    assert torch.allclose(p.grad().data(), ar.grad, rtol=1e-4, atol=1e-5)
    # a value with two readers is not folded away; other dtypes and strided operands stay on PyTorch
    h = T.exp(x * 0.5)
    both = (h + 1.0).data(), (h * 2.0).data()
    assert torch.allclose(both[0], torch.exp(a * 0.5) + 1.0) and torch.allclose(both[1], torch.exp(a * 0.5) * 2.0)
    xd = T.tensor(a.double())
    assert (T.exp(xd * 0.5) + 1.0).data().dtype == torch.float64
    xt = T.from_torch(a.t())
    assert torch.allclose((T.exp(xt * 0.5) + 1.0).data(), torch.exp(a.t() * 0.5) + 1.0)
    # into a destination: the fused program writes straight into it
    dst = T.tensor(torch.zeros(300, 77))
    mem = dst.data()
    before = plan.stats()["into_direct"]
    T.realize_into(dst, T.tanh(x * 2.0) + y)
    assert plan.stats()["into_direct"] == before + 1 and torch.allclose(mem, torch.tanh(a * 2.0) + b, atol=1e-6)
