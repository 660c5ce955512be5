"""Sparse patterns and the segment kernel under them (the reference's tensor/pattern_test.go cases:
products against a dense matrix, maxima against a loop, tied gradients, half and integer rows, empty
rows, errors, second derivatives and vmap)."""
import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200.tensor import autograd as A
from mimir_b200.tensor import errors as E
from mimir_b200.tensor.autograd import Param, backward
from mimir_b200.tensor.pattern import Pattern, segment


def _random(rows, cols, n, seed=0, empty_row=None):
    g = torch.Generator().manual_seed(seed)
    row = torch.randint(0, rows, (n,), generator=g)
    col = torch.randint(0, cols, (n,), generator=g)
    if empty_row is not None:
        row[row == empty_row] = (empty_row + 1) % rows
    return Pattern(rows, cols, row, col), row, col


def test_product_and_transpose_match_a_dense_matrix():
    p, _, _ = _random(9, 7, 40)
    D = p.dense()
    assert p.shape == (9, 7) and p.entries == 40 and p.T.shape == (7, 9) and p.T.T is p
    x, y = torch.randn(7, 3, 2), torch.randn(9, 5)
    torch.testing.assert_close(p.matmul(T.tensor(x)).data(), torch.einsum("rc,cab->rab", D, x))
    torch.testing.assert_close(p.T.matmul(T.tensor(y)).data(), D.T @ y)
    torch.testing.assert_close(p.degrees().data(), D.sum(1))
    px, g = Param(x), torch.randn(9, 3, 2)
    backward(T.sum_(p.matmul(px.value()) * T.tensor(g)))
    torch.testing.assert_close(px.grad().data(), torch.einsum("rc,rab->cab", D, g))


def test_entry_maps_are_each_others_transposes():
    p, row, col = _random(6, 5, 21, seed=3)
    r, c = p.coo()
    x, y, v = torch.randn(5, 2), torch.randn(6, 2), torch.randn(21, 2)
    torch.testing.assert_close(p.at_cols(T.tensor(x)).data(), x[c.long()])
    torch.testing.assert_close(p.at_rows(T.tensor(y)).data(), y[r.long()])
    torch.testing.assert_close(p.row_sum(T.tensor(v)).data(), torch.zeros(6, 2).index_add(0, r.long(), v))
    torch.testing.assert_close(p.col_sum(T.tensor(v)).data(), torch.zeros(5, 2).index_add(0, c.long(), v))


def test_maximum_matches_a_loop_and_shares_tied_gradients():
    p, row, col = _random(8, 6, 30, seed=1, empty_row=3)
    x = torch.randn(6, 4)
    want = torch.zeros(8, 4)
    for i in range(8):
        js = col[row == i]
        if len(js):
            want[i] = x[js].max(0).values
    torch.testing.assert_close(p.max(T.tensor(x)).data(), want)
    assert float(p.max(T.tensor(x)).data()[3].abs().max()) == 0.0
    # two columns tie for row 0's maximum: each gets half the gradient
    q = Pattern(1, 3, [0, 0, 0], [0, 1, 2])
    px = Param(torch.tensor([[2.0], [2.0], [1.0]]))
    backward(T.sum_(q.max(px.value())))
    torch.testing.assert_close(px.grad().data(), torch.tensor([[0.5], [0.5], [0.0]]))
    nan = torch.tensor([[1.0], [float("nan")], [0.0]])
    assert torch.isnan(q.max(T.tensor(nan)).data()).all()


def test_half_and_integer_rows_and_empty_rows():
    p, _, _ = _random(7, 5, 25, seed=2, empty_row=4)
    D = p.dense()
    x = torch.randn(5, 6)
    for dt in (torch.bfloat16, torch.float16):
        got = p.matmul(T.tensor(x.to(dt))).data()
        assert got.dtype == dt
        torch.testing.assert_close(got.float(), (D @ x.to(dt).float()).to(dt).float())     # summed in float32, rounded once
    xi = torch.randint(-5, 9, (5, 3), dtype=torch.int32)
    got = p.matmul(T.tensor(xi)).data()
    assert got.dtype == torch.int32 and torch.equal(got.long(), D.long() @ xi.long())
    assert float(p.matmul(T.tensor(x)).data()[4].abs().max()) == 0.0
    assert float(p.mean(T.tensor(x)).data()[4].abs().max()) == 0.0
    torch.testing.assert_close(p.mean(T.tensor(x)).data(), (D @ x) / D.sum(1).clamp(min=1)[:, None])
    empty = Pattern(3, 2, [], [])
    assert torch.equal(empty.matmul(T.tensor(torch.ones(2, 2))).data(), torch.zeros(3, 2))


def test_errors():
    with pytest.raises(E.ErrIndex):
        Pattern(2, 2, [0, 2], [0, 1])
    with pytest.raises(E.ErrIndex):
        Pattern(2, 2, [0, 1], [0, -1])
    with pytest.raises(E.ErrShape):
        Pattern(2, 2, [0, 1], [0])
    with pytest.raises(E.ErrShape):
        Pattern(-1, 2, [], [])
    p = Pattern(2, 3, [0, 1], [2, 0])
    assert isinstance(p.matmul(T.tensor(torch.ones(2, 2))).err, E.ErrShape)
    assert isinstance(p.matmul(T.tensor(torch.tensor(1.0))).err, E.ErrShape)
    assert isinstance(p.max(T.tensor(torch.ones(3, 2, dtype=torch.int32))).err, E.ErrDType)
    failed = p.matmul(T.tensor(torch.ones(2, 2)))
    assert p.T.matmul(failed).err is failed.err                  # an error is passed on, not replaced


def test_second_derivatives_forward_derivatives_and_vmap():
    p, row, col = _random(6, 5, 17, seed=5)
    D = p.dense()
    x = torch.randn(5, 3)

    def f(t):
        return T.sum_(T.exp(p.matmul(t)) * p.max(t))

    def fr(t):
        top = torch.zeros(6, 3).scatter_reduce(0, row[:, None].expand(-1, 3), t[col], "amax", include_self=False)
        return (torch.exp(D @ t) * top).sum()
    torch.testing.assert_close(A.grad(f)(T.tensor(x)).data(), torch.func.grad(fr)(x))
    torch.testing.assert_close(A.hessian(f, T.tensor(x)).data(), torch.func.hessian(fr)(x), rtol=1e-4, atol=1e-5)
    tan = torch.randn(5, 3)
    _, j = A.jvp(lambda t: p.mean(t), (T.tensor(x),), (T.tensor(tan),))
    torch.testing.assert_close(j.data(), (D @ tan) / D.sum(1).clamp(min=1)[:, None])
    xb = torch.randn(4, 5, 3)
    got = A.vmap(lambda t: p.matmul(t))(T.tensor(xb)).data()
    torch.testing.assert_close(got, torch.einsum("rc,bcd->brd", D, xb))
    got = A.vmap(lambda t: p.matmul(t), in_axes=1, out_axes=1)(T.tensor(xb.permute(1, 0, 2).contiguous())).data()
    torch.testing.assert_close(got, torch.einsum("rc,bcd->rbd", D, xb))


def test_results_do_not_depend_on_the_number_of_workers():
    from mimir_b200.ops import quant_cpu
    p, _, _ = _random(3000, 2000, 60000, seed=7)
    x = torch.randn(2000, 64)
    outs = []
    for threads in (1, 3, 8):
        quant_cpu.set_threads(threads)
        outs.append((p.matmul(T.tensor(x)).data().clone(), p.max(T.tensor(x)).data().clone()))
    quant_cpu.set_threads(0)
    for s, mx in outs[1:]:
        assert torch.equal(s, outs[0][0]) and torch.equal(mx, outs[0][1])
    r, c = p.coo()
    want = torch.zeros(3000, 64, dtype=torch.float64).index_add(0, r.long(), x.double()[c.long()])
    torch.testing.assert_close(outs[0][0].double(), want, rtol=1e-5, atol=1e-5)


def test_segment_primitive():
    x = torch.arange(12.0).reshape(4, 3)
    got = segment(T.tensor(x), [0, 2, 2, 5], [3, 0, 1, 1, 2]).data()
    torch.testing.assert_close(got, torch.stack([x[3] + x[0], torch.zeros(3), x[1] * 2 + x[2]]))
    got = segment(T.tensor(x), [0, 2, 2, 5], [3, 0, 1, 1, 2], "max").data()
    torch.testing.assert_close(got, torch.stack([x[3], torch.zeros(3), x[2]]))
