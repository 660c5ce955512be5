"""Graph section of .mim files: builder, codec, interpreter (33 primitives + standard library),
sessions with variables, trace-to-file export (reference tests: io/mim/ops_test.go,
session_test.go, export_test.go)."""
import io
import math

import pytest
import torch
import torch.nn.functional as F

from mimir_b200 import nn
from mimir_b200 import tensor as T
from mimir_b200.io import export as X
from mimir_b200.io import graph as G
from mimir_b200.io import graph_run as R
from mimir_b200.io import mim
from mimir_b200.tensor import errors as E


def run_builder(b, inputs):
    model = mim.parse(b.serialize())
    return {k: v.data() for k, v in model.run(inputs).items()}


def one(b, x_spec, body, inputs):
    """Builds main(x...) -> body(...) and runs it."""
    refs = [b.input(n, dt, dims) for n, dt, dims in x_spec]
    outs = body(*refs)
    if isinstance(outs, G.Ref):
        outs = [outs]
    for i, o in enumerate(outs):
        b.output(f"y{i}", o)
    return run_builder(b, inputs)


def test_codec_roundtrip_and_magic():
    b = G.Builder()
    x = b.input("x", "f32", [G.Sym("n", 8), 4])
    w = b.weight("w", torch.arange(4.0))
    b.output("y", b.add(b.mul(x, w), 1.0))
    raw = b.finish().encode()
    assert raw[:4] == b"MB2G"
    g = G.Graph.decode(raw)
    assert [v.name for v in g.values][:2] == ["x", "w"]
    assert isinstance(g.values[0].dims[0], G.Sym) and g.values[0].dims[0].bound == 8
    assert G.Graph.decode(g.encode()).encode() == raw
    with pytest.raises(E.ErrUnsupported):
        G.Graph.decode(b"XXXX" + raw[4:])
    with pytest.raises(G.FormatError):
        G.Graph.decode(raw[:20])


def test_unary_and_binary_primitives():
    x = torch.tensor([[0.5, 2.0, 4.0], [1.0, 9.0, 16.0]])
    b = G.Builder()
    out = one(b, [("x", "f32", [2, 3])],
              lambda r: [b.neg(r), b.recip(r), b.sqrt(r), b.exp2(r), b.log2(r), b.sin(r), b.trunc(b.mul(r, 1.7)),
                         b.add(r, r), b.mul(r, 3.0), b.max(r, 2.0), b.pow(r, 2.0)], {"x": x})
    want = [-x, 1 / x, x.sqrt(), torch.exp2(x), torch.log2(x), torch.sin(x), torch.trunc(x * 1.7), x + x, x * 3,
            torch.clamp(x, min=2.0), x ** 2]
    for i, w in enumerate(want):
        torch.testing.assert_close(out[f"y{i}"], w)


def test_integer_and_logic_primitives():
    a = torch.tensor([7, -7, 9, 0], dtype=torch.int32)
    c = torch.tensor([2, 2, -4, 5], dtype=torch.int32)
    b = G.Builder()
    out = one(b, [("a", "i32", [4]), ("c", "i32", [4])],
              lambda x, y: [b.idiv(x, y), b.imod(x, y), b.cmplt(x, y), b.cmpeq(x, x),
                            b.and_(b.cmplt(x, y), b.cmpeq(y, y)), b.or_(b.cmplt(x, y), b.cmplt(y, x)),
                            b.xor(b.cmplt(x, y), b.cmplt(y, x)), b.where(b.cmplt(x, y), x, y),
                            b.cast(x, "f32"), b.cast(b.mul(b.cast(x, "f32"), 0.5), "i32")], {"a": a, "c": c})
    assert out["y0"].tolist() == [3, -3, -2, 0]          # truncating division
    assert out["y1"].tolist() == [1, -1, 1, 0]
    assert out["y2"].tolist() == [0, 1, 0, 1]
    assert out["y3"].tolist() == [1, 1, 1, 1]
    assert out["y4"].tolist() == [0, 1, 0, 1]
    assert out["y5"].tolist() == [1, 1, 1, 1]
    assert out["y6"].tolist() == [1, 1, 1, 1]
    assert out["y7"].tolist() == [2, -7, -4, 0]
    assert out["y8"].dtype == torch.float32
    assert out["y9"].tolist() == [3, -3, 4, 0]           # float -> int rounds toward zero


def test_shifts_and_bitcast():
    a = torch.tensor([1, -16, 5, 1 << 20], dtype=torch.int32)
    b = G.Builder()
    out = one(b, [("a", "i32", [4])],
              lambda x: [b.shl(x, 3), b.shr(x, 2), b.bitcast(b.cast(x, "f32"), "i32"),
                         b.bitcast(b.bitcast(b.cast(x, "f32"), "i32"), "f32")], {"a": a})
    assert out["y0"].tolist() == [8, -128, 40, 1 << 23]
    assert out["y1"].tolist() == [0, -4, 1, 1 << 18]                 # arithmetic shift on signed integers
    assert out["y2"].tolist() == a.float().view(torch.int32).tolist()
    assert out["y3"].tolist() == a.float().tolist()
    b = G.Builder()
    with pytest.raises(E.ErrDType):
        one(b, [("a", "i32", [4])], lambda x: b.bitcast(x, "i64"), {"a": a})
    g = G.Graph(values=[G.Value("x", "input", "f32", [2]), G.Value("y", "temp", "f32", [2])])
    g.main.inputs = [0]
    g.main.ops.append(G.Op("add", [0], [1]))                         # wrong arity is refused at load
    with pytest.raises(G.FormatError):
        g.check()


def test_integer_division_by_zero_is_an_error():
    b = G.Builder()
    with pytest.raises(E.ErrDivideByZero):
        one(b, [("a", "i32", [2])], lambda x: b.idiv(x, b.const(0, "i32", [])), {"a": torch.tensor([1, 2], dtype=torch.int32)})


def test_shape_primitives():
    x = torch.arange(24.0).reshape(2, 3, 4)
    b = G.Builder()
    out = one(b, [("x", "f32", [2, 3, 4])],
              lambda r: [b.reduce(r, "add", [1]), b.reduce(r, "max", [0, 2]), b.reduce(b.add(r, 1.0), "mul", [2]),
                         b.reshape(r, [6, 4]), b.expand(b.reshape(b.reduce(r, "add", [1, 2]), [2, 1]), [2, 5]),
                         b.permute(r, [2, 0, 1]), b.pad(r, [(0, 0), (1, 2), (0, 0)], -1.0),
                         b.shrink(r, [(0, -1), (1, 3), (2, 4)])], {"x": x})
    torch.testing.assert_close(out["y0"], x.sum(1, keepdim=True))
    torch.testing.assert_close(out["y1"], x.amax((0, 2), keepdim=True))
    torch.testing.assert_close(out["y2"], (x + 1).prod(2, keepdim=True))
    torch.testing.assert_close(out["y3"], x.reshape(6, 4))
    torch.testing.assert_close(out["y4"], x.sum((1, 2)).reshape(2, 1).expand(2, 5))
    torch.testing.assert_close(out["y5"], x.permute(2, 0, 1))
    torch.testing.assert_close(out["y6"], F.pad(x, [0, 0, 1, 2], value=-1.0))
    torch.testing.assert_close(out["y7"], x[:, 1:3, 2:4])


def test_gather_clamps_and_scatter_last_wins():
    data = torch.arange(12.0).reshape(4, 3)
    idx = torch.tensor([[3, 0], [9, -2]], dtype=torch.int32)      # 9 and -2 clamp to 3 and 0
    b = G.Builder()
    out = one(b, [("d", "f32", [4, 3]), ("i", "i32", [2, 2])],
              lambda d, i: [b.gather(d, i, 0), b.gather(d, b.const(1, "i32", [1]), 1)], {"d": data, "i": idx})
    torch.testing.assert_close(out["y0"], data[torch.tensor([[3, 0], [3, 0]])])
    torch.testing.assert_close(out["y1"], data[:, 1:2])
    b = G.Builder()
    upd = torch.tensor([[1.0, 1, 1], [2, 2, 2], [3, 3, 3]])
    out = one(b, [("d", "f32", [4, 3]), ("i", "i32", [3]), ("u", "f32", [3, 3])],
              lambda d, i, u: b.scatter(d, i, u, 0),
              {"d": data, "i": torch.tensor([2, 0, 2], dtype=torch.int32), "u": upd})
    want = data.clone()
    want[0], want[2] = upd[1], upd[2]
    torch.testing.assert_close(out["y0"], want)
    torch.testing.assert_close(data, torch.arange(12.0).reshape(4, 3))      # the input is not written


def test_const_and_dequantize():
    from mimir_b200.ops.quant import quantize_q4_0
    w = torch.randn(8, 64)
    raw = quantize_q4_0(w)
    q = mim.QuantizedTensor(mim.Q4_0, (8, 64), raw)
    b = G.Builder()
    qw = b.weight("w", q)
    x = b.input("x", "f32", [2, 64])
    b.output("c", b.const(3, "i32", [2, 2]))
    b.output("dq", b.dequantize(qw))
    b.output("y", b.call1("dequant_matmul.v1", [x, qw], "f32", [2, 8]))
    b.output("y8", b.call1("dequant_matmul_a8.v1", [x, qw], "f32", [2, 8]))
    xs = torch.randn(2, 64)
    out = run_builder(b, {"x": xs})
    assert out["c"].tolist() == [[3, 3], [3, 3]] and out["c"].dtype == torch.int32
    torch.testing.assert_close(out["dq"], q.dequantize())
    torch.testing.assert_close(out["y"], xs @ q.dequantize().T)
    assert torch.nn.functional.cosine_similarity(out["y8"].flatten(), out["y"].flatten(), dim=0) > 0.999
    b2 = G.Builder()
    with pytest.raises(E.ErrUnsupported):
        one(b2, [], lambda: b2.const(1 << 40, "i32", [1]), {})


def test_while_if_and_model_composites():
    b = G.Builder()
    n = b.input("n", "i32", [])
    # sum of 0..n-1 with a while loop; then an if on its parity
    i0, s0 = b.const(0, "i32", []), b.const(0, "i32", [])
    i, s, _ = b.while_([i0, s0, n], lambda i, s, n: b.cmplt(i, n),
                       lambda i, s, n: [b.add(i, 1), b.add(s, i), n])
    b.composite("double.v1", [("i32", [])], lambda v: b.add(v, v))
    odd = b.imod(s, 2)
    r = b.if_(odd, [s], lambda v: b.call1("double.v1", [v], "i32", []), lambda v: b.neg(v), [("i32", [])])[0]
    b.output("sum", s)
    b.output("r", r)
    model = mim.parse(b.serialize())
    for k in (0, 1, 4, 6, 7):
        out = model.run({"n": torch.tensor(k, dtype=torch.int32)})
        total = k * (k - 1) // 2
        assert out["sum"].item() == total
        assert out["r"].item() == (2 * total if total % 2 else -total)


def test_symbolic_dims_bind_and_bound():
    b = G.Builder()
    x = b.input("x", "f32", [G.Sym("batch", 4), 3])
    y = b.input("y", "f32", [G.Sym("batch", 4), 3])
    b.output("z", b.reshape(b.add(x, y), [G.Sym("batch", 4), 3, 1]))
    model = mim.parse(b.serialize())
    for n in (1, 4):
        out = model.run({"x": torch.ones(n, 3), "y": torch.ones(n, 3)})
        assert tuple(out["z"].shape) == (n, 3, 1)
    with pytest.raises(E.ErrShape):
        model.run({"x": torch.ones(5, 3), "y": torch.ones(5, 3)})          # above the bound
    with pytest.raises(E.ErrShape):
        model.run({"x": torch.ones(2, 3), "y": torch.ones(3, 3)})          # one symbol, two sizes
    with pytest.raises(E.ErrShape):
        model.run({"x": torch.ones(2, 3)})                                 # missing input
    with pytest.raises(E.ErrShape):
        model.run({"x": torch.ones(2, 3), "y": torch.ones(2, 3), "w": torch.ones(1)})
    with pytest.raises(E.ErrDType):
        model.run({"x": torch.ones(2, 3, dtype=torch.float64), "y": torch.ones(2, 3)})
    assert model.inputs[0][0] == "x" and model.outputs[0][0] == "z"


def _call(name, ins, out_spec, **attrs):
    b = G.Builder()
    refs = [b.input(f"i{j}", G.dtype_name(t.dtype), list(t.shape)) for j, t in enumerate(ins)]
    outs = b.call(name, refs, out_spec, **attrs)
    for j, o in enumerate(outs):
        b.output(f"y{j}", o)
    out = run_builder(b, {f"i{j}": t for j, t in enumerate(ins)})
    return [out[f"y{j}"] for j in range(len(outs))]


def test_stdlib_against_torch():
    torch.manual_seed(0)
    x = torch.randn(2, 5, 8)
    w, bias = torch.randn(6, 8), torch.randn(6)
    g, be = torch.randn(8), torch.randn(8)
    torch.testing.assert_close(_call("matmul.v1", [x, w.T.contiguous()], [("f32", [2, 5, 6])])[0], x @ w.T)
    torch.testing.assert_close(_call("linear.v1", [x, w, bias], [("f32", [2, 5, 6])])[0], F.linear(x, w, bias))
    for name, fn in [("sigmoid", torch.sigmoid), ("tanh", torch.tanh), ("erf", torch.erf), ("exp", torch.exp),
                     ("cos", torch.cos), ("silu", F.silu), ("gelu_erf", F.gelu),
                     ("gelu_tanh", lambda v: F.gelu(v, approximate="tanh"))]:
        torch.testing.assert_close(_call(name + ".v1", [x], [("f32", [2, 5, 8])])[0], fn(x))
    xp = x.abs() + 0.1
    torch.testing.assert_close(_call("log.v1", [xp], [("f32", [2, 5, 8])])[0], xp.log())
    torch.testing.assert_close(_call("rsqrt.v1", [xp], [("f32", [2, 5, 8])])[0], xp.rsqrt())
    torch.testing.assert_close(_call("swiglu.v1", [x, x * 2], [("f32", [2, 5, 8])])[0], F.silu(x) * x * 2)
    torch.testing.assert_close(_call("geglu.v1", [x, x * 2], [("f32", [2, 5, 8])])[0],
                               F.gelu(x, approximate="tanh") * x * 2)
    torch.testing.assert_close(_call("softmax.v1", [x], [("f32", [2, 5, 8])], axis=1)[0], x.softmax(1))
    torch.testing.assert_close(_call("log_softmax.v1", [x], [("f32", [2, 5, 8])])[0], x.log_softmax(-1))
    torch.testing.assert_close(_call("layer_norm.v1", [x, g, be], [("f32", [2, 5, 8])], eps=1e-5)[0],
                               F.layer_norm(x, (8,), g, be, 1e-5))
    rms = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * g
    torch.testing.assert_close(_call("rms_norm.v1", [x, g], [("f32", [2, 5, 8])], eps=1e-6)[0], rms)
    torch.testing.assert_close(_call("mean.v1", [x], [("f32", [2, 1, 8])], axes=[1])[0], x.mean(1, keepdim=True))
    torch.testing.assert_close(_call("variance.v1", [x], [("f32", [2, 5])], axes=[2], keepdims=False, correction=1)[0],
                               x.var(2))
    torch.testing.assert_close(_call("cumsum.v1", [x], [("f32", [2, 5, 8])], axis=1)[0], x.cumsum(1))
    torch.testing.assert_close(_call("cumsum.v1", [x], [("f32", [2, 5, 8])], axis=1, reverse=True, exclusive=True)[0],
                               x.flip(1).cumsum(1).flip(1) - x)
    table, idx = torch.randn(10, 4), torch.tensor([[1, 9], [0, 3]], dtype=torch.int32)
    torch.testing.assert_close(_call("embedding.v1", [table, idx], [("f32", [2, 2, 4])])[0], table[idx.long()])
    v, i = _call("top_k.v1", [x], [("f32", [2, 5, 3]), ("i64", [2, 5, 3])], k=3)
    tv, ti = x.topk(3, -1)
    torch.testing.assert_close(v, tv)
    assert torch.equal(i, ti)
    assert torch.equal(_call("argsort.v1", [x], [("i64", [2, 5, 8])], descending=True)[0],
                       torch.argsort(x, dim=-1, descending=True, stable=True))
    img, k4 = torch.randn(2, 3, 9, 9), torch.randn(4, 3, 3, 3)
    torch.testing.assert_close(
        _call("conv2d.v1", [img, k4, torch.zeros(4)], [("f32", [2, 4, 5, 5])], strides=[2, 2], pads=[1, 1, 1, 1])[0],
        F.conv2d(img, k4, None, 2, 1), rtol=1e-4, atol=1e-4)


def test_stdlib_attention_and_rope():
    torch.manual_seed(1)
    q, k, v = torch.randn(2, 4, 6, 16), torch.randn(2, 2, 9, 16), torch.randn(2, 2, 9, 16)
    got = _call("attention.v1", [q, k, v], [("f32", [2, 4, 6, 16])], causal=True)[0]
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    keep = torch.ones(6, 9, dtype=torch.bool).tril(3)
    want = F.scaled_dot_product_attention(q, kk, vv, attn_mask=keep)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    mask = torch.randn(6, 9)
    got = _call("attention.v1", [q, k, v, mask], [("f32", [2, 4, 6, 16])], scale=0.3)[0]
    torch.testing.assert_close(got, F.scaled_dot_product_attention(q, kk, vv, attn_mask=mask, scale=0.3),
                               rtol=1e-4, atol=1e-5)
    # version 2: soft cap and sinks
    sinks = torch.randn(4)
    got = _call("attention.v2", [q, k, v, mask, sinks], [("f32", [2, 4, 6, 16])], softcap=5.0)[0]
    s = torch.tanh((q @ kk.transpose(-1, -2)) / 4.0 / 5.0) * 5.0 + mask
    p = torch.softmax(torch.cat([s, sinks.reshape(1, 4, 1, 1).expand(2, 4, 6, 1)], -1), -1)[..., :9]
    torch.testing.assert_close(got, p @ vv, rtol=1e-4, atol=1e-5)
    # rope, half-split and interleaved layouts
    x, pos = torch.randn(2, 3, 5, 8), torch.arange(5, dtype=torch.int32) + 2
    inv = 10000.0 ** (-torch.arange(0, 8, 2).float() / 8)
    ang = pos.float()[:, None] * inv
    a, b_ = x[..., :4], x[..., 4:]
    want = torch.cat([a * ang.cos() - b_ * ang.sin(), a * ang.sin() + b_ * ang.cos()], -1)
    torch.testing.assert_close(_call("rope.v1", [x, pos], [("f32", [2, 3, 5, 8])])[0], want)
    e, o = x[..., 0::2], x[..., 1::2]
    want = torch.stack([e * ang.cos() - o * ang.sin(), e * ang.sin() + o * ang.cos()], -1).flatten(-2)
    torch.testing.assert_close(_call("rope.v1", [x, pos], [("f32", [2, 3, 5, 8])], interleaved=True)[0], want)


def test_unknown_call_and_opcode_are_refused_at_load():
    b = G.Builder()
    x = b.input("x", "f32", [2])
    b.output("y", b.call1("frobnicate.v7", [x], "f32", [2]))
    with pytest.raises(E.ErrUnsupported):
        b.finish()
    g = G.Graph(values=[G.Value("x", "input", "f32", [2])])
    g.main.inputs = [0]
    g.main.ops.append(G.Op("teleport", [0], [0]))
    with pytest.raises(E.ErrUnsupported):
        g.check()
    g.main.ops[0] = G.Op("neg", [5], [0])
    with pytest.raises(G.FormatError):
        g.check()


def _kv_cache_model():
    """A one-layer cache: each run scatters its rows at ``pos`` and returns the running sum of the
    cache rows, the way a decoder's key-value cache is written a few rows per run."""
    b = G.Builder()
    rows = b.input("rows", "f32", [G.Sym("t", 4), 3])
    pos = b.input("pos", "i32", [G.Sym("t", 4)])
    cache = b.variable("cache", "f32", [8, 3])
    steps = b.variable("steps", "i32", [], init=torch.tensor(10, dtype=torch.int32))
    new = b.scatter(cache, pos, rows, 0)
    b.update(cache, new)
    b.update(steps, b.add(steps, 1))
    b.output("total", b.reduce(new, "add", [0]))
    b.output("steps", b.add(steps, 0))
    return mim.parse(b.serialize())


def test_session_variables_persist_and_reset():
    model = _kv_cache_model()
    s = model.new_session()
    o1 = s.run({"rows": torch.ones(2, 3), "pos": torch.tensor([0, 1], dtype=torch.int32)})
    assert o1["total"].data().tolist() == [[2.0, 2.0, 2.0]] and o1["steps"].item() == 10
    o2 = s.run({"rows": torch.full((1, 3), 5.0), "pos": torch.tensor([4], dtype=torch.int32)})
    assert o2["total"].data().tolist() == [[7.0, 7.0, 7.0]] and o2["steps"].item() == 11
    assert s.variable("cache")[4].tolist() == [5.0, 5.0, 5.0]
    # an independent session starts from the initial values; so does this one after reset
    other = model.new_session()
    assert other.run({"rows": torch.ones(1, 3), "pos": torch.tensor([7], dtype=torch.int32)})["steps"].item() == 10
    s.reset()
    o3 = s.run({"rows": torch.ones(1, 3), "pos": torch.tensor([0], dtype=torch.int32)})
    assert o3["total"].data().tolist() == [[1.0, 1.0, 1.0]] and o3["steps"].item() == 10
    # Model.run is one run on fresh variables
    assert model.run({"rows": torch.ones(1, 3), "pos": torch.tensor([0], dtype=torch.int32)})["steps"].item() == 10


def test_failed_run_before_computing_changes_nothing():
    model = _kv_cache_model()
    s = model.new_session()
    s.run({"rows": torch.ones(2, 3), "pos": torch.tensor([0, 1], dtype=torch.int32)})
    with pytest.raises(E.ErrShape):
        s.run({"rows": torch.ones(5, 3), "pos": torch.tensor([0] * 5, dtype=torch.int32)})     # above the bound
    out = s.run({"rows": torch.ones(1, 3), "pos": torch.tensor([2], dtype=torch.int32)})
    assert out["total"].data().tolist() == [[3.0, 3.0, 3.0]] and out["steps"].item() == 11


def test_cancelled_run():
    b = G.Builder()
    n = b.input("n", "i32", [])
    i, _ = b.while_([b.const(0, "i32", []), n], lambda i, n: b.cmplt(i, n), lambda i, n: [b.add(i, 1), n])
    b.output("i", i)
    model = mim.parse(b.serialize())
    calls = [0]

    def cancel():
        calls[0] += 1
        return calls[0] > 50
    with pytest.raises(E.MimirError):
        model.run({"n": torch.tensor(1 << 20, dtype=torch.int32)}, cancel=cancel)


def test_no_graph_section():
    model = mim.parse(mim.serialize({"w": torch.ones(2)}))
    assert not model.has_graph()
    with pytest.raises(G.NoGraph):
        model.run({})


class _Net(nn.Module):
    def __init__(self):
        self.emb = nn.Embedding(20, 16)
        self.norm = nn.LayerNorm(16)
        self.rms = nn.RMSNorm(16)
        self.fc1 = nn.Linear(16, 32)
        self.fc2 = nn.Linear(32, 16, bias=False)
        self.drop = nn.Dropout(0.5)

    def forward(self, idx):
        x = self.emb(idx)
        h = self.fc2(T.gelu(self.fc1(self.norm(x))))
        x = self.rms(x + self.drop(h))
        q = T.permute(T.reshape(x, (x.shape[0], x.shape[1], 2, 8)), (0, 2, 1, 3))
        a = T.attention(q, q, q, causal=True)
        a = T.reshape(T.permute(a, (0, 2, 1, 3)), (x.shape[0], x.shape[1], 16))
        y = T.softmax(a - T.max_(a, dim=-1, keepdim=True), -1) * 2.0 + T.mean(a, dim=1, keepdim=True)
        return T.cat([y[:, :, :4], T.relu(y[:, :, 4:])], dim=2)


def test_export_module_roundtrip(tmp_path):
    nn.manual_seed(3)
    net = _Net()
    idx = T.tensor(torch.tensor([[1, 5, 7, 2, 0], [3, 3, 19, 8, 4]], dtype=torch.int32))
    net.eval()
    want = net(idx).data()
    path = tmp_path / "net.mim"
    g = X.export(path, net, idx, input_name="tokens", output_name="y", dynamic={"tokens": {0: ("batch", 8)}})
    with mim.open(path) as model:
        assert model.verify()
        assert "fc1.weight" in model.names() and "emb.weight" in model.names()
        assert model.inputs == [("tokens", "i32", [G.Sym("batch", 8), 5])]
        got = model.run({"tokens": idx})["y"].data()
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        # the symbolic batch axis takes another size
        idx3 = T.tensor(torch.randint(0, 20, (3, 5), dtype=torch.int32))
        torch.testing.assert_close(model.run({"tokens": idx3})["y"].data(), net(idx3).data(), rtol=1e-5, atol=1e-6)
        assert model.metadata["format.producer"] == "mimir_b200"
    assert any(o.opcode == "call" and o.attrs["name"] == "attention.v1" for o in g.main.ops)


def test_export_func_to_stream_and_unsupported_op():
    w = T.tensor(torch.randn(4))

    def f(a, b):
        return T.where(a < b, a * w, b / 2.0), T.sum_(T.exp(a) + T.sqrt(T.lgamma(T.abs_(b) + 1.0) + 1.0), dim=1)

    a, b_ = T.tensor(torch.randn(3, 4)), T.tensor(torch.randn(3, 4))
    buf = io.BytesIO()
    with pytest.raises(E.ErrUnsupported) as exc:
        X.export_func(buf, f, [a, b_])
    assert "lgamma" in str(exc.value)

    def f2(a, b):
        return T.where(a < b, a * w, b / 2.0), T.sum_(T.exp(a) + T.sqrt(T.abs_(b) + 1.0), dim=1)
    X.export_func(buf, f2, [a, b_], input_names=["a", "b"], output_names=["sel", "s"])
    model = mim.parse(buf.getvalue())
    got = model.run({"a": a, "b": b_})
    want = f2(a, b_)
    torch.testing.assert_close(got["sel"].data(), want[0].data())
    torch.testing.assert_close(got["s"].data(), want[1].data())


def test_export_cnn(tmp_path):
    nn.manual_seed(5)
    net = nn.Sequential(nn.Conv2d(1, 4, 3, padding=1), nn.ReLU(), nn.Conv2d(4, 8, 3, stride=2), nn.Tanh(), nn.Flatten(),
                        nn.Linear(8 * 3 * 3, 10))
    x = T.tensor(torch.randn(2, 1, 8, 8))
    path = tmp_path / "cnn.mim"
    X.export(path, net, x)
    with mim.open(path) as model:
        torch.testing.assert_close(model.run({"input": x})["output"].data(), net(x).data(), rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_exported_model_runs_on_the_gpu(tmp_path):
    """The interpreter computes on the device of its inputs; weights move there once."""
    nn.manual_seed(3)
    net = _Net()
    idx = T.from_torch(torch.tensor([[1, 5, 7, 2, 0], [3, 3, 19, 8, 4]], dtype=torch.int32))
    path = tmp_path / "net.mim"
    X.export(path, net, idx, input_name="tokens", output_name="y")
    with mim.open(path) as model:
        cpu = model.run({"tokens": idx})["y"].data()
        s = model.new_session()
        gpu = s.run({"tokens": idx.data().cuda()})["y"].data()
        assert gpu.is_cuda
        torch.testing.assert_close(gpu.cpu(), cpu, rtol=1e-4, atol=1e-5)
    kv = _kv_cache_model().new_session()
    out = kv.run({"rows": torch.ones(2, 3).cuda(), "pos": torch.tensor([0, 1], dtype=torch.int32).cuda()})
    assert out["total"].data().cpu().tolist() == [[2.0, 2.0, 2.0]]
    out = kv.run({"rows": torch.ones(1, 3).cuda(), "pos": torch.tensor([5], dtype=torch.int32).cuda()})
    assert out["total"].data().cpu().tolist() == [[3.0, 3.0, 3.0]]


@pytest.mark.gpu
def test_repeated_shapes_are_replayed_from_a_recording(tmp_path):
    """Third and later runs of one input shape replay a CUDA graph; values, variables and a change of
    shape behave as in a plain pass."""
    nn.manual_seed(4)
    net = _Net()
    net.eval()
    path = tmp_path / "net.mim"
    idx = T.from_torch(torch.randint(0, 20, (2, 5), dtype=torch.int32))
    X.export(path, net, idx, input_name="tokens", output_name="y", dynamic={"tokens": {0: ("batch", 8)}})
    with mim.open(path) as model:
        s = model.new_session()
        for trial in range(5):
            t = torch.randint(0, 20, (2, 5), dtype=torch.int32)
            got = s.run({"tokens": t.cuda()})["y"].data().cpu()
            torch.testing.assert_close(got, net(T.from_torch(t)).data(), rtol=1e-4, atol=1e-5)
        assert any(isinstance(r, tuple) for r in s._recs.values())
        t3 = torch.randint(0, 20, (3, 5), dtype=torch.int32)      # another shape: its own recording
        torch.testing.assert_close(s.run({"tokens": t3.cuda()})["y"].data().cpu(), net(T.from_torch(t3)).data(),
                                   rtol=1e-4, atol=1e-5)
    kv, ref = _kv_cache_model().new_session(), _kv_cache_model().new_session()
    ref.replay = False
    for step in range(6):
        feed = {"rows": torch.full((1, 3), float(step + 1)), "pos": torch.tensor([step % 4], dtype=torch.int32)}
        a = kv.run({k: v.cuda() for k, v in feed.items()})
        b = ref.run({k: v.cuda() for k, v in feed.items()})
        assert torch.equal(a["total"].data(), b["total"].data()) and a["steps"].item() == b["steps"].item() == 10 + step
    assert any(isinstance(r, tuple) for r in kv._recs.values()) and not ref._recs
    torch.testing.assert_close(kv.variable("cache").cpu(), ref.variable("cache").cpu())
    kv.reset()
    out = kv.run({"rows": torch.ones(1, 3).cuda(), "pos": torch.tensor([0], dtype=torch.int32).cuda()})
    assert out["total"].data().cpu().tolist() == [[1.0, 1.0, 1.0]] and out["steps"].item() == 10
