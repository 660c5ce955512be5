"""More of the reference's committed float64 oracle files (testdata/golden/*.mim; the cases and their
meaning are in tools/golden/gen.py): gradients of the tensor ops, scans, sorting, Fourier transforms,
linear algebra and the rest of the forward cases."""
import math
import os

import pytest
import torch

from _refdir import reference_dir

GOLD = os.environ.get("MIMIR_GOLDEN_DIR") or os.path.join(reference_dir() or "", "testdata", "golden")
pytestmark = pytest.mark.skipif(not os.path.isdir(GOLD), reason="reference golden files not found")


def _open(name):
    from mimir_b200.io import mim
    return mim.open(os.path.join(GOLD, name + ".mim"))


def _inputs(m, case):
    ins, i = [], 0
    while f"{case}/in{i}" in m:
        ins.append(m.tensor(f"{case}/in{i}").clone())
        i += 1
    return ins


def _run_case(m, case, fn, tol=2e-5, int_inputs=()):
    """Forward value and, where the file has them, the gradients of sum(out * gout) with respect to
    every input that has a ``grad<i>`` entry."""
    import mimir_b200.tensor as T
    from mimir_b200.tensor.autograd import Param, backward
    ins = _inputs(m, case)
    want = m.tensor(f"{case}/out")
    diff = [i for i in range(len(ins)) if f"{case}/grad{i}" in m]
    params, args = {}, []
    for i, x in enumerate(ins):
        if i in diff:
            params[i] = Param(x.clone())
            args.append(params[i].value())
        else:
            args.append(T.tensor(x, dtype=x.dtype, device=T.CPU()))
    out = fn(*args)
    assert out.err is None, (case, out.err)
    if diff:
        gout = T.tensor(m.tensor(f"{case}/gout").clone(), device=T.CPU())
        backward(T.sum_(out * T.reshape(gout, tuple(out.shape))))
    got = out.data()
    assert tuple(got.shape) == tuple(want.shape) or got.numel() == want.numel(), (case, got.shape, want.shape)
    scale = max(1.0, float(want.float().abs().max())) if want.numel() else 1.0
    assert torch.allclose(got.reshape(want.shape).float(), want.float(), rtol=tol, atol=tol * scale), case
    for i in diff:
        g, wg = params[i].grad(), m.tensor(f"{case}/grad{i}")
        assert g is not None, f"{case}: no gradient for input {i}"
        gs = max(1.0, float(wg.abs().max()))
        assert torch.allclose(g.data().float(), wg, rtol=tol * 5, atol=tol * 5 * gs), f"{case}/grad{i}"


def test_gradients_of_tensor_ops():
    import mimir_b200.tensor as T
    G = {
        "exp": T.exp, "log": T.log, "sin": T.sin, "sqrt": T.sqrt, "recip": T.recip, "sigmoid": T.sigmoid, "tanh": T.tanh,
        "gelu": T.gelu, "silu": T.silu, "relu": T.relu, "abs": T.abs_,
        "add": T.add, "sub": T.sub, "mul": T.mul, "div": T.div, "maximum": T.maximum, "minimum": T.minimum,
        "where": lambda c, x, y: T.where(T.logical_not(T.equal(c, 0.0)), x, y),
        "sum_axes02": lambda x: T.sum_(x, (0, 2)), "max_axis2": lambda x: T.max_(x, 2), "mean_last": lambda x: T.mean(x, -1),
        "var_axis1": lambda x: T.var(x, 1), "softmax_axis1": lambda x: T.softmax(x, 1), "log_softmax": lambda x: T.log_softmax(x, -1),
        "permute_reshape": lambda x: T.reshape(T.permute(x, (2, 0, 1)), (4, 6)),
        "expand": lambda x: T.expand(x, (2, 3, 4)),
        "pad": lambda x: T.pad(x, ((1, 0), (2, 1)), -1.0),
        "shrink_flip_add": lambda x: T.flip(T.shrink(x, ((1, 4), (2, 6))), (0,)) + T.shrink(x, ((0, 3), (0, 4))),
        "unfold_overlap": lambda x: T.windows(x, 1, 4, 2), "unfold_gapped": lambda x: T.windows(x, 1, 2, 3),
        "cat": lambda x, y: T.cat([x, y], 1),
        "matmul_batched": T.matmul, "matmul_vec_mat": T.matmul,
        "gather": lambda x, i: T.gather(x, 1, i),
        "scatter_add": lambda x, i, s: T.scatter_add(x, 0, i, s),
        "conv2d": lambda x, w, b: T.conv2d(x, w, b, padding=1),
        "conv2d_grouped": lambda x, w: T.conv2d(x, w, None, stride=2, padding=1, dilation=2, groups=2),
        "max_pool2d": lambda x: T.max_pool2d(x, 2), "max_pool2d_padded": lambda x: T.max_pool2d(x, 3, 2, 1),
        "avg_pool2d": lambda x: T.avg_pool2d(x, 3, 1, 1),
        "layer_norm": lambda x, g, b: T.layer_norm(x, g, b, 1e-5),
        "attention": lambda q, k, v: T.matmul(T.softmax(T.matmul(q, T.transpose(k, -1, -2)) * (1 / math.sqrt(8)), -1), v),
        "mlp": lambda x, w1, b1, w2, b2: T.log_softmax(T.matmul(T.gelu(T.matmul(x, w1) + b1), w2) + b2, -1),
    }
    with _open("grads") as m:
        cases = sorted({n.split("/")[0] for n in m.names()})
        assert sorted(G) == cases, sorted(set(cases) ^ set(G))
        for case in cases:
            _run_case(m, case, G[case])


def test_scans():
    import mimir_b200.tensor as T
    S = {
        "cumsum_axis1": lambda x: T.cumsum(x, 1), "cumsum_last": lambda x: T.cumsum(x, -1), "cumsum_int": lambda x: T.cumsum(x, 1),
        "cummax_axis1": lambda x: T.cummax(x, 1), "cummax_axis0": lambda x: T.cummax(x, 0),
        "cummax_indices": lambda x: T.cummax_indices(x, 1),
        "logcumsumexp_last": lambda x: T.logcumsumexp(x, -1), "logcumsumexp_large": lambda x: T.logcumsumexp(x, 0),
    }
    with _open("scan") as m:
        assert sorted(S) == sorted({n.split("/")[0] for n in m.names()})
        for case, fn in S.items():
            _run_case(m, case, fn)


def test_sorting_fourier_and_linear_algebra():
    import mimir_b200.tensor as T
    eye = lambda x: T.tensor(torch.eye(x.shape[-1]))  # noqa: E731
    shift = lambda x, by: x + eye(x) * float(by)  # noqa: E731
    spd = lambda x, by: T.matmul(x, T.transpose(x, -1, -2)) + eye(x) * float(by)  # noqa: E731
    flat = lambda *ts: T.cat([T.reshape(t, (-1,)) for t in ts], 0)  # noqa: E731

    def svd_parts(x):
        u, s, vh = T.svd(x)
        return flat(s, u * u, vh * vh)

    def eigh_parts(x):
        w, v = T.eigh(x + T.transpose(x, -1, -2))
        return flat(w, v * v)
    L = {
        "sort_values": lambda x: T.sort(x, 1)[0], "sort_descending_indices": lambda x: T.cast(T.sort(x, 1, True)[1], T.int32),
        "argsort_axis0": lambda x: T.argsort(x, 0), "topk_values": lambda x: T.topk(x, 3, 1)[0],
        "topk_smallest_indices": lambda x: T.cast(T.topk(x, 2, 0, largest=False)[1], T.int32),
        "fft": lambda x: T.fft(x, 1), "fft_bluestein": lambda x: T.fft(x, 0), "ifft": lambda x: T.ifft(x, -1),
        "rfft": lambda x: T.rfft(x, -1), "irfft": lambda x: T.irfft(x, -1, 8), "irfft_odd_padded": lambda x: T.irfft(x, 0, 9),
        "cholesky": lambda x: T.cholesky(spd(x, 2)),
        "solve": lambda a, b: T.solve(shift(a, 3), b), "solve_vector": lambda a, b: T.solve(shift(a, 3), b),
        "triangular_solve_lower": lambda a, b: T.triangular_solve(shift(a, 3), b, upper=False),
        "triangular_solve_upper": lambda a, b: T.triangular_solve(shift(a, 3), b, upper=True),
        "inv": lambda x: T.inv(shift(x, 3)), "det": lambda x: T.det(shift(x, 1)),
        "slogdet_sign": lambda x: T.slogdet(x)[0], "slogdet_logabsdet": lambda x: T.slogdet(x)[1],
        "qr_tall": lambda x: flat(*T.qr(x)), "qr_wide": lambda x: flat(*T.qr(x)),
        "svd_tall": svd_parts, "svd_wide": svd_parts, "eigh": eigh_parts,
    }
    with _open("linalg") as m:
        assert sorted(L) == sorted({n.split("/")[0] for n in m.names()})
        for case, fn in L.items():
            _run_case(m, case, fn, tol=1e-4)
    # what the decompositions promise beyond the oracle values
    a = T.tensor(torch.randn(3, 5, 4))
    q, r = T.qr(a)
    assert torch.allclose(T.matmul(q, r).data(), a.data(), atol=1e-5)
    with pytest.raises(T.ErrSingular):
        T.cholesky(T.tensor(torch.tensor([[1.0, 2.0], [2.0, 1.0]]))).data()
    assert isinstance(T.inv(T.tensor(torch.ones(2, 3))).err, T.ErrShape)
    assert isinstance(T.fft(T.tensor(torch.ones(4, 3))).err, T.ErrShape)


def test_remaining_forward_cases():
    import mimir_b200.tensor as T
    O = {
        "cast_f2i": lambda x: T.cast(x, T.int32), "cast_i2f": lambda x: T.cast(x, T.float32),
        "equal": T.equal, "less": T.less, "greater": T.greater, "exp2": T.exp2, "log2": T.log2, "fmod": T.fmod, "fmod_int": T.fmod,
        "expand": lambda x: T.expand(x, (2, 3, 4)), "flip": lambda x: T.flip(x, (0, 1)),
        "gather": lambda x, i: T.gather(x, 1, i), "scatter_add": lambda x, i, s: T.scatter_add(x, 0, i, s),
        "layer_norm": lambda x, g, b: T.layer_norm(x, g, b, 1e-5),
        "attention": lambda q, k, v: T.matmul(T.softmax(T.matmul(q, T.transpose(k, -1, -2)) * (1 / math.sqrt(8)), -1), v),
        "matmul_mat_vec": T.matmul, "matmul_vec_mat": T.matmul, "matmul_transposed": lambda x, y: T.matmul(T.transpose(x, 0, 1), y),
        "mlp": lambda x, w1, b1, w2, b2: T.log_softmax(T.matmul(T.gelu(T.matmul(x, w1) + b1), w2) + b2, -1),
        "pad": lambda x: T.pad(x, ((1, 0), (2, 1)), -1.0), "permute_reshape": lambda x: T.reshape(T.permute(x, (2, 0, 1)), (4, 6)),
        "shrink": lambda x: T.shrink(x, ((1, 4), (2, 6))),
        "shrink_flip_add": lambda x: T.flip(T.shrink(x, ((1, 4), (2, 6))), (0,)) + T.shrink(x, ((0, 3), (0, 4))),
        "sum_int": lambda x: T.sum_(x, 1),
    }
    with _open("ops") as m:
        have = {n.split("/")[0] for n in m.names()}
        for case, fn in O.items():
            assert case in have, case
            ins = _inputs(m, case)
            want = m.tensor(f"{case}/out")
            got = fn(*[T.tensor(x, dtype=x.dtype, device=T.CPU()) for x in ins]).data()
            assert tuple(got.shape) == tuple(want.shape), (case, got.shape, want.shape)
            if want.dtype.is_floating_point:
                assert torch.allclose(got.float(), want, rtol=2e-5, atol=2e-6 * max(1.0, float(want.abs().max()))), case
            else:
                assert torch.equal(got.to(want.dtype), want), case


RNN_CASES = {
    # name: (kind, input size, hidden size, layers, bidirectional, batch_first, relu, bias)
    "rnn_tanh": ("rnn", 3, 4, 1, False, False, False, True),
    "rnn_relu_2layer_bidir": ("rnn", 3, 4, 2, True, False, True, True),
    "lstm": ("lstm", 3, 4, 1, False, False, False, True),
    "lstm_2layer_bidir": ("lstm", 3, 4, 2, True, False, False, True),
    "lstm_batch_first_unbiased": ("lstm", 3, 4, 1, False, True, False, False),
    "lstm_unbatched": ("lstm", 3, 4, 1, False, False, False, True),
    "gru": ("gru", 3, 4, 1, False, False, False, True),
    "gru_2layer_bidir_batch_first": ("gru", 3, 4, 2, True, True, False, True),
}


def test_recurrent_layers():
    """rnn.mim: outputs, final states and the gradients of every input, initial state and weight, for
    stacked / bidirectional / batch-first / unbiased / unbatched layers with PyTorch's weight layout."""
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from mimir_b200.tensor.autograd import Param, backward
    with _open("rnn") as m:
        assert sorted(RNN_CASES) == sorted({n.split("/")[0] for n in m.names()})
        for case, (kind, n_in, hidden, layers, bidir, batch_first, relu, bias) in RNN_CASES.items():
            ins = _inputs(m, case)
            ns = 2 if kind == "lstm" else 1
            kw = dict(bidirectional=bidir, batch_first=batch_first, bias=bias)
            layer = {"rnn": lambda: nn.RNN(n_in, hidden, layers, relu=relu, **kw), "lstm": lambda: nn.LSTM(n_in, hidden, layers, **kw),
                     "gru": lambda: nn.GRU(n_in, hidden, layers, **kw)}[kind]()
            weights = ins[1 + ns:]
            per = 4 if bias else 2
            order = []
            for k in range(layers * (2 if bidir else 1)):
                order += [layer.w_ih[k], layer.w_hh[k]] + ([layer.b_ih[k], layer.b_hh[k]] if bias else [])
            assert len(order) == len(weights) and per * len(layer.w_ih) == len(weights)
            for p, w in zip(order, weights):
                assert tuple(p.shape) == tuple(w.shape), case
                p.set(w.clone())
            x = Param(ins[0].clone())
            states = [Param(s.clone()) for s in ins[1:1 + ns]]
            res = layer.run(x.value(), *[s.value() for s in states])
            joined = T.cat([T.reshape(r, (-1,)) for r in res], 0)
            gout = T.tensor(m.tensor(f"{case}/gout").clone(), device=T.CPU())
            backward(T.sum_(joined * gout))
            assert torch.allclose(joined.data(), m.tensor(f"{case}/out"), rtol=2e-5, atol=2e-6), case
            assert torch.allclose(res[0].data(), m.tensor(f"{case}/output"), rtol=2e-5, atol=2e-6), case
            assert torch.allclose(res[1].data(), m.tensor(f"{case}/h_n"), rtol=2e-5, atol=2e-6), case
            for i, p in enumerate([x] + states + order):
                want = m.tensor(f"{case}/grad{i}")
                assert torch.allclose(p.grad().data(), want, rtol=1e-4, atol=1e-5), f"{case}/grad{i}"


def _run_module(m, case, fn, tol=2e-5):
    """``fn(ins)`` builds the layer from the case's inputs and returns the output with a map from
    input index to the ``Param`` whose gradient the file holds as ``grad<i>``."""
    import mimir_b200.tensor as T
    from mimir_b200.tensor.autograd import backward
    ins = _inputs(m, case)
    want = m.tensor(f"{case}/out")
    out, graders = fn(ins)
    assert out.err is None, (case, out.err)
    gout = T.tensor(m.tensor(f"{case}/gout").clone(), device=T.CPU())
    backward(T.sum_(out * T.reshape(gout, tuple(out.shape))))
    got = out.data()
    scale = max(1.0, float(want.abs().max()))
    assert torch.allclose(got.reshape(want.shape).float(), want.float(), rtol=tol, atol=tol * scale), case
    checked = 0
    for i in range(len(ins)):
        if f"{case}/grad{i}" not in m:
            continue
        assert i in graders, f"{case}: input {i} has a gradient in the file and no parameter here"
        g, wg = graders[i].grad(), m.tensor(f"{case}/grad{i}")
        assert g is not None, f"{case}: no gradient for input {i}"
        gs = max(1.0, float(wg.abs().max()))
        assert torch.allclose(g.data().float().reshape(wg.shape), wg, rtol=tol * 5, atol=tol * 5 * gs), f"{case}/grad{i}"
        checked += 1
    assert checked, case
    return got


def _set(params, values):
    assert len(params) == len(values)
    for p, v in zip(params, values):
        p.set(v)
    return {i + 1: p for i, p in enumerate(params)}


def test_attention_layers_and_blocks():
    """The cases of attention.mim that go through layers: rotary embeddings, RMS norm, masked and
    multi-head attention, the GPT-2 and Llama decoder blocks and the encoder layer, with the gradient
    of every parameter."""
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from mimir_b200.tensor.autograd import Param
    with _open("attention") as m:
        _run_case(m, "sdpa_bool_mask", lambda q, k, v, keep: T.attention(q, k, v, mask=T.logical_not(T.equal(keep, 0.0))))
        _run_case(m, "sdpa_mask", lambda q, k, v, mask: T.attention(q, k, v, mask=mask))
        for case, kw in {"sdpa": {}, "sdpa_causal": dict(causal=True), "sdpa_gqa": dict(causal=True, causal_offset=2),
                         "sdpa_causal_offset": dict(causal=True, causal_offset=4), "sdpa_scale": dict(scale=0.3)}.items():
            _run_case(m, case, lambda q, k, v, kw=kw: T.attention(q, k, v, **kw))
        _run_case(m, "rms_norm", lambda x, w: T.rms_norm(x, w, 1e-6))

        def rms_default(ins):
            layer = nn.RMSNorm(6)
            x = Param(ins[0])
            g = _set([layer.weight], ins[1:])
            return layer(x.value()), {0: x, **g}
        _run_module(m, "rms_norm_default_eps", rms_default)

        _run_case(m, "rope_neox", lambda x: nn.RotaryEmbedding(8, 10000.0).apply(x, 3))
        _run_case(m, "rope_interleaved", lambda x: nn.RotaryEmbedding(8, 10000.0, interleaved=True).apply(x, 3))
        scaling = dict(type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_context=64)
        _run_case(m, "rope_partial_scaled", lambda x: nn.RotaryEmbedding(8, 10000.0, scaling=scaling).apply(x, 2))

        def mha(ins):
            layer = nn.MultiheadAttention(8, 2)
            x = Param(ins[0])
            xv = x.value()
            ps = [layer.in_proj_weight, layer.in_proj_bias, layer.out_proj.weight, layer.out_proj.bias]
            g = _set(ps, ins[1:])
            return layer(xv, xv, xv), {0: x, **g}
        _run_module(m, "multihead_attention", mha)

        def mha_causal(ins):
            layer = nn.MultiheadAttention(8, 4)
            q, k, v = (Param(t) for t in ins[:3])
            ps = [layer.in_proj_weight, layer.in_proj_bias, layer.out_proj.weight, layer.out_proj.bias]
            g = {i + 3: p for i, p in enumerate(ps)}
            for p, val in zip(ps, ins[3:]):
                p.set(val)
            return layer(q.value(), k.value(), v.value(), causal=True), {0: q, 1: k, 2: v, **g}
        _run_module(m, "multihead_attention_causal", mha_causal)

        def gpt2(ins):
            b = nn.DecoderBlock(8, 2, style="gpt2")
            x = Param(ins[0])
            ps = [b.norm1.weight, b.norm1.bias, b.attn.qkv.weight, b.attn.qkv.bias, b.attn.out.weight, b.attn.out.bias,
                  b.norm2.weight, b.norm2.bias, b.mlp.up.weight, b.mlp.up.bias, b.mlp.down.weight, b.mlp.down.bias]
            g = _set(ps, ins[1:])
            return b(x.value()), {0: x, **g}
        _run_module(m, "decoder_block_gpt2", gpt2)

        def llama(ins):
            b = nn.DecoderBlock(16, 4, hidden=24, kv_heads=2, style="llama", rope=nn.RotaryEmbedding(4, 10000.0))
            x = Param(ins[0])
            ps = [b.norm1.weight, b.attn.qkv.weight, b.attn.out.weight, b.norm2.weight,
                  b.mlp.gate.weight, b.mlp.up.weight, b.mlp.down.weight]
            g = _set(ps, ins[1:])
            return b(x.value()), {0: x, **g}
        _run_module(m, "decoder_block_llama", llama)

        def encoder(ins):
            l = nn.TransformerEncoderLayer(8, 2, 16).eval()
            x = Param(ins[0])
            ps = [l.attn.qkv.weight, l.attn.qkv.bias, l.attn.out.weight, l.attn.out.bias, l.mlp.up.weight, l.mlp.up.bias,
                  l.mlp.down.weight, l.mlp.down.bias, l.norm1.weight, l.norm1.bias, l.norm2.weight, l.norm2.bias]
            g = _set(ps, ins[1:])
            return l(x.value()), {0: x, **g}
        _run_module(m, "transformer_encoder_layer", encoder)


def test_layers_of_nn_mim():
    """linear, layer norm, batch norm (with its running statistics), embedding and cross-entropy over
    an extra axis, with gradients."""
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from mimir_b200.nn import loss as L
    from mimir_b200.tensor.autograd import Param
    with _open("nn") as m:
        def linear(ins):
            layer = nn.Linear(6, 3)
            x = Param(ins[0])
            g = _set([layer.weight, layer.bias], ins[1:])
            return layer(x.value()), {0: x, **g}
        _run_module(m, "linear", linear)

        def layer_norm(ins):
            layer = nn.LayerNorm(8)
            x = Param(ins[0])
            g = _set([layer.weight, layer.bias], ins[1:])
            return layer(x.value()), {0: x, **g}
        _run_module(m, "layer_norm", layer_norm)

        for case, cls, ch in (("batch_norm1d", nn.BatchNorm1d, 5), ("batch_norm2d", nn.BatchNorm2d, 3)):
            holder = {}

            def bn(ins, cls=cls, ch=ch, holder=holder):
                layer = holder["layer"] = cls(ch)
                x = Param(ins[0])
                g = _set([layer.weight, layer.bias], ins[1:])
                return layer(x.value()), {0: x, **g}
            _run_module(m, case, bn)
            layer = holder["layer"]
            for name in ("running_mean", "running_var"):
                got, want = getattr(layer, name).value().data(), m.tensor(f"{case}/{name}")
                assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), (case, name)

        def bn_eval(ins):
            layer = nn.BatchNorm2d(3).eval()
            layer.running_mean.set(ins[1])
            layer.running_var.set(ins[2])
            x = Param(ins[0])
            layer.weight.set(ins[3])
            layer.bias.set(ins[4])
            return layer(x.value()), {0: x, 3: layer.weight, 4: layer.bias}
        _run_module(m, "batch_norm_eval", bn_eval)

        def embedding(ins):
            layer = nn.Embedding(5, 4)
            layer.weight.set(ins[1])
            return layer(T.tensor(ins[0], dtype=ins[0].dtype, device=T.CPU())), {1: layer.weight}
        _run_module(m, "embedding", embedding)

        for case, fn in {"cross_entropy_kdim": L.cross_entropy, "cross_entropy": L.cross_entropy, "nll": L.nll,
                         "mse": L.mse, "l1": L.l1, "huber": L.huber, "bce_with_logits": L.bce_with_logits}.items():
            _run_case(m, case, fn)


def test_graph_layers():
    """gnn.mim: aggregation of edge messages, the softmax over incoming edges, and the GCN / GraphSAGE /
    GAT convolutions with the gradient of every parameter."""
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from mimir_b200.tensor.autograd import Param
    with _open("gnn") as m:
        nodes = m.tensor("gcn/in0").shape[0]

        def graph(ei):
            return nn.Graph.from_edge_index(nodes, ei)

        for reduce in ("sum", "mean", "max"):
            def agg(ins, reduce=reduce):
                msg = Param(ins[0])
                return getattr(graph(ins[1]), reduce)(msg.value()), {0: msg}
            _run_module(m, f"aggregate_{reduce}", agg)

        def edge_softmax(ins):
            s = Param(ins[0])
            return graph(ins[1]).softmax(s.value()), {0: s}
        _run_module(m, "edge_softmax", edge_softmax)

        def gcn(ins):
            c = nn.GCNConv(5, 4)
            x = Param(ins[0])
            c.weight.set(ins[2]); c.bias.set(ins[3])
            return c.convolve(graph(ins[1]), x.value()), {0: x, 2: c.weight, 3: c.bias}
        _run_module(m, "gcn", gcn)

        def sage(ins):
            c = nn.SAGEConv(5, 4)
            x = Param(ins[0])
            c.neighbors.weight.set(ins[2]); c.neighbors.bias.set(ins[3]); c.root.weight.set(ins[4])
            return c.convolve(graph(ins[1]), x.value()), {0: x, 2: c.neighbors.weight, 3: c.neighbors.bias, 4: c.root.weight}
        _run_module(m, "sage", sage)

        for case, mean_heads in (("gat_concat", False), ("gat_mean", True)):
            def gat(ins, mean_heads=mean_heads):
                c = nn.GATConv(5, 3, heads=2, mean_heads=mean_heads)
                x = Param(ins[0])
                for p, v in zip((c.weight, c.att_src, c.att_dst, c.bias), ins[2:]):
                    p.set(v)
                return c.convolve(graph(ins[1]), x.value()), {0: x, 2: c.weight, 3: c.att_src, 4: c.att_dst, 5: c.bias}
            _run_module(m, case, gat)


def test_distributions_and_special_functions():
    """distributions.mim: log-probabilities, entropies, variances, CDFs and KL divergences of the eleven
    families, and the special functions under them, with the gradient of every float input."""
    import mimir_b200.tensor as T
    from mimir_b200 import distributions as D
    two = lambda cls: (lambda a, b, c, d: D.kl(cls(a, b), cls(c, d)))  # noqa: E731
    one = lambda make: (lambda a, b: D.kl(make(a), make(b)))  # noqa: E731
    cases = {
        "normal_log_prob": lambda m, s, x: D.Normal(m, s).log_prob(x),
        "normal_entropy": lambda m, s: D.Normal(m, s).entropy(),
        "normal_cdf": lambda m, s, x: D.Normal(m, s).cdf(x),
        "normal_icdf": lambda m, s, p: D.Normal(m, s).icdf(p),
        "normal_kl": two(D.Normal),
        "mvn_log_prob": lambda m, l, x: D.MultivariateNormal(m, scale_tril=l).log_prob(x),
        "mvn_entropy": lambda m, l: D.MultivariateNormal(m, scale_tril=l).entropy(),
        "mvn_variance": lambda m, l: D.MultivariateNormal(m, scale_tril=l).variance(),
        "mvn_kl": lambda a, b, c, d: D.kl(D.MultivariateNormal(a, scale_tril=b), D.MultivariateNormal(c, scale_tril=d)),
        "bernoulli_log_prob": lambda l, x: D.Bernoulli(logits=l).log_prob(x),
        "bernoulli_probs_log_prob": lambda p, x: D.Bernoulli(probs=p).log_prob(x),
        "bernoulli_entropy": lambda l: D.Bernoulli(logits=l).entropy(),
        "bernoulli_kl": one(lambda p: D.Bernoulli(probs=p)),
        "categorical_log_prob": lambda l, x: D.Categorical(logits=l).log_prob(x),
        "categorical_probs_log_prob": lambda p, x: D.Categorical(probs=p).log_prob(x),
        "categorical_entropy": lambda l: D.Categorical(logits=l).entropy(),
        "categorical_kl": one(lambda l: D.Categorical(logits=l)),
        "uniform_log_prob": lambda lo, hi, x: D.Uniform(lo, hi).log_prob(x),
        "uniform_entropy": lambda lo, hi: D.Uniform(lo, hi).entropy(),
        "uniform_kl": two(D.Uniform),
        "exponential_log_prob": lambda r, x: D.Exponential(r).log_prob(x),
        "exponential_entropy": lambda r: D.Exponential(r).entropy(),
        "exponential_kl": one(D.Exponential),
        "laplace_log_prob": lambda m, s, x: D.Laplace(m, s).log_prob(x),
        "laplace_entropy": lambda m, s: D.Laplace(m, s).entropy(),
        "laplace_kl": two(D.Laplace),
        "gamma_log_prob": lambda a, b, x: D.Gamma(a, b).log_prob(x),
        "gamma_entropy": lambda a, b: D.Gamma(a, b).entropy(),
        "gamma_kl": two(D.Gamma),
        "beta_log_prob": lambda a, b, x: D.Beta(a, b).log_prob(x),
        "beta_entropy": lambda a, b: D.Beta(a, b).entropy(),
        "beta_kl": two(D.Beta),
        "dirichlet_log_prob": lambda a, x: D.Dirichlet(a).log_prob(x),
        "dirichlet_entropy": lambda a: D.Dirichlet(a).entropy(),
        "dirichlet_variance": lambda a: D.Dirichlet(a).variance(),
        "dirichlet_kl": one(D.Dirichlet),
        "poisson_log_prob": lambda r, k: D.Poisson(r).log_prob(k),
        "poisson_entropy": lambda r: D.Poisson(r).entropy(),
        "poisson_kl": one(D.Poisson),
        "special_digamma": T.digamma, "special_erf": T.erf, "special_erfinv": T.erfinv, "special_expm1": T.expm1,
        "special_lgamma": T.lgamma, "special_lgamma_negative": T.lgamma, "special_log1p": T.log1p,
    }
    with _open("distributions") as m:
        names = {n.split("/")[0] for n in m.names()}
        assert names == set(cases), names ^ set(cases)
        for case, fn in cases.items():
            _run_case(m, case, fn, tol=5e-5)


def test_function_transforms():
    """transforms.mim: Hessian-vector products (a forward derivative of a gradient), forward derivatives,
    Jacobians, a Hessian and per-example gradients (a gradient mapped over the batch)."""
    import mimir_b200.tensor as T
    from mimir_b200.tensor import autograd as A

    def mlp_energy(x, w1, b1, w2):
        y = T.matmul(T.tanh(T.matmul(x, w1) + b1), w2)
        return T.sum_(y * y) * 0.25

    def xent(x, w, y):
        return T.neg(T.mean(T.gather(T.log_softmax(T.matmul(x, w), -1), 1, T.unsqueeze(y, 1))))

    def conv_pool(x, w, b, g):
        y = T.max_pool2d(T.conv2d(x, w, b, padding=1), 2)
        return T.sum_(y * y * g)

    def per_example(x, y, w1, b1, w2):
        logits = T.matmul(T.relu(T.matmul(x, w1) + b1), w2)
        return T.neg(T.squeeze(T.gather(T.log_softmax(logits, -1), 0, T.unsqueeze(y, 0)), 0))

    cases = {
        "hvp_mlp": ("hvp", [0, 1, 2, 3], mlp_energy),
        "hvp_cross_entropy": ("hvp", [0, 1], xent),
        "hvp_attention_causal": ("hvp", [0, 1, 2], lambda q, k, v, w: T.sum_(T.attention(q, k, v, causal=True, causal_offset=2) * w)),
        "hvp_conv_pool": ("hvp", [0, 1, 2], conv_pool),
        "hvp_logcumsumexp": ("hvp", [0], lambda x, g: T.sum_(T.logcumsumexp(x, -1) * g)),
        "jvp_mlp": ("jvp", [0, 1, 2], lambda x, w, b: T.tanh(T.matmul(x, w) + b)),
        "jvp_attention_gqa": ("jvp", [0, 1, 2], lambda q, k, v: T.attention(q, k, v)),
        "jvp_softmax_cumsum": ("jvp", [0], lambda x: T.cumsum(T.softmax(x, -1), 0)),
        "jvp_conv_avg_pool": ("jvp", [0, 1], lambda x, w: T.avg_pool2d(T.conv2d(x, w, None, padding=1), 2)),
        "jacobian_softmax": ("jac", [0], lambda x, w: T.softmax(T.matmul(x, w), -1)),
        "jacobian_rows": ("jac", [0], lambda x, w: T.sum_(T.tanh(T.matmul(x, w)), 0)),
        "hessian_logsumexp": ("hess", [0], lambda x, w: T.log(T.sum_(T.exp(T.matmul(T.sin(x), w))))),
        "per_example_mlp": ("perex", [2, 3, 4], per_example),
    }

    def close(got, want, what):
        got = got.data() if hasattr(got, "data") and callable(got.data) else got
        assert torch.allclose(got.float().reshape(want.shape), want, rtol=1e-4, atol=1e-5), what

    with _open("transforms") as m:
        assert {n.split("/")[0] for n in m.names()} == set(cases)
        for case, (kind, diff, f) in cases.items():
            ins = [T.tensor(x, dtype=x.dtype, device=T.CPU()) for x in _inputs(m, case)]

            def partial(*x, f=f, ins=ins, diff=diff):
                args = list(ins)
                for k, i in enumerate(diff):
                    args[i] = x[k]
                return f(*args)
            x = [ins[i] for i in diff]
            if kind != "perex":
                close(partial(*x), m.tensor(f"{case}/out"), case)
            if kind == "hvp":
                v = [T.tensor(m.tensor(f"{case}/vec{i}").clone()) for i in diff]
                _, hv = A.jvp(A.grad(partial, argnums=tuple(range(len(diff)))), x, v)
                for k, i in enumerate(diff):
                    close(hv[k], m.tensor(f"{case}/hvp{i}"), f"{case}/hvp{i}")
            elif kind == "jvp":
                v = [T.tensor(m.tensor(f"{case}/tan{i}").clone()) for i in diff]
                y, tan = A.jvp(partial, x, v)
                close(y, m.tensor(f"{case}/out"), case)
                close(tan, m.tensor(f"{case}/jvp"), f"{case}/jvp")
            elif kind == "jac":
                close(A.jacobian(partial, x[0]), m.tensor(f"{case}/jac"), f"{case}/jac")
            elif kind == "hess":
                close(A.hessian(partial, x[0]), m.tensor(f"{case}/hess"), f"{case}/hess")
            else:
                def one(ex_x, ex_y, f=f, x=x):
                    loss = lambda *p: f(ex_x, ex_y, *p)  # noqa: E731
                    return (loss(*x),) + tuple(A.grad(loss, argnums=(0, 1, 2))(*x))
                got = A.vmap(one)(ins[0], ins[1])
                close(got[0], m.tensor(f"{case}/out"), case)
                for k, i in enumerate(diff):
                    close(got[1 + k], m.tensor(f"{case}/pergrad{i}"), f"{case}/pergrad{i}")
