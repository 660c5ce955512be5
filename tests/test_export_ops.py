"""Every public op that a model may hold exports: ops without a word in the graph vocabulary are rebuilt from
ops that have one, and the interpreter's answer must equal the lazy layer's.  Whole picture, sound and
detection models export the same way (batch norm in inference mode, overlapping pooling, transposed
convolutions, group norm, framing)."""
import io

import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200 import audio, nn, vision
from mimir_b200.io import export as X
from mimir_b200.io import mim


def _round_trip(f, args):
    buf = io.BytesIO()
    X.export_func(buf, f, args, input_names=[f"i{k}" for k in range(len(args))], output_names=["o"])
    got = mim.parse(buf.getvalue()).run({f"i{k}": a for k, a in enumerate(args)})["o"].data()
    want = f(*args).data()
    assert got.shape == want.shape and got.dtype == want.dtype, (got.shape, want.shape, got.dtype, want.dtype)
    return float((got.double() - want.double()).abs().max())


def _cases():
    nn.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    x, y = T.tensor(torch.randn(3, 4, generator=g)), T.tensor(torch.randn(3, 4, generator=g))
    img, seq = T.tensor(torch.randn(2, 3, 8, 8, generator=g)), T.tensor(torch.randn(2, 3, 10, generator=g))
    idx = T.tensor(torch.tensor([[0, 1, 3, 2], [2, 3, 0, 0], [1, 1, 2, 3]]))
    c1, ct, ct3, ct1 = nn.Conv1d(3, 4, 3, padding=1), nn.ConvTranspose2d(3, 2, 2, 2), nn.ConvTranspose2d(3, 2, 3, 2, 1), nn.ConvTranspose1d(3, 2, 4, 2, 1)
    bn, gn = nn.BatchNorm2d(3).eval(), nn.GroupNorm(1, 3)
    bn.running_mean.set(torch.tensor([0.1, -0.2, 0.3]))
    bn.running_var.set(torch.tensor([1.5, 0.5, 2.0]))
    return {
        "softplus": (lambda a: T.softplus(a), [x]), "clamp": (lambda a: T.clamp(a, -0.5, 0.5), [x]), "clamp_low": (lambda a: T.clamp(a, 0.1, None), [x]),
        "min": (lambda a: T.min_(a, 1), [x]), "var": (lambda a: T.var(a, 1), [x]), "var_all": (lambda a: T.var(a), [x]),
        "flip": (lambda a: T.flip(a, (0, 1)), [x]), "stack": (lambda a, b: T.stack([a, b], 1), [x, y]), "split": (lambda a: T.split(a, [1, 3], 1)[1], [x]),
        "one_hot": (lambda i: T.one_hot(i, 4), [idx]), "argmax": (lambda a: T.argmax(a, 1), [x]), "argmax_rows": (lambda a: T.argmax(a, 0), [x]),
        "gather": (lambda a, i: T.gather(a, 1, i), [x, idx]), "log1p": (lambda a: T.log1p(T.abs_(a) * 1e-3), [x]), "log1p_big": (lambda a: T.log1p(T.abs_(a)), [x]),
        "expm1": (lambda a: T.expm1(a * 1e-3), [x]), "sign": (lambda a: T.sign(a), [x]), "floor": (lambda a: T.floor(a * 3.0), [x]), "ceil": (lambda a: T.ceil(a * 3.0), [x]),
        "logsumexp": (lambda a: T.logsumexp(a, 1), [x]), "abs": (lambda a: T.abs_(a), [x]), "greater": (lambda a, b: T.cast(T.greater(a, b), T.float32), [x, y]),
        "and_or": (lambda a, b: T.cast(T.logical_or(T.logical_and(T.less(a, b), T.less(a, 0.0)), T.less(1.0, b)), T.float32), [x, y]),
        "smallest": (lambda a: T.topk(a, 2, -1, False)[0], [x]), "windows": (lambda s: T.windows(s, 2, 4, 3), [seq]),
        "conv1d": (lambda s: c1(s), [seq]), "conv_transpose2d": (lambda i: ct(i), [img]), "conv_transpose2d_overlap": (lambda i: ct3(i), [img]),
        "conv_transpose1d": (lambda s: ct1(s), [seq]), "max_pool": (lambda i: T.max_pool2d(i, 2), [img]), "max_pool_overlap": (lambda i: T.max_pool2d(i, 3, 2, 1), [img]),
        "avg_pool": (lambda i: T.avg_pool2d(i, 2), [img]), "avg_pool_overlap": (lambda i: T.avg_pool2d(i, 3, 2, 1), [img]),
        "batch_norm_inference": (lambda i: bn(i), [img]), "group_norm": (lambda i: gn(i), [img]), "upsample": (lambda i: T.upsample_nearest(i, 2), [img]),
    }


@pytest.mark.parametrize("name", sorted(_cases()))
def test_op_exports_and_agrees(name):
    f, args = _cases()[name]
    assert _round_trip(f, args) < 1e-4, name


def test_group_norm_in_tensor_ops_equals_the_library_layer():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 6, 5, 5, generator=g)
    gn = nn.GroupNorm(3, 6)
    gn.weight.set(torch.randn(6, generator=g))
    gn.bias.set(torch.randn(6, generator=g))
    want = torch.nn.functional.group_norm(x, 3, gn.weight.value().data(), gn.bias.value().data(), 1e-5)
    assert torch.allclose(gn(T.tensor(x)).data(), want, atol=1e-5)
    assert isinstance(nn.GroupNorm(4, 6)(T.tensor(x)).err, T.ErrShape)


def test_whole_models_export_and_agree():
    nn.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    nets = {
        "resnet18": (vision.resnet18(10, width=8).eval(), torch.randn(2, 3, 64, 64, generator=g)),
        "resnet18_small": (vision.resnet18(5, width=8, small=True).eval(), torch.randn(2, 3, 32, 32, generator=g)),
        "mobilenet": (vision.MobileNetV2(4, width=0.25, small=True).eval(), torch.randn(2, 3, 32, 32, generator=g)),
        "unet": (vision.UNet(3, 2, width=4, depth=2).eval(), torch.randn(1, 3, 16, 16, generator=g)),
        "vit": (vision.ViT(image=32, patch=8, dim=32, depth=1, heads=2, mlp=64, classes=5).eval(), torch.randn(2, 3, 32, 32, generator=g)),
        "detector": (vision.Detector(2, vision.tiny_backbone(3, 8), head_width=8).eval(), torch.randn(1, 3, 32, 32, generator=g)),
        "wave_classifier": (audio.WaveClassifier(3, width=0.25).eval(), torch.randn(2, 3200, generator=g)),
    }
    for name, (net, x) in nets.items():
        buf = io.BytesIO()
        X.export(buf, net, x)
        got = mim.parse(buf.getvalue()).run({"input": x})["output"].data()
        want = net(T.tensor(x)).data()
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (name, float((got - want).abs().max()))


def test_recurrent_layers_and_text_classifier_export():
    from mimir_b200 import text
    nn.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    for name, net, x in (("lstm", nn.LSTM(5, 8, layers=2, batch_first=True), torch.randn(2, 6, 5, generator=g)),
                         ("gru", nn.GRU(5, 8, bidirectional=True), torch.randn(6, 2, 5, generator=g)),
                         ("rnn", nn.RNN(5, 8, relu=True, bias=False), torch.randn(6, 2, 5, generator=g))):
        f = lambda a, net=net: net(a)[0]  # noqa: E731
        buf = io.BytesIO()
        X.export_func(buf, f, [T.tensor(x)], input_names=["input"], output_names=["output"], module=net)
        got = mim.parse(buf.getvalue()).run({"input": x})["output"].data()
        assert torch.allclose(got, f(T.tensor(x)).data(), atol=1e-5), name
    ids = torch.randint(1, 50, (2, 12), generator=g)
    ids[0, 8:] = 0
    cfg = text.BertConfig(vocab=50, dim=32, layers=1, heads=2, hidden=64, max_positions=16, dropout=0.0)
    clf = text.TextClassifier(cfg, 3, pad_id=0).eval()
    buf = io.BytesIO()
    X.export(buf, clf, ids)
    other = ids.clone()
    other[1, 5:] = 0                                                  # the padding mask is computed in the graph, not baked in
    for batch in (ids, other):
        got = mim.parse(buf.getvalue()).run({"input": batch})["output"].data()
        assert torch.allclose(got, clf(T.tensor(batch)).data(), atol=1e-5)


def test_graph_layers_export_over_a_small_graph():
    """While an exporter listens, sparse patterns become products by their dense 0 / 1 matrices (constants of
    the graph), so GCN, GraphSAGE and GAT export with their graph baked in; a graph too large for that is refused."""
    from mimir_b200.tensor import pattern
    nn.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    n = 30
    src, dst = torch.randint(0, n, (90,), generator=g), torch.randint(0, n, (90,), generator=g)
    dst[dst == 7] = 8                                               # node 7 has no incoming edge
    graph = nn.Graph(n, src, dst)
    x = torch.randn(n, 6, generator=g)
    layers = {"gcn": nn.GCNConv(6, 4), "sage": nn.SAGEConv(6, 4), "gat": nn.GATConv(6, 3, heads=2)}
    fns = {k: (lambda a, l=l: l.convolve(graph, a)) for k, l in layers.items()}
    fns["max"] = lambda a: graph.max(graph.source(a))
    for name, f in fns.items():
        buf = io.BytesIO()
        X.export_func(buf, f, [T.tensor(x)], input_names=["x"], output_names=["y"], module=layers.get(name))
        got = mim.parse(buf.getvalue()).run({"x": x})["y"].data()
        assert torch.allclose(got, f(T.tensor(x)).data(), atol=1e-5), name
    old = pattern.DENSE_EXPORT_CELLS
    pattern.DENSE_EXPORT_CELLS = 100
    try:
        with pytest.raises(T.ErrUnsupported):
            X.export_func(io.BytesIO(), fns["gcn"], [T.tensor(x)])
    finally:
        pattern.DENSE_EXPORT_CELLS = old
