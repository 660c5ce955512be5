"""nn / optim / train behaviours: learning, exact resume, micro-batching, loss scaling."""
import io

import pytest
import torch


def _setup(seed=1):
    from mimir_b200 import data, nn, optim
    torch.manual_seed(0)
    X = torch.randn(256, 8)
    Y = (X @ torch.randn(8, 3)).argmax(1)
    nn.manual_seed(seed)
    model = nn.Sequential(nn.Linear(8, 32), nn.ReLU(), nn.Linear(32, 3))
    return model, optim.AdamW(model.parameters(), lr=1e-2), data.Tensors(X, Y, batch_size=32, seed=3, class_targets=True)


def test_fit_learns_reports_and_resumes_exactly(tmp_path):
    from mimir_b200 import metrics
    from mimir_b200.nn import loss as L
    from mimir_b200.train import fit
    m, o, ds = _setup()
    buf = io.StringIO()
    reps = fit(m, o, ds, loss=L.cross_entropy, epochs=4, eval=ds, metrics=[metrics.Accuracy()], progress=buf)
    assert reps[-1].loss < reps[0].loss and reps[-1].metrics["accuracy"] > 0.9
    assert buf.getvalue().count("\n") == 4
    m2, o2, _ = _setup()
    fit(m2, o2, ds, loss=L.cross_entropy, epochs=2, checkpoint=str(tmp_path))
    m3, o3, _ = _setup()
    fit(m3, o3, ds, loss=L.cross_entropy, epochs=4, checkpoint=str(tmp_path))
    for a, b in zip(m.parameters(), m3.parameters()):
        assert torch.equal(a._data, b._data)


def test_micro_batch_equals_full_batch_and_loss_scaling():
    from mimir_b200.nn import loss as L
    from mimir_b200.train import fit
    m, o, ds = _setup()
    fit(m, o, ds, loss=L.cross_entropy, epochs=2)
    m2, o2, _ = _setup()
    fit(m2, o2, ds, loss=L.cross_entropy, epochs=2, micro_batch=8)
    m3, o3, _ = _setup()
    seen = []
    fit(m3, o3, ds, loss=L.cross_entropy, epochs=2, dynamic_loss_scale=True, on_batch=seen.append)
    for a, b, c in zip(m.parameters(), m2.parameters(), m3.parameters()):
        assert torch.allclose(a._data, b._data, atol=1e-6)
        assert torch.allclose(a._data, c._data, atol=1e-5)
    assert seen[0].loss_scale == 65536.0 and not seen[0].skipped


def test_layers_run_and_cache_matches_full_sequence():
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    blk = nn.DecoderBlock(32, 4, style="llama", kv_heads=2, rope=nn.RotaryEmbedding(8)).eval()
    x = torch.randn(2, 5, 32)
    full = blk(T.tensor(x, device=T.CPU())).data()
    cache = nn.KVCache(2, 2, 16, 8)
    step = [blk(T.tensor(x[:, i:i + 1], device=T.CPU()), cache).data() for i in range(5)]
    assert torch.allclose(torch.cat(step, 1), full, atol=1e-5)
    out, h = nn.LSTM(8, 16, 2, batch_first=True)(T.tensor(torch.randn(3, 7, 8), device=T.CPU()))
    assert out.shape == (3, 7, 16) and h.shape == (2, 3, 16)
    g = nn.Graph(4, [0, 1, 2], [1, 2, 3])
    assert nn.GATConv(8, 4, 2)(T.tensor(torch.randn(4, 8), device=T.CPU()), g).data().shape == (4, 8)
    names = [n for n, _ in blk.named_params()]
    assert "attn.qkv.weight" in names and "mlp.gate.weight" in names
    ck = nn.Checkpoint(nn.Sequential(nn.Linear(4, 4), nn.Tanh()))
    plain = ck.inner
    xin = T.tensor(torch.randn(3, 4), device=T.CPU())
    T.sum_(ck(xin)).backward()
    g_ck = [p.grad().data().clone() for p in plain.parameters()]
    plain.zero_grad()
    T.sum_(plain(xin)).backward()
    for a, p in zip(g_ck, plain.parameters()):
        assert torch.allclose(a, p.grad().data(), atol=1e-6)
