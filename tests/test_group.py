"""Device groups on CPU ranks (reference: tensor/group_test.go)."""
import os
import sys

sys.path.insert(0, os.path.dirname(__file__))
import _group_worker as W

import mimir_b200.tensor as T


def test_collectives_three_ranks():
    res = T.cpus(3, W.collectives, port=29811)
    for r, out in enumerate(res):
        assert out["sum"] == [6.0] * 4 and out["mean"] == [2.0] * 4 and out["max"] == [3.0] * 4
        assert out["bcast"] == [2.0] * 4
        assert out["gather"] == [0.0, 1.0, 2.0]
        assert out["rs"] == [6.0]


def test_gradient_buckets_and_param_broadcast():
    res = T.cpus(2, W.grads, port=29812)
    assert res[0]["p0"] == res[1]["p0"]
    for out in res:
        assert out["g"] == [1.5, 1.5]          # mean of 1 and 2
        assert out["calls"] == 1               # both parameters fit one bucket


def test_data_parallel_fit_matches_single_device():
    import pytest
    single = W.single_fit()
    for mode, port in (("all_reduce", 29813), ("reduce", 29814)):
        res = T.cpus(3, W.dp_fit, mode, port=port)      # 10-row batches over 3 ranks: 4 + 4 + 2 rows
        for out in res:
            assert out["loss"] == pytest.approx(single["loss"], rel=1e-4, abs=1e-5)
            assert out["w"] == pytest.approx(single["w"], rel=1e-4, abs=1e-4)
        assert res[0]["w"] == res[1]["w"] == res[2]["w"]


def test_replicate_and_inference_view():
    import torch
    from mimir_b200 import nn
    from mimir_b200.parallel.replicas import inference, replicate
    nn.manual_seed(0)
    m = nn.Sequential(nn.Linear(4, 4), nn.BatchNorm1d(4))
    r = replicate(m)
    x = T.from_torch(torch.randn(8, 4))
    assert torch.equal(r.eval()(x).data(), m.eval()(x).data())
    r.layers[0].weight.set(torch.zeros(4, 4))
    assert m.layers[0].weight._data.abs().sum() > 0          # a copy, not a view
    v = inference(m)
    m.layers[0].weight._data.mul_(2)                          # the view follows the original's storage
    assert torch.equal(v(x).data(), m.eval()(x).data())
    assert not any(p.trainable for p in v.parameters())
