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
