"""The shared case table (``mimir_b200/utils/conformance.py``) against its float64 oracle files: on
the CPU in float32 and bfloat16; the GPU pass is ``tests/test_zy_conformance_gpu.py`` (reference: the same kerneltest cases on
every backend, backend/internal/kerneltest/kerneltest.go:58-120; oracle files as tools/golden/gen.py
writes them)."""
import os

import pytest
import torch

from mimir_b200.utils import conformance as conf


@pytest.fixture(scope="module")
def golden(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("golden"))
    counts = conf.generate(d)
    assert sum(counts.values()) == len(conf.CASES) and len(conf.CASES) >= 60
    return d


def test_oracle_files_hold_inputs_outputs_and_gradients(golden):
    from mimir_b200.io import mim
    with mim.open(os.path.join(golden, "ops.mim")) as m:
        assert m.metadata["oracle"] == "torch-float64"
        for name in ("binary_add/in0", "binary_add/in1", "binary_add/out", "binary_add/gout", "binary_add/grad0", "binary_add/grad1"):
            assert name in m
        a, b = m.tensor("binary_add/in0"), m.tensor("binary_add/in1")
        assert torch.equal(m.tensor("binary_add/out"), (a.double() + b.double()).float())
        # the gradient of a broadcast operand is the cotangent summed over the broadcast axes
        g = m.tensor("binary_add/gout").double()
        assert torch.allclose(m.tensor("binary_add/grad0").double(), g.sum(1, keepdim=True), atol=1e-6)
    again = str(golden) + "_again"
    conf.generate(again)
    for f in conf.FILES:                                    # seeded: the same bytes every time
        assert open(os.path.join(golden, f + ".mim"), "rb").read() == open(os.path.join(again, f + ".mim"), "rb").read()


def test_cpu_float32_is_conformant(golden):
    assert conf.check(golden) == []


def test_cpu_bfloat16_is_conformant_within_the_half_tolerances(golden):
    assert conf.check(golden, dtype=torch.bfloat16) == []


def test_a_wrong_kernel_is_caught_by_the_row_bound(golden, monkeypatch):
    import mimir_b200.tensor as T
    case = next(c for c in conf.CASES if c.name == "matmul_2d")

    def off_by_one_row(a, b):
        out = T.matmul(a, b)
        bump = torch.zeros(64, 40)
        bump[17] = 2e-3                                     # far below the largest value of the result
        return out + T.tensor(bump)
    monkeypatch.setattr(case, "run", off_by_one_row)
    bad = conf.check(golden, only={"matmul_2d"})
    assert len(bad) == 1 and "matmul_2d/out" in bad[0]
