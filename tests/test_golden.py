"""Golden parity against the reference's committed NumPy float64 oracle files
(testdata/golden/*.mim; generator semantics in tools/golden/gen.py)."""
import math
import os

import pytest
import torch

from _refdir import reference_dir

# MIMIR_GOLDEN_DIR names the directory of golden files directly, like the reference's own tests
GOLD = os.environ.get("MIMIR_GOLDEN_DIR") or os.path.join(reference_dir() or "", "testdata", "golden")
pytestmark = pytest.mark.skipif(not os.path.isdir(GOLD), reason="reference golden files not found "
                                                                "(MIMIR_GOLDEN_DIR / MIMIR_REFERENCE_DIR)")


def _open(name):
    from mimir_b200.io import mim
    return mim.open(os.path.join(GOLD, name + ".mim"))


def _case(m, case):
    ins, i = [], 0
    while f"{case}/in{i}" in m:
        ins.append(m.tensor(f"{case}/in{i}").clone())
        i += 1
    return ins, m.tensor(f"{case}/out").clone()


def test_elementwise_and_reduction_ops():
    import mimir_b200.tensor as T
    table = {
        "abs": T.abs_, "add": T.add, "cos": T.cos, "div": T.div, "exp": T.exp, "log": T.log, "mul": T.mul,
        "neg": T.neg, "recip": T.recip, "relu": T.relu, "sigmoid": T.sigmoid, "silu": T.silu, "sin": T.sin,
        "sqrt": T.sqrt, "sub": T.sub, "tanh": T.tanh, "maximum": T.maximum, "minimum": T.minimum,
        "gelu": T.gelu, "add_int": T.add, "mul_int": T.mul,
        "sum_all": lambda x: T.sum_(x), "sum_axis1": lambda x: T.sum_(x, 1), "sum_axes02": lambda x: T.sum_(x, (0, 2)),
        "mean_last": lambda x: T.mean(x, -1), "max_axis2": lambda x: T.max_(x, 2), "min_axis0": lambda x: T.min_(x, 0),
        "var_axis1": lambda x: T.var(x, 1), "softmax_axis1": lambda x: T.softmax(x, 1),
        "log_softmax_large": lambda x: T.log_softmax(x, -1), "matmul_2d": T.matmul, "matmul_batched": T.matmul,
        "where": lambda c, a, b: T.where(c, a, b),
    }
    with _open("ops") as m:
        for case, fn in table.items():
            ins, want = _case(m, case)
            got = fn(*[T.tensor(x, dtype=x.dtype, device=T.CPU()) for x in ins]).data()
            assert got.shape == want.shape, case
            assert torch.allclose(got.float(), want.float(), rtol=2e-5, atol=2e-6), case


def test_philox_streams_are_bit_exact():
    import mimir_b200.tensor as T
    with _open("ops") as m:
        u = T.rand((1001,), seed=7, device=T.CPU()).data()
        assert torch.equal(u, m.tensor("rand_uniform/out"))
        n = T.randn((1001,), seed=7, device=T.CPU()).data()
        assert torch.allclose(n, m.tensor("rand_normal/out"), rtol=1e-5, atol=1e-6)


def test_optimizer_rules_and_schedules():
    from mimir_b200 import optim
    from mimir_b200.tensor import Param
    cases = {
        "sgd": lambda p: optim.SGD(p, lr=0.05),
        "sgd_momentum": lambda p: optim.SGD(p, lr=0.05, momentum=0.9, weight_decay=0.01),
        "sgd_nesterov": lambda p: optim.SGD(p, lr=0.05, momentum=0.9, nesterov=True),
        "adam": lambda p: optim.Adam(p, lr=0.1),
        "adam_l2": lambda p: optim.Adam(p, lr=0.1, weight_decay=0.1),
        "adamw": lambda p: optim.AdamW(p, lr=0.1, weight_decay=0.1),
        "rmsprop": lambda p: optim.RMSprop(p, lr=0.01, alpha=0.9),
        "adagrad": lambda p: optim.Adagrad(p, lr=0.1, lr_decay=0.05, initial=0.1),
        "adadelta": lambda p: optim.Adadelta(p, lr=1.0, rho=0.9),
        "adamax": lambda p: optim.Adamax(p, lr=0.1),
        "nadam": lambda p: optim.NAdam(p, lr=0.1),
        "lion": lambda p: optim.Lion(p, lr=0.05, weight_decay=0.1),
    }
    with _open("optim") as m:
        for case, make in cases.items():
            (p0, t, s), want = _case(m, case)
            p = Param(p0.double())
            opt = make([p])
            for _ in range(5):
                p._grad = 2 * s.double() * (p._data - t.double())
                opt.step()
            assert torch.allclose(p._data.float(), want, rtol=2e-5, atol=2e-6), case
        sched = {"step": optim.StepDecay(0.1, 2, 0.5), "cosine": optim.Cosine(0.1, 0.01, 5),
                 "warmup": optim.Warmup(0.1, 0.025, 4), "exponential": optim.Exponential(0.1, 0.8),
                 "polynomial": optim.Polynomial(0.1, 5, 2.0), "onecycle": optim.OneCycle(0.1, 10, 0.3)}
        for case, f in sched.items():
            want = m.tensor(f"{case}/out")
            got = torch.tensor([f(e) for e in range(want.numel())])
            assert torch.allclose(got, want, rtol=1e-5, atol=1e-7), case


def test_losses_and_layers():
    import mimir_b200.tensor as T
    from mimir_b200.nn import loss as L
    with _open("nn") as m:
        for case, fn in {"mse": L.mse, "l1": L.l1, "bce_with_logits": L.bce_with_logits, "nll": L.nll,
                         "cross_entropy": L.cross_entropy, "huber": L.huber}.items():
            ins, want = _case(m, case)
            got = fn(*[T.tensor(x, dtype=x.dtype, device=T.CPU()) for x in ins]).data()
            assert torch.allclose(got.float().reshape(want.shape), want, rtol=2e-5, atol=2e-6), case


def test_attention_variants():
    import mimir_b200.tensor as T
    with _open("attention") as m:
        def t(x):
            return T.tensor(x, dtype=x.dtype, device=T.CPU())
        for case, kw in {"sdpa": {}, "sdpa_causal": dict(causal=True), "sdpa_gqa": dict(causal=True, causal_offset=2), "sdpa_causal_offset": dict(causal=True, causal_offset=4), "sdpa_scale": dict(scale=0.3)}.items():
            ins, want = _case(m, case)
            got = T.attention(*[t(x) for x in ins[:3]], **kw).data()
            assert torch.allclose(got, want, rtol=2e-5, atol=2e-6), case
        ins, want = _case(m, "sdpa_mask")
        got = T.attention(t(ins[0]), t(ins[1]), t(ins[2]), mask=t(ins[3])).data()
        assert torch.allclose(got, want, rtol=2e-5, atol=2e-6)


def test_quantized_formats_dequantize_bit_exact():
    from mimir_b200.ops import quant as Q
    with _open("quant") as m:
        for case, code in (("q8_0_dequantize", Q.Q8_0), ("q4_K_dequantize", Q.Q4_K), ("q6_K_dequantize", Q.Q6_K)):
            raw, want = m.tensor(f"{case}/in0"), m.tensor(f"{case}/out")
            got = Q.dequantize_raw(code, raw, want.numel()).view(want.shape)
            assert torch.equal(got, want), case
        for case, code in (("q8_0_matmul", Q.Q8_0), ("q4_K_matmul", Q.Q4_K), ("q6_K_matmul", Q.Q6_K)):
            x, raw, want = m.tensor(f"{case}/in0"), m.tensor(f"{case}/in1"), m.tensor(f"{case}/out")
            w = Q.dequantize_raw(code, raw, raw.shape[0] * x.shape[-1]).view(raw.shape[0], x.shape[-1])
            assert torch.allclose(x @ w.t(), want, rtol=2e-5, atol=2e-5), case
    # Q4_0 / Q8_0 quantise -> dequantise round trip stays within half a step
    x = torch.randn(4, 64)
    for quant, code, steps, bound in ((Q.quantize_q8_0, Q.Q8_0, 127, 0.56), (Q.quantize_q4_0, Q.Q4_0, 8, 1.01)):
        back = Q.dequantize_raw(code, quant(x), x.numel()).view(x.shape)
        step = x.reshape(-1, 32).abs().amax(1, keepdim=True) / steps
        # half a step (+ fp16 rounding of the scale); Q4_0's range [-8, 7] clips one extreme by up to a step
        assert ((back - x).reshape(-1, 32).abs() <= step * bound + 1e-5).all()
