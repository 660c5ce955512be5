"""Schedules: structural key, program cache, fusion planner (reference: internal/sched/key.go:181-231,
cache.go:22-104, fuse.go:200-362; tests internal/sched/cache_test.go)."""
import torch

import mimir_b200.tensor as T
from mimir_b200 import nn
from mimir_b200.tensor import plan


def _mlp_loss(model, x, y):
    return nn.loss.mse(model(x), y)


def test_same_structure_hits_the_cache_and_new_values_flow():
    plan.clear_cache()
    w = T.tensor(torch.randn(8, 8))
    before = plan.compiled()
    outs = []
    for i in range(4):
        x = T.tensor(torch.full((4, 8), float(i)))
        outs.append(T.sum_((x @ w) * float(i + 1)).item())
    assert plan.compiled() - before == 1, plan.stats()
    ref = [float(((torch.full((4, 8), float(i)) @ w.data()) * float(i + 1)).sum()) for i in range(4)]
    assert torch.allclose(torch.tensor(outs), torch.tensor(ref), rtol=1e-5, atol=1e-5)


def test_different_shapes_compile_again():
    plan.clear_cache()
    before = plan.compiled()
    for n in (3, 5, 3, 5):
        T.sum_(T.tensor(torch.ones(n, 4)) * 2.0).item()
    assert plan.compiled() - before == 2


def test_fusion_plan_matches_unfused_values_and_gradients():
    torch.manual_seed(0)
    nn.manual_seed(7)
    block = nn.DecoderBlock(16, 2, style="gpt2")
    x = torch.randn(2, 5, 16)

    def run():
        for p in block.parameters():
            p.zero_grad()
        out = block(T.tensor(x))
        loss = T.mean(out * out)
        loss.backward()
        return loss.item(), [p.grad().data().clone() for p in block.parameters()]

    plan.clear_cache()
    l1, g1 = run()
    st = plan.stats()
    assert st["fused"] >= 2, st          # gelu into fc, residual into the two row products
    # the same model with fusion disabled (every node scheduled on its own)
    saved = plan._plan_fusion
    plan._plan_fusion = lambda w: ({}, set())
    plan.clear_cache()
    try:
        l2, g2 = run()
    finally:
        plan._plan_fusion = saved
        plan.clear_cache()
    assert abs(l1 - l2) < 1e-6
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)


def test_fusion_keeps_a_value_that_has_another_reader():
    lin = nn.Linear(8, 8)
    x = T.tensor(torch.randn(4, 8))
    h = lin(x)
    y = T.gelu(h) + h          # h has two readers: it must be scheduled on its own
    ref_h = x.data() @ lin.weight._data.T + lin.bias._data
    ref = torch.nn.functional.gelu(ref_h, approximate="tanh") + ref_h
    assert torch.allclose(y.data(), ref, rtol=1e-5, atol=1e-6)


def test_dropout_seed_is_not_part_of_the_key_but_reaches_the_kernel():
    plan.clear_cache()
    d = nn.Dropout(0.5, seed=3)
    x = T.tensor(torch.ones(64, 64))
    before = plan.compiled()
    a = T.sum_(d(x) * 1.0).item()
    masks = [d(x).data().clone() for _ in range(3)]
    assert plan.compiled() - before <= 2          # one for the sum graph, one for the bare dropout
    assert not torch.equal(masks[0], masks[1]) and not torch.equal(masks[1], masks[2])
    assert a > 0


def test_error_in_a_cached_program_marks_the_node_of_the_current_graph():
    idx = T.tensor(torch.tensor([0, 1]), dtype=torch.int32)
    tab = T.tensor(torch.randn(4, 3))
    assert T.gather_rows(tab, idx).data().shape == (2, 3)
    bad = T.gather_rows(tab, T.tensor(torch.tensor([0, 9]), dtype=torch.int32))
    try:
        bad.data()
        raise AssertionError("expected ErrIndex")
    except T.ErrIndex:
        pass
    assert isinstance(bad.err, T.ErrIndex)
