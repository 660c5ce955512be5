"""GPT-2 engine (kernel sequence) against an fp32 PyTorch autograd restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).norm().item() / (b.float().norm().item() + 1e-8)


@pytest.mark.parametrize("attention", ["native", "sdpa"])
def test_tiny_gpt2_loss_and_grads(attention):
    from mimir_b200.models.gpt2 import GPT2Config, GPT2Engine, reference_forward_loss
    from mimir_b200.ops._util import check_error_word
    cfg = GPT2Config(n_layer=2, n_head=2, d_model=128, vocab=1000, ctx=128)
    B, T = 2, 128
    eng = GPT2Engine(cfg, B, T, seed=1, attention=attention)
    torch.manual_seed(0)
    tok = torch.randint(0, cfg.vocab, (B, T), device="cuda")
    tgt = torch.randint(0, cfg.vocab, (B, T), device="cuda")
    eng.tokens.copy_(tok.view(-1))
    eng.targets.copy_(tgt.view(-1))
    eng.forward()
    eng.loss_and_dlogits()
    eng.backward()
    assert check_error_word() == 0
    # reference uses the bf16-rounded weights the engine actually multiplies with
    eng.master.copy_(eng.params)
    loss, grads = reference_forward_loss(eng, tok, tgt)
    assert abs(eng.loss.item() - loss.item()) < 2e-2 * loss.item()
    views = eng.g
    for name in ("h.1.proj_w", "h.0.qkv_w", "h.0.fc_b", "h.1.ln1_g", "lnf_b", "wpe", "wte", "h.0.o_w"):
        assert _rel(views[name], grads[name]) < 6e-2, name


def test_trainer_loss_decreases_and_graph_matches_eager():
    from mimir_b200.models.gpt2 import GPT2Config, GPT2Engine
    from mimir_b200.train import FusedTrainer
    cfg = GPT2Config(n_layer=2, n_head=2, d_model=128, vocab=512, ctx=128)
    torch.manual_seed(0)
    tok = torch.randint(0, cfg.vocab, (4, 128))
    tgt = torch.roll(tok, -1, 1)
    losses = {}
    for use_graph in (False, True):
        eng = GPT2Engine(cfg, 4, 128, seed=3)
        tr = FusedTrainer(eng, lr=3e-3, use_graph=use_graph)
        losses[use_graph] = [tr.step(tok, tgt) for _ in range(8)]
        assert tr.launches_per_step > 0
    assert losses[True][-1] < losses[True][0] - 0.3
    for a, b in zip(losses[False], losses[True]):
        assert abs(a - b) < 5e-2
