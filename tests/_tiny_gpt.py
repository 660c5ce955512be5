"""A small GPT-2 built from the public ``nn`` layers, and its plain-PyTorch fp32 restatement
(used by the GPU tests of the lazy tensor / nn / optim / train path)."""
import torch

import mimir_b200.tensor as T
from mimir_b200 import nn
from mimir_b200.nn import loss as L

F = torch.nn.functional


class TinyGPT(nn.Module):
    def __init__(self, vocab=512, ctx=128, dim=128, heads=2, layers=2):
        self.vocab, self.ctx, self.dim, self.heads = vocab, ctx, dim, heads
        self.wte = nn.Embedding(vocab, dim)
        self.wpe = nn.Embedding(ctx, dim)
        self.blocks = [nn.DecoderBlock(dim, heads, style="gpt2") for _ in range(layers)]
        self.lnf = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, vocab, bias=False)
        self._nn_skip_pos = None      # position ids, uploaded once
        for _, p in self.named_params():       # GPT-2 sized initial weights keep bf16 well conditioned
            if p._data.dim() == 2:
                p._data.mul_(0.2)

    def forward(self, tok):
        B, Tq = tok.shape
        if self._nn_skip_pos is None or self._nn_skip_pos.device != tok.device:
            self._nn_skip_pos = T.tensor(torch.arange(self.ctx), dtype=torch.int64, device=tok.device)
        x = self.wte(tok) + self.wpe(self._nn_skip_pos[:Tq])
        for b in self.blocks:
            x = b(x)
        return self.head(self.lnf(x))


def loss_fn(vocab):
    return lambda out, y: L.cross_entropy(T.reshape(out, (-1, vocab)), T.reshape(y, (-1,)))


def torch_reference(model: TinyGPT, params: dict, tok: torch.Tensor, tgt: torch.Tensor):
    """fp32 loss of the same network from a ``{name: tensor}`` dict (autograd-ready)."""
    C, H = model.dim, model.heads
    B, Tq = tok.shape
    x = params["wte.weight"][tok] + params["wpe.weight"][:Tq]
    for i in range(len(model.blocks)):
        p = f"blocks.{i}."
        a = F.layer_norm(x, (C,), params[p + "norm1.weight"], params[p + "norm1.bias"], 1e-5)
        qkv = a @ params[p + "attn.qkv.weight"].t() + params[p + "attn.qkv.bias"]
        q, k, v = qkv.split(C, dim=-1)
        sp = lambda t: t.view(B, Tq, H, C // H).transpose(1, 2)  # noqa: E731
        o = F.scaled_dot_product_attention(sp(q), sp(k), sp(v), is_causal=True)
        x = x + o.transpose(1, 2).reshape(B, Tq, C) @ params[p + "attn.out.weight"].t() + params[p + "attn.out.bias"]
        a = F.layer_norm(x, (C,), params[p + "norm2.weight"], params[p + "norm2.bias"], 1e-5)
        h = F.gelu(a @ params[p + "mlp.up.weight"].t() + params[p + "mlp.up.bias"], approximate="tanh")
        x = x + h @ params[p + "mlp.down.weight"].t() + params[p + "mlp.down.bias"]
    x = F.layer_norm(x, (C,), params["lnf.weight"], params["lnf.bias"], 1e-5)
    logits = x @ params["head.weight"].t()
    return F.cross_entropy(logits.view(-1, model.vocab), tgt.reshape(-1).long())
