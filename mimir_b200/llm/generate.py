"""Sampling and generation (reference: examples/llama/generate.go): temperature, top-k, top-p
(nucleus), min-p, repetition penalty; greedy when the temperature is zero."""
from __future__ import annotations

import torch

from .. import tensor as T


class Sampler:
    def __init__(self, temperature: float = 0.8, top_k: int = 40, top_p: float = 0.95, min_p: float = 0.0,
                 repeat_penalty: float = 1.0, repeat_last: int = 64, seed: int = 0):
        self.temperature, self.top_k, self.top_p, self.min_p = temperature, top_k, top_p, min_p
        self.repeat_penalty, self.repeat_last = repeat_penalty, repeat_last
        self.gen = torch.Generator().manual_seed(seed)
        self.seed, self.draws = seed, 0

    def distribution(self, logits: torch.Tensor, history=()) -> torch.Tensor:
        """Probabilities [vocab] after every filter (what ``sample`` draws from)."""
        lg = logits.detach().float().cpu().clone()
        if self.repeat_penalty != 1.0 and len(history):
            idx = torch.tensor(sorted(set(history[-self.repeat_last:])))
            v = lg[idx]
            lg[idx] = torch.where(v > 0, v / self.repeat_penalty, v * self.repeat_penalty)
        if self.temperature <= 0:
            p = torch.zeros_like(lg)
            p[lg.argmax()] = 1.0
            return p
        lg = lg / self.temperature
        if 0 < self.top_k < lg.numel():
            kth = lg.topk(self.top_k).values[-1]
            lg[lg < kth] = -float("inf")
        p = torch.softmax(lg, 0)
        if self.top_p < 1.0:
            sp, order = p.sort(descending=True)
            keep = sp.cumsum(0) - sp < self.top_p      # always keeps the first token
            mask = torch.zeros_like(p, dtype=torch.bool)
            mask[order[keep]] = True
            p = torch.where(mask, p, torch.zeros_like(p))
        if self.min_p > 0:
            p = torch.where(p >= self.min_p * p.max(), p, torch.zeros_like(p))
        return p / p.sum()

    def sample_device(self, logits: torch.Tensor, history=None) -> torch.Tensor:
        """Tokens for every row of ``logits`` ``[rows, V]`` on the GPU, drawn by the fused sampling kernel
        (radix-select top-k, nucleus and min-p cuts, Philox draw); returns int32 ``[rows]`` on the device.
        ``history``: optional int64 ``[rows, n]`` of recent tokens for the repetition penalty."""
        from ..ops.sampling import sample
        if logits.dim() == 1:
            logits = logits[None]
        if self.repeat_penalty != 1.0 and history is not None and history.numel():
            logits = logits.float().clone()
            h = history[:, -self.repeat_last:].to(logits.device)
            v = logits.gather(1, h)
            logits.scatter_(1, h, torch.where(v > 0, v / self.repeat_penalty, v * self.repeat_penalty))
        self.draws += 1
        return sample(logits, self.temperature, self.top_k, self.top_p, self.min_p, self.seed, self.draws - 1)

    def sample(self, logits: torch.Tensor, history=()) -> int:
        if logits.is_cuda and logits.dim() == 1:
            hist = torch.tensor([list(history[-self.repeat_last:])], dtype=torch.int64) if len(history) else None
            return int(self.sample_device(logits, hist)[0])
        p = self.distribution(logits, history)
        return int(p.argmax()) if self.temperature <= 0 else int(torch.multinomial(p, 1, generator=self.gen))


def generate(model, prompt_ids, n: int, sampler: Sampler | None = None, stop=(), on_token=None) -> list:
    """Incremental decoding with KV caches: the prompt is one forward pass, then one token at a time."""
    sampler = sampler or Sampler(temperature=0.0)
    caches = model.new_caches(1, min(model.cfg.context, len(prompt_ids) + n))
    ids = list(prompt_ids)
    with torch.no_grad():
        logits = model.logits(T.from_torch(torch.tensor([ids])), caches).data()[0, -1]
        out = []
        for _ in range(n):
            tok = sampler.sample(logits, ids)
            if tok in stop:
                break
            out.append(tok)
            ids.append(tok)
            if on_token is not None:
                on_token(tok)
            if len(ids) >= model.cfg.context:
                break
            logits = model.logits(T.from_torch(torch.tensor([[tok]])), caches).data()[0, -1]
    return out
