"""BERT encoder (reference: text/bert.go): token + position + segment embeddings, post-norm
encoder layers, pooler, masked-LM and classification heads."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import nn
from .. import tensor as T


@dataclass
class BertConfig:
    vocab: int = 30522
    dim: int = 768
    layers: int = 12
    heads: int = 12
    hidden: int = 3072
    max_positions: int = 512
    types: int = 2
    eps: float = 1e-12
    dropout: float = 0.1

    @staticmethod
    def tiny(vocab=128):
        return BertConfig(vocab=vocab, dim=32, layers=2, heads=2, hidden=64, max_positions=64)

    @staticmethod
    def base(vocab=30522):
        """Devlin et al.'s BERT-base: 768 numbers, 12 layers of 12 heads, 512 tokens."""
        return BertConfig(vocab=vocab)

    @staticmethod
    def mini(vocab=30522):
        """Turc et al.'s BERT-mini: 256 numbers in 4 layers of 4 heads."""
        return BertConfig(vocab=vocab, dim=256, layers=4, heads=4, hidden=1024)

    @staticmethod
    def small(vocab=30522):
        """Turc et al.'s BERT-tiny: 128 numbers in 2 layers of 2 heads; small enough to teach from scratch on a
        few thousand texts."""
        return BertConfig(vocab=vocab, dim=128, layers=2, heads=2, hidden=512)


class Bert(nn.Module):
    def __init__(self, cfg: BertConfig):
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.vocab, cfg.dim)
        self.pos = nn.Embedding(cfg.max_positions, cfg.dim)
        self.typ = nn.Embedding(cfg.types, cfg.dim)
        for e in (self.tok, self.pos, self.typ):
            e.weight.set(nn.normal_init(tuple(e.weight.shape), 0.02))
        self.norm = nn.LayerNorm(cfg.dim, cfg.eps)
        self.drop = nn.Dropout(cfg.dropout)
        self.layers = [nn.TransformerEncoderLayer(cfg.dim, cfg.heads, cfg.hidden, cfg.eps, activation="gelu", dropout=0.0) for _ in range(cfg.layers)]
        self.pooler = nn.Linear(cfg.dim, cfg.dim)

    def forward(self, ids, type_ids=None, attention_mask=None):
        """ids [B, T] int; returns ``(hidden [B, T, dim], pooled [B, dim])``."""
        B, Tn = ids.shape
        pos = T.arange(Tn, dtype=torch.int64, device=ids.device)
        x = self.tok(ids) + self.pos(pos)
        x = x + self.typ(type_ids if type_ids is not None else T.zeros((B, Tn), dtype=torch.int64, device=ids.device))
        x = self.drop(self.norm(x))
        mask = None
        if attention_mask is not None:   # [B, T] of 1 / 0 -> additive [B, 1, 1, T]
            m = T.cast(attention_mask, torch.float32)
            mask = T.reshape((m - 1.0) * 1e9, (B, 1, 1, Tn))
        for l in self.layers:
            x = l(x, mask=mask)
        return x, T.tanh(self.pooler(x[:, 0]))


class BertForMaskedLM(nn.Module):
    def __init__(self, cfg: BertConfig):
        self.bert = Bert(cfg)
        self.transform, self.norm = nn.Linear(cfg.dim, cfg.dim), nn.LayerNorm(cfg.dim, cfg.eps)
        self.bias = T.Param(torch.zeros(cfg.vocab), "bias")

    def forward(self, ids, type_ids=None, attention_mask=None):
        h, _ = self.bert(ids, type_ids, attention_mask)
        h = self.norm(T.gelu(self.transform(h)))
        return T.matmul_t(h, self.bert.tok.weight.value()) + self.bias.value()   # tied output embedding


class BertForSequenceClassification(nn.Module):
    def __init__(self, cfg: BertConfig, classes: int):
        self.bert, self.drop, self.head = Bert(cfg), nn.Dropout(cfg.dropout), nn.Linear(cfg.dim, classes)

    def forward(self, ids, type_ids=None, attention_mask=None):
        return self.head(self.drop(self.bert(ids, type_ids, attention_mask)[1]))


class TextClassifier(nn.Module):
    """A BERT that reads token ids ``[B, S]`` and says a class (text/bert.go: BERT): ``encode`` gives each
    token's vector, ``features`` the pooled [CLS] vector, ``forward`` the logits.  Padding (``pad_id``) is
    hidden from attention.  ``set_head`` / ``head_parameters`` serve transfer learning."""

    def __init__(self, cfg: BertConfig, classes: int, pad_id: int = 0):
        if cfg.dim % cfg.heads:
            raise ValueError(f"BERT: {cfg.dim} features over {cfg.heads} heads")
        self.bert, self.drop, self.head = Bert(cfg), nn.Dropout(cfg.dropout), nn.Linear(cfg.dim, classes)
        self.width, self.pad_id = cfg.dim, pad_id

    def _ids(self, x):
        x = x if isinstance(x, T.Tensor) else T.tensor(torch.as_tensor(x))
        return T.cast(x, torch.int64) if x.dtype != torch.int64 else x

    def _run(self, x):
        ids = self._ids(x)
        if ids.shape[1] > self.bert.cfg.max_positions:
            raise ValueError(f"BERT: {ids.shape[1]} tokens, the model reads {self.bert.cfg.max_positions}")
        visible = T.logical_not(T.equal(ids, T.tensor(torch.tensor(self.pad_id), device=ids.device)))
        return self.bert(ids, attention_mask=visible)

    def encode(self, x):
        return self._run(x)[0]

    def features(self, x):
        return self._run(x)[1]

    def forward(self, x):
        return self.head(self.drop(self.features(x)))

    def set_head(self, classes: int) -> None:
        self.head = nn.Linear(self.width, classes)

    def head_parameters(self) -> list:
        return self.head.parameters()
