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
