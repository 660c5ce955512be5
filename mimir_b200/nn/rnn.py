"""Recurrent layers (reference: nn/rnn.go): RNN, LSTM, GRU over ``[B, T, C]`` inputs,
multi-layer, built on ``tensor.scan`` so that backward can checkpoint the loop."""
from __future__ import annotations

import math

import torch

from .. import tensor as T
from ..tensor.autograd import Param
from .module import Module, uniform_init


class _Recurrent(Module):
    gates = 1

    def __init__(self, input_size: int, hidden: int, layers: int = 1, dtype=torch.float32):
        self.hidden, self.layers = hidden, layers
        bound = 1.0 / math.sqrt(hidden)
        g = self.gates * hidden
        self.w_ih = [Param(uniform_init((g, input_size if l == 0 else hidden), bound, dtype)) for l in range(layers)]
        self.w_hh = [Param(uniform_init((g, hidden), bound, dtype)) for l in range(layers)]
        self.b_ih = [Param(uniform_init((g,), bound, dtype)) for l in range(layers)]
        self.b_hh = [Param(uniform_init((g,), bound, dtype)) for l in range(layers)]

    def cell(self, x, h, c, wi, wh, bi, bh):
        raise NotImplementedError

    def forward(self, x, state=None):
        """Returns (outputs [B, T, H], final hidden [layers, B, H])."""
        ws = [p.value() for l in range(self.layers) for p in (self.w_ih[l], self.w_hh[l], self.b_ih[l], self.b_hh[l])]
        cell, hid, nl = self.cell, self.hidden, self.layers

        def run(v, *w):
            B, Tn = v.shape[0], v.shape[1]
            if v.device.type == "meta":
                return torch.empty(B, Tn, hid, dtype=v.dtype, device="meta"), torch.empty(nl, B, hid, dtype=v.dtype, device="meta")
            seq, finals = v, []
            for l in range(nl):
                wi, wh, bi, bh = w[4 * l: 4 * l + 4]
                h = torch.zeros(B, hid, dtype=v.dtype, device=v.device)
                c = torch.zeros_like(h)
                outs = []
                xin = seq @ wi.t() + bi  # input projections for every step in one product
                for t in range(Tn):
                    h, c = cell(xin[:, t], h, c, wh, bh)
                    outs.append(h)
                seq = torch.stack(outs, 1)
                finals.append(h)
            return seq, torch.stack(finals, 0)
        return T.core._node(run, (x, *ws), {}, type(self).__name__.lower())


class RNN(_Recurrent):
    gates = 1

    def cell(self, xi, h, c, wh, bh):
        return torch.tanh(xi + h @ wh.t() + bh), c


class LSTM(_Recurrent):
    gates = 4

    def cell(self, xi, h, c, wh, bh):
        i, f, g, o = (xi + h @ wh.t() + bh).chunk(4, -1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        return torch.sigmoid(o) * torch.tanh(c), c


class GRU(_Recurrent):
    gates = 3

    def cell(self, xi, h, c, wh, bh):
        hr, hz, hn = (h @ wh.t() + bh).chunk(3, -1)
        xr, xz, xn = xi.chunk(3, -1)
        r, z = torch.sigmoid(xr + hr), torch.sigmoid(xz + hz)
        n = torch.tanh(xn + r * hn)
        return (1 - z) * n + z * h, c
