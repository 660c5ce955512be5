"""Recurrent layers (reference: nn/rnn.go:37-145): RNN, LSTM and GRU, stacked and optionally
bidirectional, over sequences laid out ``[T, B, C]`` (or ``[B, T, C]`` with ``batch_first``, or
``[T, C]`` for a single sequence), with the gate order and the two bias vectors of PyTorch's layers,
so weights move between the two.  ``run`` takes initial states and returns the final ones.
The whole recurrence is one node of the lazy graph; its gradients come from autograd over the loop.
"""
from __future__ import annotations

import math

import torch

from .. import tensor as T
from ..tensor.autograd import Param
from .module import Module, uniform_init


class _Recurrent(Module):
    gates = 1
    states = 1

    def __init__(self, input_size: int, hidden: int, layers: int = 1, bidirectional: bool = False, batch_first: bool = False,
                 bias: bool = True, dtype=torch.float32):
        """``layers`` stacked layers of ``hidden`` units; ``bidirectional`` runs every layer over the
        sequence in both directions and joins the two outputs; ``batch_first`` takes and returns
        ``[B, T, C]``; ``bias=False`` leaves the bias vectors out (nn.NumLayers, nn.Bidirectional,
        nn.BatchFirst, nn.NoBias)."""
        self.input_size, self.hidden, self.layers = input_size, hidden, layers
        self.bidirectional, self.batch_first, self.bias = bidirectional, batch_first, bias
        bound = 1.0 / math.sqrt(hidden)
        g, dirs = self.gates * hidden, 2 if bidirectional else 1
        self.w_ih, self.w_hh, self.b_ih, self.b_hh = [], [], [], []
        for l in range(layers):
            width = input_size if l == 0 else dirs * hidden
            for _ in range(dirs):                      # layer l, direction d sits at index l * dirs + d
                self.w_ih.append(Param(uniform_init((g, width), bound, dtype)))
                self.w_hh.append(Param(uniform_init((g, hidden), bound, dtype)))
                if bias:
                    self.b_ih.append(Param(uniform_init((g,), bound, dtype)))
                    self.b_hh.append(Param(uniform_init((g,), bound, dtype)))

    def cell(self, gi, gh, h, c):
        """One step: input and hidden pre-activations -> (h, c)."""
        raise NotImplementedError

    def run(self, x, *init):
        """``x`` and optional initial states ``[layers * directions, B, H]`` (zeros when left out;
        an LSTM takes ``h0, c0``) -> ``(outputs, h_n)`` or ``(outputs, h_n, c_n)``."""
        ns, dirs, nl, hid = self.states, 2 if self.bidirectional else 1, self.layers, self.hidden
        if init and len(init) != ns:
            return tuple(T.core._error_tensor(T.ErrShape(f"{type(self).__name__}: {len(init)} initial states, want {ns}"))
                         for _ in range(1 + ns))
        per = 4 if self.bias else 2
        ws = []
        for k in range(nl * dirs):
            ws += [self.w_ih[k].value(), self.w_hh[k].value()]
            if self.bias:
                ws += [self.b_ih[k].value(), self.b_hh[k].value()]
        if T.core._TRACE is not None:
            return self._run_in_ops(x, init)          # an exporter is listening: the recurrence as separate ops
        cell, batch_first, n_init = self.cell, self.batch_first, len(init)

        def fn(v, *rest):
            states, w = rest[:n_init], rest[n_init:]
            batched = v.dim() == 3
            if v.dim() not in (2, 3):
                raise T.ErrShape(f"recurrent layer input of rank {v.dim()}, want [T, B, C], [B, T, C] or [T, C]")
            seq = v if not batched else (v.transpose(0, 1) if batch_first else v)
            if not batched:
                seq = seq[:, None]
            Tn, B = seq.shape[0], seq.shape[1]
            if v.device.type == "meta":
                out = torch.empty(Tn, B, dirs * hid, dtype=v.dtype, device="meta")
                st = torch.empty(nl * dirs, B, hid, dtype=v.dtype, device="meta")
                if not batched:
                    out, st = out[:, 0], st[:, 0]
                elif batch_first:
                    out = out.transpose(0, 1)
                return (out,) + (st,) * ns
            zeros = torch.zeros(nl * dirs, B, hid, dtype=v.dtype, device=v.device)
            st = [(s if batched else s[:, None]) for s in states] if states else [zeros] * ns
            hs, cs = [], []
            for l in range(nl):
                outs = []
                for d in range(dirs):
                    k = l * dirs + d
                    wi, wh = w[per * k], w[per * k + 1]
                    bi, bh = (w[per * k + 2], w[per * k + 3]) if per == 4 else (None, None)
                    h = st[0][k]
                    c = st[1][k] if ns == 2 else None
                    gi_all = seq @ wi.t() if bi is None else seq @ wi.t() + bi        # the input products of every step at once
                    ys = [None] * Tn
                    for t in (range(Tn - 1, -1, -1) if d else range(Tn)):
                        gh = h @ wh.t() if bh is None else h @ wh.t() + bh
                        h, c = cell(gi_all[t], gh, h, c)
                        ys[t] = h
                    outs.append(torch.stack(ys))
                    hs.append(h)
                    cs.append(c)
                seq = outs[0] if dirs == 1 else torch.cat(outs, -1)
            out, hn = seq, torch.stack(hs)
            finals = (hn,) if ns == 1 else (hn, torch.stack(cs))
            if not batched:
                out, finals = out[:, 0], tuple(f[:, 0] for f in finals)
            elif batch_first:
                out = out.transpose(0, 1)
            return (out,) + finals
        return T.core._node(fn, (x, *init, *ws), {}, type(self).__name__.lower())

    def _run_in_ops(self, x, init):
        """The same recurrence unrolled in public tensor ops (one product, one cell per step), which is what a
        graph exporter can translate.  Batched input only."""
        ns, dirs, nl, hid = self.states, 2 if self.bidirectional else 1, self.layers, self.hidden
        if len(x.shape) != 3:
            return tuple(T.core._error_tensor(T.ErrShape("recurrent layer: export needs batched input [T, B, C] or [B, T, C]"))
                         for _ in range(1 + ns))
        seq = T.transpose(x, 0, 1) if self.batch_first else x
        steps, batch = seq.shape[0], seq.shape[1]
        hs, cs = [], []
        for l in range(nl):
            outs = []
            for d in range(dirs):
                k = l * dirs + d
                wi, wh = self.w_ih[k].value(), self.w_hh[k].value()
                bi, bh = (self.b_ih[k].value(), self.b_hh[k].value()) if self.bias else (None, None)
                if init:
                    h = T.reshape(T.shrink(init[0], ((k, k + 1), (0, batch), (0, hid))), (batch, hid))
                    c = T.reshape(T.shrink(init[1], ((k, k + 1), (0, batch), (0, hid))), (batch, hid)) if ns == 2 else None
                else:
                    # zeros shaped by the batch of the input, so a dynamic batch stays dynamic
                    first = T.reshape(T.shrink(seq, ((0, 1), (0, batch), (0, 1))), (batch, 1))
                    zero = T.expand(first * 0.0, (batch, hid))
                    h, c = zero, (zero if ns == 2 else None)
                gi_all = T.matmul_t(seq, wi, bi)                                  # the input products of every step at once
                ys = [None] * steps
                for t in (range(steps - 1, -1, -1) if d else range(steps)):
                    gi = T.reshape(T.shrink(gi_all, ((t, t + 1), (0, batch), (0, gi_all.shape[2]))), (batch, gi_all.shape[2]))
                    h, c = self.cell_ops(gi, T.matmul_t(h, wh, bh), h, c)
                    ys[t] = h
                outs.append(T.stack(ys, 0))
                hs.append(h)
                cs.append(c)
            seq = outs[0] if dirs == 1 else T.cat(outs, -1)
        out = T.transpose(seq, 0, 1) if self.batch_first else seq
        finals = (T.stack(hs, 0),) if ns == 1 else (T.stack(hs, 0), T.stack(cs, 0))
        return (out,) + finals

    def cell_ops(self, gi, gh, h, c):
        """``cell`` in lazy tensor ops."""
        raise NotImplementedError

    def forward(self, x, *init):
        """The outputs and the final hidden state (``run`` also gives an LSTM's final cell state)."""
        res = self.run(x, *init)
        return res[0], res[1]


class RNN(_Recurrent):
    gates = 1

    def __init__(self, input_size: int, hidden: int, layers: int = 1, relu: bool = False, **kw):
        """``relu``: ReLU instead of tanh (nn.RNNReLU)."""
        super().__init__(input_size, hidden, layers, **kw)
        self.relu = relu

    def cell(self, gi, gh, h, c):
        return (torch.relu(gi + gh) if self.relu else torch.tanh(gi + gh)), c

    def cell_ops(self, gi, gh, h, c):
        return (T.relu(gi + gh) if self.relu else T.tanh(gi + gh)), c


class LSTM(_Recurrent):
    gates = 4
    states = 2

    def cell(self, gi, gh, h, c):
        i, f, g, o = (gi + gh).chunk(4, -1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        return torch.sigmoid(o) * torch.tanh(c), c

    def cell_ops(self, gi, gh, h, c):
        H = self.hidden
        i, f, g, o = T.split(gi + gh, [H, H, H, H], -1)
        c = T.sigmoid(f) * c + T.sigmoid(i) * T.tanh(g)
        return T.sigmoid(o) * T.tanh(c), c


class GRU(_Recurrent):
    gates = 3

    def cell(self, gi, gh, h, c):
        ir, iz, inn = gi.chunk(3, -1)
        hr, hz, hn = gh.chunk(3, -1)
        r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
        n = torch.tanh(inn + r * hn)
        return (1 - z) * n + z * h, c

    def cell_ops(self, gi, gh, h, c):
        H = self.hidden
        ir, iz, inn = T.split(gi, [H, H, H], -1)
        hr, hz, hn = T.split(gh, [H, H, H], -1)
        r, z = T.sigmoid(ir + hr), T.sigmoid(iz + hz)
        n = T.tanh(inn + r * hn)
        return (1.0 - z) * n + z * h, c
