"""Graph layers (reference: nn/gnn.go): a ``Graph`` in CSR form and GCN / GraphSAGE /
GAT convolutions built on segment sums and segment softmax (tensor/pattern.go)."""
from __future__ import annotations

import math

import torch

from .. import tensor as T
from ..tensor.autograd import Param
from .module import Linear, Module, uniform_init


class Graph:
    """Directed edges ``src -> dst`` over ``n`` nodes, kept sorted by destination."""

    def __init__(self, n: int, src, dst, self_loops: bool = False):
        src, dst = torch.as_tensor(src, dtype=torch.int64), torch.as_tensor(dst, dtype=torch.int64)
        if self_loops:
            loop = torch.arange(n)
            src, dst = torch.cat([src, loop]), torch.cat([dst, loop])
        order = torch.argsort(dst, stable=True)
        self.n, self.src, self.dst = n, src[order], dst[order]
        self.in_degree = torch.bincount(self.dst, minlength=n).float()
        self.out_degree = torch.bincount(self.src, minlength=n).float()


def _aggregate(h, g: Graph, weight=None, mean=False):
    msg = h[g.src.to(h.device)]
    if weight is not None:
        msg = msg * weight.unsqueeze(-1)
    out = torch.zeros(g.n, h.shape[1], dtype=h.dtype, device=h.device).index_add_(0, g.dst.to(h.device), msg)
    if mean:
        out = out / g.in_degree.to(h.device).clamp_min(1).unsqueeze(-1)
    return out


class GCNConv(Module):
    def __init__(self, cin, cout):
        self.lin = Linear(cin, cout)

    def forward(self, x, g: Graph):
        gl = Graph(g.n, g.src, g.dst, self_loops=True)
        deg = gl.in_degree
        norm = (deg[gl.src] * deg[gl.dst]).rsqrt()
        return T.core._node(lambda h: torch.empty(h.shape, dtype=h.dtype, device="meta") if h.device.type == "meta"
                            else _aggregate(h, gl, norm.to(h.device)), (self.lin(x),), {}, "gcn")


class SAGEConv(Module):
    def __init__(self, cin, cout):
        self.self_lin, self.neigh_lin = Linear(cin, cout), Linear(cin, cout, bias=False)

    def forward(self, x, g: Graph):
        agg = T.core._node(lambda h: torch.empty(h.shape, dtype=h.dtype, device="meta") if h.device.type == "meta"
                           else _aggregate(h, g, mean=True), (x,), {}, "sage_mean")
        return self.self_lin(x) + self.neigh_lin(agg)


class GATConv(Module):
    def __init__(self, cin, cout, heads=1, slope=0.2):
        self.lin = Linear(cin, cout * heads, bias=False)
        bound = 1.0 / math.sqrt(cout)
        self.att_src = Param(uniform_init((heads, cout), bound))
        self.att_dst = Param(uniform_init((heads, cout), bound))
        self.heads, self.cout, self.slope = heads, cout, slope

    def forward(self, x, g: Graph):
        gl = Graph(g.n, g.src, g.dst, self_loops=True)
        H, C, slope = self.heads, self.cout, self.slope

        def run(h, a_s, a_d):
            if h.device.type == "meta":
                return torch.empty(h.shape[0], H * C, dtype=h.dtype, device="meta")
            hv = h.view(-1, H, C)
            src, dst = gl.src.to(h.device), gl.dst.to(h.device)
            e = torch.nn.functional.leaky_relu((hv * a_s).sum(-1)[src] + (hv * a_d).sum(-1)[dst], slope)
            emax = torch.full((gl.n, H), float("-inf"), dtype=e.dtype, device=h.device).scatter_reduce(0, dst[:, None].expand(-1, H), e, "amax")
            w = (e - emax[dst]).exp()
            denom = torch.zeros(gl.n, H, dtype=e.dtype, device=h.device).index_add_(0, dst, w)
            alpha = w / denom[dst]
            out = torch.zeros(gl.n, H, C, dtype=h.dtype, device=h.device).index_add_(0, dst, hv[src] * alpha.unsqueeze(-1))
            return out.reshape(gl.n, H * C)
        return T.core._node(run, (self.lin(x), self.att_src.value(), self.att_dst.value()), {}, "gat")
