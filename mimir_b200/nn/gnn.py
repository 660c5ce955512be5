"""Graph layers (reference: nn/gnn.go): a ``Graph`` whose edges carry messages from source to target,
and the GCN / GraphSAGE / GAT convolutions.

Node features have a row per node ``[nodes, F...]`` and edge features a row per edge ``[edges, F...]``.
``source`` / ``target`` read the features of each edge's end points, ``sum`` / ``mean`` / ``max``
aggregate edge features into the target nodes, ``softmax`` normalises edge scores over the edges into
each node, and ``adjacency()`` combines neighbours' features directly, without a tensor per edge,
which is how GCN and SAGE run.  Every one of them is a product by a sparse ``Pattern`` that the graph
builds the first time it is needed and keeps, so each is one segment kernel forward and one backward,
with results that do not depend on the number of workers.
"""
from __future__ import annotations

import math
import threading

import torch

from .. import tensor as T
from ..tensor import errors as E
from ..tensor.autograd import Param
from ..tensor.pattern import Pattern
from .module import Linear, Module, uniform_init


class Graph:
    """Directed edges ``src[e] -> dst[e]`` over ``nodes`` nodes, like PyTorch Geometric's ``edge_index``;
    repeated edges count as often as they appear.  End points outside ``[0, nodes)`` raise ``ErrIndex``."""

    def __init__(self, nodes: int, src, dst):
        src = torch.as_tensor(src).reshape(-1).to(torch.int32)
        dst = torch.as_tensor(dst).reshape(-1).to(torch.int32)
        if src.numel() != dst.numel():
            raise E.ErrShape(f"graph: {src.numel()} sources and {dst.numel()} targets")
        if src.numel() and (int(src.min()) < 0 or int(dst.min()) < 0 or int(src.max()) >= nodes or int(dst.max()) >= nodes):
            raise E.ErrIndex(f"graph: an edge end point outside [0, {nodes})")
        self.n, self.src, self.dst = int(nodes), src, dst
        self._lock = threading.Lock()
        self._patterns: dict = {}
        self._loops = None
        self._norms: dict = {}

    @classmethod
    def from_edge_index(cls, nodes: int, edge_index) -> "Graph":
        """From an integer edge index ``[2, edges]``: sources in its first row, targets in its second."""
        ei = edge_index.data() if isinstance(edge_index, T.Tensor) else torch.as_tensor(edge_index)
        if ei.dim() != 2 or ei.shape[0] != 2 or ei.dtype.is_floating_point:
            raise E.ErrShape(f"graph: edge index of shape {tuple(ei.shape)} and dtype {ei.dtype}, want integers [2, edges]")
        return cls(nodes, ei[0].cpu(), ei[1].cpu())

    @property
    def nodes(self) -> int:
        return self.n

    @property
    def edges(self) -> int:
        return int(self.src.numel())

    @property
    def in_degree(self):
        return torch.bincount(self.dst.long(), minlength=self.n).float()

    @property
    def out_degree(self):
        return torch.bincount(self.src.long(), minlength=self.n).float()

    def with_self_loops(self) -> "Graph":
        """This graph with exactly one edge from every node to itself: the loops it has are left out and
        one per node is added after the other edges (PyTorch Geometric's ``remove_self_loops`` then
        ``add_self_loops``).  The result is kept."""
        with self._lock:
            if self._loops is None:
                keep = self.src != self.dst
                loop = torch.arange(self.n, dtype=torch.int32)
                self._loops = Graph(self.n, torch.cat([self.src[keep], loop]), torch.cat([self.dst[keep], loop]))
            return self._loops

    def _pattern(self, kind: str) -> Pattern:
        with self._lock:
            p = self._patterns.get(kind)
            if p is None:
                e = torch.arange(self.edges, dtype=torch.int32)
                if kind == "source":          # edges x nodes, an entry at (e, src[e])
                    p = Pattern(self.edges, self.n, e, self.src)
                elif kind == "target":
                    p = Pattern(self.edges, self.n, e, self.dst)
                else:                          # nodes x nodes, an entry at (dst[e], src[e])
                    p = Pattern(self.n, self.n, self.dst, self.src)
                self._patterns[kind] = p
            return p

    def adjacency(self) -> Pattern:
        """The ``nodes x nodes`` pattern with an entry at ``(dst[e], src[e])`` per edge: its product sums
        the features of each node's in-neighbours."""
        return self._pattern("adjacency")

    # -- messages
    def source(self, x):
        """The features of each edge's source node ``[edges, F...]``."""
        return self._pattern("source").matmul(x)

    def target(self, x):
        """The features of each edge's target node ``[edges, F...]``."""
        return self._pattern("target").matmul(x)

    def sum(self, m):
        """Edge features ``[edges, F...]`` added into the target of each edge ``[nodes, F...]``."""
        return self._pattern("target").T.matmul(m)

    def mean(self, m):
        """Edge features averaged over the incoming edges of each node; zero for a node without any."""
        return self._pattern("target").T.mean(m)

    def max(self, m):
        """Elementwise maximum over the incoming edges of each node; zero for a node without any."""
        return self._pattern("target").T.max(m)

    def softmax(self, m):
        """Edge scores ``[edges, F...]`` normalised over the incoming edges of each node: e^m over the sum
        of e^m of the edges into the same target, after subtracting the target's largest score (no
        gradient flows through that shift: the result does not depend on it)."""
        shift = self.target(self.max(T.detach(m)))
        e = T.exp(m - shift)
        return e / self.target(self.sum(e))

    def degree_norm(self, device=None):
        """``D^-1/2``: the inverse square roots of the in-degrees (at least 1) as ``[nodes, 1]``, kept per device."""
        key = str(device.torch) if device is not None else "cpu"
        with self._lock:
            t = self._norms.get(key)
            if t is None:
                d = self.in_degree.clamp(min=1.0).rsqrt().reshape(self.n, 1)
                t = self._norms[key] = T.tensor(d, device=device) if device is not None else T.tensor(d)
            return t


def _glorot(fan_out: int, fan_in: int, dtype=torch.float32):
    return uniform_init((fan_out, fan_in), math.sqrt(6.0 / max(fan_in + fan_out, 1)), dtype)


class _Conv(Module):
    def forward(self, x, g: Graph):
        return self.convolve(g, x)


class GCNConv(_Conv):
    """Kipf and Welling's graph convolution, like PyTorch Geometric's ``GCNConv``: a self loop on every
    node, then ``D^-1/2 A D^-1/2 x W^T + b`` as one sum over the neighbours of each node.  Glorot-uniform
    weight ``[out, in]``, zero bias."""

    def __init__(self, cin: int, cout: int, bias: bool = True, dtype=torch.float32):
        self.weight = Param(_glorot(cout, cin, dtype), "weight")
        self.bias = Param(torch.zeros(cout, dtype=dtype), "bias") if bias else None

    def convolve(self, g: Graph, x):
        loops = g.with_self_loops()
        norm = loops.degree_norm(x.device)
        h = T.matmul_t(x, self.weight.value()) * norm
        y = loops.adjacency().matmul(h) * norm
        return y + self.bias.value() if self.bias is not None else y


class SAGEConv(_Conv):
    """GraphSAGE with the mean aggregator, like PyTorch Geometric's ``SAGEConv``:
    ``mean_j(x_j) Wl^T + b + x_i Wr^T`` with ``neighbors`` (bias) and ``root`` (no bias)."""

    def __init__(self, cin: int, cout: int, bias: bool = True, dtype=torch.float32):
        self.neighbors, self.root = Linear(cin, cout, bias, dtype), Linear(cin, cout, False, dtype)

    def convolve(self, g: Graph, x):
        return self.neighbors(g.adjacency().mean(x)) + self.root(x)


class GATConv(_Conv):
    """Graph attention (Velickovic et al.), like PyTorch Geometric's ``GATConv``: each head maps the
    features ``x W^T``, scores each edge j -> i by ``LeakyReLU(a_src . h_j + a_dst . h_i)``, normalises the
    scores over the edges into each node and sums the neighbours' features weighted by them; every node
    attends to itself as well.  The heads are concatenated, or averaged with ``mean_heads``; then the bias."""

    def __init__(self, cin: int, cout: int, heads: int = 1, slope: float = 0.2, mean_heads: bool = False,
                 bias: bool = True, dtype=torch.float32):
        heads = max(int(heads), 1)
        self.weight = Param(_glorot(heads * cout, cin, dtype), "weight")
        self.att_src = Param(_glorot(heads, cout, dtype), "att_src")
        self.att_dst = Param(_glorot(heads, cout, dtype), "att_dst")
        self.bias = Param(torch.zeros(cout if mean_heads else heads * cout, dtype=dtype), "bias") if bias else None
        self.heads, self.cout, self.slope, self.concat = heads, cout, float(slope), not mean_heads

    def convolve(self, g: Graph, x):
        loops, n = g.with_self_loops(), g.nodes
        h = T.reshape(T.matmul_t(x, self.weight.value()), (n, self.heads, self.cout))
        src = T.sum_(h * self.att_src.value(), -1)                       # [nodes, heads]
        dst = T.sum_(h * self.att_dst.value(), -1)
        s = loops.source(src) + loops.target(dst)
        s = T.leaky_relu(s, self.slope)
        alpha = loops.softmax(s)                                          # [edges, heads]
        y = loops.sum(loops.source(h) * T.unsqueeze(alpha, -1))
        y = T.reshape(y, (n, self.heads * self.cout)) if self.concat else T.mean(y, 1)
        return y + self.bias.value() if self.bias is not None else y
