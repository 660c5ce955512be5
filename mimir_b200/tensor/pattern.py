"""Sparse patterns: matrices whose nonzero entries all are one (reference: tensor/pattern.go).

The adjacency matrix of a graph, or the matrix that sums edge messages into nodes, combines rows of
a dense tensor without a dense matrix: row i of ``p.matmul(x)`` sums the rows j of ``x`` with an
entry (i, j).  A pattern is built once on the host and keeps its entries sorted both by row and by
column, so a product and its gradient (the product by the transpose) each are ONE segment reduction
that reads the rows it combines where they lie and writes every output row once, in a fixed order:
results do not depend on the number of workers.  The lists move to a device the first time a product
there needs them, and stay.

``segment`` is the one primitive (tensor/segment.go): float32 rows on the host run the native kernel
``mimir_cpu_segment`` over the worker pool; other dtypes and CUDA tensors gather the rows and reduce
them per segment with ``torch.segment_reduce`` (each segment is summed by one thread, in order).
The sum is a linear map whose derivative rules name its transpose, so gradients of any order, forward
derivatives and ``vmap`` go through the same kernel.
"""
from __future__ import annotations

import ctypes

import torch

from . import core as C
from . import errors as E

SUM, MAX = 0, 1


class _Entries:
    """Entries in row-major order as compressed sparse rows: the entries of row i are those from
    ``offsets[i]`` up to ``offsets[i + 1]``."""

    def __init__(self, offsets, cols, rows, by_col):
        self.lists = {"offsets": offsets, "cols": cols, "rows": rows, "by_col": by_col,
                      "all": torch.arange(cols.numel() + 1, dtype=torch.int32),
                      "degrees": (offsets[1:] - offsets[:-1]).float()}
        self._dev = {}

    def list(self, name, device):
        """The named list on ``device`` (a torch device), cached there."""
        if device.type == "cpu":
            return self.lists[name]
        key = (name, str(device))
        t = self._dev.get(key)
        if t is None:
            t = self._dev[key] = self.lists[name].to(device)
        return t


def _offsets(keys, n):
    counts = torch.bincount(keys.long(), minlength=n) if keys.numel() else torch.zeros(n, dtype=torch.int64)
    out = torch.zeros(n + 1, dtype=torch.int32)
    out[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return out


# ------------------------------------------------------------------ the primitive
def _bind(lib):
    if not getattr(lib, "_segment_bound", False):
        lib.mimir_cpu_segment.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int]
        lib.mimir_cpu_segment.restype = ctypes.c_int
        lib._segment_bound = True
    return lib


def _segment_raw(x, offsets, lst, combine):
    """Rows of ``x`` combined in the segments that ``offsets`` cuts ``lst`` into; no autograd."""
    n_out = offsets.numel() - 1
    tail = tuple(x.shape[1:])
    if x.device.type == "cpu" and x.dtype == torch.float32 and not torch._C._functorch.is_functorch_wrapped_tensor(x):
        from .. import _native
        if _native.available():
            xc = x.contiguous()
            out = torch.empty((n_out,) + tail, dtype=torch.float32)
            inner = 1
            for d in tail:
                inner *= d
            rc = _bind(_native.lib()).mimir_cpu_segment(xc.data_ptr(), xc.shape[0], offsets.data_ptr(), lst.data_ptr(),
                                                        out.data_ptr(), n_out, inner, combine)
            if rc != 0:
                raise E.ErrIndex("segment: a list entry outside the rows of the operand")
            return out
    wide = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    rows = wide.index_select(0, lst.long())
    if not wide.dtype.is_floating_point:
        # integer rows: a prefix sum over the gathered rows, differences at the segment ends (sum only)
        if combine != SUM:
            raise E.ErrDType(f"segment maximum of {x.dtype} rows")
        sums = torch.cumsum(rows, 0)
        cs = torch.cat([torch.zeros((1,) + tail, dtype=sums.dtype, device=x.device), sums])
        o = offsets.long()
        return (cs[o[1:]] - cs[o[:-1]]).to(x.dtype)
    lengths = (offsets[1:] - offsets[:-1]).long()
    if rows.shape[0] == 0:
        out = torch.zeros((n_out,) + tail, dtype=wide.dtype, device=x.device)
    else:
        out = torch.segment_reduce(rows, "sum" if combine == SUM else "max", lengths=lengths, axis=0, unsafe=True)
        if combine == MAX:
            shape = (n_out,) + (1,) * len(tail)
            out = torch.where((lengths == 0).reshape(shape), torch.zeros((), dtype=out.dtype, device=out.device), out)
    return out.to(x.dtype)


class _SegmentSum(torch.autograd.Function):
    """``out[i] = sum_k x[lst[k]]`` over a segment per output row; ``adj`` names the lists of the
    transposed map, which is the gradient."""

    @staticmethod
    def forward(x, spec):
        offsets, lst, _ = spec.lists(x.device)
        return _segment_raw(x, offsets, lst, SUM)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.spec = inputs[1]

    @staticmethod
    def backward(ctx, g):
        return _SegmentSum.apply(g, ctx.spec.adjoint), None

    @staticmethod
    def jvp(ctx, t, _):
        return _SegmentSum.apply(t, ctx.spec)

    @staticmethod
    def vmap(info, in_dims, x, spec):
        # the batch axis moves behind the rows, among the dimensions a segment keeps
        d = in_dims[0]
        if d is None:
            return _SegmentSum.apply(x, spec), None
        return _SegmentSum.apply(x.movedim(d, 1), spec), 1


class _Spec:
    """One linear map of a pattern: which entries' list holds the segment offsets, which list names
    the operand's rows, how many rows the operand must have, and the transposed map."""

    __slots__ = ("seg", "off", "src", "rows", "n_in", "adjoint")

    def __init__(self, seg, off, src, rows, n_in):
        self.seg, self.off, self.src, self.rows, self.n_in, self.adjoint = seg, off, src, rows, n_in, None

    def lists(self, device):
        offsets, lst = self.seg.list(self.off, device), self.src.list(self.rows, device)
        return offsets, lst, None

    @property
    def n_out(self):
        return self.seg.lists[self.off].numel() - 1


def _pair(a: _Spec, b: _Spec):
    a.adjoint, b.adjoint = b, a
    return a, b


def _apply(spec: _Spec, x, what: str):
    if not isinstance(x, C.Tensor):
        x = C.tensor(x)
    if x._err is not None:
        return x
    shape = tuple(x.shape)
    if not shape or shape[0] != spec.n_in:
        return C._error_tensor(E.ErrShape(f"pattern: {what} wants {spec.n_in} rows, got shape {shape}"))

    if C._TRACE is not None:
        return _as_dense_product(spec, x)

    def run(v):
        if v.device.type == "meta":
            return torch.empty((spec.n_out,) + tuple(v.shape[1:]), dtype=v.dtype, device="meta")
        return _SegmentSum.apply(v, spec)
    return C._node(run, (x,), {}, "segment", known=((spec.n_out,) + shape[1:], x.dtype))


DENSE_EXPORT_CELLS = 1 << 24


def _as_dense_product(spec: _Spec, x):
    """While a graph exporter listens, a segment sum is written as the product by its 0 / 1 / count matrix (a
    constant of the graph), which the graph vocabulary has a word for.  Meant for graphs small enough to hold
    that matrix: ``DENSE_EXPORT_CELLS`` cells at most."""
    n_out, n_in = spec.n_out, spec.n_in
    if n_out * n_in > DENSE_EXPORT_CELLS:
        return C._error_tensor(E.ErrUnsupported(f"export: a sparse pattern of {n_out} x {n_in} is too large to export as a dense matrix"))
    offsets, lst, _ = spec.lists(torch.device("cpu"))
    rows = torch.repeat_interleave(torch.arange(n_out), (offsets[1:] - offsets[:-1]).long())
    dense = torch.zeros(n_out, n_in)
    dense.index_put_((rows, lst.long()[:rows.numel()]), torch.ones(rows.numel()), accumulate=True)
    shape = tuple(x.shape)
    flat = C.reshape(x, (shape[0], -1)) if len(shape) != 2 else x
    wide = C.cast(flat, torch.float32) if flat.dtype != torch.float32 else flat
    y = C.matmul(C.tensor(dense, device=x.device), wide)
    y = C.cast(y, x.dtype) if y.dtype != x.dtype else y
    return C.reshape(y, (n_out,) + shape[1:]) if len(shape) != 2 else y


class Pattern:
    """The ``rows x cols`` pattern with an entry at ``(row[k], col[k])`` for each k, like the coordinate
    lists of ``torch.sparse_coo_tensor``; an entry listed twice counts twice.  Entries out of range
    raise ``ErrIndex``, lists of different lengths ``ErrShape`` (tensor/pattern.go:77-106)."""

    def __init__(self, rows: int, cols: int, row, col):
        row = torch.as_tensor(row).reshape(-1).to(torch.int64)
        col = torch.as_tensor(col).reshape(-1).to(torch.int64)
        if rows < 0 or cols < 0 or rows >= 2**31 - 1 or cols >= 2**31 - 1:
            raise E.ErrShape(f"pattern of {rows} x {cols}")
        if row.numel() != col.numel() or row.numel() >= 2**31 - 1:
            raise E.ErrShape(f"pattern of {row.numel()} rows and {col.numel()} columns of entries")
        if row.numel():
            bad = (row < 0) | (row >= rows) | (col < 0) | (col >= cols)
            if bool(bad.any()):
                k = int(bad.nonzero()[0])
                raise E.ErrIndex(f"entry ({int(row[k])}, {int(col[k])}) of a pattern of {rows} x {cols}")
        # sorting stably by row puts the entries in row-major order with ties in the order given; the
        # stable order of their columns then is the transpose's row-major order
        order = torch.argsort(row, stable=True)
        by_rows, by_cols = row[order].to(torch.int32), col[order].to(torch.int32)
        by_col = torch.argsort(by_cols.long(), stable=True).to(torch.int32)
        by = _Entries(_offsets(by_rows, rows), by_cols, by_rows, by_col)
        q = by_col.long()
        tr_pos = torch.empty_like(by_col)
        tr_pos[q] = torch.arange(q.numel(), dtype=torch.int32)
        tr = _Entries(_offsets(by_cols, cols), by_rows[q], by_cols[q], tr_pos)
        self.rows, self.cols, self._by, self._tr, self._t = rows, cols, by, tr, None
        n = by_cols.numel()
        # the product and the four maps between rows / columns and entries, each paired with its transpose
        mm, mm_t = _pair(_Spec(by, "offsets", by, "cols", cols), _Spec(tr, "offsets", tr, "cols", rows))
        at_cols, col_sum = _pair(_Spec(by, "all", by, "cols", cols), _Spec(tr, "offsets", by, "by_col", n))
        at_rows, row_sum = _pair(_Spec(by, "all", by, "rows", rows), _Spec(by, "offsets", by, "all", n))
        self._maps = {"matmul": mm, "matmul_t": mm_t, "at_cols": at_cols, "col_sum": col_sum, "at_rows": at_rows, "row_sum": row_sum}

    # -- description
    @property
    def shape(self):
        return self.rows, self.cols

    @property
    def entries(self) -> int:
        return int(self._by.lists["cols"].numel())

    def transpose(self) -> "Pattern":
        """The ``cols x rows`` pattern with an entry (j, i) for each (i, j) here; built on first use and kept."""
        return self._t if self._t is not None else _transpose_of(self)

    @property
    def T(self) -> "Pattern":
        return self.transpose()

    def degrees(self):
        """The float32 number of entries of each row."""
        return C.from_torch(self._by.lists["degrees"].clone())

    def coo(self):
        """``(row, col)`` int32 lists in row-major order."""
        return self._by.lists["rows"].clone(), self._by.lists["cols"].clone()

    # -- products
    def matmul(self, x):
        """Row i of the result ``[rows, D...]`` sums the rows j of ``x [cols, D...]`` with an entry (i, j),
        in the order of j; a row without entries is zero.  Half inputs are summed in float32 and rounded once."""
        return _apply(self._maps["matmul"], x, "product")

    def mean(self, x):
        """The product divided, row by row, by the number of entries of the row (zero for an empty row)."""
        y = self.matmul(x)
        if y._err is not None:
            return y
        if not y.dtype.is_floating_point:
            return C._error_tensor(E.ErrDType(f"pattern: mean of {y.dtype} rows"))
        d = torch.clamp(self._by.lists["degrees"], min=1.0).reshape((self.rows,) + (1,) * (len(y.shape) - 1))
        return y / C.tensor(d, device=y.device)

    def max(self, x):
        """Elementwise maximum of the rows j of ``x`` with an entry (i, j); zero for a row without entries;
        NaN propagates.  The gradient of an element is shared evenly between the rows that tie for it."""
        spec = self._maps["matmul"]
        if not isinstance(x, C.Tensor):
            x = C.tensor(x)
        if x._err is not None:
            return x
        shape = tuple(x.shape)
        if not shape or shape[0] != self.cols:
            return C._error_tensor(E.ErrShape(f"pattern: maximum wants {self.cols} rows, got shape {shape}"))
        if not x.dtype.is_floating_point:
            return C._error_tensor(E.ErrDType(f"pattern: maximum of {x.dtype} rows"))

        def top(v):
            if v.device.type == "meta":
                return torch.empty((spec.n_out,) + tuple(v.shape[1:]), dtype=v.dtype, device="meta")
            offsets, lst, _ = spec.lists(v.device)
            return _segment_raw(v.detach(), offsets, lst, MAX)
        if C._TRACE is not None:
            # an exporter listens: the maximum over a row's entries from the dense 0 / 1 matrix (small graphs)
            if self.rows * self.cols > DENSE_EXPORT_CELLS:
                return C._error_tensor(E.ErrUnsupported(f"export: a sparse pattern of {self.rows} x {self.cols} is too large to export as a dense matrix"))
            has = C.tensor((self.dense() > 0).float().reshape((self.rows, self.cols) + (1,) * (len(shape) - 1)), device=x.device)
            cand = C.where(C.less(0.0, has), C.unsqueeze(x, 0), -float("inf"))
            top_rows = C.max_(cand, 1)
            deg = C.tensor(self._by.lists["degrees"].reshape((self.rows,) + (1,) * (len(shape) - 1)), device=x.device)
            best = C.where(C.less(0.0, deg), top_rows, 0.0)
        else:
            best = C.detach(C._node(top, (C.detach(x),), {}, "segment_max", known=((self.rows,) + shape[1:], x.dtype)))
        # the maximum again as a sum over the entries that hold it, divided by their number: the same
        # value, and a linear map of x whose derivatives share a tie evenly
        picked = self.at_cols(x)
        hit = C.cast(C.equal(C.detach(picked), self.at_rows(best)), x.dtype)
        n = C.maximum(self.row_sum(hit), 1.0)
        y = self.row_sum(picked * hit) / n
        return C.where(C.equal(best, best), y, best)          # a NaN maximum stays NaN

    # -- maps between rows / columns and entries ([entries, D...] in row-major order)
    def at_cols(self, x):
        """The row of ``x [cols, D...]`` at the column of each entry."""
        return _apply(self._maps["at_cols"], x, "column gather")

    def col_sum(self, v):
        """``v [entries, D...]`` summed over the entries of each column."""
        return _apply(self._maps["col_sum"], v, "column sum")

    def at_rows(self, y):
        """The row of ``y [rows, D...]`` at the row of each entry."""
        return _apply(self._maps["at_rows"], y, "row gather")

    def row_sum(self, v):
        """``v [entries, D...]`` summed over the entries of each row."""
        return _apply(self._maps["row_sum"], v, "row sum")

    def dense(self):
        """The pattern as a dense float32 matrix (entries listed twice count twice)."""
        r, c = self.coo()
        out = torch.zeros(self.rows, self.cols)
        out.index_put_((r.long(), c.long()), torch.ones(r.numel()), accumulate=True)
        return out


def _transpose_of(p: Pattern) -> Pattern:
    r, c = p.coo()
    t = Pattern(p.cols, p.rows, c, r)
    t._t, p._t = p, t
    return t


def segment(x, offsets, lst, combine="sum"):
    """The primitive by itself: rows ``x[lst[k]]`` combined per segment ``[offsets[i], offsets[i+1])``;
    ``combine`` is "sum" or "max".  No derivative is recorded: patterns carry the rules."""
    offsets = torch.as_tensor(offsets, dtype=torch.int32)
    lst = torch.as_tensor(lst, dtype=torch.int32)
    code = {"sum": SUM, "max": MAX}[combine]
    if not isinstance(x, C.Tensor):
        x = C.tensor(x)

    def run(v):
        if v.device.type == "meta":
            return torch.empty((offsets.numel() - 1,) + tuple(v.shape[1:]), dtype=v.dtype, device="meta")
        return _segment_raw(v.detach(), offsets.to(v.device), lst.to(v.device), code)
    return C.detach(C._node(run, (x,), {}, "segment"))
