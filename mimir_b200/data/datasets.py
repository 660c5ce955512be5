"""Dataset readers (reference: data/datasets/): MNIST IDX files, CSV (one file or shards),
Parquet shards, tensors mapped from a ``.mim`` file, and synthetic generators."""
from __future__ import annotations

import csv as _csv
import glob
import gzip
import os
import struct

import torch

from . import FunctionSource, Source, Stream, Tensors


# ------------------------------------------------------------------ MNIST (IDX)
def read_idx(path: str) -> torch.Tensor:
    """IDX1 / IDX3 ubyte file (optionally .gz) -> uint8 tensor."""
    op = gzip.open if path.endswith(".gz") else open
    with op(path, "rb") as f:
        data = f.read()
    zero, dtype, ndim = struct.unpack(">HBB", data[:4])
    if zero != 0 or dtype != 0x08:
        raise ValueError(f"{path}: not an unsigned-byte IDX file")
    dims = struct.unpack(">" + "I" * ndim, data[4:4 + 4 * ndim])
    body = data[4 + 4 * ndim:]
    n = 1
    for d in dims:
        n *= d
    if len(body) < n:
        raise ValueError(f"{path}: truncated ({len(body)} of {n} bytes)")
    return torch.frombuffer(bytearray(body[:n]), dtype=torch.uint8).view(*dims)


def write_idx(path: str, t: torch.Tensor) -> None:
    t = t.to(torch.uint8).contiguous()
    with open(path, "wb") as f:
        f.write(struct.pack(">HBB", 0, 0x08, t.dim()) + struct.pack(">" + "I" * t.dim(), *t.shape) + t.numpy().tobytes())


def mnist(directory: str, train: bool = True, batch_size: int = 128, shuffle: bool = True, seed: int = 0,
          normalize: bool = True) -> Tensors:
    """Images [N, 1, 28, 28] float32 (mean 0.1307 / std 0.3081 when ``normalize``), labels int64."""
    stem = "train" if train else "t10k"
    def find(kind):
        for ext in ("", ".gz"):
            for sep in ("-", "."):
                p = os.path.join(directory, f"{stem}-{kind}{sep}idx{3 if kind == 'images' else 1}-ubyte{ext}")
                if os.path.exists(p):
                    return p
        raise FileNotFoundError(f"no {stem} {kind} IDX file in {directory}")
    x = read_idx(find("images")).float().div(255.0).unsqueeze(1)
    if normalize:
        x = (x - 0.1307) / 0.3081
    y = read_idx(find("labels")).long()
    return Tensors(x, y, batch_size=batch_size, shuffle=shuffle, seed=seed)


# ------------------------------------------------------------------------- CSV
def _read_csv_native(path: str, header: bool):
    """``(names, table)`` of a CSV file of plain numbers parsed by ``mimir_cpu_csv_parse`` (pieces of the file
    in parallel), or None when the file needs the general reader (quotes, a field that is not a number, ragged
    lines)."""
    import ctypes

    import numpy as np

    from .. import _native
    with open(path, "rb") as f:
        first = f.readline()
    if not first.strip() or b'"' in first:
        return None
    names = next(_csv.reader([first.decode("utf-8", "replace").rstrip("\r\n")]))
    raw = np.fromfile(path, dtype=np.uint8)
    skip = len(first) if header else 0
    if not header:
        names = [f"c{i}" for i in range(len(names))]
    if (raw[skip:] == ord('"')).any():
        return None
    lib = _native.lib()
    if not getattr(lib, "_csv_bound", False):
        lib.mimir_cpu_csv_lines.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        lib.mimir_cpu_csv_lines.restype = ctypes.c_longlong
        lib.mimir_cpu_csv_parse.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong]
        lib.mimir_cpu_csv_parse.restype = ctypes.c_longlong
        lib._csv_bound = True
    at, size = raw.ctypes.data + skip, int(raw.size) - skip
    rows = lib.mimir_cpu_csv_lines(at, size)
    table = torch.empty(max(rows, 0), len(names), dtype=torch.float64)
    if rows < 0 or lib.mimir_cpu_csv_parse(at, size, len(names), table.data_ptr(), rows) != rows:
        return None
    return names, table


def read_csv(path: str, label: str | int | None = -1, header: bool = True, dtype=torch.float32):
    """Numeric CSV -> ``(X, y, feature_names)``; ``label`` names or indexes the target column (None: no target)."""
    data = names = None
    fast = _read_csv_native(path, header)
    if fast is not None:
        names, data = fast
    else:
        with open(path, newline="") as f:
            rows = list(_csv.reader(f))
        names = rows[0] if header else [f"c{i}" for i in range(len(rows[0]))]
        body = rows[1:] if header else rows
        data = torch.tensor([[float(v) if v != "" else float("nan") for v in r] for r in body], dtype=torch.float64)
    li = None if label is None else (names.index(label) if isinstance(label, str) else label % len(names))
    if li is None:
        return data.to(dtype), None, names
    keep = [i for i in range(len(names)) if i != li]
    return data[:, keep].to(dtype), data[:, li].to(dtype), [names[i] for i in keep]


def csv(path: str, label=-1, header=True, batch_size=32, shuffle=True, seed=0) -> Tensors:
    X, y, _ = read_csv(path, label, header)
    return Tensors(X, y, batch_size=batch_size, shuffle=shuffle, seed=seed)


class _CSVShard(Source):
    def __init__(self, path, label, header, chunk):
        self.path, self.label, self.header, self.chunk = path, label, header, chunk

    def read(self):
        X, y, _ = read_csv(self.path, self.label, self.header)
        for i in range(0, X.shape[0], self.chunk):
            yield X[i:i + self.chunk], (None if y is None else y[i:i + self.chunk])


def csv_shards(pattern: str, label=-1, header=True, batch_size=32, chunk=4096, **kw) -> Stream:
    paths = sorted(glob.glob(pattern))
    if not paths:
        raise FileNotFoundError(f"no files match {pattern!r}")
    return Stream([_CSVShard(p, label, header, chunk) for p in paths], batch_size=batch_size, **kw)


# --------------------------------------------------------------------- Parquet
class _ParquetShard(Source):
    def __init__(self, path, features, label, classes=None):
        self.path, self.features, self.label = path, features, label
        self.classes = {c: i for i, c in enumerate(classes)} if classes else None

    def read(self):
        from ..io import parquet
        f = parquet.File(self.path)
        feats = self.features or [c for c in f.columns if c != self.label]
        for g in range(f.row_groups):
            X, y = f.matrix(feats, self.label, g)
            if self.classes is not None and isinstance(y, list):
                try:
                    y = torch.tensor([self.classes[v] for v in y], dtype=torch.int64)
                except KeyError as e:
                    raise ValueError(f"{self.path}: label {e.args[0]!r} is not one of {list(self.classes)}") from None
            yield X, y


def parquet_shards(pattern, features=None, label: str | None = None, batch_size=32, classes=None, **kw) -> Stream:
    """A stream over the row groups of Parquet files (a glob pattern or a list of paths), decoded by
    the native reader.  ``classes``: the names a string label column may hold, mapped to 0, 1, ...
    (datasets.ParquetShards with datasets.Classes)."""
    paths = sorted(glob.glob(pattern)) if isinstance(pattern, str) else list(pattern)
    if not paths:
        raise FileNotFoundError(f"no files match {pattern!r}")
    return Stream([_ParquetShard(p, features, label, classes) for p in paths], batch_size=batch_size, **kw)


# ------------------------------------------------------------------ .mim mapped
def mapped(path: str, x: str = "x", y: str | None = "y", batch_size=32, shuffle=True, seed=0) -> Tensors:
    """Tensors ``x`` / ``y`` of a ``.mim`` file, read through the memory map (no copy until batched)."""
    from ..io import mim
    m = mim.open(path)
    ds = Tensors(m.tensor(x), m.tensor(y) if y and y in m else None, batch_size=batch_size, shuffle=shuffle, seed=seed)
    ds._keepalive = m
    return ds


# -------------------------------------------------------------------- synthetic
class _SyntheticShard(Source):
    """Rows generated as they are read: features uniform in [-1, 1), target 1 where a fixed direction
    of the feature space is positive (separable), every chunk a function of (seed, shard, chunk) only."""

    def __init__(self, rows: int, features: int, seed: int, shard: int, chunk: int = 65536):
        self.rows, self.features, self.seed, self.shard, self.chunk = rows, features, seed, shard, chunk
        g = torch.Generator().manual_seed(seed * 2654435761 % (1 << 62))
        self.w = torch.randn(features, generator=g)

    def read(self):
        done, c = 0, 0
        while done < self.rows:
            n = min(self.chunk, self.rows - done)
            g = torch.Generator().manual_seed((self.seed * 1000003 + self.shard) * 1000003 + c)
            x = torch.rand(n, self.features, generator=g) * 2.0 - 1.0
            yield x, (x @ self.w > 0).long()
            done += n
            c += 1


def synthetic(rows: int, features: int = 32, shards: int = 1, seed: int = 0, batch_size: int = 32, **kw) -> Stream:
    """A stream of ``rows`` generated rows over ``shards`` shards in constant memory, for scale tests
    and benchmarks (datasets.Synthetic, data/datasets/synthetic.go): nothing is stored, so the row
    count is free; the same seed gives the same rows."""
    rows, features, shards = max(int(rows), 0), max(int(features), 1), max(int(shards), 1)
    per, extra = divmod(rows, shards)
    srcs = [_SyntheticShard(per + (1 if i < extra else 0), features, seed, i) for i in range(shards)]
    return Stream([s for s in srcs if s.rows], batch_size=batch_size, **kw)


def synthetic_classification(rows=1024, features=16, classes=4, batch_size=32, seed=0, noise=0.5) -> Tensors:
    g = torch.Generator().manual_seed(seed)
    centers = torch.randn(classes, features, generator=g) * 2
    y = torch.randint(0, classes, (rows,), generator=g)
    return Tensors(centers[y] + noise * torch.randn(rows, features, generator=g), y, batch_size=batch_size, seed=seed)


def synthetic_regression(rows=1024, features=8, batch_size=32, seed=0, noise=0.1) -> Tensors:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(features, generator=g)
    X = torch.randn(rows, features, generator=g)
    return Tensors(X, X @ w + noise * torch.randn(rows, generator=g), batch_size=batch_size, seed=seed)


def synthetic_tokens(rows=256, seq=64, vocab=256, batch_size=8, seed=0) -> Tensors:
    """Next-token pairs from a random first-order Markov chain (learnable, unlike uniform noise)."""
    g = torch.Generator().manual_seed(seed)
    trans = torch.softmax(torch.randn(vocab, vocab, generator=g) * 2, 1)
    toks = torch.zeros(rows, seq + 1, dtype=torch.long)
    toks[:, 0] = torch.randint(0, vocab, (rows,), generator=g)
    for t in range(seq):
        toks[:, t + 1] = torch.multinomial(trans[toks[:, t]], 1, generator=g).squeeze(1)
    return Tensors(toks[:, :-1], toks[:, 1:], batch_size=batch_size, seed=seed)
