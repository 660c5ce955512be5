"""Parquet reading for flat schemas (reference: io/parquet/parquet.go:15-53, reader.go:122-260).

The decoder is this package's own (``csrc/parquet.cpp`` in the native library: Thrift compact
footer and page headers, data pages V1 / V2, PLAIN / RLE / dictionary / DELTA_BINARY_PACKED /
DELTA_LENGTH_BYTE_ARRAY / DELTA_BYTE_ARRAY / BYTE_STREAM_SPLIT, Snappy decoded in place, gzip and
zstd through the system libraries).  One column chunk of one row group is decoded per call, so a
data set streams shard by shard and row group by row group.  A column is read by its physical type;
its logical type is reported, not applied.  Nested columns, INT96, encrypted files and the LZ4 /
Brotli / LZO codecs are listed but refused with ``ErrUnsupported``; a malformed file fails with
``ErrFormat`` whatever its bytes.  There is no writer in the reference; ``write`` here produces test
and export files through pyarrow.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from .. import _native

BOOLEAN, INT32, INT64, INT96, FLOAT, DOUBLE, BYTE_ARRAY, FIXED_LEN_BYTE_ARRAY = range(8)
TYPE_NAMES = ["BOOLEAN", "INT32", "INT64", "INT96", "FLOAT", "DOUBLE", "BYTE_ARRAY", "FIXED_LEN_BYTE_ARRAY"]
_NP = {BOOLEAN: np.uint8, INT32: np.int32, INT64: np.int64, FLOAT: np.float32, DOUBLE: np.float64}
_CONVERTED = {0: "UTF8", 1: "MAP", 2: "MAP_KEY_VALUE", 3: "LIST", 4: "ENUM", 5: "DECIMAL", 6: "DATE", 7: "TIME_MILLIS",
              8: "TIME_MICROS", 9: "TIMESTAMP_MILLIS", 10: "TIMESTAMP_MICROS", 11: "UINT_8", 12: "UINT_16", 13: "UINT_32",
              14: "UINT_64", 15: "INT_8", 16: "INT_16", 17: "INT_32", 18: "INT_64", 19: "JSON", 20: "BSON", 21: "INTERVAL"}


class ParquetError(Exception):
    pass


class ErrFormat(ParquetError):
    """A malformed file."""


class ErrUnsupported(ParquetError):
    """A feature of the format that this reader does not implement."""


@dataclass(frozen=True)
class Column:
    """A leaf column of the schema (reference: parquet.go:112-135)."""
    name: str            # the path in the schema, "a.b" for a nested column
    type: int            # physical type
    nullable: bool
    nested: bool         # below a group or repeated: listed, cannot be read
    type_length: int     # FIXED_LEN_BYTE_ARRAY
    logical: str         # LogicalType or ConvertedType name, "" when absent
    scale: int = 0
    precision: int = 0

    @property
    def type_name(self) -> str:
        return TYPE_NAMES[self.type] if 0 <= self.type < 8 else f"TYPE({self.type})"


def _bind(lib):
    if getattr(lib, "_pq_bound", False):
        return lib
    c = ctypes
    lib.mimir_pq_open.argtypes = [c.c_char_p, c.POINTER(c.c_void_p)]
    lib.mimir_pq_close.argtypes = [c.c_void_p]
    lib.mimir_pq_close.restype = None
    lib.mimir_pq_last_error.argtypes = [c.c_void_p]
    lib.mimir_pq_last_error.restype = c.c_char_p
    lib.mimir_pq_counts.argtypes = [c.c_void_p, c.POINTER(c.c_longlong), c.POINTER(c.c_int), c.POINTER(c.c_int)]
    lib.mimir_pq_column.argtypes = [c.c_void_p, c.c_int, c.c_char_p, c.c_int, c.c_char_p, c.c_int, c.POINTER(c.c_int)]
    lib.mimir_pq_group_rows.argtypes = [c.c_void_p, c.c_int]
    lib.mimir_pq_group_rows.restype = c.c_longlong
    lib.mimir_pq_meta.argtypes = [c.c_void_p, c.c_int, c.POINTER(c.c_char_p), c.POINTER(c.c_longlong),
                                  c.POINTER(c.c_char_p), c.POINTER(c.c_longlong)]
    lib.mimir_pq_decode.argtypes = [c.c_void_p, c.c_int, c.c_int]
    lib.mimir_pq_result.argtypes = [c.c_void_p, c.POINTER(c.c_int), c.POINTER(c.c_longlong), c.POINTER(c.c_void_p),
                                    c.POINTER(c.c_longlong), c.POINTER(c.c_void_p), c.POINTER(c.c_void_p),
                                    c.POINTER(c.c_longlong)]
    lib.mimir_pq_decode_into.argtypes = [c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_longlong, c.c_void_p, c.POINTER(c.c_longlong)]
    lib._pq_bound = True
    return lib


def _raise(code: int, msg: str):
    if code == 2:
        raise ErrUnsupported("parquet: unsupported feature: " + msg)
    if code == 3:
        raise OSError("parquet: " + msg)
    if code == 4:
        raise IndexError("parquet: " + msg)
    raise ErrFormat("parquet: malformed file: " + msg)


class File:
    """An open Parquet file: its metadata and a mapping of its bytes."""

    def __init__(self, path: str):
        self._lib = _bind(_native.lib())
        self._h = ctypes.c_void_p()
        self.path = str(path)
        rc = self._lib.mimir_pq_open(self.path.encode(), ctypes.byref(self._h))
        if rc:
            _raise(rc, (self._lib.mimir_pq_last_error(None) or b"").decode("utf-8", "replace"))
        rows, groups, cols = ctypes.c_longlong(), ctypes.c_int(), ctypes.c_int()
        self._lib.mimir_pq_counts(self._h, ctypes.byref(rows), ctypes.byref(groups), ctypes.byref(cols))
        self.rows, self.row_groups = rows.value, groups.value
        self._cols: list[Column] = []
        name, logical, info = ctypes.create_string_buffer(1024), ctypes.create_string_buffer(64), (ctypes.c_int * 7)()
        for i in range(cols.value):
            self._lib.mimir_pq_column(self._h, i, name, 1024, logical, 64, info)
            lg = logical.value.decode() or _CONVERTED.get(info[4], "")
            self._cols.append(Column(name.value.decode("utf-8", "replace"), info[0], bool(info[2]), bool(info[3]), info[1], lg,
                                     info[5], info[6]))
        self._index = {c.name: i for i, c in enumerate(self._cols)}

    # ---- metadata -------------------------------------------------------------------------
    def close(self) -> None:
        if self._h:
            self._lib.mimir_pq_close(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def columns(self) -> list:
        return [c.name for c in self._cols]

    def column_info(self) -> list:
        return list(self._cols)

    def column(self, name: str) -> int:
        """Index of the column called ``name``; ``KeyError`` when there is none."""
        return self._index[name]

    def row_group_rows(self, group: int) -> int:
        n = self._lib.mimir_pq_group_rows(self._h, group)
        if n < 0:
            raise IndexError(f"parquet: no row group {group}")
        return n

    def _meta(self, i):
        k, v = ctypes.c_char_p(), ctypes.c_char_p()
        kl, vl = ctypes.c_longlong(), ctypes.c_longlong()
        n = self._lib.mimir_pq_meta(self._h, i, ctypes.byref(k), ctypes.byref(kl), ctypes.byref(v), ctypes.byref(vl))
        key = ctypes.string_at(k, kl.value) if kl.value else b""
        val = ctypes.string_at(v, vl.value) if i >= 0 and vl.value else b""
        return n, key, val

    @property
    def created_by(self) -> str:
        return self._meta(-1)[1].decode("utf-8", "replace")

    def metadata(self) -> dict:
        n = self._meta(-1)[0]
        out = {}
        for i in range(n):
            _, k, v = self._meta(i)
            out[k.decode("utf-8", "replace")] = v
        return out

    def schema(self) -> dict:
        return {c.name: c.type_name + (f"({c.logical})" if c.logical else "") for c in self._cols}

    # ---- data -------------------------------------------------------------------------------
    def read_column(self, group: int, column, strings: bool = True):
        """Decodes one column chunk.  Returns ``(values, nulls)``: ``values`` is a torch tensor for
        numeric and boolean columns (nulls hold 0), a list of ``str`` / ``bytes`` for BYTE_ARRAY and
        FIXED_LEN_BYTE_ARRAY (nulls hold ``None``); ``nulls`` is a bool tensor, or ``None`` for a
        required column."""
        ci = self._index[column] if isinstance(column, str) else int(column)
        col = self._cols[ci] if 0 <= ci < len(self._cols) else None
        if col is not None and col.type in _NP and not col.nested:
            return self._read_fixed(int(group), ci, col)
        rc = self._lib.mimir_pq_decode(self._h, int(group), ci)
        if rc:
            _raise(rc, (self._lib.mimir_pq_last_error(self._h) or b"").decode("utf-8", "replace"))
        ty, cnt, nb, nc = ctypes.c_int(), ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_longlong()
        vals, offs, nulls = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        self._lib.mimir_pq_result(self._h, ctypes.byref(ty), ctypes.byref(cnt), ctypes.byref(vals), ctypes.byref(nb),
                                  ctypes.byref(offs), ctypes.byref(nulls), ctypes.byref(nc))
        n, col = cnt.value, self._cols[ci]
        null_t = None
        if col.nullable:
            null_t = torch.from_numpy(np.frombuffer(ctypes.string_at(nulls, n), np.uint8).astype(bool)) if n else torch.zeros(0, dtype=torch.bool)
        raw = ctypes.string_at(vals, nb.value) if nb.value else b""
        if col.type in _NP:
            arr = np.frombuffer(raw, _NP[col.type]).copy()
            t = torch.from_numpy(arr)
            return (t.bool() if col.type == BOOLEAN else t), null_t
        if col.type == FIXED_LEN_BYTE_ARRAY:
            w = col.type_length
            items = [raw[i * w:(i + 1) * w] for i in range(n)]
        else:
            o = np.frombuffer(ctypes.string_at(offs, (n + 1) * 8), np.int64) if n else np.zeros(1, np.int64)
            text = strings and col.logical in ("STRING", "UTF8", "ENUM", "JSON")
            items = [raw[o[i]:o[i + 1]] for i in range(n)]
            if text:
                items = [b.decode("utf-8", "replace") for b in items]
        if null_t is not None and nc.value:
            mask = null_t.tolist()
            items = [None if m else v for v, m in zip(items, mask)]
        return items, null_t

    def _read_fixed(self, group: int, ci: int, col, out: torch.Tensor | None = None):
        """A numeric / boolean column chunk decoded straight into a tensor (``out``: a contiguous
        destination of the chunk's length and the column's dtype)."""
        n = self.row_group_rows(group)
        np_dt = _NP[col.type]
        if out is None:
            out = torch.from_numpy(np.empty(n, dtype=np_dt))
        nulls = torch.empty(n, dtype=torch.uint8) if col.nullable else None
        nc = ctypes.c_longlong()
        rc = self._lib.mimir_pq_decode_into(self._h, group, ci, out.data_ptr(), n * out.element_size(),
                                            nulls.data_ptr() if nulls is not None else None, ctypes.byref(nc))
        if rc:
            _raise(rc, (self._lib.mimir_pq_last_error(self._h) or b"").decode("utf-8", "replace"))
        if nulls is not None:
            nulls = nulls.bool() if nc.value else torch.zeros(n, dtype=torch.bool)
        return (out.bool() if col.type == BOOLEAN else out), nulls

    def read(self, columns=None, row_group: int | None = None) -> dict:
        """Column name -> tensor (numeric / bool; nulls of float columns become NaN) or list
        (strings / bytes), over one row group or the whole file."""
        names = list(columns) if columns is not None else [c.name for c in self._cols if not c.nested]
        groups = [row_group] if row_group is not None else list(range(self.row_groups))
        out = {}
        for name in names:
            parts = []
            for g in groups:
                v, nulls = self.read_column(g, name)
                if torch.is_tensor(v) and nulls is not None and bool(nulls.any()):
                    if not v.dtype.is_floating_point:
                        v = v.double()
                    v = v.masked_fill(nulls, float("nan"))
                parts.append(v)
            if not parts:
                ty = self._cols[self._index[name]].type
                out[name] = torch.zeros(0, dtype=torch.from_numpy(np.zeros(0, _NP[ty])).dtype) if ty in _NP else []
            elif torch.is_tensor(parts[0]):
                dt = torch.float64 if any(p.dtype == torch.float64 for p in parts) else parts[0].dtype
                out[name] = torch.cat([p.to(dt) for p in parts]) if len(parts) > 1 else parts[0]
            else:
                out[name] = [x for p in parts for x in p]
        return out

    def iter_row_groups(self, columns=None):
        """Yields ``read(columns, g)`` for every row group in file order."""
        for g in range(self.row_groups):
            yield self.read(columns, g)

    def matrix(self, features, label=None, row_group: int | None = None, dtype=torch.float32):
        """``(X [rows, features], y)`` of one row group or the whole file.  Feature columns whose file
        type already is ``dtype`` and that hold no nulls are decoded straight into the rows of one
        ``[features, rows]`` buffer, of which ``X`` is the transposed view."""
        features = list(features)
        if row_group is not None:
            fast = {torch.float32: FLOAT, torch.float64: DOUBLE, torch.int32: INT32, torch.int64: INT64}.get(dtype)
            infos = [self._cols[self._index[f]] for f in features]
            if fast is not None and all(c.type == fast and not c.nested for c in infos):
                n = self.row_group_rows(row_group)
                buf = torch.empty(len(features), n, dtype=dtype)
                for k, f in enumerate(features):
                    _, nulls = self._read_fixed(row_group, self._index[f], infos[k], buf[k])
                    if nulls is not None and bool(nulls.any()):
                        if not dtype.is_floating_point:
                            break
                        buf[k].masked_fill_(nulls, float("nan"))
                else:
                    y = self.read([label], row_group)[label] if label else None
                    return buf.t(), y
        cols = self.read(features + ([label] if label else []), row_group)
        X = torch.stack([cols[f].to(dtype) for f in features], 1)
        return X, (cols[label] if label else None)


def open(path: str) -> File:   # noqa: A001 - mirrors parquet.OpenFile
    return File(path)


def write(path: str, columns: dict, compression: str = "snappy", row_group_size: int | None = None, **kw) -> None:
    """Writes tensors / lists as a flat Parquet file through pyarrow (tests and data-set export;
    the reference has no writer either)."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    arrays = {k: (pa.array(v.cpu().numpy()) if torch.is_tensor(v) else (v if isinstance(v, pa.Array) else pa.array(v)))
              for k, v in columns.items()}
    pq.write_table(pa.table(arrays), path, compression=compression, row_group_size=row_group_size, **kw)
