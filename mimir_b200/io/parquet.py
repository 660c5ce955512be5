"""Parquet reading for flat schemas (reference: io/parquet/ — its own decoder of the format; here
the column chunks are decoded by the Arrow C++ reader that ships with pyarrow, which covers the
same encodings and Snappy / gzip / zstd pages)."""
from __future__ import annotations

import numpy as np
import torch


class File:
    def __init__(self, path: str):
        import pyarrow.parquet as pq
        self._pf = pq.ParquetFile(path)
        self.path = path

    @property
    def columns(self) -> list:
        return list(self._pf.schema_arrow.names)

    @property
    def rows(self) -> int:
        return self._pf.metadata.num_rows

    @property
    def row_groups(self) -> int:
        return self._pf.metadata.num_row_groups

    def schema(self) -> dict:
        return {f.name: str(f.type) for f in self._pf.schema_arrow}

    def read(self, columns=None, row_group: int | None = None) -> dict:
        """Column name -> torch tensor (numeric / bool) or list (strings, nested)."""
        tbl = self._pf.read_row_group(row_group, columns=columns) if row_group is not None else self._pf.read(columns=columns)
        out = {}
        for name in tbl.column_names:
            col = tbl.column(name)
            try:
                arr = col.to_numpy(zero_copy_only=False)
                if arr.dtype == object or arr.dtype.kind in "US":
                    out[name] = col.to_pylist()
                else:
                    out[name] = torch.from_numpy(np.array(arr, copy=True))
            except Exception:
                out[name] = col.to_pylist()
        return out

    def matrix(self, features, label=None, row_group: int | None = None, dtype=torch.float32):
        cols = self.read(list(features) + ([label] if label else []), row_group)
        X = torch.stack([cols[f].to(dtype) for f in features], 1)
        return X, (cols[label] if label else None)


def write(path: str, columns: dict, compression: str = "snappy", row_group_size: int | None = None) -> None:
    """Writes tensors / lists as a flat Parquet file (used by tests and by dataset export)."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    arrays = {k: (pa.array(v.cpu().numpy()) if torch.is_tensor(v) else pa.array(v)) for k, v in columns.items()}
    pq.write_table(pa.table(arrays), path, compression=compression, row_group_size=row_group_size)
