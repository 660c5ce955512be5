"""GGUF reader and GGUF -> ``.mim`` conversion.

The reference reads language models from ``.mim`` files that an external importer
(``mim-import`` of the mimir-model module, see tools/gguf/llama.py:4-13 in the reference) makes
from GGUF files "copying the tensors byte for byte and the GGUF metadata as it is".  This module
is that importer: it parses GGUF versions 2 and 3 (header, typed key-value metadata, tensor
table, aligned data section), maps every tensor whose type the container knows (F32, F16, BF16,
F64, I8, I16, I32, I64 and the block formats Q8_0, Q4_0, Q4_K, Q6_K) without touching its bytes, and
writes weights plus metadata into one ``.mim`` file that ``llm.Model.load`` opens.

GGUF stores a tensor's dimensions innermost first; shapes here are outermost first (row-major),
so a ``[n_out, n_in]`` weight has ``ne = (n_in, n_out)`` in the file.

    python -m mimir_b200.io.gguf model.gguf model.mim
"""
from __future__ import annotations

import mmap
import os
import struct
import sys
import warnings

import numpy as np
import torch

from . import mim
from .metadata import UInt64

MAGIC = 0x46554747  # "GGUF" little endian

# value types of the key-value section
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9

# ggml tensor types -> (torch dtype or .mim block code, values per block, bytes per block)
_DENSE = {0: (torch.float32, 4), 1: (torch.float16, 2), 30: (torch.bfloat16, 2), 28: (torch.float64, 8),
          24: (torch.int8, 1), 25: (torch.int16, 2), 26: (torch.int32, 4), 27: (torch.int64, 8)}
_BLOCK = {2: (mim.Q4_0, 32, 18), 8: (mim.Q8_0, 32, 34), 12: (mim.Q4_K, 256, 144), 14: (mim.Q6_K, 256, 210)}
_TYPE_NAMES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K",
               11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 15: "Q8_K", 30: "BF16"}


class GGUFError(ValueError):
    pass


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError("file ends inside its header")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GGUFError("file ends inside a string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="surrogateescape")
        self.pos += n
        return s

    def value(self, ty):
        if ty in _SCALARS:
            v = self.take(_SCALARS[ty])
            return UInt64(v) if ty == 10 else v
        if ty == _STRING:
            return self.string()
        if ty == _ARRAY:
            ety, n = self.take("<I"), self.take("<Q")
            if ety in _SCALARS:
                fmt = _SCALARS[ety][1]
                size = struct.calcsize(fmt)
                if self.pos + n * size > len(self.buf):
                    raise GGUFError("file ends inside an array")
                arr = np.frombuffer(self.buf, dtype=np.dtype("<" + fmt), count=n, offset=self.pos)
                self.pos += n * size
                if fmt in "fd":
                    return [float(x) for x in arr]
                if fmt == "?":
                    return [int(x) for x in arr]
                return [int(x) for x in arr]
            if ety == _STRING:
                return [self.string() for _ in range(n)]
            if ety == _ARRAY:
                return [self.value(_ARRAY) for _ in range(n)]
            raise GGUFError(f"array of unknown value type {ety}")
        raise GGUFError(f"unknown value type {ty}")


class GGUFFile:
    """A parsed GGUF file: ``metadata`` (dict), ``tensors`` (name -> (shape, ggml type, offset, bytes)).
    Tensor data stays in the file mapping until ``tensor`` is called."""

    def __init__(self, path):
        self.path = os.fspath(path)
        self._f = open(self.path, "rb")
        try:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:
            self._f.close()
            raise GGUFError("empty file") from None
        buf = memoryview(self._map)
        c = _Cursor(buf)
        if len(buf) < 24 or c.take("<I") != MAGIC:
            raise GGUFError("not a GGUF file")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GGUFError(f"GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.metadata = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = c.value(c.take("<I"))
        infos = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            if nd > 8:
                raise GGUFError(f"tensor {name!r} has {nd} dimensions")
            ne = [c.take("<Q") for _ in range(nd)]
            infos.append((name, tuple(reversed(ne)), c.take("<I"), c.take("<Q")))
        self.alignment = int(self.metadata.get("general.alignment", 32))
        if self.alignment <= 0 or self.alignment & (self.alignment - 1):
            raise GGUFError(f"alignment {self.alignment} is not a power of two")
        self.data_start = (c.pos + self.alignment - 1) // self.alignment * self.alignment
        self.tensors = {}
        for name, shape, ty, off in infos:
            n = 1
            for s in shape:
                n *= s
            if ty in _DENSE:
                nbytes = n * _DENSE[ty][1]
            elif ty in _BLOCK:
                _, per, size = _BLOCK[ty]
                if not shape or shape[-1] % per:
                    raise GGUFError(f"tensor {name!r}: rows of {shape[-1] if shape else 0} values do not fill "
                                    f"{_TYPE_NAMES[ty]} blocks of {per}")
                nbytes = n // per * size
            else:
                nbytes = None           # a type the container cannot hold; reported when it is asked for
            if nbytes is not None and self.data_start + off + nbytes > len(buf):
                raise GGUFError(f"tensor {name!r} reaches past the end of the file")
            self.tensors[name] = (shape, ty, off, nbytes)
        self._buf = buf

    def tensor(self, name: str):
        """The tensor as a torch view over the mapping (dense types) or a ``QuantizedTensor``."""
        shape, ty, off, nbytes = self.tensors[name]
        if nbytes is None:
            raise GGUFError(f"tensor {name!r} has ggml type {_TYPE_NAMES.get(ty, ty)}, which .mim files do not hold")
        raw = np.frombuffer(self._buf, dtype=np.uint8, count=nbytes, offset=self.data_start + off)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the mapping is read-only; so are the views
            t = torch.from_numpy(raw)
        if ty in _DENSE:
            return t.view(_DENSE[ty][0]).view(shape) if nbytes else torch.empty(shape, dtype=_DENSE[ty][0])
        return mim.QuantizedTensor(_BLOCK[ty][0], shape, t)

    def close(self):
        self._buf = None
        try:
            self._map.close()
        except BufferError:
            pass        # tensors handed out still view the mapping; it goes with them
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def _mim_metadata(md: dict) -> dict:
    """Metadata the typed ``.mim`` section can hold: scalars, strings and flat arrays; nested arrays
    (not used by any model architecture key) are dropped."""
    out = {}
    for k, v in md.items():
        if isinstance(v, list):
            if any(isinstance(e, list) for e in v):
                continue
            if v and all(isinstance(e, str) for e in v):
                out[k] = v
            elif all(isinstance(e, float) for e in v):
                out[k] = [float(e) for e in v]
            elif all(isinstance(e, (int, bool)) for e in v):
                out[k] = [int(e) for e in v]
            elif not v:
                out[k] = []
        else:
            out[k] = v
    return out


def convert(gguf_path, mim_path, skip_unsupported: bool = False) -> dict:
    """Writes the GGUF file's tensors (bytes unchanged) and metadata as a ``.mim`` file.  Returns a
    summary ``{"tensors": n, "skipped": [names], "bytes": total}``."""
    with GGUFFile(gguf_path) as g:
        tensors, skipped, total = {}, [], 0
        for name, (shape, ty, off, nbytes) in g.tensors.items():
            if nbytes is None:
                if not skip_unsupported:
                    raise GGUFError(f"tensor {name!r} has ggml type {_TYPE_NAMES.get(ty, ty)}, which .mim files "
                                    f"do not hold (pass skip_unsupported=True to leave it out)")
                skipped.append(name)
                continue
            tensors[name] = g.tensor(name)
            total += nbytes
        mim.write_tensors(mim_path, tensors, metadata=_mim_metadata(g.metadata))
        tensors.clear()
    return {"tensors": len(g.tensors) - len(skipped), "skipped": skipped, "bytes": total}


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print("usage: python -m mimir_b200.io.gguf <in.gguf> <out.mim>", file=sys.stderr)
        return 2
    info = convert(argv[0], argv[1], skip_unsupported=True)
    print(f"{info['tensors']} tensors, {info['bytes']} bytes" +
          (f", skipped {len(info['skipped'])}: {', '.join(info['skipped'][:5])}" if info["skipped"] else ""))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
