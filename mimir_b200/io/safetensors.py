"""safetensors reader / writer and safetensors -> ``.mim`` conversion.

The reference's models and test oracles arrive as GGUF or safetensors files that an external
importer turns into ``.mim`` (tools/gguf/llama.py:4-13 of the reference converts
``<name>.logits.safetensors`` that way).  The format is an 8-byte little-endian header length, a JSON
header ``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`` and the raw
little-endian tensor bytes; tensors are mapped, not copied, until they are written out.

    python -m mimir_b200.io.safetensors model.safetensors model.mim
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import sys
import warnings

import numpy as np
import torch

from . import mim

_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """``tensors``: name -> (dtype, shape, begin, end); ``metadata``: the header's string map."""

    def __init__(self, path):
        self._f = open(os.fspath(path), "rb")
        try:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:
            self._f.close()
            raise SafetensorsError("empty file") from None
        buf = memoryview(self._map)
        if len(buf) < 8:
            raise SafetensorsError("file is shorter than its header length")
        (n,) = struct.unpack_from("<Q", buf, 0)
        if n > len(buf) - 8 or n > (100 << 20):
            raise SafetensorsError(f"header of {n} bytes does not fit the file")
        try:
            header = json.loads(bytes(buf[8:8 + n]).decode("utf-8"))
        except (ValueError, UnicodeDecodeError) as exc:
            raise SafetensorsError(f"header does not parse: {exc}") from None
        if not isinstance(header, dict):
            raise SafetensorsError("header is not an object")
        self.metadata = {str(k): str(v) for k, v in (header.pop("__metadata__", None) or {}).items()}
        self._data = 8 + n
        self.tensors = {}
        for name, info in header.items():
            try:
                dt, shape, (begin, end) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"tensor {name!r}: malformed entry") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"tensor {name!r}: dtype {dt} is not supported")
            count = 1
            for s in shape:
                count *= s
            size = count * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if begin < 0 or end - begin != size or self._data + end > len(buf):
                raise SafetensorsError(f"tensor {name!r}: {end - begin} bytes at [{begin}, {end}) for "
                                       f"{count} values of {dt}")
            self.tensors[name] = (_DTYPES[dt], shape, begin, end)
        self._buf = buf

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, begin, end = self.tensors[name]
        if end == begin:
            return torch.empty(shape, dtype=dt)
        raw = np.frombuffer(self._buf, dtype=np.uint8, count=end - begin, offset=self._data + begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the mapping is read-only; so are the views
            t = torch.from_numpy(raw)
        if dt == torch.bool:
            return (t != 0).view(shape)
        return t.view(dt).view(shape)

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


def load(path) -> dict:
    """All tensors of the file, copied out of the mapping."""
    with SafetensorsFile(path) as f:
        return {n: f.tensor(n).clone() for n in f.tensors}


def save(path, tensors: dict, metadata: dict | None = None) -> None:
    """Writes ``tensors`` (name -> torch tensor) in name order, 8-byte aligned header."""
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} is not supported")
        raw = (t.to(torch.uint8) if t.dtype == torch.bool else t).reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    body = json.dumps(header, separators=(",", ":")).encode("utf-8")
    body += b" " * (-len(body) % 8)
    tmp = os.fspath(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(body)) + body)
        for raw in blobs:
            f.write(raw)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, os.fspath(path))


def convert(src, mim_path) -> int:
    """safetensors -> ``.mim``: tensors byte for byte (bool as uint8), the string metadata as it is.
    Returns the number of tensors."""
    with SafetensorsFile(src) as f:
        tensors = {}
        for n in f.tensors:
            t = f.tensor(n)
            tensors[n] = t.to(torch.uint8) if t.dtype == torch.bool else t
        mim.write_tensors(mim_path, tensors, metadata=dict(f.metadata) or None)
        n = len(tensors)
        tensors.clear()
    return n


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print("usage: python -m mimir_b200.io.safetensors <in.safetensors> <out.mim>", file=sys.stderr)
        return 2
    print(f"{convert(argv[0], argv[1])} tensors")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
