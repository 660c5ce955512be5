"""``.mim`` model / checkpoint files (reference: io/mim/mim.go:193-226,
weights.go:50-201, write.go:54-167).

``open(path)`` maps the file read-only through the native library and returns a
:class:`Model` whose tensors are zero-copy views over the mapping;
``write_tensors`` / ``save`` produce files byte-compatible with the reference
writer (verified by rewriting every sample file of the reference bit for bit).
"""
from __future__ import annotations

import ctypes
import math
import os

import numpy as np
import torch

from .. import _native
from . import metadata as _md

# dtype codes of the container (io/mim/dtype.go:32-35,118-123)
F32, F16, BF16, U8, I32, I64 = 1, 2, 3, 6, 9, 11
Q8_0, Q4_0, Q4_K, Q6_K = 64, 65, 66, 67
_TORCH = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16, U8: torch.uint8,
          I32: torch.int32, I64: torch.int64}
_CODE = {v: k for k, v in _TORCH.items()}
# quantized block layouts: (values per block, bytes per block)
QUANT_BLOCK = {Q8_0: (32, 34), Q4_0: (32, 18), Q4_K: (256, 144), Q6_K: (256, 210)}
SECTION_WEIGHTS, SECTION_METADATA, SECTION_GRAPH, SECTION_TRAINING = 1, 2, 3, 4


class MimError(RuntimeError):
    pass


class QuantizedTensor:
    """A block-quantized tensor kept in its file encoding (ggml layouts)."""

    def __init__(self, code: int, shape, raw: torch.Tensor):
        self.code, self.shape, self.raw = code, tuple(shape), raw

    @property
    def kind(self) -> str:
        return {Q8_0: "q8_0", Q4_0: "q4_0", Q4_K: "q4_k", Q6_K: "q6_k"}[self.code]

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        from ..ops.quant import dequantize
        return dequantize(self, dtype)

    def numel(self) -> int:
        return math.prod(self.shape)


def _lib():
    lib = _native.lib()
    if not getattr(lib, "_mim_declared", False):
        vp, c = ctypes.c_void_p, ctypes
        lib.mimir_mim_last_error.restype = c.c_char_p
        lib.mimir_mim_open.argtypes = [c.c_char_p, c.POINTER(vp)]
        lib.mimir_mim_parse.argtypes = [vp, c.c_uint64, c.POINTER(vp)]
        lib.mimir_mim_close.argtypes = [vp]
        lib.mimir_mim_close.restype = None
        lib.mimir_mim_info.argtypes = [vp] + [c.POINTER(c.c_int)] * 6
        lib.mimir_mim_base.argtypes = [vp]
        lib.mimir_mim_base.restype = vp
        lib.mimir_mim_size.argtypes = [vp]
        lib.mimir_mim_size.restype = c.c_uint64
        lib.mimir_mim_tensor.argtypes = [vp, c.c_int, c.POINTER(c.c_char_p), c.POINTER(c.c_int),
                                         c.POINTER(c.c_int), c.POINTER(c.c_int), c.POINTER(c.c_uint64),
                                         c.POINTER(c.c_uint64), c.POINTER(c.c_uint64)]
        lib.mimir_mim_table.argtypes = [vp, vp, vp, c.c_char_p, c.c_longlong]
        lib.mimir_mim_table.restype = c.c_longlong
        lib.mimir_mim_section.argtypes = [vp, c.c_int, c.POINTER(c.c_int), c.POINTER(c.c_int),
                                          c.POINTER(c.c_uint64), c.POINTER(c.c_uint64), c.c_char_p]
        lib.mimir_mim_verify.argtypes = [vp]
        lib.mimir_mim_writer_new.argtypes = [c.c_int, c.c_int, c.c_int]
        lib.mimir_mim_writer_new.restype = vp
        lib.mimir_mim_writer_free.argtypes = [vp]
        lib.mimir_mim_writer_free.restype = None
        lib.mimir_mim_writer_add_tensor.argtypes = [vp, c.c_char_p, c.c_int, c.c_int, c.c_int,
                                                    c.POINTER(c.c_uint64), vp, c.c_uint64]
        lib.mimir_mim_writer_set_section.argtypes = [vp, c.c_int, c.c_int, vp, c.c_uint64]
        lib.mimir_mim_writer_write.argtypes = [vp, c.c_char_p]
        lib.mimir_mim_writer_serialize.argtypes = [vp, c.POINTER(c.POINTER(c.c_uint8)), c.POINTER(c.c_uint64)]
        lib.mimir_mim_free_buffer.argtypes = [c.POINTER(c.c_uint8)]
        lib.mimir_mim_free_buffer.restype = None
        lib._mim_declared = True
    return lib


def _check(rc: int) -> None:
    if rc != 0:
        raise MimError(_lib().mimir_mim_last_error().decode())


class Model:
    """An open ``.mim`` file.  Tensors are views over the read-only mapping."""

    def __init__(self, handle, keepalive=None):
        lib = _lib()
        self._h, self._keep = handle, keepalive
        vals = [ctypes.c_int() for _ in range(6)]
        lib.mimir_mim_info(handle, *[ctypes.byref(v) for v in vals])
        self.major, self.minor, self.alignment, nt, ns, mmf = (v.value for v in vals)
        self.legacy_magic = bool(mmf)
        size = size_total = lib.mimir_mim_size(handle)
        base = lib.mimir_mim_base(handle)
        self._buf = (ctypes.c_uint8 * size).from_address(base)
        self._np = np.frombuffer(self._buf, dtype=np.uint8)
        self._index = {}
        self._table_order = []        # tensor names in table order: graph values refer to tensors by this index
        off, nb = ctypes.c_uint64(), ctypes.c_uint64()
        if nt:
            # the whole table in one call, checked with array arithmetic: a file of 20 000 tensors opens in milliseconds
            need = lib.mimir_mim_table(handle, None, None, None, 0)
            meta = np.zeros((nt, 12), dtype=np.uint64)
            ends = np.zeros(nt, dtype=np.uint32)
            blob = ctypes.create_string_buffer(max(int(need), 1))
            if lib.mimir_mim_table(handle, meta.ctypes.data, ends.ctypes.data, blob, int(need)) < 0:
                _check(-1)
            raw = blob.raw[:need]
            dts, ranks = meta[:, 0].astype(np.int64), meta[:, 1].astype(np.int64)
            dims = meta[:, 2:10].astype(np.int64)
            live = np.arange(8)[None, :] < ranks[:, None]
            counts = np.where(live, dims, 1).prod(1)
            want = meta[:, 11].astype(np.int64).copy()          # dtypes this reader does not decode: refused when asked for
            for code, tdt in _TORCH.items():
                sel = dts == code
                if sel.any():
                    want[sel] = counts[sel] * torch.empty((), dtype=tdt).element_size()
            for code, (per, bsize) in QUANT_BLOCK.items():
                sel = dts == code
                if sel.any():
                    want[sel] = np.where(counts[sel] % per == 0, counts[sel] // per * bsize, -1)
            offs, lens = meta[:, 10].astype(np.int64), meta[:, 11].astype(np.int64)
            bad = np.nonzero((want != lens) | (offs + lens > size_total) | (offs < 0) | (lens < 0))[0]
            starts = np.concatenate([[0], ends[:-1]]).tolist()
            ends_l, dts_l, ranks_l, dims_l, offs_l, lens_l = ends.tolist(), dts.tolist(), ranks.tolist(), dims.tolist(), offs.tolist(), lens.tolist()
            if bad.size:
                i = int(bad[0])
                nm = raw[starts[i]:ends_l[i]].decode("utf-8", "replace")
                lib.mimir_mim_close(handle)
                self._h = None
                raise MimError(f"tensor {nm!r}: {lens_l[i]} bytes at offset {offs_l[i]} for shape {dims_l[i][:ranks_l[i]]} "
                               f"of dtype code {dts_l[i]}")
            text = raw.decode("utf-8")
            if len(text) == len(raw):                             # ASCII names: byte offsets are character offsets
                order = [text[a:b] for a, b in zip(starts, ends_l)]
            else:
                order = [raw[a:b].decode("utf-8") for a, b in zip(starts, ends_l)]
            self._table_order = order
            self._index = {nm: (dts_l[i], tuple(dims_l[i][:ranks_l[i]]), offs_l[i], lens_l[i]) for i, nm in enumerate(order)}
        self.sections = []
        kind, flags = ctypes.c_int(), ctypes.c_int()
        h32 = ctypes.create_string_buffer(32)
        for i in range(ns):
            _check(lib.mimir_mim_section(handle, i, ctypes.byref(kind), ctypes.byref(flags),
                                         ctypes.byref(off), ctypes.byref(nb), h32))
            self.sections.append(dict(kind=kind.value, flags=flags.value, offset=off.value,
                                      length=nb.value, sha256=bytes(h32.raw)))
        self._metadata = None

    # -- inspection
    def names(self):
        return sorted(self._index)

    def __contains__(self, name):
        return name in self._index

    def info(self, name):
        dt, shape, _, nb = self._index[name]
        return dt, shape, nb

    def section_bytes(self, kind: int):
        for s in self.sections:
            if s["kind"] == kind:
                return bytes(self._np[s["offset"]: s["offset"] + s["length"]])
        return None

    @property
    def metadata(self) -> dict:
        if self._metadata is None:
            raw = self.section_bytes(SECTION_METADATA)
            self._metadata = _md.decode(raw) if raw else {}
        return self._metadata

    def training(self):
        """Training section (counters, hyper-parameters, extras) or None."""
        raw = self.section_bytes(SECTION_TRAINING)
        return _md.decode(raw) if raw else None

    # -- graph runtime (reference: Model.Run / NewSession / Inputs / Outputs, io/mim/mim.go:164-330)
    def has_graph(self) -> bool:
        return self.section_bytes(SECTION_GRAPH) is not None

    def program(self):
        """The file's graph as a runnable program (parsed once)."""
        if getattr(self, "_program", None) is None:
            from . import graph as _g, graph_run as _gr
            raw = self.section_bytes(SECTION_GRAPH)
            if raw is None:
                raise _g.NoGraph("the file has no graph section")
            from . import mmfg as _mmfg
            if _mmfg.is_reference_encoding(raw):       # written by the reference: its binary tables
                graph = _mmfg.decode(raw, self._table_order)
            else:
                graph = _g.Graph.decode(raw)
            self._program = _gr.Program(graph, self.tensor)
        return self._program

    def graph(self):
        return self.program().g

    @property
    def inputs(self):
        """(name, dtype, dims) of every input of the main program."""
        return [(v.name, v.dtype, list(v.dims)) for v in self.program().inputs]

    @property
    def outputs(self):
        return [(n, v.dtype, list(v.dims)) for n, v in self.program().outputs]

    def run(self, inputs: dict, cancel=None) -> dict:
        """Computes the outputs from the inputs, keyed by name, on fresh variables."""
        return self.program().run(inputs, cancel=cancel)

    def new_session(self):
        """A session whose variables start from their initial values, independent of other sessions."""
        return self.program().new_session()

    def verify(self) -> bool:
        """Re-hashes every section against the SHA-256 in the index."""
        return _lib().mimir_mim_verify(self._h) == 0

    # -- tensors
    def tensor(self, name: str):
        """Zero-copy tensor over the mapping (clone before writing to it)."""
        if name not in self._index:
            raise KeyError(name)
        dt, shape, off, nb = self._index[name]
        raw = torch.from_numpy(self._np[off: off + nb])
        if dt in _TORCH:
            return raw.view(_TORCH[dt]).view(shape)
        if dt in QUANT_BLOCK:
            return QuantizedTensor(dt, shape, raw)
        raise MimError(f"tensor {name!r}: unknown dtype code {dt}")

    def load(self, device="cpu", prefix: str = "", dequantize: bool = False) -> dict:
        """All tensors under ``prefix`` as a name -> tensor dict on ``device``."""
        out = {}
        for n in self.names():
            if not n.startswith(prefix):
                continue
            t = self.tensor(n)
            if isinstance(t, QuantizedTensor):
                t = t.dequantize() if dequantize else QuantizedTensor(t.code, t.shape, t.raw.to(device))
            else:
                t = t.to(device) if str(device) != "cpu" else t.clone()
            if dequantize and not isinstance(t, QuantizedTensor):
                t = t.to(device)
            out[n[len(prefix):]] = t
        return out

    def close(self):
        if self._h:
            self._np = self._buf = None
            _lib().mimir_mim_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def open(path) -> Model:  # noqa: A001 - mirrors mim.Open
    h = ctypes.c_void_p()
    _check(_lib().mimir_mim_open(os.fspath(path).encode(), ctypes.byref(h)))
    return Model(h)


def parse(data: bytes) -> Model:
    buf = ctypes.create_string_buffer(data, len(data))
    h = ctypes.c_void_p()
    _check(_lib().mimir_mim_parse(ctypes.cast(buf, ctypes.c_void_p), len(data), ctypes.byref(h)))
    return Model(h, keepalive=buf)


def _writer(tensors: dict, metadata=None, graph=None, training=None, alignment=4096, minor=2,
            legacy_magic=False, extra_sections=None):
    lib = _lib()
    w = lib.mimir_mim_writer_new(alignment, minor, int(legacy_magic))
    keep = []
    for name, t in tensors.items():
        if isinstance(t, QuantizedTensor):
            code, shape, raw = t.code, t.shape, t.raw.detach().cpu().contiguous()
        else:
            t = t.detach().cpu().contiguous()
            if t.dtype not in _CODE:
                raise MimError(f"tensor {name!r}: dtype {t.dtype} has no .mim code")
            code, shape, raw = _CODE[t.dtype], tuple(t.shape), t.reshape(-1).view(torch.uint8)
        raw = raw.reshape(-1)
        keep.append(raw)
        dims = (ctypes.c_uint64 * 8)(*shape, *([0] * (8 - len(shape))))
        nm = name.encode("utf-8")
        _check(lib.mimir_mim_writer_add_tensor(w, nm, len(nm), code, len(shape), dims,
                                               raw.data_ptr() if raw.numel() else None, raw.numel()))
    def put(kind, flags, data):
        b = ctypes.create_string_buffer(data, len(data))
        _check(lib.mimir_mim_writer_set_section(w, kind, flags, ctypes.cast(b, ctypes.c_void_p), len(data)))
    if metadata is not None:
        put(SECTION_METADATA, 0, metadata if isinstance(metadata, bytes)
            else _md.encode(metadata, b"MMFM" if legacy_magic else b"MIMM"))
    if graph is not None:
        put(SECTION_GRAPH, 1, graph)
    if training is not None:
        put(SECTION_TRAINING, 0, training if isinstance(training, bytes) else _md.encode(training))
    for kind, (flags, data) in (extra_sections or {}).items():
        put(kind, flags, data)
    return w, keep


def write_tensors(path, tensors: dict, metadata=None, training=None, graph=None, alignment=4096,
                  minor=2, legacy_magic=False) -> None:
    """Writes ``tensors`` (name -> tensor) atomically: temp file, fsync, rename."""
    w, keep = _writer(tensors, metadata, graph, training, alignment, minor, legacy_magic)
    try:
        _check(_lib().mimir_mim_writer_write(w, os.fspath(path).encode()))
    finally:
        _lib().mimir_mim_writer_free(w)


def serialize(tensors: dict, metadata=None, training=None, graph=None, alignment=4096, minor=2,
              legacy_magic=False) -> bytes:
    w, keep = _writer(tensors, metadata, graph, training, alignment, minor, legacy_magic)
    try:
        out, n = ctypes.POINTER(ctypes.c_uint8)(), ctypes.c_uint64()
        _check(_lib().mimir_mim_writer_serialize(w, ctypes.byref(out), ctypes.byref(n)))
        data = ctypes.string_at(out, n.value)
        _lib().mimir_mim_free_buffer(out)
        return data
    finally:
        _lib().mimir_mim_writer_free(w)


def save(path, module_or_state, metadata=None, training=None) -> None:
    """Saves a module's named parameters/buffers (or a state dict) as ``.mim``."""
    state = module_or_state.state_dict() if hasattr(module_or_state, "state_dict") else module_or_state
    write_tensors(path, {k: v for k, v in state.items() if torch.is_tensor(v) or isinstance(v, QuantizedTensor)},
                  metadata=metadata, training=training)


def lora_info(model: "Model"):
    """``{"rank", "alpha", "base", "targets"}`` of a LoRA adapter file, None for other files
    (mim.Model.LoRA in the reference)."""
    md = model.metadata
    if md.get("adapter.type") != "lora":
        return None
    targets = sorted({n.rsplit(".", 1)[0] for n in model.names() if n.endswith(".lora_a")})
    return {"rank": int(md.get("adapter.lora.rank", 0)), "alpha": float(md.get("adapter.lora.alpha", 0.0)),
            "base": md.get("adapter.base", ""), "targets": targets}


def apply_lora(module, adapter: "Model") -> int:
    """Wraps the ``nn.Linear`` layers an adapter file names (``<path>.lora_a`` / ``<path>.lora_b``, paths as
    in ``module.named_params()`` without the ``.weight`` suffix) in ``LoRALinear`` and loads the factors;
    returns how many layers were adapted (mim.Model.ApplyLoRA)."""
    from ..nn.module import Linear, LoRALinear
    info = lora_info(adapter)
    if info is None:
        raise MimError("not a LoRA adapter file")
    done = 0
    for path in info["targets"]:
        owner, attr = module, None
        parts = path.split(".")
        for i, part in enumerate(parts):
            last = i == len(parts) - 1
            holder = owner
            owner = owner[int(part)] if isinstance(owner, (list, tuple)) else (owner[part] if isinstance(owner, dict) else getattr(owner, part))
            if last:
                attr = (holder, part)
        holder, part = attr
        lin = owner
        if isinstance(lin, LoRALinear):
            wrapped = lin
        elif isinstance(lin, Linear):
            wrapped = LoRALinear(lin, info["rank"], info["alpha"])
            if isinstance(holder, list):
                holder[int(part)] = wrapped
            elif isinstance(holder, dict):
                holder[part] = wrapped
            else:
                setattr(holder, part, wrapped)
        else:
            raise MimError(f"{path}: not a Linear layer")
        wrapped.lora_a.set(adapter.tensor(path + ".lora_a").clone().to(wrapped.lora_a.dtype))
        wrapped.lora_b.set(adapter.tensor(path + ".lora_b").clone().to(wrapped.lora_b.dtype))
        done += 1
    return done


def describe(path, out=None) -> None:
    """Prints what a ``.mim`` file holds: version, sections with their hashes, tensors, metadata keys
    and, when there is a graph this package can read, its inputs and outputs."""
    import sys
    out = out or sys.stdout
    names = {SECTION_WEIGHTS: "weights", SECTION_METADATA: "metadata", SECTION_GRAPH: "graph",
             SECTION_TRAINING: "training"}
    dts = {F32: "f32", F16: "f16", BF16: "bf16", U8: "u8", Q8_0: "q8_0", Q4_0: "q4_0", Q4_K: "q4_k", Q6_K: "q6_k"}
    with open(path) as m:
        print(f"{path}: version {m.major}.{m.minor}, alignment {m.alignment}, hashes "
              f"{'ok' if m.verify() else 'MISMATCH'}", file=out)
        for s in m.sections:
            print(f"  section {names.get(s['kind'], s['kind'])}: {s['length']} bytes, sha256 {s['sha256'].hex()[:16]}…",
                  file=out)
        for n in m.names():
            dt, shape, nb = m.info(n)
            torch_dt = _TORCH.get(dt)
            label = dts.get(dt) or (str(torch_dt).replace("torch.", "") if torch_dt is not None else f"dtype {dt}")
            print(f"  tensor {n}: {label} {list(shape)} ({nb} bytes)", file=out)
        md = m.metadata
        for k in sorted(md):
            v = md[k]
            text = f"[{len(v)} values]" if isinstance(v, list) and len(v) > 8 else repr(v)
            print(f"  metadata {k} = {text}", file=out)
        if m.has_graph():
            try:
                print(f"  graph inputs {m.inputs}", file=out)
                print(f"  graph outputs {m.outputs}", file=out)
            except Exception as exc:  # noqa: BLE001 - a graph in another encoding is reported, not fatal
                print(f"  graph: {exc}", file=out)


if __name__ == "__main__":
    import sys
    if len(sys.argv) != 2:
        print("usage: python -m mimir_b200.io.mim <file.mim>", file=sys.stderr)
        raise SystemExit(2)
    describe(sys.argv[1])
