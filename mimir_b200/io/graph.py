"""Graph section of a ``.mim`` file: data model, codec, builder, interpreter, sessions, export.

What the reference's ``io/mim`` runtime offers (``Model.Run`` / ``NewSession`` / ``Session.Run`` /
``Reset``, io/mim/session.go:48-252; the 33 primitive opcodes, io/mim/ops.go:282-392; the
standard-library composites ``name.vN``, io/mim/stdlib.go:33-68; ``Export`` / ``ExportFunc``,
io/mim/export.go:55-105) is provided here over this package's container:

* a graph is a table of **values** (name, kind, dtype, dims; a dim is an int or a named symbol with
  an upper bound), a list of **subgraphs** (subgraph 0 is the main program; ``while`` / ``if`` /
  model-defined composites name others by index) and, for sessions, **variables**: values that
  keep their contents from one run to the next (a KV cache) and take the value of another value
  of the main program when a run ends.
* the 33 primitives the reference runs have its meaning (``shl`` / ``shr`` / ``bitcast``, which the
  format defines and the reference's interpreter refuses, run here too): ``and`` / ``or`` are mul / max on 0-1 integers,
  ``reduce`` takes ``mode`` add | max | mul and keeps the reduced axes with size 1, ``gather`` takes
  slices along an axis at clamped positions, ``scatter`` replaces slices along an axis (the last
  of repeated positions wins), ``reshape`` / ``expand`` / ``const`` take their target from the
  declared shape of their output.
* two byte encodings are read: the reference's binary tables (magic ``MMFG`` / ``MIMG``; decoded by
  ``io/mmfg.py``, so graph files written by the reference run here and give its expected
  outputs) and this package's own (magic ``MB2G``, a version word and one UTF-8 JSON document),
  which is what ``export`` writes.

The interpreter computes with torch tensors on the device of its inputs (float composites in
fp32, outputs cast to their declared dtypes, as the reference's stdlib does) and returns lazy
``Tensor`` leaves.  ``export`` traces a module or a function through the public tensor ops
(``tensor.core`` reports each outermost op while a trace is active) and writes weights,
metadata and graph into one file that ``open(path).run({...})`` reproduces.
"""
from __future__ import annotations

import json
import math
import struct
import threading
from dataclasses import dataclass, field

import torch

from ..tensor import errors as E

MAGIC = b"MB2G"
VERSION = 1

OPCODES = (
    "neg", "recip", "sqrt", "exp2", "log2", "sin", "trunc", "cast",
    "add", "mul", "max", "pow", "idiv", "imod", "and", "or", "xor", "cmplt", "cmpeq", "where",
    "reduce", "reshape", "expand", "permute", "pad", "shrink", "gather", "scatter",
    "const", "dequantize", "call", "while", "if",
    # opcodes of the format that the reference's interpreter refuses as unsupported (io/mim/ops.go:256-258)
    "shl", "shr", "bitcast",
)
assert len(OPCODES) == 36

# inputs, outputs of the fixed-arity opcodes (reference: the arity table, io/mim/ops.go:228-238)
ARITY = {**{c: (1, 1) for c in ("neg", "recip", "sqrt", "exp2", "log2", "sin", "trunc", "cast", "reduce", "reshape",
                                "expand", "permute", "pad", "shrink", "dequantize", "bitcast")},
         **{c: (2, 1) for c in ("add", "mul", "max", "pow", "idiv", "imod", "and", "or", "xor", "cmplt", "cmpeq",
                                "gather", "shl", "shr")},
         "where": (3, 1), "scatter": (3, 1), "const": (0, 1)}

KINDS = ("input", "weight", "const", "variable", "temp")

DTYPES = {
    "f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "f64": torch.float64,
    "i8": torch.int8, "i16": torch.int16, "i32": torch.int32, "i64": torch.int64, "u8": torch.uint8,
    "bool": torch.bool,
}
QUANT_DTYPES = ("q8_0", "q4_0", "q4_k", "q6_k")
_NAME_OF = {v: k for k, v in DTYPES.items()}


def dtype_name(dt) -> str:
    if isinstance(dt, str):
        if dt not in DTYPES and dt not in QUANT_DTYPES:
            raise E.ErrDType(f"graph: unknown dtype {dt!r}")
        return dt
    if dt not in _NAME_OF:
        raise E.ErrDType(f"graph: dtype {dt} has no graph type")
    return _NAME_OF[dt]


class FormatError(E.MimirError):
    """The graph section is damaged or inconsistent (reference: mim.ErrFormat)."""


class NoGraph(E.MimirError):
    """The file has no graph section (reference: mim.ErrNoGraph)."""


@dataclass
class Sym:
    """A symbolic dimension: any size from 1 to ``bound``, the same wherever the name appears."""
    name: str
    bound: int = 1 << 31


@dataclass
class Value:
    name: str
    kind: str
    dtype: str
    dims: list          # ints or Sym
    store: str = ""     # weights / consts / variables: name of the stored tensor ("" = zeros for variables)


@dataclass
class Op:
    opcode: str
    inputs: list
    outputs: list
    attrs: dict = field(default_factory=dict)


@dataclass
class Subgraph:
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)
    ops: list = field(default_factory=list)


@dataclass
class Graph:
    values: list = field(default_factory=list)
    subgraphs: list = field(default_factory=lambda: [Subgraph()])
    composites: dict = field(default_factory=dict)   # "name.vN" -> subgraph index
    updates: dict = field(default_factory=dict)      # variable value index -> value index of its next contents
    output_names: list = field(default_factory=list)

    @property
    def main(self) -> Subgraph:
        return self.subgraphs[0]

    # ----------------------------------------------------------------- codec
    def encode(self) -> bytes:
        def dim(d):
            return d if isinstance(d, int) else {"sym": d.name, "max": d.bound}

        def attr(v):
            if isinstance(v, torch.dtype):
                return {"dtype": dtype_name(v)}
            if isinstance(v, SubgraphRef):
                return {"subgraph": v.index}
            return v
        doc = {
            "values": [[v.name, v.kind, v.dtype, [dim(d) for d in v.dims], v.store] for v in self.values],
            "subgraphs": [{"in": s.inputs, "out": s.outputs,
                           "ops": [[o.opcode, o.inputs, o.outputs, {k: attr(a) for k, a in o.attrs.items()}]
                                   for o in s.ops]} for s in self.subgraphs],
            "composites": self.composites,
            "updates": {str(k): v for k, v in self.updates.items()},
            "outputs": self.output_names,
        }
        body = json.dumps(doc, separators=(",", ":"), allow_nan=True).encode("utf-8")
        return MAGIC + struct.pack("<II", VERSION, len(body)) + body

    @staticmethod
    def decode(raw: bytes) -> "Graph":
        raw = bytes(raw)
        if raw[:4] != MAGIC:
            raise E.ErrUnsupported("graph section is not in this package's encoding (no MB2G magic); the "
                                   "reference's own graph encoding is defined outside its source tree")
        if len(raw) < 12:
            raise FormatError("graph section is truncated")
        version, n = struct.unpack_from("<II", raw, 4)
        if version != VERSION:
            raise E.ErrUnsupported(f"graph section version {version}, this reader knows {VERSION}")
        if 12 + n > len(raw):
            raise FormatError("graph section is truncated")
        try:
            doc = json.loads(raw[12:12 + n].decode("utf-8"))
        except (ValueError, UnicodeDecodeError) as exc:
            raise FormatError(f"graph section does not parse: {exc}") from None

        def dim(d):
            return d if isinstance(d, int) else Sym(d["sym"], int(d["max"]))

        def attr(v):
            if isinstance(v, dict) and "dtype" in v:
                return DTYPES[v["dtype"]]
            if isinstance(v, dict) and "subgraph" in v:
                return SubgraphRef(int(v["subgraph"]))
            return v
        try:
            g = Graph(values=[Value(n_, k, dt, [dim(d) for d in dims], st) for n_, k, dt, dims, st in doc["values"]],
                      subgraphs=[Subgraph(s["in"], s["out"], [Op(o[0], o[1], o[2], {k: attr(a) for k, a in o[3].items()})
                                                              for o in s["ops"]]) for s in doc["subgraphs"]],
                      composites={k: int(v) for k, v in doc.get("composites", {}).items()},
                      updates={int(k): int(v) for k, v in doc.get("updates", {}).items()},
                      output_names=list(doc.get("outputs", [])))
        except (KeyError, TypeError, ValueError) as exc:
            raise FormatError(f"graph section is malformed: {exc!r}") from None
        g.check()
        return g

    # ------------------------------------------------------------ validation
    def check(self) -> None:
        """Structural checks done once at load: indices in range, opcodes and kinds known, every
        value computed before it is read (reference: Model.check, io/mim/ops.go:241-280)."""
        nv = len(self.values)
        if not self.subgraphs:
            raise FormatError("graph without a main program")
        for v in self.values:
            if v.kind not in KINDS:
                raise FormatError(f"value {v.name!r}: unknown kind {v.kind!r}")
            if v.dtype not in DTYPES and v.dtype not in QUANT_DTYPES:
                raise FormatError(f"value {v.name!r}: unknown dtype {v.dtype!r}")
        for si, s in enumerate(self.subgraphs):
            for i in list(s.inputs) + list(s.outputs):
                if not 0 <= i < nv:
                    raise FormatError(f"subgraph {si}: value index {i} out of range")
            for o in s.ops:
                if o.opcode not in OPCODES:
                    raise E.ErrUnsupported(f"graph: unknown opcode {o.opcode!r}")
                want = ARITY.get(o.opcode)
                if want is not None and (len(o.inputs), len(o.outputs)) != want:
                    raise FormatError(f"{o.opcode} with {len(o.inputs)} inputs and {len(o.outputs)} outputs, "
                                      f"want {want[0]} and {want[1]}")
                if o.opcode == "while" and len(o.inputs) != len(o.outputs):
                    raise FormatError(f"while with {len(o.inputs)} inputs and {len(o.outputs)} outputs")
                if o.opcode == "if" and not o.inputs:
                    raise FormatError("if without a condition")
                for i in list(o.inputs) + list(o.outputs):
                    if not 0 <= i < nv:
                        raise FormatError(f"{o.opcode}: value index {i} out of range")
                for a in o.attrs.values():
                    if isinstance(a, SubgraphRef) and not 0 <= a.index < len(self.subgraphs):
                        raise FormatError(f"{o.opcode}: subgraph {a.index} out of range")
                if o.opcode == "call":
                    name = o.attrs.get("name", "")
                    if name not in self.composites and name not in STDLIB:
                        raise E.ErrUnsupported(f"graph: call of {name!r}, which is neither a standard-library "
                                               f"composite nor one of the model's own")
        for var, nxt in self.updates.items():
            if not 0 <= var < nv or self.values[var].kind != "variable" or not 0 <= nxt < nv:
                raise FormatError(f"update of value {var} is not an update of a variable")
        for name, si in self.composites.items():
            if not 0 < si < len(self.subgraphs):
                raise FormatError(f"composite {name!r}: subgraph {si} out of range")


@dataclass(frozen=True)
class SubgraphRef:
    index: int


# =============================================================================================
# Builder
# =============================================================================================

class Ref:
    """Handle of one value inside a ``Builder``; arithmetic on handles appends ops."""
    __slots__ = ("b", "index")

    def __init__(self, b: "Builder", index: int):
        self.b, self.index = b, index

    @property
    def value(self) -> Value:
        return self.b.g.values[self.index]

    @property
    def dims(self):
        return list(self.value.dims)

    @property
    def dtype(self) -> str:
        return self.value.dtype

    def __add__(self, o): return self.b.add(self, o)
    def __radd__(self, o): return self.b.add(o, self)
    def __mul__(self, o): return self.b.mul(self, o)
    def __rmul__(self, o): return self.b.mul(o, self)
    def __neg__(self): return self.b.neg(self)
    def __sub__(self, o): return self.b.add(self, self.b.neg(self.b.lift(o, self)))
    def __rsub__(self, o): return self.b.add(self.b.lift(o, self), self.b.neg(self))
    def __truediv__(self, o): return self.b.mul(self, self.b.recip(self.b.lift(o, self)))


def _bcast(a, b):
    out = []
    for x, y in zip(([1] * (len(b) - len(a)) + list(a)), ([1] * (len(a) - len(b)) + list(b))):
        if isinstance(x, int) and x == 1:
            out.append(y)
        elif isinstance(y, int) and y == 1:
            out.append(x)
        else:
            if isinstance(x, int) and isinstance(y, int) and x != y:
                raise E.ErrShape(f"graph: dims {a} and {b} do not broadcast")
            out.append(x)
    return out


class Builder:
    """Builds a ``Graph`` op by op.  Every method returns ``Ref`` handles of the outputs."""

    def __init__(self):
        self.g = Graph()
        self.tensors: dict = {}          # stored tensors (weights, constants, initial variable contents)
        self._cur = self.g.subgraphs[0]
        self._n = 0

    # --------------------------------------------------------------- values
    def _value(self, name, kind, dtype, dims, store="") -> Ref:
        self.g.values.append(Value(name or f"%{len(self.g.values)}", kind, dtype_name(dtype), list(dims), store))
        return Ref(self, len(self.g.values) - 1)

    def input(self, name: str, dtype, dims) -> Ref:
        r = self._value(name, "input", dtype, dims)
        self._cur.inputs.append(r.index)
        return r

    def weight(self, name: str, tensor, kind: str = "weight") -> Ref:
        """A stored tensor: a torch tensor or a ``QuantizedTensor`` kept in its block encoding."""
        from .mim import QuantizedTensor
        if isinstance(tensor, QuantizedTensor):
            self.tensors[name] = tensor
            return self._value(name, kind, tensor.kind, tensor.shape, store=name)
        tensor = tensor.detach()
        self.tensors[name] = tensor
        return self._value(name, kind, tensor.dtype, tensor.shape, store=name)

    def variable(self, name: str, dtype, dims, init=None) -> Ref:
        """A value that a session keeps between runs; it starts as ``init`` (or zeros)."""
        store = ""
        if init is not None:
            store = f"{name}.init"
            self.tensors[store] = init.detach()
        return self._value(name, "variable", dtype, dims, store=store)

    def update(self, variable: Ref, new: Ref) -> None:
        self.g.updates[variable.index] = new.index

    def output(self, name: str, ref: Ref) -> None:
        self.g.main.outputs.append(ref.index)
        self.g.output_names.append(name)

    def lift(self, x, like: Ref) -> Ref:
        if isinstance(x, Ref):
            return x
        return self.const(float(x) if not isinstance(x, (bool, int)) else x, like.dtype, [])

    # ------------------------------------------------------------------ ops
    def op(self, opcode, inputs, outs, **attrs):
        """Appends one op; ``outs`` is a list of (dtype, dims).  Returns the output handles."""
        refs = [self._value("", "temp", dt, dims) for dt, dims in outs]
        self._cur.ops.append(Op(opcode, [r.index for r in inputs], [r.index for r in refs], attrs))
        return refs

    def _un(self, code, x):
        return self.op(code, [x], [(x.dtype, x.dims)])[0]

    def neg(self, x): return self._un("neg", x)
    def recip(self, x): return self._un("recip", x)
    def sqrt(self, x): return self._un("sqrt", x)
    def exp2(self, x): return self._un("exp2", x)
    def log2(self, x): return self._un("log2", x)
    def sin(self, x): return self._un("sin", x)
    def trunc(self, x): return self._un("trunc", x)

    def cast(self, x, dtype):
        return self.op("cast", [x], [(dtype, x.dims)], to=DTYPES[dtype_name(dtype)])[0]

    def _bin(self, code, a, b, dtype=None):
        like = a if isinstance(a, Ref) else b
        a, b = self.lift(a, like), self.lift(b, like)
        return self.op(code, [a, b], [(dtype or a.dtype, _bcast(a.dims, b.dims))])[0]

    def add(self, a, b): return self._bin("add", a, b)
    def mul(self, a, b): return self._bin("mul", a, b)
    def max(self, a, b): return self._bin("max", a, b)
    def pow(self, a, b): return self._bin("pow", a, b)
    def idiv(self, a, b): return self._bin("idiv", a, b)
    def imod(self, a, b): return self._bin("imod", a, b)
    def and_(self, a, b): return self._bin("and", a, b)
    def or_(self, a, b): return self._bin("or", a, b)
    def xor(self, a, b): return self._bin("xor", a, b)
    def shl(self, a, b): return self._bin("shl", a, b)
    def shr(self, a, b): return self._bin("shr", a, b)

    def bitcast(self, x, dtype):
        """Reinterprets the bits as another type of the same width."""
        return self.op("bitcast", [x], [(dtype, x.dims)], to=DTYPES[dtype_name(dtype)])[0]

    def cmplt(self, a, b): return self._bin("cmplt", a, b, "i32")
    def cmpeq(self, a, b): return self._bin("cmpeq", a, b, "i32")

    def where(self, c, a, b):
        a = self.lift(a, b if isinstance(b, Ref) else c)
        b = self.lift(b, a)
        return self.op("where", [c, a, b], [(a.dtype, _bcast(c.dims, _bcast(a.dims, b.dims)))])[0]

    def reduce(self, x, mode, axes):
        axes = [a % len(x.dims) for a in axes]
        dims = [1 if i in axes else d for i, d in enumerate(x.dims)]
        return self.op("reduce", [x], [(x.dtype, dims)], mode=mode, axes=axes)[0]

    def reshape(self, x, dims): return self.op("reshape", [x], [(x.dtype, dims)])[0]
    def expand(self, x, dims): return self.op("expand", [x], [(x.dtype, dims)])[0]

    def permute(self, x, perm):
        perm = [p % len(x.dims) for p in perm]
        return self.op("permute", [x], [(x.dtype, [x.dims[p] for p in perm])], perm=perm)[0]

    def pad(self, x, pads, value=0.0):
        """``pads``: (before, after) per axis."""
        dims = []
        for d, (lo, hi) in zip(x.dims, pads):
            if not isinstance(d, int) and (lo or hi):
                raise E.ErrUnsupported("graph: pad of a symbolic dimension")
            dims.append(d + lo + hi if isinstance(d, int) else d)
        flat = [int(v) for p in pads for v in p]
        return self.op("pad", [x], [(x.dtype, dims)], pads=flat, value=float(value))[0]

    def shrink(self, x, ranges):
        """``ranges``: (begin, end) per axis; end -1 means to the end."""
        dims, begin, end = [], [], []
        for d, (lo, hi) in zip(x.dims, ranges):
            begin.append(int(lo))
            end.append(int(hi))
            if hi == -1:
                dims.append(d - lo if isinstance(d, int) else d)
            else:
                dims.append(hi - lo)
        return self.op("shrink", [x], [(x.dtype, dims)], begin=begin, end=end)[0]

    def gather(self, data, idx, axis=0):
        axis %= len(data.dims)
        return self.op("gather", [data, idx], [(data.dtype if data.dtype not in QUANT_DTYPES else "f32",
                                                data.dims[:axis] + idx.dims + data.dims[axis + 1:])], axis=axis)[0]

    def scatter(self, data, idx, updates, axis=0):
        return self.op("scatter", [data, idx, updates], [(data.dtype, data.dims)], axis=axis % len(data.dims))[0]

    def const(self, value, dtype="f32", dims=()):
        return self.op("const", [], [(dtype, list(dims))], value=value)[0]

    def dequantize(self, x): return self.op("dequantize", [x], [("f32", x.dims)])[0]

    def call(self, name, inputs, outs, **attrs):
        """Calls a standard-library composite (``"softmax.v1"``) or one defined with ``composite``."""
        return self.op("call", inputs, outs, name=name, **attrs)

    def call1(self, name, inputs, dtype, dims, **attrs):
        return self.call(name, inputs, [(dtype, dims)], **attrs)[0]

    # ------------------------------------------------------------ subgraphs
    def subgraph(self, in_specs, body) -> SubgraphRef:
        """Builds a subgraph: ``body(*refs)`` receives one handle per (dtype, dims) of ``in_specs`` and
        returns the output handles."""
        sg = Subgraph()
        self.g.subgraphs.append(sg)
        index = len(self.g.subgraphs) - 1
        prev, self._cur = self._cur, sg
        try:
            ins = []
            for dt, dims in in_specs:
                r = self._value("", "temp", dt, dims)
                sg.inputs.append(r.index)
                ins.append(r)
            outs = body(*ins)
            if isinstance(outs, Ref):
                outs = [outs]
            sg.outputs = [o.index for o in outs]
        finally:
            self._cur = prev
        return SubgraphRef(index)

    def composite(self, name: str, in_specs, body) -> None:
        self.g.composites[name] = self.subgraph(in_specs, body).index

    def while_(self, carried, cond, body):
        """Runs ``body`` on the carried values while ``cond`` (one i32 / bool scalar) holds."""
        specs = [(r.dtype, r.dims) for r in carried]
        c, b = self.subgraph(specs, cond), self.subgraph(specs, body)
        return self.op("while", carried, specs, cond=c, body=b)

    def if_(self, pred, operands, then, otherwise, outs):
        specs = [(r.dtype, r.dims) for r in operands]
        t, e = self.subgraph(specs, then), self.subgraph(specs, otherwise)
        return self.op("if", [pred] + list(operands), outs, then=t, **{"else": e})

    # -------------------------------------------------------------- writing
    def finish(self) -> Graph:
        self.g.check()
        return self.g

    def write(self, path, metadata=None) -> None:
        from . import mim
        mim.write_tensors(path, self.tensors, metadata=metadata, graph=self.finish().encode())

    def serialize(self, metadata=None) -> bytes:
        from . import mim
        return mim.serialize(self.tensors, metadata=metadata, graph=self.finish().encode())


STDLIB: dict = {}   # name.vN -> implementation, filled by graph_run

from . import graph_run as _graph_run  # noqa: E402,F401 - registers the standard library
