"""Decoder of the reference's binary graph section (magic ``MMFG`` in files written by the format's
first release, ``MIMG`` since), into this package's ``Graph`` model.

The reference keeps the encoding in a separate module that is not part of its source tree; the
layout below was recovered from the nine sample files the reference ships
(io/mim/testdata/{pytorch,onnx,llama}/*.mim) and checked by running each against its
``expected.json``.  Everything is little endian.

* header, 16 bytes: magic, u16 major, u16 minor, u32, u32; then eleven (u64 offset, u64 count)
  pairs, one per table, offsets from the start of the section:
  0 string bytes, 1 strings (u32 offset, u32 length), 2 symbols (u32 name, u32 0, u64 upper bound),
  3 integers (i64: dimensions and integer-list attributes), 4 values (8 x u32), 5 ops (8 x u32),
  6 value indices (u32: operand lists), 7 attributes (u32 key, u32 type, i64 count, i64 value),
  8 subgraphs (8 x u32), 9 composites, 10 variable updates (u32 variable, u32 next value).
* value: name string, dtype code (the container's codes), offset of its dimensions in table 3,
  then rank | kind << 8 | flags << 16, then the index of its stored tensor in the file's
  (name-sorted) tensor table.  A negative dimension -1 - k is symbol k.  Kinds: 0 temporary,
  1 input, 2 output, 3 weight, 4 variable, 5 constant.
* op: opcode, offset and count of its inputs in table 6, the same for outputs, offset and count of
  its attributes in table 7.
* attribute types: 1 integer, 2 integer list (count, offset into table 3), 3 float (the value's
  bits are an IEEE double), 4 string (index into table 1), 5 dtype code, 6 subgraph index.
* subgraph: first op, op count, then offset and count of inputs and of outputs in table 6.
"""
from __future__ import annotations

import struct

import torch

from ..tensor import errors as E
from . import graph as G

MAGICS = (b"MMFG", b"MIMG")

# opcode numbers of the format; the order of the binary group around and / or / xor was fixed by
# the sample graphs (``le`` = or(cmplt, cmpeq), ``not`` = xor(x, true))
OPCODE = {1: "neg", 2: "recip", 3: "sqrt", 4: "exp2", 5: "log2", 6: "sin", 7: "trunc", 8: "cast", 9: "bitcast",
          10: "add", 11: "mul", 12: "max", 13: "pow", 14: "idiv", 15: "imod", 16: "shl", 17: "shr", 18: "and",
          19: "or", 20: "xor", 21: "cmplt", 22: "cmpeq", 23: "where", 24: "reduce", 25: "reshape", 26: "expand",
          27: "permute", 28: "pad", 29: "shrink", 30: "gather", 31: "scatter", 32: "const", 33: "dequantize",
          34: "call", 35: "while", 36: "if"}
DTYPE = {1: "f32", 2: "f16", 3: "bf16", 4: "f64", 5: "i8", 6: "u8", 7: "i16", 9: "i32", 11: "i64", 13: "bool",
         64: "q8_0", 65: "q4_0", 66: "q4_k", 67: "q6_k"}
KIND = {0: "temp", 1: "input", 2: "temp", 3: "weight", 4: "variable", 5: "const"}


def is_reference_encoding(raw) -> bool:
    return bytes(raw[:4]) in MAGICS


def decode(raw, tensor_names) -> G.Graph:
    """``raw``: the section's bytes; ``tensor_names``: the names of the file's tensor table in table
    order (sorted bytewise), which stored values refer to by index."""
    raw = bytes(raw)
    if raw[:4] not in MAGICS:
        raise E.ErrUnsupported("graph section: unknown magic")
    if len(raw) < 16 + 11 * 16:
        raise G.FormatError("graph section is truncated")
    tabs = [struct.unpack_from("<QQ", raw, 16 + 16 * i) for i in range(11)]
    width = [1, 8, 16, 8, 32, 32, 4, 24, 32, 16, 8]
    for (off, n), w in zip(tabs, width):
        if off + n * w > len(raw):
            raise G.FormatError("graph section: a table runs past the end of the section")

    def rows(i, fmt):
        off, n = tabs[i]
        size = struct.calcsize(fmt)
        return [struct.unpack_from(fmt, raw, off + size * k) for k in range(n)]
    pool = raw[tabs[0][0]: tabs[0][0] + tabs[0][1]]
    try:
        strings = [pool[o: o + l].decode("utf-8") for o, l in rows(1, "<II")]
    except UnicodeDecodeError:
        raise G.FormatError("graph section: a string is not UTF-8") from None
    symbols = [G.Sym(strings[n], min(int(bound), 1 << 62)) for n, _, bound in rows(2, "<IIQ")]
    ints = [r[0] for r in rows(3, "<q")]
    vals, ops = rows(4, "<8I"), rows(5, "<8I")
    idx = [r[0] for r in rows(6, "<I")]
    attrs = rows(7, "<IIqq")
    subs = rows(8, "<8I")
    updates = rows(10, "<II")
    tensor_names = list(tensor_names)

    def dims_of(off, rank):
        out = []
        for d in ints[off: off + rank]:
            if d >= 0:
                out.append(int(d))
            else:
                k = -1 - d
                if k >= len(symbols):
                    raise G.FormatError("graph section: a dimension names a symbol that does not exist")
                out.append(symbols[k])
        return out

    g = G.Graph()
    g.subgraphs = []
    outputs_named = {}
    try:
        for i, (name, dt, doff, packed, store, *_rest) in enumerate(vals):
            rank, kind = packed & 0xFF, (packed >> 8) & 0xFF
            if dt not in DTYPE or kind not in KIND:
                raise G.FormatError(f"graph section: value {i} has dtype code {dt}, kind {kind}")
            nm = strings[name] or f"%{i}"
            st = ""
            if kind in (3, 5) or (kind == 4 and store < len(tensor_names) and _is_init(tensor_names, store, nm)):
                if store >= len(tensor_names):
                    raise G.FormatError(f"graph section: value {nm!r} names tensor {store} of {len(tensor_names)}")
                st = tensor_names[store]
            g.values.append(G.Value(nm, KIND[kind], DTYPE[dt], dims_of(doff, rank), st))
            if kind == 2:
                outputs_named[i] = strings[name]

        def attr_value(key, typ, count, value):
            if typ == 1:
                return int(value)
            if typ == 2:       # plain integers: -1 in a shrink's ``end`` means "to the end of the dimension"
                return [int(x) for x in ints[value: value + count]]
            if typ == 3:
                return struct.unpack("<d", struct.pack("<q", value))[0]
            if typ == 4:
                return strings[value]
            if typ == 5:
                return G.DTYPES.get(DTYPE.get(int(value), ""), DTYPE.get(int(value)))
            if typ == 6:
                return G.SubgraphRef(int(value))
            raise E.ErrUnsupported(f"graph section: attribute {key!r} has type code {typ}")

        all_ops = []
        for (code, ioff, nin, ooff, nout, aoff, nattr, _flags) in ops:
            if code not in OPCODE:
                raise E.ErrUnsupported(f"graph section: opcode {code}")
            at = {}
            for (k, typ, count, value) in attrs[aoff: aoff + nattr]:
                at[strings[k]] = attr_value(strings[k], typ, count, value)
            if OPCODE[code] == "call":
                at["name"] = f"{at.get('name', '')}.v{at.pop('version', 1)}"
            if OPCODE[code] == "cast" and "to" in at:
                at["dtype"] = at["to"]
            all_ops.append(G.Op(OPCODE[code], idx[ioff: ioff + nin], idx[ooff: ooff + nout], at))
        for (first, nops, ioff, nin, ooff, nout, *_r) in subs:
            g.subgraphs.append(G.Subgraph(idx[ioff: ioff + nin], idx[ooff: ooff + nout], all_ops[first: first + nops]))
    except IndexError:
        raise G.FormatError("graph section: an index points outside its table") from None
    if not g.subgraphs:
        raise G.FormatError("graph without a main program")
    g.output_names = [g.values[o].name for o in g.subgraphs[0].outputs]
    g.updates = {int(a): int(b) for a, b in updates}
    # the main program's declared inputs also list the variables: a session supplies those itself
    main = g.subgraphs[0]
    main.inputs = [i for i in main.inputs if g.values[i].kind == "input"]
    g.check()
    return g


def _is_init(names, store, value_name) -> bool:
    """A variable's stored tensor (its initial contents), when the file has one under its name."""
    return 0 <= store < len(names) and names[store] in (value_name, value_name + ".init")
