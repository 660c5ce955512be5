"""Damaged files are refused with the reader's own error, never with a crash or a stray exception
(the reference fuzzes its .mim parser the same way: io/mim/fuzz_test.go)."""
import random
import struct

import pytest
import torch

from mimir_b200.io import gguf, mim
from mimir_b200.io import graph as G
from mimir_b200.io import safetensors as st
from mimir_b200.tensor import errors as E


def _mutations(good: bytes, n: int, seed: int):
    rng = random.Random(seed)
    for _ in range(n):
        data = bytearray(good)
        mode = rng.randrange(4)
        if mode == 0:
            for _ in range(rng.randrange(1, 8)):
                data[rng.randrange(len(data))] = rng.randrange(256)
        elif mode == 1:
            data = data[:rng.randrange(len(data))]
        elif mode == 2:
            pos = rng.randrange(0, min(len(data), 600))
            data[pos:pos + 8] = rng.randbytes(8)
        else:
            pos = rng.randrange(len(data))
            data[pos:pos + 4] = b"\xff\xff\xff\xff"
        yield bytes(data)


def _model_bytes():
    b = G.Builder()
    x = b.input("x", "f32", [2, 4])
    w = b.weight("w", torch.randn(4, 4))
    b.output("y", b.call1("linear.v1", [x, w], "f32", [2, 4]))
    return b.serialize(metadata={"a": 1, "s": "hello", "l": [1, 2, 3], "f": [0.5], "t": ["x", "yy"]})


def test_mim_parser_and_graph_runtime_survive_damage():
    ok = 0
    for data in _mutations(_model_bytes(), 600, 1):
        try:
            m = mim.parse(data)
        except (mim.MimError, ValueError):
            continue
        try:
            m.metadata  # noqa: B018
            for n in m.names():
                m.tensor(n)
            m.verify()
            if m.has_graph():
                m.run({"x": torch.ones(2, 4)})
            ok += 1
        except (mim.MimError, E.MimirError, ValueError, KeyError):
            pass
        finally:
            m.close()
    assert ok > 0                                  # damage inside tensor data still parses


def test_graph_decoder_survives_damage():
    b = G.Builder()
    x = b.input("x", "i32", [])
    i, _ = b.while_([b.const(0, "i32", []), x], lambda i, n: b.cmplt(i, n), lambda i, n: [b.add(i, 1), n])
    b.output("i", i)
    good = b.finish().encode()
    for data in _mutations(good, 600, 2):
        try:
            G.Graph.decode(data)
        except E.MimirError:
            pass


def test_gguf_reader_survives_damage(tmp_path):
    from test_gguf import _sample
    path, _ = _sample(tmp_path)
    good = path.read_bytes()
    p = tmp_path / "f.gguf"
    for data in _mutations(good, 500, 3):
        p.write_bytes(data)
        try:
            with gguf.GGUFFile(p) as g:
                for n in g.tensors:
                    try:
                        g.tensor(n)
                    except gguf.GGUFError:
                        pass
        except gguf.GGUFError:
            pass


def test_safetensors_reader_survives_damage(tmp_path):
    good_path = tmp_path / "g.safetensors"
    st.save(good_path, {"w": torch.randn(3, 5), "i": torch.arange(4)}, metadata={"k": "v"})
    good = good_path.read_bytes()
    p = tmp_path / "f.safetensors"
    for data in _mutations(good, 500, 4):
        p.write_bytes(data)
        try:
            with st.SafetensorsFile(p) as f:
                for n in f.tensors:
                    f.tensor(n)
        except st.SafetensorsError:
            pass
