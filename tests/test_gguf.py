"""GGUF reader and GGUF -> .mim conversion, on files written here byte by byte."""
import struct

import pytest
import torch

from mimir_b200.io import gguf, mim
from mimir_b200.ops import quant as Q


def _s(x: str) -> bytes:
    b = x.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key, ty, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", ty) + payload


def write_gguf(path, metadata: list, tensors: list, alignment=32, version=3):
    """metadata: already encoded key-value records; tensors: (name, shape outermost first, ggml type, bytes)."""
    head = struct.pack("<IIQQ", gguf.MAGIC, version, len(tensors), len(metadata)) + b"".join(metadata)
    infos, blobs, off = b"", [], 0
    for name, shape, ty, raw in tensors:
        infos += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        infos += struct.pack("<IQ", ty, off)
        blobs.append((off, raw))
        off = (off + len(raw) + alignment - 1) // alignment * alignment
    body = head + infos
    body += b"\0" * (-len(body) % alignment)
    data = bytearray(off)
    for o, raw in blobs:
        data[o:o + len(raw)] = raw
    with open(path, "wb") as f:
        f.write(body + bytes(data))


def _sample(tmp_path, alignment=32):
    torch.manual_seed(0)
    w32 = torch.randn(3, 5)
    w16 = torch.randn(4, 8).half()
    wbf = torch.randn(2, 16).bfloat16()
    q8 = Q.quantize_q8_0(torch.randn(6, 64))
    q4 = Q.quantize_q4_0(torch.randn(4, 32))
    md = [
        _kv("general.architecture", 8, _s("llama")),
        _kv("general.alignment", 4, struct.pack("<I", alignment)),
        _kv("llama.block_count", 4, struct.pack("<I", 2)),
        _kv("llama.rope.freq_base", 6, struct.pack("<f", 10000.0)),
        _kv("llama.context_length", 10, struct.pack("<Q", 1 << 33)),
        _kv("flag", 7, struct.pack("<?", True)),
        _kv("offset", 5, struct.pack("<i", -7)),
        _kv("tokenizer.ggml.tokens", 9, struct.pack("<IQ", 8, 3) + _s("<s>") + _s("a") + _s("é")),
        _kv("tokenizer.ggml.scores", 9, struct.pack("<IQ", 6, 3) + struct.pack("<3f", 0.0, -1.5, -2.0)),
        _kv("tokenizer.ggml.token_type", 9, struct.pack("<IQ", 5, 3) + struct.pack("<3i", 3, 1, 1)),
    ]
    tensors = [("a.weight", (3, 5), 0, w32.numpy().tobytes()), ("b.weight", (4, 8), 1, w16.numpy().tobytes()),
               ("c.weight", (2, 16), 30, wbf.view(torch.int16).numpy().tobytes()),
               ("d.weight", (6, 64), 8, q8.numpy().tobytes()), ("e.weight", (4, 32), 2, q4.numpy().tobytes())]
    path = tmp_path / "m.gguf"
    write_gguf(path, md, tensors, alignment)
    return path, dict(a=w32, b=w16, c=wbf, d=q8, e=q4)


@pytest.mark.parametrize("alignment", [32, 64])
def test_read_metadata_and_tensors(tmp_path, alignment):
    path, want = _sample(tmp_path, alignment)
    with gguf.GGUFFile(path) as g:
        assert g.version == 3 and g.alignment == alignment
        md = g.metadata
        assert md["general.architecture"] == "llama" and md["llama.block_count"] == 2
        assert md["llama.context_length"] == 1 << 33 and md["flag"] is True and md["offset"] == -7
        assert md["tokenizer.ggml.tokens"] == ["<s>", "a", "é"]
        assert md["tokenizer.ggml.scores"] == [0.0, -1.5, -2.0] and md["tokenizer.ggml.token_type"] == [3, 1, 1]
        assert torch.equal(g.tensor("a.weight"), want["a"]) and torch.equal(g.tensor("b.weight"), want["b"])
        assert torch.equal(g.tensor("c.weight"), want["c"])
        d = g.tensor("d.weight")
        assert isinstance(d, mim.QuantizedTensor) and d.kind == "q8_0" and d.shape == (6, 64)
        assert torch.equal(d.raw.clone(), want["d"].reshape(-1))
        assert g.tensor("e.weight").kind == "q4_0"


def test_convert_copies_bytes_and_metadata(tmp_path):
    path, want = _sample(tmp_path)
    out = tmp_path / "m.mim"
    info = gguf.convert(path, out)
    assert info["tensors"] == 5 and not info["skipped"]
    with mim.open(out) as m:
        assert m.verify()
        assert torch.equal(m.tensor("a.weight"), want["a"]) and torch.equal(m.tensor("c.weight"), want["c"])
        d = m.tensor("d.weight")
        assert d.kind == "q8_0" and torch.equal(d.raw.clone(), want["d"].reshape(-1))
        torch.testing.assert_close(d.dequantize(), Q.dequantize_raw(Q.Q8_0, want["d"].reshape(-1), 6 * 64).view(6, 64))
        md = m.metadata
        assert md["general.architecture"] == "llama" and md["llama.block_count"] == 2
        assert md["tokenizer.ggml.tokens"] == ["<s>", "a", "é"]
        assert md["tokenizer.ggml.scores"] == [0.0, -1.5, -2.0]
    assert gguf.main([str(path), str(tmp_path / "cli.mim")]) == 0


def test_unsupported_and_damaged_files(tmp_path):
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 40)
    with pytest.raises(gguf.GGUFError):
        gguf.GGUFFile(bad)
    write_gguf(tmp_path / "v9.gguf", [], [], version=9)
    with pytest.raises(gguf.GGUFError):
        gguf.GGUFFile(tmp_path / "v9.gguf")
    # a Q5_K tensor (type 13) cannot be held: refused by convert unless skipped
    p = tmp_path / "q5.gguf"
    write_gguf(p, [], [("x", (1, 256), 13, b"\0" * 176), ("y", (2, 2), 0, b"\0" * 16)])
    with pytest.raises(gguf.GGUFError):
        gguf.convert(p, tmp_path / "q5.mim")
    info = gguf.convert(p, tmp_path / "q5.mim", skip_unsupported=True)
    assert info["skipped"] == ["x"] and info["tensors"] == 1
    # truncated data section
    path, _ = _sample(tmp_path)
    raw = path.read_bytes()
    (tmp_path / "cut.gguf").write_bytes(raw[:-40])
    with pytest.raises(gguf.GGUFError):
        gguf.GGUFFile(tmp_path / "cut.gguf")
    # rows that do not fill blocks
    write_gguf(tmp_path / "odd.gguf", [], [("x", (2, 40), 8, b"\0" * 85)])
    with pytest.raises(gguf.GGUFError):
        gguf.GGUFFile(tmp_path / "odd.gguf")


def test_converted_llama_loads_and_matches_the_package_writer(tmp_path):
    """A tiny Llama written with the gguf package (when present) converts and loads as a model."""
    gg = pytest.importorskip("gguf")
    import numpy as np
    from mimir_b200 import llm
    rng = np.random.default_rng(0)
    d, ff, heads, kv, vocab, layers = 32, 64, 4, 2, 48, 2
    w = gg.GGUFWriter(str(tmp_path / "tiny.gguf"), "llama")
    w.add_block_count(layers); w.add_context_length(64); w.add_embedding_length(d); w.add_feed_forward_length(ff)
    w.add_head_count(heads); w.add_head_count_kv(kv); w.add_layer_norm_rms_eps(1e-5); w.add_rope_freq_base(10000.0)
    w.add_vocab_size(vocab)
    names = {"token_embd.weight": (vocab, d), "output_norm.weight": (d,), "output.weight": (vocab, d)}
    for i in range(layers):
        names.update({f"blk.{i}.attn_norm.weight": (d,), f"blk.{i}.ffn_norm.weight": (d,),
                      f"blk.{i}.attn_q.weight": (d, d), f"blk.{i}.attn_k.weight": (d // heads * kv, d),
                      f"blk.{i}.attn_v.weight": (d // heads * kv, d), f"blk.{i}.attn_output.weight": (d, d),
                      f"blk.{i}.ffn_gate.weight": (ff, d), f"blk.{i}.ffn_up.weight": (ff, d),
                      f"blk.{i}.ffn_down.weight": (d, ff)})
    vals = {n: (rng.standard_normal(s) * 0.1).astype(np.float32) for n, s in names.items()}
    for n, v in vals.items():
        w.add_tensor(n, v)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    with gguf.GGUFFile(tmp_path / "tiny.gguf") as g:
        assert g.metadata["llama.block_count"] == layers
        for n, v in vals.items():
            assert torch.equal(g.tensor(n), torch.from_numpy(v))
    gguf.convert(tmp_path / "tiny.gguf", tmp_path / "tiny.mim")
    model = llm.Model.load(str(tmp_path / "tiny.mim"))
    from mimir_b200 import tensor as T
    logits = model.logits(T.from_torch(torch.tensor([[1, 2, 3]]))).data()
    assert logits.shape == (1, 3, vocab) and torch.isfinite(logits).all()
