"""safetensors reader / writer / importer; cross-checked with the safetensors package when present."""
import json
import struct

import pytest
import torch

from mimir_b200.io import mim
from mimir_b200.io import safetensors as st


def _tensors():
    torch.manual_seed(0)
    return {"w": torch.randn(3, 5), "h": torch.randn(4, 2).half(), "b": torch.randn(7).bfloat16(),
            "i": torch.arange(6, dtype=torch.int64).reshape(2, 3), "m": torch.tensor([True, False, True]),
            "empty": torch.zeros(0, 4)}


def test_roundtrip_and_convert(tmp_path):
    ts = _tensors()
    p = tmp_path / "a.safetensors"
    st.save(p, ts, metadata={"format": "pt", "step": 12})
    with st.SafetensorsFile(p) as f:
        assert f.metadata == {"format": "pt", "step": "12"}
        assert set(f.tensors) == set(ts)
        for n, t in ts.items():
            got = f.tensor(n)
            assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t), n
    back = st.load(p)
    assert all(torch.equal(back[n], t) for n, t in ts.items())
    assert st.convert(p, tmp_path / "a.mim") == len(ts)
    with mim.open(tmp_path / "a.mim") as m:
        assert torch.equal(m.tensor("w"), ts["w"]) and torch.equal(m.tensor("b"), ts["b"])
        assert m.tensor("m").tolist() == [1, 0, 1]
        assert m.metadata["format"] == "pt"
    assert st.main([str(p), str(tmp_path / "cli.mim")]) == 0


def test_matches_the_safetensors_package(tmp_path):
    pkg = pytest.importorskip("safetensors.torch")
    ts = {k: v for k, v in _tensors().items() if k != "empty"}
    pkg.save_file(ts, str(tmp_path / "pkg.safetensors"), metadata={"k": "v"})
    with st.SafetensorsFile(tmp_path / "pkg.safetensors") as f:
        assert f.metadata == {"k": "v"}
        for n, t in ts.items():
            assert torch.equal(f.tensor(n), t)
    st.save(tmp_path / "ours.safetensors", ts)
    theirs = pkg.load_file(str(tmp_path / "ours.safetensors"))
    assert all(torch.equal(theirs[n], t) for n, t in ts.items())


def test_damaged_files(tmp_path):
    (tmp_path / "short").write_bytes(b"\x01\x02")
    with pytest.raises(st.SafetensorsError):
        st.SafetensorsFile(tmp_path / "short")
    (tmp_path / "big").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(st.SafetensorsError):
        st.SafetensorsFile(tmp_path / "big")
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    (tmp_path / "size").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(st.SafetensorsError):
        st.SafetensorsFile(tmp_path / "size")
    hdr = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    (tmp_path / "dt").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(st.SafetensorsError):
        st.SafetensorsFile(tmp_path / "dt")
