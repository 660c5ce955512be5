"""The .mim reader / writer against the reference's own sample files."""
import glob
import os

import pytest
import torch

from _refdir import reference_dir

REF = reference_dir()
FILES = sorted(glob.glob(os.path.join(REF, "**", "*.mim"), recursive=True)) if REF else []
needs_ref = pytest.mark.skipif(not FILES, reason="reference sample files not mounted")


@needs_ref
def test_every_sample_file_rewrites_bit_for_bit():
    from mimir_b200.io import mim
    assert len(FILES) >= 26
    for path in FILES:
        original = open(path, "rb").read()
        with mim.open(path) as m:
            assert m.verify(), path
            tensors = {n: m.tensor(n) for n in sorted(m.names(), key=lambda n: m._index[n][2])}
            again = mim.serialize(tensors, metadata=m.section_bytes(mim.SECTION_METADATA),
                                  graph=m.section_bytes(mim.SECTION_GRAPH), alignment=m.alignment,
                                  minor=m.minor, legacy_magic=m.legacy_magic)
        assert again == original, path


@needs_ref
def test_golden_optimizer_file_contents():
    from mimir_b200.io import mim
    with mim.open(os.path.join(REF, "testdata/golden/optim.mim")) as m:
        assert m.metadata["oracle"] == "numpy" and m.metadata["seed"] == "20261015"
        t = m.tensor("adadelta/in0")
        assert t.dtype == torch.float32 and t.shape == (8,)


def test_write_read_round_trip_with_typed_metadata(tmp_path):
    from mimir_b200.io import mim
    from mimir_b200.io.metadata import UInt64
    tensors = {"b": torch.arange(6, dtype=torch.int32).view(2, 3), "a.w": torch.randn(300, 1000),
               "c": torch.randn(4).bfloat16(), "d": torch.tensor(3, dtype=torch.int64)}
    md = {"general.architecture": "llama", "llama.block_count": 2, "x.f": 1.5, "x.b": True,
          "x.u": UInt64(3), "ids": [1, 2, 3], "scores": [0.5, 1.25], "tokens": ["a", "bc", ""]}
    path = tmp_path / "m.mim"
    mim.write_tensors(path, tensors, metadata=md, training={"epochs": 2, "steps": 10, "lr": 1e-3})
    with mim.open(path) as m:
        assert m.verify()
        assert m.names() == sorted(tensors)
        for k, v in tensors.items():
            assert torch.equal(m.tensor(k), v)
        assert m.metadata == md and isinstance(m.metadata["x.u"], UInt64)
        assert m.training() == {"epochs": 2, "steps": 10, "lr": 1e-3}
        # a large tensor starts on a 4 KiB boundary inside the weights section
        assert m._index["a.w"][2] % 4096 == 0
    data = open(path, "rb").read()
    with pytest.raises(mim.MimError):
        mim.parse(data[:-1])


def test_describe_lists_sections_tensors_metadata_and_graph(tmp_path):
    import io as _io
    import torch
    from mimir_b200 import nn
    from mimir_b200 import tensor as T
    from mimir_b200.io import export, mim
    p = tmp_path / "d.mim"
    export.export(p, nn.Sequential(nn.Linear(4, 3), nn.ReLU()), T.tensor(torch.randn(2, 4)),
                  metadata={"general.name": "tiny"})
    buf = _io.StringIO()
    mim.describe(p, out=buf)
    text = buf.getvalue()
    for want in ("hashes ok", "section weights", "section graph", "tensor layers.0.weight: f32 [3, 4]",
                 "metadata general.name = 'tiny'", "graph inputs [('input', 'f32', [2, 4])]"):
        assert want in text, text
