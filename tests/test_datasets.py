"""Dataset readers and the Parquet reader (reference: data/datasets/*_test.go, io/parquet/*_test.go)."""
import os

import pytest

import torch

from mimir_b200.data import datasets
from mimir_b200.io import mim, parquet


def test_mnist_idx_round_trip(tmp_path):
    img = torch.randint(0, 256, (10, 28, 28), dtype=torch.uint8)
    lab = torch.arange(10, dtype=torch.uint8)
    datasets.write_idx(os.path.join(tmp_path, "train-images-idx3-ubyte"), img)
    datasets.write_idx(os.path.join(tmp_path, "train-labels-idx1-ubyte"), lab)
    ds = datasets.mnist(str(tmp_path), batch_size=4, shuffle=False, normalize=False)
    batches = list(ds)
    assert [b.x.shape[0] for b in batches] == [4, 4, 2]
    assert torch.equal((batches[0].x.data() * 255).round().to(torch.uint8)[:, 0], img[:4])
    assert batches[2].y.data().tolist() == [8, 9]


def test_csv_and_shards(tmp_path):
    for k in range(2):
        with open(os.path.join(tmp_path, f"s{k}.csv"), "w") as f:
            f.write("a,b,y\n")
            for i in range(5):
                f.write(f"{i + 10 * k},{2 * i},{i % 2}\n")
    X, y, names = datasets.read_csv(os.path.join(tmp_path, "s0.csv"), "y")
    assert names == ["a", "b"] and X.shape == (5, 2) and y.tolist() == [0, 1, 0, 1, 0]
    st = datasets.csv_shards(os.path.join(tmp_path, "s*.csv"), "y", batch_size=4)
    rows = torch.cat([b.x.data() for b in st])
    assert rows.shape == (10, 2) and rows[:, 0].tolist() == [0, 1, 2, 3, 4, 10, 11, 12, 13, 14]


def test_parquet_reader_and_shards(tmp_path):
    p = os.path.join(tmp_path, "d.parquet")
    cols = {"f0": torch.arange(100).float(), "f1": torch.arange(100).double() * 2, "label": torch.arange(100) % 3,
            "name": [f"r{i}" for i in range(100)]}
    for comp in ("snappy", "gzip", "zstd"):
        parquet.write(p, cols, compression=comp, row_group_size=40)
        f = parquet.File(p)
        assert f.rows == 100 and f.row_groups == 3 and f.columns == ["f0", "f1", "label", "name"]
        got = f.read()
        assert torch.equal(got["f0"], cols["f0"]) and got["name"][7] == "r7" and got["label"].dtype == torch.int64
        X, y = f.matrix(["f0", "f1"], "label", row_group=1)
        assert X.shape == (40, 2) and X[0].tolist() == [40.0, 80.0] and y[0] == 40 % 3
    st = datasets.parquet_shards(p, ["f0", "f1"], "label", batch_size=32)
    assert sum(b.x.shape[0] for b in st) == 100


def test_mapped_and_synthetic(tmp_path):
    p = os.path.join(tmp_path, "d.mim")
    mim.write_tensors(p, {"x": torch.arange(24.0).view(6, 4), "y": torch.arange(6)})
    ds = datasets.mapped(p, batch_size=4, shuffle=False)
    b = list(ds)
    assert b[0].x.data()[1].tolist() == [4.0, 5, 6, 7] and b[1].y.data().tolist() == [4, 5]
    c = datasets.synthetic_classification(rows=64, classes=3, batch_size=16)
    assert len(list(c)) == 4
    t = datasets.synthetic_tokens(rows=8, seq=16, vocab=32, batch_size=4)
    b0 = next(iter(t))
    assert b0.x.shape == (4, 16) and b0.y.shape == (4, 16)
    assert datasets.synthetic_regression(rows=10, batch_size=5).rows() == 10


def test_streamed_statistics_normalize_and_named_classes(tmp_path):
    """README "Scale": statistics in one parallel pass over the shards, applied as the stream is read;
    a string label column mapped through its class names."""
    from mimir_b200 import data
    torch.manual_seed(0)
    paths, Xs = [], []
    for k in range(3):
        n = 500 + 37 * k
        X = torch.randn(n, 4) * torch.tensor([1.0, 5.0, 0.1, 2.0]) + torch.tensor([0.0, 10.0, -3.0, 1.0])
        Xs.append(X)
        p = os.path.join(tmp_path, f"s{k}.parquet")
        parquet.write(p, {"a": X[:, 0], "b": X[:, 1], "c": X[:, 2], "d": X[:, 3],
                          "label": ["yes" if v > 0 else "no" for v in X[:, 0].tolist()]}, row_group_size=200)
        paths.append(p)
    allX = torch.cat(Xs)
    src = datasets.parquet_shards(paths, ["a", "b", "c", "d"], "label", classes=("no", "yes"), batch_size=128)
    mean, std = data.statistics(src)
    assert torch.allclose(mean, allX.mean(0), atol=1e-4) and torch.allclose(std, allX.std(0), rtol=1e-4)
    st = datasets.parquet_shards(paths, ["a", "b", "c", "d"], "label", classes=("no", "yes"), batch_size=128,
                                 normalize=(mean, std), class_targets=True, shuffle_buffer=256, seed=3)
    xs, ys = [], []
    for b in st:
        xs.append(b.x.data())
        ys.append(b.y.data())
    Xn, Y = torch.cat(xs), torch.cat(ys)
    assert Xn.shape == allX.shape and Y.dtype == torch.int64
    assert torch.allclose(Xn.mean(0), torch.zeros(4), atol=1e-3) and torch.allclose(Xn.std(0), torch.ones(4), atol=1e-3)
    assert int(Y.sum()) == int((allX[:, 0] > 0).sum())
    assert torch.equal(Y, (Xn[:, 0] * std[0] + mean[0] > 0).long())                 # labels stayed with their rows through the shuffle
    with pytest.raises(ValueError, match="maybe"):
        p = os.path.join(tmp_path, "bad.parquet")
        parquet.write(p, {"a": torch.zeros(2), "label": ["yes", "maybe"]})
        list(datasets.parquet_shards(p, ["a"], "label", classes=("no", "yes")))


def test_native_csv_reader_equals_the_general_one(tmp_path):
    """Plain numeric files are parsed in native code, pieces of the file in parallel; the general reader is the
    oracle (and the fallback for quoted or non-numeric fields): empty fields, blank lines, CRLF, signs, exponents,
    a last line without a line end, and a file large enough to be cut into pieces."""
    import numpy as np
    from mimir_b200.data import datasets
    small = tmp_path / "s.csv"
    small.write_text("a,b,c\r\n1,,3\r\n\r\n+4.5, 5e-1 ,nan\r\n7,8,9")
    X, y, names = datasets.read_csv(str(small))
    assert names == ["a", "b"] and X.shape == (3, 2) and torch.isnan(X[0, 1]) and torch.isnan(y[1])
    assert X[1].tolist() == [4.5, 0.5] and y.tolist()[::2] == [3.0, 9.0]
    big = tmp_path / "b.csv"
    table = np.random.default_rng(0).standard_normal((30000, 9))
    np.savetxt(big, table, delimiter=",", header=",".join(f"c{i}" for i in range(9)), comments="", fmt="%.9g")
    assert big.stat().st_size > (1 << 20)
    Xn, yn, _ = datasets.read_csv(str(big), label="c3")
    native = datasets._read_csv_native
    try:
        datasets._read_csv_native = lambda *a: None
        Xg, yg, _ = datasets.read_csv(str(big), label="c3")
    finally:
        datasets._read_csv_native = native
    assert torch.equal(Xn, Xg) and torch.equal(yn, yg) and Xn.shape == (30000, 8)
    quoted = tmp_path / "q.csv"
    quoted.write_text('a,b\n1,"2"\n')
    assert datasets._read_csv_native(str(quoted), True) is None and datasets.read_csv(str(quoted))[1].tolist() == [2.0]
    ragged = tmp_path / "r.csv"
    ragged.write_text("a,b\n1,2\n3\n")
    assert datasets._read_csv_native(str(ragged), True) is None
    bare = tmp_path / "n.csv"
    bare.write_text("1,2\n3,4\n")
    assert datasets.read_csv(str(bare), header=False)[0].tolist() == [[1.0], [3.0]]
